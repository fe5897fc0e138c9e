"""Each part alone against the plain functions, and a toy architecture built from outside the package.

The toy architecture is defined here and registered through the public registries only; no file of the
framework knows it. It holds a mixer with state of its own (an exponential moving average), an
attention layer with a window (a page group of its own whose pages are given back as the window moves),
a layer that runs twice, a schedule entry that reads another entry's cache, a feed-forward that routes every
token to one of three experts, a position encoding that is not rotary (a decay with distance), a mixer whose
per-token storage is one pool of pages of a size of its own, and the decoder's optional ends (embedding multiplier,
logit scale and softcap).
"""

from dataclasses import dataclass, field

import numpy as np
import pytest
import torch

import plain_lfm2 as plain
import tiny
import traces
from akas_b200.cache import CacheManager
from akas_b200.config import (AttentionSpec, EngineConfig, LayerSpec, ModelSpec, PartSpec, RMSNormSpec, RopeSpec,
                              ScheduleEntry, ShortConvSpec, SwiGLUSpec, register_architecture)
from akas_b200.engine.batch import BatchLayout, StepEntry, fill_batch
from akas_b200.engine.runner import ModelRunner
from akas_b200.ops import reference
from akas_b200.parts import (Block, FeedForward, Mixer, PagedSpec, Param, Part, Runtime, StateSpec, build_part, register_ffn,
                             register_mixer, register_position)
from akas_b200.weights import write_random_model


def _devices():
    out = [pytest.param("cpu", id="cpu-reference-ops")]
    out.append(pytest.param("cuda:0", id="gpu", marks=pytest.mark.gpu))
    return out


def _runtime(device, dtype=torch.float32):
    if device == "cpu":
        return Runtime(dtype, torch.device("cpu"), reference)
    from akas_b200.ops import cuda

    cuda.require()
    return Runtime(dtype, torch.device(device), cuda)


def _context(rt, cache, lengths):
    """A StepContext for fresh requests of the given lengths, each run whole."""
    from akas_b200.engine.runner import ModelRunner as _R

    entries = []
    for i, n in enumerate(lengths):
        cache.admit(i)
        cache.reserve(i, n)
        entries.append(StepEntry(i, [0] * n, ()))
    lay = BatchLayout(sum(lengths), len(lengths), 0, cache.table_widths)
    host = torch.zeros(lay.size, dtype=torch.int32)
    mq, mc = fill_batch(host.numpy(), lay, entries, cache)
    dev = host.to(rt.device)
    shim = type("S", (), {"cache": cache})()
    return _R._context(shim, dev, lay, mq, mc, False)


def _rel(got, want):
    """Largest difference relative to the largest reference value (float32 results of size 40 carry 5e-6)."""
    return ((got - want).abs().max() / want.abs().max()).item()


def _rand(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64) * scale


@pytest.mark.parametrize("device", _devices())
def test_rmsnorm_part(device):
    rt = _runtime(device)
    for zero_centered in (False, True):
        part = build_part("norm", RMSNormSpec(50, 1e-6, zero_centered), rt)
        w = _rand((50,), 1)
        part.load(lambda name: w.float().to(rt.device))
        x = _rand((7, 50), 2, 3.0)
        want = plain.rms_norm(x, w + 1 if zero_centered else w, 1e-6)
        got = part.forward(x.float().to(rt.device), out_dtype=torch.float32).double().cpu()
        assert _rel(got, want) < 1e-5


@pytest.mark.parametrize("device", _devices())
@pytest.mark.parametrize("taps,bias", [(3, False), (5, True)])
def test_short_conv_part(device, taps, bias):
    rt = _runtime(device)
    c = 40
    part = build_part("mixer", ShortConvSpec(c, taps, bias), rt)
    w = {"in_proj.weight": _rand((3 * c, c), 1, 0.3), "conv.weight": _rand((c, 1, taps), 2), "out_proj.weight": _rand((c, c), 3, 0.3),
         "conv.bias": _rand((c,), 4), "in_proj.bias": _rand((3 * c,), 8), "out_proj.bias": _rand((c,), 9)}
    biases = {"conv.bias", "in_proj.bias", "out_proj.bias"}  # the option gives all three or none
    assert set(part.params()) == set(w) - (set() if bias else biases)
    part.load(lambda name: w[name].float().to(rt.device))
    cache = CacheManager([part.cache()], 8, 64, 2, 32, device=rt.device)
    lengths = [11, 4]
    ctx = _context(rt, cache, lengths)
    x = _rand((sum(lengths), c), 5)
    state_before = cache.views[0].state.clone()
    peek = part.forward(x.float().to(rt.device), ctx, cache.views[0], write=False).double().cpu()
    assert torch.equal(cache.views[0].state, state_before)  # a layer that reads another's state leaves it alone
    h = _rand((sum(lengths), c), 6)
    got = part.forward(x.float().to(rt.device), ctx, cache.views[0]).double().cpu()
    assert torch.equal(got, peek)
    assert not torch.equal(cache.views[0].state, state_before)
    at = 0
    for n in lengths:
        want = plain.short_conv(x[at:at + n], w["in_proj.weight"], w["conv.weight"].reshape(c, taps),
                                w["conv.bias"] if bias else None, w["out_proj.weight"],
                                w["in_proj.bias"] if bias else None, w["out_proj.bias"] if bias else None)
        assert _rel(got[at:at + n], want) < 1e-5
        at += n
    # with a residual the result is residual + mixer(x), the output bias included; the state moved on by then, so
    # fresh requests run the same tokens again
    cache2 = CacheManager([part.cache()], 8, 64, 2, 32, device=rt.device)
    ctx2 = _context(rt, cache2, lengths)
    summed = part.forward(x.float().to(rt.device), ctx2, cache2.views[0], residual=h.float().to(rt.device)).double().cpu()
    assert _rel(summed, h.float().double() + got) < 1e-5


@pytest.mark.parametrize("device", _devices())
@pytest.mark.parametrize("heads,kv,dim,window,rotary", [(4, 2, 16, None, None), (3, 1, 32, 6, None), (2, 2, 48, None, 16)])
def test_attention_part(device, heads, kv, dim, window, rotary):
    rt = _runtime(device)
    c = 40
    spec = AttentionSpec(c, heads, kv, dim, qk_norm=RMSNormSpec(dim, 1e-6), position=RopeSpec(dim, 1e4, rotary), window=window)
    part = build_part("mixer", spec, rt)
    w = {"q_proj.weight": _rand((heads * dim, c), 1, 0.3), "k_proj.weight": _rand((kv * dim, c), 2, 0.3),
         "v_proj.weight": _rand((kv * dim, c), 3, 0.3), "out_proj.weight": _rand((c, heads * dim), 4, 0.3),
         "q_norm.weight": _rand((dim,), 5) + 1, "k_norm.weight": _rand((dim,), 6) + 1}
    assert set(part.params()) == set(w)
    part.load(lambda name: w[name].float().to(rt.device))
    cache = CacheManager([part.cache()], 4, 64, 2, 32, device=rt.device)
    lengths = [13, 6]
    ctx = _context(rt, cache, lengths)
    x = _rand((sum(lengths), c), 7)
    h = torch.zeros((sum(lengths), c), dtype=torch.float32, device=rt.device)
    got = part.forward(x.float().to(rt.device), ctx, cache.views[0], residual=h).double().cpu()
    at = 0
    for n in lengths:
        want = plain.attention(x[at:at + n], w["q_proj.weight"], w["k_proj.weight"], w["v_proj.weight"],
                               w["out_proj.weight"], w["q_norm.weight"], w["k_norm.weight"], 1e-6, heads, kv, dim,
                               1e4, window, rotary)
        assert _rel(got[at:at + n], want) < 1e-5
        at += n


@pytest.mark.parametrize("device", _devices())
def test_swiglu_part_and_block(device):
    rt = _runtime(device)
    c, f = 24, 56
    w = {"ff.w1.weight": _rand((f, c), 1, 0.3), "ff.w3.weight": _rand((f, c), 2, 0.3), "ff.w2.weight": _rand((c, f), 3, 0.3),
         "mix.in_proj.weight": _rand((3 * c, c), 4, 0.3), "mix.conv.weight": _rand((c, 1, 3), 5),
         "mix.out_proj.weight": _rand((c, c), 6, 0.3), "n1": _rand((c,), 7) + 1, "n2": _rand((c,), 8) + 1}
    spec = LayerSpec(ShortConvSpec(c, 3), SwiGLUSpec(c, f), RMSNormSpec(c, 1e-5), RMSNormSpec(c, 1e-5), "mix.", "ff.", "n1", "n2")
    block = Block(spec, rt)
    assert set(block.params()) == set(w)
    block.load(lambda name: w[name].float().to(rt.device))
    cache = CacheManager([block.mixer.cache()], 8, 64, 1, 32, device=rt.device)
    ctx = _context(rt, cache, [9])
    h = _rand((9, c), 9)
    got = block.forward(h.float().to(rt.device), ctx, cache.views[0]).double().cpu()
    x = plain.rms_norm(h, w["n1"], 1e-5)
    h1 = h + plain.short_conv(x, w["mix.in_proj.weight"], w["mix.conv.weight"].reshape(c, 3), None, w["mix.out_proj.weight"])
    want = h1 + plain.swiglu(plain.rms_norm(h1, w["n2"], 1e-5), w["ff.w1.weight"], w["ff.w3.weight"], w["ff.w2.weight"])
    assert _rel(got, want) < 1e-5


# --------------------------------------------------------------------------- a toy architecture


class EmaMixer(Mixer):
    """s_t = decay * s_{t-1} + x_t W^T, out_t = s_t: one vector of state per request."""

    def params(self):
        c = self.spec.options["width"]
        return {"proj.weight": Param((c, c)), "decay": Param((c,), role="vector", mean=0.5)}

    def load(self, get):
        self.w, self.decay = get("proj.weight"), get("decay")

    def cache(self):
        return StateSpec((self.spec.options["width"],))

    def forward(self, x, ctx, cache=None, residual=None, write=True):
        u = self.rt.ops.linear(x, self.w, out_dtype=torch.float32)
        out = torch.zeros_like(u)
        slots, at = ctx.slots.tolist(), 0
        for r, count in enumerate(ctx.query_lens):  # how many tokens each request brings is known on the host
            s = cache.state[slots[r]].clone()
            for t in range(at, at + count):
                s = self.decay * s + u[t]
                out[t] = s
            cache.state[slots[r]] = s
            at += count
        return residual.add_(out) if residual is not None else out.to(x.dtype)


@dataclass(frozen=True)
class LatentPages(PagedSpec):
    """One pool, one vector per token, pages of two tokens whatever the engine's page size is."""

    width: int = 0
    page_size: int = 2
    dtype: torch.dtype = torch.float32
    window: int = None

    def pools(self, page_size):
        return {"latent": (page_size, self.width)}


class PrefixMeanMixer(Mixer):
    """z_t = x_t W^T goes into the request's pages; out_t is the mean of z_s over s <= t, read back from the pages."""

    def params(self):
        c = self.spec.options["width"]
        return {"proj.weight": Param((c, c))}

    def load(self, get):
        self.w = get("proj.weight")

    def cache(self):
        return LatentPages(width=self.spec.options["width"])

    def forward(self, x, ctx, cache=None, residual=None, write=True):
        z = self.rt.ops.linear(x, self.w, out_dtype=torch.float32)
        table, page = ctx.block_table(cache.group).long(), cache.page_size
        seq, pos = ctx.seq_of_token.long(), ctx.positions.long()
        live = (seq >= 0).nonzero().flatten()
        if write:
            cache.latent[table[seq[live], pos[live] // page], pos[live] % page] = z[live]
        out = torch.zeros_like(z)
        for t in live.tolist():
            upto = torch.arange(int(pos[t]) + 1, device=x.device)
            out[t] = cache.latent[table[seq[t], upto // page], upto % page].mean(dim=0)
        return residual.add_(out) if residual is not None else out.to(x.dtype)


class RoutedFeedForward(FeedForward):
    """Every token goes to the expert whose router logit is largest (lowest index among equals); the expert's
    output, relu(x U^T) D^T, is weighted by the softmax probability of that logit. Router and softmax in float32."""

    def params(self):
        o = self.spec.options
        p = {"router.weight": Param((o["experts"], o["width"]))}
        for e in range(o["experts"]):
            p[f"experts.{e}.up.weight"] = Param((o["hidden"], o["width"]))
            p[f"experts.{e}.down.weight"] = Param((o["width"], o["hidden"]))
        return p

    def load(self, get):
        n = self.spec.options["experts"]
        self.router = get("router.weight")
        self.up = [get(f"experts.{e}.up.weight") for e in range(n)]
        self.down = [get(f"experts.{e}.down.weight") for e in range(n)]

    def forward(self, x, ctx, residual=None):
        ops = self.rt.ops
        logits = ops.linear(x, self.router, out_dtype=torch.float32)
        weight, expert = torch.softmax(logits, dim=-1).max(dim=-1)
        out = torch.zeros((x.shape[0], self.spec.options["width"]), dtype=torch.float32, device=x.device)
        for e in range(len(self.up)):
            rows = (expert == e).nonzero().flatten()
            if rows.numel():
                hidden = torch.relu(ops.linear(x[rows].contiguous(), self.up[e], out_dtype=torch.float32)).to(x.dtype)
                out[rows] = ops.linear(hidden, self.down[e], out_dtype=torch.float32) * weight[rows, None]
        return residual.add_(out) if residual is not None else out.to(x.dtype)


class DecayPosition(Part):
    """q_t *= g^t, k_t *= g^-t per channel pair rate g: a score then carries g^(t - s), a decay with distance.
    No tables for the fused rotary kernel, so the attention mixer calls ``apply`` and stores k and v after it."""

    def apply(self, q, k, ctx):
        rate = float(self.spec.options["rate"])
        pos = ctx.positions.to(torch.float32)[:, None]
        return (q.float() * rate ** pos).to(q.dtype), (k.float() * rate ** -pos).to(k.dtype)


@dataclass(frozen=True)
class ToyConfig:
    width: int = 32
    vocab: int = 50
    window: int = 12
    architecture = "ToyHybridForTests"

    @classmethod
    def from_dict(cls, data):
        return cls(data["width"], data["vocab"], data["window"])

    def to_dict(self):
        return dict(architectures=[self.architecture], width=self.width, vocab=self.vocab, window=self.window)

    def model_spec(self):
        c = self.width
        norm = RMSNormSpec(c, 1e-5)

        def layer(i, mixer, ffn=SwiGLUSpec(c, 48)):
            p = f"layers.{i}."
            return LayerSpec(mixer, ffn, norm, norm, p + "mixer.", p + "ffn.", p + "norm1", p + "norm2")

        attn = dict(qk_norm=RMSNormSpec(16, 1e-5), position=RopeSpec(16, 1e4))
        return ModelSpec(
            architecture=self.architecture, hidden_size=c, vocab_size=self.vocab,
            layers=(layer(0, PartSpec("ema_for_tests", {"width": c})),
                    layer(1, AttentionSpec(c, 2, 1, 16, window=self.window, **attn)),
                    layer(2, AttentionSpec(c, 2, 2, 16, **attn)),
                    layer(3, AttentionSpec(c, 2, 1, 16, qk_norm=None, position=PartSpec("decay_for_tests", {"rate": 0.97})),
                          PartSpec("routed_for_tests", {"width": c, "hidden": 40, "experts": 3})),
                    layer(4, PartSpec("prefix_mean_for_tests", {"width": c})),
                    layer(5, ShortConvSpec(c, 3, bias=True))),
            final_norm=norm, embedding_name="embed", final_norm_name="final_norm", head_name=None,
            # layer 1 runs twice, each time with a cache of its own; the fifth entry reads entry 2's keys and values; the
            # convolution layer runs twice in a row, each time with a state of its own
            schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(1), ScheduleEntry(2, cache=2),
                      ScheduleEntry(3), ScheduleEntry(4), ScheduleEntry(5), ScheduleEntry(5)),
            embedding_multiplier=1.7, logit_scale=0.4, logit_softcap=2.5,
        )


def _toy_plain(cfg, w, tokens):
    """The toy model, whole sequence, float64, from the plain part functions."""
    c, T = cfg.width, len(tokens)
    h = w["embed"][torch.as_tensor(tokens)] * 1.7
    kept = {}

    def attn(i, x, window, heads, kv, shared=None, decay=None):
        p = f"layers.{i}.mixer."
        d = 16
        pos = torch.arange(T)
        if decay is not None:  # no QK-norm, decay position: q_t g^t, k_t g^-t
            q = (x @ w[p + "q_proj.weight"].T).reshape(T, heads, d) * decay ** pos[:, None, None].double()
            k = (x @ w[p + "k_proj.weight"].T).reshape(T, kv, d) * decay ** -pos[:, None, None].double()
            v = (x @ w[p + "v_proj.weight"].T).reshape(T, kv, d)
        else:
            q = plain.rms_norm((x @ w[p + "q_proj.weight"].T).reshape(T, heads, d), w[p + "q_norm.weight"], 1e-5)
            cos, sin = plain.rope_tables(torch.arange(T), d, 1e4, torch.float64)
            q = plain.apply_rope(q, cos, sin)
            if shared is None:
                k = plain.rms_norm((x @ w[p + "k_proj.weight"].T).reshape(T, kv, d), w[p + "k_norm.weight"], 1e-5)
                k, v = plain.apply_rope(k, cos, sin), (x @ w[p + "v_proj.weight"].T).reshape(T, kv, d)
            else:
                k, v = shared
        seen = pos[None, :] <= pos[:, None]
        if window:
            seen &= pos[None, :] > pos[:, None] - window
        kk, vv = k.repeat_interleave(heads // kv, 1), v.repeat_interleave(heads // kv, 1)
        score = (torch.einsum("thd,shd->hts", q, kk) * d ** -0.5).masked_fill(~seen[None], float("-inf"))
        out = torch.einsum("hts,shd->thd", torch.softmax(score, -1), vv).reshape(T, heads * d)
        return out @ w[p + "out_proj.weight"].T, (k, v)

    for n, (i, shared) in enumerate(((0, None), (1, None), (2, None), (1, None), (2, 2), (3, None), (4, None), (5, None),
                                     (5, None))):
        p = f"layers.{i}."
        x = plain.rms_norm(h, w[p + "norm1"], 1e-5)
        if i == 0:
            u = x @ w[p + "mixer.proj.weight"].T
            s, rows = torch.zeros(c, dtype=torch.float64), []
            for t in range(T):
                s = w[p + "mixer.decay"] * s + u[t]
                rows.append(s)
            mixed = torch.stack(rows)
        elif i == 3:
            mixed, kept[n] = attn(i, x, None, 2, 1, decay=0.97)
        elif i == 4:
            z = x @ w[p + "mixer.proj.weight"].T
            mixed = torch.cumsum(z, 0) / torch.arange(1, T + 1, dtype=torch.float64)[:, None]
        elif i == 5:
            m = p + "mixer."
            mixed = plain.short_conv(x, w[m + "in_proj.weight"], w[m + "conv.weight"].reshape(c, 3), w[m + "conv.bias"],
                                     w[m + "out_proj.weight"], w[m + "in_proj.bias"], w[m + "out_proj.bias"])
        else:
            mixed, kept[n] = attn(i, x, cfg.window if i == 1 else None, 2, 1 if i == 1 else 2,
                                  kept[shared] if shared is not None else None)
        h = h + mixed
        f = p + "ffn."
        y = plain.rms_norm(h, w[p + "norm2"], 1e-5)
        if i == 3:  # routed: the expert with the largest router logit, weighted by its softmax probability
            prob = torch.softmax(y @ w[f + "router.weight"].T, -1)
            weight, expert = prob.max(-1)
            routed = torch.zeros_like(h)
            for t in range(T):
                e = int(expert[t])
                routed[t] = torch.relu(y[t] @ w[f + f"experts.{e}.up.weight"].T) @ w[f + f"experts.{e}.down.weight"].T * weight[t]
            h = h + routed
        else:
            h = h + plain.swiglu(y, w[f + "w1.weight"], w[f + "w3.weight"], w[f + "w2.weight"])
    logits = plain.rms_norm(h, w["final_norm"], 1e-5) @ w["embed"].T * 0.4
    return 2.5 * torch.tanh(logits / 2.5)


@pytest.mark.parametrize("device", _devices())
def test_toy_architecture_is_registered_built_and_stepped(device, tmp_path):
    register_mixer("ema_for_tests", EmaMixer)
    register_ffn("routed_for_tests", RoutedFeedForward)
    register_position("decay_for_tests", DecayPosition)
    register_mixer("prefix_mean_for_tests", PrefixMeanMixer)
    register_architecture(ToyConfig.architecture, ToyConfig)
    cfg = ToyConfig()
    folder = write_random_model(tmp_path / "toy", cfg, seed=3, std=0.2, dtype="float32")
    from safetensors.torch import load_file

    w = {k: v.double() for k, v in load_file(str(folder / "model.safetensors")).items()}
    reqs = {f"t{i}": p for i, p in enumerate(tiny.prompts(cfg.vocab, [41, 3, 30, 17, 26], seed=9))}
    want = {rid: _toy_plain(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    ops = reference if device == "cpu" else None
    page = 4

    def runner(tokens):
        config = EngineConfig(dtype="float32", device=device, page_size=page, max_tokens=tokens, max_requests=4,
                              context=48, cuda_graphs=False)
        return ModelRunner(folder, config, ops=ops)

    r = runner(48)
    assert len(r.cache.groups) == 3 and [type(v).__name__ for v in r.cache.views] == [
        "StateCache", "PagedCache", "PagedCache", "PagedCache", "NoneType", "PagedCache", "PagedCache", "StateCache",
        "StateCache"]
    assert r.cache.views[7].state.data_ptr() != r.cache.views[8].state.data_ptr()  # the layer named twice: two states
    latent = r.cache.views[6]
    assert latent.page_size == 2 and latent.latent.shape == (24, 2, cfg.width) and r.cache.table_widths == [12, 12, 24]
    steps, peak = traces.mixed(reqs, {rid: max(1, len(t) - 6) for rid, t in reqs.items()}, seed=2, live=3, page=page)
    for name, trace, pool in (("whole", traces.whole(reqs), 48), ("portions", traces.portions(reqs), 48),
                              ("tail", traces.tail_decoded(reqs, 8), 48), ("mixed", steps, peak)):
        r = runner(pool)
        got = traces.replay(r, trace)
        for rid in reqs:
            bad = traces.first_bad(got[rid], want[rid], 2e-5)
            assert bad is None, f"{name}: {rid} first differs at {bad}: {traces.worst(got[rid], want[rid])}"
        assert r.cache.min_free_pages() == r.cache.num_pages
    # a summary of the past cannot be read by a second entry: after the owner has run it has moved past the step's tokens
    from dataclasses import replace
    from akas_b200.models.decoder import Decoder

    spec = cfg.model_spec()
    shared = replace(spec, schedule=spec.schedule[:8] + (ScheduleEntry(5, cache=7),))
    with pytest.raises(ValueError, match="cache of its own"):
        Decoder(shared, r.model.rt)
    # the windowed group gave pages back while the request was still running
    r = runner(48)
    r.step([StepEntry("w", reqs["t0"], ())])
    full, win = r.cache.blocks("w", r.cache.views[2].group), r.cache.blocks("w", r.cache.views[1].group)
    assert all(p >= 0 for p in full) and sum(p < 0 for p in win) == (41 - cfg.window + 1) // page
