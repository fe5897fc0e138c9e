"""A block: a mixer and a feed-forward, each behind its norm, around a float32 residual stream.

``pre_norm`` (the only arrangement LFM2 uses, src/akas/models/lfm2/_composition.py:189,308-309,356
in kreasof-ai/akas): h += mixer(norm(h)); h += ffn(norm(h)). Other arrangements are
added to ``ARRANGEMENTS`` as functions of (block, h, ctx, cache, write).
"""

from __future__ import annotations

from .base import Runtime, build_part


def _normed(norm, part, h):
    """The norm's output for ``part``: left to the part's first product when both sides can do that."""
    if getattr(part, "takes_normed", False) and hasattr(norm, "lazy"):
        return norm.lazy(h)
    return norm.forward(h)


def _pre_norm(block, h, ctx, cache, write):
    h = block.mixer.forward(_normed(block.mixer_norm, block.mixer, h), ctx, cache, residual=h, write=write)
    return block.ffn.forward(_normed(block.ffn_norm, block.ffn, h), ctx, residual=h)


ARRANGEMENTS = {"pre_norm": _pre_norm}


class Block:
    def __init__(self, spec, runtime: Runtime):
        if spec.arrangement not in ARRANGEMENTS:
            raise KeyError(f"unknown block arrangement {spec.arrangement!r}; known: {sorted(ARRANGEMENTS)}")
        self.spec = spec
        self.mixer = build_part("mixer", spec.mixer, runtime)
        self.ffn = build_part("ffn", spec.ffn, runtime)
        self.mixer_norm = build_part("norm", spec.mixer_norm, runtime)
        self.ffn_norm = build_part("norm", spec.ffn_norm, runtime)
        self._run = ARRANGEMENTS[spec.arrangement]
        # Whether every part of the block reaches its tensors through the runtime's operations only (see Part.chain_safe)
        self.chain_safe = all(getattr(part, "chain_safe", False) for part in (self.mixer, self.ffn, self.mixer_norm, self.ffn_norm))

    def params(self):
        """Checkpoint name -> Param for everything this block holds."""
        s = self.spec
        out = {s.mixer_prefix + k: v for k, v in self.mixer.params().items()}
        out.update({s.ffn_prefix + k: v for k, v in self.ffn.params().items()})
        (norm_param,) = self.mixer_norm.params().values()
        out[s.mixer_norm_name] = norm_param
        (norm_param,) = self.ffn_norm.params().values()
        out[s.ffn_norm_name] = norm_param
        return out

    def load(self, get):
        s = self.spec
        self.mixer.load(lambda name: get(s.mixer_prefix + name))
        self.ffn.load(lambda name: get(s.ffn_prefix + name))
        self.mixer_norm.load(lambda _name: get(s.mixer_norm_name))
        self.ffn_norm.load(lambda _name: get(s.ffn_norm_name))

    def forward(self, h, ctx, cache=None, write=True):
        return self._run(self, h, ctx, cache, write)
