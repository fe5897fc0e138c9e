"""Each kernel alone against its plain PyTorch statement, at sizes other than the engine's.

Sizes are chosen to hit tails: widths and vocabularies that are no power of two, head sizes 16 to 256
in steps of 16, group sizes 1 to 8 and odd ones, pages of 8 to 64, padding tokens, empty requests.
"""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from akas_b200.ops import cuda, reference

    cuda.require()
    return cuda, reference


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


def _close(a, b, dtype, what="", k=64):
    """``k``: length of the float32 sums behind the values; their rounding grows like its square root."""
    tol = 2e-6 * max(1.0, (k / 64) ** 0.5) if dtype == torch.float32 else 1e-2
    a, b = a.double(), b.double()
    scale = max(b.abs().max().item(), 1e-6)
    err = (a - b).abs().max().item() / scale
    assert err <= tol, f"{what}: relative error {err:.3g} > {tol}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(ops, dtype):
    cuda, ref = ops
    table = _rand((37, 50), dtype, 1)
    ids = torch.tensor([0, 36, 5, 5, 17], dtype=torch.int32, device=DEV)
    assert torch.equal(cuda.embedding(ids, table), ref.embedding(ids, table))


@pytest.mark.parametrize("dtype", DTYPES)
def test_add_bias_and_scale_cap(ops, dtype):
    cuda, ref = ops
    x, bias = _rand((9, 70), torch.float32, 4, 3.0), _rand((70,), torch.float32, 5)
    got, want = cuda.add_bias(x.clone(), bias, dtype), ref.add_bias(x.clone(), bias, dtype)
    assert got.dtype == dtype and torch.equal(got, want)  # one add, one rounding
    for scale, cap in ((1.7, 0.0), (0.4, 2.5), (1.0, 30.0)):
        got, want = cuda.scale_cap(x.clone(), scale, cap), ref.scale_cap(x.clone(), scale, cap)
        assert torch.allclose(got, want, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("c", [16, 48, 100, 2048, 3000])
def test_rmsnorm(ops, dtype, c):
    cuda, ref = ops
    x = _rand((7, c), torch.float32, 2, 3.0)
    w = _rand((c,), torch.float32, 3) + 1
    for zero_centered in (False, True):
        _close(cuda.rmsnorm(x, w, 1e-6, zero_centered, dtype), ref.rmsnorm(x, w, 1e-6, zero_centered, dtype), dtype)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    _close(cuda.rmsnorm(x, w, 1e-5, False, dtype, rows), ref.rmsnorm(x, w, 1e-5, False, dtype, rows), dtype)
    xt = x.to(dtype)  # input in the compute dtype too
    _close(cuda.rmsnorm(xt, w, 1e-5, False, dtype), ref.rmsnorm(xt, w, 1e-5, False, dtype), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(ops, dtype):
    cuda, ref = ops
    gu = _rand((5, 2 * 33), dtype, 4, 4.0)
    _close(cuda.swiglu(gu), ref.swiglu(gu), dtype)


@pytest.mark.parametrize("n,k,o", [(1, 64, 50), (17, 100, 37), (70, 52, 130), (200, 96, 192), (3, 50, 9), (129, 257, 65)])
def test_linear_float32(ops, n, k, o):
    cuda, ref = ops
    x, w = _rand((n, k), torch.float32, 5), _rand((o, k), torch.float32, 6)
    want = x.double() @ w.double().T
    _close(cuda.linear(x, w), want, torch.float32, "product")
    res = _rand((n, o), torch.float32, 7)
    got = cuda.linear(x, w, residual=res.clone())
    _close(got, res.double() + want, torch.float32, "product + residual")


def test_linear_float32_rows_do_not_depend_on_the_batch(ops):
    cuda, _ = ops
    x, w = _rand((300, 96), torch.float32, 8), _rand((130, 96), torch.float32, 9)
    whole = cuda.linear(x, w)
    for rows in (slice(0, 1), slice(5, 22), slice(100, 164), slice(299, 300)):
        assert torch.equal(cuda.linear(x[rows].contiguous(), w), whole[rows])
    # a wide w: up to 16 rows go through the kernel that streams w once; the same bits as the tiled kernel
    for k, o in ((200, 400), (520, 257), (1028, 300)):
        x, w = _rand((300, k), torch.float32, 8), _rand((o, k), torch.float32, 9)
        whole = cuda.linear(x, w)
        res = _rand((300, o), torch.float32, 10)
        added = cuda.linear(x, w, residual=res.clone())
        for rows in (slice(0, 1), slice(7, 10), slice(40, 48), slice(100, 109), slice(284, 300)):
            assert torch.equal(cuda.linear(x[rows].contiguous(), w), whole[rows])
            assert torch.equal(cuda.linear(x[rows].contiguous(), w, residual=res[rows].clone()), added[rows])


@pytest.mark.parametrize("n,k,o", [(1, 64, 50), (17, 104, 37), (70, 56, 130), (300, 96, 192), (8, 2048, 321)])
def test_linear_bfloat16(ops, n, k, o):
    cuda, ref = ops
    x, w = _rand((n, k), torch.bfloat16, 5), _rand((o, k), torch.bfloat16, 6)
    want = x.double() @ w.double().T
    _close(cuda.linear(x, w), want, torch.bfloat16, "bf16 out")
    _close(cuda.linear(x, w, out_dtype=torch.float32), want, torch.float32, "f32 out")
    res = _rand((n, o), torch.float32, 7)
    _close(cuda.linear(x, w, residual=res.clone()), res.double() + want, torch.float32, "accumulate")
    with pytest.raises(ValueError):  # an inner size that is no multiple of 8 is refused, not miscomputed
        cuda.linear(_rand((n, 60), torch.bfloat16, 5), _rand((o, 60), torch.bfloat16, 6))


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("k,o", [(64, 50), (192, 320), (2048, 37), (8192, 64), (96, 40)])
def test_skinny_products_for_few_tokens(ops, m, k, o, monkeypatch):
    """The decode-step product kernel: plain, float32 out, accumulate, SwiGLU, and with the norm riding along."""
    cuda, ref = ops
    monkeypatch.setattr(cuda, "decode_products", "skinny")
    x, w = _rand((m, k), torch.bfloat16, 5), _rand((o, k), torch.bfloat16, 6, 0.05)
    want = x.double() @ w.double().T
    _close(cuda.linear(x, w), want, torch.bfloat16, "bf16 out")
    _close(cuda.linear(x, w, out_dtype=torch.float32), want, torch.float32, "f32 out", k)
    res = _rand((m, o), torch.float32, 7)
    _close(cuda.linear(x, w, residual=res.clone()), res.double() + want, torch.float32, "accumulate", k)
    w2 = _rand((2 * o, k), torch.bfloat16, 8, 0.05)
    _close(cuda.linear_swiglu(x, w2), ref.linear_swiglu(x, w2), torch.bfloat16, "swiglu")
    # the norm inside the product: float32 rows of a larger residual stream, gathered by index
    h = _rand((m + 5, k), torch.float32, 9, 3.0)
    nw = _rand((k,), torch.float32, 10) + 1
    rows = torch.arange(m + 4, 4, -1, dtype=torch.int32, device=DEV)[:m].contiguous()
    for zero_centered in (False, True):
        got = cuda.norm_linear(h, nw, 1e-6, zero_centered, w, torch.float32, rows)
        _close(got, ref.norm_linear(h, nw, 1e-6, zero_centered, w, torch.float32, rows), torch.bfloat16, "norm + product")
    got = cuda.norm_linear(h[:m].contiguous(), nw, 1e-5, False, w2, None, None, True)
    _close(got, ref.norm_linear(h[:m].contiguous(), nw, 1e-5, False, w2, None, None, True), torch.bfloat16, "norm + swiglu")
    # more tokens than the kernel takes: the library path gives the same
    big = _rand((40, k), torch.float32, 11)
    _close(cuda.norm_linear(big, nw, 1e-5, False, w), ref.norm_linear(big, nw, 1e-5, False, w), torch.bfloat16, "many tokens")
    assert cuda.skinny_status() == 0  # no bounded wait inside the kernel ran out


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 17, 40, 64, 128])
@pytest.mark.parametrize("k,o", [(64, 50), (192, 320), (2048, 37), (8192, 64), (96, 40), (2048, 1000), (1024, 2048),
                                 (520, 3000), (256, 20000)])
def test_streamed_products_for_few_tokens(ops, m, k, o, monkeypatch):
    """The decode-step product kernel on the tensor cores: plain, float32 out, accumulate, SwiGLU, and with the norm
    riding along; one and several parts of K (few and many output channels), ragged edges in every direction."""
    cuda, ref = ops
    monkeypatch.setattr(cuda, "decode_products", "stream")
    # the kernel itself answers, not the path behind it: every read-out with bfloat16 activations, and the fused norm
    # where the normalised activations fit in shared memory
    assert all(cuda._stream_takes(m, o, k, False, mode) for mode in (0, 1, 2)) and cuda._stream_takes(m, 2 * o, k, False, 3)
    if m <= 16 and k <= 2048:
        assert all(cuda._stream_takes(m, o, k, True, mode) for mode in (0, 1)) and cuda._stream_takes(m, 2 * o, k, True, 3)
    x, w = _rand((m, k), torch.bfloat16, 5), _rand((o, k), torch.bfloat16, 6, 0.05)
    want = x.double() @ w.double().T
    _close(cuda.linear(x, w), want, torch.bfloat16, "bf16 out")
    _close(cuda.linear(x, w, out_dtype=torch.float32), want, torch.float32, "f32 out", k)
    res = _rand((m, o), torch.float32, 7)
    _close(cuda.linear(x, w, residual=res.clone()), res.double() + want, torch.float32, "accumulate", k)
    w2 = _rand((2 * o, k), torch.bfloat16, 8, 0.05)
    _close(cuda.linear_swiglu(x, w2), ref.linear_swiglu(x, w2), torch.bfloat16, "swiglu")
    h = _rand((m + 5, k), torch.float32, 9, 3.0)
    nw = _rand((k,), torch.float32, 10) + 1
    rows = torch.arange(m + 4, 4, -1, dtype=torch.int32, device=DEV)[:m].contiguous()
    for zero_centered in (False, True):
        got = cuda.norm_linear(h, nw, 1e-6, zero_centered, w, torch.float32, rows)
        _close(got, ref.norm_linear(h, nw, 1e-6, zero_centered, w, torch.float32, rows), torch.bfloat16, "norm + product")
    got = cuda.norm_linear(h[:m].contiguous(), nw, 1e-5, False, w, None, None)
    _close(got, ref.norm_linear(h[:m].contiguous(), nw, 1e-5, False, w, None, None), torch.bfloat16, "norm + product, bf16")
    got = cuda.norm_linear(h[:m].contiguous(), nw, 1e-5, False, w2, None, None, True)
    _close(got, ref.norm_linear(h[:m].contiguous(), nw, 1e-5, False, w2, None, None, True), torch.bfloat16, "norm + swiglu")
    # twice the same call gives the same bits: parts of K are added in a fixed order
    a, b = cuda.linear(x, w, out_dtype=torch.float32), cuda.linear(x, w, out_dtype=torch.float32)
    assert torch.equal(a, b)
    assert cuda.stream_status() == 0  # no bounded wait inside the kernel ran out


@pytest.mark.parametrize("m,k,o", [(17, 64, 48), (64, 128, 256), (100, 96, 200), (128, 2048, 320), (300, 192, 1000),
                                   (2048, 256, 512), (333, 2048, 2056), (40, 128, 333), (70, 64, 1001)])
def test_tensor_memory_products_for_prompt_portions(ops, m, k, o):
    """The one-block tcgen05 kernel (TMA in, accumulators in tensor memory, masked read-outs: the route of widths
    whose rows TMA cannot write) with its three read-outs, at sizes that leave ragged tiles in every direction."""
    cuda, ref = ops
    x, w = _rand((m, k), torch.bfloat16, 5), _rand((o, k), torch.bfloat16, 6, 0.05)
    want = x.double() @ w.double().T
    _close(cuda.block_product(x, w), want, torch.bfloat16, "bf16 out")
    _close(cuda.block_product(x, w, out_dtype=torch.float32), want, torch.float32, "f32 out", k)
    res = _rand((m, o), torch.float32, 7)
    _close(cuda.block_product(x, w, residual=res.clone()), res.double() + want, torch.float32, "accumulate", k)
    if o % 8 == 0:  # gate and up rows come by TMA in boxes of 8
        w2 = _rand((2 * o, k), torch.bfloat16, 8, 0.05)
        _close(cuda.block_product(x, w2, swiglu_out=True), ref.linear_swiglu(x, w2), torch.bfloat16, "swiglu")
    assert cuda.gemm_tcgen05_status() == 0


@pytest.mark.parametrize("m,k,o", [(17, 64, 48), (256, 128, 256), (300, 264, 520), (2048, 256, 512), (333, 2048, 2056),
                                   (1000, 1024, 1160), (130, 2048, 6144), (2048, 512, 16384), (4100, 320, 8200)])
def test_products_on_pairs_of_sms(ops, m, k, o):
    """The cta_group::2 kernel (each block of a pair stages half of a tile's channels; read-outs staged in shared memory
    and written by TMA), all four read-outs, at sizes that leave ragged tiles in every direction, more tiles than
    pairs, and tiles of every width."""
    cuda, ref = ops
    x, w = _rand((m, k), torch.bfloat16, 5), _rand((o, k), torch.bfloat16, 6, 0.05)
    want = x.double() @ w.double().T
    _close(cuda.paired_product(x, w), want, torch.bfloat16, "bf16 out")
    got = cuda.paired_product(x, w, out_dtype=torch.float32)
    assert got.dtype == torch.float32
    _close(got, want, torch.bfloat16, "f32 out")
    h = _rand((m, o), torch.float32, 7, 2.0)
    h0 = h.clone()
    assert cuda.paired_product(x, w, residual=h) is h
    _close(h, h0.double() + want, torch.bfloat16, "added into the residual stream")
    w2 = _rand((2 * o, k), torch.bfloat16, 8, 0.05)
    _close(cuda.paired_product(x, w2, swiglu_out=True), ref.linear_swiglu(x, w2), torch.bfloat16, "swiglu")
    assert cuda.gemm_pair_status() == 0


@pytest.mark.parametrize("m,k,o", [(17, 64, 48), (64, 2048, 6144), (33, 264, 520), (128, 8192, 2048), (100, 200, 2056),
                                   (64, 2048, 65536), (20, 1024, 40), (96, 704, 1160), (48, 128, 40000), (64, 8192, 2048),
                                   (33, 4096, 1000), (70, 6912, 1536)])
def test_products_of_few_rows_stream_the_weights(ops, m, k, o):
    """The one-block tcgen05 kernel for 17 to 128 tokens (tiles as wide as gives every SM one; token rows past the batch
    are never loaded), all four read-outs, at inner sizes that are and are not multiples of 64 (one copy per stage, a
    copy per step), widths that leave ragged tiles, more tiles than SMs, and one narrow tile."""
    cuda, ref = ops
    x, w = _rand((m, k), torch.bfloat16, 5), _rand((o, k), torch.bfloat16, 6, 0.05)
    want = x.double() @ w.double().T
    _close(cuda.rows_product(x, w), want, torch.bfloat16, "bf16 out")
    got = cuda.rows_product(x, w, out_dtype=torch.float32)
    assert got.dtype == torch.float32
    _close(got, want, torch.bfloat16, "f32 out")
    h = _rand((m, o), torch.float32, 7, 2.0)
    h0 = h.clone()
    assert cuda.rows_product(x, w, residual=h) is h
    _close(h, h0.double() + want, torch.bfloat16, "added into the residual stream")
    if o <= 20000:
        w2 = _rand((2 * o, k), torch.bfloat16, 8, 0.05)
        _close(cuda.rows_product(x, w2, swiglu_out=True), ref.linear_swiglu(x, w2), torch.bfloat16, "swiglu")
    assert cuda.gemm_rows_status() == 0
    with pytest.raises(ValueError, match="at most 128"):
        cuda.rows_product(_rand((129, k), torch.bfloat16, 9), w)


@pytest.mark.parametrize("m,c,f,v,taps", [(1, 128, 320, 500, 3), (8, 256, 9216, 1000, 3), (5, 192, 448, 777, 4),
                                         (13, 128, 6912, 300, 2), (16, 2048, 8192, 4096, 3), (3, 64, 64, 40, 5)])
def test_decode_chain_runs_a_layer_as_one_launch(ops, m, c, f, v, taps, monkeypatch):
    """Embedding, norm + in projection, short convolution with its state, out projection into the residual stream,
    norm + gate/up + SwiGLU, down projection (inner sizes up to 9,216: more than the two activation segments that
    shared memory holds, so they roll), norm of gathered rows + head: recorded into one chain and run as one launch,
    against the same functions of the plain module, with padding tokens, and twice in a row (the barrier word
    resets itself)."""
    cuda, ref = ops
    monkeypatch.setattr(cuda, "decode_chain", "1")
    bf = torch.bfloat16
    table = _rand((v, c), bf, 1, 0.5)
    w_in, w_out = _rand((3 * c, c), bf, 2, c ** -0.5), _rand((c, c), bf, 3, c ** -0.5)
    w_gu, w_down = _rand((2 * f, c), bf, 4, c ** -0.5), _rand((c, f), bf, 5, f ** -0.5)
    n1, n2, n3 = (_rand((c,), torch.float32, 6 + i) * 0.2 + 1 for i in range(3))
    conv_w, conv_b = _rand((c, taps), torch.float32, 9), _rand((c,), torch.float32, 10)
    ids = torch.randint(0, v, (m,), generator=torch.Generator().manual_seed(11), dtype=torch.int32).to(DEV)
    live = max(1, m - 2) if m > 2 else m  # the last tokens are padding
    seq = torch.tensor(list(range(live)) + [-1] * (m - live), dtype=torch.int32, device=DEV)
    slots = torch.tensor([(3 * r + 1) % 20 for r in range(live)] + [-1] * (m - live), dtype=torch.int32, device=DEV)
    rows = torch.tensor(list(range(live))[::-1], dtype=torch.int32, device=DEV)
    state0 = _rand((20, taps - 1, c), torch.float32, 12)

    def layer(o, state):
        h = o.embedding(ids, table)
        bcx = o.norm_linear(h, n1, 1e-5, False, w_in)
        y = o.short_conv(bcx, conv_w, conv_b, state, None, seq, slots, decode_only=True) if o is cuda else \
            ref.short_conv(bcx, conv_w, conv_b, state, torch.arange(live + 1, dtype=torch.int32, device=DEV), seq, slots[:live])
        h = o.linear(y, w_out, residual=h)
        act = o.norm_linear(h, n2, 1e-5, False, w_gu, swiglu_out=True)
        h = o.linear(act, w_down, residual=h)
        return h, o.norm_linear(h, n3, 1e-6, True, table, out_dtype=torch.float32, rows=rows)

    s_ref = state0.clone()
    h_want, logits_want = layer(ref, s_ref)
    for _ in range(2):
        s_got = state0.clone()
        before = cuda.launch_count
        assert cuda.chain_begin(m)
        h_got, logits_got = layer(cuda, s_got)
        assert cuda.launch_count == before  # nothing has run yet
        cuda.chain_end()
        assert cuda.launch_count == before + 1
        _close(h_got[:live], h_want[:live], bf, "residual stream")
        _close(logits_got, logits_want, bf, "logits of gathered rows")
        _close(s_got, s_ref, bf, "conv state")  # built from activations that were rounded to bfloat16
    assert cuda.chain_status() == 0
    # an operation that cannot join (a float32 product) makes the pending ones run first
    assert cuda.chain_begin(m)
    h = cuda.embedding(ids, table)
    before = cuda.launch_count
    cuda.rmsnorm(h, n1, 1e-5, False, torch.float32)
    assert cuda.launch_count == before + 2
    cuda.chain_end()


@pytest.mark.parametrize("m,c,k,taps,bias", [(8, 2048, 2048, 3, False), (5, 72, 128, 4, True), (13, 1024, 512, 2, False),
                                             (1, 64, 64, 3, True), (16, 200, 320, 5, False)])
def test_in_projection_and_short_conv_as_one_kernel(ops, m, c, k, taps, bias):
    """A decode step's RMSNorm, in projection and gated short convolution in one launch, against the product and the
    convolution kernel one after the other: the read-out rounds the projection to bfloat16 as the product would and
    then does the convolution's arithmetic in its order, so the two differ only where the product by itself cut K into
    parts (another order of the float32 sum) and a value lay on a rounding boundary: fewer than one element in a hundred,
    by one step of bfloat16. State included; padding tokens give zeros and touch no state; ``write=False`` leaves the
    state as it was."""
    cuda, ref = ops
    h = _rand((m, k), torch.float32, 1, 2.0)
    norm_w = _rand((k,), torch.float32, 2) * 0.2 + 1
    w_in = _rand((3 * c, k), torch.bfloat16, 3, k ** -0.5)
    conv_w, conv_b = _rand((c, taps), torch.float32, 4), (_rand((c,), torch.float32, 5) if bias else None)
    live = max(1, m - 2) if m > 2 else m
    seq = torch.tensor(list(range(live)) + [-1] * (m - live), dtype=torch.int32, device=DEV)
    slots = torch.tensor([(5 * r + 2) % 24 for r in range(live)], dtype=torch.int32, device=DEV)
    state0 = _rand((24, taps - 1, c), torch.float32, 6)
    for write in (True, False):
        s_two, s_one = state0.clone(), state0.clone()
        bcx = cuda.norm_linear(h, norm_w, 1e-5, False, w_in)
        want = cuda.short_conv(bcx, conv_w, conv_b, s_two, None, seq, slots, decode_only=True, write=write)
        before = cuda.launch_count
        got = cuda.norm_linear_short_conv(h, norm_w, 1e-5, False, w_in, conv_w, conv_b, s_one, seq, slots, write=write)
        assert got is not None and cuda.launch_count == before + 1
        _close(got, want, torch.bfloat16, "output")
        _close(s_one, s_two, torch.bfloat16, "state")
        assert (got != want).float().mean() < 0.01 and (s_one != s_two).float().mean() < 0.01
        assert torch.equal(s_one, state0) != write
        assert not got[live:].any()
    assert cuda.skinny_status() == 0
    assert cuda.norm_linear_short_conv(_rand((17, k), torch.float32, 7), norm_w, 1e-5, False, w_in, conv_w, conv_b, state0, seq,
                                       slots) is None  # more tokens than the decode kernels take: the caller runs the two


def test_short_conv_decode_kernel_equals_the_general_one(ops):
    cuda, ref = ops
    c, taps = 72, 4
    seq = torch.tensor([0, 1, 2, -1], dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, 1, 2, 3, 3], dtype=torch.int32, device=DEV)
    slots = torch.tensor([5, 0, 2, -1], dtype=torch.int32, device=DEV)
    for dtype in DTYPES:
        bcx = _rand((4, 3 * c), dtype, 10)
        w, b = _rand((c, taps), torch.float32, 11), _rand((c,), torch.float32, 12)
        state = _rand((8, taps - 1, c), torch.float32, 13)
        s1, s2 = state.clone(), state.clone()
        got = cuda.short_conv(bcx, w, b, s1, cu, seq, slots, decode_only=True)
        want = cuda.short_conv(bcx, w, b, s2, cu, seq, slots)
        assert torch.equal(got, want) and torch.equal(s1, s2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_kv_store_of_separate_rows(ops, dtype):
    """Keys rewritten by a position encoding of its own (a fresh tensor) and values still inside the qkv buffer:
    rows of different pitch go to the same pages."""
    cuda, ref = ops
    kh, d, page, n = 2, 32, 4, 9
    qkv = _rand((n, (3 + 2 * kh) * d), dtype, 40)
    k = _rand((n, kh * d), dtype, 41)
    v = qkv[:, (3 + kh) * d:]
    table = torch.tensor([[5, 2, 7], [1, -1, -1]], dtype=torch.int32, device=DEV)
    seq = torch.tensor([0] * 6 + [1, 1, -1], dtype=torch.int32, device=DEV)
    pos = torch.tensor([3, 4, 5, 6, 7, 8, 0, 1, 0], dtype=torch.int32, device=DEV)
    pools = [_rand((8, kh, page, d), dtype, 42 + i) for i in range(4)]
    pools[2].copy_(pools[0]), pools[3].copy_(pools[1])
    cuda.kv_store(k, v, pools[0], pools[1], table, seq, pos, page)
    ref.kv_store(k, v, pools[2], pools[3], table, seq, pos, page)
    assert torch.equal(pools[0], pools[2]) and torch.equal(pools[1], pools[3])


def _batch(lengths, pad=0):
    """cu_seqlens, seq_of_token, for requests of the given lengths, plus ``pad`` padding tokens."""
    cu = [0]
    seq = []
    for r, n in enumerate(lengths):
        cu.append(cu[-1] + n)
        seq += [r] * n
    seq += [-1] * pad
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return t(cu), t(seq)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,bias", [(2, False), (3, False), (4, True), (7, True)])
def test_short_conv(ops, dtype, taps, bias):
    cuda, ref = ops
    c = 72
    lengths = [5, 1, 0, 2, 9, 1]
    cu, seq = _batch(lengths, pad=2)
    n = sum(lengths) + 2
    slots = torch.tensor([3, 0, 5, 6, 1, -1], dtype=torch.int32, device=DEV)
    bcx = _rand((n, 3 * c), dtype, 10)
    w = _rand((c, taps), torch.float32, 11)
    b = _rand((c,), torch.float32, 12) if bias else None
    state = _rand((8, taps - 1, c), torch.float32, 13)
    s1, s2 = state.clone(), state.clone()
    got = cuda.short_conv(bcx, w, b, s1, cu, seq, slots)
    want = ref.short_conv(bcx, w, b, s2, cu, seq, slots)
    _close(got, want, dtype, "output")
    _close(s1, s2, torch.float32, "state")
    for untouched in (2, 4, 5, 7):  # slots of no live request, and of the request with no tokens
        assert torch.equal(s1[untouched], state[untouched])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,bias", [(2, True), (3, False), (4, True), (5, False)])
def test_short_conv_of_prompt_portions(ops, dtype, taps, bias):
    """Many tokens: the sliding-window kernel (2 to 4 taps). Requests start and end inside a thread's run of
    tokens, one has a single token, one is shorter than the window, and padding follows."""
    cuda, ref = ops
    c = 136
    lengths = [130, 1, 3, 0, 77, 2, 61, 9]
    cu, seq = _batch(lengths, pad=5)
    n = sum(lengths) + 5
    slots = torch.tensor([3, 0, 5, 6, 1, 7, -1, 2], dtype=torch.int32, device=DEV)
    bcx = _rand((n, 3 * c), dtype, 10)
    w = _rand((c, taps), torch.float32, 11)
    b = _rand((c,), torch.float32, 12) if bias else None
    state = _rand((8, taps - 1, c), torch.float32, 13)
    s1, s2 = state.clone(), state.clone()
    got = cuda.short_conv(bcx, w, b, s1, cu, seq, slots)
    want = ref.short_conv(bcx, w, b, s2, cu, seq, slots)
    _close(got, want, dtype, "output")
    _close(s1, s2, torch.float32, "state")
    assert torch.equal(s1[4], state[4]) and torch.equal(s1[6], state[6])  # no live request, no tokens


def test_rope_tables(ops):
    cuda, ref = ops
    pos = torch.tensor([0, 1, 77, 4095, 131071], dtype=torch.int32, device=DEV)
    for theta, rot in ((1e4, 16), (1e6, 64), (5e5, 48)):
        inv = (torch.tensor(theta, dtype=torch.float64) ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).to(DEV)
        c1, s1 = cuda.rope_tables(pos, inv)
        c2, s2 = ref.rope_tables(pos, inv)
        assert (c1 - c2).abs().max() <= 1.2e-7 and (s1 - s2).abs().max() <= 1.2e-7


def _pools(pages, kh, page, d, dtype, seed):
    return _rand((pages, kh, page, d), dtype, seed), _rand((pages, kh, page, d), dtype, seed + 1)


def _tables(contexts, page, pages, seed, max_blocks=None):
    """A block table whose pages are a random permutation: neighbouring positions lie in far pages."""
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(pages, generator=g).tolist()
    need = [-(-c // page) for c in contexts]
    max_blocks = max_blocks or max(need) + 1
    bt = torch.full((len(contexts), max_blocks), -1, dtype=torch.int32)
    for r, n in enumerate(need):
        for b in range(n):
            bt[r, b] = perm.pop()
    return bt.to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("h,kh,d,rot,page", [(6, 2, 48, 32, 8), (4, 4, 16, 16, 16), (8, 1, 128, 128, 64), (3, 1, 256, 64, 8)])
def test_qk_norm_rope_store(ops, dtype, h, kh, d, rot, page):
    cuda, ref = ops
    lengths, starts = [3, 1, 6], [5, 40, 0]
    cu, seq = _batch(lengths, pad=1)
    pos = torch.tensor([s + j for s, n in zip(starts, lengths) for j in range(n)] + [0], dtype=torch.int32, device=DEV)
    n = pos.numel()
    bt = _tables([s + l for s, l in zip(starts, lengths)], page, 40, 3)
    qkv = _rand((n, (h + 2 * kh) * d), dtype, 20)
    qw, kw = _rand((d,), torch.float32, 21) + 1, _rand((d,), torch.float32, 22) + 1
    inv = (torch.tensor(1e4, dtype=torch.float64) ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).to(DEV)
    cos, sin = ref.rope_tables(pos, inv)
    for norm, rope in ((True, True), (False, True), (True, False)):
        k1, v1 = _pools(40, kh, page, d, dtype, 30)
        k2, v2 = k1.clone(), v1.clone()
        a, b = qkv.clone(), qkv.clone()
        args = (h, kh, d, qw if norm else None, kw if norm else None, 1e-5, False, cos if rope else None, sin if rope else None)
        q1 = cuda.qk_norm_rope_store(a, *args, k1, v1, bt, seq, pos, page)
        q2 = ref.qk_norm_rope_store(b, *args, k2, v2, bt, seq, pos, page)
        _close(q1, q2, dtype, "q")
        _close(a[:-1], b[:-1], dtype, "k in place")
        _close(k1, k2, dtype, "key pages")
        assert torch.equal(v1, v2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("h,kh,d,page,window", [
    (4, 2, 16, 16, None), (3, 1, 32, 8, None), (8, 8, 64, 64, None), (6, 2, 48, 8, 37), (16, 2, 128, 32, None),
    (5, 1, 80, 16, 100), (32, 8, 64, 64, None), (7, 7, 256, 8, None),
])
def test_paged_attention(ops, dtype, h, kh, d, page, window):
    cuda, ref = ops
    # a prompt portion that starts mid-page, two decoded tokens with long and short contexts, a first token
    lengths, starts = [37, 1, 1, 1, 70], [29, 333, 64, 0, 0]
    cu, seq = _batch(lengths, pad=2)
    pos = torch.tensor([s + j for s, n in zip(starts, lengths) for j in range(n)] + [0, 0], dtype=torch.int32, device=DEV)
    contexts = [s + l for s, l in zip(starts, lengths)]
    pages = sum(-(-c // page) for c in contexts) + 3
    bt = _tables(contexts, page, pages, 4)
    k, v = _pools(pages, kh, page, d, dtype, 40)
    q = _rand((pos.numel(), h * d), dtype, 42)
    scale = d ** -0.5
    want = ref.paged_attention(q, k, v, bt, seq, pos, scale, window, page)
    got = cuda.paged_attention(q, k, v, bt, seq, pos, scale, window, page)
    _close(got, want, dtype, "mixed batch")


class _Prompt:
    decode_only = False

    def __init__(self, cu, lengths):
        self.cu_seqlens = cu
        self.query_lens = tuple(lengths)
        self.memo = {}
        self.max_context = 0


@pytest.mark.parametrize("h,kh,d,page,window", [
    (4, 2, 16, 16, None), (3, 1, 32, 8, None), (8, 2, 64, 64, None), (6, 2, 64, 8, 37), (16, 2, 128, 32, None),
    (5, 1, 128, 16, 100), (32, 8, 64, 64, 70), (2, 2, 16, 4, None), (4, 1, 64, 128, None), (6, 3, 64, 256, 200),
    (2, 2, 64, 64, 129),
])
@pytest.mark.parametrize("kernel", ["tcgen05", "mma"])
def test_prompt_attention_on_tensor_cores(ops, h, kh, d, page, window, kernel, monkeypatch):
    """Portions that start mid-page and mid-tile, of 1 to 300 tokens, beside decoded tokens with long contexts; with
    the tensor-memory kernel (head size 64 and pages of 64 keys or more; the others fall to mma.sync) and with the
    mma.sync kernel. What the pages hold past the end of a request is poisoned: it must not be looked at."""
    cuda, ref = ops
    monkeypatch.setattr(cuda, "prompt_attention", kernel)
    dtype = torch.bfloat16
    lengths, starts = [37, 1, 200, 1, 64, 65, 0, 130, 300, 128], [29, 333, 0, 64, 64, 100, 5, 700, 100, 128]
    cu, seq = _batch(lengths)
    pos = torch.tensor([s + j for s, n in zip(starts, lengths) for j in range(n)], dtype=torch.int32, device=DEV)
    contexts = [s + l for s, l in zip(starts, lengths)]
    pages = sum(-(-c // page) for c in contexts) + 3
    bt = _tables(contexts, page, pages, 4)
    k, v = _pools(pages, kh, page, d, dtype, 40)
    for r, context in enumerate(contexts):  # past the end of every request: not a number
        last = int(bt[r, (context - 1) // page]) if context else -1
        if last >= 0 and context % page:
            k[last, :, context % page:] = float("nan")
            v[last, :, context % page:] = float("nan")
    q = _rand((pos.numel(), h * d), dtype, 42)
    scale = d ** -0.5
    want = ref.paged_attention(q, k, v, bt, seq, pos, scale, window, page)
    got = cuda.paged_attention(q, k, v, bt, seq, pos, scale, window, page, _Prompt(cu, lengths))
    _close(got, want, dtype, "tensor-core prompt attention")
    assert cuda.prefill_attention_tc_status() == 0
    general = cuda.paged_attention(q, k, v, bt, seq, pos, scale, window, page)
    _close(general, want, dtype, "general kernel")


@pytest.mark.parametrize("h,kh,d,page,window", [(8, 2, 64, 64, None), (4, 2, 16, 16, 300), (6, 1, 128, 32, None), (32, 8, 64, 64, None)])
@pytest.mark.parametrize("mode", ["split", "tiles"])
def test_decoded_tokens_at_the_front_of_a_mixed_step(ops, h, kh, d, page, window, mode, monkeypatch):
    """Five decoded tokens with contexts of 1 to 2,000 keys, then portions of 130, 1 and 70 tokens: with "split" the
    five go to the split-key kernel and the prompt kernels start at the sixth request; with "tiles"
    everything runs as query tiles. Both write every row of the one output, and both are the plain attention."""
    cuda, ref = ops
    monkeypatch.setattr(cuda, "mixed_attention", mode)
    dtype = torch.bfloat16
    lengths, starts = [1, 1, 1, 1, 1, 130, 1, 70], [1999, 0, 63, 64, 700, 50, 300, 0]
    cu, seq = _batch(lengths)
    pos = torch.tensor([s + j for s, n in zip(starts, lengths) for j in range(n)], dtype=torch.int32, device=DEV)
    contexts = [s + l for s, l in zip(starts, lengths)]
    pages = sum(-(-c // page) for c in contexts) + 3
    bt = _tables(contexts, page, pages, 14)
    k, v = _pools(pages, kh, page, d, dtype, 70)
    q = _rand((pos.numel(), h * d), dtype, 72)
    ctx = _Prompt(cu, lengths)
    ctx.max_context = max(contexts)
    before = cuda.launch_count
    got = cuda.paged_attention(q, k, v, bt, seq, pos, d ** -0.5, window, page, ctx)
    # split keys, their merge (a kernel of its own unless the TMA-fed kernel merges in its clusters), the prompt tiles
    merged = d == 64 and page % 64 == 0
    assert cuda.launch_count - before == ((2 if merged else 3) if mode == "split" else 1)
    _close(got, ref.paged_attention(q, k, v, bt, seq, pos, d ** -0.5, window, page), dtype, mode)
    assert cuda.decode_attention_status() == 0 and cuda.prefill_attention_tc_status() == 0


@pytest.mark.parametrize("kernel", ["tcgen05", "mma"])
def test_prompt_attention_when_the_maximum_keeps_growing(ops, kernel, monkeypatch):
    """Random scores find their maximum in the first tile of keys. Here one channel of the keys grows with the
    position, so the row maximum of the queries that look along it rises a little with every tile (the output so far
    is rescaled on some tiles and left on others), falls for the queries that look the other way, and two keys far
    apart stand out by a wide margin."""
    cuda, ref = ops
    monkeypatch.setattr(cuda, "prompt_attention", kernel)
    dtype, h, kh, d, page = torch.bfloat16, 4, 2, 64, 64
    lengths, starts = [520, 300, 1], [200, 0, 900]
    cu, seq = _batch(lengths)
    pos = torch.tensor([s + j for s, n in zip(starts, lengths) for j in range(n)], dtype=torch.int32, device=DEV)
    contexts = [s + l for s, l in zip(starts, lengths)]
    pages = sum(-(-c // page) for c in contexts) + 2
    bt = _tables(contexts, page, pages, 9)
    k, v = _pools(pages, kh, page, d, dtype, 60)
    q = _rand((pos.numel(), h * d), dtype, 62)
    q.view(-1, h, d)[:, :, 0] = torch.where(torch.arange(pos.numel(), device=DEV) % 3 == 0, -6.0, 6.0)[:, None].to(dtype)
    tables = bt.cpu()
    for r, context in enumerate(contexts):
        where = torch.arange(context)
        value = where / 30.0 + 25.0 * ((where == 310) | (where == 650))
        k[tables[r, where // page].long().to(DEV), :, (where % page).to(DEV), 0] = value.to(DEV, dtype)[:, None]
    scale = d ** -0.5
    want = ref.paged_attention(q, k, v, bt, seq, pos, scale, None, page)
    got = cuda.paged_attention(q, k, v, bt, seq, pos, scale, None, page, _Prompt(cu, lengths))
    _close(got, want, dtype, "prompt attention under a rising maximum")
    assert cuda.prefill_attention_tc_status() == 0


class _Decode:
    decode_only = True

    def __init__(self, max_context):
        self.max_context = max_context


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("h,kh,d,page,window", [
    (4, 2, 16, 16, None), (3, 1, 32, 8, None), (32, 8, 64, 64, None), (6, 1, 48, 8, 300), (16, 2, 128, 32, None),
    (24, 1, 64, 16, None), (5, 5, 256, 64, None), (8, 2, 64, 128, 300), (4, 4, 64, 256, None), (32, 8, 64, 64, 1000),
])
@pytest.mark.parametrize("items", ["auto", "1"])
def test_paged_attention_decode_split(ops, dtype, h, kh, d, page, window, items, monkeypatch):
    """Split-key decode attention; head size 64 with pages of 64 keys or more takes the TMA-fed kernels in bfloat16:
    a block per (token, KV head, key part), or (items "1") a fixed number of blocks that walk those items.
    What the pages hold past the end of a request is poisoned: it must not be looked at."""
    cuda, ref = ops
    monkeypatch.setattr(cuda, "decode_items", items)
    contexts = [1, 2, 33, 700, 1500, 257, 64, 128]
    cu, seq = _batch([1] * len(contexts), pad=2)
    pos = torch.tensor([c - 1 for c in contexts] + [0, 0], dtype=torch.int32, device=DEV)
    pages = sum(-(-c // page) for c in contexts) + 3
    bt = _tables(contexts, page, pages, 6)
    k, v = _pools(pages, kh, page, d, dtype, 50)
    for r, context in enumerate(contexts):
        if context % page:
            last = int(bt[r, (context - 1) // page])
            k[last, :, context % page:] = float("nan")
            v[last, :, context % page:] = float("nan")
    q = _rand((pos.numel(), h * d), dtype, 52)
    scale = d ** -0.5
    want = ref.paged_attention(q, k, v, bt, seq, pos, scale, window, page)
    got = cuda.paged_attention(q, k, v, bt, seq, pos, scale, window, page, _Decode(max(contexts)))
    _close(got, want, dtype, "split decode")
    assert cuda.decode_attention_status() == 0
    assert torch.equal(got[-2:], torch.zeros_like(got[-2:]))


@pytest.mark.parametrize("h,kh,page,window,rot,norm", [
    (32, 8, 64, None, 64, True), (24, 1, 128, 300, 32, True), (4, 4, 256, None, 64, False), (8, 2, 64, 1000, 16, True),
    (6, 2, 64, None, 0, True),
])
@pytest.mark.parametrize("items", ["auto", "1"])
def test_decode_attention_from_the_qkv_product(ops, h, kh, page, window, rot, norm, items, monkeypatch):
    """Norm and rotation of q and k, the write into the pages and split-key attention as one kernel, against the two
    kernels that do the same: every bit of the output and of the pages. The page rows that the step's own tokens go to
    are poisoned beforehand, so a block that attended to what its load found there instead of the token would show;
    24 heads over one key/value head make two tiles of query rows, of which only the first writes the pages. With
    items "1" both sides run on the kernel whose blocks walk the items."""
    cuda, ref = ops
    monkeypatch.setattr(cuda, "decode_items", items)
    d, dtype = 64, torch.bfloat16
    contexts = [1, 2, 33, 700, 1500, 257, 64, 128, 65]
    cu, seq = _batch([1] * len(contexts), pad=2)
    pos = torch.tensor([c - 1 for c in contexts] + [0, 0], dtype=torch.int32, device=DEV)
    n = pos.numel()
    pages = sum(-(-c // page) for c in contexts) + 3
    bt = _tables(contexts, page, pages, 6)
    k0, v0 = _pools(pages, kh, page, d, dtype, 50)
    for r, context in enumerate(contexts):
        last = int(bt[r, (context - 1) // page])
        k0[last, :, (context - 1) % page:] = float("nan")
        v0[last, :, (context - 1) % page:] = float("nan")
    qkv = _rand((n, (h + 2 * kh) * d), dtype, 20)
    qw, kw = (_rand((d,), torch.float32, 21) + 1, _rand((d,), torch.float32, 22) + 1) if norm else (None, None)
    cos = sin = None
    if rot:
        inv = (torch.tensor(1e4, dtype=torch.float64) ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).to(DEV)
        cos, sin = ref.rope_tables(pos, inv)
    scale, step = d ** -0.5, _Decode(max(contexts))
    prep = (h, kh, d, qw, kw, 1e-5, False, cos, sin)
    k1, v1, k2, v2 = k0.clone(), v0.clone(), k0.clone(), v0.clone()
    q = cuda.qk_norm_rope_store(qkv.clone(), *prep, k1, v1, bt, seq, pos, page)
    want = cuda.paged_attention(q, k1, v1, bt, seq, pos, scale, window, page, step)
    got = cuda.qkv_decode_attention(qkv.clone(), *prep, k2, v2, bt, seq, pos, scale, window, page, step)
    assert got is not None and cuda.decode_attention_status() == 0
    assert torch.equal(got, want)
    live = torch.ones_like(k1, dtype=torch.bool)
    for r, context in enumerate(contexts):  # (what lies past a request's end stays poisoned)
        live[int(bt[r, (context - 1) // page]), :, context % page if context % page else page:] = False
    assert torch.equal(k1[live], k2[live]) and torch.equal(v1[live], v2[live])
    assert not torch.isnan(k2[live]).any()
    _close(got, ref.paged_attention(q, k1, v1, bt, seq, pos, scale, window, page), dtype, "against the plain statement")
    # a layer that only reads the pages: nothing written, the pages attended as they are
    q = cuda.qk_norm_rope_store(qkv.clone(), *prep, None, None, bt, seq, pos, page)
    want = cuda.paged_attention(q, k1, v1, bt, seq, pos, scale, window, page, step)
    before = k1.clone()
    got = cuda.qkv_decode_attention(qkv.clone(), *prep, k1, v1, bt, seq, pos, scale, window, page, step, write=False)
    assert torch.equal(got, want) and torch.equal(k1[live], before[live])


def test_decode_attention_with_more_items_than_blocks(ops, monkeypatch):
    """66 requests of 8 key/value heads with contexts from 1 to 3,000 keys: more (token, KV head, key part) items than
    blocks fit the GPU, so the blocks walk them (two rounds, the ring of tiles running on from item to item, empty
    parts and padding tokens among them); then 130 requests with the walking kernel asked for (four rounds)."""
    cuda, ref = ops
    h, kh, d, page, dtype = 32, 8, 64, 64, torch.bfloat16
    g = torch.Generator().manual_seed(5)
    for extra, items in ((60, "auto"), (124, "1")):
        monkeypatch.setattr(cuda, "decode_items", items)
        contexts = [1, 2, 63, 64, 65, 3000] + torch.randint(1, 2500, (extra,), generator=g).tolist()
        cu, seq = _batch([1] * len(contexts), pad=3)
        pos = torch.tensor([c - 1 for c in contexts] + [0, 0, 0], dtype=torch.int32, device=DEV)
        pages = sum(-(-c // page) for c in contexts) + 3
        bt = _tables(contexts, page, pages, 6)
        k, v = _pools(pages, kh, page, d, dtype, 50)
        for r, context in enumerate(contexts):
            if context % page:
                last = int(bt[r, (context - 1) // page])
                k[last, :, context % page:] = float("nan")
                v[last, :, context % page:] = float("nan")
        q = _rand((pos.numel(), h * d), dtype, 52)
        step = _Decode(max(contexts))
        assert cuda.decode_plan(len(contexts) + 3, h, kh, d, page, step.max_context, dtype)[1]
        want = ref.paged_attention(q, k, v, bt, seq, pos, d ** -0.5, None, page)
        got = cuda.paged_attention(q, k, v, bt, seq, pos, d ** -0.5, None, page, step)
        _close(got, want, dtype, "walking the items")
        assert cuda.decode_attention_status() == 0
        assert torch.equal(got[-3:], torch.zeros_like(got[-3:]))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key(ops, dtype):
    """One key among a thousand, far back and in a page of its own, is made to dominate: random values
    would hide a kernel that drops it."""
    cuda, ref = ops
    h, kh, d, page = 4, 2, 64, 16
    ctx, far = 1000, 131
    cu, seq = _batch([1, 5])
    pos = torch.tensor([ctx - 1] + list(range(ctx - 5, ctx)), dtype=torch.int32, device=DEV)
    pages = 2 * (-(-ctx // page)) + 2
    bt = _tables([ctx, ctx], page, pages, 8)
    k, v = _pools(pages, kh, page, d, dtype, 60)
    q = _rand((6, h * d), dtype, 62)
    for r in range(2):
        pg, off = int(bt[r, far // page]), far % page
        for kvh in range(kh):
            qh = q[0 if r == 0 else 3, kvh * 2 * d : kvh * 2 * d + d].float()
            k[pg, kvh, off] = (qh / qh.norm() * 40).to(dtype)
            v[pg, kvh, off] = 7.0
    scale = d ** -0.5
    want = ref.paged_attention(q, k, v, bt, seq, pos, scale, None, page)
    assert want[0, :d].float().mean() > 6  # the far key does dominate
    _close(cuda.paged_attention(q, k, v, bt, seq, pos, scale, None, page), want, dtype, "generic")
    one = cuda.paged_attention(q[:1].contiguous(), k, v, bt[:1].contiguous(), seq[:1], pos[:1], scale, None, page, _Decode(ctx))
    _close(one, want[:1], dtype, "split decode")


def test_argmax_ties_go_to_the_lowest_index(ops):
    cuda, ref = ops
    x = _rand((5, 1000), torch.float32, 70)
    x[0, 17] = x[0, 900] = 50.0
    x[1, 999] = 60.0
    x[2, 0] = x[2, 1] = 70.0
    x[3] = 1.0
    assert cuda.argmax(x).tolist() == ref.argmax(x).tolist() == [17, 999, 0, 0, int(x[4].argmax())]
    big = _rand((3, 65536 + 3), torch.float32, 71)
    assert cuda.argmax(big).tolist() == big.argmax(dim=-1).tolist()


def test_sample(ops):
    cuda, ref = ops
    v = 777
    logits = _rand((6, v), torch.float32, 80, 2.0)
    t = lambda vals, dt: torch.tensor(vals, dtype=dt, device=DEV)
    temp = t([0.0, 1.0, 0.7, 1.3, 1.0, 1.0], torch.float32)
    top_k = t([0, 0, 5, 0, 1, 50], torch.int32)
    top_p = t([1.0, 1.0, 1.0, 0.6, 1.0, 0.9], torch.float32)
    for seed in range(20):
        u = torch.rand(6, generator=torch.Generator().manual_seed(seed)).to(DEV)
        got, want = cuda.sample(logits, temp, top_k, top_p, u), ref.sample(logits, temp, top_k, top_p, u)
        assert got.tolist() == want.tolist(), (seed, got.tolist(), want.tolist())
    assert cuda.sample(logits, temp, top_k, top_p, u)[0] == logits[0].argmax()
    assert cuda.sample(logits, temp, top_k, top_p, u)[4] == logits[4].argmax()
    # equal logits at the cut: top-k keeps exactly k, the lower ids of the equals; top-p cuts inside a run of equals
    tied = torch.full((4, 64), -3.0, device=DEV)
    tied[:, [5, 9, 20, 33, 40, 41, 50]] = torch.tensor([2.0, 1.0, 1.0, 1.0, 1.0, 0.5, 1.0], device=DEV)
    temp4, k4 = t([1.0, 1.0, 0.5, 1.0], torch.float32), t([3, 4, 0, 64], torch.int32)
    p4 = t([1.0, 1.0, 0.7, 0.7], torch.float32)
    seen = [set() for _ in range(4)]
    for seed in range(200):
        u = torch.rand(4, generator=torch.Generator().manual_seed(100 + seed)).to(DEV)
        got, want = cuda.sample(tied, temp4, k4, p4, u), ref.sample(tied, temp4, k4, p4, u)
        assert got.tolist() == want.tolist(), (seed, got.tolist(), want.tolist())
        for r in range(4):
            seen[r].add(int(got[r]))
    assert seen[0] == {5, 9, 20} and seen[1] == {5, 9, 20, 33}, seen  # not every token equal to the k-th
    assert seen[2] == {5, 9, 20} and seen[3] == {5, 9, 20, 33, 40}, seen  # top-p stops inside the run of equals
    # frequencies follow softmax(logits / T)
    small = torch.tensor([[0.0, 1.0, 2.0, -1.0]], device=DEV).repeat(4096, 1)
    u = torch.rand(4096, generator=torch.Generator().manual_seed(1)).to(DEV)
    ones = torch.ones(4096, device=DEV)
    picks = cuda.sample(small, ones * 0.8, torch.zeros(4096, dtype=torch.int32, device=DEV), ones, u)
    freq = torch.bincount(picks.long(), minlength=4).float() / 4096
    want = torch.softmax(small[0] / 0.8, dim=-1)
    assert (freq - want).abs().max() < 0.03


@pytest.mark.parametrize("m,v,w", [(1, 300, 5), (5, 1000, 17), (3, 65536, 96), (2, 4099, 1)])
def test_adjust_logits(ops, m, v, w):
    """Softcap, then the repetition penalty once per token of the history (tokens repeated in the history, empty
    places, rows without either)."""
    cuda, ref = ops
    logits = _rand((m, v), torch.float32, 31, 4.0)
    g = torch.Generator().manual_seed(32)
    history = torch.randint(0, v, (m, w), generator=g, dtype=torch.int32)
    history[:, w // 2:] = history[:, : w - w // 2].clone()  # every token of the first half again
    if w > 2:
        history[0, -1] = -1
    history = history.to(DEV)
    softcap = torch.tensor([0.0, 15.0, 3.0, 0.0, 7.5][:m], dtype=torch.float32, device=DEV)
    penalty = torch.tensor([2.4, 1.0, 1.3, 0.5, 2.4][:m], dtype=torch.float32, device=DEV)
    want = ref.adjust_logits(logits.clone(), softcap, penalty, history)
    got = cuda.adjust_logits(logits.clone(), softcap, penalty, history)
    assert torch.allclose(got, want, rtol=1e-6, atol=1e-6), (got - want).abs().max()
    # and what it is for: the argmax moves away from a penalised token
    row = torch.zeros((1, v), dtype=torch.float32, device=DEV)
    row[0, 7], row[0, 9] = 2.0, 1.5
    seen = torch.tensor([[7]], dtype=torch.int32, device=DEV)
    one, none = torch.tensor([2.0], device=DEV), torch.tensor([0.0], device=DEV)
    assert int(cuda.argmax(cuda.adjust_logits(row.clone(), none, one, seen))) == 9
