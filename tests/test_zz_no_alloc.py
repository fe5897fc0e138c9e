"""The entry point that allocates nothing: akas_decode_attention_bf16_noalloc (akas_b200/csrc/noalloc.h).

Some callers of the kernels cannot allocate device memory at the moment they need decode attention: a
serving process that has given every free byte to its page pool, a loop that must not stall on cudaMalloc,
a host that reaches this library through its C symbols and has no allocator to lend. For them the
split-key scratch lives in a static device array inside the library. This test calls that entry point
through its exported C symbol, twice in a row with different inputs and different numbers of splits (the
array keeps the first call's contents, which the second must not read), and compares each result with
the allocating entry point given scratch from torch. It is collected last so that a run which stops at the
first failure has already run every other test.
"""

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NOALLOC_FLOATS = 1 << 20
TOO_LARGE = -2


def _library():
    from akas_b200.ops import build

    path = build.ensure_built(["attention_decode"])["attention_decode"]
    lib = ctypes.CDLL(str(path))
    common = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p]
    lib.akas_decode_attention_bf16_noalloc.argtypes = common + [c_float] + [c_int] * 7 + [c_void_p]
    lib.akas_decode_attention_bf16_noalloc.restype = c_int
    lib.akas_decode_attention_bf16.argtypes = common + [c_void_p, c_void_p, c_float] + [c_int] * 7 + [c_void_p]
    lib.akas_decode_attention_bf16.restype = c_int
    lib.akas_decode_attention_bf16_noalloc_needs.argtypes = [c_int] * 4
    lib.akas_decode_attention_bf16_noalloc_needs.restype = c_longlong
    lib.akas_noalloc_error_string.argtypes = [c_int]
    lib.akas_noalloc_error_string.restype = ctypes.c_char_p
    return lib


def _case(seed, contexts, heads, kv_heads, dim, page):
    g = torch.Generator().manual_seed(seed)
    n = len(contexts)
    pages = sum(-(-c // page) for c in contexts) + 2
    perm = torch.randperm(pages, generator=g).tolist()
    table = torch.full((n, max(-(-c // page) for c in contexts) + 1), -1, dtype=torch.int32)
    for r, c in enumerate(contexts):
        for b in range(-(-c // page)):
            table[r, b] = perm.pop()
    rand = lambda *shape: torch.randn(*shape, generator=g).to(torch.bfloat16).to(DEV)
    return dict(
        q=rand(n, heads * dim), k=rand(pages, kv_heads, page, dim), v=rand(pages, kv_heads, page, dim),
        table=table.to(DEV), seq=torch.arange(n, dtype=torch.int32, device=DEV),
        pos=torch.tensor([c - 1 for c in contexts], dtype=torch.int32, device=DEV),
        n=n, heads=heads, kv_heads=kv_heads, dim=dim, page=page,
    )


def _run(lib, case, splits, noalloc):
    out = torch.full_like(case["q"], float("nan"))
    stream = torch.cuda.current_stream().cuda_stream
    head = (case["q"].data_ptr(), case["k"].data_ptr(), case["v"].data_ptr(), case["table"].data_ptr(),
            case["table"].shape[1], case["seq"].data_ptr(), case["pos"].data_ptr(), out.data_ptr())
    tail = (case["dim"] ** -0.5, 0, case["page"], case["n"], case["heads"], case["kv_heads"], case["dim"], splits, stream)
    if noalloc:
        err = lib.akas_decode_attention_bf16_noalloc(*head, *tail)
    else:
        part_o = torch.empty((case["n"], case["heads"], splits, case["dim"]), dtype=torch.float32, device=DEV)
        part_ml = torch.empty((case["n"], case["heads"], splits, 2), dtype=torch.float32, device=DEV)
        err = lib.akas_decode_attention_bf16(*head, part_o.data_ptr(), part_ml.data_ptr(), *tail)
    torch.cuda.synchronize()
    return err, out


def test_entry_point_without_allocation_matches_the_allocating_one():
    lib = _library()
    first = _case(1, [700, 33, 1500, 1], heads=8, kv_heads=2, dim=64, page=16)
    second = _case(2, [64, 900, 257], heads=6, kv_heads=1, dim=128, page=64)
    from akas_b200.ops import reference

    for case, splits in ((first, 6), (second, 3), (first, 1)):
        err, got = _run(lib, case, splits, noalloc=True)
        assert err == 0, lib.akas_noalloc_error_string(err).decode()
        err, want = _run(lib, case, splits, noalloc=False)
        assert err == 0
        assert torch.isfinite(got.float()).all()
        scale = want.float().abs().max().item()
        assert (got.float() - want.float()).abs().max().item() <= 1e-2 * scale  # the kernel tests' bfloat16 tolerance
        # and against the plain statement of the operation, which shares no kernel with either entry point
        plain = reference.paged_attention(case["q"], case["k"], case["v"], case["table"], case["seq"], case["pos"],
                                          case["dim"] ** -0.5, None, case["page"])
        assert (got.float() - plain.float()).abs().max().item() <= 1e-2 * plain.float().abs().max().item()


def test_sizes_beyond_the_scratch_are_refused_with_a_clear_error():
    lib = _library()
    case = _case(3, [100] * 4, heads=8, kv_heads=2, dim=64, page=16)
    assert lib.akas_decode_attention_bf16_noalloc_needs(4, 8, 6, 64) == 4 * 8 * 6 * 66
    assert lib.akas_decode_attention_bf16_noalloc_needs(4, 8, 1, 64) == 0  # one split needs no scratch
    too_many = NOALLOC_FLOATS // (4 * 8 * 66) + 1
    assert lib.akas_decode_attention_bf16_noalloc_needs(4, 8, too_many, 64) > NOALLOC_FLOATS
    big = 2 ** 31 - 1  # a product that does not fit 64 bits is still "too many", never a small number
    assert lib.akas_decode_attention_bf16_noalloc_needs(big, big, big, big) > NOALLOC_FLOATS
    err, out = _run(lib, case, too_many, noalloc=True)
    assert err == TOO_LARGE
    assert torch.isnan(out.float()).all()  # nothing was launched
    message = lib.akas_noalloc_error_string(err).decode()
    assert "AKAS_DECODE_NOALLOC_FLOATS" in message and "fewer splits" in message
    err, _ = _run(lib, case, 4, noalloc=True)  # the entry point still works afterwards
    assert err == 0
