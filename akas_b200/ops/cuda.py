"""The compiled sm_100a kernels behind the signatures that the parts call.

Every function takes torch CUDA tensors, allocates its output with torch, and
launches the kernel of ``akas_b200/csrc`` on torch's current stream through the
library's C entry point. ``akas_b200.ops.reference`` states the same functions in
plain PyTorch. A missing compiler, a failed build or a launch error raises; there
is no other path.
"""

from __future__ import annotations

import ctypes
import functools
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Iterable, Optional

import torch

from . import build

name = "cuda-sm100a"

_F32, _BF16 = 0, 1
_CODE = {torch.float32: _F32, torch.bfloat16: _BF16}
_WORKSPACE_BYTES = 64 << 20
_workspaces = {}
launch_count = 0  # kernels launched through this module since import (library products count as one)

_SIGNATURES = {
    "elementwise": {
        "akas_embedding": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "akas_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p],
        "akas_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "akas_take_tokens": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "akas_zero_row": [c_void_p, c_longlong, c_int, c_int, c_longlong, c_void_p],
        "akas_add_bias": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "akas_scale_cap": [c_void_p, c_float, c_float, c_longlong, c_void_p],
    },
    "conv": {
        "akas_short_conv": [c_void_p] * 8 + [c_int] * 6 + [c_void_p],
        "akas_short_conv_decode": [c_void_p] * 7 + [c_int] * 5 + [c_void_p],
    },
    "rope": {
        "akas_rope_tables": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "akas_qk_norm_rope_store": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_int,
                                    c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                    c_int, c_int, c_int, c_void_p],
        "akas_kv_store": [c_void_p, c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                          c_int, c_int, c_int, c_int, c_int, c_void_p],
    },
    "attention": {
        "akas_paged_attention": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float,
                                 c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "akas_paged_attention_decode": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                        c_int, c_void_p],
    },
    "attention_prefill": {
        "akas_prefill_attention_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                        c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    },
    "attention_prefill_tc": {
        "akas_prefill_attention_tc": [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                      c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "akas_prefill_attention_tc_status": [],
    },
    "attention_decode": {
        "akas_decode_attention_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                       c_void_p],
        "akas_decode_attention_bf16_paged": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                             c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int,
                                             c_int, c_int, c_void_p],
        "akas_decode_attention_from_qkv": [c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_int, c_int,
                                           c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                           c_void_p],
        "akas_decode_attention_items": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_int, c_int,
                                        c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                        c_void_p],
        "akas_decode_attention_items_places": [c_int, c_int],
        "akas_decode_attention_status": [],
    },
    "gemm_tcgen05": {
        "akas_gemm_tcgen05": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "akas_gemm_tcgen05_status": [],
    },
    "gemm_pair": {
        "akas_gemm_pair": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "akas_gemm_pair_status": [],
    },
    "gemm_rows": {
        "akas_gemm_rows": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "akas_gemm_rows_takes": [c_int, c_int, c_int, c_int],
        "akas_gemm_rows_status": [],
    },
    "gemm_stream": {
        "akas_stream_gemm": [c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                             c_int, c_void_p],
        "akas_stream_gemm_takes": [c_int, c_int, c_int, c_int, c_int],
        "akas_stream_gemm_status": [],
    },
    "skinny_gemm": {
        "akas_skinny_gemm": [c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                             c_int, c_int, c_void_p],
        "akas_skinny_gemm_conv": [c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                  c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "akas_skinny_gemm_status": [],
    },
    "decode_chain": {
        "akas_chain_set_scratch": [c_void_p],
        "akas_chain_scratch_words": [],
        "akas_chain_begin": [],
        "akas_chain_count": [],
        "akas_chain_takes": [c_int] * 5,
        "akas_chain_gemm": [c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int],
        "akas_chain_conv": [c_void_p] * 7 + [c_int] * 4,
        "akas_chain_embed": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int],
        "akas_chain_run": [c_void_p],
        "akas_chain_status": [],
    },
    "sgemm": {
        "akas_sgemm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    },
    "gemm_bf16": {
        "akas_gemm_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_longlong,
                           c_void_p],
    },
    "sampling": {
        "akas_argmax": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "akas_sample": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "akas_adjust_logits": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    },
}

_functions = {}


def libraries_for(dtype: torch.dtype) -> list:
    """The kernel files a model of this compute dtype needs under the switches as they stand: what a first call
    compiles. A file that only a switch's other value needs (the library arm of the products, the tcgen05 decode
    products, the decode chain) is built when that value is first used."""
    names = ["elementwise", "conv", "rope", "attention", "sampling"]
    if dtype == torch.float32:
        return names + ["sgemm"]
    names += ["gemm_tcgen05", "gemm_pair", "gemm_rows", "skinny_gemm", "attention_prefill", "attention_prefill_tc", "attention_decode"]
    if products == "library":
        names.append("gemm_bf16")
    if decode_products == "stream":
        names.append("gemm_stream")
    if decode_chain == "1":
        names.append("decode_chain")
    return names


def require(names: Optional[Iterable[str]] = None) -> None:
    """Builds (if need be) and loads the named kernel files, or all of them; raises if that fails."""
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device: akas_b200's kernels run on an NVIDIA B200 (sm_100a) only")
    names = list(names) if names is not None else list(_SIGNATURES)
    build.ensure_built(names)
    for n in names:
        _bind(n)
    if "decode_chain" in names:
        _chain_barrier_word(torch.device("cuda", torch.cuda.current_device()))


def _bind(lib_name: str) -> None:
    lib = build.library(lib_name)
    for fn_name, argtypes in _SIGNATURES[lib_name].items():
        if fn_name not in _functions:
            fn = getattr(lib, fn_name)
            fn.argtypes = argtypes
            fn.restype = c_int
            _functions[fn_name] = fn


def _fn(lib_name: str, fn_name: str):
    fn = _functions.get(fn_name)
    if fn is None:
        _bind(lib_name)
        fn = _functions[fn_name]
    return fn


def _check(err: int, what: str, kernels: int = 1) -> None:
    global launch_count
    launch_count += kernels
    if err:
        if err >= 2000:
            detail = f"cuBLASLt found no algorithm (status {err - 2000})"
        elif err >= 1000:
            detail = f"cuBLAS status {err - 1000}"
        else:
            detail = f"CUDA error {err}"
        raise RuntimeError(f"{what} failed: {detail}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The handle of torch's current stream on the current device (every launch goes there)."""
    if _raw_stream is not None:  # the same value as below without building a Stream object per launch
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _code(t: torch.Tensor) -> int:
    try:
        return _CODE[t.dtype]
    except KeyError:
        raise TypeError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}") from None


def _dense(t: torch.Tensor, what: str) -> torch.Tensor:
    if not t.is_contiguous():
        raise ValueError(f"{what} must be contiguous")
    return t


# --------------------------------------------------------------------------- chained decode steps
#
# A decode step is a chain of small operations: products for a handful of tokens, the short convolution, the
# embedding look-up. Between ``chain_begin`` and ``chain_end`` (the decoder brackets a decode step with them) the
# functions below that can join a chain do not launch: they allocate their output, add themselves to a program, and
# return; the program runs as ONE persistent launch (csrc/decode_chain.cu) when an operation comes that cannot join
# (every other function of this module flushes first), when it is full, or at ``chain_end``. A part that touches
# tensors by other means than this module's functions must not run inside a chain: the decoder flushes before any
# block whose parts do not declare ``chain_safe``. Chains are off unless AKAS_B200_DECODE_CHAIN=1: measured on the
# 1.2B shape at 8 tokens a chained step takes 1.03 ms against 0.89 ms for one launch per operation (a meeting of the
# whole grid inside a kernel costs what a kernel boundary with a programmatic dependent launch costs, and one block
# per SM keeps fewer bytes in flight than two); both are tested.
decode_chain = os.environ.get("AKAS_B200_DECODE_CHAIN", "0")
if decode_chain not in ("0", "1"):
    raise ValueError(f"AKAS_B200_DECODE_CHAIN must be 0 or 1, got {decode_chain!r}")
_CHAIN_ROWS = 16
_chain_open = False
_chain_keep = []  # tensors of the program under construction, kept alive until it has been launched
_chain_words = {}
_chain_answers = {}


def _chain_barrier_word(device):
    """The words of device memory that the blocks of a chain meet on and count tiles in (zeroed once; the kernel
    leaves them as it found them)."""
    word = _chain_words.get(device)
    if word is None:
        count = int(_fn("decode_chain", "akas_chain_scratch_words")())
        word = _chain_words[device] = torch.zeros(count, dtype=torch.int32, device=device)
        _check(_fn("decode_chain", "akas_chain_set_scratch")(_ptr(word)), "chain scratch", kernels=0)
    return word


def chain_begin(num_tokens: int) -> bool:
    """Opens a chain for a decode step of ``num_tokens`` tokens; False if chains are off or the step is too large."""
    global _chain_open
    device = torch.device("cuda", torch.cuda.current_device())
    if decode_chain != "1" or num_tokens > _CHAIN_ROWS or _chain_open or device not in _chain_words:
        return False  # (no barrier word: the chain's library was not asked for, as for a float32 model)
    _fn("decode_chain", "akas_chain_begin")()
    _chain_open = True
    return True


def chain_flush() -> None:
    """Launches what the chain holds so far; the chain stays open."""
    if _chain_open and _fn("decode_chain", "akas_chain_count")():
        err = _fn("decode_chain", "akas_chain_run")(_stream())
        _chain_keep.clear()
        _check(err, "decode chain")


def chain_end() -> None:
    global _chain_open
    try:
        chain_flush()
    finally:
        _chain_open = False
        _chain_keep.clear()


def chain_status() -> int:
    """0 unless a bounded wait inside the chain kernel has run out on this device. Synchronises."""
    return int(_fn("decode_chain", "akas_chain_status")())


def _chain_takes(m: int, o: int, k: int, in_mode: int, mode: int) -> bool:
    if not _chain_open or m > _CHAIN_ROWS:
        return False
    key = (m > 8, o % 2, k, in_mode, mode)
    answer = _chain_answers.get(key)
    if answer is None:
        answer = _chain_answers[key] = bool(_fn("decode_chain", "akas_chain_takes")(m, o, k, in_mode, mode))
    return answer


_CHAIN_OPS = int(os.environ.get("AKAS_B200_CHAIN_OPS", "24"))  # the most operations of one launch


def _chain_add(fn_name: str, keep, *args) -> None:
    """Adds an operation to the open chain (launching the chain first when it is full)."""
    fn = _fn("decode_chain", fn_name)
    if _fn("decode_chain", "akas_chain_count")() >= _CHAIN_OPS:
        chain_flush()
    err = fn(*args)
    if err == 1:  # the program is full
        chain_flush()
        err = fn(*args)
    if err:
        raise RuntimeError(f"{fn_name} failed: error {err}")
    _chain_keep.extend(keep)


def _flushes(fn):
    """An operation that cannot join a chain: whatever the chain holds runs first."""
    @functools.wraps(fn)
    def flushed(*args, **kwargs):
        if _chain_open:
            chain_flush()
        return fn(*args, **kwargs)
    return flushed


# --------------------------------------------------------------------------- elementwise


def embedding(token_ids, table):
    n, c = token_ids.numel(), table.shape[1]
    out = torch.empty((n, c), dtype=torch.float32, device=table.device)
    if _chain_open and n <= _CHAIN_ROWS:
        _chain_add("akas_chain_embed", (token_ids, table, out), _ptr(token_ids), _ptr(_dense(table, "table")), _ptr(out), n, c,
                   _code(table))
        return out
    _check(_fn("elementwise", "akas_embedding")(_ptr(token_ids), _ptr(_dense(table, "table")), _ptr(out), n, c,
                                               _code(table), _stream()), "embedding")
    return out


@_flushes
def take_tokens(token_ids, source, previous):
    """token_ids[i] = previous[source[i]] where source[i] >= 0 (all int32, in place)."""
    _check(_fn("elementwise", "akas_take_tokens")(_ptr(token_ids), _ptr(source), _ptr(previous), previous.numel(),
                                                 token_ids.numel(), _stream()), "take_tokens")


@_flushes
def rmsnorm(x, weight, eps, zero_centered, out_dtype, rows=None):
    c = x.shape[-1]
    _dense(x, "x")
    lead = x.shape[:-1]
    m = rows.numel() if rows is not None else x.numel() // c
    out_shape = (m, c) if rows is not None else (*lead, c)
    out = torch.empty(out_shape, dtype=out_dtype, device=x.device)
    _check(_fn("elementwise", "akas_rmsnorm")(_ptr(x), _ptr(weight), _ptr(out), _ptr(rows), m, c, float(eps),
                                             int(bool(zero_centered)), _code(x), _CODE[out_dtype], _stream()),
           "rmsnorm")
    return out


@_flushes
def swiglu(gate_up):
    n, f2 = gate_up.shape
    out = torch.empty((n, f2 // 2), dtype=gate_up.dtype, device=gate_up.device)
    _check(_fn("elementwise", "akas_swiglu")(_ptr(_dense(gate_up, "gate_up")), _ptr(out), n, f2 // 2, _code(gate_up),
                                            _stream()), "swiglu")
    return out


@_flushes
def add_bias(x, bias, out_dtype=None):
    """x [N, C] float32 plus bias [C] float32, rounded once to ``out_dtype``; in place when that is float32."""
    n, c = x.shape
    if x.dtype != torch.float32 or bias.dtype != torch.float32 or bias.numel() != c:
        raise ValueError("add_bias takes float32 x [N, C] and a float32 bias [C]")
    target = out_dtype or torch.float32
    out = x if target == torch.float32 else torch.empty((n, c), dtype=target, device=x.device)
    _check(_fn("elementwise", "akas_add_bias")(_ptr(_dense(x, "x")), _ptr(bias), _ptr(out), n, c, _CODE[target], _stream()),
           "add_bias")
    return out


@_flushes
def scale_cap(x, scale=1.0, cap=0.0):
    """In place on float32 x: times ``scale``, then ``cap * tanh(x / cap)`` where ``cap`` > 0."""
    if x.dtype != torch.float32:
        raise TypeError("scale_cap takes float32")
    _check(_fn("elementwise", "akas_scale_cap")(_ptr(_dense(x, "x")), float(scale), float(cap), x.numel(), _stream()),
           "scale_cap")
    return x


@_flushes
def zero_rows(state, slot):
    """state[:, slot] = 0 for a contiguous tensor [layers, slots, ...]."""
    row = state[0, 0].numel()
    if state.dtype != torch.float32 or not state.is_contiguous():
        state[:, slot].zero_()
        return
    _check(_fn("elementwise", "akas_zero_row")(_ptr(state), row, int(slot), state.shape[0], state[0].numel(), _stream()),
           "zero_rows")


# --------------------------------------------------------------------------- matrix products


def _workspace(device):
    ws = _workspaces.get(device)
    if ws is None:
        ws = _workspaces[device] = torch.empty(_WORKSPACE_BYTES, dtype=torch.uint8, device=device)
    return ws


def linear(x, w, out_dtype=None, residual=None):
    """x [N, K] times w [O, K] transposed. With ``residual`` (float32 [N, O]) the product is added into it."""
    n, k = x.shape
    o = w.shape[0]
    if w.shape[1] != k:
        raise ValueError(f"linear: x has {k} columns, w has {w.shape[1]}")
    _dense(x, "x")
    _dense(w, "w")
    if x.dtype != w.dtype:
        raise TypeError(f"linear: x is {x.dtype}, w is {w.dtype}")
    if residual is not None:
        if residual.dtype != torch.float32 or residual.shape != (n, o) or not residual.is_contiguous():
            raise ValueError("linear: residual must be contiguous float32 [N, O]")
    if x.dtype == torch.float32:
        if _chain_open:
            chain_flush()
        out = residual if residual is not None else torch.empty((n, o), dtype=torch.float32, device=x.device)
        _check(_fn("sgemm", "akas_sgemm")(_ptr(x), _ptr(w), _ptr(out), _ptr(residual), n, o, k, _stream()), "sgemm")
        if residual is None and out_dtype not in (None, torch.float32):
            out = out.to(out_dtype)
        return out
    if x.dtype != torch.bfloat16:
        raise TypeError(f"linear takes float32 or bfloat16, got {x.dtype}")
    target = out_dtype or torch.bfloat16
    mode = _OUT_ACC if residual is not None else _OUT_F32 if target == torch.float32 else _OUT_BF16
    if _chain_takes(n, o, k, 0, mode):
        out = residual if residual is not None else torch.empty((n, o), dtype=target, device=x.device)
        _chain_add("akas_chain_gemm", (x, w, out), _ptr(x), None, None, 0.0, 0, _ptr(w), _ptr(out), n, o, k, 0, mode)
        return out
    if _chain_open:
        chain_flush()
    if _stream_takes(n, o, k, False, mode):
        # few tokens: the weights are streamed once through the tensor cores
        out = residual if residual is not None else torch.empty((n, o), dtype=target, device=x.device)
        _stream_product(x, None, None, 0.0, False, False, w, out, n, o, k, mode)
        return out
    if _skinny_fits(n, k):
        out = residual if residual is not None else torch.empty((n, o), dtype=target, device=x.device)
        _skinny(x, None, None, 0.0, False, w, out, n, o, k, 0, mode)
        return out
    if k % 8:
        raise ValueError(f"bfloat16 matrix products need an inner size that is a multiple of 8, got {k}")
    route = _product_route(k, o, mode)
    if route == "paired":
        return paired_product(x, w, out_dtype=target, residual=residual)
    if route == "block":
        return block_product(x, w, out_dtype=target, residual=residual)
    if residual is not None:
        out, out_f32, acc = residual, 1, 1
    else:
        out = torch.empty((n, o), dtype=target, device=x.device)
        out_f32, acc = int(target == torch.float32), 0
    ws = _workspace(x.device)
    _check(_fn("gemm_bf16", "akas_gemm_bf16")(_ptr(x), _ptr(w), _ptr(out), n, o, k, out_f32, acc, _ptr(ws),
                                             ws.numel(), _stream()), f"bfloat16 product [{n}x{k}] x [{o}x{k}]^T")
    return out


def _skinny_fits(m: int, k: int) -> bool:
    """Whether the skinny kernel takes this product: few tokens, an inner size that is a multiple of 64 (its TMA
    boxes), and activations that fit in shared memory beside the ring of weight chunks."""
    tokens = 8 if m <= 8 else 16
    return decode_products == "skinny" and m <= _SKINNY_ROWS and k % 64 == 0 and 1024 + 8 * 8192 + tokens * 512 + tokens * (k + 32) * 2 <= 226 * 1024


_SKINNY_ROWS = 16
# Which kernels run the products of more than 16 tokens (prompt portions, mixed steps, large decode batches). "own"
# (default; "auto" and "tcgen05" mean the same): the hand-written tcgen05 kernels everywhere: the kernel for pairs of
# SMs (gemm_pair.cu, TMA-written read-outs) for every product whose output rows TMA can write, the one-block kernel
# (gemm_tcgen05.cu, masked read-outs) for the rest. "library": cuBLASLt everywhere, with SwiGLU as a kernel of its
# own: the arm that the hand-written kernels are measured against.
products = os.environ.get("AKAS_B200_PRODUCTS", "own")
if products not in ("own", "auto", "tcgen05", "library"):
    raise ValueError(f"AKAS_B200_PRODUCTS must be own or library, got {products!r}")


def _product_route(k: int, o: int, mode: int) -> str:
    """Which kernel runs a product of more than 16 tokens with inner size k and o output channels (for SwiGLU the
    stacked 2F): "paired", "block", "library", or (SwiGLU only) "unfused"."""
    if products == "library":
        return "library"
    if mode == _OUT_SWIGLU:
        return "paired" if o % 16 == 0 else "unfused"  # unfused: the plain product, then the SwiGLU kernel
    pitch_ok = o % 8 == 0 if mode == _OUT_BF16 else o % 4 == 0
    return "paired" if pitch_ok else "block"


_sms = 0


def _sm_count() -> int:
    global _sms
    if not _sms:
        _sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _sms


@_flushes
def block_product(x, w, swiglu_out: bool = False, out_dtype=None, residual=None):
    """The same products on the one-block tcgen05 kernel (gemm_tcgen05.cu), whose masked read-outs take any width:
    the route of sizes whose rows TMA cannot write (a pitch that is no multiple of 16 bytes). A float32 result is
    summed into zeros."""
    n, k = x.shape
    o = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != k or k % 8:
        raise ValueError("block_product takes bfloat16 [N, K] and [O, K] with K a multiple of 8")
    kernels = 1
    if swiglu_out:
        if o % 16:
            raise ValueError("block_product: the stacked gate and up matrices need a height that is a multiple of 16")
        out, epilogue = torch.empty((n, o // 2), dtype=torch.bfloat16, device=x.device), 2
    elif residual is not None:
        out, epilogue = residual, 1
    elif out_dtype == torch.float32:
        out, epilogue, kernels = torch.zeros((n, o), dtype=torch.float32, device=x.device), 1, 2
    else:
        out, epilogue = torch.empty((n, o), dtype=torch.bfloat16, device=x.device), 0
    _check(_fn("gemm_tcgen05", "akas_gemm_tcgen05")(_ptr(_dense(x, "x")), _ptr(_dense(w, "w")), _ptr(out), n, o, k, epilogue,
                                                   _stream()), f"tcgen05 product [{n}x{k}] x [{o}x{k}]^T", kernels=kernels)
    return out


def _tma_product(name, x, w, swiglu_out, out_dtype, residual):
    """The checks and the output of a product whose read-out TMA writes: (out, epilogue code)."""
    n, k = x.shape
    o = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != k or k % 8:
        raise ValueError(f"{name} takes bfloat16 [N, K] and [O, K] with K a multiple of 8")
    if swiglu_out:
        if o % 16:
            raise ValueError(f"{name}: the stacked gate and up matrices need a height that is a multiple of 16")
        return torch.empty((n, o // 2), dtype=torch.bfloat16, device=x.device), 2
    if residual is not None:
        if residual.dtype != torch.float32 or residual.shape != (n, o) or not residual.is_contiguous() or o % 4:
            raise ValueError(f"{name}: residual must be contiguous float32 [N, O] with O a multiple of 4")
        return residual, 1
    if out_dtype == torch.float32:
        if o % 4:
            raise ValueError(f"{name}: a float32 result needs a width that is a multiple of 4")
        return torch.empty((n, o), dtype=torch.float32, device=x.device), 3
    if o % 8:
        raise ValueError(f"{name}: a bfloat16 result needs a width that is a multiple of 8")
    return torch.empty((n, o), dtype=torch.bfloat16, device=x.device), 0


# Products of 17 to 128 tokens (decode steps of many requests, short portions) stream the weights through every SM
# (gemm_rows.cu); AKAS_B200_ROWS_PRODUCTS=0 gives them to the kernel for pairs of SMs like longer portions.
_ROWS_MAX = 128
rows_products = os.environ.get("AKAS_B200_ROWS_PRODUCTS", "1") != "0"
_rows_answers = {}


def _rows_takes(n: int, o: int, k: int, epilogue: int) -> bool:
    if not rows_products or n > _ROWS_MAX:
        return False
    key = (torch.cuda.current_device(), n, o, k, epilogue)
    answer = _rows_answers.get(key)
    if answer is None:
        answer = _rows_answers[key] = bool(_fn("gemm_rows", "akas_gemm_rows_takes")(n, o, k, epilogue))
    return answer


@_flushes
def rows_product(x, w, swiglu_out: bool = False, out_dtype=None, residual=None):
    """x [N, K] times w [O, K] transposed for at most 128 tokens: the weights streamed once through all SMs, the
    read-outs of ``paired_product``."""
    n, k = x.shape
    o = w.shape[0]
    out, epilogue = _tma_product("rows_product", x, w, swiglu_out, out_dtype, residual)
    if not _rows_takes(n, o, k, epilogue):
        raise ValueError(f"rows_product does not take [{n}x{k}] x [{o}x{k}]^T (at most {_ROWS_MAX} tokens)")
    _check(_fn("gemm_rows", "akas_gemm_rows")(_ptr(_dense(x, "x")), _ptr(_dense(w, "w")), _ptr(out), n, o, k, epilogue,
                                             _stream()), f"streamed tcgen05 product [{n}x{k}] x [{o}x{k}]^T")
    return out


def gemm_rows_status() -> int:
    """0 unless a bounded wait inside the kernel of ``rows_product`` has run out on this device. Synchronises."""
    return int(_fn("gemm_rows", "akas_gemm_rows_status")())


@_flushes
def paired_product(x, w, swiglu_out: bool = False, out_dtype=None, residual=None, few_rows=True):
    """x [N, K] times w [O, K] transposed on pairs of SMs. bfloat16 out by default; float32 out with ``out_dtype``;
    added into ``residual`` (float32 [N, O]) when that is given; with ``swiglu_out`` w is the stacked [2F, K] gate and
    up matrices and the result is swiglu of the product, bfloat16 [N, F]. Up to 128 tokens go to ``rows_product``
    unless ``few_rows`` is False."""
    n, k = x.shape
    o = w.shape[0]
    out, epilogue = _tma_product("paired_product", x, w, swiglu_out, out_dtype, residual)
    if few_rows and _rows_takes(n, o, k, epilogue):
        _check(_fn("gemm_rows", "akas_gemm_rows")(_ptr(_dense(x, "x")), _ptr(_dense(w, "w")), _ptr(out), n, o, k, epilogue,
                                                 _stream()), f"streamed tcgen05 product [{n}x{k}] x [{o}x{k}]^T")
        return out
    _check(_fn("gemm_pair", "akas_gemm_pair")(_ptr(_dense(x, "x")), _ptr(_dense(w, "w")), _ptr(out), n, o, k, epilogue,
                                             _stream()), f"paired tcgen05 product [{n}x{k}] x [{o}x{k}]^T")
    return out


def gemm_pair_status() -> int:
    """0 unless a bounded wait inside the paired-SM product kernel has run out on this device. Synchronises."""
    return int(_fn("gemm_pair", "akas_gemm_pair_status")())


def gemm_tcgen05_status() -> int:
    """0 unless a bounded wait inside the tcgen05 product kernel has run out on this device. Synchronises."""
    return int(_fn("gemm_tcgen05", "akas_gemm_tcgen05_status")())


_OUT_BF16, _OUT_F32, _OUT_ACC, _OUT_SWIGLU = 0, 1, 2, 3


# Which kernel runs the products of decode steps (few tokens): "skinny", the mma.sync kernel, for up to 16 tokens;
# "stream", the tcgen05 kernel that streams the weights through the tensor cores (K split over a thread-block
# cluster where output channels are few), for up to _STREAM_ROWS tokens. Measured on the 1.2B shape at 8 tokens
# the skinny kernel is the faster one (1.01 ms a step against 1.35 ms), so it is the default; both are tested.
decode_products = os.environ.get("AKAS_B200_DECODE_PRODUCTS", "skinny")
if decode_products not in ("stream", "skinny"):
    raise ValueError(f"AKAS_B200_DECODE_PRODUCTS must be stream or skinny, got {decode_products!r}")
_STREAM_ROWS = 128
_stream_answers = {}


def _stream_takes(m: int, o: int, k: int, in_norm: bool, mode: int) -> bool:
    if decode_products != "stream" or m > _STREAM_ROWS or k % 8:
        return False
    key = (m, o, k, in_norm, mode)
    answer = _stream_answers.get(key)
    if answer is None:
        answer = _stream_answers[key] = bool(_fn("gemm_stream", "akas_stream_gemm_takes")(m, o, k, int(in_norm), mode))
    return answer


def _stream_product(x, rows, norm_w, eps, zero_centered, in_norm, w, out, m, o, k, mode):
    _check(_fn("gemm_stream", "akas_stream_gemm")(_ptr(x), _ptr(rows), _ptr(norm_w), float(eps), int(bool(zero_centered)),
                                                 int(in_norm), _ptr(w), _ptr(out), m, o, k, mode, _stream()),
           f"streamed product [{m}x{k}] x [{o}x{k}]^T")


def stream_status() -> int:
    """0 unless a bounded wait inside the streamed product kernel has run out on this device (then its results
    since are not valid). Synchronises with the device."""
    return int(_fn("gemm_stream", "akas_stream_gemm_status")())


def _skinny(x, rows, norm_w, eps, zero_centered, w, out, m, o, k, in_mode, out_mode):
    _check(_fn("skinny_gemm", "akas_skinny_gemm")(_ptr(x), _ptr(rows), _ptr(norm_w), float(eps), int(bool(zero_centered)),
                                                 _ptr(w), _ptr(out), m, o, k, in_mode, out_mode, _stream()),
           f"skinny product [{m}x{k}] x [{o}x{k}]^T")


def skinny_status() -> int:
    """0 unless a bounded wait inside the skinny product kernel has run out on this device (then its results
    since are not valid). Synchronises with the device."""
    return int(_fn("skinny_gemm", "akas_skinny_gemm_status")())


def linear_swiglu(x, w_gate_up):
    """swiglu(x . w^T) with w the stacked [2F, K] gate and up matrices: [N, F] in x's dtype."""
    n, k = x.shape
    f2 = w_gate_up.shape[0]
    if x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and f2 % 2 == 0 and _chain_takes(n, f2, k, 0, _OUT_SWIGLU):
        out = torch.empty((n, f2 // 2), dtype=torch.bfloat16, device=x.device)
        _chain_add("akas_chain_gemm", (x, w_gate_up, out), _ptr(_dense(x, "x")), None, None, 0.0, 0,
                   _ptr(_dense(w_gate_up, "w")), _ptr(out), n, f2, k, 0, _OUT_SWIGLU)
        return out
    if _chain_open:
        chain_flush()
    if x.dtype == torch.bfloat16 and f2 % 2 == 0 and _stream_takes(n, f2, k, False, _OUT_SWIGLU):
        out = torch.empty((n, f2 // 2), dtype=torch.bfloat16, device=x.device)
        _stream_product(_dense(x, "x"), None, None, 0.0, False, False, _dense(w_gate_up, "w"), out, n, f2, k, _OUT_SWIGLU)
        return out
    if x.dtype == torch.bfloat16 and f2 % 2 == 0 and _skinny_fits(n, k):
        out = torch.empty((n, f2 // 2), dtype=torch.bfloat16, device=x.device)
        _skinny(_dense(x, "x"), None, None, 0.0, False, _dense(w_gate_up, "w"), out, n, f2, k, 0, _OUT_SWIGLU)
        return out
    if x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and k % 8 == 0 and \
            _product_route(k, f2, _OUT_SWIGLU) == "paired":
        # SwiGLU in the read-out of the product: the [N, 2F] intermediate is never written
        return paired_product(x, w_gate_up, swiglu_out=True)
    return swiglu(linear(x, w_gate_up))


def norm_linear(h, norm_weight, eps, zero_centered, w, out_dtype=None, rows=None, swiglu_out=False):
    """linear(rmsnorm(h[rows]), w), optionally through swiglu: the norm rides in the product for few tokens."""
    m = rows.numel() if rows is not None else h.shape[0]
    k, o = h.shape[1], w.shape[0]
    target = torch.bfloat16 if swiglu_out else (out_dtype or torch.bfloat16)
    mode = _OUT_SWIGLU if swiglu_out else _OUT_F32 if target == torch.float32 else _OUT_BF16
    fusable = w.dtype == torch.bfloat16 and h.dtype == torch.float32 and h.is_contiguous() and (not swiglu_out or o % 2 == 0)
    if fusable and _chain_takes(m, o, k, 1, mode):
        out = torch.empty((m, o // 2 if swiglu_out else o), dtype=target, device=h.device)
        _chain_add("akas_chain_gemm", (h, rows, norm_weight, w, out), _ptr(h), _ptr(rows), _ptr(norm_weight), float(eps),
                   int(bool(zero_centered)), _ptr(_dense(w, "w")), _ptr(out), m, o, k, 1, mode)
        return out
    if _chain_open:
        chain_flush()
    if fusable and _stream_takes(m, o, k, True, mode):
        out = torch.empty((m, o // 2 if swiglu_out else o), dtype=target, device=h.device)
        _stream_product(h, rows, norm_weight, eps, zero_centered, True, _dense(w, "w"), out, m, o, k, mode)
        return out
    if fusable and _skinny_fits(m, k):
        out = torch.empty((m, o // 2 if swiglu_out else o), dtype=target, device=h.device)
        _skinny(h, rows, norm_weight, eps, zero_centered, _dense(w, "w"), out, m, o, k, 1, mode)
        return out
    x = rmsnorm(h, norm_weight, eps, zero_centered, w.dtype, rows)
    return linear_swiglu(x, w) if swiglu_out else linear(x, w, out_dtype=out_dtype)


# A decode step's in projection and gated short convolution as one kernel (csrc/skinny_gemm.cu, read-out "conv"):
# AKAS_B200_FUSED_CONV=0 runs them as the product and the convolution kernel.
fused_conv = os.environ.get("AKAS_B200_FUSED_CONV", "1") != "0"


def norm_linear_short_conv(h, norm_weight, eps, zero_centered, w_in, taps, bias, state, seq_of_token, slots, write=True):
    """``short_conv(norm_linear(h, ...), ...)`` for a decode step (every token the single token of its request) in one
    launch, or None where the fused kernel does not take the sizes (the caller then runs the two by themselves)."""
    m, k = h.shape
    c3 = w_in.shape[0]
    c, l = c3 // 3, taps.shape[1]
    if not fused_conv or _chain_open or w_in.dtype != torch.bfloat16 or h.dtype != torch.float32 or not h.is_contiguous() \
            or c3 % 3 or c % 8 or not 2 <= l <= 16 or not _skinny_fits(m, k) or state.dtype != torch.float32:
        return None
    out = torch.empty((m, c), dtype=torch.bfloat16, device=h.device)
    _check(_fn("skinny_gemm", "akas_skinny_gemm_conv")(
        _ptr(h), None, _ptr(norm_weight), float(eps), int(bool(zero_centered)), _ptr(_dense(w_in, "w")), _ptr(out), m, c, k, 1,
        _ptr(taps), _ptr(bias), _ptr(state), _ptr(seq_of_token), _ptr(slots), l, int(bool(write)), _stream()),
        f"fused in projection and short convolution [{m}x{k}] x [{c3}x{k}]^T")
    return out


# --------------------------------------------------------------------------- mixers


def short_conv(bcx, taps, bias, state, cu_seqlens, seq_of_token, slots, decode_only=False, write=True):
    """The gated short convolution over the flat batch; ``write=False`` reads the state and leaves it as it is."""
    n, c3 = bcx.shape
    c, l = c3 // 3, taps.shape[1]
    out = torch.empty((n, c), dtype=bcx.dtype, device=bcx.device)
    if decode_only and _chain_open and n <= _CHAIN_ROWS and bcx.dtype == torch.bfloat16:
        _chain_add("akas_chain_conv", (bcx, taps, bias, state, seq_of_token, slots, out), _ptr(_dense(bcx, "bcx")), _ptr(taps),
                   _ptr(bias), _ptr(state), _ptr(seq_of_token), _ptr(slots), _ptr(out), n, c, l, int(bool(write)))
        return out
    if _chain_open:
        chain_flush()
    if decode_only:
        _check(_fn("conv", "akas_short_conv_decode")(_ptr(_dense(bcx, "bcx")), _ptr(taps), _ptr(bias), _ptr(state),
                                                    _ptr(seq_of_token), _ptr(slots), _ptr(out), n, c, l, _code(bcx),
                                                    int(bool(write)), _stream()), "short_conv_decode")
        return out
    _check(_fn("conv", "akas_short_conv")(_ptr(_dense(bcx, "bcx")), _ptr(taps), _ptr(bias), _ptr(state),
                                         _ptr(cu_seqlens), _ptr(seq_of_token), _ptr(slots), _ptr(out), n,
                                         slots.numel(), c, l, _code(bcx), int(bool(write)), _stream()), "short_conv",
           kernels=2 if write else 1)
    return out


def rope_tables(positions, inv_freq):
    n, half = positions.numel(), inv_freq.numel()
    cos = torch.empty((n, half), dtype=torch.float32, device=positions.device)
    sin = torch.empty_like(cos)
    _check(_fn("rope", "akas_rope_tables")(_ptr(positions), _ptr(inv_freq), _ptr(cos), _ptr(sin), n, half, _stream()),
           "rope_tables")
    return cos, sin


@_flushes
def qk_norm_rope_store(qkv, heads, kv_heads, head_dim, q_weight, k_weight, eps, zero_centered, cos, sin,
                       k_pool, v_pool, block_table, seq_of_token, positions, page_size):
    n = qkv.shape[0]
    _dense(qkv, "qkv")
    if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
        raise ValueError("qkv width does not match (heads + 2 kv_heads) * head_dim")
    q = torch.empty((n, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    rotary = 2 * cos.shape[1] if cos is not None else 0
    _check(_fn("rope", "akas_qk_norm_rope_store")(
        _ptr(qkv), _ptr(q), _ptr(q_weight), _ptr(k_weight), float(eps), int(bool(zero_centered)), _ptr(cos), _ptr(sin),
        rotary, _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1], _ptr(seq_of_token),
        _ptr(positions), page_size, n, heads, kv_heads, head_dim, _code(qkv), _stream()), "qk_norm_rope_store")
    return q


@_flushes
def kv_store(k, v, k_pool, v_pool, block_table, seq_of_token, positions, page_size):
    n = k.shape[0]
    kh, d = k_pool.shape[1], k_pool.shape[3]
    if k.stride(1) != 1 or v.stride(1) != 1:
        raise ValueError("kv_store: k and v must have unit inner stride")
    _check(_fn("rope", "akas_kv_store")(_ptr(k), _ptr(v), k.stride(0), v.stride(0), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
                                       block_table.shape[1], _ptr(seq_of_token), _ptr(positions), page_size, n, kh, d,
                                       _code(k_pool), _stream()), "kv_store")


# Which kernel runs attention over prompt portions in bfloat16: "mma" (the mma.sync kernel, 64-query tiles),
# "tcgen05" (the tensor-memory kernel, 128-query tiles, where it takes the sizes: head size 64, page size a multiple
# of 64) or "auto": the tensor-memory kernel when the step's requests mostly bring more than 64 tokens. Measured on
# the 1.2B shape: 222 against 182 TFLOP/s at 2,048 tokens, 392 against 220 at 8,192 (mma.sync peaks at 550 here).
prompt_attention = os.environ.get("AKAS_B200_PROMPT_ATTENTION", "auto")
if prompt_attention not in ("auto", "tcgen05", "mma"):
    raise ValueError(f"AKAS_B200_PROMPT_ATTENTION must be auto, tcgen05 or mma, got {prompt_attention!r}")


# How the decoded tokens of a step that also holds prompt portions are attended: "split" (default), by the split-key
# decode kernel, or "tiles", inside the prompt kernels as query tiles with one live row each.
mixed_attention = os.environ.get("AKAS_B200_MIXED_ATTENTION", "split")
if mixed_attention not in ("split", "tiles"):
    raise ValueError(f"AKAS_B200_MIXED_ATTENTION must be split or tiles, got {mixed_attention!r}")


def decode_attention_status() -> int:
    """0 unless a bounded wait inside the TMA-fed decode-attention kernel has run out on this device."""
    return int(_fn("attention_decode", "akas_decode_attention_status")())


def prefill_attention_tc_status() -> int:
    """0 unless a bounded wait inside the tcgen05 prompt-attention kernel has run out on this device."""
    return int(_fn("attention_prefill_tc", "akas_prefill_attention_tc_status")())


_DECODE_BLOCKS = int(os.environ.get("AKAS_B200_DECODE_BLOCKS", "300"))
_DECODE_SPLITS = int(os.environ.get("AKAS_B200_DECODE_SPLITS", "0"))  # a number of key parts for every step, for measurements


def decode_splits(num_tokens: int, kv_heads: int, head_tiles: int, max_context: int) -> int:
    """How many parts the keys of a decoding request are cut into, from sizes known on the host: enough blocks for
    two per SM (measured on a B200 at 2,048 to 4,096 keys: a block's fixed cost, its query load, barriers and the
    partial result it writes for the merge, outweighs a fuller GPU beyond that; 8 requests of 8 KV heads run fastest
    in 4 to 5 parts, 0.861 ms a step against 0.888 ms in 16), two parts even where the requests alone give that many
    (64 requests: 44.8k tokens/s in 2 parts, 43.4k in 1, 44.4k in 4), and at least four 64-key tiles per part."""
    blocks = max(1, num_tokens * kv_heads * head_tiles)
    want = _DECODE_SPLITS or max(-(-_DECODE_BLOCKS // blocks), 2)
    most = max(1, -(-max_context // 256))
    return max(1, min(want, most, 64))


_decode_cluster_merge = os.environ.get("AKAS_B200_DECODE_CLUSTER_MERGE", "1") != "0"


def _merges_in_cluster(blocks: int, splits: int, head_dim: int, page_size: int) -> bool:
    """Whether the decode attention kernel merges its key parts itself (they form a thread-block cluster: the TMA-fed
    kernel, 2 to 8 parts, up to four blocks per SM in all) instead of leaving them to a second kernel; the rule of
    csrc/attention_decode.cu::launch_tma."""
    return (_decode_cluster_merge and 2 <= splits <= 8 and head_dim == 64 and page_size % 64 == 0
            and blocks * splits <= 4 * _sm_count())


# Decode attention by blocks that walk the step's items instead of a block per item: "auto" (where a block per item
# would come to more blocks than the GPU holds at once: alone and with a cold L2, 64 requests of 2,048 keys take 50 us
# against 58 us), "0" never, "1" wherever the kernel takes the sizes.
decode_items = os.environ.get("AKAS_B200_DECODE_ITEMS", "auto")
if decode_items not in ("auto", "0", "1"):
    raise ValueError(f"AKAS_B200_DECODE_ITEMS must be auto, 0 or 1, got {decode_items!r}")
_items_places_cache = {}


def _items_places(heads: int, kv_heads: int) -> int:
    key = (torch.cuda.current_device(), heads // kv_heads)
    if key not in _items_places_cache:
        _items_places_cache[key] = int(_fn("attention_decode", "akas_decode_attention_items_places")(heads, kv_heads))
    return _items_places_cache[key]


def decode_plan(num_tokens: int, heads: int, kv_heads: int, head_dim: int, page_size: int, keys: int, dtype):
    """(key parts, whether the blocks walk the items) for a decode step's attention, from sizes known on the host."""
    head_tiles = -(-(heads // kv_heads) // 16)
    splits = decode_splits(num_tokens, kv_heads, head_tiles, keys)
    if dtype != torch.bfloat16 or head_dim != 64 or page_size % 64 or decode_items == "0":
        return splits, False
    blocks = num_tokens * kv_heads * head_tiles
    if splits > 8 and keys <= 4096 and _merges_in_cluster(blocks, 8, head_dim, page_size):
        # up to 8 tiles a part: 8 parts that meet inside their cluster, rather than more parts and a kernel that merges
        # them (one request of 2,048 keys: 1,495 against 1,478 tokens/s)
        splits = 8
    if decode_items == "auto" and not 3 * _sm_count() < blocks * splits <= 8 * _sm_count():
        # up to three blocks per SM all run at once; far more than the GPU holds are spread well by the hardware as they
        # come (128 requests of 8,192 keys: 40.1k tokens/s with a block per item, 37.7k with blocks that walk them,
        # whose items are dealt out beforehand); in between, the last round would run part empty (32 requests: 24.5k
        # against 25.9k, at 8,192 keys 18.3k against 20.4k)
        return splits, False
    # (the same parts: measured at 64 requests of 2,048 keys, 48.1k tokens/s in 2 parts, 47.3k in 3, 46.4k in 6 and
    # 44.3k in 11 against 47.2k with a block per item: what an item costs beside its tiles is not hidden by the ring)
    return splits, _items_places(heads, kv_heads) > 0


def _decode_attention(q, n, out, k_pool, v_pool, block_table, seq_of_token, positions, scale, win, page_size, keys):
    """Split-key attention of the first ``n`` tokens of q, each the single token of its request, into out[:n]."""
    kh, d = k_pool.shape[1], k_pool.shape[3]
    heads = q.shape[1] // d
    group = heads // kh
    if q.dtype == torch.bfloat16 and d in (16, 32, 64, 128):
        # tensor-core kernel: the query heads of a group are the rows of one tile
        splits, walks = decode_plan(n, heads, kh, d, page_size, keys, q.dtype)
        part_o = part_ml = None
        if splits > 1:
            part_o = torch.empty((n, heads, splits, d), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((n, heads, splits, 2), dtype=torch.float32, device=q.device)
        if walks:
            err = _fn("attention_decode", "akas_decode_attention_items")(
                _ptr(q), None, None, None, 0.0, 0, None, None, 0, 0, _ptr(k_pool), _ptr(v_pool), k_pool.shape[0],
                _ptr(block_table), block_table.shape[1], _ptr(seq_of_token), _ptr(positions), _ptr(out), _ptr(part_o),
                _ptr(part_ml), float(scale), win, page_size, n, heads, kh, d, splits, _stream())
            if err != 3999:
                _check(err, "decode_attention (items)", kernels=2 if splits > 1 else 1)
                return
            splits = decode_splits(n, kh, -(-group // 16), keys)  # (pointers that the kernel does not take)
            if splits > 1:
                part_o = torch.empty((n, heads, splits, d), dtype=torch.float32, device=q.device)
                part_ml = torch.empty((n, heads, splits, 2), dtype=torch.float32, device=q.device)
        _check(_fn("attention_decode", "akas_decode_attention_bf16_paged")(
            _ptr(q), _ptr(k_pool), _ptr(v_pool), k_pool.shape[0], _ptr(block_table), block_table.shape[1], _ptr(seq_of_token),
            _ptr(positions), _ptr(out), _ptr(part_o), _ptr(part_ml), float(scale), win, page_size, n, heads, kh, d,
            splits, _stream()), "decode_attention", kernels=2 if splits > 1 and not _merges_in_cluster(n * kh * -(-group // 16), splits, d, page_size) else 1)
        return
    gt = 8 if group >= 8 else 4 if group > 2 else group
    splits = decode_splits(n, kh, -(-group // gt), keys)
    part_o = torch.empty((n, heads, splits, d), dtype=torch.float32, device=q.device)
    part_ml = torch.empty((n, heads, splits, 2), dtype=torch.float32, device=q.device)
    _check(_fn("attention", "akas_paged_attention_decode")(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1], _ptr(seq_of_token),
        _ptr(positions), _ptr(out), _ptr(part_o), _ptr(part_ml), float(scale), win, page_size, n, heads, kh, d,
        splits, _code(q), _stream()), "paged_attention_decode", kernels=2)


# Whether a decode step's attention layers run as one kernel from the qkv product on (norm and rotation of q and k, the
# write into the pages and attention; measured on the 1.2B shape: 6 launches fewer a step).
fused_qkv_attention = os.environ.get("AKAS_B200_FUSED_QKV_ATTENTION", "1") != "0"


@_flushes
def qkv_decode_attention(qkv, heads, kv_heads, head_dim, q_weight, k_weight, eps, zero_centered, cos, sin, k_pool, v_pool,
                         block_table, seq_of_token, positions, scale, window, page_size, ctx, write=True):
    """``paged_attention(qk_norm_rope_store(qkv, ...), ...)`` for a decode step (every token the single token of its
    request) in one launch, or None where the fused kernel does not take the sizes or the dtype (the caller then runs
    the two by themselves). With ``write=False`` the pages are read as they are and nothing is written."""
    if not fused_qkv_attention or qkv.dtype != torch.bfloat16 or head_dim != 64 or page_size % 64 or k_pool.dtype != torch.bfloat16:
        return None
    n = qkv.shape[0]
    _dense(qkv, "qkv")
    if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
        raise ValueError("qkv width does not match (heads + 2 kv_heads) * head_dim")
    rotary = 2 * cos.shape[1] if cos is not None else 0
    if rotary % 16:
        return None
    win = int(window) if window else 0
    group = heads // kv_heads
    splits, walks = decode_plan(n, heads, kv_heads, head_dim, page_size, win if win else ctx.max_context, qkv.dtype)
    merged = splits == 1 or (not walks and _merges_in_cluster(n * kv_heads * -(-group // 16), splits, head_dim, page_size))
    out = torch.empty((n, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty((n, heads, splits, head_dim), dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty((n, heads, splits, 2), dtype=torch.float32, device=qkv.device)
    prep = (_ptr(qkv), _ptr(q_weight), _ptr(k_weight), float(eps), int(bool(zero_centered)), _ptr(cos), _ptr(sin), rotary,
            int(bool(write)), _ptr(k_pool), _ptr(v_pool), k_pool.shape[0], _ptr(block_table), block_table.shape[1],
            _ptr(seq_of_token), _ptr(positions), _ptr(out), _ptr(part_o), _ptr(part_ml), float(scale), win, page_size, n,
            heads, kv_heads, head_dim, splits, _stream())
    if walks:
        err = _fn("attention_decode", "akas_decode_attention_items")(None, *prep)
    else:
        err = _fn("attention_decode", "akas_decode_attention_from_qkv")(*prep)
    if err == 3999:
        return None
    _check(err, "decode attention from qkv", kernels=1 if merged else 2)
    return out


def _leading_single_tokens(ctx) -> int:
    """How many requests at the front of the step bring exactly one token (the scheduler puts decoding requests first)."""
    lens = getattr(ctx, "query_lens", ()) if ctx is not None else ()
    count = 0
    while count < len(lens) and lens[count] == 1:
        count += 1
    return count


@_flushes
def paged_attention(q, k_pool, v_pool, block_table, seq_of_token, positions, scale, window, page_size, ctx=None):
    n = q.shape[0]
    kh, d = k_pool.shape[1], k_pool.shape[3]
    heads = q.shape[1] // d
    _dense(q, "q")
    out = torch.empty_like(q)
    win = int(window) if window else 0
    if ctx is not None and ctx.decode_only:
        _decode_attention(q, n, out, k_pool, v_pool, block_table, seq_of_token, positions, scale, win, page_size,
                          win if win else ctx.max_context)
        return out
    tensor_cores = q.dtype == torch.bfloat16 and d in (16, 32, 64, 128)
    # A step that mixes portions of prompts with decoded tokens: the single tokens at its front go to the split-key
    # kernel (one block per request, key/value head and part of the keys) instead of a 64-query tile each of which one
    # row is alive; the prompt kernels then start at the first request that brings more. Two launches, one output.
    first = _leading_single_tokens(ctx) if tensor_cores and mixed_attention == "split" else 0
    lens = ctx.query_lens[first:] if first else (getattr(ctx, "query_lens", ()) if ctx is not None else ())
    if first:
        _decode_attention(q, first, out, k_pool, v_pool, block_table, seq_of_token, positions, scale, win, page_size,
                          win if win else ctx.max_context)
        if not lens:
            return out
    tiles, wide = sum(-(-c // 64) for c in lens), sum(-(-c // 128) for c in lens)
    requests = len(lens) if first else (ctx.cu_seqlens.numel() - 1 if tiles else 0)
    # the prompt kernels find their tiles from cu_seqlens and address block tables by request: both start at `first`
    cu = ctx.cu_seqlens[first:] if tiles else None
    table = block_table[first:] if first else block_table
    # A 128-query tile of the tensor-memory kernel costs about what a 64-query tile of the mma.sync kernel costs
    # (measured: 1.8 times the throughput): it pays when requests bring more than 64 tokens, not for single tokens.
    tensor_memory = prompt_attention == "tcgen05" or (prompt_attention == "auto" and 0 < wide and wide <= 0.9 * tiles)
    if q.dtype == torch.bfloat16 and tensor_memory and d == 64 and page_size % 64 == 0 and 0 < tiles <= 65535:
        # prompt portions, head size 64, pages of whole half tiles: 128-query tiles on tcgen05
        err = _fn("attention_prefill_tc", "akas_prefill_attention_tc")(
            _ptr(q), _ptr(k_pool), _ptr(v_pool), k_pool.shape[0] * k_pool.shape[1] * k_pool.shape[2], _ptr(table),
            block_table.shape[1], _ptr(cu), _ptr(positions), _ptr(out), float(scale), win, page_size, tiles, n,
            heads, kh, d, requests, _stream())
        if err != 3999:
            _check(err, "prefill_attention_tc")
            return out
    if tensor_cores and 0 < tiles <= 65535:
        # prompt portions (and whatever decodes beside them): 64-query tiles on the tensor cores
        _check(_fn("attention_prefill", "akas_prefill_attention_bf16")(
            _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(table), block_table.shape[1], _ptr(cu),
            _ptr(positions), _ptr(out), float(scale), win, page_size, tiles, heads, kh, d, requests,
            _stream()), "prefill_attention")
        return out
    _check(_fn("attention", "akas_paged_attention")(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1], _ptr(seq_of_token),
        _ptr(positions), _ptr(out), float(scale), win, page_size, n, heads, kh, d, _code(q), _stream()),
        "paged_attention")
    return out


# --------------------------------------------------------------------------- sampling


@_flushes
def argmax(logits):
    m, v = logits.shape
    out = torch.empty((m,), dtype=torch.int32, device=logits.device)
    parts = max(1, min(64, v // 1024, 592 // max(m, 1)))  # slices of the vocabulary, at least 1024 entries each
    part_val = torch.empty((m, parts), dtype=torch.float32, device=logits.device)
    part_idx = torch.empty((m, parts), dtype=torch.int32, device=logits.device)
    _check(_fn("sampling", "akas_argmax")(_ptr(_dense(logits, "logits")), _ptr(out), _ptr(part_val), _ptr(part_idx), m,
                                         v, parts, _stream()), "argmax", kernels=2)
    return out


@_flushes
def adjust_logits(logits, softcap, penalty, history):
    """In place on float32 logits [M, V]: softcap (float32 [M], 0 = none), then the repetition penalty (float32 [M],
    1 = none) on the tokens of ``history`` (int32 [M, W], -1 where empty)."""
    m, v = logits.shape
    if logits.dtype != torch.float32 or history.dtype != torch.int32 or history.shape[0] != m:
        raise ValueError("adjust_logits takes float32 logits [M, V] and an int32 history [M, W]")
    _check(_fn("sampling", "akas_adjust_logits")(_ptr(_dense(logits, "logits")), _ptr(_dense(softcap, "softcap")),
                                                 _ptr(_dense(penalty, "penalty")), _ptr(_dense(history, "history")),
                                                 history.shape[1], m, v, _stream()), "adjust_logits")
    return logits


@_flushes
def sample(logits, temperature, top_k, top_p, uniform):
    m, v = logits.shape
    out = torch.empty((m,), dtype=torch.int32, device=logits.device)
    _check(_fn("sampling", "akas_sample")(_ptr(_dense(logits, "logits")), _ptr(temperature), _ptr(top_k), _ptr(top_p),
                                         _ptr(uniform), _ptr(out), m, v, _stream()), "sample")
    return out
