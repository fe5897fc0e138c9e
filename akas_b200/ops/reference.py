"""Plain PyTorch statements of every kernel, with the kernels' own signatures.

Each function here says, in a few tensor expressions, what the CUDA kernel of
the same name in ``akas_b200.ops.cuda`` computes: same arguments, same layouts
of pages, block tables and state slots, same in-place effects. The kernel tests
compare each kernel with its neighbour here, and the step function's host logic
(batches, pages, slots) can be exercised on a CPU by handing this module to the
runner as ``ops``. The engine never picks it by itself: without the compiled
kernels it fails.

Layouts. Pages: ``[num_pages, kv_heads, page_size, head_dim]``. Block table:
int32 ``[requests, max_blocks]``, ``-1`` where a request holds no page. Flat
batch: ``seq_of_token[N]`` names each token's request (row of the block table and
of ``slots``; ``-1`` marks padding that must touch nothing), ``positions[N]`` its
absolute position, ``cu_seqlens[R + 1]`` the extent of each request's tokens.
"""

from __future__ import annotations

import torch

name = "reference"


def embedding(token_ids, table):
    return table[token_ids.long()].to(torch.float32)


def rmsnorm(x, weight, eps, zero_centered, out_dtype, rows=None):
    if rows is not None:
        x = x[rows.long()]
    xf = x.to(torch.float32)
    w = weight.to(torch.float32)
    if zero_centered:
        w = w + 1.0
    y = xf * torch.rsqrt((xf * xf).mean(dim=-1, keepdim=True) + eps) * w
    return y.to(out_dtype)


def linear(x, w, out_dtype=None, residual=None):
    """x [N, K] times w [O, K] transposed, float32 accumulation; ``residual`` (float32) is added to in place."""
    y = x.to(torch.float32) @ w.to(torch.float32).T
    if residual is not None:
        residual += y
        return residual
    return y.to(out_dtype or x.dtype)


def swiglu(gate_up):
    f = gate_up.shape[-1] // 2
    g = gate_up[:, :f].to(torch.float32)
    u = gate_up[:, f:].to(torch.float32)
    return (g / (1 + torch.exp(-g)) * u).to(gate_up.dtype)


def linear_swiglu(x, w_gate_up):
    return swiglu(linear(x, w_gate_up))


def norm_linear(h, norm_weight, eps, zero_centered, w, out_dtype=None, rows=None, swiglu_out=False):
    x = rmsnorm(h, norm_weight, eps, zero_centered, w.dtype, rows)
    return linear_swiglu(x, w) if swiglu_out else linear(x, w, out_dtype=out_dtype)


def short_conv(bcx, taps, bias, state, cu_seqlens, seq_of_token, slots, decode_only=False, write=True):
    n, c3 = bcx.shape
    c = c3 // 3
    l = taps.shape[1]
    bf = bcx.to(torch.float32)
    u = bf[:, :c] * bf[:, 2 * c :]
    gate = bf[:, c : 2 * c]
    out = torch.zeros((n, c), dtype=torch.float32, device=bcx.device)
    cu = cu_seqlens.tolist()
    for r, slot in enumerate(slots.tolist()):
        a, b = cu[r], cu[r + 1]
        if slot < 0 or b <= a:
            continue
        hist = torch.cat((state[slot], u[a:b]), dim=0)  # [L-1 + n_r, C], oldest first
        acc = torch.zeros((b - a, c), dtype=torch.float32, device=bcx.device)
        for j in range(l):
            acc = acc + hist[j : j + b - a] * taps[:, j]
        if bias is not None:
            acc = acc + bias
        out[a:b] = gate[a:b] * acc
        if write:
            state[slot] = hist[-(l - 1) :]
    return out.to(bcx.dtype)


def add_bias(x, bias, out_dtype=None):
    """x float32 [N, C] plus bias [C], rounded once to ``out_dtype``; in place when that is float32."""
    if out_dtype in (None, torch.float32):
        return x.add_(bias)
    return (x + bias).to(out_dtype)


def scale_cap(x, scale=1.0, cap=0.0):
    """In place on float32 x: times ``scale``, then ``cap * tanh(x / cap)`` where ``cap`` > 0."""
    x.mul_(scale)
    if cap > 0:
        x.copy_(cap * torch.tanh(x / cap))
    return x


def rope_tables(positions, inv_freq):
    ang = positions.to(torch.float64)[:, None] * inv_freq[None, :]
    return torch.cos(ang).to(torch.float32), torch.sin(ang).to(torch.float32)


def _page_addresses(block_table, seq_of_token, positions, page_size):
    live = seq_of_token >= 0
    seq = seq_of_token.clamp(min=0).long()
    pos = positions.long()
    page = block_table[seq, pos // page_size].long()
    return live, page, pos % page_size


def kv_store(k, v, k_pool, v_pool, block_table, seq_of_token, positions, page_size):
    """k, v: [N, kv_heads * head_dim] -> pages at each live token's (page, offset)."""
    kh, d = k_pool.shape[1], k_pool.shape[3]
    live, page, off = _page_addresses(block_table, seq_of_token, positions, page_size)
    k_pool[page[live], :, off[live]] = k.reshape(-1, kh, d)[live].to(k_pool.dtype)
    v_pool[page[live], :, off[live]] = v.reshape(-1, kh, d)[live].to(v_pool.dtype)


def qk_norm_rope_store(qkv, heads, kv_heads, head_dim, q_weight, k_weight, eps, zero_centered, cos, sin,
                       k_pool, v_pool, block_table, seq_of_token, positions, page_size):
    """Per-head RMSNorm of q and k, rotation of both, k (in place in ``qkv``) and v into the pages; returns q."""
    n = qkv.shape[0]
    d = head_dim
    q = qkv[:, : heads * d].reshape(n, heads, d).to(torch.float32)
    k = qkv[:, heads * d : (heads + kv_heads) * d].reshape(n, kv_heads, d).to(torch.float32).clone()  # written back below
    if q_weight is not None:
        q = rmsnorm(q, q_weight, eps, zero_centered, torch.float32)
        k = rmsnorm(k, k_weight, eps, zero_centered, torch.float32)
    if cos is not None:
        half = cos.shape[1]

        def rotate(x):
            left, right, rest = x[..., :half], x[..., half : 2 * half], x[..., 2 * half :]
            c, s = cos[:, None, :], sin[:, None, :]
            return torch.cat((left * c - right * s, left * s + right * c, rest), dim=-1)

        q, k = rotate(q), rotate(k)
    qkv[:, heads * d : (heads + kv_heads) * d] = k.reshape(n, kv_heads * d).to(qkv.dtype)
    if k_pool is not None:
        kv_store(qkv[:, heads * d : (heads + kv_heads) * d], qkv[:, (heads + kv_heads) * d :], k_pool, v_pool,
                 block_table, seq_of_token, positions, page_size)
    return q.reshape(n, heads * d).to(qkv.dtype)


def paged_attention(q, k_pool, v_pool, block_table, seq_of_token, positions, scale, window, page_size, ctx=None):
    n = q.shape[0]
    kh, d = k_pool.shape[1], k_pool.shape[3]
    heads = q.shape[1] // d
    group = heads // kh
    out = torch.zeros((n, heads * d), dtype=torch.float32, device=q.device)
    seqs, poss = seq_of_token.tolist(), positions.tolist()
    for t in range(n):
        r, p = seqs[t], poss[t]
        if r < 0:
            continue
        first = 0 if window is None else max(0, p - window + 1)
        idx = torch.arange(first, p + 1, device=q.device)
        pages = block_table[r, idx // page_size].long()
        offs = idx % page_size
        keys = k_pool[pages, :, offs].to(torch.float32)  # [S, kh, d]
        vals = v_pool[pages, :, offs].to(torch.float32)
        qt = q[t].reshape(kh, group, d).to(torch.float32)
        scores = torch.einsum("kgd,skd->kgs", qt, keys) * scale
        prob = torch.softmax(scores, dim=-1)
        out[t] = torch.einsum("kgs,skd->kgd", prob, vals).reshape(heads * d)
    return out.to(q.dtype)


def argmax(logits):
    """Greedy token per row; ties go to the lowest index."""
    top = logits.max(dim=-1, keepdim=True).values
    v = logits.shape[-1]
    idx = torch.arange(v, device=logits.device).expand_as(logits)
    return torch.where(logits == top, idx, v).min(dim=-1).values.to(torch.int32)


def sample(logits, temperature, top_k, top_p, uniform):
    """Per row with temperature T: T <= 0 is the argmax. Else w_i = exp((x_i - max x) / T); tokens are ranked by
    logit, larger first, equal logits by id, lower first (the order of the reference's rank loop,
    src/akas/ops/vocabulary/kernel.py:586-622). Token i is kept iff its rank is below top_k (top_k <= 0 or >= V:
    no limit) and the kept tokens ranked before it hold at most top_p of the kept mass (top_p >= 1: no limit);
    the result is the first kept i, in index order, whose running kept mass exceeds uniform * (kept mass)."""
    out = argmax(logits).clone()
    m, v = logits.shape
    for r in range(m):
        t = float(temperature[r])
        if t <= 0:
            continue
        x = logits[r].to(torch.float32)
        w = torch.exp((x - x.max()) * torch.tensor(1.0 / t, dtype=torch.float32, device=x.device)).double()
        order = torch.sort(x, descending=True, stable=True).indices  # equal logits: the lower id first
        rank = torch.empty(v, dtype=torch.long, device=x.device)
        rank[order] = torch.arange(v, device=x.device)
        keep = torch.ones(v, dtype=torch.bool, device=x.device)
        k = int(top_k[r])
        if 0 < k < v:
            keep &= rank < k
        p = float(top_p[r])
        if p < 1.0:
            kept_w = torch.where(keep, w, torch.zeros_like(w))
            before = torch.cumsum(kept_w[order], 0) - kept_w[order]  # kept mass ranked before each token
            keep &= before[rank] <= p * kept_w.sum()
        kept_w = torch.where(keep, w, torch.zeros_like(w))
        run = torch.cumsum(kept_w, 0)
        hit = torch.nonzero(keep & (run > float(uniform[r]) * run[-1]))
        out[r] = int(hit[0]) if len(hit) else int(torch.nonzero(keep)[-1])
    return out


def adjust_logits(logits, softcap, penalty, history):
    """The stages before top-k of the reference's sampler (src/akas/ops/vocabulary/kernel.py:556-577), in place:
    x = c tanh(x / c) where the row's softcap c > 0; then every token of the row's history (-1: none), once, becomes
    x / q if x > 0 else x * q where the row's penalty q != 1."""
    for r in range(logits.shape[0]):
        c, q = float(softcap[r]), float(penalty[r])
        if c > 0:
            logits[r] = c * torch.tanh(logits[r] / c)
        if q != 1.0:
            tokens = torch.unique(history[r][history[r] >= 0]).long()
            x = logits[r, tokens]
            logits[r, tokens] = torch.where(x > 0, x / q, x * q)
    return logits


def take_tokens(token_ids, source, previous):
    live = source >= 0
    token_ids[live] = previous[source[live].long()]


def zero_rows(state, slot):
    state[:, slot].zero_()
