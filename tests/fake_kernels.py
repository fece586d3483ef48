"""Plain PyTorch stand-ins for the kernel table, one function per kernel.

Two uses.  (1) CPU tests hand this module to the engine in place of the CUDA kernel
table, so that the step function, the cache and the scheduler are exercised without a
GPU; the product itself has no such path.  (2) GPU tests compare every CUDA kernel with
the function of the same name here.  Arithmetic is done in float64 and rounded once to
the output type, so these are references, not imitations of the kernels' rounding.

Formulas: the same reference lines the kernels cite (kernels/cuda/generic/norm.cuh,
kernels/cuda/dense/dense_norm_rope.cuh, dense_attn.cuh, dense_common.cuh:120-126,166-180,
kernels/metal/dense/dense_short_conv.metal:31-68, kernels/cuda/generic/glu.cuh:35-57).
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def require():
    return None


def embed(ids, table, feed_index=None, fed_tokens=None, scale=1.0):
    ids = ids.long()
    if feed_index is not None:
        fed = fed_tokens.long()[feed_index.long().clamp(min=0)]
        ids = torch.where(feed_index.long() >= 0, fed, ids)
    return (table[ids].to(F64) * scale).to(torch.float32)


def stream_add(residual, deltas, vector, in_place=True):
    """``residual + sum(deltas) + vector`` (the vector the same for every row), float32; written
    into ``residual`` or, with ``in_place=False``, into rows of its own."""
    total = residual.to(F64)
    for d in deltas:
        total = total + d.to(F64)
    if vector is not None:
        total = total + vector.to(F64)
    if in_place:
        residual.copy_(total.to(residual.dtype))
        return residual
    return total.to(residual.dtype)


def add_dyt(residual, deltas, alpha, w, b, out_dtype, rows=None):
    """``tanh(alpha * x) * w + b`` of ``x = residual + sum(deltas)``; without ``rows`` the sum is
    stored back into ``residual``."""
    if rows is None:
        if deltas:
            total = residual.to(F64)
            for d in deltas:
                total = total + d.to(F64)
            residual.copy_(total.to(residual.dtype))
        x = residual.to(F64)
    else:
        idx = rows.long()
        x = residual[idx]
        for d in deltas:  # summed in float32, as the stored residual would be
            x = (x.to(F64) + d[idx].to(F64)).to(residual.dtype)
        x = x.to(F64)
    return (torch.tanh(alpha * x) * w.to(F64) + b.to(F64)).to(out_dtype)


def gather_rows(x, rows):
    return x[rows.long()].clone()


def rmsnorm(x, w, eps, out_dtype):
    x64 = x.to(F64)
    y = x64 / torch.sqrt((x64 * x64).mean(-1, keepdim=True) + eps) * w.to(F64)
    return y.to(out_dtype)


def add_rmsnorm(residual, delta, w, eps, out_dtype, rows=None):
    if rows is None:
        residual += delta.to(residual.dtype)
        return rmsnorm(residual, w, eps, out_dtype)
    idx = rows.long()
    summed = residual[idx] + delta[idx].to(residual.dtype)
    return rmsnorm(summed, w, eps, out_dtype)


def linear(x, w, out_dtype, bias=None):
    y = x.to(F64) @ w.to(F64).T
    if bias is not None:
        y = y + bias.to(F64)
    return y.to(out_dtype)


def swiglu(gate_up):
    inter = gate_up.shape[1] // 2
    g = gate_up[:, :inter].to(F64)
    u = gate_up[:, inter:].to(F64)
    return (g / (1.0 + torch.exp(-g)) * u).to(gate_up.dtype)


def linear_swiglu(x, gate_up, out_dtype):
    y = x.to(F64) @ gate_up.to(F64).T
    inter = y.shape[1] // 2
    g, u = y[:, :inter], y[:, inter:]
    return (g / (1.0 + torch.exp(-g)) * u).to(out_dtype)


def _glu(g, u, act, limit):
    """The gated pair: "silu", "gelu_tanh" or "swish_clamped" (see ``linear_glu``)."""
    if act == "silu":
        return g / (1.0 + torch.exp(-g)) * u
    if act == "gelu_tanh":
        return 0.5 * g * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g + 0.044715 * g ** 3))) * u
    if act == "swish_clamped":
        g, u = torch.clamp(g, max=limit), torch.clamp(u, min=-limit, max=limit)
        return g / (1.0 + torch.exp(-1.702 * g)) * (u + 1.0)
    raise ValueError(f"gated pair {act!r}")


def linear_glu(x, gate_up, out_dtype, act, limit=0.0):
    """``act(x @ gate^T, x @ up^T)`` for ``gate_up = [gate; up]``: "silu" ``silu(g) u``; "gelu_tanh"
    ``gelu(g) u`` in its tanh form; "swish_clamped" ``g' sigmoid(1.702 g') (u' + 1)`` with
    ``g' = min(g, limit)`` and ``u' = clamp(u, -limit, limit)``."""
    y = x.to(F64) @ gate_up.to(F64).T
    inter = y.shape[1] // 2
    return _glu(y[:, :inter], y[:, inter:], act, limit).to(out_dtype)


class ScaledRows:
    def __init__(self, x, partials, eps):
        self.x, self.partials, self.eps = x, partials, eps


def linear_into_stream(x, w, residual, next_norm_w, eps, bias=None):
    """The pair the CUDA table offers for up to 64 bfloat16 rows; here for any type, so that
    the parts' handling of it runs on the CPU too."""
    if x.shape[0] > 64:
        return None  # as the CUDA table: short steps only
    summed = residual + linear(x, w, torch.float32, bias)
    rows = (summed.to(F64) * next_norm_w.to(F64)).to(x.dtype)
    return summed, ScaledRows(rows, (summed.to(F64) ** 2).sum(-1, keepdim=True).T.contiguous(), eps)


def linear_scaled(rows, w, out_dtype, glu=False):
    k = rows.x.shape[1]
    inv = 1.0 / torch.sqrt(rows.partials.sum(0) / k + rows.eps)
    y = (rows.x.to(F64) @ w.to(F64).T) * inv[:, None]
    if glu:
        inter = y.shape[1] // 2
        g, u = y[:, :inter], y[:, inter:]
        y = g / (1.0 + torch.exp(-g)) * u
    return y.to(out_dtype)


def linear_add_rmsnorm(x, w, residual, norm_w, eps, out_dtype):
    return add_rmsnorm(residual, linear(x, w, out_dtype), norm_w, eps, out_dtype)


def linear_short_conv(x, in_proj, taps, bias, state, step):
    """``x`` is a tensor or ``ScaledRows``, as in the CUDA table."""
    if isinstance(x, ScaledRows):
        return short_conv(linear_scaled(x, in_proj, x.x.dtype), taps, bias, state, step)
    return short_conv(linear(x, in_proj, x.dtype), taps, bias, state, step)


def short_conv(proj, taps, bias, state, step):
    """y[t] = c[t] * (sum_j taps[:, j] * u[t - (L-1) + j] + bias); u = b * x; the state of
    each sequence's slot holds the last L-1 values of u (float32) and is updated."""
    T, H3 = proj.shape
    H = H3 // 3
    L = taps.shape[1]
    p = proj.to(F64)
    b, c, x = p[:, :H], p[:, H : 2 * H], p[:, 2 * H :]
    u = b * x
    y = torch.zeros(T, H, dtype=F64)
    q_start = step.q_start.tolist()
    slots = step.state_slots.tolist()
    for s in range(step.num_seqs):
        a, e = q_start[s], q_start[s + 1]
        full = torch.cat([state[slots[s]].to(F64), u[a:e]], dim=0)  # [(L-1) + n, H]
        n = e - a
        acc = torch.zeros(n, H, dtype=F64)
        for j in range(L):
            acc += taps[:, j].to(F64)[None, :] * full[j : j + n]
        if bias is not None:
            acc += bias.to(F64)[None, :]
        y[a:e] = c[a:e] * acc
        state[slots[s]] = full[-(L - 1) :].to(state.dtype)
    return y.to(proj.dtype)


def _cache_rows(block_table, seq_of_token, positions, page_size):
    pages = block_table.long()[seq_of_token.long(), (positions // page_size).long()]
    return pages * page_size + (positions % page_size).long()


def qk_norm_rope_store(qkv, heads, kv_heads, head_dim, q_w, k_w, eps, inv_freq, rotary_dim, step,
                       k_cache, v_cache, block_table, page_size, store, interleaved=False):
    T = qkv.shape[0]
    d = head_dim
    x = qkv.to(F64)
    q = x[:, : heads * d].reshape(T, heads, d)
    pos = step.positions.to(F64)

    def norm(v, w):
        if w is None:
            return v
        return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * w.to(F64)

    def rotate(v):
        if not rotary_dim:
            return v
        half = rotary_dim // 2
        # the angle in float64 from the float32 frequency table the kernel is given: a kernel that
        # forms it in float32 is off by up to position * 2^-24 radians, which its test allows for
        angle = step.positions.to(F64)[:, None] * inv_freq.to(F64)[None, :]
        cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
        out = v.clone()
        if interleaved:  # pairs of neighbours (2i, 2i + 1)
            a, b = v[..., 0:rotary_dim:2], v[..., 1:rotary_dim:2]
            out[..., 0:rotary_dim:2] = a * cos - b * sin
            out[..., 1:rotary_dim:2] = a * sin + b * cos
            return out
        a, b = v[..., :half], v[..., half:rotary_dim]
        out[..., :half] = a * cos - b * sin
        out[..., half:rotary_dim] = a * sin + b * cos
        return out

    q = rotate(norm(q, q_w))
    if kv_heads and store:
        k = x[:, heads * d : (heads + kv_heads) * d].reshape(T, kv_heads, d)
        v = x[:, (heads + kv_heads) * d :].reshape(T, kv_heads, d)
        k = rotate(norm(k, k_w))
        rows = _cache_rows(block_table, step.seq_of_token, step.positions, page_size)
        k_cache.view(-1, kv_heads, d)[rows] = k.to(k_cache.dtype)
        v_cache.view(-1, kv_heads, d)[rows] = v.to(v_cache.dtype)
    return q.reshape(T, heads * d).to(qkv.dtype)


def paged_attention(q, heads, kv_heads, head_dim, k_cache, v_cache, block_table, page_size, scale, window, step):
    T = q.shape[0]
    d = head_dim
    group = heads // kv_heads
    q64 = q.to(F64).reshape(T, heads, d)
    kf = k_cache.view(-1, kv_heads, d)
    vf = v_cache.view(-1, kv_heads, d)
    out = torch.zeros(T, heads, d, dtype=F64)
    seq = step.seq_of_token.tolist()
    pos = step.positions.tolist()
    for t in range(T):
        lo = max(0, pos[t] + 1 - window) if window else 0
        ps = torch.arange(lo, pos[t] + 1)
        pages = block_table[seq[t]].long()[(ps // page_size)]
        rows = pages * page_size + ps % page_size
        k = kf[rows].to(F64)  # [n, kv, d]
        v = vf[rows].to(F64)
        for h in range(heads):
            g = h // group
            s = (k[:, g, :] @ q64[t, h]) * scale
            p = torch.softmax(s, dim=0)
            out[t, h] = p @ v[:, g, :]
    return out.reshape(T, heads * d).to(q.dtype)


CARRIES_STATUS = True
GAVE_UP = "a kernel gave up waiting on a barrier; what it wrote is not valid"
STATUS_WORD = [0]  # a test sets it to imitate a kernel whose bounded wait ran out


def hand_over_status(status_out):
    if status_out is not None:
        status_out[0] = STATUS_WORD[0]
        STATUS_WORD[0] = 0


def suppress(logits, rows, ids):
    logits[rows.long(), ids.long()] = float("-inf")
    return logits


def argmax(logits, out=None, status_out=None):
    """Lowest id among the finite maxima (crates/shiso-engine/src/sampling.rs:91-154)."""
    hand_over_status(status_out)
    picks = torch.argmax(torch.where(torch.isfinite(logits), logits, torch.full_like(logits, float("-inf"))), dim=-1).to(torch.int32)
    if out is None:
        return picks
    out.copy_(picks)
    return out


# --------------------------------------------------------------------------- hashed-pair embedding, stream copies


def _step_ids(ids, feed_index, fed_tokens):
    ids = ids.long()
    if feed_index is not None:
        fed = fed_tokens.long()[feed_index.long().clamp(min=0)]
        ids = torch.where(feed_index.long() >= 0, fed, ids)
    return ids


def embed_hashed_pair(ids, table, pair_table, scale, buckets, mul_prev, mul_cur, step, state, feed_index=None, fed_tokens=None):
    """``scale * table[id] + pair_table[hash(previous id, id)]``; a sequence's first token takes
    row ``buckets``.  ``state[slot, 0]`` holds a request's last token + 1."""
    ids = _step_ids(ids, feed_index, fed_tokens).tolist()
    q_start, slots, starts = step.q_start.tolist(), step.state_slots.tolist(), step.start_pos.tolist()
    out = torch.zeros(len(ids), table.shape[1], dtype=F64)
    for s in range(step.num_seqs):
        a, e = q_start[s], q_start[s + 1]
        if e <= a:
            continue
        for t in range(a, e):
            if t > a:
                prev = ids[t - 1]
            elif starts[s] == 0:
                prev = None
            else:
                prev = int(state[slots[s], 0]) - 1
            row = buckets if prev is None else (prev * mul_prev + ids[t] * mul_cur) % buckets
            out[t] = table[ids[t]].to(F64) * scale + pair_table[row].to(F64)
        state[slots[s], 0] = ids[e - 1] + 1
    return out.to(torch.float32)


def _mixed_lanes(source, y, mix, write, copies):
    lanes = source.to(F64) if source.dim() == 3 else source.to(F64).unsqueeze(0).expand(copies, -1, -1)
    if y is None:
        return lanes
    return torch.einsum("sr,std->rtd", mix.to(F64), lanes) + write.to(F64)[:, None, None] * y.to(F64)[None]


def hyper_mix_read(source, y, mix, write, copies, read, weight, eps, out_dtype):
    new = _mixed_lanes(source, y, mix, write, copies)
    lanes = None
    if y is not None:
        if source.dim() == 3:
            source.copy_(new.to(source.dtype))
            lanes = source
        else:
            lanes = new.to(torch.float32).contiguous()
        new = lanes.to(F64)  # what the next sublayer reads is what was stored
    u = torch.einsum("s,std->td", read.to(F64), new)
    x = u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps) * weight.to(F64)
    return lanes, x.to(out_dtype)


def hyper_mix_sum(source, y, mix, write):
    copies = source.shape[0] if source.dim() == 3 else mix.shape[0]
    return _mixed_lanes(source, y, mix, write, copies).sum(0).to(torch.float32)


# --------------------------------------------------------------------------- time mixing, recurrences


def token_shift_blend(x, mu, state, step):
    T, H = x.shape
    x64 = x.to(F64)
    prev = torch.zeros_like(x64)
    q_start, slots = step.q_start.tolist(), step.state_slots.tolist()
    for s in range(step.num_seqs):
        a, e = q_start[s], q_start[s + 1]
        if e <= a:
            continue
        prev[a] = state[slots[s]].to(F64)
        prev[a + 1 : e] = x64[a : e - 1]
        state[slots[s]] = x64[e - 1].to(state.dtype)
    return (x64[None] + (prev - x64)[None] * mu.to(F64)[:, None, :]).to(x.dtype)


def unary(x, kind, out_dtype):
    x64 = x.to(F64)
    if kind == "tanh":
        return torch.tanh(x64).to(out_dtype)
    if kind == "silu":
        return (x64 / (1.0 + torch.exp(-x64))).to(out_dtype)
    if kind == "relu2":
        return (torch.relu(x64) ** 2).to(out_dtype)
    if kind == "copy":
        return x64.to(out_dtype)
    raise ValueError(kind)


def decay_recurrence(q, k, v, out, state, step, heads, dim, vdim, eps, *, decay_logits=None, decay_bias=None, bonus=None,
                     head_decay=None, head_loss=None, inv_freq=None, rotary_dim=0, key_scale=1.0, out_weight=None, gate=None,
                     out_scale=1.0):
    """Per head ``S[dim, vdim]``.  With ``decay_logits``: ``w = exp(-exp(logits + bias))`` per key
    channel, ``o = (S + diag(bonus) k v^T)^T q`` and then ``S = diag(w) S + k v^T``.  With
    ``head_decay``: ``S = decay S + k v^T`` and then ``o = S^T q``; q and k are rotated (half-split
    pairs of the first ``rotary_dim`` channels) and k multiplied by ``key_scale`` first.  ``o`` is
    brought to unit RMS per head, times ``out_weight``, times ``silu(gate)``, times ``out_scale``."""
    T = q.shape[0]
    q64 = q.to(F64).reshape(T, heads, dim).clone()
    k64 = k.to(F64).reshape(T, heads, dim).clone()
    v64 = v.to(F64).reshape(T, heads, vdim)
    if rotary_dim:
        half = rotary_dim // 2
        angle = step.positions.to(F64)[:, None] * inv_freq.to(F64)[None, :]
        cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
        for x in (q64, k64):
            a, b = x[..., :half].clone(), x[..., half:rotary_dim].clone()
            x[..., :half] = a * cos - b * sin
            x[..., half:rotary_dim] = b * cos + a * sin
    k64 = k64 * key_scale
    if decay_logits is not None:
        w = torch.exp(-torch.exp(decay_logits.to(F64) + decay_bias.to(F64))).reshape(T, heads, dim)
    o = torch.zeros(T, heads, vdim, dtype=F64)
    q_start, slots = step.q_start.tolist(), step.state_slots.tolist()
    for s in range(step.num_seqs):
        S = state[slots[s]].to(F64)
        for t in range(q_start[s], q_start[s + 1]):
            kv = k64[t][:, :, None] * v64[t][:, None, :]
            if decay_logits is not None:
                o[t] = torch.einsum("hi,hij->hj", q64[t], S + bonus.to(F64)[:, :, None] * kv)
                S = w[t][:, :, None] * S + kv
            else:
                S = head_decay.to(F64)[:, None, None] * S + kv
                o[t] = torch.einsum("hi,hij->hj", q64[t], S)
        if q_start[s + 1] > q_start[s]:
            state[slots[s]] = S.to(state.dtype)
    o = (o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps)).reshape(T, heads * vdim)
    if out_weight is not None:
        o = o * out_weight.to(F64)
    if gate is not None:
        g = gate.to(F64)
        o = o * (g / (1.0 + torch.exp(-g)))
    out.copy_((o * out_scale).to(out.dtype))
    return out


# --------------------------------------------------------------------------- windowed attention with pooled blocks


def store_kv(k, v, kv_heads, dim, vdim, step, k_cache, v_cache, block_table, page_size):
    rows = _cache_rows(block_table, step.seq_of_token, step.positions, page_size)
    T = k.shape[0]
    k_cache.view(-1, kv_heads, dim)[rows] = k.reshape(T, kv_heads, dim).to(k_cache.dtype)
    v_cache.view(-1, kv_heads, vdim)[rows] = v.reshape(T, kv_heads, vdim).to(v_cache.dtype)


def pool_kv(k_cache, v_cache, block_table, pooled_k, pooled_v, pooled_table, page_size, pool, step):
    """For every row whose position ends a block of ``pool`` positions: the means of the block's
    cached keys and values, stored as row ``position // pool`` of the pooled caches."""
    kf, vf = k_cache.flatten(0, 1), v_cache.flatten(0, 1)
    pkf, pvf = pooled_k.flatten(0, 1), pooled_v.flatten(0, 1)
    seq, pos = step.seq_of_token.tolist(), step.positions.tolist()
    for t in range(len(pos)):
        if (pos[t] + 1) % pool:
            continue
        ps = torch.arange(pos[t] + 1 - pool, pos[t] + 1)
        rows = block_table[seq[t]].long()[ps // page_size] * page_size + ps % page_size
        b = pos[t] // pool
        at = int(pooled_table[seq[t], b // page_size]) * page_size + b % page_size
        pkf[at] = kf[rows].to(F64).mean(0).to(pooled_k.dtype)
        pvf[at] = vf[rows].to(F64).mean(0).to(pooled_v.dtype)


def pooled_window_attention(q, heads, k_cache, v_cache, block_table, pooled_k, pooled_v, pooled_table, page_size, scale,
                            window, pool, step, out, out_scale=1.0):
    T = q.shape[0]
    kv_heads, d, dv = k_cache.shape[2], k_cache.shape[3], v_cache.shape[3]
    group = heads // kv_heads
    q64 = q.to(F64).reshape(T, heads, d)
    kf, vf = k_cache.flatten(0, 1), v_cache.flatten(0, 1)
    pkf, pvf = pooled_k.flatten(0, 1), pooled_v.flatten(0, 1)
    res = torch.zeros(T, heads, dv, dtype=F64)
    seq, pos = step.seq_of_token.tolist(), step.positions.tolist()
    for t in range(T):
        i = pos[t]
        ps = torch.arange(max(0, i - window + 1), i + 1)
        rows = block_table[seq[t]].long()[ps // page_size] * page_size + ps % page_size
        keys, values = kf[rows].to(F64), vf[rows].to(F64)
        blocks = max(0, (i - window + 1) // pool)
        if blocks:
            bs = torch.arange(blocks)
            prow = pooled_table[seq[t]].long()[bs // page_size] * page_size + bs % page_size
            keys = torch.cat([pkf[prow].to(F64), keys])
            values = torch.cat([pvf[prow].to(F64), values])
        for h in range(heads):
            g = h // group
            p = torch.softmax((keys[:, g] @ q64[t, h]) * scale, dim=0)
            res[t, h] = p @ values[:, g]
    out.copy_((res.reshape(T, heads * dv) * out_scale).to(out.dtype))
    return out


# --------------------------------------------------------------------------- layer norm, parallel layers


def add_layernorm(residual, deltas, w, eps, out_dtype, rows=None):
    """``residual`` plus every tensor of ``deltas`` (summed in place without ``rows``), then
    ``(x - mean) / sqrt(var + eps) * w``."""
    if rows is None:
        for d in deltas:
            residual += d.to(residual.dtype)
        x = residual.to(F64)
    else:
        idx = rows.long()
        x = residual[idx].clone()
        for d in deltas:
            x = x + d[idx].to(residual.dtype)
        x = x.to(F64)
    dev = x - x.mean(-1, keepdim=True)
    return (dev / torch.sqrt((dev * dev).mean(-1, keepdim=True) + eps) * w.to(F64)).to(out_dtype)


# --------------------------------------------------------------------------- causal convolution, scalar-decay recurrences


def _sigmoid(x):
    return 1.0 / (1.0 + torch.exp(-x))


def causal_conv(x, taps, bias, state, step, silu=True):
    """``y_t[c] = bias[c] + sum_j taps[c, j] x_{t-(L-1)+j}[c]`` per sequence, then silu; the state
    of each sequence's slot holds its last ``L - 1`` inputs (float32) and is updated."""
    T, C = x.shape
    L = taps.shape[1]
    x64 = x.to(F64)
    y = torch.zeros(T, C, dtype=F64)
    q_start, slots = step.q_start.tolist(), step.state_slots.tolist()
    for s in range(step.num_seqs):
        a, e = q_start[s], q_start[s + 1]
        if e == a:
            continue
        full = torch.cat([state[slots[s]].to(F64), x64[a:e]], dim=0)
        acc = torch.zeros(e - a, C, dtype=F64)
        for j in range(L):
            acc += taps[:, j].to(F64)[None, :] * full[j : j + e - a]
        if bias is not None:
            acc += bias.to(F64)[None, :]
        y[a:e] = acc
        state[slots[s]] = full[-(L - 1):].to(state.dtype)
    if silu:
        y = y * _sigmoid(y)
    return y.to(x.dtype)


def state_recurrence(q, k, v, state, step, heads, groups, dim, vdim, *, silu_inputs=False, head_loss=None,
                     dt=None, dt_bias=None, a_log=None, skip=None):
    """Per head ``S[dim, vdim]``: ``S = a S + b k v^T``, ``o = S^T q + skip v``.  With ``head_loss``:
    ``a = 1 - head_loss[h]``, ``b = 1``.  With ``dt``: ``b = softplus(dt + dt_bias[h])``,
    ``a = exp(-exp(a_log[h]) b)``.  Head ``h`` reads q and k of group ``h // (heads / groups)``;
    ``silu_inputs`` applies silu to q, k and v first.  Returns float32 ``[T, heads * vdim]``."""
    T = q.shape[0]
    q64, k64, v64 = q.to(F64), k.to(F64), v.to(F64)
    if silu_inputs:
        q64, k64, v64 = q64 * _sigmoid(q64), k64 * _sigmoid(k64), v64 * _sigmoid(v64)
    per = heads // groups
    q64 = q64.reshape(T, groups, dim).repeat_interleave(per, dim=1)
    k64 = k64.reshape(T, groups, dim).repeat_interleave(per, dim=1)
    v64 = v64.reshape(T, heads, vdim)
    if dt is not None:
        z = dt.to(F64) + dt_bias.to(F64)
        b = torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))
        a = torch.exp(-torch.exp(a_log.to(F64)) * b)
    else:
        a = (1.0 - head_loss.to(F64))[None, :].expand(T, heads)
        b = torch.ones(T, heads, dtype=F64)
    o = torch.zeros(T, heads, vdim, dtype=F64)
    q_start, slots = step.q_start.tolist(), step.state_slots.tolist()
    for s in range(step.num_seqs):
        if q_start[s + 1] == q_start[s]:
            continue
        S = state[slots[s]].to(F64)
        for t in range(q_start[s], q_start[s + 1]):
            S = a[t][:, None, None] * S + b[t][:, None, None] * k64[t][:, :, None] * v64[t][:, None, :]
            o[t] = torch.einsum("hi,hij->hj", q64[t], S)
        state[slots[s]] = S.to(state.dtype)
    if skip is not None:
        o = o + skip.to(F64)[None, :, None] * v64
    return o.reshape(T, heads * vdim).to(torch.float32)


def group_rmsnorm(x, weight, eps, groups, out_dtype, gate=None, gate_mode=None):
    """Rows in ``groups`` equal parts, each divided by its own root mean square, times ``weight``.
    ``gate_mode`` ``"silu_before"``: the rows are multiplied by ``silu(gate)`` first;
    ``"sigmoid_after"``: the result is multiplied by ``sigmoid(gate)``."""
    T, W = x.shape
    y = x.to(F64)
    if gate_mode == "silu_before":
        g = gate.to(F64)
        y = y * g * _sigmoid(g)
    y = y.reshape(T, groups, W // groups)
    y = (y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)).reshape(T, W) * weight.to(F64)
    if gate_mode == "sigmoid_after":
        y = y * _sigmoid(gate.to(F64))
    return y.to(out_dtype)


# --------------------------------------------------------------------------- latent attention


def _rotate_rows(v, positions, inv_freq, rotary_dim, magnitude=1.0, interleaved=False):
    if not rotary_dim:
        return v
    half = rotary_dim // 2
    angle = positions.to(F64)[:, None] * inv_freq.to(F64)[None, :]
    cos, sin = torch.cos(angle) * magnitude, torch.sin(angle) * magnitude
    while cos.dim() < v.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    out = v.clone()
    if interleaved:  # pair i: the neighbours (2i, 2i + 1)
        a, b = v[..., 0:rotary_dim:2], v[..., 1:rotary_dim:2]
        out[..., 0:rotary_dim:2] = a * cos - b * sin
        out[..., 1:rotary_dim:2] = b * cos + a * sin
        return out
    a, b = v[..., :half], v[..., half:rotary_dim]
    out[..., :half] = a * cos - b * sin
    out[..., half:rotary_dim] = b * cos + a * sin
    return out


def latent_store(rows, rank, norm_w, eps, inv_freq, rotary_dim, step, k_cache, block_table, page_size, magnitude=1.0,
                 interleaved=False):
    """Each row ``[latent (rank) | shared key part]``: the latent RMS-normed with ``norm_w``, the
    rest rotated by the row's position; stored as the position's row of the cache."""
    x = rows.to(F64)
    c = x[:, :rank]
    c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * norm_w.to(F64)
    shared = _rotate_rows(x[:, rank:], step.positions, inv_freq, rotary_dim, magnitude, interleaved)
    at = _cache_rows(block_table, step.seq_of_token, step.positions, page_size)
    k_cache.view(-1, k_cache.shape[-1])[at] = torch.cat([c, shared], dim=-1).to(k_cache.dtype)


def rotate_heads(x, out, inv_freq, rotary_dim, step, magnitude=1.0, interleaved=False):
    """``x[T, H, P]`` rotated by each row's position into ``out[T, H, P]`` (both may be column ranges)."""
    out.copy_(_rotate_rows(x.to(F64), step.positions, inv_freq, rotary_dim, magnitude, interleaved).to(out.dtype))


def head_linear(x, w, out, gate=None):
    """``out[t, h] = w[h] x[t, h]`` for ``x[T, H, K]``, ``w[H, N, K]``, ``out[T, H, N]``; with
    ``gate[T, H]`` the head's result is multiplied by ``sigmoid(gate[t, h])``."""
    y = torch.einsum("thk,hnk->thn", x.to(F64), w.to(F64))
    if gate is not None:
        y = y * _sigmoid(gate.to(F64))[:, :, None]
    out.copy_(y.to(out.dtype))


def latent_attention(q_lat, rank, k_cache, block_table, page_size, scale, step):
    """Causal softmax attention of ``q_lat[T, H, D]`` against cached rows of ``D``; the values are
    the first ``rank`` entries of the same rows.  Returns ``[T, H, rank]``."""
    T, H, D = q_lat.shape
    q64 = q_lat.to(F64)
    kf = k_cache.view(-1, D)
    out = torch.zeros(T, H, rank, dtype=F64)
    seq, pos = step.seq_of_token.tolist(), step.positions.tolist()
    for t in range(T):
        ps = torch.arange(0, pos[t] + 1)
        at = block_table[seq[t]].long()[ps // page_size] * page_size + ps % page_size
        k = kf[at].to(F64)
        p = torch.softmax((q64[t] @ k.T) * scale, dim=-1)  # [H, n]
        out[t] = p @ k[:, :rank]
    return out.to(q_lat.dtype)


# --------------------------------------------------------------------------- mixture of experts


def moe_route(logits, top, group_count, group_keep, scale, sigmoid=False, renormalize=False, correction=None, renorm_eps=0.0):
    """Expert ids (int32 ``[T, top]``, best first) and weights (float32) of every row.  Groups and
    experts are ranked by score + ``correction``; the weights are the scores themselves."""
    T, E = logits.shape
    z = logits.to(F64)
    s = _sigmoid(z) if sigmoid else torch.softmax(z, dim=-1)
    choice = s if correction is None else s + correction.to(F64)
    per = E // group_count
    best = choice.reshape(T, group_count, per).max(-1).values
    order = torch.sort(best, dim=-1, descending=True, stable=True).indices[:, :group_keep]
    kept = torch.zeros(T, group_count, dtype=torch.bool, device=logits.device)
    kept.scatter_(1, order, True)
    allowed = kept[:, :, None].expand(T, group_count, per).reshape(T, E)
    masked = torch.where(allowed, choice, torch.full_like(s, float("-inf")))
    ids = torch.sort(masked, dim=-1, descending=True, stable=True).indices[:, :top]
    w = torch.gather(s, 1, ids)
    if renormalize:
        w = w / (w.sum(-1, keepdim=True) + renorm_eps)
    return ids.to(torch.int32), (w * scale).to(torch.float32)


def routed_experts(x, ids, weights, gate_up, down, extra=None, act="silu", limit=0.0, extra_gate=None, identity=0):
    """``sum_j weights[t, j] * expert_{ids[t, j]}(x[t])`` (+ ``extra``, times ``sigmoid(extra_gate[t])``
    where one is given), in ``x``'s type.  An id from the number of stacked matrices on is an
    identity expert: its output is ``x[t]``."""
    T, H = x.shape
    x64 = x.to(F64)
    out = torch.zeros(T, H, dtype=F64)
    if extra is not None:
        out = extra.to(F64).clone()
        if extra_gate is not None:
            out = out * _sigmoid(extra_gate.to(F64)).reshape(T, 1)
    inter = gate_up.shape[1] // 2
    for t in range(T):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            if e >= gate_up.shape[0]:
                assert e < gate_up.shape[0] + identity, f"choice {e} beyond the experts and identity experts"
                out[t] += float(weights[t, j]) * x64[t]
                continue
            y = gate_up[e].to(F64) @ x64[t]
            mid = _glu(y[:inter], y[inter:], act, limit)
            out[t] += float(weights[t, j]) * (down[e].to(F64) @ mid)
    return out.to(x.dtype)


# --------------------------------------------------------------------------- attention with a parameterised mask and weighting


def head_prepare_store(proj, heads, kv_heads, dim, vdim, q_w, k_w, eps, norm_order, inv_freq, rotary_dim, magnitude, step,
                       k_cache, v_cache, block_table, page_size, store=True):
    T = proj.shape[0]
    x = proj.to(F64)
    q_cols, k_cols = heads * dim, kv_heads * dim

    def norm(v, w):
        v = v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)
        return v if w is None else v * w.to(F64)

    def prepare(v, w):
        if norm_order == "before":
            v = norm(v, w)
        if rotary_dim:
            v = _rotate_rows(v, step.positions, inv_freq, rotary_dim, magnitude)
        if norm_order == "after":
            v = norm(v, w)
        return v

    q = prepare(x[:, :q_cols].reshape(T, heads, dim), q_w)
    proj[:, :q_cols] = q.reshape(T, q_cols).to(proj.dtype)
    if store:
        k = prepare(x[:, q_cols : q_cols + k_cols].reshape(T, kv_heads, dim), k_w)
        v = proj[:, q_cols + k_cols : q_cols + k_cols + kv_heads * vdim].reshape(T, kv_heads, vdim)
        rows = _cache_rows(block_table, step.seq_of_token, step.positions, page_size)
        k_cache.view(-1, kv_heads, dim)[rows] = k.to(k_cache.dtype)
        v_cache.view(-1, kv_heads, vdim)[rows] = v.to(v_cache.dtype)
    return proj[:, :q_cols]


def joined_norm_store(proj, heads, kv_heads, dim, vdim, q_w, k_w, eps, q_temperature, values_from_keys, step, k_cache, v_cache,
                      block_table, page_size):
    """``proj[T, heads*dim | kv_heads*dim | (kv_heads*vdim) | ...]``: one RMS norm over all query
    columns together (weight ``q_w[heads*dim]``) and one over all key columns; the queries times
    ``1 + coef * ln(floor((p + 1) / every) + 1)`` when ``q_temperature = (coef, every)``; queries
    written back in place, keys to the cache; the values are the key columns as they came
    (``values_from_keys``) or the value columns."""
    T = proj.shape[0]
    x = proj.to(F64)
    q_cols, k_cols = heads * dim, kv_heads * dim

    def norm(v, w):
        return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * w.to(F64)

    q = norm(x[:, :q_cols], q_w)
    if q_temperature is not None:
        coef, every = q_temperature
        q = q * (1.0 + coef * torch.log(torch.floor((step.positions.to(F64) + 1.0) / every) + 1.0))[:, None]
    k = norm(x[:, q_cols : q_cols + k_cols], k_w)
    if values_from_keys:
        v = proj[:, q_cols : q_cols + k_cols].clone()
    else:
        v = proj[:, q_cols + k_cols : q_cols + k_cols + kv_heads * vdim]
    proj[:, :q_cols] = q.to(proj.dtype)
    rows = _cache_rows(block_table, step.seq_of_token, step.positions, page_size)
    k_cache.view(-1, kv_heads, dim)[rows] = k.reshape(T, kv_heads, dim).to(k_cache.dtype)
    v_cache.view(-1, kv_heads, vdim)[rows] = v.reshape(T, kv_heads, vdim).to(v_cache.dtype)
    return proj[:, :q_cols]


def masked_attention(q, heads, k_cache, v_cache, block_table, page_size, scale, mask, size, keep_first, step, *, sigmoid=False,
                     key_bias=None, softcap=None, gate=None, general=False, gate_per_element=False):
    T = q.shape[0]
    kv_heads, dim, vdim = k_cache.shape[2], k_cache.shape[3], v_cache.shape[3]
    q64 = q.to(F64).reshape(T, heads, dim)
    kf, vf = k_cache.view(-1, kv_heads, dim), v_cache.view(-1, kv_heads, vdim)
    out = torch.zeros(T, heads, vdim, dtype=F64)
    seq, pos = step.seq_of_token.tolist(), step.positions.tolist()
    for t in range(T):
        i = pos[t]
        if mask == "chunk":
            seen = list(range(i // size * size, i + 1))
        else:
            first = max(0, i - size + 1)
            seen = list(range(min(keep_first, first))) + list(range(first, i + 1))
        ps = torch.tensor(seen)
        pages = block_table[seq[t]].long()[ps // page_size]
        assert (pages >= 0).all(), f"row {t} at position {i} reads a page that went back"
        rows = pages * page_size + ps % page_size
        k, v = kf[rows].to(F64), vf[rows].to(F64)
        for h in range(heads):
            g = h // (heads // kv_heads)
            s = (k[:, g, :] @ q64[t, h]) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            if sigmoid:
                w = torch.sigmoid(s + (float(key_bias[h]) if key_bias is not None else 0.0))
            else:
                w = torch.softmax(s, dim=0)
            out[t, h] = w @ v[:, g, :]
            if gate is not None and gate_per_element:
                out[t, h] *= torch.sigmoid(gate[t, h * vdim : (h + 1) * vdim].to(F64))
            elif gate is not None:
                out[t, h] *= torch.sigmoid(gate[t, h].to(F64))
    return out.reshape(T, heads * vdim).to(q.dtype)


def norm_into(residual, y, w, eps, want_rows=True):
    y64 = y.to(F64)
    total = residual.to(F64) + y64 / torch.sqrt((y64 * y64).mean(-1, keepdim=True) + eps) * w.to(F64)
    residual.copy_(total.to(residual.dtype))
    if not want_rows:
        return None
    return residual if y.dtype == torch.float32 else residual.to(y.dtype)


def polynorm(z, coefficients, eps, out_dtype):
    z64 = z.to(F64)
    a, b, c, e = (float(v) for v in coefficients)

    def unit(u):
        return u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps)

    return (a * unit(z64) + b * unit(z64 * z64) + c * unit(z64 ** 3) + e).to(out_dtype)
