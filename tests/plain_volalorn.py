"""Volalorn, stated plainly: in float64, one function per mechanism, masks written out key by key.

This is the tests' oracle.  It shares nothing with the engine: it reads the configuration
document and a dict of tensors and works on a whole sequence ``x[T, width]`` at positions
``0 .. T-1``.

A layer norms what its sublayers give back, not what they read: ``x <- x + g1 * unit(mixer(x))``,
then ``x <- x + g2 * unit(ff(x))``, where ``unit(y) = y / sqrt(mean(y^2) + eps)`` and ``g`` is one
number.  Mixers: ``attention`` (grouped-query, rotation with stretched frequencies, unit-RMS
queries and keys, capped scores, keys of the own chunk only, a sigmoid per key instead of a
softmax, a gate per head) and ``attention_2`` (grouped-query with biases, weighted RMS norm of
queries and keys before the rotation, a sliding window that also keeps the first tokens,
softmax).  Feed-forward: ``W_down poly(W_up x)`` with a polynomial of unit-RMS powers.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def _w(tensors, name):
    return tensors[name].to(F64)


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose weight is one number."""
    return unit_rms(x, eps) * g.reshape(())


def frequencies(rot):
    """Rotation frequency of every pair, and the factor on cos and sin.  Without ``scaling`` the
    ladder is ``base^(-2i/dims)`` and the factor 1.  With it, pair ``i`` is blended between the
    ladder's value and that value divided by ``factor``, by a ramp over the pair index that runs
    from the pair turning ``fast`` times in ``original`` positions to the one turning ``slow`` times."""
    dims, base = rot["dims"], float(rot["base"])
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    s = rot.get("scaling")
    if s is None:
        return torch.tensor(f, dtype=F64), 1.0

    def pair_turning(times):
        return dims * math.log(s["original"] / (2.0 * math.pi * times)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_turning(s["fast"])), 0)
    hi = min(math.ceil(pair_turning(s["slow"])), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / s["factor"] * ramp + f[i] * (1.0 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(s["factor"]) + 1.0


def rotate(x, positions, rot):
    """``x[T, heads, D]``: entry ``i`` of the first ``dims`` is paired with ``i + dims/2``."""
    freq, factor = frequencies(rot)
    dims = rot["dims"]
    half = dims // 2
    angle = positions.to(F64)[:, None] * freq[None, :]
    cos, sin = (torch.cos(angle) * factor)[:, None, :], (torch.sin(angle) * factor)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def sees_chunk(i, j, size):
    return j <= i and i // size == j // size


def sees_window(i, j, size, keep_first):
    return j <= i and (i - j < size or j < keep_first)


def visibility(positions, sees):
    """``[T, T]`` booleans: row ``a`` sees key ``b``; asked key by key."""
    p = [int(v) for v in positions]
    return torch.tensor([[sees(i, j) for j in p] for i in p], dtype=torch.bool)


def chunk_sigmoid_attention(tensors, p, m, h, eps, positions=None):
    T = h.shape[0]
    positions = torch.arange(T) if positions is None else positions
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ _w(tensors, f"{p}.q").T).reshape(T, H, D)
    k = (h @ _w(tensors, f"{p}.k").T).reshape(T, G, D)
    v = (h @ _w(tensors, f"{p}.v").T).reshape(T, G, V)
    q = unit_rms(rotate(q, positions, m["rot"]), eps)
    k = unit_rms(rotate(k, positions, m["rot"]), eps)
    bias = _w(tensors, f"{p}.pb")
    gate = torch.sigmoid(h @ _w(tensors, f"{p}.g").T)  # [T, H]
    cap = m.get("softcap")
    seen = visibility(positions, lambda i, j: sees_chunk(i, j, m["mask"]["size"]))
    out = torch.zeros((T, H, V), dtype=F64)
    for head in range(H):
        kv = head // (H // G)
        score = q[:, head] @ k[:, kv].T * m["scale"]
        if cap is not None:
            score = cap * torch.tanh(score / cap)
        weight = torch.where(seen, torch.sigmoid(score + bias[head]), torch.zeros((), dtype=F64))  # not normalised over keys
        out[:, head] = (weight @ v[:, kv]) * gate[:, head : head + 1]
    return out.reshape(T, H * V) @ _w(tensors, f"{p}.o").T


def window_softmax_attention(tensors, p, m, h, eps, positions=None):
    T = h.shape[0]
    positions = torch.arange(T) if positions is None else positions
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ _w(tensors, f"{p}.q").T + _w(tensors, f"{p}.q.b")).reshape(T, H, D)
    k = (h @ _w(tensors, f"{p}.k").T + _w(tensors, f"{p}.k.b")).reshape(T, G, D)
    v = (h @ _w(tensors, f"{p}.v").T + _w(tensors, f"{p}.v.b")).reshape(T, G, V)
    q = rotate(unit_rms(q, eps) * _w(tensors, f"{p}.q.norm"), positions, m["rot"])
    k = rotate(unit_rms(k, eps) * _w(tensors, f"{p}.k.norm"), positions, m["rot"])
    size, keep = m["mask"]["size"], m["mask"].get("keep_first", 0)
    seen = visibility(positions, lambda i, j: sees_window(i, j, size, keep))
    out = torch.zeros((T, H, V), dtype=F64)
    for head in range(H):
        kv = head // (H // G)
        score = q[:, head] @ k[:, kv].T * m["scale"]
        weight = torch.softmax(torch.where(seen, score, torch.full((), -math.inf, dtype=F64)), dim=-1)
        out[:, head] = weight @ v[:, kv]
    return out.reshape(T, H * V) @ _w(tensors, f"{p}.o").T


def poly_norm(z, coefficients, eps):
    a, b, c, e = (float(t) for t in coefficients)
    return a * unit_rms(z, eps) + b * unit_rms(z * z, eps) + c * unit_rms(z * z * z, eps) + e


def dense_ff(tensors, p, h, eps):
    z = h @ _w(tensors, f"{p}.up").T
    return poly_norm(z, _w(tensors, f"{p}.act"), eps) @ _w(tensors, f"{p}.down").T


MIXERS = {"attention": chunk_sigmoid_attention, "attention_2": window_softmax_attention}


def forward(doc, tensors, tokens, after_layer=None):
    """Logits ``[T, vocab]`` (float64) of a whole sequence; ``after_layer(i, x)`` sees the
    residual rows after every layer."""
    eps = doc["norm"]["eps"]
    x = _w(tensors, "embed")[torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(doc["layers"]):
        y = MIXERS[layer["type"]](tensors, f"l{i}.mix", layer["mixer"], x, eps)
        x = x + scalar_norm(y, _w(tensors, f"l{i}.norm1"), eps)
        if layer.get("mlp") is not None:
            x = x + scalar_norm(dense_ff(tensors, f"l{i}.mlp", x, eps), _w(tensors, f"l{i}.norm2"), eps)
        if after_layer is not None:
            after_layer(i, x)
    x = scalar_norm(x, _w(tensors, "final.norm"), eps)
    return x @ _w(tensors, "head").T * doc.get("logit_scale", 1.0)
