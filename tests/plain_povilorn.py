"""Povilorn, stated plainly: a whole sequence at a time, in float64, one function per mechanism.

This is the tests' oracle.  It shares nothing with the engine: it reads the configuration
document and a dict of tensors.  Notation: ``x`` is the residual stream ``[T, width]``, ``h`` a
sublayer's normed input, ``p`` a row's position in its sequence (from 0), ``eps`` the layers'
epsilon.

A layer is pre-norm, ``x <- x + mixer(N1(x))`` then ``x <- x + ff(N2(x))``, where a norm is a
squashing without statistics, ``N(x) = tanh(alpha x) * w + b``.  Mixers: ``attention`` (grouped
queries, values that are the keys, one RMS norm over all heads together, a query temperature
that grows with the position, an elementwise output gate) and ``latent_attention`` (keys and
values expanded from a cached latent, one rotated key part shared by the heads, neighbouring
rotation pairs on a stretched frequency ladder).  Feed-forwards: ``dense`` (a gated pair with
the tanh form of gelu) and ``moe`` (a softmax router with a correction on the choice, groups,
identity experts, clamped experts, a gated shared expert).  A run of layers may repeat; every
pass begins by adding a vector of its own, and every pass after the first the embedding rows.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def _w(tensors, name):
    return tensors[name].to(F64)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z**3)))


def squash_norm(x, tensors, name):
    """``tanh(alpha x) * w + b``: no mean, no variance, no epsilon."""
    return torch.tanh(_w(tensors, f"{name}.alpha") * x) * _w(tensors, name) + _w(tensors, f"{name}.b")


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def softmax_causal(scores):
    """``scores[T, T]`` (row = query position): softmax over the keys ``j <= i``."""
    T = scores.shape[0]
    hidden = torch.triu(torch.ones((T, T), dtype=torch.bool), diagonal=1)
    return torch.softmax(scores.masked_fill(hidden, float("-inf")), dim=-1)


# --------------------------------------------------------------------------- mixers


def query_temperature(positions, coef, every):
    """``1 + coef * ln(floor((p + 1) / every) + 1)``."""
    return 1.0 + coef * torch.log(torch.floor((positions.to(F64) + 1.0) / every) + 1.0)


def attention(tensors, prefix, m, h, eps):
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    positions = torch.arange(T)
    q = h @ _w(tensors, f"{prefix}.q").T + _w(tensors, f"{prefix}.q.b")
    k = h @ _w(tensors, f"{prefix}.k").T + _w(tensors, f"{prefix}.k.b")
    v = k  # as projected: the keys before their norm
    q = rms_norm(q, _w(tensors, f"{prefix}.q.norm"), eps)  # over all heads' entries together
    k = rms_norm(k, _w(tensors, f"{prefix}.k.norm"), eps)
    if m.get("q_temp") is not None:
        q = q * query_temperature(positions, m["q_temp"]["coef"], m["q_temp"]["every"])[:, None]
    q, k, v = q.view(T, H, D), k.view(T, G, D), v.view(T, G, V)
    out = torch.zeros((T, H, V), dtype=F64)
    for a in range(H):
        g = a // (H // G)
        weights = softmax_causal(q[:, a] @ k[:, g].T * m["scale"])
        out[:, a] = weights @ v[:, g]
    gate = torch.sigmoid(h @ _w(tensors, f"{prefix}.g").T)
    return (out.reshape(T, H * V) * gate) @ _w(tensors, f"{prefix}.o").T


def stretched_ladder(rot):
    """Frequencies of the pairs and the factor on cosine and sine."""
    dims, base = rot["dims"], rot["base"]
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    s = rot.get("scaling")
    if s is None:
        return f, 1.0

    def pair_of(turns):
        return dims * math.log(s["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(s["fast"])), 0)
    hi = min(math.ceil(pair_of(s["slow"])), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / s["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(s["factor"]) + 1.0


def rotate_neighbours(x, positions, rot):
    """Entries ``2i`` and ``2i + 1`` of the first ``rot.dims`` entries of ``x[T, ..., D]`` turn by
    ``p * f_i``; the rest pass."""
    dims = rot["dims"]
    f, magnitude = stretched_ladder(rot)
    angle = positions.to(F64)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = (torch.cos(angle) * magnitude).view(shape), (torch.sin(angle) * magnitude).view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    turned = torch.stack([u * cos - v * sin, v * cos + u * sin], dim=-1).flatten(-2)
    return torch.cat([turned, x[..., dims:]], dim=-1)


def latent_attention(tensors, prefix, m, h, eps):
    H, D, P, V, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    positions = torch.arange(T)
    q = (h @ _w(tensors, f"{prefix}.q").T).view(T, H, D + P)
    down = h @ _w(tensors, f"{prefix}.dkv").T
    c = rms_norm(down[:, :R], _w(tensors, f"{prefix}.dkv.norm"), eps)
    k_rot = rotate_neighbours(down[:, R:], positions, m["rot"])  # one for all heads
    q_rot = rotate_neighbours(q[:, :, D:], positions, m["rot"])
    k_plain = (c @ _w(tensors, f"{prefix}.uk").T).view(T, H, D)
    values = (c @ _w(tensors, f"{prefix}.uv").T).view(T, H, V)
    out = torch.zeros((T, H, V), dtype=F64)
    for a in range(H):
        scores = (q[:, a, :D] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        out[:, a] = softmax_causal(scores) @ values[:, a]
    return out.reshape(T, H * V) @ _w(tensors, f"{prefix}.o").T


# --------------------------------------------------------------------------- feed-forwards


def dense_ff(tensors, prefix, h):
    return (gelu_tanh(h @ _w(tensors, f"{prefix}.gate").T) * (h @ _w(tensors, f"{prefix}.up").T)) @ _w(tensors, f"{prefix}.down").T


def clamped_expert(tensors, prefix, h, limit):
    g = torch.clamp(h @ _w(tensors, f"{prefix}.gate").T, max=limit)
    u = torch.clamp(h @ _w(tensors, f"{prefix}.up").T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ _w(tensors, f"{prefix}.down").T


def route(choice, top, count, keep):
    """``choice[T, E]`` -> a boolean ``[T, E]`` of the ``top`` best entries among the ``keep`` best
    of ``count`` groups of neighbours; a group is as good as its best entry."""
    T, E = choice.shape
    best = choice.view(T, count, E // count).max(-1).values
    kept = torch.zeros((T, count), dtype=torch.bool)
    kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
    open_ = kept[:, :, None].expand(T, count, E // count).reshape(T, E)
    ranked = choice.masked_fill(~open_, float("-inf"))
    chosen = torch.zeros((T, E), dtype=torch.bool)
    chosen.scatter_(1, ranked.topk(top, dim=-1).indices, True)
    return chosen


def route_margin(choice, chosen, count):
    """Per token: how far the nearest decision was from falling the other way (the smallest gap
    between a chosen and an unchosen entry among the open ones, and between a kept and a dropped
    group).  Rows with a tiny margin may route differently in reduced precision."""
    T, E = choice.shape
    inf = float("inf")
    lowest_in = choice.masked_fill(~chosen, inf).min(-1).values
    highest_out = choice.masked_fill(chosen, -inf).max(-1).values
    margin = lowest_in - highest_out
    best = choice.view(T, count, E // count).max(-1).values
    order = best.sort(-1, descending=True).values
    gaps = order[:, :-1] - order[:, 1:]
    if gaps.numel():
        margin = torch.minimum(margin, gaps.min(-1).values)
    return margin


def moe_ff(tensors, prefix, mlp, h, margins=None):
    r = mlp["router"]
    experts, identity = r["experts"], r.get("identity", 0)
    scores = torch.softmax(h @ _w(tensors, f"{prefix}.router").T, dim=-1)  # over experts and identity experts
    choice = scores + _w(tensors, f"{prefix}.correction")
    groups = r.get("groups") or {"count": 1, "keep": 1}
    chosen = route(choice, r["top"], groups["count"], groups["keep"])
    if margins is not None:
        margins.append(route_margin(choice, chosen, groups["count"]))
    picked = scores * chosen
    weights = picked / (picked.sum(-1, keepdim=True) + 1e-20)
    out = torch.zeros_like(h)
    for e in range(experts):
        rows = chosen[:, e].nonzero().flatten()
        if rows.numel():
            out[rows] += weights[rows, e : e + 1] * clamped_expert(tensors, f"{prefix}.e{e}", h[rows], mlp["expert"]["limit"])
    for e in range(experts, experts + identity):
        out += weights[:, e : e + 1] * h
    if mlp.get("shared") is not None:
        gate = torch.sigmoid(h @ _w(tensors, f"{prefix}.shared.sg").T)  # one number per token
        out = out + gate * clamped_expert(tensors, f"{prefix}.shared", h, mlp["shared"]["limit"])
    return out


# --------------------------------------------------------------------------- the model

MIXERS = {"attention": attention, "latent_attention": latent_attention}


def run_order(doc):
    """``(layer, pass number or None)`` in running order; the pass number stands at a pass's first layer."""
    n = len(doc["layers"])
    loop = doc.get("loop")
    if loop is None:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], n)]


def forward(doc, tensors, tokens, after_layer=None, margins=None):
    """Logits ``[T, vocab]`` (float64) of a whole sequence; ``after_layer(run, x)`` sees the
    residual rows after every layer run; ``margins`` is given one ``route_margin`` per routed run."""
    eps = doc["norm"]["eps"]
    first = _w(tensors, "embed")[torch.as_tensor(tokens, dtype=torch.long)] * (doc.get("embedding") or {}).get("scale", 1.0)
    x = first.clone()
    for run, (i, begins) in enumerate(run_order(doc)):
        layer = doc["layers"][i]
        if begins is not None:
            if begins > 0:
                x = x + first
            x = x + _w(tensors, "loop.step")[begins]
        x = x + MIXERS[layer["type"]](tensors, f"l{i}.mix", layer["mixer"], squash_norm(x, tensors, f"l{i}.norm1"), eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = squash_norm(x, tensors, f"l{i}.norm2")
            x = x + (dense_ff(tensors, f"l{i}.mlp", h) if mlp["kind"] == "dense" else moe_ff(tensors, f"l{i}.mlp", mlp, h, margins))
        if after_layer is not None:
            after_layer(run, x)
    return squash_norm(x, tensors, "final.norm") @ _w(tensors, "head").T
