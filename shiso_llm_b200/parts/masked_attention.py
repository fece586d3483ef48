"""Grouped-query attention whose mask, weighting and head preparation are parameters.

``q = W_q h (+ b_q)`` in ``heads`` of ``dim``, ``k = W_k h (+ b_k)`` in ``kv_heads`` of ``dim``,
``v = W_v h (+ b_v)`` in ``kv_heads`` of ``vdim``; query head ``a`` reads KV head
``a // (heads / kv_heads)``.  With ``values = "keys"`` there is no ``W_v``: the values are the keys as
projected (bias included), before any norm, so ``vdim = dim``.  Then, per query and key head:

  * ``head_norm``: none, or an RMS norm over ``dim`` taken ``"before"`` or ``"after"`` the
    rotation, with one ``[dim]`` weight for the queries and one for the keys (shared by the
    heads) or, without names for them, no weight at all (a unit norm); or ``"joined"``: ONE RMS
    norm over all query heads' entries together and one over all key heads', with weights of
    ``[heads * dim]`` and ``[kv_heads * dim]`` (no rotation goes with it);
  * the position encoding on the first ``rotary_dim`` entries (half-split pairs; cosine and sine
    times the encoding's ``magnitude``).

``q_temperature = {"coef": c, "every": n}`` multiplies the query at position ``p`` by
``1 + c * ln(floor((p + 1) / n) + 1)`` (with the joined norm).  ``score = (q . k) * scale``, then ``softcap * tanh(score / softcap)`` if a cap is given.  What
position ``i`` sees (``mask``):

  * ``{"kind": "window", "size": w, "keep_first": f}``: ``j <= i`` with ``i - j < w`` or ``j < f``
    (the kept first tokens stay at their true positions);
  * ``{"kind": "chunk", "size": c}``: ``j <= i`` with ``j // c == i // c``, chunks counted from
    position 0 of the sequence wherever a prompt was cut;
  * ``{"kind": "causal"}``: every ``j <= i`` (a window that never ends; the cache keeps everything).

``weights``: ``"softmax"`` over the visible keys, or ``"sigmoid"``: every visible key weighs
``sigmoid(score + key_bias[head])`` and nothing is normalised.  ``gate`` names a ``[heads,
hidden]`` matrix: head ``a``'s output is multiplied by ``sigmoid((W_g h)_a)``; with ``gate_per =
"element"`` the matrix is ``[heads * vdim, hidden]`` and every entry of the concatenated heads has
a gate of its own.  Output: ``W_o`` on the concatenated heads.

The projections are joined into one matrix ``[q | k | v | gate]`` when bound, so one product
feeds the kernel that prepares the heads in place and stores keys and values.  The cache keeps
the last ``size`` positions (a chunk never reaches further back than that) and, for a window
that keeps first tokens, the pages that hold those.
"""

from __future__ import annotations

import torch

from ..config.errors import UnsupportedShape
from ..weights.spec import NORMAL, ONES, VECTOR, ZEROS, TensorSpec
from .base import MIXERS, POSITION_ENCODINGS, DeferredLinear, Mixer, PagedKV
from .plan import PartSpec

MAX_HEAD_DIM = 256  # what the kernels keep of a head in a warp's registers
EVERYTHING = 1 << 30  # the size of a window that never ends


@MIXERS.register("masked_attention")
class MaskedAttention(Mixer):
    """``params``: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``v_head_dim``,
    ``scale``, ``mask``, ``weights``, optionally ``softcap``, ``head_norm`` (+ ``eps``, ``q_norm``,
    ``k_norm``), ``position``, ``key_bias``, ``gate`` (+ ``gate_per``), ``values``, ``q_temperature``,
    ``q_bias`` / ``k_bias`` / ``v_bias``, and the names ``q_proj``, ``k_proj``, ``v_proj``, ``out_proj``."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.kv_heads = int(p["num_kv_heads"])
        self.dim = int(p["head_dim"])
        self.vdim = int(p.get("v_head_dim") or self.dim)
        self.scale = float(p["scale"])
        self.softcap = float(p["softcap"]) if p.get("softcap") is not None else None
        if self.heads % self.kv_heads:
            raise UnsupportedShape("num_kv_heads", self.kv_heads, f"does not divide {self.heads} query heads")
        if not 0 < self.dim <= MAX_HEAD_DIM or not 0 < self.vdim <= MAX_HEAD_DIM:
            raise UnsupportedShape("head sizes", (self.dim, self.vdim), f"the attention kernels take head sizes up to {MAX_HEAD_DIM}")
        if self.softcap is not None and self.softcap <= 0.0:
            raise UnsupportedShape("softcap", self.softcap, "a cap on the scores is positive")
        mask = p["mask"]
        self.mask = mask["kind"]
        self.causal = self.mask == "causal"
        if self.causal:  # a window that reaches back to the start, whatever the length
            self.mask, self.size, self.keep_first = "window", EVERYTHING, 0
        else:
            self.size = int(mask["size"])
            self.keep_first = int(mask.get("keep_first") or 0)
        if self.mask not in ("window", "chunk") or self.size < 1 or self.keep_first < 0:
            raise UnsupportedShape("mask", dict(mask), "kind 'window', 'chunk' or 'causal', size at least 1, keep_first not negative")
        if self.mask == "chunk" and self.keep_first:
            raise UnsupportedShape("mask", dict(mask), "a chunk keeps no first tokens")
        self.weights = p.get("weights", "softmax")
        if self.weights not in ("softmax", "sigmoid"):
            raise UnsupportedShape("weights", self.weights, "expected 'softmax' or 'sigmoid'")
        self.head_norm = p.get("head_norm")
        if self.head_norm not in (None, "before", "after", "joined"):
            raise UnsupportedShape("head_norm", self.head_norm, "expected None, 'before', 'after' or 'joined'")
        self.eps = float(p.get("eps", 0.0))
        self.values = p.get("values", "projected")
        if self.values not in ("projected", "keys"):
            raise UnsupportedShape("values", self.values, "expected 'projected' or 'keys'")
        if self.values == "keys" and self.vdim != self.dim:
            raise UnsupportedShape("v_head_dim", self.vdim, f"values that are the keys have the keys' size {self.dim}")
        self.gate_per = p.get("gate_per", "head")
        if self.gate_per not in ("head", "element"):
            raise UnsupportedShape("gate_per", self.gate_per, "expected 'head' or 'element'")
        temperature = p.get("q_temperature")
        self.q_temperature = (float(temperature["coef"]), int(temperature["every"])) if temperature is not None else None
        if self.q_temperature is not None and self.q_temperature[1] < 1:
            raise UnsupportedShape("q_temperature", dict(temperature), "the positions are counted in runs of at least 1")
        self.position = POSITION_ENCODINGS.build(p.get("position") or PartSpec("none"), env, self.dim)
        joined = self.head_norm == "joined"
        if joined and self.position.rotary()[1]:
            raise UnsupportedShape("position", p["position"].kind, "the kernel of the joined norm does not rotate")
        if (self.values == "keys" or self.q_temperature is not None) and not joined:
            raise UnsupportedShape("head_norm", self.head_norm, "values that are the keys and a query temperature come with the joined norm's kernel")
        if joined and (p.get("q_norm") is None or p.get("k_norm") is None):
            raise UnsupportedShape("head_norm", self.head_norm, "the joined norm has a weight for the queries and one for the keys")
        if getattr(self.position, "interleaved", False):
            raise UnsupportedShape("position", p["position"].kind, "the kernel that prepares the heads rotates half-split pairs")
        self.names = {k: p.get(k) for k in ("q_proj", "k_proj", "v_proj", "out_proj", "q_bias", "k_bias", "v_bias", "q_norm", "k_norm",
                                             "key_bias", "gate")}
        if self.names["key_bias"] is not None and self.weights != "sigmoid":
            raise UnsupportedShape("key_bias", self.names["key_bias"], "a bias per head on the scores changes nothing under a softmax")
        self.in_matrix = self.in_bias = self.out_matrix = None
        self.q_weight = self.k_weight = self.key_bias = None

    @property
    def q_cols(self):
        return self.heads * self.dim

    @property
    def kv_cols(self):
        return self.kv_heads * (self.dim + (self.vdim if self.values == "projected" else 0))

    @property
    def gate_cols(self):
        return self.heads * (self.vdim if self.gate_per == "element" else 1)

    def sub_parts(self):
        return [self.position]

    def tensor_specs(self):
        n = self.names
        specs = [
            TensorSpec(n["q_proj"], (self.heads * self.dim, self.hidden)),
            TensorSpec(n["k_proj"], (self.kv_heads * self.dim, self.hidden)),
            TensorSpec(n["out_proj"], (self.hidden, self.heads * self.vdim)),
        ]
        if self.values == "projected":
            specs.append(TensorSpec(n["v_proj"], (self.kv_heads * self.vdim, self.hidden)))
        for key, rows in (("q_bias", self.heads * self.dim), ("k_bias", self.kv_heads * self.dim), ("v_bias", self.kv_heads * self.vdim)):
            if n[key] is not None and not (key == "v_bias" and self.values == "keys"):
                specs.append(TensorSpec(n[key], (rows,), VECTOR, NORMAL))
        joined = self.head_norm == "joined"
        for key, heads in (("q_norm", self.heads), ("k_norm", self.kv_heads)):
            if n[key] is not None:
                specs.append(TensorSpec(n[key], (heads * self.dim if joined else self.dim,), VECTOR, ONES))
        if n["key_bias"] is not None:
            specs.append(TensorSpec(n["key_bias"], (self.heads,), VECTOR, ZEROS))
        if n["gate"] is not None:
            specs.append(TensorSpec(n["gate"], (self.gate_cols, self.hidden)))
        return specs

    def bind(self, tensors):
        n = self.names
        projected = ("q_proj", "k_proj", "v_proj") if self.values == "projected" else ("q_proj", "k_proj")
        mats = [tensors[n[k]] for k in projected]
        if n["gate"] is not None:
            mats.append(tensors[n["gate"]])
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.in_matrix = torch.cat(mats, dim=0).contiguous()
        if any(n[k] is not None for k in ("q_bias", "k_bias", "v_bias")):
            rows = (self.heads * self.dim, self.kv_heads * self.dim, self.kv_heads * self.vdim)
            parts = [tensors[n[k]].to(torch.float32) if n[k] is not None else torch.zeros(r, dtype=torch.float32, device=self.in_matrix.device)
                     for k, r in zip(("q_bias", "k_bias", "v_bias")[: len(projected)], rows)]
            if n["gate"] is not None:
                parts.append(torch.zeros(self.gate_cols, dtype=torch.float32, device=self.in_matrix.device))
            self.in_bias = torch.cat(parts).contiguous()
        self.out_matrix = tensors[n["out_proj"]]
        self.q_weight = tensors[n["q_norm"]] if n["q_norm"] is not None else None
        self.k_weight = tensors[n["k_norm"]] if n["k_norm"] is not None else None
        self.key_bias = tensors[n["key_bias"]] if n["key_bias"] is not None else None

    def cache_spec(self):
        return PagedKV(self.kv_heads, self.dim, None if self.causal else self.size, self.vdim, keep_first=self.keep_first)

    def forward(self, x, step, cache):
        ops = self.env.ops
        proj = ops.linear(x, self.in_matrix, self.env.dtype, self.in_bias)
        inv_freq, rotary_dim = self.position.rotary()
        table = step.block_tables[cache.group]
        from_qkv = getattr(ops, "decode_attention_from_qkv", None)
        gate = proj[:, self.q_cols + self.kv_cols :] if self.names["gate"] is not None else None
        more = {"gate_per_element": True} if gate is not None and self.gate_per == "element" else {}
        if self.head_norm == "joined":
            q = ops.joined_norm_store(
                proj, self.heads, self.kv_heads, self.dim, self.vdim, self.q_weight, self.k_weight, self.eps, self.q_temperature,
                self.values == "keys", step, cache.k, cache.v, table, cache.page_size,
            )
            out = ops.masked_attention(
                q, self.heads, cache.k, cache.v, table, cache.page_size, self.scale, self.mask, self.size, self.keep_first, step,
                sigmoid=self.weights == "sigmoid", key_bias=self.key_bias, softcap=self.softcap, gate=gate, **more,
            )
            return DeferredLinear(ops, out, self.out_matrix, self.env.dtype)
        if (
            from_qkv is not None and self.mask == "window" and self.weights == "softmax" and self.softcap is None
            and self.names["gate"] is None and self.head_norm == "before" and self.q_weight is not None and self.k_weight is not None
            and self.dim == self.vdim and float(getattr(self.position, "magnitude", 1.0)) == 1.0
        ):
            # steps of single tokens, heads of 64 rotated whole: norm, rotation, cache store and
            # attention in the one launch the framework's other attention layers take (None otherwise)
            attn = from_qkv(
                proj, self.heads, self.kv_heads, self.dim, self.q_weight, self.k_weight, self.eps, inv_freq, rotary_dim, step,
                cache.k, cache.v, table, cache.page_size, True, self.scale, self.size, keep_first=self.keep_first,
            )
            if attn is not None:
                return DeferredLinear(ops, attn, self.out_matrix, self.env.dtype)
        q = ops.head_prepare_store(
            proj, self.heads, self.kv_heads, self.dim, self.vdim, self.q_weight, self.k_weight, self.eps, self.head_norm,
            inv_freq, rotary_dim, float(getattr(self.position, "magnitude", 1.0)), step, cache.k, cache.v, table, cache.page_size,
        )
        out = ops.masked_attention(
            q, self.heads, cache.k, cache.v, table, cache.page_size, self.scale, self.mask, self.size, self.keep_first, step,
            sigmoid=self.weights == "sigmoid", key_bias=self.key_bias, softcap=self.softcap, gate=gate, **more,
        )
        return DeferredLinear(ops, out, self.out_matrix, self.env.dtype)
