"""Latent attention: softmax attention whose keys and values are expanded from a small cached
latent, with one rotated key part shared by all heads.

Queries go through a latent of their own: ``c_q = rmsnorm(W_dq h) * w_q``, ``q = W_uq c_q``, laid
out head by head as ``[dim plain | rot_dim rotated]`` - or, without ``q_rank``, straight from the
input: ``q = W_q h`` (name ``q_proj``).  ``W_dkv h`` has ``kv_rank + rot_dim``
rows: the first ``kv_rank``, RMS-normed with a weight, are the latent ``c``; the last ``rot_dim``
(not normed) are rotated by the position and shared by all heads.  Head ``h`` has the plain
key ``W_uk[h] c`` and the value ``W_uv[h] c``; its score against position ``j`` is

    (q_plain . W_uk[h] c_j + q_rot . k_rot_j) * scale,

causal, with an ordinary softmax.  The head's output is multiplied by ``sigmoid(W_g h)_h`` where
a ``gate`` is named, and the joined heads are projected.  The rotation may pair neighbours or
halves and carry a magnitude on cosine and sine (the position encoding says which).

Only ``c`` and the rotated key part are cached: one row of ``kv_rank + rot_dim`` per position,
for all heads.  The expansion never happens: the plain query is carried into the latent space
(``q_lat[h] = W_uk[h]^T q_plain``, a product per head), scores are taken against the cached row
``[c | k_rot]`` directly, the softmax weights sum the latents, and ``W_uv[h]`` is applied once
to that sum (a product per head, with the gate in its epilogue).  The three projections that
read ``h`` (query latent, key/value latent, gate) are one product.
"""

from __future__ import annotations

import torch

from ..config.errors import UnsupportedShape
from ..weights.spec import ONES, VECTOR, TensorSpec
from .base import MIXERS, POSITION_ENCODINGS, DeferredLinear, Mixer, PagedKV, project

MAX_LATENT_ROW = 1024  # kv_rank + rot_dim a CTA of the attention kernel keeps of a query in shared memory
MAX_LATENT_RANK = 512  # kv_rank: a lane of the attention kernel sums up to 16 latent entries per head


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """``params``: ``hidden_size``, ``num_heads``, ``head_dim`` (plain), ``rot_dim``, ``v_head_dim``,
    ``q_rank`` (None: no query latent), ``kv_rank``, ``scale``, ``eps``, ``position`` (a PartSpec, over
    ``rot_dim``) and names ``q_down``, ``q_norm``, ``q_up`` (or ``q_proj``), ``kv_down``, ``kv_norm``,
    ``k_up``, ``v_up``, ``gate`` (optional), ``out_proj``."""

    takes_deferred_norm = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.dim = int(p["head_dim"])
        self.rot = int(p["rot_dim"])
        self.vdim = int(p["v_head_dim"])
        self.q_rank = int(p["q_rank"]) if p.get("q_rank") is not None else None
        self.kv_rank = int(p["kv_rank"])
        self.scale = float(p["scale"])
        self.eps = float(p["eps"])
        if self.kv_rank + self.rot > MAX_LATENT_ROW:
            raise UnsupportedShape("kv_rank + rot_dim", self.kv_rank + self.rot, f"the attention kernel takes cached rows of up to {MAX_LATENT_ROW}")
        if self.kv_rank > MAX_LATENT_RANK:
            raise UnsupportedShape("kv_rank", self.kv_rank, f"the attention kernel takes latents of up to {MAX_LATENT_RANK}")
        self.position = POSITION_ENCODINGS.build(p["position"], env, self.rot)
        self.magnitude = float(getattr(self.position, "magnitude", 1.0))
        self.interleaved = bool(getattr(self.position, "interleaved", False))
        # what the rotation kernels are told beyond the usual (half-split pairs, no magnitude)
        self.rotation = {}
        if self.magnitude != 1.0:
            self.rotation["magnitude"] = self.magnitude
        if self.interleaved:
            self.rotation["interleaved"] = True
        wanted = ("q_down", "q_norm", "q_up") if self.q_rank is not None else ("q_proj",)
        self.names = {k: p[k] for k in wanted + ("kv_down", "kv_norm", "k_up", "v_up", "out_proj")}
        self.names["gate"] = p.get("gate")
        self.in_matrix = self.w = None

    def sub_parts(self):
        return [self.position]

    def tensor_specs(self):
        n, H = self.names, self.heads
        if self.q_rank is not None:
            specs = [TensorSpec(n["q_down"], (self.q_rank, self.hidden)), TensorSpec(n["q_norm"], (self.q_rank,), VECTOR, ONES),
                     TensorSpec(n["q_up"], (H * (self.dim + self.rot), self.q_rank))]
        else:
            specs = [TensorSpec(n["q_proj"], (H * (self.dim + self.rot), self.hidden))]
        specs += [
            TensorSpec(n["kv_down"], (self.kv_rank + self.rot, self.hidden)), TensorSpec(n["kv_norm"], (self.kv_rank,), VECTOR, ONES),
            TensorSpec(n["k_up"], (H * self.dim, self.kv_rank)), TensorSpec(n["v_up"], (H * self.vdim, self.kv_rank)),
            TensorSpec(n["out_proj"], (self.hidden, H * self.vdim)),
        ]
        if n["gate"] is not None:
            specs.append(TensorSpec(n["gate"], (H, self.hidden)))
        return specs

    def bind(self, tensors):
        n, H = self.names, self.heads
        mats = [tensors[n["q_down" if self.q_rank is not None else "q_proj"]], tensors[n["kv_down"]]]
        if n["gate"] is not None:
            mats.append(tensors[n["gate"]])
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.in_matrix = torch.cat(mats, dim=0).contiguous()
        self.w = {k: tensors[n[k]] for k in (("q_norm", "q_up") if self.q_rank is not None else ()) + ("kv_norm", "out_proj")}
        # per head: the key expansion transposed, [kv_rank, dim] (it carries queries into the latent
        # space), and the value expansion as stored, [vdim, kv_rank]
        self.w["k_up_t"] = tensors[n["k_up"]].reshape(H, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w["v_up"] = tensors[n["v_up"]].reshape(H, self.vdim, self.kv_rank).contiguous()

    def cache_spec(self):
        # one row [latent | rotated key part] per position for all heads, and no value rows: values are the latent
        return PagedKV(1, self.kv_rank + self.rot, None, 0)

    def forward(self, x, step, cache):
        ops, w, dtype = self.env.ops, self.w, self.env.dtype
        H, R, P = self.heads, self.kv_rank, self.rot
        proj = project(ops, x, self.in_matrix, dtype)
        T = proj.shape[0]
        a = self.q_rank if self.q_rank is not None else H * (self.dim + P)  # the query's columns (its latent's)
        b = a + R + P
        inv_freq, rotary_dim = self.position.rotary()
        table = step.block_tables[cache.group]
        if cache.owner:
            ops.latent_store(proj[:, a:b], R, w["kv_norm"], self.eps, inv_freq, rotary_dim, step, cache.k, table, cache.page_size,
                             **self.rotation)
        if self.q_rank is not None:
            cq = ops.group_rmsnorm(proj[:, :a], w["q_norm"], self.eps, 1, dtype)
            q = ops.linear(cq, w["q_up"], dtype).view(T, H, self.dim + P)
        else:
            q = proj[:, :a].unflatten(1, (H, self.dim + P))  # a column range of the projection's rows
        q_lat = torch.empty((T, H, R + P), dtype=dtype, device=q.device)
        ops.head_linear(q[:, :, : self.dim], w["k_up_t"], q_lat[:, :, :R])
        ops.rotate_heads(q[:, :, self.dim :], q_lat[:, :, R:], inv_freq, rotary_dim, step, **self.rotation)
        mixed = ops.latent_attention(q_lat, R, cache.k, table, cache.page_size, self.scale, step)  # [T, H, R]
        out = torch.empty((T, H, self.vdim), dtype=dtype, device=q.device)
        ops.head_linear(mixed, w["v_up"], out, gate=proj[:, b:] if self.names["gate"] is not None else None)
        return DeferredLinear(ops, out.view(T, H * self.vdim), w["out_proj"], dtype)

