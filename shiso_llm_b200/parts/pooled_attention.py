"""Sliding-window attention that also sees one pooled key and value per block of old tokens.

Grouped-query softmax attention without biases: ``q = W_q h`` in ``heads`` of ``dim``,
``k = W_k h`` in ``kv_heads`` of ``dim``, ``v = W_v h`` in ``kv_heads`` of ``vdim``; query
head ``h`` reads KV head ``h // (heads / kv_heads)``; ``score = (q . k) * scale``.  A position
encoding may rotate ``q`` and ``k`` (none by default).  Position ``i`` sees

  * the tokens ``j`` with ``0 <= i - j < window``, and
  * for every block ``b`` of ``pool`` consecutive positions that lies wholly behind the window,
    ``b * pool + pool - 1 <= i - window``, ONE key and ONE value: the means of the block's
    keys and values as the cache holds them,

all in one softmax.  A token that has left the window while its block is not yet behind it
is not seen at all.

Two caches per run entry: keys and values per position in pages of the compute type, of
which only the last ``max(window, pool)`` positions are ever read again (older pages go
back to the pool), and the blocks' means in float32, one row per ``pool`` positions, kept
for the request's life.  A step stores its keys and values, then forms the mean of every
block whose last position it brought (from the cache, so a block may have begun in an
earlier step), then attends.  The mixer also serves as a branch of ``parallel_mixer``.
"""

from __future__ import annotations

import torch

from ..config.errors import UnsupportedShape
from ..weights.spec import TensorSpec
from .attention import MAX_HEAD_DIM
from .base import MIXERS, POSITION_ENCODINGS, DeferredLinear, Mixer, PagedKV, project
from .plan import PartSpec


@MIXERS.register("pooled_window_attention")
class PooledWindowAttention(Mixer):
    """``params``: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``,
    ``v_head_dim``, ``scale``, ``window``, ``pool``, optionally ``position``, and names
    ``q_proj``, ``k_proj``, ``v_proj``, ``out_proj``."""

    takes_deferred_norm = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.kv_heads = int(p["num_kv_heads"])
        self.dim = int(p["head_dim"])
        self.vdim = int(p.get("v_head_dim") or self.dim)
        self.scale = float(p["scale"])
        self.window = int(p["window"])
        self.pool = int(p["pool"])
        if self.heads % self.kv_heads:
            raise UnsupportedShape("num_kv_heads", self.kv_heads, f"does not divide {self.heads} query heads")
        if not 0 < self.dim <= MAX_HEAD_DIM or not 0 < self.vdim <= MAX_HEAD_DIM:
            raise UnsupportedShape("head sizes", (self.dim, self.vdim), f"the attention kernels take head sizes up to {MAX_HEAD_DIM}")
        if self.window < 1 or self.pool < 1:
            raise UnsupportedShape("window / pool", (self.window, self.pool), "both are at least 1")
        self.position = POSITION_ENCODINGS.build(p.get("position") or PartSpec("none"), env, self.dim)
        if float(getattr(self.position, "magnitude", 1.0)) != 1.0:
            raise UnsupportedShape("position", type(self.position).__name__, "this mixer's kernels rotate without a magnitude on cosine and sine")
        if self.position.rotary()[1]:
            raise UnsupportedShape("position", p["position"].kind, "the store kernel of this mixer keeps keys as they are projected")
        self.names = {k: p[k] for k in ("q_proj", "k_proj", "v_proj", "out_proj")}
        self.in_matrix = self.out_matrix = None

    @property
    def in_width(self):
        return self.heads * self.dim + self.kv_heads * (self.dim + self.vdim)

    @property
    def out_width(self):
        return self.heads * self.vdim

    def sub_parts(self):
        return [self.position]

    def tensor_specs(self):
        n = self.names
        return [
            TensorSpec(n["q_proj"], (self.heads * self.dim, self.hidden)),
            TensorSpec(n["k_proj"], (self.kv_heads * self.dim, self.hidden)),
            TensorSpec(n["v_proj"], (self.kv_heads * self.vdim, self.hidden)),
            TensorSpec(n["out_proj"], (self.hidden, self.heads * self.vdim)),
        ]

    def bind(self, tensors):
        n = self.names
        mats = [tensors[n[k]] for k in ("q_proj", "k_proj", "v_proj")]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.in_matrix = torch.cat(mats, dim=0).contiguous()
        self.out_matrix = tensors[n["out_proj"]]

    def cache_spec(self):
        return (
            PagedKV(self.kv_heads, self.dim, max(self.window, self.pool), self.vdim),
            PagedKV(self.kv_heads, self.dim, None, self.vdim, torch.float32, every=self.pool),
        )

    def mix(self, proj, step, cache, out, out_scale=1.0):
        """``proj[T, in_width]`` (rows may be strided) -> ``out[T, out_width]``, times ``out_scale``."""
        ops = self.env.ops
        tokens, blocks = cache
        q_cols, k_cols = self.heads * self.dim, self.kv_heads * self.dim
        ops.store_kv(proj[:, q_cols : q_cols + k_cols], proj[:, q_cols + k_cols :], self.kv_heads, self.dim, self.vdim, step,
                     tokens.k, tokens.v, step.block_tables[tokens.group], tokens.page_size)
        ops.pool_kv(tokens.k, tokens.v, step.block_tables[tokens.group], blocks.k, blocks.v, step.block_tables[blocks.group],
                    tokens.page_size, self.pool, step)
        ops.pooled_window_attention(
            proj[:, :q_cols], self.heads, tokens.k, tokens.v, step.block_tables[tokens.group],
            blocks.k, blocks.v, step.block_tables[blocks.group], tokens.page_size, self.scale, self.window, self.pool,
            step, out, out_scale,
        )

    def forward(self, x, step, cache):
        ops = self.env.ops
        proj = project(ops, x, self.in_matrix, self.env.dtype)
        out = torch.empty((proj.shape[0], self.out_width), dtype=self.env.dtype, device=proj.device)
        self.mix(proj, step, cache, out)
        return DeferredLinear(ops, out, self.out_matrix, self.env.dtype)
