"""Retention: linear attention with one fixed decay per head, no softmax and no denominator.

``q = W_q h`` and ``k = W_k h`` in heads of ``dim``, ``v = W_v h`` in heads of ``vdim``.  A
position encoding rotates ``q`` and ``k`` (not ``v``); ``k`` is then multiplied by
``dim^(-1/2)``.  Per head, with a state ``S[key, value]`` that starts at zero,

    S_t = decay_h * S_{t-1} + k_t v_t^T,        o_t = S_t^T q_t.

Each head's ``o_t`` is brought to unit RMS (no weight), the joined heads are multiplied by
``silu(W_g h)`` and projected.  The state is float32 and carried per request.

The four input projections are one product.  One launch walks each sequence's tokens in
order with a head's state in registers; it rotates and scales on load and applies unit RMS
and the gate on store.  The mixer also serves as a branch of ``parallel_mixer``: it then
reads its columns of the joint product and writes its columns of the joint output.
"""

from __future__ import annotations

import torch

from ..config.errors import UnsupportedShape
from ..weights.spec import TensorSpec
from .base import MIXERS, POSITION_ENCODINGS, DeferredLinear, FixedState, Mixer, project
from .wkv import MAX_STATE_DIM, MAX_STATE_SIZE


@MIXERS.register("retention")
class Retention(Mixer):
    """``params``: ``hidden_size``, ``num_heads``, ``head_dim``, ``v_head_dim``, ``decay`` (one
    per head), ``eps``, ``position`` (a PartSpec), and names ``q_proj``, ``k_proj``, ``v_proj``,
    ``g_proj``, ``out_proj``."""

    takes_deferred_norm = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.dim = int(p["head_dim"])
        self.vdim = int(p["v_head_dim"])
        self.eps = float(p["eps"])
        decays = [float(d) for d in p["decay"]]
        if len(decays) != self.heads:
            raise UnsupportedShape("decay", decays, f"one decay per head is needed, {self.heads} heads")
        if not 0 < self.dim <= MAX_STATE_DIM or not 0 < self.vdim <= MAX_STATE_DIM or self.dim * self.vdim > MAX_STATE_SIZE:
            raise UnsupportedShape("head sizes", (self.dim, self.vdim), f"the recurrence kernel takes states up to {MAX_STATE_DIM} rows or columns and {MAX_STATE_SIZE} values")
        fits = getattr(env.ops, "recurrence_supported", None)
        if fits is not None and not fits(self.dim, self.vdim):
            raise UnsupportedShape("head sizes", (self.dim, self.vdim), "the recurrence kernel has no layout for a state of this shape")
        self.decays = torch.tensor(decays, dtype=torch.float64).to(torch.float32).to(env.device)
        # what the kernel multiplies by: S - (1 - decay) S, with 1 - decay formed in float64
        self.losses = (1.0 - torch.tensor(decays, dtype=torch.float64)).to(torch.float32).to(env.device)
        self.position = POSITION_ENCODINGS.build(p["position"], env, self.dim)
        if float(getattr(self.position, "magnitude", 1.0)) != 1.0:
            raise UnsupportedShape("position", type(self.position).__name__, "this mixer's kernels rotate without a magnitude on cosine and sine")
        if getattr(self.position, "interleaved", False):
            raise UnsupportedShape("position", p["position"].kind, "the recurrence kernel rotates half-split pairs")
        self.names = {k: p[k] for k in ("q_proj", "k_proj", "v_proj", "g_proj", "out_proj")}
        self.in_matrix = self.out_matrix = None

    # sizes of the columns this mixer reads (q, k, v, gate) and writes
    @property
    def in_width(self):
        return 2 * self.heads * self.dim + 2 * self.heads * self.vdim

    @property
    def out_width(self):
        return self.heads * self.vdim

    def sub_parts(self):
        return [self.position]

    def tensor_specs(self):
        qk, vg, n = self.heads * self.dim, self.heads * self.vdim, self.names
        return [
            TensorSpec(n["q_proj"], (qk, self.hidden)), TensorSpec(n["k_proj"], (qk, self.hidden)),
            TensorSpec(n["v_proj"], (vg, self.hidden)), TensorSpec(n["g_proj"], (vg, self.hidden)),
            TensorSpec(n["out_proj"], (self.hidden, vg)),
        ]

    def bind(self, tensors):
        n = self.names
        mats = [tensors[n[k]] for k in ("q_proj", "k_proj", "v_proj", "g_proj")]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.in_matrix = torch.cat(mats, dim=0).contiguous()
        self.out_matrix = tensors[n["out_proj"]]

    def cache_spec(self):
        return FixedState((self.heads, self.dim, self.vdim))

    def mix(self, proj, step, cache, out, out_scale=1.0):
        """``proj[T, in_width]`` (rows may be strided) -> ``out[T, out_width]``, times ``out_scale``."""
        qk, vg = self.heads * self.dim, self.heads * self.vdim
        inv_freq, rotary_dim = self.position.rotary()
        self.env.ops.decay_recurrence(
            proj[:, :qk], proj[:, qk : 2 * qk], proj[:, 2 * qk : 2 * qk + vg], out, cache.state, step,
            self.heads, self.dim, self.vdim, self.eps,
            head_decay=self.decays, head_loss=self.losses, inv_freq=inv_freq, rotary_dim=rotary_dim, key_scale=self.dim ** -0.5,
            gate=proj[:, 2 * qk + vg :], out_scale=out_scale,
        )

    def forward(self, x, step, cache):
        ops = self.env.ops
        proj = project(ops, x, self.in_matrix, self.env.dtype)
        out = torch.empty((proj.shape[0], self.out_width), dtype=self.env.dtype, device=proj.device)
        self.mix(proj, step, cache, out)
        return DeferredLinear(ops, out, self.out_matrix, self.env.dtype)
