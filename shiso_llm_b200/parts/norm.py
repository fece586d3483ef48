"""RMS normalisation: ``y = x * rsqrt(mean(x^2) + eps) * w`` with the statistics in float32.

The weight multiplies directly, not as ``1 + w`` (kernels/cuda/generic/norm.cuh:86-93).
``add_apply`` is the fused residual-add + norm that closes every block
(norm.cuh:105-165; crates/shiso-engine/src/layers.rs:2476-2498): the stored sum is
what is normalised.

``offset`` (default 0) is added to the stored weight once, when it is bound: a checkpoint
that keeps its norm weights around zero and applies ``1 + w`` asks for ``offset = 1`` and
every kernel runs unchanged.  ``scalar`` says that the checkpoint holds ONE number for all
coordinates (a tensor without dimensions): it is spread over the row when bound.  ``gain``
(default 1) is a constant multiplied into the weight when bound - a scale on the logits
rides on the final norm this way.

``add_normed`` is the other way round from ``add_apply``: the norm is taken of a sublayer's
OUTPUT, and that is added to the residual, ``x <- x + norm(y)``; the sublayers of such a layer
read the residual itself, so the kernel also hands back the new residual in the compute type.
"""

from __future__ import annotations

import torch

from ..weights.spec import NORMAL, ONES, VECTOR, TensorSpec
from .base import NORMS, Norm


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.tensor_name = spec.params["tensor"]
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.offset = float(spec.params.get("offset", 0.0))
        self.scalar = bool(spec.params.get("scalar", False))
        self.gain = float(spec.params.get("gain", 1.0))
        self.weight = None

    def tensor_specs(self):
        if self.scalar:
            return [TensorSpec(self.tensor_name, (), VECTOR, NORMAL if self.offset != 0.0 else ONES, init_std=0.1)]
        if self.offset != 0.0:  # stored around zero
            return [TensorSpec(self.tensor_name, (self.size,), VECTOR, NORMAL, init_std=0.1)]
        return [TensorSpec(self.tensor_name, (self.size,), VECTOR, ONES)]

    def bind(self, tensors):
        self.weight = tensors[self.tensor_name]
        if self.scalar:
            self.weight = self.weight.to(torch.float32).reshape(1).expand(self.size).contiguous()
        if self.offset != 0.0:
            self.weight = (self.weight.to(torch.float32) + self.offset).contiguous()
        if self.gain != 1.0:
            self.weight = (self.weight.to(torch.float32) * self.gain).contiguous()

    def rms_params(self):
        """``(weight, eps)``: what a kernel that normalises inside a product needs."""
        return self.weight, self.eps

    def apply(self, x):
        return self.env.ops.rmsnorm(x, self.weight, self.eps, self.env.dtype)

    def add_apply(self, residual, delta, rows=None):
        return self.env.ops.add_rmsnorm(residual, delta, self.weight, self.eps, self.env.dtype, rows)

    def add_normed(self, residual, y, want_rows=True):
        """``residual += norm(y)`` in float32, in place; returns the new residual rows in the
        compute type (what the next sublayer reads), or None when they are not wanted."""
        return self.env.ops.norm_into(residual, y, self.weight, self.eps, want_rows)

    def add_apply_linear(self, residual, deferred):
        """``residual += deferred.x @ deferred.w^T`` and the norm of the sum, fused where the
        kernel table can (decode-sized bfloat16 steps)."""
        return self.env.ops.linear_add_rmsnorm(deferred.x, deferred.w, residual, self.weight, self.eps, self.env.dtype)


@NORMS.register("layernorm")
class LayerNorm(Norm):
    """``y = (x - mean) / sqrt(var + eps) * w`` with a weight and no bias; the variance is the
    mean of the squared deviations; statistics in float32.  ``add_apply`` takes one block
    output or a tuple of them (a layer whose mixer and feed-forward read the same rows leaves
    two): they are added to the residual in float32 by the kernel that normalises."""

    takes_several = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.tensor_name = spec.params["tensor"]
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.tensor_name, (self.size,), VECTOR, ONES)]

    def bind(self, tensors):
        self.weight = tensors[self.tensor_name]

    def apply(self, x):
        return self.env.ops.add_layernorm(x, (), self.weight, self.eps, self.env.dtype, None)

    def add_apply(self, residual, delta, rows=None):
        deltas = tuple(delta) if isinstance(delta, (tuple, list)) else (delta,)
        return self.env.ops.add_layernorm(residual, deltas, self.weight, self.eps, self.env.dtype, rows)


@NORMS.register("dyt")
class DynamicTanh(Norm):
    """``y = tanh(alpha x) * w + b``: a squashing element by element, with no mean, no variance and
    no epsilon.  ``alpha`` is one number in the checkpoint (a tensor without dimensions), ``w`` and
    ``b`` are vectors; names ``tensor`` (the weight), ``alpha`` and ``bias`` (absent: the weight's
    name with ``.alpha`` / ``.b`` added).  Evaluated in float32; ``add_apply`` adds one block output
    or a tuple of them to the float32 residual in the kernel that squashes."""

    takes_several = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.tensor_name = spec.params["tensor"]
        self.alpha_name = spec.params.get("alpha") or self.tensor_name + ".alpha"
        self.bias_name = spec.params.get("bias") or self.tensor_name + ".b"
        self.size = int(spec.params["size"])
        self.weight = self.bias = None
        self.alpha = 1.0

    def tensor_specs(self):
        return [
            TensorSpec(self.tensor_name, (self.size,), VECTOR, ONES),
            TensorSpec(self.bias_name, (self.size,), VECTOR, NORMAL, init_std=0.02),
            TensorSpec(self.alpha_name, (), VECTOR, NORMAL, init_mean=0.5, init_std=0.05),
        ]

    def bind(self, tensors):
        self.weight, self.bias = tensors[self.tensor_name], tensors[self.bias_name]
        self.alpha = float(tensors[self.alpha_name].to(torch.float32))  # a launch parameter

    def apply(self, x):
        return self.env.ops.add_dyt(x, (), self.alpha, self.weight, self.bias, self.env.dtype, None)

    def add_apply(self, residual, delta, rows=None):
        deltas = tuple(delta) if isinstance(delta, (tuple, list)) else (delta,)
        return self.env.ops.add_dyt(residual, deltas, self.alpha, self.weight, self.bias, self.env.dtype, rows)
