"""SwiGLU feed-forward: ``W_down (silu(W_gate x) * (W_up x))``.

The gate and up matrices are stored apart in the checkpoint and run as one paired
projection (crates/shiso-engine/src/ffn.rs:234-239); here they are joined into one
``[2I, H]`` matrix when bound, so one product yields ``[gate | up]`` rows; the activation
(kernels/cuda/generic/glu.cuh:35-57: alpha 1, no clamp) is applied in the product's epilogue
for decode-sized batches and by a kernel of its own otherwise.  ``activation`` chooses another
gated pair than silu: ``"gelu_tanh"``, ``act(g) * u`` with the tanh form of gelu, or
``"swish_clamped"`` with a ``limit`` L: ``g' = min(g, L)``, ``u' = clamp(u, -L, L)``,
``g' sigmoid(1.702 g') (u' + 1)``.

``relu2_ff`` is ``W_down relu(W_up x)^2``; ``routed_experts`` a mixture of gated experts
behind a router with group-limited choice; ``polynorm_ff`` is ``W_down act(W_up x)`` with a
polynomial of unit-RMS powers as the activation (see the classes).
"""

from __future__ import annotations

import torch

from ..config.errors import UnsupportedShape
from ..weights.spec import NORMAL, VECTOR, TensorSpec
from .base import FEED_FORWARDS, DeferredLinear, FeedForward, project

MAX_EXPERTS = 256  # what the routing kernel keeps of a token's scores in a warp's registers ...
MAX_TOP = 16  # ... and how many choices it makes per token
GLU_ACTIVATIONS = ("silu", "gelu_tanh", "swish_clamped")


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    takes_deferred_norm = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        self.names = (p["gate"], p["up"], p["down"])
        self.activation = p.get("activation", "silu")
        if self.activation not in GLU_ACTIVATIONS:
            raise UnsupportedShape("activation", self.activation, f"expected one of {GLU_ACTIVATIONS}")
        self.limit = float(p.get("limit") or 0.0)
        if self.activation == "swish_clamped" and self.limit <= 0.0:
            raise UnsupportedShape("limit", p.get("limit"), "a clamped pair needs a positive limit")
        self.act = None if self.activation == "silu" else (self.activation, self.limit)
        self.gate_up = None
        self.down = None

    def tensor_specs(self):
        gate, up, down = self.names
        return [
            TensorSpec(gate, (self.inter, self.hidden)),
            TensorSpec(up, (self.inter, self.hidden)),
            TensorSpec(down, (self.hidden, self.inter)),
        ]

    def bind(self, tensors):
        gate, up, down = self.names
        g, u = tensors[gate], tensors[up]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.gate_up = torch.cat([g, u], dim=0).contiguous()
        self.down = tensors[down]

    def forward(self, x, step):
        ops = self.env.ops
        mid = project(ops, x, self.gate_up, self.env.dtype, glu=True, act=self.act)
        return DeferredLinear(ops, mid, self.down, self.env.dtype)


@FEED_FORWARDS.register("relu2_ff")
class Relu2FeedForward(FeedForward):
    """``W_down relu(W_up x)^2``; names ``up`` and ``down``."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        self.names = (p["up"], p["down"])
        self.up = self.down = None

    def tensor_specs(self):
        up, down = self.names
        return [TensorSpec(up, (self.inter, self.hidden)), TensorSpec(down, (self.hidden, self.inter))]

    def bind(self, tensors):
        self.up, self.down = tensors[self.names[0]], tensors[self.names[1]]

    def forward(self, x, step):
        ops = self.env.ops
        mid = ops.unary(project(ops, x, self.up, self.env.dtype), "relu2", self.env.dtype)
        return DeferredLinear(ops, mid, self.down, self.env.dtype)


@FEED_FORWARDS.register("polynorm_ff")
class PolyNormFeedForward(FeedForward):
    """``W_down act(W_up x)`` with ``act(z) = a N(z) + b N(z^2) + c N(z^3) + e``: powers element by
    element, ``N(u) = u / sqrt(mean(u^2) + eps)`` over a token's ``intermediate_size`` values,
    statistics in float32.  Names ``up``, ``down`` and ``act`` (the four numbers a, b, c, e)."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        self.eps = float(p["eps"])
        self.names = (p["up"], p["down"], p["act"])
        self.up = self.down = self.coefficients = None

    def tensor_specs(self):
        up, down, act = self.names
        return [TensorSpec(up, (self.inter, self.hidden)), TensorSpec(down, (self.hidden, self.inter)),
                TensorSpec(act, (4,), VECTOR, NORMAL, init_mean=0.4, init_std=0.3)]

    def bind(self, tensors):
        self.up, self.down, self.coefficients = (tensors[n] for n in self.names)

    def forward(self, x, step):
        ops = self.env.ops
        mid = ops.polynorm(project(ops, x, self.up, self.env.dtype), self.coefficients, self.eps, self.env.dtype)
        return DeferredLinear(ops, mid, self.down, self.env.dtype)


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    """A mixture of gated experts ``W_down (silu(W_gate x) * (W_up x))``, ``top`` of ``experts``
    per token, plus an optional feed-forward that every token runs (``shared``, a PartSpec).

    Router: logits ``W_router x`` in float32; scores are their softmax over all experts
    (``scores = "softmax"``) or their sigmoids (``"sigmoid"``).  Experts form ``group_count``
    equal groups of neighbours; a group's score is its largest score, and only experts of the
    ``group_keep`` best groups can be chosen (one group of all experts: no limit).  The ``top``
    largest scores among those win (the lower index on a tie); a token's weights are the
    chosen scores - divided by their sum (plus ``renorm_eps``) with ``renormalize`` - times
    ``scale``.  ``correction`` names a vector that is added to the scores for the CHOICE only
    (groups and experts are ranked by score + correction; a group that is not kept cannot be
    chosen however its corrected scores compare); the weights use the scores themselves.

    The last ``identity`` of the router's ``experts`` outputs are identity experts: no matrices,
    their output is the token's input itself, times the weight.  ``activation`` / ``limit`` are
    the experts' gated pair (as for ``swiglu``).  ``shared_gate`` names a ``[1, hidden]`` matrix:
    the shared feed-forward's output is multiplied by ``sigmoid(W_sg x)``, one number per token;
    its row rides on the router's product.

    The expert matrices are stacked ``[experts, 2 ff, hidden]`` (gate over up) and
    ``[experts, hidden, ff]`` when bound; a step's (token, choice) pairs are grouped by expert
    on the device and each group runs as row tiles of one launch, so nothing about the routing
    reaches the host and a captured step can be replayed."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        self.experts = int(p["experts"])
        self.top = int(p["top"])
        self.group_count = int(p.get("group_count", 1))
        self.group_keep = int(p.get("group_keep", self.group_count))
        self.scale = float(p.get("scale", 1.0))
        self.scores = p.get("scores", "softmax")
        self.renormalize = bool(p.get("renormalize", False))
        self.renorm_eps = float(p.get("renorm_eps", 0.0))
        self.identity = int(p.get("identity", 0))
        self.correction_name = p.get("correction")
        self.shared_gate_name = p.get("shared_gate")
        self.activation = p.get("activation", "silu")
        self.limit = float(p.get("limit") or 0.0)
        if self.activation not in GLU_ACTIVATIONS or (self.activation == "swish_clamped" and self.limit <= 0.0):
            raise UnsupportedShape("expert activation", (self.activation, self.limit), f"one of {GLU_ACTIVATIONS}; a clamped pair needs a positive limit")
        if not 0 <= self.identity < self.experts:
            raise UnsupportedShape("identity experts", self.identity, f"fewer than the router's {self.experts} outputs")
        if self.shared_gate_name is not None and p.get("shared") is None:
            raise UnsupportedShape("shared_gate", self.shared_gate_name, "a gate on a shared feed-forward that is absent")
        if self.scores not in ("softmax", "sigmoid"):
            raise UnsupportedShape("router scores", self.scores, "expected 'softmax' or 'sigmoid'")
        if not 0 < self.top <= self.experts or self.experts % self.group_count or not 0 < self.group_keep <= self.group_count:
            raise UnsupportedShape("router", (self.experts, self.top, self.group_count, self.group_keep), "top <= experts, groups must divide the experts, keep <= groups")
        if self.group_keep * (self.experts // self.group_count) < self.top:
            raise UnsupportedShape("router groups", (self.group_count, self.group_keep), f"the kept groups hold fewer than {self.top} experts")
        if self.experts > MAX_EXPERTS or self.top > MAX_TOP:
            raise UnsupportedShape("router", (self.experts, self.top), f"the routing kernel takes up to {MAX_EXPERTS} experts and {MAX_TOP} choices")
        self.router_name = p["router"]
        self.expert_names = tuple(p["expert_names"])
        if len(self.expert_names) != self.experts - self.identity:
            raise ValueError(f"{len(self.expert_names)} sets of names for {self.experts - self.identity} experts with matrices")
        self.shared = FEED_FORWARDS.build(p["shared"], env) if p.get("shared") is not None else None
        self.router = self.gate_up = self.down = self.correction = None

    def sub_parts(self):
        return [self.shared] if self.shared is not None else []

    def tensor_specs(self):
        specs = [TensorSpec(self.router_name, (self.experts, self.hidden))]
        for names in self.expert_names:
            specs += [TensorSpec(names["gate"], (self.inter, self.hidden)), TensorSpec(names["up"], (self.inter, self.hidden)),
                      TensorSpec(names["down"], (self.hidden, self.inter))]
        if self.shared is not None:
            specs += self.shared.tensor_specs()
        if self.correction_name is not None:
            specs.append(TensorSpec(self.correction_name, (self.experts,), VECTOR, NORMAL, init_std=0.02))
        if self.shared_gate_name is not None:
            specs.append(TensorSpec(self.shared_gate_name, (1, self.hidden)))
        return specs

    def bind(self, tensors):
        self.router = tensors[self.router_name]
        if self.shared_gate_name is not None:  # one more row of the router's product
            gate = tensors[self.shared_gate_name]
            if gate.dtype != self.router.dtype:
                gate, self.router = gate.float(), self.router.float()
            # (rows up to a multiple of eight are zeros: the tensor-memory products for long portions take such matrices)
            pad = torch.zeros((-(self.experts + 1) % 8, self.hidden), dtype=gate.dtype, device=gate.device)
            self.router = torch.cat([self.router, gate, pad], dim=0).contiguous()
        self.correction = tensors[self.correction_name] if self.correction_name is not None else None
        mats = [tensors[n[k]] for n in self.expert_names for k in ("gate", "up", "down")]
        wide = len({m.dtype for m in mats}) > 1
        pick = (lambda m: m.float()) if wide else (lambda m: m)
        self.gate_up = torch.stack([torch.cat([pick(tensors[n["gate"]]), pick(tensors[n["up"]])], dim=0) for n in self.expert_names]).contiguous()
        self.down = torch.stack([pick(tensors[n["down"]]) for n in self.expert_names]).contiguous()
        if self.shared is not None:
            self.shared.bind(tensors)

    def forward(self, x, step):
        ops = self.env.ops
        logits = ops.linear(x, self.router, torch.float32)
        more = {}
        if self.correction is not None:
            more["correction"] = self.correction
        if self.renorm_eps:
            more["renorm_eps"] = self.renorm_eps
        ids, weights = ops.moe_route(logits[:, : self.experts], self.top, self.group_count, self.group_keep, self.scale,
                                     self.scores == "sigmoid", self.renormalize, **more)
        extra = None
        if self.shared is not None:
            extra = self.shared.forward(x, step)
            if isinstance(extra, DeferredLinear):
                extra = extra.materialize()
        more = {}
        if self.activation != "silu":
            more["act"], more["limit"] = self.activation, self.limit
        if self.shared_gate_name is not None:
            more["extra_gate"] = logits[:, self.experts : self.experts + 1]  # [T, 1] float32 logits
        if self.identity:
            more["identity"] = self.identity
        return ops.routed_experts(x, ids, weights, self.gate_up, self.down, extra, **more)
