"""Povilorn: typed configuration and model plan.

A pre-norm decoder whose norms are squashings without statistics (``tanh(alpha x) * w + b``).
A layer's mixer is ``attention`` - grouped-query softmax attention without rotation, whose values
are the keys as projected, with one RMS norm over all query heads together and one over all key
heads, a query temperature that grows with the logarithm of the position, and an elementwise
sigmoid gate before the output projection - or ``latent_attention`` - keys and values expanded
from a cached latent, one rotated key part shared by the heads, queries straight from the input,
neighbouring rotation pairs on a stretched frequency ladder with a magnitude.  Its feed-forward
is ``dense`` (a gated pair with the tanh form of gelu), ``moe`` (softmax router over experts and
identity experts, a correction on the choice, groups, renormalised weights, clamped experts and a
gated shared expert) or absent.  A stretch of layers may run several times with the same weights,
each pass with caches of its own; every pass starts by adding a vector of its own to the stream
and, from the second on, the embedding's output.  The embedding is scaled; the head has a matrix
of its own.

config.json keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``,
``loop.{start, stop, times}`` and ``layers``: a list of ``{"type", "mixer", "mlp"}`` with, for
``attention``, ``mixer.{heads, kv_heads, dim, vdim, scale, q_temp.{coef, every}}``; for
``latent_attention``, ``mixer.{heads, dim, rot_dim, vdim, kv_rank, scale, rot.{dims, base,
scaling.{factor, original, fast, slow}}}``; and ``mlp.{kind, ff}`` or ``mlp.{kind, expert.{ff,
limit}, router.{experts, identity, top, groups.{count, keep}}, shared.{ff, limit}}`` or null.
Tensor names: ``embed``, ``head``, ``final.norm{, .alpha, .b}``, ``loop.step`` and, for layer
``i``, ``l<i>.norm1/2{, .alpha, .b}``, ``l<i>.mix.*`` (``q, q.b, k, k.b, q.norm, k.norm, g, o`` /
``q, dkv, dkv.norm, uk, uv, o``), ``l<i>.mlp.{gate, up, down}`` or ``l<i>.mlp.{router, correction,
e<j>.{gate, up, down}, shared.{gate, up, down, sg}}``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping, Optional

from ..parts.plan import LayerSpec, ModelPlan, PartSpec, RunEntry
from .errors import ConfigMissing, InvalidValue
from .registry import register_architecture

ARCHITECTURE = "Povilorn"
ATTENTION = "attention"
LATENT = "latent_attention"
DENSE = "dense"
MOE = "moe"
RENORM_EPS = 1e-20  # added to the sum of a token's chosen scores before they are divided by it
LOOP_VECTORS = "loop.step"


def _get(document: Mapping[str, Any], path: str):
    at = document
    for key in path.split("."):
        if not isinstance(at, Mapping) or key not in at or at[key] is None:
            raise ConfigMissing(path)
        at = at[key]
    return at


def _int(document, path: str, least: int = 1) -> int:
    value = _get(document, path)
    if isinstance(value, bool) or not isinstance(value, int) or value < least:
        raise InvalidValue(path, value, f"expected an integer of at least {least}")
    return value


def _num(document, path: str) -> float:
    value = _get(document, path)
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise InvalidValue(path, value, "expected a number")
    return float(value)


@dataclass(frozen=True)
class PovilornConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple  # the documents of the layers, checked
    embedding_scale: float = 1.0
    loop: Optional[tuple] = None  # (start, stop, times)

    @classmethod
    def from_dict(cls, document: Mapping[str, Any]) -> "PovilornConfig":
        if document.get("architecture") != ARCHITECTURE:
            raise InvalidValue("architecture", document.get("architecture"), f"expected {ARCHITECTURE!r}")
        vocab, width = _int(document, "vocab"), _int(document, "width")
        eps = _num(document, "norm.eps")
        if not 0.0 < eps < 1.0:
            raise InvalidValue("norm.eps", eps, "expected a small positive number")
        embedding = document.get("embedding") or {}
        scale = _num(document, "embedding.scale") if embedding.get("scale") is not None else 1.0
        layers = _get(document, "layers")
        if not isinstance(layers, list) or not layers:
            raise InvalidValue("layers", layers, "expected a non-empty list of layers")
        for i, layer in enumerate(layers):
            cls._check_layer(i, layer)
        loop = None
        if document.get("loop") is not None:
            loop = (_int(document, "loop.start", 0), _int(document, "loop.stop", 0), _int(document, "loop.times", 1))
            if not loop[0] <= loop[1] <= len(layers):
                raise InvalidValue("loop", document["loop"], f"start <= stop <= {len(layers)} layers is needed")
        return cls(vocab=vocab, width=width, eps=eps, layers=tuple(copy.deepcopy(layers)), embedding_scale=scale, loop=loop)

    @staticmethod
    def _check_layer(i: int, layer) -> None:
        at = f"layers[{i}]"
        if not isinstance(layer, Mapping):
            raise InvalidValue(at, layer, "expected an object")
        kind = layer.get("type")
        if kind == ATTENTION:
            for key in ("heads", "kv_heads", "dim", "vdim"):
                _int(layer, f"mixer.{key}")
            _num(layer, "mixer.scale")
            m = layer["mixer"]
            if m["heads"] % m["kv_heads"]:
                raise InvalidValue(f"{at}.mixer.kv_heads", m["kv_heads"], f"does not divide {m['heads']} query heads")
            if m["vdim"] != m["dim"]:
                raise InvalidValue(f"{at}.mixer.vdim", m["vdim"], f"the values are the keys, of size dim = {m['dim']}")
            if m.get("q_temp") is not None:
                _num(layer, "mixer.q_temp.coef"), _int(layer, "mixer.q_temp.every")
        elif kind == LATENT:
            for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "rot.dims"):
                _int(layer, f"mixer.{key}")
            _num(layer, "mixer.scale")
            m = layer["mixer"]
            if _num(layer, "mixer.rot.base") <= 0:
                raise InvalidValue(f"{at}.mixer.rot.base", m["rot"]["base"], "expected a positive base")
            if m["rot"]["dims"] % 2 or m["rot"]["dims"] > m["rot_dim"]:
                raise InvalidValue(f"{at}.mixer.rot.dims", m["rot"]["dims"], f"must be even and at most rot_dim = {m['rot_dim']}")
            if m["rot"].get("scaling") is not None:
                for key in ("factor", "original", "fast", "slow"):
                    _num(layer, f"mixer.rot.scaling.{key}")
        else:
            raise InvalidValue(f"{at}.type", kind, f"expected {ATTENTION!r} or {LATENT!r}")
        mlp = layer.get("mlp")
        if mlp is None:
            return
        if mlp.get("kind") == DENSE:
            _int(layer, "mlp.ff")
        elif mlp.get("kind") == MOE:
            experts, top = _int(layer, "mlp.router.experts"), _int(layer, "mlp.router.top")
            identity = _int(layer, "mlp.router.identity", 0) if mlp["router"].get("identity") is not None else 0
            _int(layer, "mlp.expert.ff")
            if _num(layer, "mlp.expert.limit") <= 0:
                raise InvalidValue(f"{at}.mlp.expert.limit", mlp["expert"]["limit"], "expected a positive limit")
            outputs = experts + identity
            if top > outputs:
                raise InvalidValue(f"{at}.mlp.router.top", top, f"more than the {outputs} experts and identity experts")
            groups = mlp["router"].get("groups")
            if groups is not None:
                count, keep = _int(layer, "mlp.router.groups.count"), _int(layer, "mlp.router.groups.keep")
                if outputs % count or keep > count:
                    raise InvalidValue(f"{at}.mlp.router.groups", groups, f"count must divide the {outputs} router outputs and keep be at most count")
                if keep * (outputs // count) < top:
                    raise InvalidValue(f"{at}.mlp.router.groups", groups, f"{keep} groups hold fewer than top = {top} experts")
            if mlp.get("shared") is not None:
                _int(layer, "mlp.shared.ff")
                if _num(layer, "mlp.shared.limit") <= 0:
                    raise InvalidValue(f"{at}.mlp.shared.limit", mlp["shared"]["limit"], "expected a positive limit")
        else:
            raise InvalidValue(f"{at}.mlp.kind", mlp.get("kind"), f"expected {DENSE!r} or {MOE!r}")

    def to_dict(self) -> dict:
        document = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                    "embedding": {"scale": self.embedding_scale}, "layers": copy.deepcopy(list(self.layers))}
        if self.loop is not None:
            document["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        return document

    def run_order(self) -> list:
        """``(layer, pass)`` in running order: ``pass`` is the number of the pass that begins with
        this run of the layer, or None."""
        n = len(self.layers)
        if self.loop is None or self.loop[0] == self.loop[1]:  # (a stretch without layers has no pass to begin)
            return [(i, None) for i in range(n)]
        start, stop, times = self.loop
        order = [(i, None) for i in range(start)]
        for t in range(times):
            order += [(i, t if i == start else None) for i in range(start, stop)]
        return order + [(i, None) for i in range(stop, n)]


def _position_spec(rot: Mapping[str, Any]) -> PartSpec:
    scaling = rot.get("scaling")
    if scaling is None:
        return PartSpec("rope_half_split", {"theta": rot["base"], "rotary_dim": rot["dims"], "interleaved": True})
    return PartSpec("rope_stretched", {
        "theta": rot["base"], "rotary_dim": rot["dims"], "interleaved": True, "factor": scaling["factor"],
        "original": scaling["original"], "fast": scaling["fast"], "slow": scaling["slow"],
    })


def _mixer_spec(kind: str, m: Mapping[str, Any], p: str, width: int, eps: float) -> PartSpec:
    if kind == ATTENTION:
        return PartSpec("masked_attention", {
            "hidden_size": width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"],
            "scale": m["scale"], "mask": {"kind": "causal"}, "weights": "softmax", "values": "keys", "head_norm": "joined", "eps": eps,
            "q_temperature": dict(m["q_temp"]) if m.get("q_temp") is not None else None, "gate_per": "element",
            "q_proj": f"{p}.q", "k_proj": f"{p}.k", "q_bias": f"{p}.q.b", "k_bias": f"{p}.k.b", "q_norm": f"{p}.q.norm",
            "k_norm": f"{p}.k.norm", "gate": f"{p}.g", "out_proj": f"{p}.o",
        })
    return PartSpec("latent_attention", {
        "hidden_size": width, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"], "v_head_dim": m["vdim"],
        "q_rank": None, "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": eps, "position": _position_spec(m["rot"]),
        "q_proj": f"{p}.q", "kv_down": f"{p}.dkv", "kv_norm": f"{p}.dkv.norm", "k_up": f"{p}.uk", "v_up": f"{p}.uv", "gate": None,
        "out_proj": f"{p}.o",
    })


def _pair_names(p: str) -> dict:
    return {"gate": f"{p}.gate", "up": f"{p}.up", "down": f"{p}.down"}


def _ff_spec(mlp: Mapping[str, Any], p: str, width: int) -> PartSpec:
    if mlp["kind"] == DENSE:
        return PartSpec("swiglu", {"hidden_size": width, "intermediate_size": mlp["ff"], "activation": "gelu_tanh", **_pair_names(p)})
    r = mlp["router"]
    identity = r.get("identity") or 0
    groups = r.get("groups") or {"count": 1, "keep": 1}
    shared = None
    if mlp.get("shared") is not None:
        shared = PartSpec("swiglu", {"hidden_size": width, "intermediate_size": mlp["shared"]["ff"], "activation": "swish_clamped",
                                     "limit": mlp["shared"]["limit"], **_pair_names(f"{p}.shared")})
    return PartSpec("routed_experts", {
        "hidden_size": width, "intermediate_size": mlp["expert"]["ff"], "experts": r["experts"] + identity, "identity": identity,
        "top": r["top"], "group_count": groups["count"], "group_keep": groups["keep"], "scale": 1.0, "scores": "softmax",
        "renormalize": True, "renorm_eps": RENORM_EPS, "correction": f"{p}.correction", "activation": "swish_clamped",
        "limit": mlp["expert"]["limit"], "router": f"{p}.router",
        "expert_names": tuple(_pair_names(f"{p}.e{e}") for e in range(r["experts"])),
        "shared": shared, "shared_gate": f"{p}.shared.sg" if shared is not None else None,
    })


def build_plan(config: PovilornConfig) -> ModelPlan:
    width, eps = config.width, config.eps

    def norm(name: str) -> PartSpec:
        return PartSpec("dyt", {"tensor": name, "size": width})

    layers = []
    for i, layer in enumerate(config.layers):
        prefix = f"l{i}"
        mlp = layer.get("mlp")
        layers.append(LayerSpec(
            name=prefix,
            block=PartSpec("pre_norm"),
            mixer=_mixer_spec(layer["type"], layer["mixer"], f"{prefix}.mix", width, eps),
            mixer_norm=norm(f"{prefix}.norm1"),
            feed_forward=_ff_spec(mlp, f"{prefix}.mlp", width) if mlp is not None else None,
            feed_forward_norm=norm(f"{prefix}.norm2") if mlp is not None else None,
        ))
    order = tuple(
        RunEntry(layer=i, add_first=bool(begins), add_vector=(LOOP_VECTORS, begins) if begins is not None else None)
        for i, begins in config.run_order()
    )
    unused = tuple(name for i, layer in enumerate(config.layers) if layer.get("mlp") is None
                   for name in (f"l{i}.norm2", f"l{i}.norm2.alpha", f"l{i}.norm2.b"))
    if not any(entry.add_vector is not None for entry in order):
        unused += (LOOP_VECTORS,)
    return ModelPlan(
        architecture=ARCHITECTURE,
        hidden_size=width,
        vocab_size=config.vocab,
        embedding=PartSpec("token_embedding", {"tensor": "embed", "vocab_size": config.vocab, "hidden_size": width,
                                               "scale": config.embedding_scale}),
        layers=tuple(layers),
        order=order,
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": config.vocab, "hidden_size": width, "tied_to": None, "tensor": "head"}),
        unused_tensors=unused,
    )


register_architecture(ARCHITECTURE, PovilornConfig, build_plan)
