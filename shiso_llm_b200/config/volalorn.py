"""Volalorn: typed configuration and model plan.

A decoder whose layers norm what a sublayer gives back, ``x <- x + norm1(mixer(x))`` and then
``x <- x + norm2(ff(x))``: the sublayers read the stream itself, and every norm of the model is
an RMS norm with ONE number as its weight.  A layer's mixer is ``attention`` (grouped-query,
no biases, rotation with an optionally stretched ladder, then a unit RMS norm of queries and
keys, scores capped by ``softcap * tanh(. / softcap)``, keys of the row's own chunk only, one
``sigmoid(score + pb[head])`` per key instead of a softmax, a sigmoid gate per head before the
output projection) or ``attention_2`` (grouped-query with biases, a weighted RMS norm of
queries and keys before the rotation, a sliding window that also keeps the sequence's first
tokens, softmax).  Its feed-forward is ``dense`` (``W_down act(W_up x)`` with a polynomial of
unit-RMS powers as ``act``) or absent.  The head has a matrix of its own; logits are scaled by
``logit_scale``, which rides on the final norm's weight.

config.json keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``logit_scale`` (absent:
1) and ``layers``: a list of ``{"type", "mixer", "mlp"}`` with ``mixer.{heads, kv_heads, dim,
vdim, scale, mask.{size, keep_first}, rot.{dims, base, scaling.{factor, original, fast, slow}},
softcap}`` (``keep_first`` belongs to ``attention_2`` and may be absent: none kept; ``scaling``
and ``softcap`` may be absent: a plain ladder, no cap) and ``mlp.{kind, ff}`` or null.
Tensor names: ``embed``, ``final.norm``, ``head`` and, for layer ``i``, ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.{q, k, v, o}`` plus ``{pb, g}`` (attention) or ``{q.b, k.b, v.b,
q.norm, k.norm}`` (attention_2), and ``l<i>.mlp.{up, down, act}``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping

from ..parts.plan import LayerSpec, ModelPlan, PartSpec, RunEntry
from .errors import InvalidValue
from .registry import register_architecture
from .zetavik import _get, _int, _num

ARCHITECTURE = "Volalorn"
CHUNKED = "attention"
WINDOWED = "attention_2"
DENSE = "dense"


@dataclass(frozen=True)
class VolalornConfig:
    vocab: int
    width: int
    eps: float
    logit_scale: float
    layers: tuple  # the documents of the layers, checked

    @classmethod
    def from_dict(cls, document: Mapping[str, Any]) -> "VolalornConfig":
        if document.get("architecture") != ARCHITECTURE:
            raise InvalidValue("architecture", document.get("architecture"), f"expected {ARCHITECTURE!r}")
        vocab, width = _int(document, "vocab"), _int(document, "width")
        eps = _num(document, "norm.eps")
        if not 0.0 < eps < 1.0:
            raise InvalidValue("norm.eps", eps, "expected a small positive number")
        logit_scale = _num(document, "logit_scale") if document.get("logit_scale") is not None else 1.0
        layers = _get(document, "layers")
        if not isinstance(layers, list) or not layers:
            raise InvalidValue("layers", layers, "expected a non-empty list of layers")
        for i, layer in enumerate(layers):
            cls._check_layer(i, layer)
        return cls(vocab=vocab, width=width, eps=eps, logit_scale=logit_scale, layers=tuple(copy.deepcopy(layers)))

    @staticmethod
    def _check_layer(i: int, layer) -> None:
        at = f"layers[{i}]"
        if not isinstance(layer, Mapping):
            raise InvalidValue(at, layer, "expected an object")
        kind = layer.get("type")
        if kind not in (CHUNKED, WINDOWED):
            raise InvalidValue(f"{at}.type", kind, f"expected {CHUNKED!r} or {WINDOWED!r}")
        for key in ("heads", "kv_heads", "dim", "vdim", "mask.size", "rot.dims"):
            _int(layer, f"mixer.{key}")
        _num(layer, "mixer.scale")
        m = layer["mixer"]
        if m["heads"] % m["kv_heads"]:
            raise InvalidValue(f"{at}.mixer.kv_heads", m["kv_heads"], f"does not divide {m['heads']} heads")
        if _num(layer, "mixer.rot.base") <= 1.0:
            raise InvalidValue(f"{at}.mixer.rot.base", m["rot"]["base"], "expected a base above 1")
        if m["rot"]["dims"] % 2 or m["rot"]["dims"] > m["dim"]:
            raise InvalidValue(f"{at}.mixer.rot.dims", m["rot"]["dims"], f"must be even and at most dim = {m['dim']}")
        if m["rot"].get("scaling") is not None:
            for key in ("factor", "original", "fast", "slow"):
                if _num(layer, f"mixer.rot.scaling.{key}") <= 0.0:
                    raise InvalidValue(f"{at}.mixer.rot.scaling.{key}", m["rot"]["scaling"][key], "expected a positive number")
            if m["rot"]["scaling"]["factor"] < 1.0:
                raise InvalidValue(f"{at}.mixer.rot.scaling.factor", m["rot"]["scaling"]["factor"], "a stretch is at least 1")
        if m.get("softcap") is not None and _num(layer, "mixer.softcap") <= 0.0:
            raise InvalidValue(f"{at}.mixer.softcap", m["softcap"], "a cap on the scores is positive")
        keep = m["mask"].get("keep_first")
        if keep is not None:
            if kind == CHUNKED:
                raise InvalidValue(f"{at}.mixer.mask.keep_first", keep, "a chunked mask keeps no first tokens")
            _int(layer, "mixer.mask.keep_first", 0)
        mlp = layer.get("mlp")
        if mlp is None:
            return
        if not isinstance(mlp, Mapping) or mlp.get("kind") != DENSE:
            raise InvalidValue(f"{at}.mlp.kind", mlp.get("kind") if isinstance(mlp, Mapping) else mlp, f"expected {DENSE!r}")
        _int(layer, "mlp.ff")

    def to_dict(self) -> dict:
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "logit_scale": self.logit_scale, "layers": copy.deepcopy(list(self.layers))}


def _position_spec(rot: Mapping[str, Any]) -> PartSpec:
    params = {"theta": rot["base"], "rotary_dim": rot["dims"]}
    scaling = rot.get("scaling")
    if scaling is None:
        return PartSpec("rope_half_split", params)
    return PartSpec("rope_stretched", {**params, **{k: scaling[k] for k in ("factor", "original", "fast", "slow")}})


def _mixer_spec(kind: str, m: Mapping[str, Any], p: str, width: int, eps: float) -> PartSpec:
    common = {
        "hidden_size": width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"],
        "scale": m["scale"], "softcap": m.get("softcap"), "eps": eps, "position": _position_spec(m["rot"]),
        "q_proj": f"{p}.q", "k_proj": f"{p}.k", "v_proj": f"{p}.v", "out_proj": f"{p}.o",
    }
    if kind == CHUNKED:
        return PartSpec("masked_attention", {
            **common, "mask": {"kind": "chunk", "size": m["mask"]["size"]}, "weights": "sigmoid", "head_norm": "after",
            "key_bias": f"{p}.pb", "gate": f"{p}.g",
        })
    return PartSpec("masked_attention", {
        **common, "mask": {"kind": "window", "size": m["mask"]["size"], "keep_first": m["mask"].get("keep_first") or 0},
        "weights": "softmax", "head_norm": "before", "q_norm": f"{p}.q.norm", "k_norm": f"{p}.k.norm",
        "q_bias": f"{p}.q.b", "k_bias": f"{p}.k.b", "v_bias": f"{p}.v.b",
    })


def _scalar_norm(name: str, width: int, eps: float, gain: float = 1.0) -> PartSpec:
    return PartSpec("rmsnorm", {"tensor": name, "size": width, "eps": eps, "scalar": True, "gain": gain})


def build_plan(config: VolalornConfig) -> ModelPlan:
    width, eps = config.width, config.eps
    layers, unused = [], []
    for i, layer in enumerate(config.layers):
        prefix = f"l{i}"
        mlp = layer.get("mlp")
        ff = ff_norm = None
        if mlp is not None:
            ff = PartSpec("polynorm_ff", {"hidden_size": width, "intermediate_size": mlp["ff"], "eps": eps,
                                          "up": f"{prefix}.mlp.up", "down": f"{prefix}.mlp.down", "act": f"{prefix}.mlp.act"})
            ff_norm = _scalar_norm(f"{prefix}.norm2", width, eps)
        else:
            unused.append(f"{prefix}.norm2")
        layers.append(LayerSpec(
            name=prefix,
            block=PartSpec("output_norm"),
            mixer=_mixer_spec(layer["type"], layer["mixer"], f"{prefix}.mix", width, eps),
            mixer_norm=_scalar_norm(f"{prefix}.norm1", width, eps),
            feed_forward=ff,
            feed_forward_norm=ff_norm,
        ))
    return ModelPlan(
        architecture=ARCHITECTURE,
        hidden_size=width,
        vocab_size=config.vocab,
        embedding=PartSpec("token_embedding", {"tensor": "embed", "vocab_size": config.vocab, "hidden_size": width}),
        layers=tuple(layers),
        order=tuple(RunEntry(layer=i) for i in range(len(layers))),
        final_norm=_scalar_norm("final.norm", width, eps, gain=config.logit_scale),
        head=PartSpec("linear_head", {"vocab_size": config.vocab, "hidden_size": width, "tied_to": None, "tensor": "head"}),
        unused_tensors=tuple(unused),
    )


register_architecture(ARCHITECTURE, VolalornConfig, build_plan)
