"""Token embedding and the output head.

Embedding: ``x_t = E[id_t]`` (crates/shiso-engine/src/layers.rs:1341-1357), times ``scale`` where a
model gives one (the product is formed in float32, so a table kept in 16 bits loses nothing to it).
Head: logits for the requested rows only, against the embedding table when tied or a
matrix of its own otherwise (layers.rs:2616-2681).  Logits are float32.

``hashed_pair_embedding`` adds, to the scaled token row, a row of a second table chosen by a
hash of (previous token, token): ``x_t = scale * E[id_t] + B[(id_{t-1} * a + id_t * b) mod n]``,
and ``B[n]`` (a row of its own behind the hashed ones) for a sequence's first token.  The
previous token is the last row's of the same sequence in the step, or, for a portion's first
row, what the request's state slot holds (token + 1; zero: no token yet).
"""

from __future__ import annotations

import torch

from ..weights.spec import TensorSpec
from .base import EMBEDDINGS, HEADS, Embedding, FixedState, Head, project


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Embedding):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.tensor_name = spec.params["tensor"]
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.scale = float(spec.params.get("scale", 1.0))
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.tensor_name, (self.vocab, self.hidden))]

    def bind(self, tensors):
        self.weight = tensors[self.tensor_name]

    def table(self):
        return self.weight

    def forward(self, step):
        feed = getattr(step, "feed_index", None)
        more = {"scale": self.scale} if self.scale != 1.0 else {}
        if feed is None:
            return self.env.ops.embed(step.token_ids, self.weight, **more)
        return self.env.ops.embed(step.token_ids, self.weight, feed, step.fed_tokens, **more)


@EMBEDDINGS.register("hashed_pair_embedding")
class HashedPairEmbedding(Embedding):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.tensor_name = p["tensor"]
        self.pair_name = p["pair_tensor"]
        self.vocab = int(p["vocab_size"])
        self.hidden = int(p["hidden_size"])
        self.scale = float(p.get("scale", 1.0))
        self.buckets = int(p["buckets"])
        self.mul_prev = int(p["mul_prev"])
        self.mul_cur = int(p["mul_cur"])
        if self.buckets <= 0:
            raise ValueError(f"a hashed table needs at least one bucket, got {self.buckets}")
        # the hash is formed in 64-bit integers on the device
        self.weight = self.pair = None

    def tensor_specs(self):
        return [
            TensorSpec(self.tensor_name, (self.vocab, self.hidden)),
            TensorSpec(self.pair_name, (self.buckets + 1, self.hidden)),
        ]

    def bind(self, tensors):
        self.weight = tensors[self.tensor_name]
        self.pair = tensors[self.pair_name]

    def table(self):
        return self.weight

    def cache_spec(self):
        return FixedState((1,), torch.int32)  # the request's last token + 1

    def forward(self, step, cache=None):
        return self.env.ops.embed_hashed_pair(
            step.token_ids, self.weight, self.pair, self.scale, self.buckets, self.mul_prev, self.mul_cur,
            step, cache.state, getattr(step, "feed_index", None), getattr(step, "fed_tokens", None),
        )


@HEADS.register("linear_head")
class LinearHead(Head):
    takes_deferred_norm = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.vocab = int(p["vocab_size"])
        self.hidden = int(p["hidden_size"])
        self.tied_to = p.get("tied_to")
        self.tensor_name = p.get("tensor")
        if (self.tied_to is None) == (self.tensor_name is None):
            raise ValueError("a head is either tied to a table or has a tensor of its own")
        self.weight = None

    def tensor_specs(self):
        if self.tied_to is not None:
            return []
        return [TensorSpec(self.tensor_name, (self.vocab, self.hidden))]

    def bind(self, tensors):
        self.weight = tensors[self.tied_to if self.tied_to is not None else self.tensor_name]

    def forward(self, x):
        """Float32 logits of the rows ``x``, a tensor or a ``DeferredNorm``."""
        return project(self.env.ops, x, self.weight, torch.float32)
