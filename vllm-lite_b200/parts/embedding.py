"""Token embedding: x[t] = table[id[t]], a row gather into the float32 residual stream, no scaling
(crates/model/src/causal_lm/mod.rs:28-46 of the reference).

An embedding part offers
    declare(spec) -> {relative tensor name: TensorDecl}            static
    __init__(spec, weights, ctx)
    __call__(step, x)        fills x float32 [T, hidden] from step.tokens (and step.positions if it likes)
    tied_weight()            the [vocab, hidden] matrix an output head may share, or None
and may say `graph_safe = True` (parts/base.py)."""
from __future__ import annotations

from .registry import EMBEDDINGS
from .spec import EmbeddingSpec, TensorDecl


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding:
    graph_safe = True

    @staticmethod
    def declare(spec: EmbeddingSpec) -> dict:
        return {"weight": TensorDecl((spec.vocab_size, spec.hidden_size))}

    def __init__(self, spec: EmbeddingSpec, weights: dict, ctx):
        self.spec = spec
        self.table = weights["weight"]

    def tied_weight(self):
        return self.table

    def __call__(self, step, x):
        from ..csrc import ops
        return ops.embed(step.tokens, self.table, x, step.err)     # an id outside the table is flagged, not read
