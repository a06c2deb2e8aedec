"""Output head: logits = h W^T in float32, no bias; W is the embedding's table when the head is tied
(crates/model/src/causal_lm/weights.rs:19-36 of the reference).

An output head offers
    declare(spec) -> {relative tensor name: TensorDecl}            static
    __init__(spec, weights, ctx, embedding)      embedding: the model's embedding part
    __call__(h, step) -> float32 [rows, vocab]   h: the final norm's output on the wanted rows
and may say `graph_safe = True` (parts/base.py)."""
from __future__ import annotations

import torch

from .linear import Linear
from .registry import HEADS
from .spec import HeadSpec, TensorDecl


@HEADS.register("linear_head")
class LinearHead:
    graph_safe = True

    @staticmethod
    def declare(spec: HeadSpec) -> dict:
        return {} if spec.tied else {"weight": TensorDecl((spec.vocab_size, spec.hidden_size))}

    def __init__(self, spec: HeadSpec, weights: dict, ctx, embedding=None):
        self.spec = spec
        if spec.tied:
            weight = embedding.tied_weight() if embedding is not None else None
            if weight is None or tuple(weight.shape) != (spec.vocab_size, spec.hidden_size):
                raise ValueError("a tied output head needs an embedding that shares a [vocab, hidden] table")
        else:
            weight = weights["weight"]
        self.proj = Linear(weight)

    def __call__(self, h, step):
        return self.proj(h, step, "logits", out_dtype=torch.float32)
