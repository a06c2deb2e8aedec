"""A causal language model assembled from a `ModelPlan`:
embedding -> the calls of the running order -> final norm -> output head
(crates/model/src/causal_lm/mod.rs:180-221 of the reference).  Only the rows
whose logits are wanted go through the final norm and the head."""
from __future__ import annotations

import torch

from .base import BuildContext, Residual, prefixed, sub_weights
from .registry import BLOCKS, EMBEDDINGS, HEADS, NORMS
from .spec import ModelPlan, TensorDecl


def declare_model(plan: ModelPlan) -> dict:
    """Every tensor the model binds: {checkpoint name: TensorDecl}."""
    emb, head = plan.embedding_spec, plan.head_spec
    d = prefixed(EMBEDDINGS.get(emb.kind).declare(emb), plan.embed_prefix)
    for i, block in enumerate(plan.layers):
        d.update(prefixed(BLOCKS.get(block.kind).declare(block), plan.layer_prefix.format(i)))
    d.update(prefixed(NORMS.get(plan.final_norm.kind).declare(plan.final_norm), plan.final_norm_prefix))
    d.update(prefixed(HEADS.get(head.kind).declare(head), plan.head_prefix))
    return d


def cache_needs(plan: ModelPlan) -> list:
    """The need of every entry of the running order (None for an entry that
    keeps nothing or that reads another entry's cache)."""
    needs = []
    for call in plan.order:
        block = plan.layers[call.layer]
        needs.append(None if call.cache_of is not None else BLOCKS.get(block.kind).cache_need(block))
    return needs


class CausalLM:
    def __init__(self, plan: ModelPlan, weights: dict, ctx: BuildContext):
        plan.validate()
        self.plan = plan
        self.ctx = ctx
        emb, head = plan.embedding_spec, plan.head_spec
        self.embedding = EMBEDDINGS.get(emb.kind)(emb, sub_weights(weights, plan.embed_prefix), ctx)
        self.layers = [BLOCKS.get(b.kind)(b, sub_weights(weights, plan.layer_prefix.format(i)), ctx)
                       for i, b in enumerate(plan.layers)]
        self.final_norm = NORMS.get(plan.final_norm.kind)(plan.final_norm,
                                                          sub_weights(weights, plan.final_norm_prefix), ctx)
        self.head = HEADS.get(head.kind)(head, sub_weights(weights, plan.head_prefix), ctx, embedding=self.embedding)
        self.graph_safe = all(getattr(part, "graph_safe", False) for part in [self.embedding, self.head] + self.layers)

    def forward(self, step, caches) -> torch.Tensor:
        """Logits float32 [len(step.logit_rows), vocab]."""
        ws = step.workspace
        x = ws.get(step.tag + "residual", (step.num_tokens, self.plan.hidden_size), torch.float32)
        self.embedding(step, x)
        residual = Residual(x)
        order = self.plan.order
        for i, (call, cache) in enumerate(zip(order, caches)):
            layer = self.layers[call.layer]
            if getattr(layer, "chains_norms", False):
                # a block may leave the next block's first norm in factored form (parts/base.py, ScaledRows)
                nxt = self.layers[order[i + 1].layer] if i + 1 < len(order) else None
                ask = getattr(nxt, "input_norm_for_fusion", None)
                layer(residual, step, cache, next_norm=ask(step.num_tokens) if ask else None)
            else:
                layer(residual, step, cache)
        R = step.logit_rows.shape[0]
        if R == 0:
            return ws.get(step.tag + "logits", (0, self.plan.vocab_size), torch.float32)
        h = self.final_norm(residual.x, residual.pending, step, rows=step.logit_rows, tag="final_norm")   # pending: the last block has no next norm
        return self.head(h, step)
