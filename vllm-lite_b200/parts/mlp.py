"""SwiGLU feed-forward: down(silu(gate(h)) * up(h)), no biases
(crates/model/src/components/mlp/swiglu.rs:18-31 of the reference).  gate and up
are bound by their own names and stacked at load time into one matrix: blocks of 8
gate rows followed by their 8 up rows (plain halves when the width is no multiple
of 8), so that a product kernel holds matching gate and up values in one tile and
can apply the activation itself.  Row order does not touch any row's arithmetic."""
from __future__ import annotations

import torch

from .linear import Linear
from .registry import FEED_FORWARDS
from .spec import SwiGLUSpec, TensorDecl


@FEED_FORWARDS.register("swiglu")
class SwiGLU:
    graph_safe = True

    @staticmethod
    def declare(spec: SwiGLUSpec) -> dict:
        return {"gate_proj.weight": TensorDecl((spec.intermediate_size, spec.hidden_size)),
                "up_proj.weight": TensorDecl((spec.intermediate_size, spec.hidden_size)),
                "down_proj.weight": TensorDecl((spec.hidden_size, spec.intermediate_size))}

    def __init__(self, spec: SwiGLUSpec, weights: dict, ctx):
        self.spec = spec
        self.dtype = ctx.dtype
        gate, up = weights["gate_proj.weight"], weights["up_proj.weight"]
        inter, hidden = spec.intermediate_size, spec.hidden_size
        self.group = 8 if inter % 8 == 0 else 0
        if self.group:
            g = self.group
            stacked = torch.stack([gate.view(inter // g, g, hidden), up.view(inter // g, g, hidden)], dim=1)
            stacked = stacked.reshape(2 * inter, hidden)
        else:
            stacked = torch.cat([gate, up], dim=0)
        self.gate_up = Linear(stacked.contiguous())
        self.down = Linear(weights["down_proj.weight"])

    def factors_norms(self, M) -> bool:
        """For M rows: the input may come as `ScaledRows` and the result may go `into_stream`."""
        from ..csrc import ops
        return self.group == ops.SWIGLU_GROUP and self.gate_up.factors_norms(M) and self.down.factors_norms(M)

    def __call__(self, h, step, sink=None):
        act = self.gate_up.swiglu(h, step, "mlp.gate_up", self.group)
        if sink is not None:
            return self.down.into_stream(act, sink, step, "mlp.down")
        return self.down(act, step, "mlp.down")
