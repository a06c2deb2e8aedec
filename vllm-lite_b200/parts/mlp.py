"""SwiGLU feed-forward: down(silu(gate(h)) * up(h)), no biases
(crates/model/src/components/mlp/swiglu.rs:18-31 of the reference).  gate and up
are bound by their own names and stacked at load time into one [gate | up] matrix."""
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
        self.gate_up = Linear(torch.cat([weights["gate_proj.weight"], weights["up_proj.weight"]], dim=0).contiguous())
        self.down = Linear(weights["down_proj.weight"])

    def __call__(self, h, step):
        from ..csrc import ops
        gu = self.gate_up(h, step, "mlp.gate_up")
        act = step.workspace.get(step.tag + "mlp.act", (h.shape[0], self.spec.intermediate_size), self.dtype)
        ops.silu_mul(gu, act)
        return self.down(act, step, "mlp.down")
