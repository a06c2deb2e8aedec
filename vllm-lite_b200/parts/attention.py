"""Grouped-query attention with per-head norm of q and k before the rotation.

project -> head norm -> rotation -> cache write -> attention over the pages ->
output projection (crates/model/src/components/attention/rope_gqa.rs:261-305 of
the reference).  The three projections are bound by their own tensor names and
stacked at load time into one [q | k | v] matrix, which keeps every output row's
arithmetic unchanged.  A prompt portion, a continuation and a decoded token are
the same case: every token's key and value are written first, then each query
reads positions 0..its own (or its window) from the pages.
"""
from __future__ import annotations

import torch

from ..cache.spec import PagedKV
from .base import sub_weights
from .linear import Linear
from .registry import MIXERS, NORMS, POSITIONS
from .spec import AttentionSpec, TensorDecl


MAX_HEAD_DIM = 256


def check_attention_sizes(spec: AttentionSpec):
    """What the attention kernels take, checked when a model is planned or built instead of in its first
    step: head sizes in steps of 16 up to 256, and kv heads that divide the query heads."""
    if spec.num_heads <= 0 or spec.num_kv_heads <= 0 or spec.num_heads % spec.num_kv_heads:
        raise ValueError(f"{spec.num_kv_heads} kv heads do not divide {spec.num_heads} query heads")
    if spec.head_dim % 16 or not 16 <= spec.head_dim <= MAX_HEAD_DIM:
        raise ValueError(f"head_dim {spec.head_dim}: the attention kernels take multiples of 16 from 16 to {MAX_HEAD_DIM}")
    if spec.qk_norm is not None and spec.qk_norm.size != spec.head_dim:
        raise ValueError("the head norm runs over head_dim")
    if spec.window is not None and spec.window <= 0:
        raise ValueError(f"window {spec.window} must be positive (None reads every earlier key)")


@MIXERS.register("gqa_attention")
class GqaAttention:
    graph_safe = True          # launches only stream-ordered kernels: a step can be captured in a CUDA graph

    @staticmethod
    def declare(spec: AttentionSpec) -> dict:
        qd, kvd = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        d = {"q_proj.weight": TensorDecl((qd, spec.hidden_size)),
             "k_proj.weight": TensorDecl((kvd, spec.hidden_size)),
             "v_proj.weight": TensorDecl((kvd, spec.hidden_size)),
             "o_proj.weight": TensorDecl((spec.hidden_size, qd))}
        if spec.bias:
            d.update({"q_proj.bias": TensorDecl((qd,)), "k_proj.bias": TensorDecl((kvd,)),
                      "v_proj.bias": TensorDecl((kvd,))})
        if spec.qk_norm is not None:
            for side in ("q_norm.", "k_norm."):
                for name, decl in NORMS.get(spec.qk_norm.kind).declare(spec.qk_norm).items():
                    d[side + name] = decl
        if spec.position is not None:
            for name, decl in POSITIONS.get(spec.position.kind).declare(spec.position).items():
                d["rotary." + name] = decl
        return d

    @staticmethod
    def cache_need(spec: AttentionSpec):
        return PagedKV(spec.num_kv_heads, spec.head_dim, spec.window)

    def __init__(self, spec: AttentionSpec, weights: dict, ctx):
        check_attention_sizes(spec)
        self.spec = spec
        self.dtype = ctx.dtype
        qkv = torch.cat([weights["q_proj.weight"], weights["k_proj.weight"], weights["v_proj.weight"]], dim=0)
        bias = None
        if spec.bias:
            bias = torch.cat([weights["q_proj.bias"].float(), weights["k_proj.bias"].float(),
                              weights["v_proj.bias"].float()], dim=0)
        self.qkv_proj = Linear(qkv.contiguous(), bias)
        self.o_proj = Linear(weights["o_proj.weight"])
        self.q_norm = self.k_norm = None
        # The kernel that rotates and writes the cache also applies an RMS norm to every head.  A head norm
        # that says it is one (`fused_rms()` -> (weight, eps)) runs there; any other kind must change the
        # heads itself (`apply_heads`), and the kernel is then given no norm.
        self.fused_head_norm = None
        if spec.qk_norm is not None:
            cls = NORMS.get(spec.qk_norm.kind)
            self.q_norm = cls(spec.qk_norm, sub_weights(weights, "q_norm."), ctx)
            self.k_norm = cls(spec.qk_norm, sub_weights(weights, "k_norm."), ctx)
            if hasattr(self.q_norm, "fused_rms"):
                (qw, eps), (kw, _) = self.q_norm.fused_rms(), self.k_norm.fused_rms()
                self.fused_head_norm = (qw, kw, eps)
            elif not hasattr(self.q_norm, "apply_heads"):
                raise TypeError(f"norm kind {spec.qk_norm.kind!r} cannot serve as a head norm: it offers neither "
                                f"fused_rms() nor apply_heads(qkv, first_head, num_heads, head_dim, step)")
        self.position = None
        if spec.position is not None:
            self.position = POSITIONS.get(spec.position.kind)(spec.position, sub_weights(weights, "rotary."), ctx)
        self.scale = spec.scale if spec.scale is not None else spec.head_dim ** -0.5

    def factors_norms(self, M) -> bool:
        """For M rows: the input may come as `ScaledRows` and the result may go `into_stream`."""
        return self.qkv_proj.factors_norms(M) and self.o_proj.factors_norms(M)

    def __call__(self, h, step, cache, sink=None):
        from ..csrc import ops
        s = self.spec
        group = step.groups[cache.group]
        qkv = self.qkv_proj(h, step, "attn.qkv")
        fused = self.position.fused_rotary() if self.position is not None else None
        if self.position is not None and fused is None:
            # an encoding that the fused kernel does not know acts on the q and k parts of qkv itself
            # (after the projections, before the head norm's kernel writes the cache)
            self.position.apply(qkv, step.positions, s.num_heads, s.num_kv_heads, s.head_dim, step)
        inv_freq, rot = fused if fused is not None else (None, 0)
        if self.q_norm is not None and self.fused_head_norm is None:
            # a head norm of a kind of its own: it edits the q heads and the k heads of qkv in place
            self.q_norm.apply_heads(qkv, 0, s.num_heads, s.head_dim, step)
            self.k_norm.apply_heads(qkv, s.num_heads, s.num_kv_heads, s.head_dim, step)
        qw, kw, eps = self.fused_head_norm if self.fused_head_norm is not None else (None, None, 0.0)
        slots = group.slots if cache.writes else None
        from . import attention_dispatch
        fold = None
        if attention_dispatch.folds_head_work(qkv.dtype, step, s, group, qkv.shape[0]):
            fold = (qw, kw, eps, inv_freq, rot, slots)          # the attention kernel does it on the way
        else:
            ops.qk_norm_rope_write(qkv, step.positions, slots, qw, kw, eps, inv_freq, rot, cache.k, cache.v,
                                   s.num_heads, s.num_kv_heads, s.head_dim, step.err)
        out = step.workspace.get(step.tag + "attn.out", (qkv.shape[0], s.num_heads * s.head_dim), self.dtype)
        attention_dispatch.run(qkv, out, cache, group, step, s, self.scale, fold=fold)
        if sink is not None:
            return self.o_proj.into_stream(out, sink, step, "attn.o")
        return self.o_proj(out, step, "attn.o")
