"""Chooses the attention kernel for a step.

Every kernel computes the same function of (query token, its request's pages);
which one runs depends on the dtype and on the shape of the step only.
"""
from __future__ import annotations


def run(qkv, out, cache, group, step, spec, scale):
    from ..csrc import ops
    return ops.paged_attention(qkv, out, cache.k, cache.v, group.block_table, step.req_index, step.positions,
                               spec.num_heads, spec.num_kv_heads, spec.head_dim, scale, spec.window, step.err)
