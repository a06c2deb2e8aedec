"""Chooses the attention kernel for a step.

Every kernel computes the same function of (query token, its request's pages);
which one runs depends on the dtype and on the shape of the step only.  The
float32 path always takes the one kernel whose order of additions depends on
positions alone, so its results are bit-for-bit independent of the batch.  In
bfloat16 a step of single tokens (decoding) takes the kernel that splits each
token's key range over many blocks.
"""
from __future__ import annotations

import torch


def run(qkv, out, cache, group, step, spec, scale):
    from ..csrc import ops
    args = (qkv, out, cache.k, cache.v, group.block_table, step.req_index, step.positions,
            spec.num_heads, spec.num_kv_heads, spec.head_dim, scale, spec.window)
    if qkv.dtype == torch.bfloat16 and step.max_query_len == 1:
        T = qkv.shape[0]
        S, n_acc, n_ml = ops.decode_attention_scratch(T, spec.num_heads, spec.head_dim, group.max_context)
        part_acc = step.workspace.get(step.tag + "attn.part_acc", (n_acc,), torch.float32)
        part_ml = step.workspace.get(step.tag + "attn.part_ml", (n_ml,), torch.float32)
        return ops.decode_attention(*args, group.max_context, part_acc, part_ml, step.err)
    return ops.paged_attention(*args, step.err)
