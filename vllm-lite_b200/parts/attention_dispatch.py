"""Chooses the attention kernel for a step.

Every kernel computes the same function of (query token, its request's pages);
which one runs depends on the dtype and on the shape of the step only.  The
float32 path always takes the one kernel whose order of additions depends on
positions alone, so its results are bit-for-bit independent of the batch.  In
bfloat16 the tensor-core kernels run: requests that bring one token (decoding)
go to the kernel that splits each token's key range over many blocks, requests
that bring a portion of a prompt to one that walks tiles of query tokens (the
tcgen05 kernel when a portion is long enough to fill its 128-row tiles and it
takes the head and page size, else the mma.sync kernel); a step that holds both
kinds launches both, each on its own tokens.
"""
from __future__ import annotations

import torch

from .base import QUERY_TILE


FOLD_MAX_CHUNKS = 4      # most chunks per token with which the decode attention still does the head work itself


def folds_head_work(dtype, step, spec, group, num_tokens) -> bool:
    """Whether `run` will do the head norm, the rotation and the cache write of this step itself (pass `fold`),
    so that the mixer launches no kernel for them: a decode step (every request brings one token) that the
    block-per-chunk kernel serves with few chunks per token (every chunk's block prepares the query heads
    again).  Measured at Qwen3-8B sizes, a step with / without: batch 8 at 4,096 keys (4 chunks) 3.77 / 3.79 ms,
    batch 16 at 1,024 keys (1 chunk) 3.99 / 4.06; batch 4 (8 chunks) 3.635 / 3.61, batch 1 (16 chunks) 3.07 / 3.065."""
    from ..csrc import ops
    if not (ops.flash_supported(dtype, spec.head_dim) and step.max_query_len == 1):
        return False
    if ops.flash_decode_streams(dtype, num_tokens, spec.num_kv_heads, spec.head_dim, group.page_size, group.max_context):
        return False
    chunk = ops.decode_chunk_for(num_tokens, spec.num_kv_heads, group.max_context, head_dim=spec.head_dim)
    return -(-int(group.max_context) // chunk) <= FOLD_MAX_CHUNKS


def _decode(ops, args, step, spec, group, num_tokens, max_context, token_index=None, fold=None):
    chunk = ops.decode_chunk_for(num_tokens, spec.num_kv_heads, max_context, head_dim=spec.head_dim)
    S, n_acc, n_ml = ops.decode_attention_scratch(num_tokens, spec.num_heads, spec.head_dim, max_context, chunk)
    part_acc = step.workspace.get(step.tag + "attn.part_acc", (n_acc,), torch.float32)
    part_ml = step.workspace.get(step.tag + "attn.part_ml", (n_ml,), torch.float32)
    # one set of counters for all layers of a step shape: every launch leaves them zero
    arrivals = step.workspace.zeros(step.tag + "attn.arrivals", ops.flash_decode_arrivals(num_tokens, spec.num_heads, spec.num_kv_heads),
                                    torch.int32)
    return ops.flash_decode(*args, max_context, part_acc, part_ml, step.err, chunk=chunk, token_index=token_index,
                            arrivals=arrivals, fold=fold)


def run(qkv, out, cache, group, step, spec, scale, fold=None):
    """`fold` (only where `folds_head_work` said so): (q_weight, k_weight, eps, inv_freq, rotary_dim, slots) of the
    head work that the mixer left undone."""
    from ..csrc import ops
    if fold is not None and not folds_head_work(qkv.dtype, step, spec, group, qkv.shape[0]):
        raise ValueError("this step's attention kernel does not fold the head norm and rotation in")
    args = (qkv, out, cache.k, cache.v, group.block_table, step.req_index, step.positions,
            spec.num_heads, spec.num_kv_heads, spec.head_dim, scale, spec.window)
    if ops.flash_supported(qkv.dtype, spec.head_dim):
        if step.max_query_len == 1:
            return _decode(ops, args, step, spec, group, qkv.shape[0], group.max_context, fold=fold)
        if step.query_tiles is not None:
            tile_args = (qkv, out, cache.k, cache.v, group.block_table, step.query_tiles,
                         spec.num_heads, spec.num_kv_heads, spec.head_dim, scale, spec.window, step.err)
            if step.max_query_len > 64 and ops.flash_tc5_supported(qkv.dtype, spec.head_dim, group.page_size):
                ops.flash_prefill_tc5(*tile_args)
            else:
                ops.flash_prefill(*tile_args, tile_rows=QUERY_TILE)
            if step.single_tokens is not None:
                _decode(ops, args, step, spec, group, step.single_tokens.shape[0], step.single_context,
                        token_index=step.single_tokens)
            return out
    return ops.paged_attention(*args, step.err)
