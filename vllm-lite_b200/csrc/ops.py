"""Python face of the CUDA kernels: one function per exported entry point.

Tensors are torch CUDA tensors used as plain device buffers; the kernels run on
torch's current stream.  Arguments are checked here (dtype, contiguity, sizes)
so that a kernel never sees a pointer that does not match its shape arguments.
A non-zero return code of an entry point raises `KernelError`.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}
_ERRORS = {-2: "a size this kernel does not take", -3: "inconsistent arguments",
           -4: "the problem does not fit the built-in scratch memory"}


class KernelError(RuntimeError):
    pass


def dtype_code(dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 and bfloat16, got {dtype}") from None


_SIGNATURES = {
    ("embed_norm", "vl_embed"): [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    ("embed_norm", "vl_add_rmsnorm"): [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
    ("embed_norm", "vl_add_bias"): [c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p],
    ("embed_norm", "vl_cast"): [c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p],
    ("rope_cache", "vl_qk_norm_rope_write"): [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int,
                                              c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_longlong, c_int,
                                              c_void_p, c_void_p],
    ("attention", "vl_paged_attention"): [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                          c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                          c_float, c_int, c_void_p, c_void_p],
    ("attention", "vl_decode_attention"): [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                           c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                           c_float, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    ("attention", "vl_decode_attention_merge"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                 c_int, c_int, c_void_p, c_void_p],
    ("flash_attn", "vl_flash_prefill"): [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                         c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    ("flash_tc5", "vl_flash_prefill_tc5"): [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                            c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    ("flash_attn", "vl_flash_decode"): [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                        c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int,
                                        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    ("flash_attn", "vl_flash_decode_fused"): [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                              c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int,
                                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_float, c_void_p, c_int, c_void_p, c_void_p],
    ("flash_decode_tma", "vl_flash_decode_tma"): [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                  c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int,
                                                  c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    ("activation", "vl_silu_mul"): [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    ("gemm_f32", "vl_gemm_f32_nt"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    ("gemm_bf16", "vl_gemm_bf16_small_m"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                            c_void_p, c_int, c_void_p],
    ("gemm_bf16", "vl_gemm_bf16_small_m_fused"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                  c_void_p, c_int, c_void_p, c_int, c_float, c_int, c_void_p, c_int,
                                                  c_void_p, c_void_p, c_void_p, c_void_p],
    ("gemm_tc5", "vl_gemm_bf16_tc5"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                       c_void_p, c_int, c_void_p],
    ("gemm_tc5_pair", "vl_gemm_bf16_tc5_pair"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                 c_void_p, c_int, c_void_p],
    ("memprobe", "vl_read_only"): [c_void_p, c_longlong, c_void_p, c_void_p],
    ("sampling", "vl_apply_penalties"): [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_void_p, c_void_p],
    ("sampling", "vl_sample"): [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_void_p],
}
_functions = {}
launch_count = 0          # kernels of this library launched so far (graph replays add theirs)


_pdl = False              # whether launches carry the programmatic-dependent-launch attribute: off unless the
                          # engine turns it on for a step of few tokens (the paired tcgen05 product never has it)
_pdl_libs = {}


def set_pdl(on: bool):
    """Launch the kernels that follow with (or without) the attribute that lets a kernel start while
    the one before it in the stream drains.  Every library holds the switch for its own launches."""
    global _pdl
    on = bool(on)
    if on != _pdl:
        _pdl = on
        for setter in _pdl_libs.values():
            setter(int(on))


def _fn(lib: str, name: str, defines=None):
    key = (lib, name, build._variant(defines))
    f = _functions.get(key)
    if f is None:
        handle = build.load(lib, defines)
        if key[::2] not in _pdl_libs and hasattr(handle, "vl_set_pdl"):
            setter = handle.vl_set_pdl
            setter.argtypes, setter.restype = [c_int], None
            setter(int(_pdl))
            _pdl_libs[key[::2]] = setter
        f = getattr(handle, name)
        f.argtypes = _SIGNATURES[(lib, name)]
        f.restype = c_int
        _functions[key] = f
    return f


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _check(code: int, name: str):
    global launch_count
    if code == 0:
        launch_count += 1
        return
    if code < 0:
        raise KernelError(f"{name} refused its arguments: {_ERRORS.get(code, code)}")
    raise KernelError(f"{name}: CUDA error {code} at launch")


def _need(t, dtype, name, ndim=None):
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor; the engine has no CPU path")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} must have {ndim} dimensions, got {tuple(t.shape)}")


# ---------------------------------------------------------------- embed / norm
def embed(ids, table, out, err):
    """out[t, :] = table[ids[t], :] as float32.  ids int32 [T]; out float32 [T, H]."""
    _need(ids, torch.int32, "ids", 1); _need(table, None, "table", 2); _need(out, torch.float32, "out", 2)
    T, (V, H) = ids.shape[0], table.shape
    if out.shape != (T, H):
        raise KernelError(f"out must be [{T}, {H}], got {tuple(out.shape)}")
    _check(_fn("embed_norm", "vl_embed")(_ptr(ids), _ptr(table), dtype_code(table.dtype), _ptr(out), T, H, V,
                                         _ptr(err), _stream()), "vl_embed")
    return out


def add_rmsnorm(x, delta, weight, eps, out, rows=None):
    """x float32 [T, H] (+= delta when given and rows is None); out[r] = rmsnorm(x[row r] (+ delta)) * weight."""
    _need(x, torch.float32, "x", 2); _need(weight, torch.float32, "weight", 1); _need(out, None, "out", 2)
    H = x.shape[1]
    R = x.shape[0] if rows is None else rows.shape[0]
    if weight.shape[0] != H or out.shape != (R, H):
        raise KernelError(f"norm shapes disagree: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if delta is not None:
        _need(delta, out.dtype, "delta", 2)
        if delta.shape != x.shape:
            raise KernelError(f"delta {tuple(delta.shape)} must match x {tuple(x.shape)}")
    if rows is not None:
        _need(rows, torch.int32, "rows", 1)
    _check(_fn("embed_norm", "vl_add_rmsnorm")(_ptr(x), _ptr(delta), _ptr(rows), _ptr(weight), _ptr(out),
                                               dtype_code(out.dtype), R, H, float(eps), _stream()), "vl_add_rmsnorm")
    return out


def add_bias(y, bias):
    """y[r, c] += bias[c] in place; y float32 or bfloat16 [rows, cols], bias float32 [cols]."""
    _need(y, None, "y", 2); _need(bias, torch.float32, "bias", 1)
    if bias.shape[0] != y.shape[1]:
        raise KernelError(f"add_bias: bias has {bias.shape[0]} entries for rows of {y.shape[1]}")
    _check(_fn("embed_norm", "vl_add_bias")(_ptr(y), dtype_code(y.dtype), _ptr(bias), y.shape[0], y.shape[1], _stream()),
           "vl_add_bias")
    return y


def cast(src, out):
    _need(src, None, "src"); _need(out, None, "out")
    if src.numel() != out.numel():
        raise KernelError("cast: sizes differ")
    _check(_fn("embed_norm", "vl_cast")(_ptr(src), dtype_code(src.dtype), _ptr(out), dtype_code(out.dtype),
                                        src.numel(), _stream()), "vl_cast")
    return out


# ---------------------------------------------------------------- rope + cache
def qk_norm_rope_write(qkv, positions, slots, q_weight, k_weight, eps, inv_freq, rotary_dim,
                       k_cache, v_cache, num_heads, num_kv_heads, head_dim, err):
    """In place on the q part of qkv [T, (nq + 2 nkv) hd]; k and v go to the cache
    [pages, nkv, page_size, hd] at `slots` (int32 [T]; negative: no write)."""
    _need(qkv, None, "qkv", 2); _need(positions, torch.int32, "positions", 1)
    T = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim or positions.shape[0] != T:
        raise KernelError(f"qkv {tuple(qkv.shape)} does not match heads {num_heads}+2*{num_kv_heads} x {head_dim}")
    page_size, num_slots = 1, 0
    if slots is not None:
        _need(slots, torch.int32, "slots", 1)
        _need(k_cache, qkv.dtype, "k_cache", 4); _need(v_cache, qkv.dtype, "v_cache", 4)
        if k_cache.shape != v_cache.shape or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim:
            raise KernelError(f"cache {tuple(k_cache.shape)} does not match kv heads {num_kv_heads} x {head_dim}")
        page_size = k_cache.shape[2]
        num_slots = k_cache.shape[0] * page_size
    for w, n in ((q_weight, "q_weight"), (k_weight, "k_weight")):
        if w is not None:
            _need(w, torch.float32, n, 1)
            if w.shape[0] != head_dim:
                raise KernelError(f"{n} must have head_dim={head_dim} entries")
    if inv_freq is not None:
        _need(inv_freq, torch.float32, "inv_freq", 1)
        if inv_freq.shape[0] * 2 != rotary_dim:
            raise KernelError("inv_freq must have rotary_dim / 2 entries")
    _check(_fn("rope_cache", "vl_qk_norm_rope_write")(
        _ptr(qkv), dtype_code(qkv.dtype), _ptr(positions), _ptr(slots), _ptr(q_weight), _ptr(k_weight), float(eps),
        _ptr(inv_freq), int(rotary_dim if inv_freq is not None else 0), _ptr(k_cache) if slots is not None else None,
        _ptr(v_cache) if slots is not None else None, T, num_heads, num_kv_heads, head_dim, page_size, num_slots,
        qkv.shape[1], _ptr(err), _stream()), "vl_qk_norm_rope_write")
    return qkv


# ---------------------------------------------------------------- attention
def paged_attention(qkv, out, k_cache, v_cache, block_table, req_index, positions,
                    num_heads, num_kv_heads, head_dim, scale, window, err):
    """out [T, nq*hd] = attention of the q part of qkv over the pages of each token's request."""
    _need(qkv, None, "qkv", 2); _need(out, qkv.dtype, "out", 2)
    _need(k_cache, qkv.dtype, "k_cache", 4); _need(v_cache, qkv.dtype, "v_cache", 4)
    _need(block_table, torch.int32, "block_table", 2)
    _need(req_index, torch.int32, "req_index", 1); _need(positions, torch.int32, "positions", 1)
    T = qkv.shape[0]
    if out.shape != (T, num_heads * head_dim) or req_index.shape[0] != T or positions.shape[0] != T:
        raise KernelError("paged_attention: token counts or widths disagree")
    if qkv.shape[1] < num_heads * head_dim:
        raise KernelError("paged_attention: qkv rows are narrower than the query heads")
    if k_cache.shape != v_cache.shape or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim:
        raise KernelError(f"cache {tuple(k_cache.shape)} does not match kv heads {num_kv_heads} x {head_dim}")
    _check(_fn("attention", "vl_paged_attention")(
        _ptr(qkv), qkv.shape[1], _ptr(out), dtype_code(qkv.dtype), _ptr(k_cache), _ptr(v_cache),
        _ptr(block_table), block_table.shape[1], _ptr(req_index), _ptr(positions),
        T, num_heads, num_kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0],
        float(scale), int(window or 0), _ptr(err), _stream()), "vl_paged_attention")
    return out


DECODE_CHUNK = 256        # key positions per block of the split decode kernel


def decode_attention_scratch(num_tokens, num_heads, head_dim, max_context, chunk=DECODE_CHUNK):
    """(splits, floats of part_acc, floats of part_ml) that `decode_attention` needs."""
    S = max(1, -(-int(max_context) // chunk))
    return S, num_tokens * num_heads * S * head_dim, num_tokens * num_heads * S * 2


def decode_attention(qkv, out, k_cache, v_cache, block_table, req_index, positions, num_heads, num_kv_heads,
                     head_dim, scale, window, max_context, part_acc, part_ml, err, chunk=DECODE_CHUNK):
    """Same function as `paged_attention`, for steps of few tokens per request: the key range of
    a token is split over blocks of `chunk` positions and merged.  `max_context` bounds
    position + 1 of every token; part_acc / part_ml are float32 scratch (see
    `decode_attention_scratch`)."""
    _need(qkv, None, "qkv", 2); _need(out, qkv.dtype, "out", 2)
    _need(k_cache, qkv.dtype, "k_cache", 4); _need(v_cache, qkv.dtype, "v_cache", 4)
    _need(block_table, torch.int32, "block_table", 2)
    _need(req_index, torch.int32, "req_index", 1); _need(positions, torch.int32, "positions", 1)
    _need(part_acc, torch.float32, "part_acc"); _need(part_ml, torch.float32, "part_ml")
    T = qkv.shape[0]
    if out.shape != (T, num_heads * head_dim) or req_index.shape[0] != T or positions.shape[0] != T:
        raise KernelError("decode_attention: token counts or widths disagree")
    if k_cache.shape != v_cache.shape or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim:
        raise KernelError(f"cache {tuple(k_cache.shape)} does not match kv heads {num_kv_heads} x {head_dim}")
    S, need_acc, need_ml = decode_attention_scratch(T, num_heads, head_dim, max_context, chunk)
    if part_acc.numel() < need_acc or part_ml.numel() < need_ml:
        raise KernelError(f"decode_attention: scratch too small ({part_acc.numel()} < {need_acc})")
    _check(_fn("attention", "vl_decode_attention")(
        _ptr(qkv), qkv.shape[1], _ptr(out), dtype_code(qkv.dtype), _ptr(k_cache), _ptr(v_cache),
        _ptr(block_table), block_table.shape[1], _ptr(req_index), _ptr(positions),
        T, num_heads, num_kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0],
        float(scale), int(window or 0), chunk, S, _ptr(part_acc), _ptr(part_ml), _ptr(err), _stream()),
        "vl_decode_attention")
    global launch_count
    launch_count += 1           # two kernels: the split pass and the merge
    return out


_max_clusters = {}


def flash_decode_max_cluster(head_dim) -> int:
    """Most chunks of a token that `vl_flash_decode` merges as the blocks of one cluster: 16 where the device
    takes clusters beyond the portable 8, else 8."""
    v = _max_clusters.get(head_dim)
    if v is None:
        fn = build.load("flash_attn", {"FA_HD": head_dim}).vl_flash_decode_max_cluster
        fn.restype = c_int
        v = _max_clusters[head_dim] = int(fn())
    return v


def decode_chunk_for(num_tokens, num_kv_heads, max_context, target_blocks=256, head_dim=None) -> int:
    """Key positions per block of the split decode kernels: the largest of 256..1024 that still
    gives most of the 148 SMs two blocks (a block's start-up is paid once per chunk; measured at
    batch 8, context 4,096: 4.80 / 4.55 / 4.38 ms a step with chunks of 256 / 512 / 1,024)."""
    ctx = int(max_context)
    for chunk in (1024, 512):
        if num_tokens * num_kv_heads * -(-ctx // chunk) >= target_blocks:
            return chunk
    # Too few blocks either way.  What bounds so few blocks is a warp's own pace (2,200 cycles for its 16
    # keys of every 64), so the shortest chunks win whose blocks still merge as one cluster per token (8
    # blocks, 16 where the device takes it) and have an SM each: one request at 4,096 keys, 16 chunks of 256
    # against 8 of 512: 3.24 -> 3.08 ms a step; two requests (256 blocks, two to an SM): 3.26 -> 3.43, so not there
    if head_dim is not None and flash_supported(torch.bfloat16, head_dim):
        most = flash_decode_max_cluster(head_dim)
        for chunk in (128, 256, 512, 1024):
            chunks = -(-ctx // chunk)
            if chunks <= most and num_tokens * num_kv_heads * chunks <= 2 * sm_pairs():
                return chunk
    return 512 if -(-ctx // 512) <= 8 else 256


def flash_supported(dtype, head_dim) -> bool:
    """The tensor-core attention kernels take bfloat16 and head sizes in steps of 16 up to 256."""
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256


def _flash_checks(qkv, k_cache, v_cache, block_table, num_heads, num_kv_heads, head_dim):
    _need(qkv, torch.bfloat16, "qkv", 2)
    _need(k_cache, torch.bfloat16, "k_cache", 4); _need(v_cache, torch.bfloat16, "v_cache", 4)
    _need(block_table, torch.int32, "block_table", 2)
    if qkv.shape[1] < num_heads * head_dim or qkv.shape[1] % 8:
        raise KernelError("flash attention: qkv rows are too narrow or not 16-byte aligned")
    if k_cache.shape != v_cache.shape or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim:
        raise KernelError(f"cache {tuple(k_cache.shape)} does not match kv heads {num_kv_heads} x {head_dim}")


def flash_prefill(qkv, out, k_cache, v_cache, block_table, tiles, num_heads, num_kv_heads, head_dim, scale, window, err,
                  tile_rows=64):
    """Tensor-core (mma.sync) attention for prompt portions.  `tiles` int32 [n, 4]: (row of the block
    table, index of the tile's first token in the step, tokens (<= tile_rows), position of the first
    token); the tiles of a step cover every token that the kernel is to serve once."""
    _flash_checks(qkv, k_cache, v_cache, block_table, num_heads, num_kv_heads, head_dim)
    _need(out, torch.bfloat16, "out", 2); _need(tiles, torch.int32, "tiles", 2)
    if out.shape != (qkv.shape[0], num_heads * head_dim) or tiles.shape[1] != 4:
        raise KernelError("flash_prefill: shapes disagree")
    _check(_fn("flash_attn", "vl_flash_prefill", {"FA_HD": head_dim})(
        _ptr(qkv), qkv.shape[1], _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
        _ptr(tiles), tiles.shape[0], int(tile_rows), num_heads, num_kv_heads, head_dim, k_cache.shape[2],
        k_cache.shape[0], float(scale), int(window or 0), _ptr(err), _stream()), "vl_flash_prefill")
    return out


FLASH_TC5_TILE = 128


def flash_tc5_supported(dtype, head_dim, page_size) -> bool:
    """The tcgen05 attention kernel takes bfloat16, head sizes 64 and 128, and pages of a multiple of
    8 positions that divide 64 or are a multiple of it."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and page_size % 8 == 0
            and (64 % page_size == 0 if page_size < 64 else page_size % 64 == 0))


def flash_prefill_tc5(qkv, out, k_cache, v_cache, block_table, tiles, num_heads, num_kv_heads, head_dim, scale, window, err):
    """Attention for prompt portions on the tcgen05 tensor cores; `tiles` as for `flash_prefill`,
    up to 128 tokens each."""
    _flash_checks(qkv, k_cache, v_cache, block_table, num_heads, num_kv_heads, head_dim)
    _need(out, torch.bfloat16, "out", 2); _need(tiles, torch.int32, "tiles", 2)
    if out.shape != (qkv.shape[0], num_heads * head_dim) or tiles.shape[1] != 4:
        raise KernelError("flash_prefill_tc5: shapes disagree")
    if not flash_tc5_supported(qkv.dtype, head_dim, k_cache.shape[2]):
        raise KernelError(f"flash_prefill_tc5: head size {head_dim} / page size {k_cache.shape[2]} not taken")
    _check(_fn("flash_tc5", "vl_flash_prefill_tc5", {"FA_HD": head_dim})(
        _ptr(qkv), qkv.shape[1], _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
        _ptr(tiles), tiles.shape[0], num_heads, num_kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0],
        float(scale), int(window or 0), _ptr(err), _stream()), "vl_flash_prefill_tc5")
    return out


_merge_caps = {}


def _own_merge_cap(head_dim) -> int:
    """Most chunks per token that `vl_flash_decode` of this head size merges itself."""
    cap = _merge_caps.get(head_dim)
    if cap is None:
        cap = _merge_caps[head_dim] = int(build.load("flash_attn", {"FA_HD": head_dim}).vl_flash_decode_own_merge_cap())
    return cap


def flash_decode_arrivals(num_tokens, num_heads, num_kv_heads) -> int:
    """Counters (int32) that `flash_decode` needs in `arrivals` for this many tokens."""
    return num_tokens * num_kv_heads * -(-(num_heads // num_kv_heads) // 16)


STREAM_DECODE_MIN_KEYS = 8 * 49152      # tokens x KV heads x context bound from which the persistent TMA kernel is used


def flash_decode_streams(dtype, num_tokens, num_kv_heads, head_dim, page_size, max_context) -> bool:
    """Whether `flash_decode` left to itself serves such a step with the persistent TMA kernel (else a block per chunk).
    Measured (Qwen3-8B heads, pages of 64): it wins from 64-position pages on (TMA boxes of 8 KB, not 2 KB) when
    the step streams enough keys to keep every SM's block busy: 16 tokens x 4,096 keys 55.8 us against 60.0 for a
    block per chunk, 64 x 4,096: 170 against 188, 8 x 16,384: 96 against 108; at 8 x 4,096 and below the block per
    chunk, which merges in the same launch, is level or ahead."""
    return (flash_tc5_supported(dtype, head_dim, page_size) and page_size >= 64
            and num_tokens * num_kv_heads * int(max_context) >= STREAM_DECODE_MIN_KEYS)


def flash_decode(qkv, out, k_cache, v_cache, block_table, req_index, positions, num_heads, num_kv_heads,
                 head_dim, scale, window, max_context, part_acc, part_ml, err, chunk=DECODE_CHUNK, token_index=None,
                 stream_kernel=None, arrivals=None, fold=None):
    """Tensor-core version of `decode_attention` (bfloat16): every block takes a chunk of a token's
    keys; the chunks are merged by the block that finishes last (`arrivals`: int32 counters,
    `flash_decode_arrivals` of them, zero before the first call and left zero) or, without
    `arrivals`, by a second kernel.
    The split pass is the persistent TMA kernel where it takes the head size, pages hold at
    least 64 positions and the step reads STREAM_DECODE_MIN_KEYS keys or more (`stream_kernel`: None =
    that rule, True / False to force; it always merges with the second kernel), else a block per chunk.
    `token_index` (int32) restricts the launch to some tokens of the step (the others' rows of `out`
    are left alone); the scratch is then sized for that many tokens.
    `fold` = (q_weight, k_weight, eps, inv_freq, rotary_dim, slots) folds the step's `qk_norm_rope_write`
    into the block-per-chunk kernel (the TMA kernel does not take it): qkv then holds the rows as the
    projection left them, every token is the last of its request, and the token's key and value are
    written to the cache by this launch (slots None: not written).  The same bits as the two kernels in turn."""
    _flash_checks(qkv, k_cache, v_cache, block_table, num_heads, num_kv_heads, head_dim)
    _need(out, torch.bfloat16, "out", 2)
    _need(req_index, torch.int32, "req_index", 1); _need(positions, torch.int32, "positions", 1)
    _need(part_acc, torch.float32, "part_acc"); _need(part_ml, torch.float32, "part_ml")
    T = qkv.shape[0]
    if out.shape != (T, num_heads * head_dim) or req_index.shape[0] != T or positions.shape[0] != T:
        raise KernelError("flash_decode: token counts or widths disagree")
    if token_index is not None:
        _need(token_index, torch.int32, "token_index", 1)
        T = token_index.shape[0]
    S, need_acc, need_ml = decode_attention_scratch(T, num_heads, head_dim, max_context, chunk)
    if part_acc.numel() < need_acc or part_ml.numel() < need_ml:
        raise KernelError(f"flash_decode: scratch too small ({part_acc.numel()} < {need_acc})")
    if stream_kernel is None:
        stream_kernel = fold is None and flash_decode_streams(qkv.dtype, T, num_kv_heads, head_dim, k_cache.shape[2], max_context)
    if fold is not None and (stream_kernel or token_index is not None):
        raise KernelError("flash_decode: the folded norm and rotation go with the block-per-chunk kernel and whole steps")
    args = (_ptr(qkv), qkv.shape[1], _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
            _ptr(req_index), _ptr(positions), T, num_heads, num_kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0],
            float(scale), int(window or 0), chunk, S, _ptr(part_acc), _ptr(part_ml), _ptr(err), _ptr(token_index))
    if stream_kernel:
        _check(_fn("flash_decode_tma", "vl_flash_decode_tma", {"FA_HD": head_dim})(*args, _stream()), "vl_flash_decode_tma")
    else:
        if arrivals is not None and S > _own_merge_cap(head_dim):
            arrivals = None
        if arrivals is not None:
            _need(arrivals, torch.int32, "arrivals", 1)
            if arrivals.numel() < flash_decode_arrivals(T, num_heads, num_kv_heads):
                raise KernelError("flash_decode: too few arrival counters")
        if fold is None:
            _check(_fn("flash_attn", "vl_flash_decode", {"FA_HD": head_dim})(
                *args, _ptr(out) if arrivals is not None else None, _ptr(arrivals), _stream()), "vl_flash_decode")
        else:
            qw, kw, eps, inv_freq, rot, slots = fold
            for t, n in ((qw, "q_weight"), (kw, "k_weight"), (inv_freq, "inv_freq")):
                if t is not None:
                    _need(t, torch.float32, n, 1)
            if (qw is None) != (kw is None) or (qw is not None and (qw.shape[0] != head_dim or kw.shape[0] != head_dim)):
                raise KernelError("flash_decode: the head norm's weights do not match the head size")
            if inv_freq is not None and inv_freq.shape[0] * 2 != rot:
                raise KernelError("flash_decode: inv_freq does not match the rotary dimension")
            if slots is not None:
                _need(slots, torch.int32, "slots", 1)
                if slots.shape[0] < T:
                    raise KernelError("flash_decode: fewer slots than tokens")
            if qkv.shape[1] < (num_heads + 2 * num_kv_heads) * head_dim:
                raise KernelError("flash_decode: the rows do not hold q, k and v")
            _check(_fn("flash_attn", "vl_flash_decode_fused", {"FA_HD": head_dim})(
                *args, _ptr(out) if arrivals is not None else None, _ptr(arrivals),
                _ptr(qw), _ptr(kw), float(eps), _ptr(inv_freq), int(rot if inv_freq is not None else 0), _ptr(slots),
                _stream()), "vl_flash_decode_fused")
        if arrivals is not None:
            return out
    _check(_fn("attention", "vl_decode_attention_merge")(
        _ptr(part_acc), _ptr(part_ml), _ptr(positions), _ptr(out), dtype_code(out.dtype), T, num_heads, head_dim,
        chunk, S, int(window or 0), _ptr(token_index), _stream()), "vl_decode_attention_merge")
    return out


# ---------------------------------------------------------------- feed-forward
SWIGLU_GROUP = 8          # gate/up interleave that the matrix-product kernels' fused activation expects


def silu_mul(gate_up, out, group=0):
    """out[t, i] = silu(gate_i) * up_i of gate_up [T, 2I].  group = 0: gate columns, then up columns;
    group = g: blocks of g gate columns followed by their g up columns."""
    _need(gate_up, None, "gate_up", 2); _need(out, gate_up.dtype, "out", 2)
    T, I2 = gate_up.shape
    if I2 % 2 or out.shape != (T, I2 // 2):
        raise KernelError("silu_mul: out must be [T, I] for gate_up [T, 2I]")
    _check(_fn("activation", "vl_silu_mul")(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), T, I2 // 2, int(group),
                                            _stream()), "vl_silu_mul")
    return out


# ---------------------------------------------------------------- matrix products
def gemm_f32(a, w, out):
    """out[M, N] = a[M, K] @ w[N, K]^T in true float32 (FFMA, fixed order over K)."""
    _need(a, torch.float32, "a", 2); _need(w, torch.float32, "w", 2); _need(out, torch.float32, "out", 2)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_f32: shapes disagree a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _check(_fn("gemm_f32", "vl_gemm_f32_nt")(_ptr(a), _ptr(w), _ptr(out), M, N, K, K, K, N, _stream()), "vl_gemm_f32_nt")
    return out


SMALL_M = 16              # most rows of the weight-streaming product, which is also what its kernel takes; measured at
                          # Qwen3-8B sizes, context 4,096: batch 12 decodes in 5.00 ms against 5.18 ms with the library
                          # product from 9 rows on, batch 16 in 5.42 against 5.60 (the norms and SwiGLU run inside it)


def gemm_bf16_small_m_ok(M, K) -> bool:
    return 0 < M <= SMALL_M and K % 8 == 0


def _gemm_shapes(a, w, out, swiglu):
    _need(a, torch.bfloat16, "a", 2); _need(w, torch.bfloat16, "w", 2); _need(out, None, "out", 2)
    M, K = a.shape
    N = w.shape[0]
    width = N // 2 if swiglu else N
    if w.shape[1] != K or out.shape != (M, width) or (swiglu and N % (2 * SWIGLU_GROUP)):
        raise KernelError(f"gemm_bf16: shapes disagree a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}"
                          + (" (fused SwiGLU)" if swiglu else ""))
    return M, N, K, width


NORM_PARTIALS = 1024      # vectors of 16 partial sums a product kernel may leave (at least its number of blocks)


def gemm_bf16_small_m(a, w, out, err=None, swiglu=False, scaled=None, sink=None):
    """out[M, N] = a[M, K] @ w[N, K]^T for M <= 16: bfloat16 operands, float32 accumulation,
    out bfloat16 or float32.  Bound by one read of w.  swiglu: w holds blocks of 8 gate rows and
    their 8 up rows, out is [M, N/2] = silu(gate) * up.
    scaled = (partial float32 [>= count, 16], count, eps, size): the rows of `a` are an RMS norm's
    output without its scales; row m of the result is scaled by 1/sqrt(sum_b partial[b, m]/size + eps).
    sink = (x float32 [M, N], next_weight float32 [N], partial_out float32 [NORM_PARTIALS, 16]): the
    result is added into x, out receives bf16(x * next_weight) and partial_out the sums of squares of x
    block by block; returns the number of vectors written instead of out."""
    M, N, K, width = _gemm_shapes(a, w, out, swiglu)
    ss_in, count, eps, size = (None, 0, 0.0, 0) if scaled is None else scaled
    x, next_w, ss_out = (None, None, None) if sink is None else sink
    if scaled is not None:
        _need(ss_in, torch.float32, "partial", 2)
        if ss_in.shape[1] != 16 or not 0 < count <= ss_in.shape[0] or size != K:
            raise KernelError("gemm_bf16_small_m: partial sums do not match the product")
    grid = ctypes.c_int(0)
    if sink is not None:
        _need(x, torch.float32, "x", 2); _need(next_w, torch.float32, "next_weight", 1)
        _need(ss_out, torch.float32, "partial_out", 2)
        if x.shape != (M, N) or next_w.shape[0] != N or ss_out.shape != (NORM_PARTIALS, 16) or swiglu:
            raise KernelError("gemm_bf16_small_m: the stream, the next weight or the partial sums do not match")
    _check(_fn("gemm_bf16", "vl_gemm_bf16_small_m_fused")(
        _ptr(a), _ptr(w), _ptr(out), dtype_code(out.dtype), M, N, K, K, K, width, _ptr(err), int(swiglu),
        _ptr(ss_in), int(count), float(eps), int(size), _ptr(x), N, _ptr(next_w), _ptr(ss_out),
        ctypes.addressof(grid) if sink is not None else None, _stream()), "vl_gemm_bf16_small_m")
    if sink is not None:
        if not 0 < grid.value <= NORM_PARTIALS:
            raise KernelError(f"gemm_bf16_small_m: {grid.value} blocks do not fit the partial sums")
        return grid.value
    return out


# From this many rows on the tcgen05 kernels are used: 1,024 where the activation is fused into the product
# (the library would need a kernel of its own for it: level at 1,024 rows, ahead beyond), 2,048 for a plain
# product (measured at 1,024 rows, q/k/v and down of Qwen3-8B: 58 and 82 us against the library's 41 and 73;
# at 2,048 rows 81 and 156 against 72 and 137; at 4,096 rows 158 and 358 against 165 and 314).
TC5_MIN_M = 1024
TC5_MIN_M_PLAIN = 2048


def gemm_bf16_tc5_ok(M, K, fused=False) -> bool:
    return M >= (TC5_MIN_M if fused else TC5_MIN_M_PLAIN) and K % 8 == 0


def gemm_bf16_tc5(a, w, out, err=None, swiglu=False):
    """out[M, N] = a[M, K] @ w[N, K]^T on the tcgen05 tensor cores (TMA tiles, accumulators in
    TMEM): bfloat16 operands, float32 accumulation, out bfloat16 or float32.  For many rows.
    swiglu: as in `gemm_bf16_small_m`."""
    M, N, K, width = _gemm_shapes(a, w, out, swiglu)
    _check(_fn("gemm_tc5", "vl_gemm_bf16_tc5")(_ptr(a), _ptr(w), _ptr(out), dtype_code(out.dtype), M, N, K,
                                               K, K, width, _ptr(err), int(swiglu), _stream()), "vl_gemm_bf16_tc5")
    return out


_sm_pairs = None


def sm_pairs() -> int:
    """Pairs of SMs of the current device (what a kernel of two-block clusters can keep busy)."""
    global _sm_pairs
    if _sm_pairs is None:
        _sm_pairs = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count // 2
    return _sm_pairs


def gemm_bf16_tc5_pair(a, w, out, err=None, swiglu=False):
    """As `gemm_bf16_tc5`, with two SMs on one 256 x 256 tile (tcgen05.mma.cta_group::2): each SM
    brings its rows of a and half of the tile's rows of w into shared memory."""
    M, N, K, width = _gemm_shapes(a, w, out, swiglu)
    _check(_fn("gemm_tc5_pair", "vl_gemm_bf16_tc5_pair")(_ptr(a), _ptr(w), _ptr(out), dtype_code(out.dtype), M, N, K,
                                                         K, K, width, _ptr(err), int(swiglu), _stream()),
           "vl_gemm_bf16_tc5_pair")
    return out


# ---------------------------------------------------------------- measurement
def read_only(buf, nbytes=None, sink=None):
    """Streams the first `nbytes` bytes of `buf` from memory once and does nothing with them: the time of
    this launch is what any kernel that must read as many bytes is measured against (bench.py --read-ceiling)."""
    _need(buf, None, "buf")
    total = buf.numel() * buf.element_size()
    nbytes = total if nbytes is None else int(nbytes)
    if not 0 < nbytes <= total or nbytes % 16:
        raise KernelError(f"read_only: {nbytes} bytes of a buffer of {total} (a multiple of 16 is wanted)")
    _check(_fn("memprobe", "vl_read_only")(_ptr(buf), nbytes, _ptr(sink), _stream()), "vl_read_only")


# ---------------------------------------------------------------- sampling
def apply_penalties(logits, seen_off=None, seen_ids=None, repeat=None, presence=None,
                    bias_off=None, bias_ids=None, bias_vals=None):
    _need(logits, torch.float32, "logits", 2)
    R, V = logits.shape
    _check(_fn("sampling", "vl_apply_penalties")(
        _ptr(logits), logits.stride(0), R, V, _ptr(seen_off), _ptr(seen_ids), _ptr(repeat), _ptr(presence),
        _ptr(bias_off), _ptr(bias_ids), _ptr(bias_vals), _stream()), "vl_apply_penalties")
    return logits


def sample(logits, temperature, top_k, top_p, uniform, out_token, out_logprob=None):
    _need(logits, torch.float32, "logits", 2); _need(out_token, torch.int32, "out_token", 1)
    R, V = logits.shape
    for t, dt, n in ((temperature, torch.float32, "temperature"), (top_k, torch.int32, "top_k"),
                     (top_p, torch.float32, "top_p"), (uniform, torch.float32, "uniform"),
                     (out_logprob, torch.float32, "out_logprob")):
        if t is not None:
            _need(t, dt, n, 1)
            if t.shape[0] < R:
                raise KernelError(f"{n} has fewer entries than rows")
    _check(_fn("sampling", "vl_sample")(
        _ptr(logits), logits.stride(0), R, V, _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(uniform),
        _ptr(out_token), _ptr(out_logprob), _stream()), "vl_sample")
    return out_token
