"""The decode-attention entry point that carries its own scratch memory, called through its
exported C symbol as an embedding program would call it, against the entry point that takes
scratch buffers from the caller.  Two calls in a row share the built-in scratch; a problem that
does not fit is refused before anything is launched.  The file name makes pytest collect it last."""
import ctypes
from ctypes import c_float, c_int, c_void_p

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ERR_SCRATCH = -4
SCRATCH_FLOATS = 4 * 1024 * 1024


def entry_point():
    from vllm_lite_b200.csrc import build
    lib = ctypes.CDLL(str(build.library_path("attention")))
    fn = lib.vl_decode_attention_no_alloc
    fn.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p, c_void_p]
    fn.restype = c_int
    return fn


def problem(seed, dtype, lens, nq=8, nkv=2, hd=64, page=16, window=0, empty=()):
    """Single decode tokens of requests of the given lengths over shuffled pages.  `empty` lists
    places of the batch that hold no request (position -1: they read nothing, their rows become zero)."""
    g = torch.Generator().manual_seed(seed)
    blocks = [-(-n // page) for n in lens]
    pages = sum(blocks) + 2
    perm = np.random.default_rng(seed).permutation(pages).tolist()
    kc = torch.randn(pages, nkv, page, hd, generator=g).to(dtype)
    vc = torch.randn(pages, nkv, page, hd, generator=g).to(dtype)
    table = torch.full((len(lens), max(blocks)), -1, dtype=torch.int32)
    for b, nb in enumerate(blocks):
        for i in range(nb):
            table[b, i] = perm.pop()
    T = len(lens)
    qkv = torch.randn(T, (nq + 2 * nkv) * hd, generator=g).to(dtype)
    req = torch.arange(T, dtype=torch.int32)
    pos = torch.tensor([-1 if b in empty else n - 1 for b, n in enumerate(lens)], dtype=torch.int32)
    return dict(qkv=qkv.to(DEV), kc=kc.to(DEV), vc=vc.to(DEV), table=table.to(DEV), req=req.to(DEV), pos=pos.to(DEV),
                nq=nq, nkv=nkv, hd=hd, page=page, ctx=max(lens), window=window,
                host=dict(qkv=qkv, kc=kc, vc=vc, table=table, pos=pos))


def plain_attention(p):
    """The same attention written out on the CPU in float32, from the problem's host copies: keys and
    values are gathered page by page through the block table, one softmax per head.  It shares nothing
    with the kernels, so a wrong offset into the scratch shows here even where both entry points agree."""
    h = p["host"]
    nq, nkv, hd, page, window = p["nq"], p["nkv"], p["hd"], p["page"], p["window"]
    T = h["qkv"].shape[0]
    out = torch.zeros(T, nq * hd)
    for t in range(T):
        pos = int(h["pos"][t])
        if pos < 0:
            continue
        lo = max(0, pos - window + 1) if window else 0
        idx = torch.arange(lo, pos + 1)
        pg, off = h["table"][t][idx // page].long(), idx % page
        q = h["qkv"][t, :nq * hd].float().view(nq, hd)
        for head in range(nq):
            kh = head // (nq // nkv)
            k = h["kc"][pg, kh, off].float()
            v = h["vc"][pg, kh, off].float()
            w = torch.softmax((k @ q[head]) * hd ** -0.5, dim=0)
            out[t, head * hd:(head + 1) * hd] = w @ v
    return out


def run_existing(p):
    from vllm_lite_b200.csrc import ops
    T = p["qkv"].shape[0]
    out = torch.zeros(T, p["nq"] * p["hd"], device=DEV, dtype=p["qkv"].dtype)
    S, n_acc, n_ml = ops.decode_attention_scratch(T, p["nq"], p["hd"], p["ctx"])
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.decode_attention(p["qkv"], out, p["kc"], p["vc"], p["table"], p["req"], p["pos"], p["nq"], p["nkv"], p["hd"],
                         p["hd"] ** -0.5, p["window"], p["ctx"], torch.empty(n_acc, device=DEV), torch.empty(n_ml, device=DEV), err)
    assert int(err.item()) == 0
    return out


def run_no_alloc(fn, p, chunk=256):
    from vllm_lite_b200.csrc import ops
    T = p["qkv"].shape[0]
    out = torch.zeros(T, p["nq"] * p["hd"], device=DEV, dtype=p["qkv"].dtype)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    S = -(-p["ctx"] // chunk)
    rc = fn(p["qkv"].data_ptr(), p["qkv"].shape[1], out.data_ptr(), ops.dtype_code(out.dtype), p["kc"].data_ptr(),
            p["vc"].data_ptr(), p["table"].data_ptr(), p["table"].shape[1], p["req"].data_ptr(), p["pos"].data_ptr(),
            T, p["nq"], p["nkv"], p["hd"], p["page"], p["kc"].shape[0], p["hd"] ** -0.5, p["window"], chunk, S,
            err.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return rc, out, int(err.item())


def poison_scratch(fn, dtype):
    """Fills the built-in scratch with NaN through the entry point itself: a large problem whose values
    are all NaN leaves NaN partial results in every element that a smaller call may later own.  A call
    that read an element it had not written itself would then show NaN in its output."""
    p = problem(9, dtype, [1024] * 24, nq=16, nkv=2, hd=128)       # 24 * 16 * 4 * 130 floats = 800 KB of partials
    p["vc"].fill_(float("nan"))
    rc, out, _ = run_no_alloc(fn, p)
    assert rc == 0 and bool(torch.isnan(out.float()).all())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_calls_in_a_row_match_the_entry_point_with_caller_scratch(dtype):
    fn = entry_point()
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    first = problem(1, dtype, [700, 3, 257, 1024])
    second = problem(2, dtype, [64, 900])                 # other sizes: the scratch is laid out anew
    windowed = problem(4, dtype, [600, 31, 300, 5], window=100, empty=(2,))   # a window and an empty place
    for p in (first, second, windowed, first):            # ... and the first problem once more
        poison_scratch(fn, dtype)                         # what the call before left must not matter
        rc, got, err = run_no_alloc(fn, p)
        assert rc == 0 and err == 0
        # both entry points run the same kernels on the same values in the same order: equal bit for bit
        assert torch.equal(got, run_existing(p))
        # and right, by a plain implementation of its own
        assert torch.allclose(got.float().cpu(), plain_attention(p), **tol)
        assert float(got.float().abs().max()) > 0
    assert bool((got.float()[1] != 0).any())
    rc, got, err = run_no_alloc(fn, windowed)
    assert rc == 0 and err == 0 and bool((got[2] == 0).all())     # the empty place: zeros, nothing read


def test_a_problem_beyond_the_built_in_scratch_is_refused():
    fn = entry_point()
    p = problem(3, torch.bfloat16, [300, 40])
    T, nq, hd = 2, p["nq"], p["hd"]
    too_many_chunks = SCRATCH_FLOATS // (T * nq * (hd + 2)) + 1
    out = torch.full((T, nq * hd), 7.0, device=DEV, dtype=torch.bfloat16)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    from vllm_lite_b200.csrc import ops
    rc = fn(p["qkv"].data_ptr(), p["qkv"].shape[1], out.data_ptr(), ops.dtype_code(out.dtype), p["kc"].data_ptr(),
            p["vc"].data_ptr(), p["table"].data_ptr(), p["table"].shape[1], p["req"].data_ptr(), p["pos"].data_ptr(),
            T, nq, p["nkv"], hd, p["page"], p["kc"].shape[0], hd ** -0.5, 0, 256, too_many_chunks,
            err.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == ERR_SCRATCH
    assert bool((out == 7.0).all())                        # nothing ran
