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


def problem(seed, dtype, lens, nq=8, nkv=2, hd=64, page=16):
    """Single decode tokens of requests of the given lengths over shuffled pages."""
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
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    return dict(qkv=qkv.to(DEV), kc=kc.to(DEV), vc=vc.to(DEV), table=table.to(DEV), req=req.to(DEV), pos=pos.to(DEV),
                nq=nq, nkv=nkv, hd=hd, page=page, ctx=max(lens))


def run_existing(p):
    from vllm_lite_b200.csrc import ops
    T = p["qkv"].shape[0]
    out = torch.zeros(T, p["nq"] * p["hd"], device=DEV, dtype=p["qkv"].dtype)
    S, n_acc, n_ml = ops.decode_attention_scratch(T, p["nq"], p["hd"], p["ctx"])
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.decode_attention(p["qkv"], out, p["kc"], p["vc"], p["table"], p["req"], p["pos"], p["nq"], p["nkv"], p["hd"],
                         p["hd"] ** -0.5, 0, p["ctx"], torch.empty(n_acc, device=DEV), torch.empty(n_ml, device=DEV), err)
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
            T, p["nq"], p["nkv"], p["hd"], p["page"], p["kc"].shape[0], p["hd"] ** -0.5, 0, chunk, S,
            err.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return rc, out, int(err.item())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_calls_in_a_row_match_the_entry_point_with_caller_scratch(dtype):
    fn = entry_point()
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    first = problem(1, dtype, [700, 3, 257, 1024])
    second = problem(2, dtype, [64, 900])                 # other sizes: the scratch is laid out anew
    for p in (first, second):
        rc, got, err = run_no_alloc(fn, p)
        assert rc == 0 and err == 0
        want = run_existing(p)
        assert torch.allclose(got.float(), want.float(), **tol)
        assert float(got.float().abs().max()) > 0
    rc, again, _ = run_no_alloc(fn, first)                # and the first problem once more
    assert rc == 0 and torch.allclose(again.float(), run_existing(first).float(), **tol)


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
