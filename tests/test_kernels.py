"""Each CUDA kernel alone against a plain float32 reference of the same operation,
at sizes other than the engine's tiny configurations: head sizes in steps of 16,
odd head counts and groups, widths and vocabularies that are no power of two."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from vllm_lite_b200.csrc import ops as o
    return o


def err_word():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(dtype):
    V, Hd = 1000 + 7, 200 + 8
    table = torch.randn(V, Hd, device=DEV).to(dtype)
    ids = torch.tensor([0, V - 1, 5, 5, 999], dtype=torch.int32, device=DEV)
    out = torch.empty(5, Hd, device=DEV)
    e = err_word()
    ops().embed(ids, table, out, e)
    assert torch.equal(out, table[ids.long()].float()) and int(e.item()) == 0
    bad = torch.tensor([3, V], dtype=torch.int32, device=DEV)
    out2 = torch.ones(2, Hd, device=DEV)
    ops().embed(bad, table, out2, e)
    assert int(e.item()) & 1 and torch.equal(out2[1], torch.zeros(Hd, device=DEV))   # flagged, not read


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [48, 1000, 5120 + 16])
def test_add_rmsnorm(dtype, H):
    T, eps = 7, 3e-5
    x = torch.randn(T, H, device=DEV) * 3
    delta = torch.randn(T, H, device=DEV).to(dtype)
    w = (1 + 0.1 * torch.randn(H, device=DEV))
    ref_x = x + delta.float()
    ref = P.rms_norm(ref_x.cpu(), w.cpu(), eps)
    x1, out = x.clone(), torch.empty(T, H, device=DEV, dtype=dtype)
    ops().add_rmsnorm(x1, delta, w, eps, out)
    assert torch.equal(x1, ref_x)                                    # the stream now holds the sum
    assert torch.allclose(out.float().cpu(), ref, **tol(dtype))
    out0 = torch.empty(T, H, device=DEV, dtype=dtype)                # no pending delta
    ops().add_rmsnorm(x.clone(), None, w, eps, out0)
    assert torch.allclose(out0.float().cpu(), P.rms_norm(x.cpu(), w.cpu(), eps), **tol(dtype))
    rows = torch.tensor([6, 2, 2], dtype=torch.int32, device=DEV)     # picked rows leave the stream alone
    x2, outr = x.clone(), torch.empty(3, H, device=DEV, dtype=dtype)
    ops().add_rmsnorm(x2, delta, w, eps, outr, rows=rows)
    assert torch.equal(x2, x) and torch.allclose(outr.float().cpu(), ref[[6, 2, 2]], **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul_and_cast(dtype):
    T, I = 5, 333
    gu = (torch.randn(T, 2 * I, device=DEV) * 4).to(dtype)
    out = torch.empty(T, I, device=DEV, dtype=dtype)
    ops().silu_mul(gu, out)
    g, u = gu.float()[:, :I], gu.float()[:, I:]
    assert torch.allclose(out.float(), g / (1 + torch.exp(-g)) * u, **tol(dtype))
    I8 = 40                                                 # blocks of 8 gate columns and their 8 up columns
    gi = (torch.randn(T, 2 * I8, device=DEV) * 4).to(dtype)
    outi = torch.empty(T, I8, device=DEV, dtype=dtype)
    ops().silu_mul(gi, outi, group=8)
    blocks = gi.float().view(T, I8 // 8, 2, 8)
    gg, uu = blocks[:, :, 0].reshape(T, I8), blocks[:, :, 1].reshape(T, I8)
    assert torch.allclose(outi.float(), gg / (1 + torch.exp(-gg)) * uu, **tol(dtype))
    src = torch.randn(1000, device=DEV)
    b = torch.empty(1000, device=DEV, dtype=torch.bfloat16)
    ops().cast(src, b)
    assert torch.equal(b, src.to(torch.bfloat16))
    back = torch.empty(1000, device=DEV)
    ops().cast(b, back)
    assert torch.equal(back, b.float())


@pytest.mark.parametrize("M,N,K", [(1, 333, 96), (70, 130, 257), (200, 64, 1000), (3, 5, 7)])
def test_gemm_f32_is_true_float32_and_batch_invariant(M, N, K):
    a, w = torch.randn(M, K, device=DEV), torch.randn(N, K, device=DEV)
    out = torch.empty(M, N, device=DEV)
    ops().gemm_f32(a, w, out)
    ref = (a.double().cpu() @ w.double().cpu().T)
    assert float((out.cpu().double() - ref).abs().max()) <= 2e-6 * K ** 0.5 * float(ref.abs().max() + 1)
    # TF32 would err by about 1e-3 relative; this bound is three orders tighter
    one = torch.empty(1, N, device=DEV)
    ops().gemm_f32(a[M - 1:M].contiguous(), w, one)
    assert torch.equal(one[0], out[M - 1])                            # a row alone == the row in the batch


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(1, 333, 96), (8, 6144, 4096), (9, 50, 200), (13, 1000, 264), (16, 160, 4096),
                                   (5, 17, 8), (16, 4096, 12288), (7, 100, 520), (3, 40, 2056)])
def test_gemm_bf16_small_m(M, N, K, out_dtype):
    torch.manual_seed(M * N)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    out = torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype)
    ops().gemm_bf16_small_m(a, w, out)
    ref = a.double() @ w.double().T
    scale = float(ref.abs().max())
    if out_dtype == torch.float32:                        # exact products, float32 sums
        assert float((out.double() - ref).abs().max()) <= 1e-5 * scale * (K ** 0.5)
    else:
        assert float((out.double() - ref).abs().max()) <= 2 ** -8 * scale + 1e-6
    # a row's result does not depend on the other rows of the launch: bit for bit among launches of the
    # same class of row counts (1..8, 9..16; the classes differ in how K is cut into stages)
    m2 = 1 if M <= 8 else 9
    other = torch.randn(m2, K, device=DEV).to(torch.bfloat16)
    other[m2 - 1] = a[M - 1]
    again = torch.empty(m2, N, device=DEV, dtype=out_dtype)
    ops().gemm_bf16_small_m(other, w, again)
    assert torch.equal(again[m2 - 1], out[M - 1])


@pytest.mark.parametrize("kernel", ["gemm_bf16_tc5", "gemm_bf16_tc5_pair"])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 512), (2048, 6144, 4096), (300, 1000, 264), (1, 333, 96),
                                   (130, 128, 72), (17, 40, 8), (257, 4096, 12288)])
def test_gemm_bf16_tcgen05(kernel, M, N, K, out_dtype):
    """Tiles of 128 x 256 (or 128 x 128) on one SM, or of 256 x 256 on a pair of SMs, through TMA and
    TMEM; ragged M, N and K are zero-filled."""
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    out = torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype)
    e = err_word()
    getattr(ops(), kernel)(a, w, out, e)
    assert int(e.item()) == 0
    ref = a.double() @ w.double().T
    scale = float(ref.abs().max())
    if out_dtype == torch.float32:
        assert float((out.double() - ref).abs().max()) <= 1e-5 * scale * (K ** 0.5)
    else:
        assert float((out.double() - ref).abs().max()) <= 2 ** -8 * scale + 1e-6


@pytest.mark.parametrize("M,H,K,N2,swiglu", [(1, 96, 64, 80, False), (8, 4096, 4096, 6144, False), (5, 200, 520, 48, True),
                                               (13, 1000, 264, 64, True), (16, 4096, 12288, 24576, True)])
def test_gemm_small_m_with_fused_norms(M, H, K, N2, swiglu):
    """Two products with an RMS norm between them and no kernel for the norm: the first adds its
    result into the float32 stream and leaves the norm's input times the norm's weight and the
    sums of squares; the second scales its rows."""
    torch.manual_seed(M + H)
    eps = 1e-5
    x = torch.randn(M, H, device=DEV) * 3
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w1 = (torch.randn(H, K, device=DEV) * 0.05).to(torch.bfloat16)
    nw = 1 + 0.1 * torch.randn(H, device=DEV)
    w2 = (torch.randn(N2, H, device=DEV) * 0.05).to(torch.bfloat16)
    x_new = x.double() + a.double() @ w1.double().T
    h = x_new / torch.sqrt((x_new * x_new).mean(dim=1, keepdim=True) + eps) * nw.double()
    y = h @ w2.double().T
    if swiglu:                                   # rows of w2: blocks of 8 gate rows and their 8 up rows
        y = y.view(M, N2 // 16, 2, 8)
        y = (torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]).reshape(M, N2 // 2)
    stream = x.clone()
    rows = torch.empty(M, H, device=DEV, dtype=torch.bfloat16)
    partial = torch.full((ops().NORM_PARTIALS, 16), float("nan"), device=DEV)
    count = ops().gemm_bf16_small_m(a, w1, rows, err_word(), sink=(stream, nw, partial))
    assert 0 < count <= ops().NORM_PARTIALS
    assert float((stream.double() - x_new).abs().max()) <= 1e-5 * float(x_new.abs().max()) * K ** 0.5
    assert torch.allclose(rows.double(), x_new * nw.double(), atol=2 ** -7 * float(x_new.abs().max()), rtol=0)
    ss = partial[:count, :M].double().sum(dim=0)
    assert torch.allclose(ss, (x_new * x_new).sum(dim=1), rtol=1e-5)
    out = torch.empty(M, N2 // 2 if swiglu else N2, device=DEV, dtype=torch.bfloat16)
    ops().gemm_bf16_small_m(rows, w2, out, err_word(), swiglu=swiglu, scaled=(partial, count, eps, H))
    assert float((out.double() - y).abs().max()) <= 2e-2 * float(y.abs().max()) + 1e-3


def pair_width_cases():
    plain = [(256, 512, 64), (2048, 4096, 4096), (300, 1000, 264), (1, 333, 96), (130, 128, 72), (513, 1100, 520)]
    cases = [(M, N, K, False, dt) for M, N, K in plain for dt in (torch.bfloat16, torch.float32)]
    return cases + [(300, 1024, 200, True, torch.bfloat16), (2048, 3200, 1024, True, torch.bfloat16)]   # the activation writes bfloat16


@pytest.mark.parametrize("width", ["256", "512"])
@pytest.mark.parametrize("M,N,K,swiglu,out_dtype", pair_width_cases())
def test_gemm_bf16_pair_widths(M, N, K, swiglu, out_dtype, width, monkeypatch):
    """The paired product with tiles of 256 x 256 (two accumulators) and of 256 x 512 (one accumulator of all 512
    columns of tensor memory, two products per 16 columns of K): both widths forced in turn, ragged M, N and K,
    several tiles per pair of SMs, the activation in the epilogue."""
    monkeypatch.setenv("VLLM_LITE_B200_PAIR_WIDTH", width)
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    out = torch.full((M, N // 2 if swiglu else N), float("nan"), device=DEV, dtype=out_dtype)
    e = err_word()
    ops().gemm_bf16_tc5_pair(a, w, out, e, swiglu=swiglu)
    assert int(e.item()) == 0
    ref = a.double() @ w.double().T
    if swiglu:
        ref = ref.view(M, N // 16, 2, 8)
        ref = (torch.nn.functional.silu(ref[:, :, 0]) * ref[:, :, 1]).reshape(M, N // 2)
    scale = float(ref.abs().max())
    if out_dtype == torch.float32:
        assert float((out.double() - ref).abs().max()) <= 1e-5 * scale * (K ** 0.5)
    else:
        assert float((out.double() - ref).abs().max()) <= 2 ** -7 * scale + 1e-6


@pytest.mark.parametrize("kernel,M", [("small_m", 1), ("small_m", 8), ("small_m", 13), ("tc5", 128), ("tc5", 300), ("tc5", 2048),
                                      ("tc5_pair", 300), ("tc5_pair", 2048)])
@pytest.mark.parametrize("I,K", [(160, 96), (12288, 4096), (24, 64)])
def test_gemm_with_fused_swiglu(kernel, M, I, K):
    """W interleaves 8 gate rows with their 8 up rows; the kernel writes silu(gate) * up."""
    torch.manual_seed(M + I)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    gate = (torch.randn(I, K, device=DEV) * 0.05).to(torch.bfloat16)
    up = (torch.randn(I, K, device=DEV) * 0.05).to(torch.bfloat16)
    w = torch.stack([gate.view(I // 8, 8, K), up.view(I // 8, 8, K)], dim=1).reshape(2 * I, K).contiguous()
    out = torch.full((M, I), float("nan"), device=DEV, dtype=torch.bfloat16)
    e = err_word()
    fn = {"small_m": ops().gemm_bf16_small_m, "tc5": ops().gemm_bf16_tc5, "tc5_pair": ops().gemm_bf16_tc5_pair}[kernel]
    fn(a, w, out, e, swiglu=True)
    assert int(e.item()) == 0
    g, u = a.double() @ gate.double().T, a.double() @ up.double().T
    ref = g / (1 + torch.exp(-g)) * u
    assert float((out.double() - ref).abs().max()) <= 2 ** -7 * float(ref.abs().max()) + 1e-6


def plain_head_norm_rope(x, w, eps, pos, theta, rot):
    """x [T, heads, hd] -> norm over hd, then rotate the first `rot` features."""
    y = P.rms_norm(x, w, eps) if w is not None else x
    if rot:
        y = torch.cat([P.rope(y[..., :rot], pos, theta), y[..., rot:]], dim=-1)
    return y


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,rot,page", [(6, 3, 48, 48, 4), (5, 1, 80, 32, 16), (8, 8, 16, 16, 8), (4, 2, 256, 256, 32)])
def test_qk_norm_rope_write(dtype, nq, nkv, hd, rot, page):
    T, pages, theta, eps = 9, 6, 50000.0, 1e-5
    qkv = torch.randn(T, (nq + 2 * nkv) * hd, device=DEV).to(dtype)
    pos = torch.tensor([0, 1, 2, 40000, 7, 8, 9, 10, 300], dtype=torch.int32, device=DEV)
    slot_list = [5, page, 3, 2 * page + 1, -1, pages * page - 1, 0, 7, 2]
    slots = torch.tensor(slot_list, dtype=torch.int32, device=DEV)
    qw, kw = 1 + 0.1 * torch.randn(hd, device=DEV), 1 + 0.1 * torch.randn(hd, device=DEV)
    from vllm_lite_b200.parts.rope import inverse_frequencies
    inv = torch.from_numpy(inverse_frequencies(rot, theta)).to(DEV)
    assert np.array_equal(inverse_frequencies(rot, theta), P.rope_inv_freq(rot, theta).numpy())
    kc = torch.full((pages, nkv, page, hd), 77.0, device=DEV, dtype=dtype)
    vc = torch.full((pages, nkv, page, hd), 77.0, device=DEV, dtype=dtype)
    src = qkv.float().cpu()
    e = err_word()
    ops().qk_norm_rope_write(qkv, pos, slots, qw, kw, eps, inv, rot, kc, vc, nq, nkv, hd, e)
    assert int(e.item()) == 0
    q_ref = plain_head_norm_rope(src[:, :nq * hd].view(T, nq, hd), qw.cpu(), eps, pos.tolist(), theta, rot)
    k_ref = plain_head_norm_rope(src[:, nq * hd:(nq + nkv) * hd].view(T, nkv, hd), kw.cpu(), eps, pos.tolist(), theta, rot)
    v_ref = src[:, (nq + nkv) * hd:].view(T, nkv, hd)
    assert torch.allclose(qkv[:, :nq * hd].float().cpu().view(T, nq, hd), q_ref, **tol(dtype))
    touched = torch.zeros(pages, page, dtype=torch.bool)
    for t, s in enumerate(slot_list):
        if s < 0:
            continue
        p, o = divmod(s, page)
        touched[p, o] = True
        assert torch.allclose(kc[p, :, o].float().cpu(), k_ref[t], **tol(dtype)), t
        assert torch.equal(vc[p, :, o].float().cpu(), v_ref[t]), t
    untouched = ~touched
    assert bool((kc.float().cpu().permute(0, 2, 1, 3)[untouched] == 77.0).all())     # other slots keep their contents
    assert bool((vc.float().cpu().permute(0, 2, 1, 3)[untouched] == 77.0).all())
    # a slot outside the pool is flagged and skipped
    ops().qk_norm_rope_write(qkv, pos, torch.full((T,), pages * page, dtype=torch.int32, device=DEV),
                             qw, kw, eps, inv, rot, kc, vc, nq, nkv, hd, e)
    assert int(e.item()) & 2


@pytest.mark.parametrize("nq,nkv,hd", [(8, 2, 128), (3, 1, 64), (5, 5, 32), (2, 1, 256)])
def test_qk_norm_rope_write_many_tokens(nq, nkv, hd):
    """From 256 tokens on, bfloat16 steps with wholly rotated heads of a power-of-two size take the
    kernel with 16-byte accesses: against the plain functions and against the other kernel."""
    dtype = torch.bfloat16
    T, page, theta, eps = 300, 16, 1e6, 1e-6
    pages = T // page + 2
    torch.manual_seed(hd)
    qkv = torch.randn(T, (nq + 2 * nkv) * hd, device=DEV).to(dtype)
    pos = torch.arange(T, dtype=torch.int32, device=DEV) + 17
    perm = torch.randperm(pages * page)[:T]
    perm[5] = -1                                        # a token that writes no cache
    slots = perm.to(torch.int32).to(DEV)
    qw, kw = 1 + 0.1 * torch.randn(hd, device=DEV), 1 + 0.1 * torch.randn(hd, device=DEV)
    from vllm_lite_b200.parts.rope import inverse_frequencies
    inv = torch.from_numpy(inverse_frequencies(hd, theta)).to(DEV)
    src = qkv.float().cpu()
    outs = []
    for rows in (T, 100):                               # 300 rows: the wide kernel; 3 x 100 rows: the other one
        q2 = qkv.clone()
        kc = torch.full((pages, nkv, page, hd), 77.0, device=DEV, dtype=dtype)
        vc = torch.full((pages, nkv, page, hd), 77.0, device=DEV, dtype=dtype)
        e = err_word()
        for lo_ in range(0, T, rows):
            ops().qk_norm_rope_write(q2[lo_:lo_ + rows], pos[lo_:lo_ + rows], slots[lo_:lo_ + rows], qw, kw, eps, inv, hd,
                                     kc, vc, nq, nkv, hd, e)
        assert int(e.item()) == 0
        outs.append((q2[:, :nq * hd].float().cpu(), kc.float().cpu(), vc.float().cpu()))
    q_ref = plain_head_norm_rope(src[:, :nq * hd].view(T, nq, hd), qw.cpu(), eps, pos.tolist(), theta, hd)
    k_ref = plain_head_norm_rope(src[:, nq * hd:(nq + nkv) * hd].view(T, nkv, hd), kw.cpu(), eps, pos.tolist(), theta, hd)
    v_ref = src[:, (nq + nkv) * hd:].view(T, nkv, hd)
    for q_out, kc, vc in outs:
        assert torch.allclose(q_out.view(T, nq, hd), q_ref, **tol(dtype))
        for t in range(T):
            s_ = int(slots[t])
            if s_ < 0:
                continue
            assert torch.allclose(kc[s_ // page, :, s_ % page], k_ref[t], **tol(dtype)), t
            assert torch.equal(vc[s_ // page, :, s_ % page], v_ref[t]), t
        written = torch.zeros(pages * page, dtype=torch.bool)
        written[slots[slots >= 0].long().cpu()] = True
        assert bool((kc.permute(0, 2, 1, 3).reshape(pages * page, -1)[~written] == 77.0).all())
    assert torch.allclose(outs[0][0], outs[1][0], atol=2e-2, rtol=2e-2) and torch.equal(outs[0][2], outs[1][2])


def paged_reference(q, keys, values, pos, scale, window):
    """q [nq, hd] at position pos against keys/values [n, nkv, hd] (n > pos)."""
    nq, nkv = q.shape[0], keys.shape[1]
    lo = 0 if not window else max(0, pos - window + 1)
    out = torch.empty_like(q)
    for h in range(nq):
        kh = h // (nq // nkv)
        s = (keys[lo:pos + 1, kh] @ q[h]) * scale
        p = torch.softmax(s, dim=0)
        out[h] = p @ values[lo:pos + 1, kh]
    return out


def build_paged(seqs_kv, nkv, hd, page, dtype, shuffle_seed=0, order="shuffled"):
    """Scatter each sequence's keys/values into pages; returns caches and block table.  `order`: the pages
    a sequence gets are "shuffled", "in a row" (neighbours in the pool, as a fresh pool hands them out) or
    in "runs" (neighbours but for a swap every few pages)."""
    total_pages = sum(-(-k.shape[0] // page) for k, _ in seqs_kv) + 3
    if order == "shuffled":
        perm = np.random.default_rng(shuffle_seed).permutation(total_pages).tolist()
    else:
        perm = list(range(total_pages))
        if order == "runs":
            for i in range(5, total_pages - 1, 7):
                perm[i], perm[i + 1] = perm[i + 1], perm[i]
        perm.reverse()                            # pop() hands out the front first
    kc = torch.full((total_pages, nkv, page, hd), float("nan"), dtype=dtype)
    vc = torch.full((total_pages, nkv, page, hd), float("nan"), dtype=dtype)
    max_blocks = max(-(-k.shape[0] // page) for k, _ in seqs_kv)
    table = torch.full((len(seqs_kv), max_blocks), -1, dtype=torch.int32)
    for b, (k, v) in enumerate(seqs_kv):
        for blk in range(-(-k.shape[0] // page)):
            pg = perm.pop()
            table[b, blk] = pg
            n = min(page, k.shape[0] - blk * page)
            kc[pg, :, :n] = k[blk * page:blk * page + n].transpose(0, 1).to(dtype)
            vc[pg, :, :n] = v[blk * page:blk * page + n].transpose(0, 1).to(dtype)
    return kc.to(DEV), vc.to(DEV), table.to(DEV)


@pytest.mark.parametrize("kernel,dtype", [("paged", torch.float32), ("paged", torch.bfloat16), ("flash", torch.bfloat16),
                                          ("flash_split", torch.bfloat16)])
@pytest.mark.parametrize("nq,nkv,hd,page,window", [(6, 2, 48, 4, 0), (5, 5, 16, 16, 0), (8, 1, 128, 16, 0),
                                                   (3, 1, 80, 8, 37), (4, 2, 256, 32, 0)])
def test_paged_attention_ragged(kernel, dtype, nq, nkv, hd, page, window):
    """A batch of a prompt portion, a continuation and two single tokens, pages shuffled."""
    torch.manual_seed(nq * 100 + hd)
    lens = [45, 130, 1, 77]                      # keys present per request
    new = [45, 20, 1, 1]                         # query tokens of this step per request (the last `new` positions)
    seqs = [(torch.randn(n, nkv, hd), torch.randn(n, nkv, hd)) for n in lens]
    kc, vc, table = build_paged(seqs, nkv, hd, page, dtype)
    rows, req, pos = [], [], []
    for b, (n, c) in enumerate(zip(lens, new)):
        for p_ in range(n - c, n):
            req.append(b); pos.append(p_)
    T = len(req)
    q = torch.randn(T, nq, hd)
    qkv = torch.zeros(T, (nq + 2 * nkv) * hd)
    qkv[:, :nq * hd] = q.view(T, -1)
    qkv = qkv.to(DEV).to(dtype)
    out = torch.empty(T, nq * hd, device=DEV, dtype=dtype)
    e = err_word()
    scale = hd ** -0.5
    if kernel in ("flash", "flash_split"):      # tiles of up to 64 tokens per request, as the engine cuts them
        tiles, single, t0 = [], [], 0
        for b, (n, c) in enumerate(zip(lens, new)):
            if c == 1 and kernel == "flash_split":        # single tokens go to the decode kernel, by index
                single.append(t0)
            else:
                for lo_ in range(0, c, 64):
                    tiles.append([b, t0 + lo_, min(64, c - lo_), n - c + lo_])
            t0 += c
        ops().flash_prefill(qkv, out, kc, vc, table, torch.tensor(tiles, dtype=torch.int32, device=DEV),
                            nq, nkv, hd, scale, window, e)
        if single:
            ctx = max(lens[req[t]] for t in single)
            S, n_acc, n_ml = ops().decode_attention_scratch(len(single), nq, hd, ctx, 64)
            ops().flash_decode(qkv, out, kc, vc, table, torch.tensor(req, dtype=torch.int32, device=DEV),
                               torch.tensor(pos, dtype=torch.int32, device=DEV), nq, nkv, hd, scale, window, ctx,
                               torch.full((n_acc,), float("nan"), device=DEV), torch.full((n_ml,), float("nan"), device=DEV),
                               e, chunk=64, token_index=torch.tensor(single, dtype=torch.int32, device=DEV),
                               arrivals=torch.zeros(ops().flash_decode_arrivals(len(single), nq, nkv), dtype=torch.int32, device=DEV))
    else:
        ops().paged_attention(qkv, out, kc, vc, table, torch.tensor(req, dtype=torch.int32, device=DEV),
                              torch.tensor(pos, dtype=torch.int32, device=DEV), nq, nkv, hd, scale, window, e)
    assert int(e.item()) == 0
    qd = qkv[:, :nq * hd].float().cpu().view(T, nq, hd)
    for t in range(T):
        k, v = seqs[req[t]]
        ref = paged_reference(qd[t], k.to(dtype).float(), v.to(dtype).float(), pos[t], scale, window)
        assert torch.allclose(out[t].float().cpu().view(nq, hd), ref, **tol(dtype)), (t, req[t], pos[t])


@pytest.mark.parametrize("nq,nkv,hd,page,window", [(2, 1, 64, 16, 0), (6, 2, 64, 8, 37), (5, 5, 64, 64, 0),
                                                   (4, 2, 128, 16, 0), (8, 1, 128, 32, 150), (3, 3, 128, 128, 0),
                                                   (32, 8, 128, 16, 0)])
@pytest.mark.parametrize("order", ["shuffled", "in a row", "runs"])
def test_flash_tc5_prefill(nq, nkv, hd, page, window, order):
    """The tcgen05 kernel on a ragged batch: a whole prompt of several tiles, a continuation that
    starts inside a page, a short portion, a single token; pages shuffled; every cache slot that no
    query may read holds NaN, which would show in the output."""
    dtype = torch.bfloat16
    torch.manual_seed(nq * 100 + hd + page)
    lens = [300, 471, 130, 77]                    # keys present per request
    new = [300, 200, 3, 1]                        # query tokens of this step per request (the last `new` positions)
    seqs = [(torch.randn(n, nkv, hd), torch.randn(n, nkv, hd)) for n in lens]
    kc, vc, table = build_paged(seqs, nkv, hd, page, dtype, order=order)     # neighbouring pages come in one box
    req, pos, tiles, t0 = [], [], [], 0
    for b, (n, c) in enumerate(zip(lens, new)):
        for p_ in range(n - c, n):
            req.append(b); pos.append(p_)
        for lo_ in range(0, c, 128):
            tiles.append([b, t0 + lo_, min(128, c - lo_), n - c + lo_])
        t0 += c
    T = len(req)
    q = torch.randn(T, nq, hd)
    qkv = torch.zeros(T, (nq + 2 * nkv) * hd)
    qkv[:, :nq * hd] = q.view(T, -1)
    qkv = qkv.to(DEV).to(dtype)
    out = torch.full((T, nq * hd), 9.0, device=DEV, dtype=dtype)
    e = err_word()
    scale = hd ** -0.5
    ops().flash_prefill_tc5(qkv, out, kc, vc, table, torch.tensor(tiles, dtype=torch.int32, device=DEV),
                            nq, nkv, hd, scale, window, e)
    assert int(e.item()) == 0
    qd = qkv[:, :nq * hd].float().cpu().view(T, nq, hd)
    worst = 0.0
    for t in range(T):
        k, v = seqs[req[t]]
        ref = paged_reference(qd[t], k.to(dtype).float(), v.to(dtype).float(), pos[t], scale, window)
        got = out[t].float().cpu().view(nq, hd)
        worst = max(worst, float((got - ref).abs().max()))
        assert torch.allclose(got, ref, **tol(dtype)), (t, req[t], pos[t], worst)


def run_attention(kernel, qkv, out, kc, vc, table, req, pos, nq, nkv, hd, scale, window, e):
    if kernel == "paged":
        return ops().paged_attention(qkv, out, kc, vc, table, req, pos, nq, nkv, hd, scale, window, e)
    if kernel == "flash_prefill":          # every token a tile of its own
        tiles = torch.tensor([[int(req[i]), i, 1, int(pos[i])] for i in range(qkv.shape[0]) if int(pos[i]) >= 0],
                             dtype=torch.int32, device=DEV)
        return ops().flash_prefill(qkv, out, kc, vc, table, tiles, nq, nkv, hd, scale, window, e)
    ctx = int(pos.max()) + 1
    S, n_acc, n_ml = ops().decode_attention_scratch(qkv.shape[0], nq, hd, ctx)
    pa = torch.full((n_acc,), float("nan"), device=DEV)
    pm = torch.full((n_ml,), float("nan"), device=DEV)
    if kernel.startswith("flash_decode"):       # "flash_decode", "flash_decode64", "flash_decode1024": the chunk size;
        stream = kernel.endswith("tma")         # "...tma": the persistent TMA kernel, else a block per chunk;
        own = kernel.endswith("own")            # "...own": the chunks are merged by the kernel's last block
        kernel = kernel[:-3] if stream or own else kernel
        assert not stream or ops().flash_tc5_supported(qkv.dtype, hd, kc.shape[2]), "a case the TMA kernel does not take"
        chunk = int(kernel[len("flash_decode"):] or 256)
        S, n_acc, n_ml = ops().decode_attention_scratch(qkv.shape[0], nq, hd, ctx, chunk)
        pa = torch.full((n_acc,), float("nan"), device=DEV)
        pm = torch.full((n_ml,), float("nan"), device=DEV)
        arrivals = torch.zeros(ops().flash_decode_arrivals(qkv.shape[0], nq, nkv), dtype=torch.int32, device=DEV) if own else None
        if own:                                 # a launch before this one has left the counters as it must
            ops().flash_decode(qkv, torch.empty_like(out), kc, vc, table, req, pos, nq, nkv, hd, scale, window, ctx, pa, pm, e,
                               chunk=chunk, stream_kernel=False, arrivals=arrivals)
            assert int(arrivals.abs().sum()) == 0
            pa.fill_(float("nan")); pm.fill_(float("nan"))
        return ops().flash_decode(qkv, out, kc, vc, table, req, pos, nq, nkv, hd, scale, window, ctx, pa, pm, e, chunk=chunk,
                                  stream_kernel=stream, arrivals=arrivals)
    return ops().decode_attention(qkv, out, kc, vc, table, req, pos, nq, nkv, hd, scale, window, ctx, pa, pm, e)


def attention_cases():
    """(kernel, dtype): the tensor-core kernels exist in bfloat16 only."""
    return [("paged", torch.float32), ("paged", torch.bfloat16), ("decode", torch.float32), ("decode", torch.bfloat16),
            ("flash_decode", torch.bfloat16), ("flash_decode64", torch.bfloat16), ("flash_decode1024", torch.bfloat16),
            ("flash_decodeown", torch.bfloat16), ("flash_decode64own", torch.bfloat16), ("flash_decode1024own", torch.bfloat16),
            ("flash_decodetma", torch.bfloat16), ("flash_decode64tma", torch.bfloat16), ("flash_decode1024tma", torch.bfloat16),
            ("flash_prefill", torch.bfloat16)]


def decode_split_cases():
    """Every decode kernel at every shape it takes: the persistent TMA kernel is listed only with the
    head and page sizes it is built for (head size 64 or 128, pages of 8, 16, 32 or a multiple of 64)."""
    from vllm_lite_b200.csrc.ops import flash_tc5_supported
    shapes = [(6, 2, 48, 4, 0), (5, 5, 16, 16, 0), (32, 8, 128, 16, 0), (3, 1, 80, 8, 300), (16, 2, 256, 32, 0),
              (7, 1, 64, 16, 0), (40, 2, 32, 16, 0), (20, 1, 128, 64, 500), (4, 2, 64, 8, 0), (6, 3, 128, 128, 0)]
    cases = []
    for kernel, dtype in attention_cases():
        if kernel == "paged":
            continue
        for nq, nkv, hd, page, window in shapes:
            if kernel.endswith("tma") and not flash_tc5_supported(dtype, hd, page):
                continue
            cases.append((kernel, dtype, nq, nkv, hd, page, window))
    return cases


@pytest.mark.parametrize("kernel,dtype,nq,nkv,hd,page,window", decode_split_cases())
def test_decode_attention_split(kernel, dtype, nq, nkv, hd, page, window):
    """Single tokens of requests of very different lengths (one token, a chunk's edge, several
    chunks), pages shuffled; a padded token at position -1 yields zeros."""
    torch.manual_seed(nq * 10 + hd)
    lens = [1, 255, 256, 257, 700, 1030]
    seqs = [(torch.randn(n, nkv, hd), torch.randn(n, nkv, hd)) for n in lens]
    # pages shuffled, and in a row as a fresh pool hands them out
    for order in ("shuffled", "in a row"):
        _decode_attention_split(kernel, dtype, nq, nkv, hd, page, window, lens, seqs, order)


def _decode_attention_split(kernel, dtype, nq, nkv, hd, page, window, lens, seqs, order):
    kc, vc, table = build_paged(seqs, nkv, hd, page, dtype, order=order)
    T = len(lens) + 1
    req = torch.tensor(list(range(len(lens))) + [0], dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lens] + [-1], dtype=torch.int32, device=DEV)
    qkv = torch.zeros(T, (nq + 2 * nkv) * hd)
    qkv[:, :nq * hd] = torch.randn(T, nq * hd)
    qkv = qkv.to(DEV).to(dtype)
    out = torch.full((T, nq * hd), 5.0, device=DEV, dtype=dtype)
    e = err_word()
    scale = hd ** -0.5
    run_attention(kernel, qkv, out, kc, vc, table, req, pos, nq, nkv, hd, scale, window, e)
    assert int(e.item()) == 0
    qd = qkv[:, :nq * hd].float().cpu().view(T, nq, hd)
    for t, n in enumerate(lens):
        k, v = seqs[t]
        ref = paged_reference(qd[t], k.to(dtype).float(), v.to(dtype).float(), n - 1, scale, window)
        assert torch.allclose(out[t].float().cpu().view(nq, hd), ref, **tol(dtype)), (t, n, order)
    if kernel != "flash_prefill":
        assert bool((out[T - 1] == 0).all())


@pytest.mark.parametrize("nq,nkv,hd,page", [(8, 2, 128, 64), (6, 3, 64, 16), (4, 1, 32, 8)])
def test_decode_attention_merges_up_to_16_chunks_in_a_cluster(nq, nkv, hd, page):
    """Few tokens with 9 to 16 chunks each: the chunks of a token are the blocks of one cluster (beyond the
    portable 8 where the device takes it, else the last block to arrive merges); requests of other lengths
    beside them leave some blocks of a cluster without keys."""
    most = ops().flash_decode_max_cluster(hd)
    assert most in (8, 16)
    torch.manual_seed(nq + hd)
    lens = [1000, 577, 3]
    seqs = [(torch.randn(n, nkv, hd), torch.randn(n, nkv, hd)) for n in lens]
    _decode_attention_split("flash_decode64own", torch.bfloat16, nq, nkv, hd, page, 0, lens, seqs, "shuffled")
    _decode_attention_split("flash_decode64own", torch.bfloat16, nq, nkv, hd, page, 400, lens, seqs, "in a row")


@pytest.mark.parametrize("nq,nkv,hd,page,rot,norm,chunk,window,write", [
    (32, 8, 128, 64, 128, True, 1024, 0, True), (8, 2, 128, 16, 128, True, 256, 0, True), (6, 3, 64, 16, 32, True, 64, 0, True),
    (4, 1, 32, 8, 32, False, 64, 300, True), (40, 2, 32, 16, 0, True, 256, 0, True), (7, 1, 64, 16, 64, True, 512, 0, False),
    (16, 2, 256, 32, 256, True, 256, 0, True), (5, 5, 16, 16, 16, True, 64, 0, True)])
def test_decode_attention_with_the_norm_and_rotation_folded_in(nq, nkv, hd, page, rot, norm, chunk, window, write):
    """A decode step two ways: the kernel that norms and rotates the heads and writes the cache, then the decode
    attention; and the decode attention doing all of it on the way.  The same bits: the output rows, and the
    key and value that the step leaves in the cache (requests of one token, of a page's last and first row,
    of a chunk's edges, a padded place; groups of more than 8 and more than 16 heads; a call that writes no cache)."""
    torch.manual_seed(nq * hd + page)
    lens = [1, page, page + 1, 255, 256, 257, 700, 1030]
    seqs = [(torch.randn(n, nkv, hd), torch.randn(n, nkv, hd)) for n in lens]
    kc, vc, table = build_paged(seqs, nkv, hd, page, torch.bfloat16)
    T = len(lens) + 1
    req = torch.tensor(list(range(len(lens))) + [0], dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lens] + [-1], dtype=torch.int32, device=DEV)
    slots = torch.tensor([int(table[b, (n - 1) // page]) * page + (n - 1) % page for b, n in enumerate(lens)] + [-1],
                         dtype=torch.int32, device=DEV)
    raw = (torch.randn(T, (nq + 2 * nkv) * hd) * 1.5).to(DEV).to(torch.bfloat16)
    qw = (1 + 0.1 * torch.randn(hd)).to(DEV) if norm else None
    kw = (1 + 0.1 * torch.randn(hd)).to(DEV) if norm else None
    inv_freq = (10000.0 ** (-torch.arange(0, rot, 2).float() / rot)).to(DEV) if rot else None
    eps, scale, ctx = 1e-5, hd ** -0.5, max(lens)
    S, n_acc, n_ml = ops().decode_attention_scratch(T, nq, hd, ctx, chunk)
    results = []
    for fold in (False, True):
        k2, v2, qkv = kc.clone(), vc.clone(), raw.clone()
        out = torch.full((T, nq * hd), 5.0, device=DEV, dtype=torch.bfloat16)
        pa, pm = torch.full((n_acc,), float("nan"), device=DEV), torch.full((n_ml,), float("nan"), device=DEV)
        arrivals = torch.zeros(ops().flash_decode_arrivals(T, nq, nkv), dtype=torch.int32, device=DEV)
        e = err_word()
        the_slots = slots if write else None
        if not fold:
            ops().qk_norm_rope_write(qkv, pos, the_slots, qw, kw, eps, inv_freq, rot, k2, v2, nq, nkv, hd, e)
        ops().flash_decode(qkv, out, k2, v2, table, req, pos, nq, nkv, hd, scale, window, ctx, pa, pm, e, chunk=chunk,
                           stream_kernel=False, arrivals=arrivals,
                           fold=(qw, kw, eps, inv_freq, rot, the_slots) if fold else None)
        assert int(e.item()) == 0 and int(arrivals.abs().sum()) == 0
        results.append((out, k2, v2))
    (o0, k0, v0), (o1, k1, v1) = results
    same = lambda a, b: torch.equal(a.view(torch.int16), b.view(torch.int16))        # bit for bit, NaN fill included
    assert same(k0, k1) and same(v0, v1) and same(o0, o1)
    if not write:                               # the cache is as it was: the token's key is what another call left there
        assert same(k1, kc) and same(v1, vc)
    assert bool((o1[T - 1] == 0).all())


@pytest.mark.parametrize("kernel,dtype", attention_cases())
@pytest.mark.parametrize("far,window", [(3, 0), (640, 0), (15, 0), (16, 0), (63, 0), (64, 0), (255, 0), (256, 0),
                                        (700, 300), (699, 300)])
def test_attention_finds_one_far_key(kernel, dtype, far, window):
    """One key among a thousand is made to stand out by scaling it and the query; the
    output must be that key's value (or, when the window excludes it, must not be)."""
    nq, nkv, hd, page, n = 2, 1, 64, 16, 1000
    torch.manual_seed(far)
    k, v = torch.randn(n, nkv, hd) * 0.1, torch.randn(n, nkv, hd)
    direction = torch.nn.functional.normalize(torch.randn(hd), dim=0)
    k[far, 0] = direction * 8
    q = (direction * 40).expand(nq, hd).contiguous()
    kc, vc, table = build_paged([(k, v)], nkv, hd, page, dtype, shuffle_seed=far)
    qkv = torch.zeros(1, (nq + 2 * nkv) * hd)
    qkv[0, :nq * hd] = q.view(-1)
    qkv = qkv.to(DEV).to(dtype)
    out = torch.empty(1, nq * hd, device=DEV, dtype=dtype)
    e = err_word()
    run_attention(kernel, qkv, out, kc, vc, table, torch.zeros(1, dtype=torch.int32, device=DEV),
                  torch.tensor([n - 1], dtype=torch.int32, device=DEV), nq, nkv, hd, hd ** -0.5, window, e)
    got = out.float().cpu().view(nq, hd)
    target = v[far, 0].to(dtype).float()
    inside = (not window) or far >= n - window
    if inside:
        assert torch.allclose(got[0], target, atol=3e-2) and torch.allclose(got[1], target, atol=3e-2)
    else:
        assert float((got[0] - target).abs().max()) > 0.3


@pytest.mark.parametrize("V", [333, 5000, 151936])
def test_sampling_greedy_and_temperature(V):
    torch.manual_seed(V)
    R = 6
    logits = torch.randn(R, V, device=DEV) * 3
    logits[1, 7] = logits[1, 400 % V] = 50.0                         # a tie: the lowest index wins
    logits[2, 5] = float("nan")
    tok = torch.empty(R, dtype=torch.int32, device=DEV)
    ops().sample(logits, None, None, None, None, tok)
    host = logits.cpu().tolist()
    assert tok.cpu().tolist() == [P.argmax([(-math.inf if x != x else x) for x in row]) for row in host]
    assert tok[1].item() == 7
    temp = torch.tensor([0.8, 1.0, 0.0, 1.7, 0.3, 1.0], device=DEV)
    u = torch.tensor([0.0, 0.37, 0.5, 0.93, 0.61, 0.999999], device=DEV)
    lp = torch.empty(R, device=DEV)
    ops().sample(logits, temp, torch.zeros(R, dtype=torch.int32, device=DEV), torch.ones(R, device=DEV), u, tok, lp)
    for r in range(R):
        t = float(temp[r])
        got = int(tok[r])
        if t == 0:
            assert got == P.argmax([(-math.inf if x != x else x) for x in host[r]])
            continue
        c = np.cumsum(P.temperature_probs(host[r], t))
        lo = c[got - 1] if got > 0 else 0.0
        # u falls into the chosen token's interval of the CDF (up to fixed-point rounding)
        assert lo - 1e-5 <= float(u[r]) <= c[got] + 1e-5, (r, got, lo, c[got])
        assert abs(float(lp[r]) - math.log(P.temperature_probs(host[r], t)[got])) < 1e-3


def test_sampling_top_k_top_p_and_penalties():
    torch.manual_seed(3)
    V = 1000
    base = torch.randn(4, V, device=DEV) * 2
    host = base.cpu().tolist()
    tok = torch.empty(4, dtype=torch.int32, device=DEV)
    temp = torch.ones(4, device=DEV)
    # top-k: whatever u is, the draw lies among the k largest
    kept_k = [set(np.argsort(host[r])[-5:].tolist()) for r in range(4)]
    for uval in (0.0, 0.3, 0.77, 0.9999):
        ops().sample(base, temp, torch.full((4,), 5, dtype=torch.int32, device=DEV), torch.ones(4, device=DEV),
                     torch.full((4,), uval, device=DEV), tok)
        assert all(int(tok[r]) in kept_k[r] for r in range(4))
    # top-p: the draw lies in the plain implementation's nucleus, and every nucleus token can be reached
    for top_p in (0.1, 0.5, 0.9):
        keep = [set(P.top_p_keep(host[r], top_p)) for r in range(4)]
        seen = [set() for _ in range(4)]
        for uval in np.linspace(0, 0.99999, 97):
            ops().sample(base, temp, torch.zeros(4, dtype=torch.int32, device=DEV), torch.full((4,), top_p, device=DEV),
                         torch.full((4,), float(uval), device=DEV), tok)
            for r in range(4):
                assert int(tok[r]) in keep[r], (top_p, uval, r)
                seen[r].add(int(tok[r]))
        assert all(len(seen[r]) >= min(len(keep[r]), 3) for r in range(4))
    # penalties and bias, ragged lists
    logits = base.clone()
    seen_ids = [[1, 5, 9], [], [0], [2, 3]]
    off = torch.tensor([0, 3, 3, 4, 6], dtype=torch.int32, device=DEV)
    ids = torch.tensor([1, 5, 9, 0, 2, 3], dtype=torch.int32, device=DEV)
    rep = torch.tensor([1.5, 1.0, 2.0, 1.0], device=DEV)
    pres = torch.tensor([0.0, 0.0, 0.25, 1.0], device=DEV)
    boff = torch.tensor([0, 0, 2, 2, 2], dtype=torch.int32, device=DEV)
    bids = torch.tensor([7, V + 5], dtype=torch.int32, device=DEV)
    bvals = torch.tensor([4.0, 1.0], device=DEV)
    ops().apply_penalties(logits, off, ids, rep, pres, boff, bids, bvals)
    for r in range(4):
        ref = P.apply_presence_penalty(P.apply_repeat_penalty(host[r], seen_ids[r], float(rep[r])), seen_ids[r], float(pres[r]))
        if r == 1:
            ref = P.apply_logit_bias(ref, {7: 4.0, V + 5: 1.0})
        assert torch.allclose(logits[r].cpu(), torch.tensor(ref), atol=1e-6)
