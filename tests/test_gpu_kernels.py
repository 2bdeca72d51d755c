"""Each sm_100a kernel driven alone through the C launch layer (include/shv_seq_kernels.h) against the numpy oracle."""
import ctypes as C

import numpy as np
import pytest

from oracle import seq_oracle as O
from shield_sisa_b200 import binding, weights as W
from tests.helpers import dev, rel_err, stream_ptr, sync

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return binding.load_library(True)


def ok(rc):
    assert rc == 0, f"launcher returned cudaError {rc}"


def gemm_args(M, N, K, A, Wt, Cm, ldc, c_dtype=0, bias=None, act=0, R=None, ldr=0, r_div=1.0, swiglu=0):
    g = binding.GemmArgs()
    g.M, g.N, g.K = M, N, K
    g.A, g.lda, g.W, g.ldw = A.data_ptr(), K, Wt.data_ptr(), K
    g.C, g.ldc, g.c_dtype = Cm.data_ptr(), ldc, c_dtype
    g.bias = bias.data_ptr() if bias is not None else None
    g.act = act
    g.R = R.data_ptr() if R is not None else None
    g.ldr, g.r_div, g.swiglu = ldr, r_div, swiglu
    return g


def silu(x):
    return x / (1.0 + np.exp(-x))


# ---------------------------------------------------------------------------------------------- fp32 GEMM
@pytest.mark.parametrize("M,N,K", [(1, 576, 384), (3, 384, 384), (321, 2316, 384), (700, 384, 768), (130, 128, 960)])
def test_gemm_f32_plain(L, M, N, K):
    import torch
    rng = np.random.default_rng(M + N)
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    ldc = (N + 3) // 4 * 4 + 4
    A, Wt = dev(a), dev(w)
    Cm = torch.full((M, ldc), 7.0, device="cuda")
    ok(L.shvk_gemm_f32(gemm_args(M, N, K, A, Wt, Cm, ldc), stream_ptr()))
    sync()
    got = Cm.cpu().numpy()
    ref = a.astype(np.float64) @ w.astype(np.float64).T
    assert np.abs(got[:, :N] - ref).max() < 2e-5
    assert (got[:, N:] == 7.0).all()                       # columns beyond N are never written


def test_gemm_f32_epilogues(L):
    import torch
    rng = np.random.default_rng(5)
    M, K = 333, 384
    a = rng.standard_normal((M, K)).astype(np.float32)
    # bias + SiLU
    w = (rng.standard_normal((128, K)) / 20).astype(np.float32)
    b = rng.standard_normal(128).astype(np.float32)
    Cm = torch.zeros((M, 128), device="cuda")
    A, Wt, Bt = dev(a), dev(w), dev(b)
    ok(L.shvk_gemm_f32(gemm_args(M, 128, K, A, Wt, Cm, 128, bias=Bt, act=1), stream_ptr()))
    sync()
    assert np.abs(Cm.cpu().numpy() - silu(a.astype(np.float64) @ w.T + b)).max() < 2e-5
    # residual in place with divisor
    w = (rng.standard_normal((384, K)) / 20).astype(np.float32)
    r = rng.standard_normal((M, 384)).astype(np.float32)
    H, Wt = dev(r), dev(w)
    ok(L.shvk_gemm_f32(gemm_args(M, 384, K, A, Wt, H, 384, R=H, ldr=384, r_div=float(np.float32(np.sqrt(2.0)))),
                       stream_ptr()))
    sync()
    assert np.abs(H.cpu().numpy() - (r + (a.astype(np.float64) @ w.T) / np.sqrt(2.0))).max() < 2e-5
    # SwiGLU: interleaved (gate, up) rows -> silu(gate) * up
    w = (rng.standard_normal((1920, K)) / 20).astype(np.float32)
    Cm = torch.zeros((M, 960), device="cuda")
    Wt = dev(w)
    ok(L.shvk_gemm_f32(gemm_args(M, 1920, K, A, Wt, Cm, 960, swiglu=1), stream_ptr()))
    sync()
    full = a.astype(np.float64) @ w.T
    assert np.abs(Cm.cpu().numpy() - silu(full[:, 0::2]) * full[:, 1::2]).max() < 2e-5


def test_gemm_f32_rows_do_not_depend_on_the_batch(L):
    import torch
    rng = np.random.default_rng(9)
    a = rng.standard_normal((400, 768)).astype(np.float32)
    w = rng.standard_normal((384, 768)).astype(np.float32)
    Wt, A, A1 = dev(w), dev(a), dev(a[257:258])
    big = torch.zeros((400, 384), device="cuda")
    ok(L.shvk_gemm_f32(gemm_args(400, 384, 768, A, Wt, big, 384), stream_ptr()))
    one = torch.zeros((1, 384), device="cuda")
    ok(L.shvk_gemm_f32(gemm_args(1, 384, 768, A1, Wt, one, 384), stream_ptr()))
    sync()
    assert torch.equal(big[257], one[0])                   # bitwise


# ---------------------------------------------------------------------------------------------- tensor-core GEMM
def tc_plan(L, g, dtype_code):
    buf = (C.c_char * 1024)()
    addr = (C.addressof(buf) + 63) & ~63
    ok(L.shvk_gemm_tc_plan(g, dtype_code, addr))
    return buf, addr


def tc_status(L):
    st = C.c_int(-1)
    ok(L.shvk_gemm_tc_status(C.byref(st)))
    return st.value


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (321, 2316, 384), (1000, 384, 768), (642, 1068, 384), (257, 384, 960)])
def test_gemm_tc_plain(L, dtype, M, N, K):
    import torch
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float16
    rng = np.random.default_rng(N + K)
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    A, Wt = dev(a, tdt), dev(w, tdt)
    ldc = (N + 3) // 4 * 4 + 4
    Cm = torch.full((M, ldc), 7.0, device="cuda")
    g = gemm_args(M, N, K, A, Wt, Cm, ldc)
    keep, plan = tc_plan(L, g, binding.DTYPES[dtype])
    ok(L.shvk_gemm_tc(plan, stream_ptr()))
    sync()
    assert tc_status(L) == 0
    got = Cm.cpu().numpy()
    ref = A.float().cpu().numpy().astype(np.float64) @ Wt.float().cpu().numpy().astype(np.float64).T
    assert np.abs(got[:, :N] - ref).max() < 1e-4           # operands are exact in 16 bits; only fp32 accumulation differs
    # fewer than eight padding columns may be written along with the row (zeros), so that rows end on a whole sector
    assert ((got[:, N:] == 0.0) | (got[:, N:] == 7.0)).all()


def test_gemm_tc_epilogues_and_partial_rows(L):
    import torch
    rng = np.random.default_rng(21)
    M, K = 1500, 384
    a = rng.standard_normal((M, K)).astype(np.float32)
    A = dev(a, torch.bfloat16)
    a16 = A.float().cpu().numpy().astype(np.float64)
    # SwiGLU into 16-bit storage
    w = (rng.standard_normal((1920, K)) / 20).astype(np.float32)
    Wt = dev(w, torch.bfloat16)
    w16 = Wt.float().cpu().numpy().astype(np.float64)
    Cm = torch.zeros((M, 960), device="cuda", dtype=torch.bfloat16)
    g = gemm_args(M, 1920, K, A, Wt, Cm, 960, c_dtype=1, swiglu=1)
    keep, plan = tc_plan(L, g, 1)
    ok(L.shvk_gemm_tc_rows(plan, 777, stream_ptr()))       # only the first 777 rows
    sync()
    full = a16 @ w16.T
    ref = silu(full[:, 0::2]) * full[:, 1::2]
    got = Cm.float().cpu().numpy()
    assert rel_err(got[:777], ref[:777]) < 1e-2            # bf16 rounding of the output
    assert (got[777:] == 0).all()
    # residual in place / sqrt(2), fp32 output; bias
    w = (rng.standard_normal((384, K)) / 20).astype(np.float32)
    Wt = dev(w, torch.bfloat16)
    w16 = Wt.float().cpu().numpy().astype(np.float64)
    r = rng.standard_normal((M, 384)).astype(np.float32)
    H = dev(r)
    g = gemm_args(M, 384, K, A, Wt, H, 384, R=H, ldr=384, r_div=float(np.float32(np.sqrt(2.0))))
    keep2, plan2 = tc_plan(L, g, 1)
    ok(L.shvk_gemm_tc(plan2, stream_ptr()))
    sync()
    assert np.abs(H.cpu().numpy() - (r + (a16 @ w16.T) / np.sqrt(2.0))).max() < 1e-4
    b = rng.standard_normal(384).astype(np.float32)
    Cm = torch.zeros((M, 384), device="cuda")
    Bt = dev(b)
    g = gemm_args(M, 384, K, A, Wt, Cm, 384, bias=Bt)
    keep3, plan3 = tc_plan(L, g, 1)
    ok(L.shvk_gemm_tc(plan3, stream_ptr()))
    sync()
    assert np.abs(Cm.cpu().numpy() - (a16 @ w16.T + b)).max() < 1e-4
    assert tc_status(L) == 0


def test_gemm_tc_rows_do_not_depend_on_the_batch(L):
    import torch
    rng = np.random.default_rng(33)
    a = rng.standard_normal((900, 384)).astype(np.float32)
    w = rng.standard_normal((2316, 384)).astype(np.float32)
    A, Wt = dev(a, torch.float16), dev(w, torch.float16)
    big = torch.zeros((900, 2320), device="cuda")
    k1, p1 = tc_plan(L, gemm_args(900, 2316, 384, A, Wt, big, 2320), 2)
    ok(L.shvk_gemm_tc(p1, stream_ptr()))
    one_a = A[515:516].contiguous()
    one = torch.zeros((1, 2320), device="cuda")
    k2, p2 = tc_plan(L, gemm_args(1, 2316, 384, one_a, Wt, one, 2320), 2)
    ok(L.shvk_gemm_tc(p2, stream_ptr()))
    sync()
    assert torch.equal(big[515], one[0])


# ---------------------------------------------------------------------------------------------- fused feed-forward block
@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
def test_ffn_fused_equals_the_two_gemm_path(L, dtype):
    """One launch (hidden layer on the SM) against up + SwiGLU and down + residual as two tensor-core GEMMs: bitwise, on a
    row count that is not a multiple of the 128-row block, and row-independent."""
    import torch
    code = binding.DTYPES[dtype]
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float16
    rng = np.random.default_rng(91)
    M, K, F = 128 * 150 + 77, 384, 960                     # more row blocks than SMs: every CTA walks two
    xn = dev(rng.standard_normal((M, K)).astype(np.float32), tdt)
    wu = dev((rng.standard_normal((2 * F, K)) / 20).astype(np.float32), tdt)
    wd = dev((rng.standard_normal((K, F)) / 30).astype(np.float32), tdt)
    h0 = rng.standard_normal((M, K)).astype(np.float32)
    # two-kernel path
    H2 = dev(h0)
    hid = torch.zeros((M, F), device="cuda", dtype=tdt)
    k1, p1 = tc_plan(L, gemm_args(M, 2 * F, K, xn, wu, hid, F, c_dtype=code, swiglu=1), code)
    k2, p2 = tc_plan(L, gemm_args(M, K, F, hid, wd, H2, K, R=H2, ldr=K), code)
    ok(L.shvk_gemm_tc(p1, stream_ptr()))
    ok(L.shvk_gemm_tc(p2, stream_ptr()))
    # fused
    H1 = dev(h0)
    buf = (C.c_char * 1024)()
    plan = (C.addressof(buf) + 63) & ~63
    ok(L.shvk_ffn_fused_plan(xn.data_ptr(), M, wu.data_ptr(), wd.data_ptr(), H1.data_ptr(), code, plan))
    ok(L.shvk_ffn_fused(plan, M, stream_ptr()))
    sync()
    assert tc_status(L) == 0
    assert torch.equal(H1, H2)
    # against float64 on a sample of rows
    rows = np.array([0, 1, 127, 128, 5000, M - 78, M - 1])
    x64 = xn[rows].float().cpu().numpy().astype(np.float64)
    full = x64 @ wu.float().cpu().numpy().astype(np.float64).T
    hid64 = silu(full[:, 0::2]) * full[:, 1::2]
    ref = h0[rows] + hid64 @ wd.float().cpu().numpy().astype(np.float64).T
    assert rel_err(H1[rows].cpu().numpy(), ref) < (8e-3 if dtype == "bf16" else 1e-3)
    # fewer rows through the same plan: the rows computed are the same bits, the others untouched
    H3 = dev(h0)
    ok(L.shvk_ffn_fused_plan(xn.data_ptr(), M, wu.data_ptr(), wd.data_ptr(), H3.data_ptr(), code, plan))
    ok(L.shvk_ffn_fused(plan, 333, stream_ptr()))
    sync()
    assert torch.equal(H3[:333], H1[:333])
    assert torch.equal(H3[333:], dev(h0)[333:])


# ---------------------------------------------------------------------------------------------- exact tier on tensor cores
def split_operands(L, a, w):
    """Device [lo | hi] of a and [hi | lo | hi] of w through shvk_split_tf32, checked against the definition."""
    import torch
    M, K = a.shape
    N = w.shape[0]
    A, Wm = dev(a), dev(w)
    A2 = torch.zeros((M, 2 * K), device="cuda")
    W3 = torch.zeros((N, 3 * K), device="cuda")
    ok(L.shvk_split_tf32(A.data_ptr(), K, K, M, A2.data_ptr(), 2 * K, 0, stream_ptr()))
    ok(L.shvk_split_tf32(Wm.data_ptr(), K, K, N, W3.data_ptr(), 3 * K, 1, stream_ptr()))
    sync()
    a2 = A2.cpu().numpy()
    lo, hi = a2[:, :K], a2[:, K:]
    assert ((hi.view(np.uint32) & 0x1fff) == 0).all() and ((lo.view(np.uint32) & 0x1fff) == 0).all()   # TF32-representable
    assert np.abs(hi - a).max() <= np.abs(a).max() * 2.0 ** -11
    resid = np.abs(a.astype(np.float64) - hi.astype(np.float64) - lo.astype(np.float64))
    assert (resid <= np.abs(a) * 2.0 ** -21 + 1e-45).all()
    w3 = W3.cpu().numpy()
    np.testing.assert_array_equal(w3[:, :K], w3[:, 2 * K:])
    return A2, W3


@pytest.mark.parametrize("M,N,K", [(700, 2316, 384), (333, 384, 768), (257, 1068, 384)])
def test_gemm_tc_split_tf32_matches_float64(L, M, N, K):
    import torch
    rng = np.random.default_rng(N + K + 1)
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    A2, W3 = split_operands(L, a, w)
    ldc = (N + 3) // 4 * 4 + 4
    Cm = torch.full((M, ldc), 7.0, device="cuda")
    g = gemm_args(M, N, K, A2, W3, Cm, ldc)
    g.lda, g.ldw = 2 * K, 3 * K
    keep, plan = tc_plan(L, g, 0)
    ok(L.shvk_gemm_tc(plan, stream_ptr()))
    sync()
    assert tc_status(L) == 0
    got = Cm.cpu().numpy()[:, :N]
    ref = a.astype(np.float64) @ w.astype(np.float64).T
    err = np.abs(got - ref).max()
    # the SIMT fp32 chain it replaces, for scale
    chain = np.abs((a @ w.T).astype(np.float64) - ref).max()
    scale = np.abs(ref).max()
    print(f"split-TF32 GEMM {M}x{N}x{K}: max abs err {err:.2e} (fp32 matmul on the host: {chain:.2e}), max |ref| {scale:.2f}")
    assert err < 2e-6 * max(1.0, scale)                    # fp32-class: a few ulp of the largest output


def test_gemm_tc_split_tf32_epilogues_and_row_independence(L):
    import torch
    rng = np.random.default_rng(77)
    M, K = 900, 384
    a = rng.standard_normal((M, K)).astype(np.float32)
    # SwiGLU, fp32 output
    w = (rng.standard_normal((1920, K)) / 20).astype(np.float32)
    A2, W3 = split_operands(L, a, w)
    Cm = torch.zeros((M, 960), device="cuda")
    g = gemm_args(M, 1920, K, A2, W3, Cm, 960, c_dtype=0, swiglu=1)
    g.lda, g.ldw = 2 * K, 3 * K
    keep, plan = tc_plan(L, g, 0)
    ok(L.shvk_gemm_tc_rows(plan, 777, stream_ptr()))
    sync()
    full = a.astype(np.float64) @ w.astype(np.float64).T
    ref = silu(full[:, 0::2]) * full[:, 1::2]
    got = Cm.cpu().numpy()
    assert np.abs(got[:777] - ref[:777]).max() < 2e-6 * max(1.0, np.abs(ref).max())
    assert (got[777:] == 0).all()
    # one row alone equals the row inside the batch, bitwise
    one = torch.zeros((1, 960), device="cuda")
    one_a = A2[515:516].contiguous()
    g1 = gemm_args(1, 1920, K, one_a, W3, one, 960, c_dtype=0, swiglu=1)
    g1.lda, g1.ldw = 2 * K, 3 * K
    k1, p1 = tc_plan(L, g1, 0)
    ok(L.shvk_gemm_tc(p1, stream_ptr()))
    sync()
    assert torch.equal(Cm[515], one[0])
    # residual in place / sqrt(2) with K = 960 (the FFN down projection)
    K2 = 960
    a2 = rng.standard_normal((M, K2)).astype(np.float32)
    w2 = (rng.standard_normal((384, K2)) / 30).astype(np.float32)
    A22, W32 = split_operands(L, a2, w2)
    r = rng.standard_normal((M, 384)).astype(np.float32)
    H = dev(r)
    g = gemm_args(M, 384, K2, A22, W32, H, 384, R=H, ldr=384, r_div=float(np.float32(np.sqrt(2.0))))
    g.lda, g.ldw = 2 * K2, 3 * K2
    keep2, plan2 = tc_plan(L, g, 0)
    ok(L.shvk_gemm_tc(plan2, stream_ptr()))
    sync()
    ref = r.astype(np.float64) + (a2.astype(np.float64) @ w2.astype(np.float64).T) / float(np.float32(np.sqrt(2.0)))
    assert np.abs(H.cpu().numpy() - ref).max() < 2e-6 * max(1.0, np.abs(ref).max())
    assert tc_status(L) == 0


# ---------------------------------------------------------------------------------------------- row kernels
def test_assemble_norm_and_rmsnorm(L, weight_files):
    import torch
    _, w = weight_files("W3", 1)
    B = 3
    tok = W.synth_tokens(B, 4)
    T = dev(tok)
    ptrs = np.array([T.data_ptr() + i * 6144 * 4 for i in range(B * 20)], dtype=np.uint64)
    P = dev(ptrs.view(np.int64))
    pos = O.positions(w, np.dtype(np.float32))
    nw = (1.0 + 0.1 * np.random.default_rng(0).standard_normal(384)).astype(np.float32)
    h = torch.zeros((B * 321, 384), device="cuda")
    d_pos, d_ro, d_nw = dev(pos), dev(w["readout"].reshape(384)), dev(nw)
    for code, tdt, tol in ((0, torch.float32, 2e-6), (1, torch.bfloat16, 8e-3), (2, torch.float16, 1e-3)):
        xn = torch.zeros((B * 321, 384), device="cuda", dtype=tdt)
        ok(L.shvk_assemble_norm(P.data_ptr(), d_pos.data_ptr(), d_ro.data_ptr(), d_nw.data_ptr(), h.data_ptr(),
                                xn.data_ptr(), code, B, stream_ptr()))
        sync()
        href = np.empty((B, 321, 384), np.float32)
        href[:, :320] = tok.reshape(B, 320, 384) + pos
        href[:, 320] = w["readout"].reshape(384)
        np.testing.assert_array_equal(h.cpu().numpy().reshape(B, 321, 384), href)
        ref = O.rms_norm(href.astype(np.float64), nw.astype(np.float64)).reshape(B * 321, 384)
        assert rel_err(xn.float().cpu().numpy(), ref) < tol
    # exact tier: the same rows as the split operand [lo | hi], from both kernels
    xs = torch.zeros((B * 321, 768), device="cuda")
    ok(L.shvk_assemble_norm(P.data_ptr(), d_pos.data_ptr(), d_ro.data_ptr(), d_nw.data_ptr(), h.data_ptr(), xs.data_ptr(), 3, B,
                            stream_ptr()))
    x32 = torch.zeros((B * 321, 384), device="cuda")
    ok(L.shvk_rmsnorm(h.data_ptr(), 384, d_nw.data_ptr(), x32.data_ptr(), 0, 384, B * 321, stream_ptr()))
    xs2 = torch.zeros((B * 321, 768), device="cuda")
    ok(L.shvk_rmsnorm(h.data_ptr(), 384, d_nw.data_ptr(), xs2.data_ptr(), 3, 768, B * 321, stream_ptr()))
    sync()
    assert torch.equal(xs, xs2)
    sp, full = xs.cpu().numpy(), x32.cpu().numpy()
    assert ((sp.view(np.uint32) & 0x1fff) == 0).all()                          # both pieces are TF32 numbers
    resid = np.abs(full.astype(np.float64) - sp[:, :384].astype(np.float64) - sp[:, 384:].astype(np.float64))
    assert (resid <= np.abs(full) * 2.0 ** -21 + 1e-45).all()
    # strided rows: the readout row of every clip
    out = torch.zeros((B, 384), device="cuda")
    ok(L.shvk_rmsnorm(h.data_ptr() + 320 * 384 * 4, 321 * 384, d_nw.data_ptr(), out.data_ptr(), 0, 384, B, stream_ptr()))
    sync()
    ref = O.rms_norm(href[:, 320].astype(np.float64), nw.astype(np.float64))
    assert np.abs(out.cpu().numpy() - ref).max() < 2e-6


# ---------------------------------------------------------------------------------------------- fused GDN scan
def gdn_inputs(w, stage, B, seed):
    """xn (float64) and the fused projection P (float32 [B*321, 2320]) of one mixer."""
    rng = np.random.default_rng(seed)
    xn = rng.standard_normal((B, 321, 384))
    m = f"{stage}.mixer"
    P = np.zeros((B, 321, 2320), np.float64)
    P[..., 0:384] = xn @ w[f"{m}.q_proj.weight"].astype(np.float64).T
    P[..., 384:768] = xn @ w[f"{m}.k_proj.weight"].astype(np.float64).T
    P[..., 768:1536] = xn @ w[f"{m}.v_proj.weight"].astype(np.float64).T
    P[..., 1536:2304] = xn @ w[f"{m}.g_proj.weight"].astype(np.float64).T
    P[..., 2304:2310] = xn @ w[f"{m}.a_proj.weight"].astype(np.float64).T
    P[..., 2310:2316] = xn @ w[f"{m}.b_proj.weight"].astype(np.float64).T
    return xn, P.reshape(B * 321, 2320).astype(np.float32)


@pytest.mark.parametrize("recipe,stage,B", [("W3", "gdn_a", 2), ("W3", "gdn_b", 1), ("W1", "gdn_a", 3)])
def test_gdn_scan_matches_oracle(L, weight_files, recipe, stage, B):
    import torch
    _, w = weight_files(recipe, 1)
    xn, P = gdn_inputs(w, stage, B, 17)
    tr = {}
    O.gdn_mixer(w, f"{stage}.mixer", xn, tr, "t")
    m = f"{stage}.mixer"
    conv_w = np.concatenate([w[f"{m}.{n}_conv1d.weight"].reshape(-1, 4) for n in "qkv"]).astype(np.float32)
    conv_b = np.concatenate([w[f"{m}.{n}_conv1d.bias"] for n in "qkv"]).astype(np.float32)
    # the synthetic files carry o_norm gain 1: test a non-trivial gain by rescaling the oracle's output
    ow = (1.0 + 0.1 * np.random.default_rng(1).standard_normal(128)).astype(np.float32)
    ref = (tr["t.o_gated"] * ow.astype(np.float64)).reshape(B * 321, 768)
    assert np.all(w[f"{m}.o_norm.weight"] == 1.0)
    Pd, d_cw, d_cb, d_al, d_dt, d_ow = dev(P), dev(conv_w), dev(conv_b), dev(w[f"{m}.A_log"]), dev(w[f"{m}.dt_bias"]), dev(ow)
    # the per-token fp32 recurrence; 16-bit outputs only round the result
    for code, tdt, tol in ((0, torch.float32, None), (1, torch.bfloat16, 2e-2), (2, torch.float16, 2e-2)):
        on = torch.zeros((B * 321, 768), device="cuda", dtype=tdt)
        ok(L.shvk_gdn_scan(Pd.data_ptr(), d_cw.data_ptr(), d_cb.data_ptr(), d_al.data_ptr(), d_dt.data_ptr(),
                           d_ow.data_ptr(), on.data_ptr(), code, B, stream_ptr()))
        sync()
        got = on.float().cpu().numpy()
        if tol is None:
            assert np.abs(got - ref).max() < 1e-4 * max(1.0, np.abs(ref).max())
        else:
            err = rel_err(got, ref)
            rms = float(np.sqrt(((got - ref) ** 2).mean() / (ref ** 2).mean()))
            print(f"gdn_scan {recipe} {stage} dtype {code}: max-rel {err:.3e} rms-rel {rms:.3e}")
            assert err < tol and rms < tol


# ---------------------------------------------------------------------------------------------- fused in-projection + 16-bit scan
PT_BLOCK = 13696          # 12,416 bytes of operand tiles and gates + 1,280 bytes added by the chunk preparation


def bf16_round(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy().astype(np.float64)


def rounded_mixer_weights(w, stage):
    """Copy of the weight dict whose mixer projections are exactly representable in bf16 (so the oracle and the kernel
    multiply the same numbers)."""
    m = f"{stage}.mixer"
    out = dict(w)
    for n in ("q_proj", "k_proj", "v_proj", "g_proj", "a_proj", "b_proj"):
        out[f"{m}.{n}.weight"] = bf16_round(w[f"{m}.{n}.weight"]).astype(np.float32)
    return out


def run_inproj(L, w, stage, xn16, B, mode=1, prep=True):
    """xn16: [B,321,384] float64 holding values representable in the mode's type (1 bf16, 2 fp16).  Returns (PT device
    buffer, keep-alive list).  prep: also run the chunk preparation, which completes the blocks for the scan."""
    import torch
    m = f"{stage}.mixer"
    fused = np.concatenate([w[f"{m}.{n}_proj.weight"] for n in ("q", "k", "v", "g", "a", "b")]).astype(np.float32)   # [2316,384]
    rows = L.shvk_gdn_inproj_rows()
    order = np.full(rows, -2, np.int32)
    L.shvk_gdn_inproj_row_order(order.ctypes.data)
    assert sorted(order[order >= 0].tolist()) == list(range(2316))          # a permutation of the fused rows, rest zero
    perm = np.zeros((rows, 384), np.float32)
    perm[order >= 0] = fused[order[order >= 0]]
    conv_w = np.concatenate([w[f"{m}.{n}_conv1d.weight"].reshape(-1, 4) for n in "qkv"]).astype(np.float32)
    conv_b = np.concatenate([w[f"{m}.{n}_conv1d.bias"] for n in "qkv"]).astype(np.float32)
    tdt = torch.bfloat16 if mode == 1 else torch.float16
    X = dev(xn16.reshape(B * 321, 384).astype(np.float32), tdt)
    Wp = dev(perm, tdt)
    d = [X, Wp, dev(conv_w), dev(conv_b), dev(w[f"{m}.A_log"]), dev(w[f"{m}.dt_bias"])]
    nbytes = L.shvk_gdn_pt_bytes(B)
    assert nbytes == B * 6 * 21 * PT_BLOCK
    pt = torch.full((nbytes,), 0x7f, device="cuda", dtype=torch.uint8)      # poison: 0x7f7f is a large finite bf16
    buf = (C.c_char * 1024)()
    plan = (C.addressof(buf) + 63) & ~63
    ok(L.shvk_gdn_inproj_plan(X.data_ptr(), B * 321, Wp.data_ptr(), d[2].data_ptr(), d[3].data_ptr(), d[4].data_ptr(),
                              d[5].data_ptr(), pt.data_ptr(), mode, plan))
    ok(L.shvk_gdn_inproj(plan, B, stream_ptr()))
    if prep:
        ok(L.shvk_gdn_chunk_prep(pt.data_ptr(), mode, B, stream_ptr()))
    sync()
    return pt, (d, buf)


def unpack_pt(pt, B, mode=1):
    """PT buffer -> q, k [B,6,336,64] (the mode's 16-bit type), v, g [B,6,336,128] (fp16), dec, beta [B,6,336]."""
    import torch
    raw = pt.cpu().numpy().reshape(B, 6, 21, PT_BLOCK)

    def tile(off, rows, tdt):
        t = np.ascontiguousarray(raw[..., off:off + rows * 32]).view(np.int16).reshape(B, 6, 21, rows, 16)
        f = torch.from_numpy(t.copy()).view(tdt).float().numpy().astype(np.float64)
        swapped = ((np.arange(rows) >> 2) & 1) == 1                            # rows whose two token halves trade places
        f[..., swapped, :] = np.concatenate([f[..., swapped, 8:], f[..., swapped, :8]], axis=-1)
        return f.transpose(0, 1, 2, 4, 3).reshape(B, 6, 336, rows)

    def gate(off):
        return np.ascontiguousarray(raw[..., off:off + 64]).view(np.float32).reshape(B, 6, 336).astype(np.float64)

    qk = torch.bfloat16 if mode == 1 else torch.float16
    return tile(0, 64, qk), tile(2048, 64, qk), tile(4096, 128, torch.float16), tile(8192, 128, torch.float16), gate(12288), gate(12352)


def unpack_ext(pt, B, mode=1):
    """What the chunk preparation added: T2, M [B,6,21,16,16] (the mode's type), exp(c), exp(c_last - c), 1/|k|,
    0.125/|q| [B,6,21,16]."""
    import torch
    raw = pt.cpu().numpy().reshape(B, 6, 21, PT_BLOCK)
    tdt = torch.bfloat16 if mode == 1 else torch.float16

    def mat(off):
        t = np.ascontiguousarray(raw[..., off:off + 512]).view(np.int16).reshape(B, 6, 21, 16, 16)
        return torch.from_numpy(t.copy()).view(tdt).float().numpy().astype(np.float64)

    def vec(off):
        return np.ascontiguousarray(raw[..., off:off + 64]).view(np.float32).reshape(B, 6, 21, 16).astype(np.float64)

    return mat(12416), mat(12928), vec(13440), vec(13504), vec(13568), vec(13632)


@pytest.mark.parametrize("mode", [1, 2])
def test_chunk_prep_matches_numpy(L, weight_files, mode):
    """The per-chunk products the scan reads (oracle/shieldv_ref.py:121-163 in WY form): from the tiles the in-projection
    wrote, T2 = (I + L)^-1 diag(beta), the decay-masked Q K^T, the decays and the norms, against float64 numpy."""
    _, w0 = weight_files("W3", 1)
    w = rounded_mixer_weights(w0, "gdn_b")
    B = 3
    rng = np.random.default_rng(23)
    rnd = bf16_round if mode == 1 else (lambda a: np.asarray(a, np.float32).astype(np.float16).astype(np.float64))
    xn = rnd(rng.standard_normal((B, 321, 384)))
    pt0, keep0 = run_inproj(L, w, "gdn_b", xn, B, mode, prep=False)
    pt, keep = run_inproj(L, w, "gdn_b", xn, B, mode)
    r0, r1 = pt0.cpu().numpy().reshape(-1, PT_BLOCK), pt.cpu().numpy().reshape(-1, PT_BLOCK)
    assert np.array_equal(r0[:, :12416], r1[:, :12416])          # the preparation leaves the tiles alone
    assert (r0[:, 12416:] == 0x7f).all()                         # and the in-projection leaves the last 1,280 bytes alone
    q, k, v, g, dec, beta = unpack_pt(pt, B, mode)
    t2, mq, eg, dj, ik, iq = unpack_ext(pt, B, mode)
    q, k = q.reshape(B, 6, 21, 16, 64), k.reshape(B, 6, 21, 16, 64)
    dec, beta = dec.reshape(B, 6, 21, 16), beta.reshape(B, 6, 21, 16)
    c = np.cumsum(dec, axis=-1)
    ik_ref = 1.0 / np.sqrt((k * k).sum(-1) + 1e-6)
    iq_ref = 0.125 / np.sqrt((q * q).sum(-1) + 1e-6)
    assert np.allclose(ik, ik_ref, rtol=1e-5) and np.allclose(iq, iq_ref, rtol=1e-5)
    assert np.allclose(eg, np.exp(c), rtol=1e-5) and np.allclose(dj, np.exp(c[..., -1:] - c), rtol=1e-5)
    dmask = np.exp(np.minimum(c[..., :, None] - c[..., None, :], 0.0))
    kk = np.einsum("...ik,...jk->...ij", k, k) * ik_ref[..., :, None] * ik_ref[..., None, :]
    lo = np.tril(np.ones((16, 16)), -1)
    Lm = beta[..., :, None] * dmask * kk * lo
    t2_ref = np.linalg.inv(np.eye(16) + Lm) * beta[..., None, :]
    m_ref = dmask * np.einsum("...ik,...jk->...ij", q, k) * iq_ref[..., :, None] * np.tril(np.ones((16, 16)))
    tol = 6e-3 if mode == 1 else 1.5e-3                          # one rounding to the operand type
    for name, got, ref in (("T2", t2, t2_ref), ("M", mq, m_ref)):
        err = np.abs(got - ref).max() / max(np.abs(ref).max(), 1.0)
        print(f"chunk prep mode {mode} {name}: max abs err / max(1, |ref|max) {err:.3e}")
        assert err < tol



@pytest.mark.parametrize("recipe,stage,B,mode", [("W3", "gdn_a", 2, 1), ("W3", "gdn_b", 3, 2), ("W1", "gdn_a", 1, 1)])
def test_gdn_inproj_tiles_match_oracle(L, weight_files, recipe, stage, B, mode):
    """The fused in-projection against the oracle's conv / SiLU / gate intermediates, on operands that are exact in
    bf16: what is left is fp32 accumulation, the tanh-form SiLU and the bf16 rounding of the tiles."""
    _, w0 = weight_files(recipe, 1)
    w = rounded_mixer_weights(w0, stage)                                      # bf16 values are exact in fp16 too at this scale
    xn = bf16_round(np.random.default_rng(29).standard_normal((B, 321, 384)))
    tr = {}
    O.gdn_mixer(w, f"{stage}.mixer", xn, tr, "t")
    pt, keep = run_inproj(L, w, stage, xn, B, mode)
    q, k, v, g, dec, beta = unpack_pt(pt, B, mode)
    assert tc_status(L) == 0
    for name, got, ref in (("q", q, tr["t.q_conv"]), ("k", k, tr["t.k_conv"]), ("v", v, tr["t.v_conv"]),
                           ("gate", g, O.silu(tr["t.gate"]))):
        ref = ref.transpose(0, 2, 1, 3)                                       # [B,6,321,*]
        err = rel_err(got[:, :, :321], ref)
        print(f"inproj {recipe} {stage} mode {mode} {name}: max-rel {err:.3e}")
        assert err < 6e-3                                                     # bf16 rounding (2^-9) + the approximate SiLU
        assert (got[:, :, 321:] == 0).all()                                   # padding token slots are zeros
    assert np.abs(dec[:, :, :321] - tr["t.g"].transpose(0, 2, 1)).max() < 2e-5 * max(1.0, np.abs(tr["t.g"]).max())
    assert np.abs(beta[:, :, :321] - tr["t.beta"].transpose(0, 2, 1)).max() < 2e-6
    assert (dec[:, :, 321:] == 0).all() and (beta[:, :, 321:] == 0).all()


@pytest.mark.parametrize("recipe,stage,B", [("W3", "gdn_a", 2), ("W3", "gdn_b", 1), ("W1", "gdn_a", 3)])
def test_gdn_inproj_scan_matches_oracle(L, weight_files, recipe, stage, B):
    """In-projection + scan of the 16-bit modes against the oracle's gated delta-rule output."""
    import torch
    _, w0 = weight_files(recipe, 1)
    w = rounded_mixer_weights(w0, stage)
    xn = bf16_round(np.random.default_rng(17).standard_normal((B, 321, 384)))
    tr = {}
    O.gdn_mixer(w, f"{stage}.mixer", xn, tr, "t")
    ow = (1.0 + 0.1 * np.random.default_rng(1).standard_normal(128)).astype(np.float32)
    ref = (tr["t.o_gated"] * ow.astype(np.float64)).reshape(B * 321, 768)
    d_ow = dev(ow)
    for code, tdt in ((1, torch.bfloat16), (2, torch.float16)):
        pt, keep = run_inproj(L, w, stage, xn, B, code)                       # the tiles' operand type follows the mode
        on = torch.full((B * 321 + 8, 768), 9.0, device="cuda", dtype=tdt)
        ok(L.shvk_gdn_scan_t(pt.data_ptr(), d_ow.data_ptr(), on.data_ptr(), code, B, stream_ptr()))
        sync()
        st = C.c_int(-1)
        ok(L.shvk_gdn_scan_status(C.byref(st)))
        assert st.value == 0
        got = on.float().cpu().numpy()
        assert (got[B * 321:] == 9.0).all()                                   # nothing is written past the last clip
        err = rel_err(got[:B * 321], ref)
        rms = float(np.sqrt(((got[:B * 321] - ref) ** 2).mean() / (ref ** 2).mean()))
        print(f"inproj+scan {recipe} {stage} dtype {code}: max-rel {err:.3e} rms-rel {rms:.3e}")
        assert err < 2e-2 and rms < 2e-2


def test_gdn_inproj_scan_clips_are_independent(L, weight_files):
    """A clip's tiles and outputs are bitwise the same alone and inside a batch, whatever its neighbours hold
    (non-finite neighbours included: the padding token slots of a clip never carry the next clip's values)."""
    import torch
    _, w0 = weight_files("W3", 1)
    w = rounded_mixer_weights(w0, "gdn_a")
    xn = bf16_round(np.random.default_rng(41).standard_normal((3, 321, 384)))
    xn_bad = xn.copy()
    xn_bad[2] = np.inf                                                        # the clip after clip 1 is garbage
    ow = dev(np.ones(128, np.float32))
    outs = []
    for x, B, pick in ((xn_bad, 3, 1), (xn[1:2], 1, 0)):
        pt, keep = run_inproj(L, w, "gdn_a", x, B)
        on = torch.zeros((B * 321, 768), device="cuda", dtype=torch.bfloat16)
        ok(L.shvk_gdn_scan_t(pt.data_ptr(), ow.data_ptr(), on.data_ptr(), 1, B, stream_ptr()))
        sync()
        outs.append((pt.reshape(B, -1)[pick].clone(), on.reshape(B, 321, 768)[pick].clone()))
    assert torch.equal(outs[0][0], outs[1][0])
    assert torch.equal(outs[0][1], outs[1][1])
    assert torch.isfinite(outs[0][1].float()).all()


def test_starved_launches_give_up_and_the_status_clears(L, weight_files):
    """A bounded wait that runs out: the tensor-core GEMM, the scan, the fused in-projection and the fused feed-forward
    block are each launched once with their input withheld.
    Each must return by itself with its status word set and nothing else disturbed; after the words are cleared the
    same launches work normally."""
    import torch
    rng = np.random.default_rng(3)
    M, N, K = 1000, 384, 768
    a, wm = rng.standard_normal((M, K)).astype(np.float32), (rng.standard_normal((N, K)) / 30).astype(np.float32)
    A, Wt = dev(a, torch.bfloat16), dev(wm, torch.bfloat16)
    Cm = torch.zeros((M, N), device="cuda")
    keep, plan = tc_plan(L, gemm_args(M, N, K, A, Wt, Cm, N), 1)
    words = torch.zeros(8, dtype=torch.int32).pin_memory()

    def fetch():
        ok(L.shvk_status_fetch_async(words.data_ptr(), stream_ptr()))
        sync()
        return words[:3].tolist()

    assert fetch() == [0, 0, 0]
    ok(L.shvk_gemm_tc_rows_starved(plan, M, 1024, stream_ptr()))
    sync()                                                                    # returns: the waits are bounded
    assert tc_status(L) != 0 and fetch()[0] != 0
    ok(L.shvk_status_clear_async(stream_ptr()))
    assert fetch() == [0, 0, 0]
    ok(L.shvk_gemm_tc(plan, stream_ptr()))
    sync()
    assert tc_status(L) == 0
    ref = A.float().cpu().numpy().astype(np.float64) @ Wt.float().cpu().numpy().astype(np.float64).T
    assert np.abs(Cm.cpu().numpy() - ref).max() < 1e-4
    # the scan
    _, w0 = weight_files("W3", 1)
    w = rounded_mixer_weights(w0, "gdn_a")
    xn = bf16_round(rng.standard_normal((2, 321, 384)))
    pt, keep2 = run_inproj(L, w, "gdn_a", xn, 2)
    ow = dev(np.ones(128, np.float32))
    on = torch.full((2 * 321, 768), 5.0, device="cuda", dtype=torch.bfloat16)
    ok(L.shvk_gdn_scan_t_starved(pt.data_ptr(), ow.data_ptr(), on.data_ptr(), 1, 2, 1024, stream_ptr()))
    sync()
    assert fetch()[2] == 1 and (on == 5.0).all()                              # gave up before writing anything
    ok(L.shvk_status_clear_async(stream_ptr()))
    ok(L.shvk_gdn_scan_t(pt.data_ptr(), ow.data_ptr(), on.data_ptr(), 1, 2, stream_ptr()))
    sync()
    assert fetch() == [0, 0, 0] and torch.isfinite(on.float()).all() and not (on == 5.0).all()
    # the fused in-projection (its waits report through the tensor-core GEMM word)
    d, buf = keep2
    plan_in = (C.addressof(buf) + 63) & ~63
    ref_pt = pt.clone()
    ok(L.shvk_gdn_inproj_starved(plan_in, 2, 1024, stream_ptr()))
    sync()
    assert fetch()[0] != 0
    ok(L.shvk_status_clear_async(stream_ptr()))
    ok(L.shvk_gdn_inproj(plan_in, 2, stream_ptr()))
    sync()
    assert fetch() == [0, 0, 0] and torch.equal(pt, ref_pt)
    # the fused feed-forward block
    Mf = 700
    xf = dev(rng.standard_normal((Mf, 384)).astype(np.float32), torch.bfloat16)
    wu = dev((rng.standard_normal((1920, 384)) / 20).astype(np.float32), torch.bfloat16)
    wd = dev((rng.standard_normal((384, 960)) / 30).astype(np.float32), torch.bfloat16)
    h0 = rng.standard_normal((Mf, 384)).astype(np.float32)
    Hs, Hn = dev(h0), dev(h0)
    fbuf = (C.c_char * 1024)()
    fplan = (C.addressof(fbuf) + 63) & ~63
    ok(L.shvk_ffn_fused_plan(xf.data_ptr(), Mf, wu.data_ptr(), wd.data_ptr(), Hs.data_ptr(), 1, fplan))
    ok(L.shvk_ffn_fused_starved(fplan, Mf, 1024, stream_ptr()))
    sync()
    assert fetch()[0] != 0
    ok(L.shvk_status_clear_async(stream_ptr()))
    ok(L.shvk_ffn_fused_plan(xf.data_ptr(), Mf, wu.data_ptr(), wd.data_ptr(), Hn.data_ptr(), 1, fplan))
    ok(L.shvk_ffn_fused(fplan, Mf, stream_ptr()))
    sync()
    assert fetch() == [0, 0, 0]
    full = xf.float().cpu().numpy().astype(np.float64) @ wu.float().cpu().numpy().astype(np.float64).T
    ref_h = h0 + (silu(full[:, 0::2]) * full[:, 1::2]) @ wd.float().cpu().numpy().astype(np.float64).T
    assert rel_err(Hn.cpu().numpy(), ref_h) < 8e-3


# ---------------------------------------------------------------------------------------------- SISA attention + head
def test_sisa_attention_matches_oracle(L, weight_files):
    import torch
    _, w = weight_files("W3", 1)
    B = 3
    rng = np.random.default_rng(23)
    h = rng.standard_normal((B, 321, 384)) * 1.5
    tr = {}
    O.sisa_last_row(w, h, tr)
    a = "sisa.attn"
    xn = O.rms_norm(h, w["sisa.attn_norm.weight"].astype(np.float64))
    S = np.zeros((B, 321, 1072))
    S[..., 0:384] = xn @ w[f"{a}.W_K.weight"].astype(np.float64).T
    S[..., 384:768] = xn @ w[f"{a}.W_V.weight"].astype(np.float64).T
    S[..., 768:960] = xn @ w[f"{a}.W_B.weight"].astype(np.float64).T
    S[..., 960:1056] = xn @ w[f"{a}.theta_proj.weight"].astype(np.float64).T
    S[..., 1056:1062] = xn @ w[f"{a}.alpha_proj.weight"].astype(np.float64).T + w[f"{a}.alpha_proj.bias"]
    S[..., 1062:1068] = xn @ w[f"{a}.forget_proj.weight"].astype(np.float64).T + w[f"{a}.forget_proj.bias"]
    QC = np.concatenate([xn[:, 320] @ w[f"{a}.W_Q.weight"].astype(np.float64).T,
                         xn[:, 320] @ w[f"{a}.W_C.weight"].astype(np.float64).T], axis=1)
    Y = torch.zeros((B, 384), device="cuda")
    d_s, d_qc, d_lam = dev(S.reshape(B * 321, 1072).astype(np.float32)), dev(QC.astype(np.float32)), dev(w[f"{a}.lambda_raw"])
    ok(L.shvk_sisa_attn(d_s.data_ptr(), d_qc.data_ptr(), d_lam.data_ptr(), Y.data_ptr(), B, stream_ptr()))
    sync()
    assert np.abs(Y.cpu().numpy() - tr["sisa.attn_y_last"]).max() < 5e-5
    # the split row format of the 16-bit modes: K | V | B as fp16, theta | alpha | forget as fp32.  Exact for inputs
    # that are fp16 numbers: same result as the fp32 kernel on those inputs, bit for bit
    s32 = S.reshape(B * 321, 1072).astype(np.float32)
    kvb16 = s32[:, :960].astype(np.float16)
    s_rounded = s32.copy()
    s_rounded[:, :960] = kvb16.astype(np.float32)
    sg = np.zeros((B * 321, 112), np.float32)
    sg[:, :108] = s32[:, 960:1068]
    Y32, Y16 = torch.zeros((B, 384), device="cuda"), torch.zeros((B, 384), device="cuda")
    d_r, d_16, d_sg = dev(s_rounded), dev(kvb16), dev(sg)
    ok(L.shvk_sisa_attn(d_r.data_ptr(), d_qc.data_ptr(), d_lam.data_ptr(), Y32.data_ptr(), B, stream_ptr()))
    ok(L.shvk_sisa_attn_h16(d_16.data_ptr(), d_sg.data_ptr(), d_qc.data_ptr(), d_lam.data_ptr(), Y16.data_ptr(), B, stream_ptr()))
    sync()
    assert torch.equal(Y32, Y16)
    assert rel_err(Y16.cpu().numpy(), tr["sisa.attn_y_last"]) < 2e-3           # fp16 rounding of K, V, B only


def test_gemm_tc_split16_epilogue(L):
    """SISA projection shape: columns below 960 leave as fp16 rows, the rest as fp32 (+ bias) rows of pitch 112."""
    import torch
    rng = np.random.default_rng(5)
    M, N, K = 700, 1068, 384
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    bias = np.zeros(N, np.float32)
    bias[1056:] = rng.standard_normal(12).astype(np.float32)
    for code, tdt in ((1, torch.bfloat16), (2, torch.float16)):
        A, Wt, Bt = dev(a, tdt), dev(w, tdt), dev(bias)
        C16 = torch.full((M, 960), 7.0, device="cuda", dtype=torch.float16)
        Cg = torch.full((M, 112), 7.0, device="cuda")
        g = gemm_args(M, N, K, A, Wt, Cg, 112, bias=Bt)
        buf = (C.c_char * 1024)()
        plan = (C.addressof(buf) + 63) & ~63
        ok(L.shvk_gemm_tc_plan_split16(g, code, 960, C16.data_ptr(), 960, plan))
        ok(L.shvk_gemm_tc_rows(plan, 613, stream_ptr()))
        sync()
        assert tc_status(L) == 0
        ref = A.float().cpu().numpy().astype(np.float64) @ Wt.float().cpu().numpy().astype(np.float64).T + bias
        got16, gotg = C16.float().cpu().numpy(), Cg.cpu().numpy()
        assert np.abs(got16[:613] - ref[:613, :960]).max() < 4e-3          # fp16 rounding of O(1) values
        assert np.abs(gotg[:613, :108] - ref[:613, 960:]).max() < 1e-4
        assert (gotg[:613, 108:] == 0).all() or (gotg[:613, 108:] == 7.0).all()      # padding: zeros (whole sectors) or untouched
        assert (got16[613:] == 7.0).all() and (gotg[613:] == 7.0).all()
        # the fp32 part equals the plain epilogue's bits
        Cp = torch.zeros((M, 1072), device="cuda")
        k2, p2 = tc_plan(L, gemm_args(M, N, K, A, Wt, Cp, 1072, bias=Bt), code)
        ok(L.shvk_gemm_tc_rows(p2, 613, stream_ptr()))
        sync()
        assert torch.equal(Cp[:613, 960:1068], Cg[:613, :108])
        assert torch.equal(Cp[:613, :960].to(torch.float16), C16[:613])


def test_readout_row_kernels_match_oracle(L, weight_files):
    """The two fused readout-row kernels (norm + Q/C projection; W_O, FFN, final norm, head) against the oracle, on a
    batch that is not a multiple of the 16-clip tile, and bitwise independent of the batch."""
    import torch
    _, w = weight_files("W3", 1)
    B = 37
    rng = np.random.default_rng(3)
    f64 = lambda n: w[n].astype(np.float64)  # noqa: E731
    h = rng.standard_normal((B, 321, 384)) * 1.5
    y = rng.standard_normal((B, 384)) * 0.5
    a = "sisa.attn"
    # part 1
    xl = O.rms_norm(h[:, 320], f64("sisa.attn_norm.weight"))
    wqc = np.concatenate([f64(f"{a}.W_Q.weight"), f64(f"{a}.W_C.weight")])                       # [576, 384]
    H = dev(h.astype(np.float32))
    h_last = H.data_ptr() + 320 * 384 * 4
    qc = torch.zeros((B, 576), device="cuda")
    d_nw, d_wqc = dev(w["sisa.attn_norm.weight"]), dev(np.ascontiguousarray(wqc.T).astype(np.float32))
    ok(L.shvk_readout_qc(h_last, 321 * 384, d_nw.data_ptr(), d_wqc.data_ptr(), qc.data_ptr(), B, stream_ptr()))
    sync()
    h32 = H.cpu().numpy().astype(np.float64)
    xl = O.rms_norm(h32[:, 320], f64("sisa.attn_norm.weight"))
    assert np.abs(qc.cpu().numpy() - xl @ wqc.T).max() < 2e-5
    # part 2
    up = np.empty((1920, 384))
    up[0::2], up[1::2] = f64("sisa.ffn.w_gate.weight"), f64("sisa.ffn.w_up.weight")                # (gate, up) interleaved
    mats = {"wo_t": f64(f"{a}.W_O.weight").T, "ffn_norm_w": f64("sisa.ffn_norm.weight"), "up_t": up.T,
            "down_t": f64("sisa.ffn.w_down.weight").T, "final_norm_w": f64("final_norm.weight"),
            "head_w0_t": f64("head.0.weight").T, "head_b0": f64("head.0.bias"), "head_w2": f64("head.2.weight").reshape(128),
            "head_b2": f64("head.2.bias")}
    keep = {k: dev(np.ascontiguousarray(v).astype(np.float32)) for k, v in mats.items()}
    rw = binding.ReadoutWeights(**{k: v.data_ptr() for k, v in keep.items()})
    Y = dev(y.astype(np.float32))
    y32 = Y.cpu().numpy().astype(np.float64)
    x1 = h32[:, 320] + y32 @ f64(f"{a}.W_O.weight").T
    xf = O.rms_norm(x1, f64("sisa.ffn_norm.weight"))
    x2 = x1 + (silu(xf @ f64("sisa.ffn.w_gate.weight").T) * (xf @ f64("sisa.ffn.w_up.weight").T)) @ f64("sisa.ffn.w_down.weight").T
    z = O.rms_norm(x2, f64("final_norm.weight"))
    ref = silu(z @ f64("head.0.weight").T + f64("head.0.bias")) @ f64("head.2.weight").reshape(128) + f64("head.2.bias")[0]
    x2_out, logits = torch.zeros((B, 384), device="cuda"), torch.zeros(B, device="cuda")
    ok(L.shvk_readout_tail(Y.data_ptr(), h_last, 321 * 384, C.byref(rw), x2_out.data_ptr(), logits.data_ptr(), B, stream_ptr()))
    sync()
    assert np.abs(x2_out.cpu().numpy() - x2).max() < 5e-5
    assert np.abs(logits.cpu().numpy() - ref).max() < 2e-5
    # clip 20 alone (first of a tile instead of fifth, no neighbours): bitwise the same
    one = torch.zeros(1, device="cuda")
    H1, Y1 = H[20:21].contiguous(), Y[20:21].contiguous()
    ok(L.shvk_readout_tail(Y1.data_ptr(), H1.data_ptr() + 320 * 384 * 4, 321 * 384, C.byref(rw), None, one.data_ptr(), 1, stream_ptr()))
    sync()
    assert torch.equal(one[0], logits[20])
    # the clips-per-CTA variants (16 for large batches, 4, 2, 1): the same clips give the same bits in each
    Bbig = 2400
    hb = rng.standard_normal((Bbig, 384)).astype(np.float32)
    yb = (rng.standard_normal((Bbig, 384)) * 0.5).astype(np.float32)
    Hb, Yb = dev(hb), dev(yb)
    outs = {}
    for n in (Bbig, 640, 400, 37):
        lg, q = torch.zeros(n, device="cuda"), torch.zeros((n, 576), device="cuda")
        ok(L.shvk_readout_qc(Hb.data_ptr(), 384, d_nw.data_ptr(), d_wqc.data_ptr(), q.data_ptr(), n, stream_ptr()))
        ok(L.shvk_readout_tail(Yb.data_ptr(), Hb.data_ptr(), 384, C.byref(rw), None, lg.data_ptr(), n, stream_ptr()))
        sync()
        outs[n] = (lg.cpu().numpy(), q.cpu().numpy())
    for n in (640, 400, 37):
        np.testing.assert_array_equal(outs[n][0].view(np.uint32), outs[Bbig][0][:n].view(np.uint32))
        np.testing.assert_array_equal(outs[n][1].view(np.uint32), outs[Bbig][1][:n].view(np.uint32))
    x1 = hb.astype(np.float64) + yb.astype(np.float64) @ f64(f"{a}.W_O.weight").T
    xf = O.rms_norm(x1, f64("sisa.ffn_norm.weight"))
    x2 = x1 + (silu(xf @ f64("sisa.ffn.w_gate.weight").T) * (xf @ f64("sisa.ffn.w_up.weight").T)) @ f64("sisa.ffn.w_down.weight").T
    z = O.rms_norm(x2, f64("final_norm.weight"))
    ref = silu(z @ f64("head.0.weight").T + f64("head.0.bias")) @ f64("head.2.weight").reshape(128) + f64("head.2.bias")[0]
    assert np.abs(outs[Bbig][0] - ref).max() < 2e-5


def test_store_tokens(L):
    import torch
    blocks = torch.arange(4 * 6144, device="cuda", dtype=torch.float32).reshape(4, 6144)
    pool = torch.zeros((6, 6144), device="cuda")
    slots = dev(np.array([5, -1, 0, 2], np.int32))
    ok(L.shvk_store_tokens(blocks.data_ptr(), slots.data_ptr(), pool.data_ptr(), 4, stream_ptr()))
    sync()
    assert torch.equal(pool[5], blocks[0]) and torch.equal(pool[0], blocks[2]) and torch.equal(pool[2], blocks[3])
    assert (pool[[1, 3, 4]] == 0).all()
