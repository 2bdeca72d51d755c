"""GPU parity of the frame encoder: kernels one by one against numpy, and Engine::encode through the C ABI against the
float64 oracle, the golden tokens of the reference's PyTorch oracle and the reference's CPU engine.

Tolerance: fp32 mode max abs error <= 1e-4 on tokens of O(1) magnitude (recipe W5); bf16 / fp16 modes (operands of the
1x1 convolutions rounded to that type, everything else float32) max |err| / max |ref| <= 2e-2."""
import ctypes as C

import numpy as np
import pytest

from tests.helpers import dev, load_golden, rel_err, stream_ptr, sync

pytestmark = pytest.mark.gpu

TOL = 1e-4


@pytest.fixture(scope="module")
def L():
    from shield_sisa_b200 import binding
    return binding.load_library(True)


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _hardswish(x):
    return x * np.clip(x + 3.0, 0.0, 6.0) / 6.0


def test_stem_kernel(L):
    import torch
    from oracle import cnn_oracle as CO
    rng = np.random.default_rng(0)
    F = 3
    frames = rng.integers(0, 256, size=(F, 180, 320, 3), dtype=np.uint8)
    frames[0, 0, 0] = (0, 255, 0)                                           # corners exercise the padding taps
    w = (rng.standard_normal((16, 3, 3, 3)) * 0.3).astype(np.float32)
    b = rng.standard_normal(16).astype(np.float32)
    lut = np.stack([((np.arange(256, dtype=np.float32) / np.float32(255)) - CO.MEAN[c]) / CO.STD[c] for c in range(3)])
    w_tap = np.ascontiguousarray(w.transpose(2, 3, 1, 0).reshape(27, 16))   # ((kh*3 + kw)*3 + ci, co)
    out = torch.empty((F, 90, 160, 16), dtype=torch.float32, device="cuda")
    d_frames, d_lut, d_w, d_b = dev(frames), dev(lut.astype(np.float32)), dev(w_tap), dev(b)   # keep the buffers alive
    rc = L.shvk_cnn_stem(_ptr(d_frames), _ptr(d_lut), _ptr(d_w), _ptr(d_b), _ptr(out), F, stream_ptr())
    assert rc == 0
    sync()
    ref = _hardswish(CO.conv_dense(CO.normalise(frames, np.float64), w.astype(np.float64), 3, 2) + b)
    assert np.abs(out.cpu().numpy() - ref).max() < 1e-4


@pytest.mark.parametrize("k,stride,H,W,Cn,act", [(3, 1, 12, 20, 24, 1), (3, 2, 45, 80, 72, 1), (5, 2, 23, 40, 120, 2), (5, 1, 6, 10, 960, 2)])
def test_depthwise_kernel(L, k, stride, H, W, Cn, act):
    import torch
    from oracle import cnn_oracle as CO
    rng = np.random.default_rng(k * 10 + stride)
    F = 2
    x = rng.standard_normal((F, H, W, Cn)).astype(np.float32)
    w = (rng.standard_normal((Cn, 1, k, k)) * 0.4).astype(np.float32)
    b = rng.standard_normal(Cn).astype(np.float32)
    pad = (k - 1) // 2
    Ho, Wo = (H + 2 * pad - k) // stride + 1, (W + 2 * pad - k) // stride + 1
    w_tap = np.ascontiguousarray(w.reshape(Cn, k * k).T)
    out = torch.empty((F, Ho, Wo, Cn), dtype=torch.float32, device="cuda")
    d_x, d_w, d_b = dev(x), dev(w_tap), dev(b)
    rc = L.shvk_cnn_depthwise(_ptr(d_x), _ptr(d_w), _ptr(d_b), _ptr(out), F, H, W, Cn, k, stride, Ho, Wo, act, stream_ptr())
    assert rc == 0
    sync()
    ref = CO.conv_depthwise(x.astype(np.float64), w.astype(np.float64), k, stride) + b
    ref = np.maximum(ref, 0) if act == 1 else _hardswish(ref)
    assert np.abs(out.cpu().numpy() - ref).max() < 1e-5
    # wrong output size is refused, not launched
    assert L.shvk_cnn_depthwise(_ptr(d_x), _ptr(d_w), _ptr(d_b), _ptr(out), F, H, W, Cn, k, stride, Ho + 1, Wo, act,
                                stream_ptr()) != 0


@pytest.mark.parametrize("HW,Cn,CS", [(920, 72, 24), (240, 672, 168), (60, 960, 240)])
def test_se_gate_kernel(L, HW, Cn, CS):
    import torch
    rng = np.random.default_rng(HW)
    F = 3
    x = rng.standard_normal((F, HW, Cn)).astype(np.float32)
    w1 = (rng.standard_normal((CS, Cn)) / np.sqrt(Cn)).astype(np.float32)
    b1 = rng.standard_normal(CS).astype(np.float32)
    w2 = (rng.standard_normal((Cn, CS)) / np.sqrt(CS)).astype(np.float32)
    b2 = rng.standard_normal(Cn).astype(np.float32)
    n = L.shvk_cnn_se_partial_floats(F, HW, Cn)
    assert n == F * ((HW + 63) // 64) * Cn
    partial = torch.full((n,), float("nan"), dtype=torch.float32, device="cuda")      # scratch need not be cleared
    gate = torch.empty((F, Cn), dtype=torch.float32, device="cuda")
    args = [dev(x), partial, dev(w1), dev(b1), dev(w2), dev(b2), gate]
    assert L.shvk_cnn_se_gate(*[_ptr(a) for a in args], F, HW, Cn, CS, stream_ptr()) == 0
    sync()
    pooled = x.astype(np.float64).mean(axis=1)
    hid = np.maximum(pooled @ w1.T.astype(np.float64) + b1, 0)
    ref = np.clip(hid @ w2.T.astype(np.float64) + b2 + 3.0, 0, 6) / 6
    got = gate.cpu().numpy()
    assert np.abs(got - ref).max() < 1e-5
    # a frame's gate does not depend on the batch it is in
    gate1 = torch.empty((1, Cn), dtype=torch.float32, device="cuda")
    args1 = [dev(x[1:2]), partial, dev(w1), dev(b1), dev(w2), dev(b2), gate1]
    assert L.shvk_cnn_se_gate(*[_ptr(a) for a in args1], 1, HW, Cn, CS, stream_ptr()) == 0
    sync()
    assert np.array_equal(gate1.cpu().numpy()[0], got[1])


@pytest.mark.parametrize("M,N,K,act,gated,resid", [(14400, 64, 16, 1, False, False), (1000, 24, 72, 0, False, True),
                                                  (120, 160, 960, 0, True, True), (60, 960, 160, 2, False, False),
                                                  (77, 40, 120, 0, True, False)])
def test_pointwise_kernel(L, M, N, K, act, gated, resid):
    import torch
    rng = np.random.default_rng(M + N)
    rows = 60 if gated and M % 60 == 0 else (11 if gated else 1)
    A = rng.standard_normal((M, K)).astype(np.float32)
    Wt = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    gate = rng.uniform(0, 1, size=((M + rows - 1) // rows, K)).astype(np.float32) if gated else None
    R = rng.standard_normal((M, N)).astype(np.float32) if resid else None
    out = dev(R) if resid else torch.empty((M, N), dtype=torch.float32, device="cuda")      # residual in place
    g_dev = dev(gate) if gated else None
    d_a, d_w, d_b = dev(A), dev(Wt), dev(b)
    rc = L.shvk_cnn_pointwise(_ptr(d_a), _ptr(d_w), _ptr(d_b), _ptr(g_dev) if gated else None, rows,
                              _ptr(out) if resid else None, _ptr(out), M, N, K, act, stream_ptr())
    assert rc == 0
    sync()
    a64 = A.astype(np.float64)
    if gated:
        a64 = a64 * np.repeat(gate.astype(np.float64), rows, axis=0)[:M]
    ref = a64 @ Wt.T.astype(np.float64) + b
    ref = np.maximum(ref, 0) if act == 1 else _hardswish(ref) if act == 2 else ref
    if resid:
        ref = ref + R
    assert np.abs(out.cpu().numpy() - ref).max() < 2e-5


@pytest.mark.parametrize("M,N,K,act,gated,resid", [(14400, 64, 16, 1, False, False), (1000, 24, 72, 0, False, True),
                                                  (120, 160, 960, 0, True, True), (60, 960, 160, 2, False, False),
                                                  (77, 40, 120, 0, True, False), (333, 80, 184, 0, False, True),
                                                  (4000, 16, 16, 0, False, True)])
def test_pointwise_tf32_kernel(L, M, N, K, act, gated, resid):
    """Tensor-core form of the 1x1 convolution: operands rounded to TF32 (2^-11 relative), float32 accumulation."""
    import torch
    rng = np.random.default_rng(M + N + 1)
    rows = 60 if gated and M % 60 == 0 else (11 if gated else 1)
    A = rng.standard_normal((M, K)).astype(np.float32)
    Wt = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    gate = rng.uniform(0, 1, size=((M + rows - 1) // rows, K)).astype(np.float32) if gated else None
    R = rng.standard_normal((M, N)).astype(np.float32) if resid else None
    out = dev(R) if resid else torch.empty((M, N), dtype=torch.float32, device="cuda")
    g_dev = dev(gate) if gated else None
    d_a, d_w, d_b = dev(A), dev(Wt), dev(b)
    rc = L.shvk_cnn_pointwise_tf32(_ptr(d_a), _ptr(d_w), _ptr(d_b), _ptr(g_dev) if gated else None, rows,
                                   _ptr(out) if resid else None, _ptr(out), M, N, K, act, stream_ptr())
    assert rc == 0
    sync()
    a64 = A.astype(np.float64)
    if gated:
        a64 = a64 * np.repeat(gate.astype(np.float64), rows, axis=0)[:M]
    ref = a64 @ Wt.T.astype(np.float64) + b
    ref = np.maximum(ref, 0) if act == 1 else _hardswish(ref) if act == 2 else ref
    if resid:
        ref = ref + R
    got = out.cpu().numpy()
    assert np.abs(got - ref).max() < 4e-3                      # |a| |w| sqrt(K) 2^-11 with a ~ N(0,1), w ~ N(0,1/K): about 5e-4
    assert np.abs(got - ref).max() > 0                         # not the exact kernel


@pytest.mark.parametrize("ab,tol", [(1, 2.5e-2), (2, 4e-3)])
@pytest.mark.parametrize("M,N,K,act,gated,resid", [(14400, 64, 16, 1, False, False), (1000, 24, 72, 0, False, True),
                                                  (120, 160, 960, 0, True, True), (60, 960, 160, 2, False, False),
                                                  (77, 40, 120, 0, True, False), (333, 80, 184, 0, False, True),
                                                  (4000, 16, 16, 0, False, True), (700, 384, 960, 0, False, False)])
def test_pointwise_16bit_kernel(L, M, N, K, act, gated, resid, ab, tol):
    """1x1 convolution with operands rounded to bf16 (2^-9 relative) or fp16 (2^-11), float32 accumulation."""
    import torch
    rng = np.random.default_rng(M + N + 2)
    rows = 60 if gated and M % 60 == 0 else (11 if gated else 1)
    A = rng.standard_normal((M, K)).astype(np.float32)
    Wt = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    gate = rng.uniform(0, 1, size=((M + rows - 1) // rows, K)).astype(np.float32) if gated else None
    R = rng.standard_normal((M, N)).astype(np.float32) if resid else None
    out = dev(R) if resid else torch.empty((M, N), dtype=torch.float32, device="cuda")
    g_dev = dev(gate) if gated else None
    d_a, d_w, d_b = dev(A), dev(Wt), dev(b)
    rc = L.shvk_cnn_pointwise_h(_ptr(d_a), _ptr(d_w), _ptr(d_b), _ptr(g_dev) if gated else None, rows,
                                _ptr(out) if resid else None, _ptr(out), M, N, K, act, ab, stream_ptr())
    assert rc == 0
    sync()
    a64 = A.astype(np.float64)
    if gated:
        a64 = a64 * np.repeat(gate.astype(np.float64), rows, axis=0)[:M]
    ref = a64 @ Wt.T.astype(np.float64) + b
    ref = np.maximum(ref, 0) if act == 1 else _hardswish(ref) if act == 2 else ref
    if resid:
        ref = ref + R
    got = out.cpu().numpy()
    assert np.abs(got - ref).max() < tol
    # the same rounding done on the host reproduces the kernel to float32 accumulation error
    dt = torch.bfloat16 if ab == 1 else torch.float16
    a_r = torch.from_numpy(a64.astype(np.float32)).to(dt).double().numpy()
    w_r = torch.from_numpy(Wt).to(dt).double().numpy()
    ref_r = a_r @ w_r.T + b
    ref_r = np.maximum(ref_r, 0) if act == 1 else _hardswish(ref_r) if act == 2 else ref_r
    if resid:
        ref_r = ref_r + R
    assert np.abs(got - ref_r).max() < 5e-5
    assert L.shvk_cnn_pointwise_h(_ptr(d_a), _ptr(d_w), _ptr(d_b), None, 1, None, _ptr(out), M, N, K, act, 0, stream_ptr()) != 0


def test_pool_tokens_kernel(L):
    import torch
    from oracle import cnn_oracle as CO
    rng = np.random.default_rng(5)
    F = 2
    fmap = rng.standard_normal((F, 6, 10, 960)).astype(np.float32)
    out = torch.empty((F, 16, 960), dtype=torch.float32, device="cuda")
    d_map = dev(fmap)
    assert L.shvk_cnn_pool_tokens(_ptr(d_map), _ptr(out), F, stream_ptr()) == 0
    sync()
    ident = {"projection.weight": np.eye(960, dtype=np.float64)}
    ref = CO.tokens_from_map(ident, fmap.astype(np.float64))
    assert np.abs(out.cpu().numpy() - ref).max() < 1e-6


# ---------------------------------------------------------------------------------------------- whole encoder
def _encode(eng, frames, slot=0):
    import torch
    F = frames.shape[0]
    src = dev(frames)
    stream = stream_ptr()
    torch.cuda.synchronize()
    dst = _wrap_u8(eng.frames_ptr(slot), F * 172800)       # device-to-device copy of the crops into the slot buffer
    dst.copy_(src.reshape(-1))
    eng.encode(slot, F, stream)
    sync()
    return _wrap_f32(eng.tokens_ptr(slot), F * 6144).cpu().numpy().reshape(F, 16, 384).copy()


def _wrap(ptr, nbytes, typestr):
    import torch

    class _Arr:
        pass

    a = _Arr()
    a.__cuda_array_interface__ = {"shape": (nbytes // int(typestr[-1]),), "typestr": typestr, "data": (int(ptr), False),
                                  "version": 2}
    return torch.as_tensor(a, device="cuda")


def _wrap_u8(ptr, n):
    return _wrap(ptr, n, "|u1")


def _wrap_f32(ptr, n):
    return _wrap(ptr, n * 4, "<f4")


@pytest.mark.parametrize("case", ["encoder_w5_s3_f11", "encoder_w1_s1_f5"])
@pytest.mark.parametrize("mode", ["fp32", "bf16", "fp16"])
def test_encode_matches_reference(case, mode, weight_files):
    from oracle import cnn_oracle as CO, ref_cpu
    from shield_sisa_b200 import binding, weights as W
    g = load_golden(case)
    path, w = weight_files(str(g["recipe"]), int(g["weight_seed"]))
    frames = W.synth_frames(int(g["frames"]), int(g["frame_seed"]))
    eng = binding.EngineCore(path, mode, max_windows=1, max_frames=4, use_graphs=False)
    tok = _encode(eng, frames)
    assert eng.status() == 0
    # fp32 mode: max abs error <= 1e-4.  16-bit modes (16-bit operands in the 1x1 convolutions): max |err| / max |ref| <= 2e-2
    def err(ref):
        return np.abs(tok - ref).max() if mode == "fp32" else rel_err(tok, ref)
    tol = TOL if mode == "fp32" else 2e-2
    assert err(g["tokens_f64"]) <= tol                                     # reference's PyTorch oracle, float64
    assert err(CO.encode_frames(w, frames, np.float64)) <= tol
    if "tokens_cpu_engine" in g:
        assert err(g["tokens_cpu_engine"]) <= tol                          # reference's CPU engine (stored)
    if ref_cpu.available():
        cpu = ref_cpu.RefCpuEngine(path, threads=2)
        assert err(cpu.encode_frames(frames)) <= tol                       # reference's CPU engine (run here)
        cpu.close()
    print(f"encoder {case} {mode}: err vs float64 oracle {err(g['tokens_f64']):.3e}")
    eng.close()


def test_encode_frame_independence_and_graphs(weight_files):
    """A frame's tokens are bitwise the same alone, in a batch, in another order and through a padded CUDA graph."""
    from shield_sisa_b200 import binding, weights as W
    path, _ = weight_files("W5", 3)
    frames = W.synth_frames(7, 21)
    eager = binding.EngineCore(path, "fp32", max_windows=1, max_frames=16, use_graphs=False)
    graph = binding.EngineCore(path, "fp32", max_windows=1, max_frames=16, use_graphs=True)
    full = _encode(eager, frames)
    assert np.array_equal(_encode(eager, frames[3:4])[0], full[3])
    perm = np.array([6, 2, 0, 5, 1, 4, 3])
    assert np.array_equal(_encode(eager, frames[perm], slot=1), full[perm])
    assert graph.frame_bucket(7) == 8
    assert np.array_equal(_encode(graph, frames), full)
    assert np.array_equal(_encode(graph, frames), full)                    # second launch of the captured graph
    from oracle.cnn_oracle import BLOCKS
    assert eager.encode_launches() == 4 + sum(2 + (1 if e != i else 0) + (2 if se else 0) for (i, _k, e, _o, se, _a, _s) in BLOCKS)
    eager.close()
    graph.close()
