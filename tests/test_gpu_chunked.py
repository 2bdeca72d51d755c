"""Long-sequence gated delta rule (chunked WY form on the tensor cores) against the float64 recurrence of the oracle and the
golden vectors produced by the reference's own gated_delta_rule_recurrent."""
import numpy as np
import pytest

from oracle import seq_oracle as O
from shield_sisa_b200 import binding
from tests.golden.make_golden_inputs import delta_inputs
from tests.helpers import dev, load_golden, rel_err, stream_ptr, sync

pytestmark = pytest.mark.gpu
TOL = 2e-2      # max|err| / max|ref|, the bf16-mode budget


def run_chunked(L, q, k, v, g, beta, out_bf16=False):
    import torch
    b, t, h, dk = q.shape
    dv = v.shape[-1]
    Q, K, V = (dev(x.astype(np.float32), torch.bfloat16) for x in (q, k, v))
    G, Bt = dev(g.astype(np.float32)), dev(beta.astype(np.float32))
    out = torch.zeros((b, t, h, dv), device="cuda", dtype=torch.bfloat16 if out_bf16 else torch.float32)
    nws = L.shvk_gdn_chunked_workspace_bytes(b, t, h)
    assert nws == b * h * ((t + 15) // 16) * 1152
    ws = torch.full((nws,), 0xff, device="cuda", dtype=torch.uint8)            # poison: the kernels must not rely on its contents
    rc = L.shvk_gdn_chunked(Q.data_ptr(), K.data_ptr(), V.data_ptr(), G.data_ptr(), Bt.data_ptr(), out.data_ptr(),
                            1 if out_bf16 else 0, b, t, h, dk, dv, float(dk ** -0.5), ws.data_ptr(), nws, stream_ptr())
    assert rc == 0, rc
    sync()
    rounded = tuple(x.float().cpu().numpy().astype(np.float64) for x in (Q, K, V))
    return out.float().cpu().numpy().astype(np.float64), rounded


@pytest.fixture(scope="module")
def L():
    return binding.load_library(True)


@pytest.mark.parametrize("tag", ["k64v128", "k128v128"])
def test_matches_reference_recurrence_golden(L, tag):
    g = load_golden("delta_rule")
    b, t, h, dk, dv, seed = (int(x) for x in g[f"{tag}:shape"])
    q, k, v, gg, beta = delta_inputs(b, t, h, dk, dv, seed)
    got, (qr, kr, vr) = run_chunked(L, q, k, v, gg, beta)
    # against the reference's float64 output on the unrounded inputs (includes the bf16 rounding of q, k, v)
    assert rel_err(got[:, ::16], g[f"{tag}:o"]) < TOL
    # against the oracle evaluated on exactly the bf16 inputs the kernel saw
    ref = O.gated_delta_rule_recurrent(qr, kr, vr, gg.astype(np.float32).astype(np.float64),
                                       beta.astype(np.float32).astype(np.float64), dk ** -0.5)
    err = rel_err(got, ref)
    rms = float(np.sqrt(((got - ref) ** 2).mean() / (ref ** 2).mean()))
    print(f"chunked {tag}: max-rel {err:.3e} rms-rel {rms:.3e}")
    assert err < TOL and rms < TOL


@pytest.mark.parametrize("dk", [64, 128])
def test_long_sequence_stress_shape(L, dk):
    """T = 2048 (the long-sequence stress configuration, here with 2 x 3 sequences so that the float64 oracle stays short):
    ragged tail handling, causality (a prefix of a longer run equals the shorter run bitwise), bf16 output."""
    b, t, h = 2, 2048, 3
    q, k, v, gg, beta = delta_inputs(b, t, h, dk, 128, seed=3)
    got, (qr, kr, vr) = run_chunked(L, q, k, v, gg, beta)
    ref = O.gated_delta_rule_recurrent(qr, kr, vr, gg.astype(np.float32).astype(np.float64),
                                       beta.astype(np.float32).astype(np.float64), dk ** -0.5)
    assert rel_err(got, ref) < TOL
    assert rel_err(got[:, -64:], ref[:, -64:]) < TOL           # no drift at the far end
    short, _ = run_chunked(L, q[:, :1001], k[:, :1001], v[:, :1001], gg[:, :1001], beta[:, :1001])   # 1001 = 62 * 16 + 9
    np.testing.assert_array_equal(short, got[:, :1001])
    low, _ = run_chunked(L, q, k, v, gg, beta, out_bf16=True)
    assert rel_err(low, ref) < TOL


def test_rejects_unsupported_shapes(L):
    import torch
    x = torch.zeros(4096, device="cuda")
    args = [x.data_ptr()] * 6
    ws = (x.data_ptr(), 4096 * 4, stream_ptr())
    assert L.shvk_gdn_chunked(*args, 0, 1, 16, 1, 32, 128, 1.0, *ws) != 0      # DK
    assert L.shvk_gdn_chunked(*args, 0, 1, 16, 1, 64, 64, 1.0, *ws) != 0       # DV
    assert L.shvk_gdn_chunked(*args, 2, 1, 16, 1, 64, 128, 1.0, *ws) != 0      # output type
    assert L.shvk_gdn_chunked(*args, 0, 1, 16, 1, 64, 128, 1.0, x.data_ptr(), 100, stream_ptr()) != 0   # workspace too small
    assert L.shvk_gdn_chunked(*args, 0, 0, 16, 1, 64, 128, 1.0, *ws) == 0      # empty batch
