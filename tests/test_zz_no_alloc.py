"""The squeeze-excite gate for callers that cannot allocate device memory (shvk_cnn_se_gate_static).

Some hosts give the whole GPU to their own pool at start-up, or run the encoder inside a frame loop where a cudaMalloc
(a device-wide synchronisation that can also fail) is not allowed.  For them the library carries the gate's partial-sum
scratch inside its own image.  This file checks, through the C ABI, that the variant gives the same gates as
shvk_cnn_se_gate with caller scratch, on two calls in a row (the second smaller, so it runs over what the first left
in the shared array), and that a batch beyond the built-in size is refused with a message instead of being launched.
It is named to be collected last."""
import ctypes as C

import numpy as np
import pytest

from tests.helpers import dev, stream_ptr, sync

pytestmark = pytest.mark.gpu

STATIC_FLOATS = 1 << 18


def _gates(L, x, w1, b1, w2, b2, static):
    import torch
    F, HW, Cn = x.shape
    CS = w1.shape[0]
    bufs = [dev(a) for a in (x, w1, b1, w2, b2)]
    gate = torch.full((F, Cn), float("nan"), dtype=torch.float32, device="cuda")
    p = [C.c_void_p(t.data_ptr()) for t in bufs]
    if static:
        rc = L.shvk_cnn_se_gate_static(p[0], p[1], p[2], p[3], p[4], C.c_void_p(gate.data_ptr()), F, HW, Cn, CS, stream_ptr())
    else:
        partial = torch.empty(L.shvk_cnn_se_partial_floats(F, HW, Cn), dtype=torch.float32, device="cuda")
        rc = L.shvk_cnn_se_gate(p[0], C.c_void_p(partial.data_ptr()), p[1], p[2], p[3], p[4], C.c_void_p(gate.data_ptr()),
                                F, HW, Cn, CS, stream_ptr())
    assert rc == 0
    sync()
    return gate.cpu().numpy()


def test_static_scratch_gate_matches_caller_scratch_gate_twice():
    from shield_sisa_b200 import binding
    L = binding.load_library(True)
    rng = np.random.default_rng(77)
    for F, HW, Cn, CS in ((5, 240, 672, 168), (2, 920, 72, 24)):        # second call: fewer, different partial sums
        x = rng.standard_normal((F, HW, Cn)).astype(np.float32)
        w1 = (rng.standard_normal((CS, Cn)) / np.sqrt(Cn)).astype(np.float32)
        b1 = rng.standard_normal(CS).astype(np.float32)
        w2 = (rng.standard_normal((Cn, CS)) / np.sqrt(CS)).astype(np.float32)
        b2 = rng.standard_normal(Cn).astype(np.float32)
        want = _gates(L, x, w1, b1, w2, b2, static=False)
        got = _gates(L, x, w1, b1, w2, b2, static=True)
        assert np.isfinite(got).all()
        assert np.abs(got - want).max() <= 1e-5                         # the tolerance of the gate's own parity test
        assert np.array_equal(got, want)                                # and in fact the same bits: same kernels
        pooled = x.astype(np.float64).mean(axis=1)
        ref = np.clip(np.maximum(pooled @ w1.T + b1, 0) @ w2.T + b2 + 3.0, 0, 6) / 6
        assert np.abs(got - ref).max() <= 1e-5


def test_static_scratch_gate_refuses_oversize_batches():
    from shield_sisa_b200 import binding
    L = binding.load_library(True)
    F, HW, Cn = 98, 240, 672                                            # 98 * 4 * 672 floats > 2^18
    assert L.shvk_cnn_se_partial_floats(F, HW, Cn) > STATIC_FLOATS
    rc = L.shvk_cnn_se_gate_static(None, None, None, None, None, None, F, HW, Cn, 168, stream_ptr())   # refused before any launch
    assert rc != 0
    msg = binding.last_error(L)
    assert "do not fit the built-in" in msg and str(STATIC_FLOATS) in msg
    assert L.shvk_cnn_se_partial_floats(97, HW, Cn) <= STATIC_FLOATS
