"""The multi-device box on real GPUs (needs at least two): a batch sharded over two devices equals the single-device
result bit for bit, and live hops of participants placed on two devices equal whole-clip predictions bit for bit."""
import numpy as np
import pytest

from shield_sisa_b200 import binding, live, weights as W

pytestmark = pytest.mark.gpu


def gpu_count():
    import torch
    return torch.cuda.device_count()


@pytest.fixture(scope="module")
def two_gpus():
    if gpu_count() < 2:
        pytest.skip("needs two GPUs")


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
def test_sharded_batch_equals_one_device_bitwise(two_gpus, mode, weight_files):
    path, _ = weight_files("W3", 1)
    tok = W.synth_tokens(37, 19)
    with binding.CudaModel(path, mode, device=0, max_windows=64, max_host_tokens=1280) as m:
        want = m.classify(tok)
    with binding.Box(path, mode, [0, 1], max_windows=64, max_host_tokens=1280) as box:
        got = box.classify(tok)
        again = box.classify(tok[::-1].copy())[::-1]
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    np.testing.assert_array_equal(again.view(np.uint32), want.view(np.uint32))      # a clip's device does not matter


def test_live_hops_on_two_devices_match_whole_clip_predictions(two_gpus, weight_files):
    path, _ = weight_files("W5", 3)
    P, hops, new = 7, 2, 4
    total = 20 + hops * new
    crops = W.synth_frames(P * total, 43).reshape(P, total, 180, 320, 3)
    ids = [f"participant-{i}" for i in range(P)]
    with binding.CudaModel(path, "fp32", device=0, max_frames=160, max_windows=8, max_host_tokens=20) as single, \
            binding.Box(path, "fp32", [0, 1], max_sessions=P, max_frames=160, max_windows=8, max_host_tokens=20) as box:
        drv = live.BoxLiveDriver(box, ids)
        assert {d for d, _ in drv.sessions} == {0, 1}                                 # both devices hold rings
        assert all(d == box.home_device(pid) for (d, _), pid in zip(drv.sessions, ids))
        sent = 0
        for h in range(hops + 1):
            n = 20 if h == 0 else new
            logits, sizes = drv.hop(lambda p: crops[p, sent:sent + n], n)
            sent += n
            want = single.predict(crops[:, sent - 20:sent])
            np.testing.assert_array_equal(logits.view(np.uint32), want.view(np.uint32))
