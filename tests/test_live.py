"""Streaming load: ring-slot arithmetic (CPU) and, on a GPU, hops of several participants through frames + store_slots +
window_slots requests, checked against whole-clip predictions and the reference's CPU engine."""
import numpy as np
import pytest

from shield_sisa_b200 import live


def test_ring_slots_follow_the_reference_driver():
    # participant p owns [24 p, 24 p + 24); frame k lives in slot 24 p + k % 24 (bench/gpu_bench.cpp:142,159-162)
    assert live.ring_slot(0, 0) == 0 and live.ring_slot(3, 25) == 3 * 24 + 1
    store, window = live.hop_slots(2, 0, 20)
    assert store.tolist() == [48 + i for i in range(20)] and window.tolist() == store.tolist()
    store, window = live.hop_slots(2, 20, 4)
    assert store.tolist() == [48 + 20, 48 + 21, 48 + 22, 48 + 23]
    assert window.tolist() == [48 + (4 + s) % 24 for s in range(20)]
    store, window = live.hop_slots(1, 24, 4)                      # the ring wraps: frames 24..27 overwrite slots 0..3
    assert store.tolist() == [24, 25, 26, 27]
    assert window.tolist() == [24 + (8 + s) % 24 for s in range(20)]
    # a window never reads a slot that the same hop does not own or that holds a frame older than 20 hops' worth
    for sent in range(20, 80, 4):
        store, window = live.hop_slots(5, sent, 4)
        assert len(set(window.tolist())) == 20 and set(store.tolist()) <= set(window.tolist())
        assert all(5 * 24 <= s < 6 * 24 for s in window)
    with pytest.raises(ValueError):
        live.hop_slots(0, 0, 4)                                    # first hop must fill the window
    with pytest.raises(ValueError):
        live.hop_slots(0, 20, 24)


@pytest.mark.gpu
def test_live_hops_match_whole_clip_predictions(weight_files):
    from oracle import ref_cpu
    from shield_sisa_b200 import binding, weights as W
    path, _ = weight_files("W5", 3)
    P, hops, new = 5, 3, 4
    total = 20 + hops * new
    crops = W.synth_frames(P * total, 41).reshape(P, total, 180, 320, 3)
    with binding.CudaModel(path, "fp32", max_frames=64, max_windows=8, max_host_tokens=20, token_slots=24 * P) as m:
        drv = live.LiveDriver(m, P)
        sent = 0
        cpu = ref_cpu.RefCpuEngine(path, threads=4) if ref_cpu.available() else None
        for h in range(hops + 1):
            n = 20 if h == 0 else new
            logits, timings = drv.hop(crops[:, sent:sent + n])
            sent += n
            clips = crops[:, sent - 20:sent]                       # what each participant's window now covers
            want = m.predict(clips)
            np.testing.assert_array_equal(logits.view(np.uint32), want.view(np.uint32))      # rings = whole clips, bitwise
            assert all(t["batch_frames"] >= n and t["batch_windows"] >= 1 for t in timings)
            if cpu is not None:
                assert np.abs(logits - cpu.predict(clips)).max() <= 1e-4                     # reference CPU engine
        if cpu is not None:
            cpu.close()
        assert drv.frames_sent.tolist() == [total] * P
    with binding.CudaModel(path, "fp32", max_frames=32, max_windows=2, max_host_tokens=20, token_slots=24) as m:
        with pytest.raises(ValueError):
            live.LiveDriver(m, 2)
