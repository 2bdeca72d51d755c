"""Streaming load: ring-slot arithmetic (CPU) and, on a GPU, hops of several participants through frames + store_slots +
window_slots requests, checked against whole-clip predictions and the reference's CPU engine."""
import os

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


def _fake_window_score(store, window, hop):
    """Stand-in for a device: any deterministic function of what a hop request carries."""
    return float(np.dot(window.astype(np.float64) % 24, np.arange(1, 21)) + 1000.0 * hop + store.size)


def _live_rank(rank, world, port, ids, hops, out_path):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mine = live.place_participants(ids, world)[rank]
        sent = [0] * len(mine)
        rows = []
        for h in range(hops):
            new = 20 if h == 0 else 4
            for local, gi in enumerate(mine):                       # local ring index = position on this device
                store, window = live.hop_slots(local, sent[local], new)
                assert store.min() >= local * 24 and window.max() < (local + 1) * 24
                sent[local] += new
                rows.append((h, gi, _fake_window_score(store, window, h)))
        gathered = [None] * world if rank == 0 else None
        dist.gather_object(rows, gathered, dst=0)                   # host gather of the logits, as for window shards
        if rank == 0:
            table = np.full((hops, len(ids)), np.nan)
            for part in gathered:
                for h, gi, v in part:
                    assert np.isnan(table[h, gi])                   # every participant scored by exactly one device
                    table[h, gi] = v
            np.save(out_path, table)
    finally:
        dist.destroy_process_group()


def test_two_device_placement_covers_every_participant_once(tmp_path):
    import torch.multiprocessing as mp
    ids = [f"participant-{i}" for i in range(37)]
    placed = live.place_participants(ids, 2)
    assert sorted(placed[0] + placed[1]) == list(range(37)) and placed == live.place_participants(ids, 2)
    out = tmp_path / "live.npy"
    port = 31000 + os.getpid() % 2000
    mp.spawn(_live_rank, args=(2, port, ids, 3, str(out)), nprocs=2, join=True)
    table = np.load(out)
    assert np.isfinite(table).all()
    # a participant's ring arithmetic depends only on its own history, so both devices produce what one device would
    for rank_list in placed:
        for local, gi in enumerate(rank_list):
            sent = 0
            for h in range(3):
                new = 20 if h == 0 else 4
                store, window = live.hop_slots(local, sent, new)
                sent += new
                assert table[h, gi] == _fake_window_score(store, window, h)


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
