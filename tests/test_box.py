"""The multi-device box (shv_box_*) over stand-in models: placement of sessions, slot-block accounting, contiguous
sharding of batches and error reporting, without a GPU.  The stand-ins are Python callbacks behind shv_box_ops."""
import ctypes as C
import zlib

import numpy as np
import pytest

from shield_sisa_b200 import binding, sharding


class FakeModels:
    """Stand-in for the per-device models: load hands out small integer handles, classify writes
    1000 * device + (first token value of the clip), submit records which model was asked."""

    def __init__(self, fail_device=None, fail_classify=None):
        self.loaded, self.freed, self.calls, self.submits = {}, [], [], []
        self.fail_device, self.fail_classify = fail_device, fail_classify
        self.error = b""
        self.ops = binding.BoxOps(binding.LOAD_FN(self._load), binding.FREE_FN(self._free), binding.SUBMIT_FN(self._submit),
                                  binding.CLASSIFY_FN(self._classify), binding.ERROR_FN(lambda: self.error))

    def _load(self, weights, mode, device, opt):
        if device == self.fail_device:
            self.error = b"no such GPU"
            return None
        handle = 100 + device
        self.loaded[handle] = {"device": device, "mode": mode, "token_slots": opt.contents.token_slots,
                               "max_windows": opt.contents.max_windows}
        return handle

    def _free(self, m):
        self.freed.append(m)

    def _submit(self, m, req):
        self.submits.append((m, req.contents.n_windows))
        return 7000 + m

    def _classify(self, m, tokens, b, logits):
        dev = self.loaded[m]["device"]
        self.calls.append((dev, b))
        if dev == self.fail_classify:
            self.error = b"boom"
            return -1
        tok = np.ctypeslib.as_array(C.cast(tokens, C.POINTER(C.c_float)), shape=(b, 20 * 6144))
        out = np.ctypeslib.as_array(C.cast(logits, C.POINTER(C.c_float)), shape=(b,))
        out[:] = 1000.0 * dev + tok[:, 0]
        return 0


def make_box(fake, devices, max_sessions=0, **opts):
    return binding.Box("unused.weights", "fp16", devices, max_sessions=max_sessions, ops=fake.ops, **opts)


def test_box_loads_one_model_per_device_and_frees_them():
    fake = FakeModels()
    box = make_box(fake, [0, 1, 2], max_sessions=30, max_windows=77)
    assert sorted(v["device"] for v in fake.loaded.values()) == [0, 1, 2]
    # every device gets the same options; the slot pool is sized for its share of the sessions plus a quarter
    assert all(v["max_windows"] == 77 and v["mode"] == b"fp16" for v in fake.loaded.values())
    assert all(v["token_slots"] == (10 + 2 + 8) * 24 for v in fake.loaded.values())
    assert box.L.shv_box_devices(box.b) == 3 and box.model_handle(1) == 101 and box.model_handle(3) is None
    box.close()
    assert sorted(fake.freed) == [100, 101, 102]


def test_box_load_failure_names_the_device_and_releases_the_rest():
    fake = FakeModels(fail_device=1)
    with pytest.raises(RuntimeError, match="device 1: no such GPU"):
        make_box(fake, [0, 1, 2])
    assert sorted(fake.freed) == [100, 102]


def test_sessions_are_placed_by_participant_and_spill_when_a_device_is_full():
    fake = FakeModels()
    box = make_box(fake, [0, 1], max_sessions=8)            # 4 + 1 + 8 = 13 blocks per device, capped at 8
    names = [f"participant-{i}" for i in range(16)]
    placed = {}
    for n in names:
        assert box.home_device(n) == sharding.device_of_participant(n, 2) == zlib.crc32(n.encode()) % 2
        placed[n] = box.session_open(n)
    # distinct slot blocks per device, each a multiple of 24
    for d in (0, 1):
        bases = [s for (dev, s) in placed.values() if dev == d]
        assert len(bases) == len(set(bases)) == 8 and all(s % 24 == 0 and 0 <= s < 8 * 24 for s in bases)
    # the first eight of each home device stayed home; the rest spilled to the other one
    spilled = [n for n in names if placed[n][0] != box.home_device(n)]
    assert len(spilled) == abs(sum(1 for n in names if box.home_device(n) == 0) - 8)
    with pytest.raises(RuntimeError, match="max_sessions reached"):
        box.session_open("one-too-many")
    assert box.free_sessions(0) == 0 and box.free_sessions(1) == 0
    dev, base = placed[names[3]]
    box.session_close(dev, base)
    assert box.free_sessions(dev) == 1
    with pytest.raises(RuntimeError, match="not in use"):
        box.session_close(dev, base)
    assert box.session_open("newcomer") == (dev, base) or box.home_device("newcomer") != dev
    box.close()


def test_requests_go_to_the_session_device():
    fake = FakeModels()
    box = make_box(fake, [4, 5, 6], max_sessions=4)
    req = binding.Request()
    req.n_windows = 3
    assert box.submit(2, req) == 7000 + 106
    assert box.submit(0, req) == 7000 + 104
    assert fake.submits == [(106, 3), (104, 3)]
    assert box.submit(3, req) is None and "no such device" in binding.last_error(box.L)
    box.close()


@pytest.mark.parametrize("b,n", [(10, 3), (2, 4), (4096, 8), (0, 2)])
def test_batches_are_cut_into_contiguous_shards(b, n):
    fake = FakeModels()
    box = make_box(fake, list(range(n)))
    tok = np.zeros((b, 20, 16, 384), np.float32)
    tok[:, 0, 0, 0] = np.arange(b)
    got = box.classify(tok)
    for r in range(n):
        lo, hi = sharding.shard_bounds(b, n, r)
        np.testing.assert_array_equal(got[lo:hi], 1000.0 * r + np.arange(lo, hi))
    assert sorted(fake.calls) == sorted((r, sharding.shard_bounds(b, n, r)[1] - sharding.shard_bounds(b, n, r)[0])
                                        for r in range(n) if sharding.shard_bounds(b, n, r)[1] > sharding.shard_bounds(b, n, r)[0])
    box.close()


def test_a_failing_device_fails_the_batch_with_its_name():
    fake = FakeModels(fail_classify=1)
    box = make_box(fake, [0, 1])
    with pytest.raises(RuntimeError, match="device 1: boom"):
        box.classify(np.zeros((4, 20, 16, 384), np.float32))
    box.close()
