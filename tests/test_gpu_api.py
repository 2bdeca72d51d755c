"""Job API of the C ABI on a GPU: asynchronous submit / wait / callback / timing, request validation, coalescing,
device token slots, pinned buffers, and failure reporting with the failure injected on the host."""
import os
import threading

import numpy as np
import pytest

from shield_sisa_b200 import binding, weights as W

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model(weight_files):
    path, _ = weight_files("W3", 1)
    m = binding.CudaModel(path, "fp32", max_windows=16, max_host_tokens=320, token_slots=64)
    yield m
    m.close()


def blocks_of(tok):
    """[b,20,16,384] -> list of b*20 contiguous [6144] blocks (separate arrays: no two are adjacent in memory)."""
    return [np.ascontiguousarray(tok[w, f].reshape(-1)).copy() for w in range(tok.shape[0]) for f in range(20)]


def test_async_job_lifecycle(model):
    tok = W.synth_tokens(3, 21)
    want = model.classify(tok)
    out = np.full(3, -7.0, np.float32)
    seen = []
    done = threading.Event()

    def cb(job, status, user):
        seen.append((status, out.copy()))          # outputs are written before the callback runs
        done.set()

    job, keep = model.submit(3, out, window_tokens=blocks_of(tok), callback=cb)
    assert job, binding.last_error(model.L)
    assert model.job_wait(job) == 0
    assert done.wait(10)
    assert model.job_status(job) == 1 and model.job_error(job) == ""
    rc, t = model.job_timing(job)
    assert rc == 0 and t["gpu_ms"] > 0 and t["run_ms"] > 0 and t["queue_ms"] >= 0
    assert t["batch_windows"] >= 3 and t["batch_frames"] == 0
    model.job_free(job)
    np.testing.assert_array_equal(out.view(np.uint32), want.view(np.uint32))
    assert seen[0][0] == 1 and np.array_equal(seen[0][1], want)


def test_many_jobs_coalesce_and_keep_order(model):
    tok = W.synth_tokens(12, 22)
    want = model.classify(tok)
    outs, jobs, keeps = [], [], []
    for w in range(12):
        o = np.zeros(1, np.float32)
        j, k = model.submit(1, o, window_tokens=blocks_of(tok[w:w + 1]))
        assert j
        outs.append(o); jobs.append(j); keeps.append(k)
    sizes = []
    for j in jobs:
        assert model.job_wait(j) == 0
        sizes.append(model.job_timing(j)[1]["batch_windows"])
        model.job_free(j)
    got = np.concatenate(outs)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    assert max(sizes) <= 16 and sum(1 for s in sizes if s > 1) > 0      # at least some jobs shared a batch


def test_request_validation(model):
    L = model.L
    tok = W.synth_tokens(1, 23)
    out = np.zeros(1, np.float32)
    cases = [
        (dict(n_windows=0, logits_out=out), "empty request"),
        (dict(n_windows=17, logits_out=np.zeros(17, np.float32), window_tokens=[None] * 340), "more windows than max_windows"),
        (dict(n_windows=1, logits_out=None, window_tokens=blocks_of(tok)), "null logits_out"),
        (dict(n_windows=1, logits_out=out), "window entry has no token source"),
        (dict(n_windows=1, logits_out=out, window_tokens=[None] * 20), "window entry has no token source"),
        (dict(n_windows=1, logits_out=out, window_slots=[64] + [0] * 19), "window slot out of range"),
        (dict(n_windows=1, logits_out=out, window_frames=[0] * 20, window_tokens=blocks_of(tok)), "window frame index out of range"),
        (dict(n_windows=0, logits_out=out, frames=None, n_frames=1), "null frames"),
        (dict(n_windows=0, logits_out=out, frames=np.zeros(172800, np.uint8), n_frames=641), "more frames than max_frames"),
        (dict(n_windows=0, logits_out=out, frames=np.zeros(2 * 172800, np.uint8), n_frames=2, store_slots=[64, 0]),
         "store slot out of range"),
        (dict(n_windows=0, logits_out=out, frames=np.zeros(2 * 172800, np.uint8), n_frames=2, store_slots=[5, 5]),
         "duplicate store slot"),
        (dict(n_windows=1, logits_out=out, frames=np.zeros(172800, np.uint8), n_frames=1, window_frames=[1] + [0] * 19),
         "window frame index out of range"),
    ]
    for kwargs, msg in cases:
        job, keep = model.submit(**kwargs)
        assert not job, msg
        assert msg in binding.last_error(L), (msg, binding.last_error(L))
    lg = np.zeros(1, np.float32)
    assert L.shv_cuda_predict(model.m, None, 1, lg.ctypes.data) == -1 and "null argument" in binding.last_error(L)
    assert L.shv_cuda_encode_frames(model.m, None, 1, lg.ctypes.data) == -1 and "null argument" in binding.last_error(L)
    assert L.shv_cuda_encode_frames(model.m, None, 0, None) == 0 and L.shv_cuda_predict(model.m, None, 0, None) == 0
    assert L.shv_cuda_classify(model.m, None, 1, lg.ctypes.data) == -1 and "null argument" in binding.last_error(L)
    assert L.shv_cuda_classify(model.m, None, 0, None) == 0


def test_device_token_slots(model):
    """Windows read 16x384 blocks from device slots; uploads are ordered against windows like the reference's stores."""
    tok = W.synth_tokens(2, 24)
    want = model.classify(tok)
    model.upload_tokens(tok[0], np.arange(20, dtype=np.int32) + 10)
    out = np.zeros(1, np.float32)
    job, keep = model.submit(1, out, window_slots=np.arange(20) + 10)
    assert job and model.job_wait(job) == 0
    model.job_free(job)
    assert out.view(np.uint32)[0] == want.view(np.uint32)[0]
    # mixed sources in one window: even frames from slots, odd frames from host pointers
    blocks = blocks_of(tok[:1])
    slots = [10 + f if f % 2 == 0 else -1 for f in range(20)]
    ptrs = [None if f % 2 == 0 else blocks[f] for f in range(20)]
    out2 = np.zeros(1, np.float32)
    job, keep = model.submit(1, out2, window_slots=slots, window_tokens=ptrs)
    assert job and model.job_wait(job) == 0
    model.job_free(job)
    assert out2.view(np.uint32)[0] == want.view(np.uint32)[0]
    # overwrite the slots: a window submitted afterwards sees the new tokens
    model.upload_tokens(tok[1], np.arange(20, dtype=np.int32) + 10)
    out3 = np.zeros(1, np.float32)
    job, keep = model.submit(1, out3, window_slots=np.arange(20) + 10)
    assert job and model.job_wait(job) == 0
    model.job_free(job)
    assert out3.view(np.uint32)[0] == want.view(np.uint32)[1]
    with pytest.raises(RuntimeError, match="out of range"):
        model.upload_tokens(tok[0, :1], np.array([64], np.int32))
    with pytest.raises(RuntimeError, match="duplicate"):
        model.upload_tokens(tok[0, :2], np.array([3, 3], np.int32))


def test_pinned_and_pageable_tokens_agree(model):
    tok = W.synth_tokens(4, 25)
    want = model.classify(tok)
    pin = binding.PinnedBuffer(model.L, tok.shape)
    pin.array[...] = tok
    got = model.classify(pin.array)
    pin.free()
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
def test_fp16_tokens_equal_fp32_tokens_of_the_same_values(mode, weight_files):
    """shv_cuda_b200_classify_f16: tokens handed over as fp16 are widened on the device before anything reads them, so
    the logits are bitwise those of shv_cuda_classify on the same (fp16-representable) values as fp32, from pageable
    and from pinned memory, for a call that is cut into several requests."""
    path, _ = weight_files("W3", 1)
    tok16 = W.synth_tokens(37, 31).astype(np.float16)
    with binding.CudaModel(path, mode, max_windows=16, max_host_tokens=320) as m:
        want = m.classify(tok16.astype(np.float32))
        got = m.classify_f16(tok16)
        np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
        pin = binding.PinnedBuffer(m.L, tok16.shape, np.float16)
        pin.array[...] = tok16
        got_pin = m.classify_f16(pin.array)
        pin.free()
        np.testing.assert_array_equal(got_pin.view(np.uint32), want.view(np.uint32))
        # against the unrounded embeddings: what fp16 rounding of the inputs costs.  In fp32 mode that is the rounding
        # itself; in bf16 mode any perturbation of the inputs moves the bf16 roundings inside the stack, so the logits
        # move by about the mode's own error
        full = m.classify(W.synth_tokens(37, 31))
        change = np.abs(got - full).max() / max(1.0, np.abs(full).max())
        print(f"fp16 host tokens, {mode} mode: max logit change {change:.2e} relative")
        assert change < (2e-3 if mode == "fp32" else 4e-2)


def test_concurrent_callers(model):
    tok = W.synth_tokens(6, 26)
    want = model.classify(tok)
    results = [None] * 6

    def worker(i):
        results[i] = model.classify(tok[i:i + 1])

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(6)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    np.testing.assert_array_equal(np.concatenate(results).view(np.uint32), want.view(np.uint32))


def test_failed_batch_reports_nan_and_engine_recovers(weight_files):
    """The failure is raised on the host before any GPU work of the batch (SHV_CUDA_FAIL_EVERY); the GPU is never
    faulted.  Every job of the failed batch fails, its logits are NaN, the next batch is scored normally."""
    path, _ = weight_files("W3", 1)
    tok = W.synth_tokens(2, 27)
    os.environ["SHV_CUDA_FAIL_EVERY"] = "2"
    try:
        m = binding.CudaModel(path, "fp32", max_windows=4, max_host_tokens=80)
    finally:
        del os.environ["SHV_CUDA_FAIL_EVERY"]
    first = m.classify(tok)                                  # batch 1: fine
    rc, lg, err = m.classify_rc(tok)                         # batch 2: injected failure
    assert rc == -1 and np.isnan(lg).all() and "injected batch failure" in err
    out = np.zeros(2, np.float32)
    job, keep = m.submit(2, out, window_tokens=blocks_of(tok))          # batch 3: fine
    assert m.job_wait(job) == 0
    m.job_free(job)
    np.testing.assert_array_equal(out.view(np.uint32), first.view(np.uint32))
    status = []
    out4 = np.zeros(2, np.float32)
    job, keep = m.submit(2, out4, window_tokens=blocks_of(tok), callback=lambda j, s, u: status.append(s))   # batch 4
    assert m.job_wait(job) == -1 and m.job_status(job) == -1 and "injected" in m.job_error(job)
    m.job_free(job)
    assert status == [-1] and np.isnan(out4).all()
    m.close()


@pytest.mark.parametrize("kind", [1, 2])
def test_kernel_wait_that_runs_out_fails_the_batch_and_the_model_recovers(kind, weight_files):
    """A bounded wait inside a kernel that really runs out: one launch of the next batch gets no input (kind 1: a
    tensor-core GEMM whose producer withholds an operand stage; kind 2: the scan, whose chunk copy is never issued), its
    poll loop hits the limit, the kernel sets the status word and returns.  The batch fails with NaN logits, the
    scheduler clears the word, and the following batch is scored bit for bit like the one before the failure."""
    path, _ = weight_files("W3", 1)
    tok = W.synth_tokens(3, 31)
    with binding.CudaModel(path, "bf16", max_windows=4, max_host_tokens=80) as m:
        first = m.classify(tok)
        m.test_starve(kind, 1)
        rc, lg, err = m.classify_rc(tok)
        assert rc == -1 and np.isnan(lg).all() and "gave up waiting" in err
        again = m.classify(tok)
    np.testing.assert_array_equal(again.view(np.uint32), first.view(np.uint32))


def test_starve_hook_is_refused_where_it_does_not_apply(weight_files):
    path, _ = weight_files("W3", 1)
    with binding.CudaModel(path, "fp32", max_windows=2, max_host_tokens=40) as m:
        with pytest.raises(RuntimeError, match="16-bit"):
            m.test_starve(1, 1)


def test_free_completes_queued_jobs(weight_files):
    path, _ = weight_files("W1", 1)
    tok = W.synth_tokens(1, 28)
    m = binding.CudaModel(path, "fp32", max_windows=2, max_host_tokens=40)
    want = m.classify(tok)
    outs, jobs, keeps = [], [], []
    for _ in range(6):
        o = np.zeros(1, np.float32)
        j, k = m.submit(1, o, window_tokens=blocks_of(tok))
        outs.append(o); jobs.append(j); keeps.append(k)
    m.close()                                                # completes everything queued, then releases the GPU
    for j, o in zip(jobs, outs):
        assert m.L.shv_cuda_job_status(j) == 1               # jobs outlive the model
        m.L.shv_cuda_job_free(j)
        assert o.view(np.uint32)[0] == want.view(np.uint32)[0]


def test_non_finite_logit_becomes_nan(weight_files, tmp_path):
    """fp16 overflow -> non-finite result -> reported as NaN = unavailable (reference api.cu:334-338).  Produced with
    huge but finite head weights, on the host side of the contract: no GPU fault involved."""
    _, w = weight_files("W1", 1)
    big = dict(w)
    big["head.2.weight"] = np.full((1, 128), 3e38, np.float32)
    big["head.0.bias"] = np.full(128, 10.0, np.float32)
    p = tmp_path / "overflow.weights"
    W.write_shldv(p, big)
    with binding.CudaModel(p, "fp32", max_windows=2, max_host_tokens=40) as m:
        rc, lg, err = m.classify_rc(W.synth_tokens(1, 29))
    assert rc == 0 and np.isnan(lg).all()
