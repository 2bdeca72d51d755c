"""Benchmark of the SHIELD-V sequence stack (GDN-A, GDN-B x2, SISA, head) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--mode bf16|fp16|fp32] [--batch B] [--impl reference]
    python bench.py --workload live [--participants P] [--steps HOPS] [--mode fp16]     (streaming hops, see run_live)
    python bench.py --workload encoder [--frames F] [--mode bf16]                       (frame encoder alone)
    python bench.py --workload chunked [--steps K]                                      (long-sequence kernel, B=64 T=2048)

One "step" = one pass of the whole sequence stack over B clips (20 frames x 16 tokens x 384 + readout = 321 rows per
clip) per GPU.  Default workload: B = 4096 clips per GPU, bf16 mode, synthetic N(0,1) frame embeddings and seeded
random-init weights (recipe W3 of shield_sisa_b200/weights.py); clips are sharded by batch across GPUs, no
collective on the data path (weak scaling).  Rank 0 prints one JSON line:

  value      clips/s of the whole job with tokens already resident in HBM, timed with CUDA events on the launching
             stream, max over ranks
  e2e        the same metric through the C ABI (synchronous shv_cuda_classify calls covering B clips per step) with host
             buffers: pinned tokens are DMA'd to the device and logits read back inside the timed region, every step.
             The model is loaded with max_windows = --e2e-windows (default 4096); a synchronous call is cut by the library
             into requests of an eighth of that, whose uploads overlap the kernels of the requests before them (four
             buffer sets in flight), and --e2e-threads (default 2) host threads each classify their share of the batch
             so that the queue does not drain between steps (measured: one caller 87.5k clips/s, two callers 95.4k)
  roofline   for the kernel with the largest share of the step: algorithmic bytes (or flops) per launch / its mean
             launch time, measured here with CUDA events, against the measured peak in MEASURED_PEAKS.json
  cpu_baseline  the reference's exact-FP32 CPU engine (oracle/_ref) on the host cores, on a bounded sample (N=1 only)
  extras     beside the metric (N=1 only): the exact fp32 mode at B = 128, the long-sequence kernel, and the reference's own
             CUDA engine compiled for sm_100 (oracle/_ref/gpu_kbench_ref) as a same-box GPU baseline
  live_box   streaming hops of 4096 participants per GPU over all N GPUs from ONE process through one shv_box
  encoder    beside the metric (N=1 only): frames/s of the frame encoder (Engine::encode, 512 crops resident in HBM),
             its time by kernel kind and its fraction of the HBM peak under the layer-boundary byte model

`--impl reference` times the reference's own CPU implementation of this path on all host cores (rank 0 only).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "clips_per_s_gdn_sisa_stack_b4096_t20"
UNIT = "clips/s"
NTOK, D = 321, 384
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# dram__bytes_read.sum + dram__bytes_write.sum per clip of one launch, from the ncu captures at B = 512 in the 16-bit
# modes that are summarised under profiles/ (traffic grows in proportion to the clips of a launch: every clip's tiles
# are fetched and written once); scaled to the bench's B for the `traffic` key
NCU_TRAFFIC_PER_CLIP = {"gdn_scan": (883577088 + 233556480) / 512, "gdn_inproj": (128459264 + 741220608) / 512,
                        "gdn_prep": (272559104 + 60344064) / 512}
PT_TILE_BYTES_PER_CLIP = 6 * 21 * 12416  # chunk-blocked 16-bit operand tiles and gates the fused in-projection writes
PT_QK_BYTES_PER_CLIP = 6 * 21 * (4096 + 128)    # of which the chunk preparation reads q^T, k^T, decays and betas
PT_EXT_BYTES_PER_CLIP = 6 * 21 * 1280    # and what it adds to every chunk block (T2, M, decays, norms)
PT_BYTES_PER_CLIP = PT_TILE_BYTES_PER_CLIP + PT_EXT_BYTES_PER_CLIP             # what the scan reads


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def algorithmic_work(name: str, storage_bytes: int):
    """(HBM bytes, tensor flops) per clip of one launch of kernel `name`: every tensor that crosses the kernel's
    boundary is read or written once (GEMM-boundary model; weights are L2-resident and not counted)."""
    s = storage_bytes
    h = NTOK * D * 4
    xn, on, hid = NTOK * D * s, NTOK * 768 * s, NTOK * 960 * s
    p_out = NTOK * 2316 * 4
    # SISA projection row: fp32 in the exact tier; 16-bit modes: K | V | B as fp16 + theta | alpha | forget (pitch 112) as fp32
    s_out = NTOK * 1068 * 4 if s == 4 else NTOK * (960 * 2 + 112 * 4)
    table = {
        "assemble_norm": (20 * 6144 * 4 + h + xn, 0),
        "rmsnorm": (h + xn, 0),
        "gemm.in_proj": (xn + p_out, 2 * NTOK * 2316 * 384),                       # fp32 mode
        "gdn_inproj": (xn + PT_TILE_BYTES_PER_CLIP, 2 * NTOK * 2316 * 384),        # 16-bit modes: projection + conv + SiLU + gates
        "gdn_prep": (PT_QK_BYTES_PER_CLIP + PT_EXT_BYTES_PER_CLIP, 0),            # 16-bit modes: per-chunk Gram products and inverse
        "gdn_scan": ((p_out if s == 4 else PT_BYTES_PER_CLIP) + on, 0),
        "gemm.o_proj": (on + 2 * h, 2 * NTOK * 384 * 768),
        "ffn_fused": (xn + 2 * h, 2 * NTOK * 1920 * 384 + 2 * NTOK * 384 * 960),    # 16-bit modes: up + SwiGLU + down + residual
        "gemm.ffn_up": (xn + hid, 2 * NTOK * 1920 * 384),
        "gemm.ffn_down": (hid + 2 * h, 2 * NTOK * 384 * 960),
        "gemm.sisa_in": (xn + s_out, 2 * NTOK * 1068 * 384),
        "sisa_attn": (s_out, 0),
    }
    return table.get(name, (0, 0))


# launches of one classify step in the 16-bit modes, by the names the engine's profile gives them; the readout row's two
# kernels move B rows, not 321 B: the model has 124,416 bytes per clip for them
STEP_LAUNCHES_16BIT = {"assemble_norm": 1, "gdn_inproj": 3, "gdn_prep": 3, "gdn_scan": 3, "gemm.o_proj": 3, "rmsnorm": 5,
                       "ffn_fused": 2, "gemm.sisa_in": 1, "sisa_attn": 1, "readout.qc": 1, "readout.tail": 1}
MODEL_READOUT_BYTES = 124416
MODEL_BYTES_16BIT = 37471872


def boundary_model_bytes(name: str, storage_bytes: int):
    """HBM bytes per clip of kernel `name` in the fixed GEMM-boundary model the whole-stack figure (37,471,872 B per clip
    in the 16-bit modes) is built from: each GEMM its own kernel writing an fp32 projection row P [321, 2316] per token,
    one memory-bound kernel between two GEMMs.  The 16-bit build no longer has the P boundary (the in-projection's
    epilogue writes 16-bit operand tiles), so its two mixer kernels move fewer bytes than their rows of the model; the
    model's rows are what `roofline.achieved` is quoted on, the bytes that really cross are `interface_*` beside it."""
    s = storage_bytes
    p_out = NTOK * 2316 * 4
    s_row = NTOK * 1068 * 4                   # the model's fp32 SISA projection row
    rows = {"gdn_inproj": NTOK * D * s + p_out, "gdn_scan": p_out + NTOK * 768 * s,
            "gdn_prep": 0,                        # not a kernel of the model: its work is part of the scan's row
            "gemm.sisa_in": NTOK * D * s + s_row, "sisa_attn": s_row,
            "ffn_fused": NTOK * D * s + 2 * NTOK * 960 * s + 2 * NTOK * D * 4}    # up (xn, hid) + down (hid, h read and written)
    return rows.get(name, algorithmic_work(name, storage_bytes)[0])


class ClockSampler:
    """nvidia-smi clock/throttle samples of one GPU while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows = []                      # (host time when the sample was read, fields)
        self.t0 = self.t1 = None            # the timed region, host clock
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def mark_start(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        # samples read while the timed region ran (a sample describes the 100 ms before it was read, hence the slack);
        # the sampler runs from before the warm-up steps, so a short region still has the samples around it
        rows = [r for t, r in self.rows if self.t0 is None or (self.t0 <= t <= (self.t1 or t) + 0.15)]
        if not rows and self.rows and self.t0 is not None:
            nearest = min(self.rows, key=lambda tr: abs(tr[0] - self.t0))
            rows = [nearest[1]]
        for r in rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# MobileNetV3-Large block table of the frame encoder: (in, kernel, expanded, out, squeeze-excite, stride)
_ENC_BLOCKS = [(16, 3, 16, 16, 0, 1), (16, 3, 64, 24, 0, 2), (24, 3, 72, 24, 0, 1), (24, 5, 72, 40, 1, 2), (40, 5, 120, 40, 1, 1),
               (40, 5, 120, 40, 1, 1), (40, 3, 240, 80, 0, 2), (80, 3, 200, 80, 0, 1), (80, 3, 184, 80, 0, 1), (80, 3, 184, 80, 0, 1),
               (80, 3, 480, 112, 1, 1), (112, 3, 672, 112, 1, 1), (112, 5, 672, 160, 1, 2), (160, 5, 960, 160, 1, 1),
               (160, 5, 960, 160, 1, 1)]


def encoder_work():
    """(HBM bytes, flops) per frame of the frame encoder under the layer-boundary model: float32 NHWC activations, every
    tensor that crosses a kernel boundary read or written once, weights not counted."""
    h, w = 90, 160
    nbytes = 180 * 320 * 3 + h * w * 16 * 4
    flops = 2 * h * w * 16 * 27
    for cin, k, cexp, cout, se, stride in _ENC_BLOCKS:
        hw_in = h * w
        pad = (k - 1) // 2
        h, w = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
        hw_out = h * w
        if cexp != cin:
            nbytes += hw_in * (cin + cexp) * 4
            flops += 2 * hw_in * cin * cexp
        nbytes += (hw_in + hw_out) * cexp * 4
        flops += 2 * hw_out * cexp * k * k
        if se:
            nbytes += hw_out * cexp * 4
        nbytes += hw_out * (cexp + cout) * 4 + (hw_out * cout * 4 if stride == 1 and cin == cout else 0)
        flops += 2 * hw_out * cexp * cout
    nbytes += 60 * (160 + 960) * 4 + (60 + 16) * 960 * 4 + 16 * (960 + 384) * 4
    flops += 2 * 60 * 160 * 960 + 2 * 16 * 960 * 384
    return nbytes, flops


def encoder_leg(binding, torch, wpath, mode, local_rank, frames=512, steps=10, warmup=3):
    """Frames/s of Engine::encode on crops resident in HBM (CUDA events on the launching stream, graphs on)."""
    eng = binding.EngineCore(wpath, mode, device=local_rank, max_windows=1, max_frames=frames, use_graphs=True)
    crops = torch.randint(0, 256, (frames * 172800,), dtype=torch.uint8, device="cuda")

    class _Slot:
        __cuda_array_interface__ = {"shape": (frames * 172800,), "typestr": "|u1", "data": (int(eng.frames_ptr(0)), False),
                                    "version": 2}

    torch.as_tensor(_Slot(), device="cuda").copy_(crops)
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(warmup):
        eng.encode(0, frames, stream)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        eng.encode(0, frames, stream)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    kinds = {}
    for name, t in eng.profile_encode(0, frames, stream):
        kinds[name] = kinds.get(name, 0.0) + t
    nbytes, flops = encoder_work()
    pk, pk_src = peaks()
    out = {"frames_per_s": frames / (ms / 1000.0), "frames": frames, "ms_per_encode": ms, "launches": eng.encode_launches(),
           "dtype": "f32 storage; 1x1 convolutions fp32 fma (fp32 mode) or bf16 / fp16 mma with f32 accumulation (16-bit modes)", "ms_by_kernel": kinds, "algorithmic_bytes_per_frame": nbytes, "flops_per_frame": flops,
           "hbm_frac": frames * nbytes / (ms / 1000.0) / (pk["hbm_gbs"] * 1e9), "peak_source": pk_src,
           "note": "frame encoder (MobileNetV3-Large, 320x180 crops -> 16 x 384 tokens), float32 NHWC storage in every "
                   "mode; crops resident in HBM; not part of `value`"}
    eng.close()
    del eng
    torch.cuda.empty_cache()
    # whole clips through the C ABI: uint8 crops in pinned host memory -> logits in host memory (shv_cuda_predict)
    clips = 128
    model = binding.CudaModel(wpath, mode, device=local_rank, experimental=True, max_frames=640, max_windows=64, max_host_tokens=20)
    pin = binding.PinnedBuffer(model.L, (clips, 20, 172800), np.uint8)
    pin.array[...] = np.random.default_rng(5).integers(0, 256, size=(8, 20, 172800), dtype=np.uint8).repeat(clips // 8, axis=0)
    logits = np.zeros(clips, np.float32)

    def predict():
        if model.L.shv_cuda_predict(model.m, pin.ptr, clips, logits.ctypes.data):
            raise SystemExit(binding.last_error(model.L))

    predict()
    t0 = time.perf_counter()
    for _ in range(3):
        predict()
    dt = (time.perf_counter() - t0) / 3
    if not np.isfinite(logits).all():
        raise SystemExit("predict returned non-finite logits")
    out["predict"] = {"clips_per_s": clips / dt, "frames_per_s": clips * 20 / dt, "clips": clips,
                      "h2d_bytes_per_call": clips * 20 * 172800, "d2h_bytes_per_call": clips * 4,
                      "api": "one synchronous shv_cuda_predict of 128 clips (20 uint8 crops each) from pinned host memory, "
                             "max_frames 640: four jobs of 32 clips, uploads overlapping the previous job's kernels"}
    model.close()
    pin.free()
    return out


def run_live(args, rank: int, world: int, local_rank: int):
    """Streaming load (the reference's live benchmark, bench/gpu_bench.cpp:141-218): `--participants` rings of 24 device
    token slots per box; every hop each participant sends 4 new uint8 crops and scores the window of its last 20 frames
    (one request per participant: frames + store_slots + window_slots), fp16 mode by default.  With N ranks the
    participants are placed on the GPUs by live.place_participants and every rank drives its own; there is no exchange
    between ranks.  Prints windows/s and frames/s of the whole job over `--steps` hops after the 20-frame first hop (max
    over ranks of the wall time); crops start in pinned host memory, logits end in host memory."""
    import torch
    import torch.distributed as dist

    from shield_sisa_b200 import binding, live

    torch.cuda.set_device(local_rank)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    total, new = args.participants, 4
    mine = live.place_participants([f"participant-{i}" for i in range(total)], world)[rank]
    P = len(mine)
    wpath = make_weights(f"live{rank}")
    model = binding.CudaModel(wpath, args.mode, device=local_rank, experimental=True, max_frames=min(4096, max(20, P * 20)),
                              max_windows=min(4096, max(1, P)), max_host_tokens=20, token_slots=live.RING * max(1, P))
    rng = np.random.default_rng(4)
    distinct = 64                                               # distinct crops, reused across participants and hops
    pool = binding.PinnedBuffer(model.L, (distinct, 180, 320, 3), np.uint8)
    pool.array[...] = rng.integers(0, 256, size=pool.array.shape, dtype=np.uint8)
    sent = np.zeros(P, np.int64)

    def hop(n):
        logits = np.full(P, np.nan, np.float32)
        jobs, keep = [], []
        for p in range(P):
            first = (p * 7) % (distinct - n)                    # a contiguous run of the pinned pool: DMA'd without staging
            store, window = live.hop_slots(p, int(sent[p]), n)
            j, k = model.submit(1, logits[p:p + 1], window_slots=window, frames=pool.array[first:first + n], n_frames=n,
                                store_slots=store)
            if not j:
                raise SystemExit(binding.last_error(model.L))
            jobs.append(j)
            keep.append(k)
            sent[p] += n
        sizes = []
        for j in jobs:
            if model.job_wait(j) != 0:
                raise SystemExit(model.job_error(j))
            sizes.append(model.job_timing(j)[1]["batch_windows"])
            model.job_free(j)
        if not np.isfinite(logits).all():
            raise SystemExit("live run returned non-finite logits")
        return sizes

    hop(20)
    for _ in range(max(1, args.warmup)):
        hop(new)
    barrier()
    t0 = time.perf_counter()
    sizes = []
    for _ in range(args.steps):
        sizes += hop(new)
    dt = time.perf_counter() - t0
    barrier()
    if world > 1:
        t = torch.tensor([dt], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    if rank == 0:
        emit({"metric": "windows_per_s_live_hops", "value": total * args.steps / dt, "unit": "windows/s", "n_gpus": world,
              "steps": args.steps, "warmup": max(1, args.warmup), "ms_per_step": 1000.0 * dt / args.steps,
              "higher_is_better": True, "scaling": "strong",
              "dtype": {"fp32": "f32", "bf16": "bf16", "fp16": "f16"}[args.mode], "data": "synthetic",
              "frames_per_s": total * new * args.steps / dt, "mean_batch_windows": float(np.mean(sizes)) if sizes else 0.0,
              "config": {"workload": f"live hops: {total} participants over {world} GPU(s) x (4 new 320x180 uint8 crops + 1 window "
                                     f"of 20 ring slots) per hop, one request per participant through shv_cuda_submit, "
                                     f"{args.mode} mode", "participants_rank0": P, "device_bytes_rank0": model.device_bytes()},
              "h2d_bytes_per_step": total * new * 172800, "d2h_bytes_per_step": total * 4})
    model.close()
    pool.free()
    if world > 1:
        dist.destroy_process_group()


def live_box_leg(binding, wpath, mode: str, n_devices: int, participants: int, hops: int = 3, new: int = 4):
    """Streaming hops over ALL the GPUs of the box from this one process, through one shv_box (one model per device,
    sessions placed by participant id, one request per participant per hop routed to its device; BASELINE's service-load
    configuration without the session layer).  Requests are prebuilt (the ring pattern repeats every six hops), so a hop
    costs one C call per participant.  Returns windows/s and frames/s over `hops` hops after the 20-frame first hop."""
    from shield_sisa_b200 import live
    per_dev = -(-participants // n_devices)
    cap_sessions = per_dev + per_dev // 4 + 8                    # what the box provisions per device
    box = binding.Box(wpath, mode, list(range(n_devices)), max_sessions=participants, experimental=True,
                      max_frames=min(4096, max(20, cap_sessions * 20)), max_windows=min(4096, cap_sessions), max_host_tokens=20)
    L = box.L
    drv = live.BoxLiveDriver(box, [f"participant-{i}" for i in range(participants)])
    distinct = 64
    pool = binding.PinnedBuffer(L, (distinct, 180, 320, 3), np.uint8)
    pool.array[...] = np.random.default_rng(4).integers(0, 256, size=pool.array.shape, dtype=np.uint8)
    logits = np.full(participants, np.nan, np.float32)
    C = binding.C

    def requests_for(n, frames_sent):
        out = []
        for p in range(participants):
            first = (p * 7) % (distinct - n)
            store, window = live.hop_slots(0, frames_sent, n)
            base = drv.sessions[p][1]
            out.append(binding.build_request(1, logits[p:p + 1], window_slots=window + base, frames=pool.array[first:first + n],
                                             n_frames=n, store_slots=store + base))
        return out

    def run_hop(reqs):
        jobs = [L.shv_box_submit(box.b, drv.sessions[p][0], C.byref(reqs[p][0])) for p in range(participants)]
        if not all(jobs):
            raise SystemExit(binding.last_error(L))
        for j in jobs:
            if L.shv_cuda_job_wait(j) != 0:
                raise SystemExit(L.shv_cuda_job_error(j).decode())
            L.shv_cuda_job_free(j)

    run_hop(requests_for(20, 0))
    sent = 20
    phases = []
    for h in range(6):                                            # 24 / 4: the ring positions repeat after six hops
        phases.append(requests_for(new, sent))
        sent += new
    run_hop(phases[0])                                            # warm-up hop
    t0 = time.perf_counter()
    for h in range(hops):
        run_hop(phases[(h + 1) % 6])
    dt = time.perf_counter() - t0
    ok = bool(np.isfinite(logits).all())
    per_device = [sum(1 for d, _ in drv.sessions if d == i) for i in range(n_devices)]
    box.close()
    pool.free()
    if not ok:
        raise SystemExit("box live run returned non-finite logits")
    return {"windows_per_s": participants * hops / dt, "frames_per_s": participants * new * hops / dt, "participants": participants,
            "devices": n_devices, "participants_per_device": per_device, "hops": hops, "ms_per_hop": 1000.0 * dt / hops, "mode": mode,
            "what": "one process, one shv_box over all devices: 4 new uint8 crops + 1 window of 20 ring slots per participant "
                    "and hop, one request per participant routed to its device, crops in pinned host memory"}



def make_weights(tag: str):
    from shield_sisa_b200 import weights as W
    path = Path(tempfile.gettempdir()) / f"shv_bench_{os.getuid()}_{tag}" / "w3_seed1.weights"
    if not path.exists() or not Path(str(path) + ".json").exists():
        W.synth_weight_file(path, seed=1, recipe="W3")
    return path



# ---------------------------------------------------------------------------------------------- long-sequence kernel
def chunked_case(torch, L, dk: int, steps: int, warmup: int):
    """One head-dim case of the long-sequence stress configuration: B = 64, T = 2048, H = 6, DV = 128, bf16 q / k / v
    N(0,1) seed 3 with q, k L2-normalised before rounding, log decay = logsigmoid(N(0,1)), beta = sigmoid(N(0,1)),
    scale DK^-0.5, zero initial state.  Inputs (610 / 812 MB) exceed L2, so consecutive launches need no flush."""
    B, T, H, DV = 64, 2048, 6, 128
    gen = torch.Generator(device="cuda").manual_seed(3)
    rn = lambda *shape: torch.randn(*shape, device="cuda", generator=gen)  # noqa: E731
    q, k, v = rn(B, T, H, dk), rn(B, T, H, dk), rn(B, T, H, DV)
    q = (q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6)).bfloat16()
    k = (k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)).bfloat16()
    v = v.bfloat16()
    g = torch.nn.functional.logsigmoid(rn(B, T, H))
    beta = torch.sigmoid(rn(B, T, H))
    o = torch.zeros(B, T, H, DV, device="cuda", dtype=torch.bfloat16)
    nws = L.shvk_gdn_chunked_workspace_bytes(B, T, H)
    ws = torch.empty(nws, device="cuda", dtype=torch.uint8)
    stream = torch.cuda.current_stream().cuda_stream

    def run():
        rc = L.shvk_gdn_chunked(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), o.data_ptr(), 1,
                                B, T, H, dk, DV, float(dk ** -0.5), ws.data_ptr(), nws, stream)
        if rc:
            raise SystemExit(f"shvk_gdn_chunked returned cudaError {rc}")

    for _ in range(max(3, warmup)):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if not bool(torch.isfinite(o.float()).all()):
        raise SystemExit("long-sequence kernel returned non-finite outputs")
    pk, src = peaks()
    nbytes = B * T * H * (2 * dk * 2 + DV * 2 + 8 + DV * 2)          # q, k, v in, g and beta in, o out: per token and head
    # (the kernels also move q and k a second time and 72 bytes per token and head of prepared tiles: not algorithmic)
    C = 64                                                            # flops of the chunked form at chunk 64, per chunk and head
    flops = B * (T // C) * H * (2 * C * (3 * C * dk + 2 * C * DV + 3 * dk * DV) + C * C * C // 3)
    return {"head_dim": dk, "ms": ms, "tokens_per_s": B * T / (ms / 1000.0), "algorithmic_bytes": nbytes,
            "gbs": nbytes / ms / 1e6, "hbm_frac": nbytes / ms / 1e6 / pk["hbm_gbs"], "chunked_form_flops": flops,
            "tflops": flops / ms / 1e9, "tensor_frac_of_sustained": flops / ms / 1e9 / pk["bf16_tflops_sustained"],
            "peak_source": src}


def run_chunked(args, local_rank: int):
    import torch

    from shield_sisa_b200 import binding
    torch.cuda.set_device(local_rank)
    L = binding.load_library(True)
    cases = [chunked_case(torch, L, dk, args.steps, args.warmup) for dk in (64, 128)]
    emit({"metric": "tokens_per_s_gdn_chunked_b64_t2048", "value": cases[0]["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
          "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": cases[0]["ms"], "higher_is_better": True,
          "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
          "config": {"workload": "long-sequence gated delta rule, chunked WY form: B=64, T=2048, H=6, DK=64 (value) and "
                                 "DK=128, DV=128, bf16 q/k/v, seed 3", "l2": "inputs exceed L2 (610 / 812 MB per launch)"},
          "roofline": {"bound": "hbm", "achieved": cases[0]["gbs"], "peak": peaks()[0]["hbm_gbs"], "unit": "GB/s",
                       "frac": cases[0]["hbm_frac"], "kernel": "gdn_chunked", "traffic": None},
          "gpu_launches": 4 * args.steps, "cases": cases})

# ---------------------------------------------------------------------------------------------- same-box GPU baseline
def reference_gpu_engine(wpath, mode: str, windows: int = 512):
    """The reference's own CUDA engine (its sm_80-generation kernels: mma.sync, cp.async, no TMA) compiled for sm_100
    from its sources by oracle/Makefile, timed by its own kernel benchmark (bench/gpu_kbench.cu: GPU-resident tokens,
    CUDA events, graphs on, p50 over the iterations) on `windows` windows, its compiled-in maximum.  Context beside the
    headline, not the `--impl reference` arm.  None if the binary did not travel with the tree."""
    exe = ROOT / "oracle" / "_ref" / "gpu_kbench_ref"
    if not exe.exists():
        return None
    crop = Path(tempfile.gettempdir()) / f"shv_bench_{os.getuid()}_crop.npz"
    if not crop.exists():
        np.savez(crop, frames=np.random.default_rng(6).integers(0, 256, size=(20, 180, 320, 3), dtype=np.uint8))
    try:
        r = subprocess.run([str(exe), str(wpath), mode, "--frames", "20", "--windows", str(windows), "--clips", "1", "--iters", "10",
                            "--crop", str(crop)], capture_output=True, text=True, timeout=300)
    except subprocess.TimeoutExpired:
        return {"error": "gpu_kbench did not finish within 300 s"}
    if r.returncode != 0:
        return {"error": (r.stderr or r.stdout).strip()[-300:]}
    for line in r.stdout.splitlines():
        if line.startswith("{") and '"classify"' in line:
            d = json.loads(line)
            return {"clips_per_s": d["windows_per_s"], "p50_ms": d["p50_ms"], "windows": d["windows"], "mode": mode,
                    "what": "reference CUDA engine (engine/cuda, compiled for sm_100) through its own bench/gpu_kbench: "
                            "classify on GPU-resident tokens, graphs on, p50 of 10"}
    return {"error": "no classify line in gpu_kbench output"}


# ---------------------------------------------------------------------------------------------- CPU baseline
def cpu_reference_rate(weights_path, tokens_host, budget_s: float, threads: int | None = None):
    """Windows/s of the reference CPU engine (oracle/_ref) on `threads` host threads over a bounded sample of
    `tokens_host`; falls back to the numpy port of the oracle when the compiled reference did not travel."""
    from oracle import ref_cpu, seq_oracle
    cores = os.cpu_count() or 1
    if ref_cpu.available():
        threads = min(64, threads or cores)                   # a team is capped at 64 threads by the reference API
        eng = ref_cpu.RefCpuEngine(weights_path, threads=threads)
        n0 = min(len(tokens_host), max(threads, 8))
        eng.classify(tokens_host[:n0])                        # warm-up: workspaces, page-in
        t0 = time.perf_counter()
        eng.classify(tokens_host[:n0])
        rate0 = n0 / (time.perf_counter() - t0)
        n = int(min(len(tokens_host), max(n0, rate0 * budget_s)))
        t0 = time.perf_counter()
        eng.classify(tokens_host[:n])
        dt = time.perf_counter() - t0
        isa = eng.isa
        eng.close()
        return {"value": n / dt, "unit": UNIT, "cores": threads, "kind": "reference",
                "sample": f"{n} of the workload's clips, reference engine/model exact fp32 ({isa}), {threads} threads of "
                          f"{cores} host cores, one timed call after a warm-up call, {dt:.1f} s"}
    from shield_sisa_b200 import weights as W
    w = W.read_shldv(weights_path)
    n = min(len(tokens_host), 4)
    t0 = time.perf_counter()
    seq_oracle.classify_tokens(w, tokens_host[:n], np.float32)
    dt = time.perf_counter() - t0
    return {"value": n / dt, "unit": UNIT, "cores": 1, "kind": "port",
            "sample": f"{n} clips through the numpy restatement (oracle/seq_oracle.py, float32), {dt:.1f} s"}


# ---------------------------------------------------------------------------------------------- reference arm
def run_reference(args, rank: int):
    """The reference's own CPU implementation of the path on all host cores; one step = one bounded sample."""
    if rank != 0:
        return
    from shield_sisa_b200 import weights as W
    wpath = make_weights("ref")
    cores = os.cpu_count() or 1
    sample = int(os.environ.get("SHV_BENCH_REF_SAMPLE", max(64, min(args.batch, 16 * min(cores, 64)))))
    tok = W.synth_tokens(sample, seed=2)
    from oracle import ref_cpu
    times = []
    if ref_cpu.available():
        threads = min(64, cores)
        eng = ref_cpu.RefCpuEngine(wpath, threads=threads)
        for i in range(args.warmup + args.steps):
            t0 = time.perf_counter()
            eng.classify(tok)
            if i >= args.warmup:
                times.append(time.perf_counter() - t0)
        kind, desc = "reference", f"reference engine/model exact fp32 ({eng.isa})"
        eng.close()
    else:
        from oracle import seq_oracle
        threads, sample = 1, min(sample, 4)
        w = W.read_shldv(wpath)
        for i in range(min(args.warmup, 1) + args.steps):
            t0 = time.perf_counter()
            seq_oracle.classify_tokens(w, tok[:sample], np.float32)
            if i >= min(args.warmup, 1):
                times.append(time.perf_counter() - t0)
        kind, desc = "port", "numpy restatement oracle/seq_oracle.py float32"
    ms = 1000.0 * sum(times) / len(times)
    value = sample / (ms / 1000.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"GDN+SISA sequence stack, B={args.batch} clips x 321 rows x 384, {args.mode} on the GPU arm",
                   "sample_clips_per_step": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind,
                         "sample": f"{sample} clips per step, {desc}, {threads} threads of {cores} host cores"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ---------------------------------------------------------------------------------------------- our arm
def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist

    from shield_sisa_b200 import binding

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local_rank)
    host_group = None
    if world > 1 and not dist.is_initialized():
        # NCCL writes its version banner to stdout; stdout carries the one JSON line only
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        host_group = dist.new_group(backend="gloo")      # a barrier that keeps no kernel spinning on the waiting GPUs

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # Each rank's caller threads and the library's worker threads (they inherit the mask) stay on their own cores.
    affinity = None
    if world > 1 and hasattr(os, "sched_setaffinity"):
        cores = sorted(os.sched_getaffinity(0))
        per = len(cores) // world
        if per >= 2:
            affinity = cores[local_rank * per:(local_rank + 1) * per]
            os.sched_setaffinity(0, affinity)
    B, mode = args.batch, args.mode
    storage = 4 if mode == "fp32" else 2
    wpath = make_weights(f"r{rank}")
    gen = torch.Generator(device="cuda").manual_seed(2 + rank)
    tokens = torch.randn((B, 20, 16, D), device="cuda", dtype=torch.float32, generator=gen)
    stream = torch.cuda.current_stream().cuda_stream

    # ------------------------------------------------------------ device-resident throughput
    eng = binding.EngineCore(wpath, mode, device=local_rank, max_windows=B, use_graphs=True)
    eng.bind_tokens(0, tokens.data_ptr(), B, stream)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    for _ in range(args.warmup):
        eng.classify(0, B, stream)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if sampler:
        sampler.mark_start()
    ev0.record()
    for _ in range(args.steps):
        eng.classify(0, B, stream)
    ev1.record()
    barrier()
    if sampler:
        sampler.mark_end()
    ms_step = max_over_ranks(ev0.elapsed_time(ev1) / args.steps)
    clocks = sampler.stop() if sampler else None
    if eng.status() != 0:
        raise SystemExit(f"device status word {eng.status()}: a tensor-core kernel gave up waiting")
    value = world * B / (ms_step / 1000.0)

    # ------------------------------------------------------------ per-kernel times (CUDA events after every launch)
    totals, counts = {}, {}
    reps = 3
    for _ in range(reps):
        for name, ms in eng.profile(0, B, stream):
            totals[name] = totals.get(name, 0.0) + ms
            counts[name] = counts.get(name, 0) + 1
    step_ms_eager = sum(totals.values()) / reps
    pk, pk_src = peaks()
    kernels = {}
    for name, tot in totals.items():
        avg = tot / counts[name]
        nbytes, flops = algorithmic_work(name, storage)
        kernels[name] = {"launches_per_step": counts[name] // reps, "avg_ms": avg, "share": tot / reps / step_ms_eager,
                         "gbs": B * nbytes / avg / 1e6 if nbytes else None,
                         "tflops": B * flops / avg / 1e9 if flops else None}
    top = max(totals, key=totals.get)
    k = kernels[top]
    nbytes, flops = algorithmic_work(top, storage)
    model_bytes = boundary_model_bytes(top, storage)
    t_hbm = B * model_bytes / (pk["hbm_gbs"] * 1e9)
    t_tensor = B * flops / (pk["bf16_tflops_sustained"] * 1e12)
    if flops and t_tensor > t_hbm:
        roof = {"bound": "tensor", "achieved": k["tflops"], "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                "frac": k["tflops"] / pk["bf16_tflops_sustained"]}
    else:
        model_gbs = B * model_bytes / k["avg_ms"] / 1e6
        roof = {"bound": "hbm", "achieved": model_gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": model_gbs / pk["hbm_gbs"]}
    has_traffic = storage == 2 and top in NCU_TRAFFIC_PER_CLIP
    roof.update({"kernel": top, "peak_source": pk_src, "share_of_step": k["share"], "avg_launch_ms": k["avg_ms"],
                 "algorithmic_bytes_per_launch": B * model_bytes,
                 "interface_bytes_per_launch": B * nbytes, "interface_gbs": k["gbs"],
                 "interface_frac": k["gbs"] / pk["hbm_gbs"] if k["gbs"] else None,
                 "removed_boundary": ("fp32 projection row P [321 x 2316] between in-projection and scan: the model counts it "
                                      "written and read once, this build stores 16-bit operand tiles (1,564,416 B per clip) instead")
                 if model_bytes != nbytes and top.startswith("gdn_") else None,
                 "traffic": B * NCU_TRAFFIC_PER_CLIP[top] if has_traffic else None,
                 "traffic_source": "ncu capture at B = 512 (profiles/), scaled by clips" if has_traffic else None})
    # ------------------------------------------------------------ cycle counters of a development build (--dev-cycles)
    dev_cycles = None
    if args.dev_cycles and storage == 2:
        import ctypes as C
        L = binding.load_library(True)
        try:
            f_in, f_sc = L.shvk_dev_inproj_cycles, L.shvk_dev_scan_cycles
        except AttributeError:
            raise SystemExit("--dev-cycles needs the development build: python -m shield_sisa_b200.build --dev-probes")
        b_in, b_sc = (C.c_ulonglong * 88)(), (C.c_ulonglong * 32)()
        for f, b in ((f_in, b_in), (f_sc, b_sc)):
            f.argtypes, f.restype = [C.c_void_p], C.c_int
            f(b)                                          # discard what the steps above accumulated
        eng.classify(0, B, stream)
        torch.cuda.synchronize()
        f_in(b_in)
        f_sc(b_sc)

        def shares(buf, w, names, total=None):
            v = [buf[w * 8 + k] for k in range(8)]
            tot = float(v[total] if total is not None else sum(v)) or 1.0
            return {n: round(v[k] / tot, 3) for k, n in names}

        dev_cycles = {
            "note": "share of each role's cycles, one CTA (in-projection) / one CTA in 61 (scan), three launches each",
            "gdn_inproj": {
                "w_producer": shares(b_in, 0, [(0, "wait_free_stage")], 7),
                "mma_thread": shares(b_in, 1, [(0, "wait_drained_accumulator"), (1, "wait_weight_stage"), (2, "wait_token_tile")], 7),
                **{f"epilogue_warp_{w}": shares(b_in, w, [(0, "wait_full_accumulator"), (1, "first_tmem_load"),
                                                          (2, "later_tmem_loads"), (3, "tile_total")], 7) for w in range(3, 11)}},
            "gdn_scan_t": {f"warp_{w}": shares(b_sc, w, [(0, "until_block_landed"), (1, "deferred_norm"), (2, "r_and_qs"), (3, "u_and_o"),
                                                         (4, "state_update"), (5, "sum_of_squares"), (6, "barrier")]) for w in range(4)}}
        print(json.dumps(dev_cycles, indent=1), file=sys.stderr)
    alg_bytes_clip = 45853824 if mode == "fp32" else MODEL_BYTES_16BIT
    stack_frac = B * alg_bytes_clip / (ms_step / 1000.0) / (pk["hbm_gbs"] * 1e9)
    launches = eng.launches() * args.steps * world
    eng.close()
    del eng
    torch.cuda.empty_cache()

    # ------------------------------------------------------------ frame encoder beside it (rank 0, N = 1; not in `value`)
    encoder = None
    if rank == 0 and world == 1 and not args.no_encoder:
        encoder = encoder_leg(binding, torch, wpath, mode, local_rank)
        torch.cuda.empty_cache()

    # ------------------------------------------------------------ end to end through the C ABI with host buffers
    e2e = None
    if B <= 4096 and not args.no_e2e:
        mw = max(1, min(B, args.e2e_windows))
        model = binding.CudaModel(wpath, mode, device=local_rank, experimental=True, max_windows=mw,
                                  max_host_tokens=20 * mw, max_frames=1)
        pin = binding.PinnedBuffer(model.L, (B, 20, 16, D))
        pin.array[...] = tokens.cpu().numpy()
        out = np.empty(B, np.float32)
        # Callers: `nthr` host threads, each classifying its own contiguous share of the B clips with one synchronous
        # call per step (the C ABI is thread-safe on one model).  With more than one caller the scheduler's queue does
        # not drain between steps, so the upload of a call's first job overlaps the previous call's last kernels.
        nthr = max(1, min(args.e2e_threads, B))
        cuts = [B * i // nthr for i in range(nthr + 1)]

        def caller(i, n_steps, errs):
            lo, hi = cuts[i], cuts[i + 1]
            try:
                for _ in range(n_steps):
                    model.classify(pin.array[lo:hi], out[lo:hi])
            except Exception as e:                      # surfaced after the join
                errs.append(e)

        def run_steps(n_steps):
            errs = []
            if nthr == 1:
                caller(0, n_steps, errs)
            else:
                ts = [threading.Thread(target=caller, args=(i, n_steps, errs)) for i in range(nthr)]
                for th in ts:
                    th.start()
                for th in ts:
                    th.join()
            if errs:
                raise errs[0]

        run_steps(max(1, min(args.warmup, 3)))
        barrier()
        t0 = time.perf_counter()
        run_steps(args.steps)
        dt = time.perf_counter() - t0
        barrier()
        e2e_ms = max_over_ranks(1000.0 * dt / args.steps)
        # The uploads alone: the same pinned buffer in the same request-sized pieces to the device, no kernels, all ranks
        # at once.  What this rate leaves of the end-to-end rate is the host path (PCIe, host memory), not the engine.
        piece = max(1, model.limits()["max_windows"] // 8)
        src = torch.from_numpy(pin.array)
        dst = torch.empty((piece, 20, 16, D), device="cuda", dtype=torch.float32)
        copy_stream = torch.cuda.Stream()

        def upload_steps(n_steps):
            with torch.cuda.stream(copy_stream):
                for _ in range(n_steps):
                    for lo in range(0, B, piece):
                        hi = min(B, lo + piece)
                        dst[: hi - lo].copy_(src[lo:hi], non_blocking=True)
            copy_stream.synchronize()

        upload_steps(1)
        barrier()
        t0 = time.perf_counter()
        upload_steps(args.steps)
        h2d_ms = max_over_ranks(1000.0 * (time.perf_counter() - t0) / args.steps)
        barrier()
        del dst
        if not np.isfinite(out).all():
            raise SystemExit("end-to-end run returned non-finite logits")
        # Beside it (an extra key, never the headline): the same calls with the tokens handed over as fp16 through the
        # extension shv_cuda_b200_classify_f16, half the bytes to upload.  The reference's ABI fixes fp32 tokens; this shows
        # what the end-to-end rate is when the host's upload bandwidth is shared by fewer bytes.
        f16 = None
        if mode != "fp32":
            pin16 = binding.PinnedBuffer(model.L, (B, 20, 16, D), np.float16)
            pin16.array[...] = pin.array
            out16 = np.empty(B, np.float32)

            def caller16(i, n_steps, errs):
                lo, hi = cuts[i], cuts[i + 1]
                try:
                    for _ in range(n_steps):
                        model.classify_f16(pin16.array[lo:hi], out16[lo:hi])
                except Exception as e:
                    errs.append(e)

            def run16(n_steps):
                errs = []
                ts = [threading.Thread(target=caller16, args=(i, n_steps, errs)) for i in range(nthr)]
                for th in ts:
                    th.start()
                for th in ts:
                    th.join()
                if errs:
                    raise errs[0]

            run16(max(1, min(args.warmup, 3)))
            barrier()
            t0 = time.perf_counter()
            run16(args.steps)
            ms16 = max_over_ranks(1000.0 * (time.perf_counter() - t0) / args.steps)
            barrier()
            if not np.isfinite(out16).all():
                raise SystemExit("end-to-end run with fp16 tokens returned non-finite logits")
            f16 = {"value": world * B / (ms16 / 1000.0), "unit": UNIT, "ms_per_step": ms16,
                   "h2d_bytes_per_step": B * 20 * 6144 * 2 + B * 20 * 8, "d2h_bytes_per_step": B * 4,
                   "max_abs_logit_change": float(np.abs(out16 - out).max()),
                   "api": "the same callers through shv_cuda_b200_classify_f16 (extension: fp16 host tokens, widened on the device)"}
            pin16.free()
        e2e = {"value": world * B / (e2e_ms / 1000.0), "unit": UNIT, "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": B * 20 * 6144 * 4 + B * 20 * 8, "d2h_bytes_per_step": B * 4,
               "h2d_only": {"ms_per_step": h2d_ms, "gbs_per_rank": B * 20 * 6144 * 4 / h2d_ms / 1e6, "pinned": bool(src.is_pinned()),
                            "clips_per_s_if_upload_bound": world * B / (h2d_ms / 1000.0),
                            "note": "the step's token uploads alone (same pinned buffer, same piece size, no kernels), all "
                                    "ranks at once, max over ranks"},
               "api": "%d host thread(s), each one synchronous shv_cuda_classify of its B/%d clips per step; pinned host "
                      "tokens (shv_cuda_host_alloc), max_windows = %d" % (nthr, nthr, mw),
               "f16_tokens": f16}
        model.close()
        pin.free()

    # ------------------------------------------------------------ extra keys beside it (rank 0, N = 1; not in `value`)
    extras = None
    if rank == 0 and world == 1 and not args.no_extras:
        extras = {}
        # the exact tier's configuration: B = 128 clips, fp32 mode, tokens resident in HBM
        b2 = 128
        eng2 = binding.EngineCore(wpath, "fp32", device=local_rank, max_windows=b2, use_graphs=True)
        eng2.bind_tokens(0, tokens.data_ptr(), b2, stream)
        for _ in range(3):
            eng2.classify(0, b2, stream)
        torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(5):
            eng2.classify(0, b2, stream)
        a1.record()
        torch.cuda.synchronize()
        ms2 = a0.elapsed_time(a1) / 5
        extras["exact_fp32_b128"] = {"clips_per_s": b2 / (ms2 / 1000.0), "ms_per_step": ms2, "batch": b2, "dtype": "f32",
                                     "note": "GDN+SISA stack in the exact fp32 mode at B = 128, tokens resident in HBM"}
        eng2.close()
        del eng2
        torch.cuda.empty_cache()
        extras["gdn_chunked_b64_t2048"] = [chunked_case(torch, binding.load_library(True), dk, 5, 3) for dk in (64, 128)]
        torch.cuda.empty_cache()
        extras["gpu_baseline"] = reference_gpu_engine(wpath, mode if mode != "fp32" else "fp32")

    # ------------------------------------------------------------ the whole box from one process (rank 0; the others idle)
    live_box = None
    if not args.no_extras and torch.cuda.device_count() >= world:
        if host_group is not None:
            dist.barrier(group=host_group)
        if rank == 0:
            try:
                live_box = live_box_leg(binding, wpath, "fp16", world, 4096 * world)
            except (RuntimeError, SystemExit) as e:          # reported, never fatal for the headline
                live_box = {"error": str(e)[-300:]}
        if host_group is not None:
            dist.barrier(group=host_group)

    # ------------------------------------------------------------ CPU baseline beside it (rank 0, N = 1)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        n = min(B, 2048)
        cpu = cpu_reference_rate(wpath, tokens[:n].cpu().numpy(), budget_s=float(os.environ.get("SHV_BENCH_CPU_SECONDS", 15)))

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": {"fp32": "f32", "bf16": "bf16", "fp16": "f16"}[mode], "data": "synthetic",
            "config": {"workload": f"GDN+SISA sequence stack, B={B} clips per GPU x 321 rows x 384 (20 frames x 16 tokens + "
                                   f"readout), {mode} mode, weights W3 seed 1, tokens N(0,1)",
                       "l2": "inputs and activations exceed L2 (tokens 2 GB, activation arena ~20 GB per step)",
                       "graphs": True, "sharding": f"{world} x {B} clips by batch, no collective",
                       "host_cores_per_rank": len(affinity) if affinity else None},
            "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "roofline": roof, "cpu_baseline": cpu,
            "stack_hbm_fraction": {"algorithmic_bytes_per_clip": alg_bytes_clip, "frac": stack_frac,
                                   "note": "whole stack against the GEMM-boundary byte model and the measured HBM peak"},
            "kernels": kernels, "encoder": encoder, "extras": extras, "live_box": live_box,
            **({"dev_cycles": dev_cycles} if dev_cycles else {}),
        }
        emit(line)
    if world > 1:
        dist.destroy_process_group()


RESULT_FD = None     # a duplicate of the real stdout, kept for the one JSON line


def emit(line: dict):
    data = (json.dumps(line) + "\n").encode()
    os.write(RESULT_FD if RESULT_FD is not None else 1, data)


def main():
    # stdout carries the one JSON line only: everything else a library may print there (NCCL's version banner, for
    # one) is sent to stderr for the whole run
    global RESULT_FD
    sys.stdout.flush()
    RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="bf16", choices=["fp32", "bf16", "fp16"])
    ap.add_argument("--batch", type=int, default=4096)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-encoder", action="store_true", help="skip the frame-encoder leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (small cases for profiling)")
    ap.add_argument("--dev-cycles", action="store_true",
                    help="development build only (python -m shield_sisa_b200.build --dev-probes): print the per-role cycle counters "
                         "of the in-projection and the scan; the timings of such a run are not bench values")
    ap.add_argument("--no-extras", action="store_true", help="skip the extra keys (exact-tier B = 128 line, long-sequence kernel)")
    ap.add_argument("--workload", default="stack", choices=["stack", "live", "encoder", "chunked"],
                    help="stack: the headline metric (default); live: streaming hops with frames and device token rings; "
                         "encoder: the frame-encoder leg alone on --frames crops (small cases for profiling); "
                         "chunked: the long-sequence gated delta rule (B = 64, T = 2048, bf16, head dim 64 and 128)")
    ap.add_argument("--frames", type=int, default=512, help="crops per encode of the encoder workload")
    ap.add_argument("--participants", type=int, default=4096, help="participants of the live workload")
    ap.add_argument("--e2e-threads", type=int, default=2,
                    help="host threads of the end-to-end leg, each calling shv_cuda_classify on its share of the batch")
    ap.add_argument("--e2e-windows", type=int, default=4096,
                    help="scheduler option max_windows of the end-to-end leg (a synchronous call travels as requests of an "
                         "eighth of it, uploads overlapping kernels)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.workload == "encoder":
        import torch

        from shield_sisa_b200 import binding
        torch.cuda.set_device(local_rank)
        enc = encoder_leg(binding, torch, make_weights("enc"), args.mode, local_rank, frames=args.frames, steps=args.steps,
                          warmup=args.warmup)
        emit({"metric": "frames_per_s_encoder", "value": enc["frames_per_s"], "unit": "frames/s", "n_gpus": 1,
              "steps": args.steps, "warmup": args.warmup, "ms_per_step": enc["ms_per_encode"], "higher_is_better": True,
              "dtype": {"fp32": "f32", "bf16": "bf16", "fp16": "f16"}[args.mode], "data": "synthetic",
              "config": {"workload": f"frame encoder, {args.frames} crops per encode, {args.mode} mode"}, "encoder": enc})
        return
    if args.workload == "live":
        run_live(args, rank, world, local_rank)
        return
    if args.workload == "chunked":
        if rank == 0:
            run_chunked(args, local_rank)
        return
    if world != args.gpus:
        if args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
