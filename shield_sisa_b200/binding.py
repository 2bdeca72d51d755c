"""ctypes binding of libshield_v_cuda.so: the C ABI of include/shv_cuda.h, the engine-core and kernel launch layers.

`CudaModel` mirrors the reference's Python wrapper of its CPU library (bench/cpu_engine.py: load, classify, close)
for the CUDA ABI, so parity tests read like the reference's own.  Nothing here computes: a missing library raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

LIB_DIR = Path(__file__).resolve().parent / "lib"
FRAME_BYTES = 172800
TOKEN_FLOATS = 6144
DTYPES = {"fp32": 0, "bf16": 1, "fp16": 2}


class Options(C.Structure):
    _fields_ = [("max_frames", C.c_int), ("max_windows", C.c_int), ("max_host_tokens", C.c_int),
                ("token_slots", C.c_int), ("use_graphs", C.c_int), ("max_delay_us", C.c_int)]


CALLBACK = C.CFUNCTYPE(None, C.c_void_p, C.c_int, C.c_void_p)


class Request(C.Structure):
    _fields_ = [("frames", C.c_void_p), ("n_frames", C.c_size_t), ("tokens_out", C.c_void_p),
                ("store_slots", C.POINTER(C.c_int32)), ("n_windows", C.c_size_t),
                ("window_frames", C.POINTER(C.c_int32)), ("window_slots", C.POINTER(C.c_int32)),
                ("window_tokens", C.POINTER(C.c_void_p)), ("logits_out", C.c_void_p), ("callback", CALLBACK),
                ("user", C.c_void_p)]


class GemmArgs(C.Structure):
    _fields_ = [("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("A", C.c_void_p), ("lda", C.c_longlong),
                ("W", C.c_void_p), ("ldw", C.c_longlong), ("C", C.c_void_p), ("ldc", C.c_longlong),
                ("c_dtype", C.c_int), ("bias", C.c_void_p), ("act", C.c_int), ("R", C.c_void_p),
                ("ldr", C.c_longlong), ("r_div", C.c_float), ("swiglu", C.c_int)]


class ReadoutWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("wo_t", "ffn_norm_w", "up_t", "down_t", "final_norm_w", "head_w0_t", "head_b0",
                                          "head_w2", "head_b2")]


LOAD_FN = C.CFUNCTYPE(C.c_void_p, C.c_char_p, C.c_char_p, C.c_int, C.POINTER(Options))
FREE_FN = C.CFUNCTYPE(None, C.c_void_p)
SUBMIT_FN = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.POINTER(Request))
CLASSIFY_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p)
ERROR_FN = C.CFUNCTYPE(C.c_char_p)


class BoxOps(C.Structure):
    """shv_box_ops: the entry points a box reaches its per-device models through."""
    _fields_ = [("load_ex", LOAD_FN), ("free_model", FREE_FN), ("submit", SUBMIT_FN), ("classify", CLASSIFY_FN),
                ("last_error", ERROR_FN)]


_libs: dict[bool, C.CDLL] = {}


def library_path(experimental: bool = True) -> Path:
    return LIB_DIR / ("libshield_v_cuda_experimental.so" if experimental else "libshield_v_cuda.so")


def load_library(experimental: bool = True) -> C.CDLL:
    """The native library (strict, or the variant that loads 16-bit modes without a certificate)."""
    if experimental in _libs:
        return _libs[experimental]
    path = library_path(experimental)
    if not path.exists():
        raise RuntimeError(f"{path} is missing: build it with `python -m shield_sisa_b200.build` "
                           "(there is no fallback implementation)")
    L = C.CDLL(str(path))
    vp, sz, i32 = C.c_void_p, C.c_size_t, C.c_int
    sig = {
        "shv_cuda_default_options": (None, [C.POINTER(Options)]),
        "shv_cuda_load": (vp, [C.c_char_p, C.c_char_p, i32]),
        "shv_cuda_load_ex": (vp, [C.c_char_p, C.c_char_p, i32, C.POINTER(Options)]),
        "shv_cuda_free": (None, [vp]),
        "shv_cuda_last_error": (C.c_char_p, []),
        "shv_cuda_mode": (C.c_char_p, [vp]),
        "shv_cuda_fingerprint": (C.c_char_p, [vp]),
        "shv_cuda_threshold": (C.c_double, [vp]),
        "shv_cuda_compute_revision": (C.c_char_p, []),
        "shv_cuda_limits": (i32, [vp] + [C.POINTER(i32)] * 4),
        "shv_cuda_weight_bytes": (sz, [vp]),
        "shv_cuda_device_bytes": (sz, [vp]),
        "shv_cuda_encode_frames": (i32, [vp, vp, sz, vp]),
        "shv_cuda_classify": (i32, [vp, vp, sz, vp]),
        "shv_cuda_predict": (i32, [vp, vp, sz, vp]),
        "shv_cuda_submit": (vp, [vp, C.POINTER(Request)]),
        "shv_cuda_job_status": (i32, [vp]),
        "shv_cuda_job_wait": (i32, [vp]),
        "shv_cuda_job_error": (C.c_char_p, [vp]),
        "shv_cuda_job_timing": (i32, [vp] + [C.POINTER(C.c_double)] * 3 + [C.POINTER(i32)] * 2),
        "shv_cuda_job_free": (None, [vp]),
        "shv_cuda_host_alloc": (vp, [sz]),
        "shv_cuda_host_free": (None, [vp]),
        "shv_cuda_b200_upload_tokens": (i32, [vp, vp, sz, vp]),
        "shv_cuda_b200_classify_f16": (i32, [vp, vp, sz, vp]),
        "shv_cuda_b200_launches_per_batch": (i32, [vp]),
        "shv_cuda_b200_test_starve": (i32, [vp, i32, i32]),
        "shv_box_load": (vp, [C.c_char_p, C.c_char_p, C.POINTER(i32), i32, C.POINTER(Options), i32]),
        "shv_box_load_with": (vp, [C.POINTER(BoxOps), C.c_char_p, C.c_char_p, C.POINTER(i32), i32, C.POINTER(Options), i32]),
        "shv_box_free": (None, [vp]),
        "shv_box_devices": (i32, [vp]),
        "shv_box_model": (vp, [vp, i32]),
        "shv_box_home_device": (i32, [vp, C.c_char_p]),
        "shv_box_session_open": (i32, [vp, C.c_char_p, C.POINTER(i32), C.POINTER(i32)]),
        "shv_box_session_close": (i32, [vp, i32, i32]),
        "shv_box_free_sessions": (i32, [vp, i32]),
        "shv_box_submit": (vp, [vp, i32, C.POINTER(Request)]),
        "shv_box_classify": (i32, [vp, vp, sz, vp]),
        "shvb_engine_create": (vp, [C.c_char_p, C.c_char_p, i32, i32, i32]),
        "shvb_engine_create_ex": (vp, [C.c_char_p, C.c_char_p, i32, i32, i32, i32]),
        "shvb_engine_destroy": (None, [vp]),
        "shvb_engine_frames": (vp, [vp, i32]),
        "shvb_engine_tokens": (vp, [vp, i32]),
        "shvb_engine_encode": (i32, [vp, i32, i32, vp]),
        "shvb_engine_frame_bucket": (i32, [vp, i32]),
        "shvb_engine_encode_launches": (i32, [vp]),
        "shvb_engine_profile_encode": (i32, [vp, i32, i32, vp, vp, i32, C.c_char_p, i32]),
        "shvb_engine_bind_tokens": (i32, [vp, i32, vp, i32, vp]),
        "shvb_engine_classify": (i32, [vp, i32, i32, vp]),
        "shvb_engine_logits": (vp, [vp, i32]),
        "shvb_engine_read_logits": (i32, [vp, i32, vp, i32, vp]),
        "shvb_engine_window_bucket": (i32, [vp, i32]),
        "shvb_engine_launches": (i32, [vp]),
        "shvb_engine_status": (i32, [vp]),
        "shvb_engine_test_starve": (i32, [vp, i32, i32]),
        "shvb_engine_bytes": (sz, [vp, i32]),
        "shvb_engine_set_dump_dir": (i32, [vp, C.c_char_p]),
        "shvb_engine_profile": (i32, [vp, i32, i32, vp, vp, i32, C.c_char_p, i32]),
        "shvk_assemble_norm": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, vp]),
        "shvk_rmsnorm": (i32, [vp, C.c_longlong, vp, vp, i32, C.c_longlong, i32, vp]),
        "shvk_gemm_f32": (i32, [C.POINTER(GemmArgs), vp]),
        "shvk_gemm_tc_plan": (i32, [C.POINTER(GemmArgs), i32, vp]),
        "shvk_gemm_tc_plan_split16": (i32, [C.POINTER(GemmArgs), i32, i32, vp, C.c_longlong, vp]),
        "shvk_gemm_tc": (i32, [vp, vp]),
        "shvk_gemm_tc_rows": (i32, [vp, i32, vp]),
        "shvk_gemm_tc_status": (i32, [C.POINTER(i32)]),
        "shvk_gemm_tc_rows_starved": (i32, [vp, i32, i32, vp]),
        "shvk_status_fetch_async": (i32, [vp, vp]),
        "shvk_status_clear_async": (i32, [vp]),
        "shvk_gdn_inproj_rows": (i32, []),
        "shvk_gdn_inproj_row_order": (None, [vp]),
        "shvk_gdn_pt_bytes": (sz, [i32]),
        "shvk_gdn_inproj_plan": (i32, [vp, C.c_longlong, vp, vp, vp, vp, vp, vp, i32, vp]),
        "shvk_gdn_inproj": (i32, [vp, i32, vp]),
        "shvk_gdn_chunk_prep": (i32, [vp, i32, i32, vp]),
        "shvk_gdn_scan_t": (i32, [vp, vp, vp, i32, i32, vp]),
        "shvk_gdn_scan_t_starved": (i32, [vp, vp, vp, i32, i32, i32, vp]),
        "shvk_gdn_scan": (i32, [vp, vp, vp, vp, vp, vp, vp, i32, i32, vp]),
        "shvk_gdn_scan_status": (i32, [C.POINTER(i32)]),
        "shvk_gdn_chunked_workspace_bytes": (sz, [i32, i32, i32]),
        "shvk_gdn_chunked": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, C.c_float, vp, sz, vp]),
        "shvk_sisa_attn": (i32, [vp, vp, vp, vp, i32, vp]),
        "shvk_sisa_attn_h16": (i32, [vp, vp, vp, vp, vp, i32, vp]),
        "shvk_readout_qc": (i32, [vp, C.c_longlong, vp, vp, vp, i32, vp]),
        "shvk_readout_tail": (i32, [vp, vp, C.c_longlong, C.POINTER(ReadoutWeights), vp, vp, i32, vp]),
        "shvk_store_tokens": (i32, [vp, vp, vp, i32, vp]),
        "shvk_ffn_fused_plan": (i32, [vp, C.c_longlong, vp, vp, vp, i32, vp]),
        "shvk_ffn_fused": (i32, [vp, i32, vp]),
        "shvk_ffn_fused_starved": (i32, [vp, i32, i32, vp]),
        "shvk_gdn_inproj_starved": (i32, [vp, i32, i32, vp]),
        "shvk_expand_f16_tokens": (i32, [vp, i32, vp]),
        "shvk_split_tf32": (i32, [vp, C.c_longlong, i32, C.c_longlong, vp, C.c_longlong, i32, vp]),
        "shvk_cnn_stem": (i32, [vp, vp, vp, vp, vp, i32, vp]),
        "shvk_cnn_depthwise": (i32, [vp, vp, vp, vp] + [i32] * 9 + [vp]),
        "shvk_cnn_se_partial_floats": (sz, [i32, i32, i32]),
        "shvk_cnn_se_gate": (i32, [vp] * 7 + [i32] * 4 + [vp]),
        "shvk_cnn_se_gate_static": (i32, [vp] * 6 + [i32] * 4 + [vp]),
        "shvk_cnn_pointwise": (i32, [vp, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, vp]),
        "shvk_cnn_pointwise_tf32": (i32, [vp, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, vp]),
        "shvk_cnn_pointwise_h": (i32, [vp, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, i32, vp]),
        "shvk_cnn_pool_tokens": (i32, [vp, vp, i32, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _libs[experimental] = L
    return L


def last_error(L) -> str:
    return (L.shv_cuda_last_error() or b"").decode()


class PinnedBuffer:
    """Host memory from shv_cuda_host_alloc viewed as a numpy array (DMA'd without a staging copy)."""

    def __init__(self, L, shape, dtype=np.float32):
        self.L = L
        nbytes = int(np.prod(shape)) * np.dtype(dtype).itemsize
        self.ptr = L.shv_cuda_host_alloc(nbytes)
        if not self.ptr:
            raise RuntimeError(last_error(L))
        buf = (C.c_char * nbytes).from_address(self.ptr)
        self.array = np.frombuffer(buf, dtype=dtype).reshape(shape)

    def free(self):
        if self.ptr:
            self.array = None
            self.L.shv_cuda_host_free(self.ptr)
            self.ptr = None


def build_request(n_windows, logits_out, window_tokens=None, window_slots=None, window_frames=None, callback=None,
                  frames=None, n_frames=0, tokens_out=None, store_slots=None):
    """A filled shv_cuda_request and the list of objects that must stay alive until the job completes."""
    req = Request()
    keep = [logits_out]
    req.n_windows = n_windows
    req.logits_out = logits_out.ctypes.data if logits_out is not None else None
    if window_tokens is not None:
        arr = (C.c_void_p * len(window_tokens))(*[None if a is None else a.ctypes.data for a in window_tokens])
        req.window_tokens = C.cast(arr, C.POINTER(C.c_void_p))
        keep += [arr, window_tokens]
    for name, val in (("window_slots", window_slots), ("window_frames", window_frames)):
        if val is not None:
            a = np.ascontiguousarray(val, dtype=np.int32)
            setattr(req, name, a.ctypes.data_as(C.POINTER(C.c_int32)))
            keep.append(a)
    if frames is not None:
        req.frames = frames.ctypes.data
        keep.append(frames)
    req.n_frames = n_frames
    if tokens_out is not None:
        req.tokens_out = tokens_out.ctypes.data
        keep.append(tokens_out)
    if store_slots is not None:
        a = np.ascontiguousarray(store_slots, dtype=np.int32)
        req.store_slots = a.ctypes.data_as(C.POINTER(C.c_int32))
        keep.append(a)
    if callback is not None:
        cb = CALLBACK(callback)
        req.callback = cb
        keep.append(cb)
    return req, keep


class CudaModel:
    """shv_cuda_load_ex / classify / submit / free of one model on one device."""

    def __init__(self, weights, mode="fp32", device=0, experimental=True, **options):
        self.L = load_library(experimental)
        opt = Options()
        self.L.shv_cuda_default_options(C.byref(opt))
        for k, v in options.items():
            if not hasattr(opt, k):
                raise TypeError(f"unknown option {k}")
            setattr(opt, k, int(v))
        self.m = self.L.shv_cuda_load_ex(str(weights).encode(), mode.encode() if mode is not None else None, int(device),
                                         C.byref(opt))
        if not self.m:
            raise RuntimeError(last_error(self.L))

    # ---- queries
    @property
    def mode(self):
        return self.L.shv_cuda_mode(self.m).decode()

    @property
    def fingerprint(self):
        return self.L.shv_cuda_fingerprint(self.m).decode()

    @property
    def threshold(self):
        return self.L.shv_cuda_threshold(self.m)

    def limits(self):
        v = [C.c_int() for _ in range(4)]
        if self.L.shv_cuda_limits(self.m, *[C.byref(x) for x in v]):
            raise RuntimeError(last_error(self.L))
        return dict(zip(("max_frames", "max_windows", "max_host_tokens", "token_slots"), (x.value for x in v)))

    def device_bytes(self):
        return self.L.shv_cuda_device_bytes(self.m)

    def weight_bytes(self):
        return self.L.shv_cuda_weight_bytes(self.m)

    def launches_per_batch(self):
        return self.L.shv_cuda_b200_launches_per_batch(self.m)

    def test_starve(self, kind, batches=1):
        """Test hook of the experimental library: the next GPU batches starve one launch (1 GEMM, 2 scan)."""
        if self.L.shv_cuda_b200_test_starve(self.m, kind, batches):
            raise RuntimeError(last_error(self.L))

    # ---- synchronous
    def classify(self, tokens, out=None):
        """tokens [b,20,16,384] float32 (numpy, possibly a PinnedBuffer array) -> logits [b] float32."""
        t = np.ascontiguousarray(tokens, dtype=np.float32)
        if t.ndim != 4 or t.shape[1:] != (20, 16, 384):
            raise ValueError("expected [b,20,16,384] float32 tokens")
        out = np.empty(t.shape[0], np.float32) if out is None else out
        rc = self.L.shv_cuda_classify(self.m, t.ctypes.data, t.shape[0], out.ctypes.data)
        if rc:
            raise RuntimeError(last_error(self.L))
        return out

    def classify_f16(self, tokens_f16, out=None):
        """tokens [b,20,16,384] float16 (numpy, possibly a PinnedBuffer array) -> logits [b] float32
        (shv_cuda_b200_classify_f16: half the bytes to upload)."""
        t = np.ascontiguousarray(tokens_f16, dtype=np.float16)
        if t.ndim != 4 or t.shape[1:] != (20, 16, 384):
            raise ValueError("expected [b,20,16,384] float16 tokens")
        out = np.empty(t.shape[0], np.float32) if out is None else out
        if self.L.shv_cuda_b200_classify_f16(self.m, t.ctypes.data, t.shape[0], out.ctypes.data):
            raise RuntimeError(last_error(self.L))
        return out

    def encode_frames(self, frames):
        """uint8 crops [n,180,320,3] -> tokens [n,16,384] (shv_cuda_encode_frames)."""
        f = np.ascontiguousarray(frames, dtype=np.uint8).reshape(-1, FRAME_BYTES)
        out = np.zeros((f.shape[0], 16, 384), np.float32)
        if self.L.shv_cuda_encode_frames(self.m, f.ctypes.data, f.shape[0], out.ctypes.data):
            raise RuntimeError(last_error(self.L))
        return out

    def predict(self, clips):
        """uint8 clips [b,20,180,320,3] -> logits [b] (shv_cuda_predict)."""
        c = np.ascontiguousarray(clips, dtype=np.uint8).reshape(-1, 20 * FRAME_BYTES)
        out = np.zeros(c.shape[0], np.float32)
        if self.L.shv_cuda_predict(self.m, c.ctypes.data, c.shape[0], out.ctypes.data):
            raise RuntimeError(last_error(self.L))
        return out

    def classify_rc(self, tokens):
        """Like classify but returns (rc, logits, error) instead of raising."""
        t = np.ascontiguousarray(tokens, dtype=np.float32)
        out = np.zeros(t.shape[0], np.float32)
        rc = self.L.shv_cuda_classify(self.m, t.ctypes.data, t.shape[0], out.ctypes.data)
        return rc, out, last_error(self.L)

    def upload_tokens(self, blocks, slots):
        b = np.ascontiguousarray(blocks, dtype=np.float32).reshape(-1, TOKEN_FLOATS)
        s = np.ascontiguousarray(slots, dtype=np.int32)
        if self.L.shv_cuda_b200_upload_tokens(self.m, b.ctypes.data, b.shape[0], s.ctypes.data):
            raise RuntimeError(last_error(self.L))

    # ---- asynchronous
    def submit(self, n_windows, logits_out, window_tokens=None, window_slots=None, window_frames=None, callback=None,
               frames=None, n_frames=0, tokens_out=None, store_slots=None):
        """Returns (job handle or None, keepalive tuple).  window_tokens: list of numpy blocks (or None entries)."""
        req, keep = build_request(n_windows, logits_out, window_tokens, window_slots, window_frames, callback, frames, n_frames,
                                  tokens_out, store_slots)
        job = self.L.shv_cuda_submit(self.m, C.byref(req))
        return job, keep

    def job_wait(self, job):
        return self.L.shv_cuda_job_wait(job)

    def job_status(self, job):
        return self.L.shv_cuda_job_status(job)

    def job_error(self, job):
        return self.L.shv_cuda_job_error(job).decode()

    def job_timing(self, job):
        q, r, g = C.c_double(), C.c_double(), C.c_double()
        bf, bw = C.c_int(), C.c_int()
        rc = self.L.shv_cuda_job_timing(job, C.byref(q), C.byref(r), C.byref(g), C.byref(bf), C.byref(bw))
        return rc, {"queue_ms": q.value, "run_ms": r.value, "gpu_ms": g.value, "batch_frames": bf.value,
                    "batch_windows": bw.value}

    def job_free(self, job):
        self.L.shv_cuda_job_free(job)

    def close(self):
        if self.m:
            self.L.shv_cuda_free(self.m)
            self.m = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Box:
    """shv_box_*: one model per device of a box behind one object (sessions placed by participant, batches sharded)."""

    def __init__(self, weights, mode, devices, max_sessions=0, experimental=True, ops=None, **options):
        self.L = load_library(experimental)
        opt = Options()
        self.L.shv_cuda_default_options(C.byref(opt))
        for k, v in options.items():
            if not hasattr(opt, k):
                raise TypeError(f"unknown option {k}")
            setattr(opt, k, int(v))
        devs = (C.c_int * len(devices))(*devices)
        self._ops = ops                                      # keeps the stand-in callbacks alive
        if ops is None:
            self.b = self.L.shv_box_load(str(weights).encode(), mode.encode(), devs, len(devices), C.byref(opt), max_sessions)
        else:
            self.b = self.L.shv_box_load_with(C.byref(ops), str(weights).encode(), mode.encode(), devs, len(devices),
                                              C.byref(opt), max_sessions)
        if not self.b:
            raise RuntimeError(last_error(self.L))
        self.n = len(devices)

    def home_device(self, participant):
        return self.L.shv_box_home_device(self.b, participant.encode())

    def session_open(self, participant):
        """-> (device index, first of the session's 24 token slots on that device)."""
        d, s = C.c_int(-1), C.c_int(-1)
        if self.L.shv_box_session_open(self.b, participant.encode(), C.byref(d), C.byref(s)):
            raise RuntimeError(last_error(self.L))
        return d.value, s.value

    def session_close(self, device, slot_base):
        if self.L.shv_box_session_close(self.b, device, slot_base):
            raise RuntimeError(last_error(self.L))

    def free_sessions(self, device):
        return self.L.shv_box_free_sessions(self.b, device)

    def model_handle(self, device):
        return self.L.shv_box_model(self.b, device)

    def classify(self, tokens):
        t = np.ascontiguousarray(tokens, dtype=np.float32)
        out = np.empty(t.shape[0], np.float32)
        if self.L.shv_box_classify(self.b, t.ctypes.data, t.shape[0], out.ctypes.data):
            raise RuntimeError(last_error(self.L))
        return out

    def submit(self, device, request):
        """request: a filled binding.Request; returns the job handle (or None)."""
        return self.L.shv_box_submit(self.b, device, C.byref(request))

    def close(self):
        if self.b:
            self.L.shv_box_free(self.b)
            self.b = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class EngineCore:
    """shvb_engine_*: the engine core driven directly on device-resident tokens and a caller-owned stream."""

    def __init__(self, weights, mode="fp32", device=0, max_windows=512, use_graphs=True, experimental=True, max_frames=1):
        self.L = load_library(experimental)
        self.e = self.L.shvb_engine_create_ex(str(weights).encode(), mode.encode(), device, max_frames, max_windows,
                                              int(use_graphs))
        if not self.e:
            raise RuntimeError(last_error(self.L))
        self.max_windows = max_windows
        self.max_frames = max_frames

    def _ok(self, rc):
        if rc:
            raise RuntimeError(last_error(self.L))

    def bind_tokens(self, slot, device_ptr, batch, stream=0):
        self._ok(self.L.shvb_engine_bind_tokens(self.e, slot, device_ptr, batch, stream))

    def classify(self, slot, batch, stream=0):
        self._ok(self.L.shvb_engine_classify(self.e, slot, batch, stream))

    def logits_ptr(self, slot):
        return self.L.shvb_engine_logits(self.e, slot)

    def read_logits(self, slot, n, stream=0):
        out = np.empty(n, np.float32)
        self._ok(self.L.shvb_engine_read_logits(self.e, slot, out.ctypes.data, n, stream))
        return out

    def frames_ptr(self, slot):
        """Device address of the slot's uint8 crop buffer [max_frames][180][320][3]."""
        return self.L.shvb_engine_frames(self.e, slot)

    def tokens_ptr(self, slot):
        """Device address of the slot's encoded tokens [max_frames][16][384] fp32."""
        return self.L.shvb_engine_tokens(self.e, slot)

    def encode(self, slot, frames, stream=0):
        self._ok(self.L.shvb_engine_encode(self.e, slot, frames, stream))

    def frame_bucket(self, frames):
        return self.L.shvb_engine_frame_bucket(self.e, frames)

    def encode_launches(self):
        return self.L.shvb_engine_encode_launches(self.e)

    def _profile(self, fn, slot, n_items, stream):
        ms = (C.c_float * 128)()
        names = C.create_string_buffer(8192)
        n = fn(self.e, slot, n_items, stream, ms, 128, names, 8192)
        if n < 0:
            raise RuntimeError(last_error(self.L))
        return list(zip(names.value.decode().split(";"), [float(ms[i]) for i in range(n)]))

    def profile(self, slot, batch, stream=0):
        """[(kernel name, ms)] of one eager classify, one entry per launch."""
        return self._profile(self.L.shvb_engine_profile, slot, batch, stream)

    def profile_encode(self, slot, frames, stream=0):
        """[(kernel name, ms)] of one eager encode, one entry per launch."""
        return self._profile(self.L.shvb_engine_profile_encode, slot, frames, stream)

    def window_bucket(self, batch):
        return self.L.shvb_engine_window_bucket(self.e, batch)

    def launches(self):
        return self.L.shvb_engine_launches(self.e)

    def status(self):
        return self.L.shvb_engine_status(self.e)

    def bytes(self):
        return {k: self.L.shvb_engine_bytes(self.e, i) for i, k in enumerate(("weights", "activations", "slot"))}

    def set_dump_dir(self, path):
        self._ok(self.L.shvb_engine_set_dump_dir(self.e, str(path).encode() if path else b""))

    def close(self):
        if self.e:
            self.L.shvb_engine_destroy(self.e)
            self.e = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
