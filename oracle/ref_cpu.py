"""TEST INFRASTRUCTURE ONLY -- ctypes access to the reference's CPU engine built by oracle/Makefile.

`oracle/_ref/libshield_v_cpu.so` is the reference's exact-FP32 engine (engine/include/shv_cpu.h:92-128) compiled
unmodified from the reference checkout.  It is the authoritative checker for the CUDA engine and the CPU baseline the
benchmark times; the shipped engine never loads it.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

LIB = Path(__file__).resolve().parent / "_ref" / "libshield_v_cpu.so"


def available() -> bool:
    return LIB.exists()


class RefCpuEngine:
    """shv_cpu_load_ex / shv_cpu_classify / shv_cpu_free of the reference library."""

    def __init__(self, weights, threads: int = 1, mode: str = "exact", isa: str | None = None, dump_dir=None):
        if not LIB.exists():
            raise RuntimeError(f"{LIB} missing: run `make -C oracle` where the reference checkout is present")
        if dump_dir is not None:                       # read once at load (engine/model/runtime.cpp:900-906)
            os.environ["SHV_CPU_DUMP_DIR"] = str(dump_dir)
        else:
            os.environ.pop("SHV_CPU_DUMP_DIR", None)
        self.lib = C.CDLL(str(LIB))
        L = self.lib
        L.shv_cpu_load_ex.restype = C.c_void_p
        L.shv_cpu_load_ex.argtypes = [C.c_char_p, C.c_char_p, C.c_int, C.c_char_p]
        L.shv_cpu_free.argtypes = [C.c_void_p]
        L.shv_cpu_classify.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
        L.shv_cpu_classify.restype = C.c_int
        L.shv_cpu_encode_frames.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
        L.shv_cpu_encode_frames.restype = C.c_int
        L.shv_cpu_predict.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
        L.shv_cpu_predict.restype = C.c_int
        L.shv_cpu_last_error.restype = C.c_char_p
        L.shv_cpu_isa.restype = C.c_char_p
        L.shv_cpu_isa.argtypes = [C.c_void_p]
        self.threads = int(threads)
        self.h = L.shv_cpu_load_ex(str(weights).encode(), mode.encode(), self.threads, (isa or "").encode())
        os.environ.pop("SHV_CPU_DUMP_DIR", None)
        if not self.h:
            raise RuntimeError(L.shv_cpu_last_error().decode())

    @property
    def isa(self) -> str:
        return self.lib.shv_cpu_isa(self.h).decode()

    def classify(self, tokens) -> np.ndarray:
        t = np.ascontiguousarray(tokens, dtype=np.float32)
        if t.ndim != 4 or t.shape[1:] != (20, 16, 384):
            raise ValueError("expected [B,20,16,384] float32 tokens")
        out = np.empty(t.shape[0], np.float32)
        if self.lib.shv_cpu_classify(self.h, t.ctypes.data, t.shape[0], out.ctypes.data):
            raise RuntimeError(self.lib.shv_cpu_last_error().decode())
        return out

    def encode_frames(self, frames) -> np.ndarray:
        """uint8 crops [N,180,320,3] -> tokens [N,16,384] (shv_cpu_encode_frames, engine/include/shv_cpu.h:99-101)."""
        f = np.ascontiguousarray(frames, dtype=np.uint8)
        if f.ndim != 4 or f.shape[1:] != (180, 320, 3):
            raise ValueError("expected [N,180,320,3] uint8 crops")
        out = np.empty((f.shape[0], 16, 384), np.float32)
        if self.lib.shv_cpu_encode_frames(self.h, f.ctypes.data, f.shape[0], out.ctypes.data):
            raise RuntimeError(self.lib.shv_cpu_last_error().decode())
        return out

    def predict(self, clips) -> np.ndarray:
        """uint8 clips [B,20,180,320,3] -> logits [B] (shv_cpu_predict, engine/include/shv_cpu.h:111-112)."""
        c = np.ascontiguousarray(clips, dtype=np.uint8)
        if c.ndim != 5 or c.shape[1:] != (20, 180, 320, 3):
            raise ValueError("expected [B,20,180,320,3] uint8 clips")
        out = np.empty(c.shape[0], np.float32)
        if self.lib.shv_cpu_predict(self.h, c.ctypes.data, c.shape[0], out.ctypes.data):
            raise RuntimeError(self.lib.shv_cpu_last_error().decode())
        return out

    def close(self):
        if self.h:
            self.lib.shv_cpu_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def read_dump(dump_dir, name: str) -> np.ndarray:
    """A `<name>.f32` intermediate of window 0 written by the reference engine's debug hook."""
    return np.fromfile(Path(dump_dir) / f"{name}.f32", dtype="<f4")
