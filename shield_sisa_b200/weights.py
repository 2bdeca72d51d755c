"""SHLDV001 weight files for SHIELD-V: tensor table, reader, writer and seeded synthetic weights.

The engine loads the same weight file as the reference engines do (format defined by the reference's
tools/export_v.py:4-8,62-79: magic "SHLDV001", u32 count, then per tensor u32 name length, name, u32 rank,
u32 dims, u64 element count, float32 data, all little endian) plus the "<file>.json" sidecar holding the decision
threshold and the SHA-256 of the weight file (engine/cuda/api.cu:410-421, engine/cuda/model.cpp:42-55).

No trained checkpoint ships with this repository, so tests and benchmarks use seeded synthetic weights of exactly
the reference architecture.  Two recipes:

  "W1"  every learned tensor ~ N(0, 0.02), norm gains 1, BatchNorm statistics (mean 0, var 1).  Small logits; the
        gated RMSNorm runs in its eps-dominated regime.
  "W3"  as W1, but every 2-D weight of the sequence stages ~ N(0, 1/fan_in) and the short-conv taps ~ N(0, 0.25),
        which gives O(1) activations, decay factors across (0, 1) and logits of order +-1: a much stricter test.
  "W5"  as W3, and the frame encoder is scaled too: every convolution and squeeze-excite weight ~ N(0, 1/fan_in),
        the token projection ~ N(0, 1/960), BatchNorm shifts and squeeze-excite biases ~ N(0, 0.25), so that the
        feature maps stay O(1) through all 15 blocks and the encoder's tokens are O(1) (under W1 / W3 they are
        about 1e-2 and test little).

Values come from numpy's PCG64 `default_rng(seed)`, consumed in table order, so any machine regenerates the same file.
"""
from __future__ import annotations

import hashlib
import json
import struct
from pathlib import Path

import numpy as np

D, H, DK, DV, DFF, DSTATE, FRAMES = 384, 6, 64, 128, 960, 32, 20

# MobileNetV3-Large inverted-residual table (input ch, kernel, expanded ch, output ch, squeeze-excite, stride).
_MBV3 = [
    (16, 3, 16, 16, False, 1), (16, 3, 64, 24, False, 2), (24, 3, 72, 24, False, 1), (24, 5, 72, 40, True, 2),
    (40, 5, 120, 40, True, 1), (40, 5, 120, 40, True, 1), (40, 3, 240, 80, False, 2), (80, 3, 200, 80, False, 1),
    (80, 3, 184, 80, False, 1), (80, 3, 184, 80, False, 1), (80, 3, 480, 112, True, 1), (112, 3, 672, 112, True, 1),
    (112, 5, 672, 160, True, 2), (160, 5, 960, 160, True, 1), (160, 5, 960, 160, True, 1),
]


def _make_divisible(v: float, divisor: int = 8) -> int:
    new_v = max(divisor, int(v + divisor / 2) // divisor * divisor)
    if new_v < 0.9 * v:
        new_v += divisor
    return new_v


def _conv_bn(prefix: str, out_c: int, in_c: int, k: int):
    yield f"{prefix}.0.weight", (out_c, in_c, k, k)
    for leaf in ("weight", "bias", "running_mean", "running_var"):
        yield f"{prefix}.1.{leaf}", (out_c,)


def tensor_table() -> list[tuple[str, tuple[int, ...]]]:
    """Every tensor of a SHLDV001 SHIELD-V export with its shape (331 entries)."""
    t: list[tuple[str, tuple[int, ...]]] = []
    t += [("time_embedding", (FRAMES, D)), ("row_embedding", (4, D)), ("col_embedding", (4, D)),
          ("readout", (1, 1, D))]
    t += list(_conv_bn("cnn.0", 16, 3, 3))
    for i, (cin, k, cexp, cout, se, _stride) in enumerate(_MBV3):
        pre = f"cnn.{i + 1}.block"
        idx = 0
        if cexp != cin:
            t += list(_conv_bn(f"{pre}.{idx}", cexp, cin, 1))
            idx += 1
        t += list(_conv_bn(f"{pre}.{idx}", cexp, 1, k))
        idx += 1
        if se:
            cs = _make_divisible(cexp // 4, 8)
            t += [(f"{pre}.{idx}.fc1.weight", (cs, cexp, 1, 1)), (f"{pre}.{idx}.fc1.bias", (cs,)),
                  (f"{pre}.{idx}.fc2.weight", (cexp, cs, 1, 1)), (f"{pre}.{idx}.fc2.bias", (cexp,))]
            idx += 1
        t += list(_conv_bn(f"{pre}.{idx}", cout, cexp, 1))
    t += list(_conv_bn("cnn.16", 960, 160, 1))
    t += [("projection.weight", (D, 960))]
    for s in ("gdn_a", "gdn_b"):
        m = f"{s}.mixer"
        t += [(f"{s}.norm.weight", (D,)), (f"{s}.ffn_norm.weight", (D,)), (f"{m}.A_log", (H,)), (f"{m}.dt_bias", (H,)),
              (f"{m}.q_proj.weight", (H * DK, D)), (f"{m}.k_proj.weight", (H * DK, D)),
              (f"{m}.v_proj.weight", (H * DV, D)), (f"{m}.a_proj.weight", (H, D)), (f"{m}.b_proj.weight", (H, D)),
              (f"{m}.q_conv1d.weight", (H * DK, 1, 4)), (f"{m}.q_conv1d.bias", (H * DK,)),
              (f"{m}.k_conv1d.weight", (H * DK, 1, 4)), (f"{m}.k_conv1d.bias", (H * DK,)),
              (f"{m}.v_conv1d.weight", (H * DV, 1, 4)), (f"{m}.v_conv1d.bias", (H * DV,)),
              (f"{m}.g_proj.weight", (H * DV, D)), (f"{m}.o_norm.weight", (DV,)), (f"{m}.o_proj.weight", (D, H * DV)),
              (f"{s}.ffn.gate.weight", (DFF, D)), (f"{s}.ffn.up.weight", (DFF, D)), (f"{s}.ffn.down.weight", (D, DFF))]
    a = "sisa.attn"
    t += [("sisa.attn_norm.weight", (D,)), (f"{a}.lambda_raw", (H,)), (f"{a}.W_Q.weight", (D, D)),
          (f"{a}.W_K.weight", (D, D)), (f"{a}.W_V.weight", (D, D)), (f"{a}.W_O.weight", (D, D)),
          (f"{a}.W_B.weight", (H * DSTATE, D)), (f"{a}.W_C.weight", (H * DSTATE, D)),
          (f"{a}.alpha_proj.weight", (H, D)), (f"{a}.alpha_proj.bias", (H,)),
          (f"{a}.theta_proj.weight", (H * DSTATE // 2, D)), (f"{a}.forget_proj.weight", (H, D)),
          (f"{a}.forget_proj.bias", (H,)), ("sisa.ffn_norm.weight", (D,)), ("sisa.ffn.w_gate.weight", (DFF, D)),
          ("sisa.ffn.w_up.weight", (DFF, D)), ("sisa.ffn.w_down.weight", (D, DFF))]
    t += [("final_norm.weight", (D,)), ("head.0.weight", (128, D)), ("head.0.bias", (128,)),
          ("head.2.weight", (1, 128)), ("head.2.bias", (1,))]
    return t


def _is_gain(name: str, shape) -> bool:
    if name.endswith("running_mean") or name.endswith("running_var"):
        return False
    if len(shape) == 1 and "norm" in name and name.endswith(".weight"):
        return True
    return name.startswith("cnn.") and name.endswith(".1.weight") and len(shape) == 1   # BatchNorm gain


def synth_weights(seed: int = 1, recipe: str = "W3", sigma: float = 0.02) -> dict[str, np.ndarray]:
    """Seeded synthetic weights of the reference architecture (see the module docstring for the recipes)."""
    if recipe not in ("W1", "W3", "W5"):
        raise ValueError("recipe must be 'W1', 'W3' or 'W5'")
    rng = np.random.default_rng(seed)
    out: dict[str, np.ndarray] = {}
    for name, shape in tensor_table():
        if name.endswith("running_var"):
            v = np.ones(shape, np.float32)
        elif name.endswith("running_mean"):
            v = np.zeros(shape, np.float32)
        elif _is_gain(name, shape):
            v = np.ones(shape, np.float32)
        else:
            z = rng.standard_normal(shape, dtype=np.float64)
            scale = sigma
            if recipe == "W5" and (name.startswith("cnn.") or name == "projection.weight"):
                if len(shape) == 4:
                    scale = np.sqrt(1.0 / (shape[1] * shape[2] * shape[3]))
                elif len(shape) == 2:
                    scale = 1.0 / np.sqrt(shape[1])
                else:
                    scale = 0.5
            elif recipe in ("W3", "W5") and not name.startswith("cnn.") and name != "projection.weight":
                if name.endswith("conv1d.weight"):
                    scale = 0.5
                elif len(shape) == 2 and name.endswith(".weight"):
                    scale = 1.0 / np.sqrt(shape[1])
            v = (z * scale).astype(np.float32)
        out[name] = v
    return out


def sha256_file(path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


def write_shldv(path, tensors: dict[str, np.ndarray], threshold: float = 0.5) -> str:
    """Write `tensors` as a SHLDV001 file plus its "<path>.json" sidecar; returns the file's SHA-256."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "wb") as f:
        f.write(b"SHLDV001")
        f.write(struct.pack("<I", len(tensors)))
        for name, arr in tensors.items():
            v = np.ascontiguousarray(arr, dtype="<f4")
            e = name.encode()
            f.write(struct.pack("<I", len(e)))
            f.write(e)
            f.write(struct.pack("<I", v.ndim))
            f.write(struct.pack("<" + "I" * v.ndim, *v.shape))
            f.write(struct.pack("<Q", v.size))
            f.write(v.tobytes(order="C"))
    sha = sha256_file(path)
    Path(str(path) + ".json").write_text(json.dumps(
        {"format": "SHLDV001", "threshold": float(threshold), "tensor_count": len(tensors), "output_sha256": sha}))
    return sha


def read_shldv(path) -> dict[str, np.ndarray]:
    out: dict[str, np.ndarray] = {}
    with open(path, "rb") as f:
        if f.read(8) != b"SHLDV001":
            raise ValueError("not a SHLDV001 file")
        (count,) = struct.unpack("<I", f.read(4))
        for _ in range(count):
            (n,) = struct.unpack("<I", f.read(4))
            name = f.read(n).decode()
            (rank,) = struct.unpack("<I", f.read(4))
            dims = struct.unpack("<" + "I" * rank, f.read(4 * rank))
            (elements,) = struct.unpack("<Q", f.read(8))
            out[name] = np.frombuffer(f.read(4 * elements), dtype="<f4").reshape(dims).copy()
        if f.read(1):
            raise ValueError("trailing bytes")
    return out


def synth_weight_file(path, seed: int = 1, recipe: str = "W3", threshold: float = 0.5) -> dict[str, np.ndarray]:
    """Generate synthetic weights, write them to `path` (+ sidecar) and return the tensors."""
    w = synth_weights(seed, recipe)
    write_shldv(path, w, threshold)
    return w


def synth_frames(n: int, seed: int) -> np.ndarray:
    """RGB crops [n, 180, 320, 3] uint8, uniform in [0, 255]: the stand-in for face crops."""
    rng = np.random.default_rng(seed)
    return rng.integers(0, 256, size=(n, 180, 320, 3), dtype=np.uint8)


def synth_tokens(batch: int, seed: int) -> np.ndarray:
    """Frame embeddings [batch, 20, 16, 384] float32 ~ N(0, 1): the stand-in for MobileNetV3 tokens."""
    rng = np.random.default_rng(seed)
    return rng.standard_normal((batch, FRAMES, 16, D), dtype=np.float32)
