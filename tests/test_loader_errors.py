"""Load-time validation of the C ABI (weights file, sidecar, mode, options, certificate).  Every case here fails
before the first CUDA call, so it runs without a GPU; the messages are the reference loader's
(engine/cuda/model.cpp:137-179,278-279; engine/cuda/api.cu:410-461,476-499)."""
import json
import shutil
import struct

import numpy as np
import pytest

from shield_sisa_b200 import binding, weights as W


@pytest.fixture(scope="module")
def lib():
    from shield_sisa_b200 import build
    build.build()
    return binding.load_library(True)


def load_error(path, mode="fp32", experimental=True, **opts):
    with pytest.raises(RuntimeError) as e:
        binding.CudaModel(path, mode, experimental=experimental, **opts)
    return str(e.value)


def copy_weights(src, dst_dir, name="w.weights"):
    dst = dst_dir / name
    shutil.copy(src, dst)
    shutil.copy(str(src) + ".json", str(dst) + ".json")
    return dst


def test_missing_file_and_bad_magic(lib, tmp_path):
    assert "cannot open weights" in load_error(tmp_path / "nope.weights")
    bad = tmp_path / "bad.weights"
    bad.write_bytes(b"SHLDA001" + b"\0" * 64)
    assert "not a SHLDV001 weight file" in load_error(bad)


def test_unknown_mode_and_options(lib, weight_files, tmp_path):
    path, _ = weight_files("W1", 1)
    assert "unknown mode" in load_error(path, "int8")
    for bad in ({"max_windows": 0}, {"max_windows": 4097}, {"max_frames": 0}, {"max_host_tokens": (1 << 20) + 1},
                {"token_slots": -1}, {"max_delay_us": -5}):
        assert "invalid options" in load_error(path, "fp32", **bad)


def test_tensor_table_is_enforced(lib, weight_files, tmp_path):
    _, w = weight_files("W1", 1)
    missing = dict(w)
    del missing["gdn_b.mixer.A_log"]
    p = tmp_path / "missing.weights"
    W.write_shldv(p, missing)
    assert "missing tensor: gdn_b.mixer.A_log" in load_error(p)
    extra = dict(w)
    extra["zz.extra"] = np.zeros(3, np.float32)
    p = tmp_path / "extra.weights"
    W.write_shldv(p, extra)
    assert "unexpected tensor in weight file: zz.extra" in load_error(p)
    shape = dict(w)
    shape["sisa.attn.W_B.weight"] = np.zeros((191, 384), np.float32)
    p = tmp_path / "shape.weights"
    W.write_shldv(p, shape)
    assert "bad shape for sisa.attn.W_B.weight" in load_error(p)
    nonfinite = dict(w)
    nonfinite["head.0.bias"] = np.full(128, np.nan, np.float32)
    p = tmp_path / "nan.weights"
    W.write_shldv(p, nonfinite)
    assert "non-finite value in tensor: head.0.bias" in load_error(p)


def test_truncated_and_trailing_bytes(lib, weight_files, tmp_path):
    path, _ = weight_files("W1", 1)
    data = path.read_bytes()
    t = tmp_path / "trunc.weights"
    t.write_bytes(data[: len(data) // 2])
    assert "truncated" in load_error(t)
    t = tmp_path / "trail.weights"
    t.write_bytes(data + b"\0")
    assert "trailing weight data" in load_error(t)
    t = tmp_path / "count.weights"
    t.write_bytes(b"SHLDV001" + struct.pack("<I", 0))
    assert "invalid tensor count" in load_error(t)


def test_sidecar_rules(lib, weight_files, tmp_path):
    src, _ = weight_files("W1", 1)
    p = copy_weights(src, tmp_path)
    side = json.loads(open(str(p) + ".json").read())
    open(str(p) + ".json", "w").write(json.dumps({**side, "threshold": 1.5}))
    assert "threshold out of (0,1)" in load_error(p)
    open(str(p) + ".json", "w").write(json.dumps({"output_sha256": side["output_sha256"]}))
    assert "no threshold" in load_error(p)
    open(str(p) + ".json", "w").write(json.dumps({**side, "output_sha256": "0" * 64}))
    assert "does not match the weights' SHA-256" in load_error(p)
    open(str(p) + ".json", "w").write(json.dumps({"threshold": 0.5}))
    assert "no output_sha256" in load_error(p)
    (tmp_path / "w.weights.json").unlink()
    assert "cannot open" in load_error(p)


def test_strict_library_wants_a_certificate_for_16_bit_modes(lib, weight_files, tmp_path):
    src, _ = weight_files("W1", 1)
    p = copy_weights(src, tmp_path)
    sha = W.sha256_file(p)
    rev = lib.shv_cuda_compute_revision().decode()
    cert = tmp_path / "w.weights.cuda.cert"
    assert "needs a quality certificate" in load_error(p, "bf16", experimental=False)
    cert.write_text("SHIELDV_CUDA_CERT_V1\n")
    assert "expected SHIELDV_CUDA_CERT_V2" in load_error(p, "bf16", experimental=False)
    cert.write_text(f"SHIELDV_CUDA_CERT_V2\n{sha} fp16 {rev} PASS c.json abc threshold=0.5\n")
    assert "no passing certificate" in load_error(p, "bf16", experimental=False)
    cert.write_text(f"SHIELDV_CUDA_CERT_V2\n{sha} bf16 {rev} PASS c.json abc threshold=0.25\n")
    assert "does not cover the threshold" in load_error(p, "bf16", experimental=False)
    cert.write_text(f"SHIELDV_CUDA_CERT_V2\n{sha} bf16 someotherrevision PASS c.json abc threshold=0.5\n")
    assert "no passing certificate" in load_error(p, "bf16", experimental=False)
    # a matching line passes the certificate gate; without a GPU the load then stops at the first CUDA call
    cert.write_text(f"SHIELDV_CUDA_CERT_V2\n{sha} bf16 {rev} PASS c.json abc threshold=0.5\n")
    import torch
    if not torch.cuda.is_available():
        assert "CUDA error" in load_error(p, "bf16", experimental=False)
    # fp32 never needs one
    if not torch.cuda.is_available():
        assert "CUDA error" in load_error(p, "fp32", experimental=False)
