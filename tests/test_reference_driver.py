"""The reference's own API test driver (bench/gpu_bench.cpp, compiled unmodified by oracle/Makefile against this
repository's include/shv_cuda.h and linked against libshield_v_cuda_experimental.so) driving the B200 library.

Its `slots` command is the reference's row-independence test of the C ABI (bench/gpu_bench.cpp:221-272): sliding windows
assembled from device token slots, four new frames per hop, all hops queued at once so that the scheduler coalesces
them, must equal shv_cuda_predict on the same 20 frames BITWISE, and tokens encoded 60 at a time must equal tokens
encoded one by one bitwise.  The binary is built where the reference checkout is present and travels with the tree; the
data directory it reads (crop archives and the sample map) is generated here from seeded synthetic crops."""
import hashlib
import json
import os
import subprocess

import numpy as np
import pytest

from shield_sisa_b200 import weights as W
from tests.helpers import ROOT

DRIVER = ROOT / "oracle" / "_ref" / "gpu_bench"
needs_driver = pytest.mark.skipif(not DRIVER.exists(), reason="oracle/_ref/gpu_bench is built where the reference checkout is present")


@needs_driver
def test_reference_driver_is_linked_against_this_library():
    out = subprocess.run(["ldd", str(DRIVER)], capture_output=True, text=True, check=True).stdout
    line = next(ln for ln in out.splitlines() if "libshield_v_cuda_experimental.so" in ln)
    resolved = os.path.realpath(line.split("=>")[1].split("(")[0].strip())
    assert resolved == str(ROOT / "shield_sisa_b200" / "lib" / "libshield_v_cuda_experimental.so")   # through the binary's own rpath
    r = subprocess.run([str(DRIVER)], capture_output=True, text=True)
    assert r.returncode == 2 and "usage: gpu_bench" in r.stderr            # starts, loads the library, prints its usage


def make_data_dir(base, n_clips):
    """The layout bench/gpu_bench.cpp:53-77 reads: maps/orig.jsonl with one sample id per line, and one .npz per sample,
    named by the first 24 hex digits of the SHA-256 of its id, holding frames.npy uint8 [20,180,320,3]."""
    maps, crops = base / "shieldv_codec" / "maps", base / "shieldv_codec" / "crops" / "orig_bt601"
    maps.mkdir(parents=True)
    crops.mkdir(parents=True)
    frames = W.synth_frames(20 * n_clips, seed=21).reshape(n_clips, 20, 180, 320, 3)
    with open(maps / "orig.jsonl", "w") as f:
        for i in range(n_clips):
            sid = f"synthetic-{i:03d}"
            f.write(json.dumps({"sample_id": sid}) + "\n")
            np.savez(crops / (hashlib.sha256(sid.encode()).hexdigest()[:24] + ".npz"), frames=frames[i])


@needs_driver
@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["fp32", "fp16"])
def test_reference_slots_test_passes_on_this_library(mode, tmp_path):
    data = tmp_path / "data"
    make_data_dir(data, 3)
    (tmp_path / "build").mkdir()
    W.synth_weight_file(tmp_path / "build" / "shield_v.weights", seed=3, recipe="W5")   # the path the driver loads
    env = dict(os.environ, SHIELD_DATA_DIR=str(data))
    r = subprocess.run([str(DRIVER), "slots", "--mode", mode], cwd=tmp_path, env=env, capture_output=True, text=True, timeout=600)
    print(r.stdout, r.stderr)
    assert r.returncode == 0, r.stderr
    lines = [json.loads(ln) for ln in r.stdout.splitlines() if ln.startswith("{")]
    slots = next(ln for ln in lines if ln.get("what") == "slots")
    assert slots["logit_bitwise_diff"] == 0 and slots["tokens_batch60_vs_batch1_identical"] is True
    assert slots["windows"] == 11 and slots["max_coalesced_windows"] > 1     # the hops really shared GPU batches
    assert np.isfinite(slots["example"]).all()
