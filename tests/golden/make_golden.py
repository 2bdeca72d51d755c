"""Regenerates tests/golden/*.npz by running the REFERENCE's own code on seeded synthetic inputs.

Runs only where the reference checkout is present (pass its path as the first argument): it imports the
reference's PyTorch oracle (oracle/shieldv_ref.py) and, if oracle/_ref/libshield_v_cpu.so has been built by
oracle/Makefile, also runs the reference's exact-FP32 CPU engine.  The tests read only the .npz files; inputs are
regenerated from the seeds stored in them (shield_sisa_b200/weights.py), so no weights or tokens are committed.

  python tests/golden/make_golden.py /path/to/reference

Each case file holds: recipe / seeds / batch; float64 and float32 logits of the PyTorch oracle; logits of the CPU
engine; and (for the first two cases), for selected rows of the first and last window, float64 intermediates under the
oracle's trace names.
`encoder_*.npz` pins the frame encoder: float64 tokens of the PyTorch oracle (MobileNetV3 features, pooling, projection)
on seeded uint8 crops, samples of its feature map, the CPU engine's tokens and the logit of a whole clip (shv_cpu_predict).
`delta_rule.npz` pins the bare recurrence (gated_delta_rule_recurrent, float64) on a long-sequence case.
"""
from __future__ import annotations

import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py <reference checkout>")
REF = Path(sys.argv[1])
sys.path.insert(0, str(REF / "oracle"))
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402
import shieldv_ref as R  # noqa: E402  (the reference's oracle)

from shield_sisa_b200 import weights as W  # noqa: E402
from oracle import ref_cpu  # noqa: E402
from tests.golden.make_golden_inputs import delta_inputs  # noqa: E402

ROWS = np.array([0, 1, 3, 16, 65, 160, 319, 320])
KEYS = ["h0", "after_gdn_a", "after_gdn_b", "gdn_a.rep0.q_l2", "gdn_a.rep0.k_l2", "gdn_a.rep0.v_conv",
        "gdn_a.rep0.g", "gdn_a.rep0.beta", "gdn_a.rep0.o_core", "gdn_a.rep0.o_gated", "gdn_b.rep1.o_core",
        "gdn_b.rep1.h", "sisa.g", "sisa.fgate", "sisa.phi", "sisa.attn_y"]
CASES = [("w3_s1_t2_b3", "W3", 1, 2, 3, True), ("w1_s1_t1_b2", "W1", 1, 1, 2, True), ("w3_s5_t7_b2", "W3", 5, 7, 2, False)]


def run_case(name, recipe, wseed, tseed, batch, with_trace):
    tmp = Path(tempfile.mkdtemp())
    wpath = tmp / "synthetic.weights"
    W.synth_weight_file(wpath, wseed, recipe)
    tok = W.synth_tokens(batch, tseed)
    out = {"recipe": recipe, "weight_seed": wseed, "token_seed": tseed, "batch": batch, "rows": ROWS}
    with torch.no_grad():
        m64 = R.load_ref_from_weights(wpath, torch.float64)
        tr = {}
        out["logits_f64"] = m64.classify_features(torch.from_numpy(tok).double(), tr).numpy()
        m32 = R.load_ref_from_weights(wpath, torch.float32)
        out["logits_f32"] = m32.classify_features(torch.from_numpy(tok)).numpy()
    out["after_sisa_last"] = tr["after_sisa"][:, 320].numpy()
    for k in ("final_norm_row", "head_hidden"):
        out[k] = tr[k].numpy()
    for k in KEYS if with_trace else ():
        v = tr[k].numpy()
        if k.startswith("sisa.") and v.shape[1] == 6:            # [B,H,L,...] -> [B,L,H,...]
            v = np.moveaxis(v, 1, 2)
        out["trace:" + k] = v[[0, batch - 1]][:, ROWS]
    if ref_cpu.available():
        dump = Path(tempfile.mkdtemp())
        eng = ref_cpu.RefCpuEngine(wpath, threads=4)
        out["logits_cpu_engine"] = eng.classify(tok)
        eng.close()
        eng = ref_cpu.RefCpuEngine(wpath, threads=1, dump_dir=dump)
        eng.classify(tok[:1])
        eng.close()
        for k in ("h0", "after_gdn_a", "after_gdn_b"):
            out["cpu:" + k] = ref_cpu.read_dump(dump, k).reshape(321, 384)[ROWS]
        out["cpu:after_sisa_last"] = ref_cpu.read_dump(dump, "after_sisa_last")
    np.savez_compressed(HERE / f"{name}.npz", **out)
    print(name, out["logits_f64"], out.get("logits_cpu_engine"))


def encoder_case(name, recipe, wseed, fseed, frames):
    """Frame encoder: uint8 crops -> tokens, PyTorch oracle in float64 and the CPU engine."""
    from oracle import cnn_oracle as CO
    tmp = Path(tempfile.mkdtemp())
    wpath = tmp / "synthetic.weights"
    W.synth_weight_file(wpath, wseed, recipe)
    fr = W.synth_frames(frames, fseed)
    out = {"recipe": recipe, "weight_seed": wseed, "frame_seed": fseed, "frames": frames}
    with torch.no_grad():
        m64 = R.load_ref_from_weights(wpath, torch.float64)
        x = torch.from_numpy(CO.normalise(fr, np.float32)).permute(0, 3, 1, 2).double()     # prepare_clips' float32 steps
        fmap = m64.cnn_map(x)
        out["tokens_f64"] = m64.tokens_from_map(fmap).numpy()
        out["map_f64_sample"] = fmap.permute(0, 2, 3, 1).numpy()[:, ::2, ::3, ::7]           # NHWC, subsampled
    if ref_cpu.available():
        eng = ref_cpu.RefCpuEngine(wpath, threads=4)
        out["tokens_cpu_engine"] = eng.encode_frames(fr)
        clip = W.synth_frames(20, fseed + 1)[None]
        out["clip_logit_cpu_engine"] = eng.predict(clip)
        eng.close()
    np.savez_compressed(HERE / f"{name}.npz", **out)
    print(name, float(np.abs(out["tokens_f64"]).max()), out.get("clip_logit_cpu_engine"))


def delta_rule_case():
    """Bare recurrence on a long sequence: B=2, T=300, H=3, DK=64, DV=128 (and DK=DV=128), float64."""
    out = {}
    for tag, dk, dv, seed in (("k64v128", 64, 128, 3), ("k128v128", 128, 128, 4)):
        b, t, h = 2, 300, 3
        q, k, v, g, beta = delta_inputs(b, t, h, dk, dv, seed)
        o = R.gated_delta_rule_recurrent(*(torch.from_numpy(x) for x in (q, k, v, g, beta)), dk ** -0.5).numpy()
        out[f"{tag}:shape"] = np.array([b, t, h, dk, dv, seed])
        out[f"{tag}:o"] = o[:, ::16]
    np.savez_compressed(HERE / "delta_rule.npz", **out)
    print("delta_rule", {k: v.shape for k, v in out.items()})


ENCODER_CASES = [("encoder_w5_s3_f11", "W5", 3, 11, 3), ("encoder_w1_s1_f5", "W1", 1, 5, 1)]

if __name__ == "__main__":
    for case in CASES:
        run_case(*case)
    for case in ENCODER_CASES:
        encoder_case(*case)
    delta_rule_case()
