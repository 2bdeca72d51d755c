"""Pins the CPU restatement (oracle/seq_oracle.py) and the compiled reference CPU engine against the golden vectors
that tests/golden/make_golden.py produced from the reference's own PyTorch oracle."""
import numpy as np
import pytest

from tests.helpers import load_golden
from oracle import ref_cpu, seq_oracle as O
from shield_sisa_b200 import weights as W

CASES = ["w3_s1_t2_b3", "w1_s1_t1_b2", "w3_s5_t7_b2"]


def _inputs(g, weight_files):
    path, w = weight_files(str(g["recipe"]), int(g["weight_seed"]))
    return path, w, W.synth_tokens(int(g["batch"]), int(g["token_seed"]))


@pytest.mark.parametrize("case", CASES)
def test_restatement_float64_matches_reference_oracle(case, weight_files):
    g = load_golden(case)
    _, w, tok = _inputs(g, weight_files)
    tr = {}
    logits = O.classify_tokens(w, tok, np.float64, tr)
    np.testing.assert_allclose(logits, g["logits_f64"], rtol=0, atol=1e-10)
    np.testing.assert_allclose(tr["after_sisa_last"], g["after_sisa_last"], rtol=0, atol=1e-10)
    np.testing.assert_allclose(tr["head_hidden"], g["head_hidden"], rtol=0, atol=1e-10)
    rows, b = g["rows"], int(g["batch"])
    for key in [k for k in g if k.startswith("trace:")]:
        name = key[6:]
        if name == "sisa.attn_y":
            continue                                   # the restatement evaluates the readout row only
        got = tr[name][[0, b - 1]][:, rows]
        np.testing.assert_allclose(got, g[key].reshape(got.shape), rtol=0, atol=1e-10, err_msg=name)
    if "trace:sisa.attn_y" in g:                       # golden [2, rows, H, 64]; row 320 is the last selected row
        y = g["trace:sisa.attn_y"][:, -1].reshape(2, 384)
        np.testing.assert_allclose(tr["sisa.attn_y_last"][[0, b - 1]], y, rtol=0, atol=1e-10)


@pytest.mark.parametrize("case", CASES)
def test_restatement_float32_within_reference_noise(case, weight_files):
    g = load_golden(case)
    _, w, tok = _inputs(g, weight_files)
    logits = O.classify_tokens(w, tok, np.float32)
    assert np.abs(logits - g["logits_f64"]).max() < 2e-5
    assert np.abs(g["logits_f32"] - g["logits_f64"]).max() < 2e-5     # the reference's own float32 noise floor


def test_delta_rule_recurrent_and_chunked_match_reference():
    from tests.golden.make_golden_inputs import delta_inputs
    g = load_golden("delta_rule")
    for tag in ("k64v128", "k128v128"):
        b, t, h, dk, dv, seed = (int(x) for x in g[f"{tag}:shape"])
        q, k, v, gg, beta = delta_inputs(b, t, h, dk, dv, seed)
        o = O.gated_delta_rule_recurrent(q, k, v, gg, beta, dk ** -0.5)
        np.testing.assert_allclose(o[:, ::16], g[f"{tag}:o"], rtol=0, atol=1e-12)
        for chunk in (64, 32):
            oc = O.gated_delta_rule_chunked(q, k, v, gg, beta, dk ** -0.5, chunk)
            np.testing.assert_allclose(oc[:, ::16], g[f"{tag}:o"], rtol=0, atol=1e-11)


@pytest.mark.skipif(not ref_cpu.available(), reason="oracle/_ref not built (needs the reference checkout)")
@pytest.mark.parametrize("case", CASES)
def test_reference_cpu_engine_matches_golden(case, weight_files):
    g = load_golden(case)
    path, _, tok = _inputs(g, weight_files)
    eng = ref_cpu.RefCpuEngine(path, threads=2)
    logits = eng.classify(tok)
    eng.close()
    np.testing.assert_array_equal(logits, g["logits_cpu_engine"])     # the engine is bit-reproducible
    assert np.abs(logits - g["logits_f64"]).max() < 2e-5


def test_weight_file_round_trip(tmp_path, weight_files):
    path, w = weight_files("W1", 1)
    back = W.read_shldv(path)
    assert list(back) == [n for n, _ in W.tensor_table()]
    for name, shape in W.tensor_table():
        assert back[name].shape == shape
        np.testing.assert_array_equal(back[name], w[name])


# ---------------------------------------------------------------------------------------------- frame encoder
ENCODER_CASES = ["encoder_w5_s3_f11", "encoder_w1_s1_f5"]


def _encoder_inputs(g, weight_files):
    from shield_sisa_b200 import weights as W
    _, w = weight_files(str(g["recipe"]), int(g["weight_seed"]))
    return w, W.synth_frames(int(g["frames"]), int(g["frame_seed"]))


@pytest.mark.parametrize("case", ENCODER_CASES)
def test_encoder_restatement_matches_reference_oracle(case, weight_files):
    from oracle import cnn_oracle as CO
    g = load_golden(case)
    w, frames = _encoder_inputs(g, weight_files)
    trace = {}
    tok = CO.encode_frames(w, frames, np.float64, trace)
    assert np.abs(tok - g["tokens_f64"]).max() < 1e-10
    assert np.abs(trace["cnn_map"][:, ::2, ::3, ::7] - g["map_f64_sample"]).max() < 1e-10
    tok32 = CO.encode_frames(w, frames, np.float32)
    assert tok32.dtype == np.float32
    assert np.abs(tok32 - g["tokens_f64"]).max() < 2e-5


@pytest.mark.parametrize("case", ENCODER_CASES)
def test_reference_cpu_engine_encoder_matches_golden(case, weight_files):
    from oracle import ref_cpu
    from shield_sisa_b200 import weights as W
    if not ref_cpu.available():
        pytest.skip("reference CPU engine not built")
    g = load_golden(case)
    path, _ = weight_files(str(g["recipe"]), int(g["weight_seed"]))
    _, frames = _encoder_inputs(g, weight_files)
    eng = ref_cpu.RefCpuEngine(path, threads=2)
    tok = eng.encode_frames(frames)
    assert np.abs(tok - g["tokens_cpu_engine"]).max() < 1e-6        # thread count and ISA do not change its results
    assert np.abs(tok - g["tokens_f64"]).max() < 1e-5
    clip = W.synth_frames(20, int(g["frame_seed"]) + 1)[None]
    assert np.abs(eng.predict(clip) - g["clip_logit_cpu_engine"]).max() < 1e-6
    eng.close()


def test_storage_policy_floor_of_the_16_bit_modes(weight_files):
    """What the reference's own 16-bit storage policy (xn, all-row weights, on, hid rounded; everything else exact)
    costs on the golden sets, measured as the GPU tests measure the engine: max|err| / max|ref| of the logits against
    the float64 oracle.  In bf16 the policy alone reaches or passes the 2e-2 budget on sets of two or three clips
    (one logit's error is a draw of about 1e-2 of the set's largest logit), which is why the GPU tests judge the logits
    of such small sets against 3e-2 and apply 2e-2 to the stage outputs and to logits of sets of 64 clips."""
    from oracle import lowp_policy
    from shield_sisa_b200 import weights as W
    from tests.helpers import load_golden, rel_err
    worst = {"bf16": 0.0, "fp16": 0.0}
    for case in ("w3_s1_t2_b3", "w1_s1_t1_b2", "w3_s5_t7_b2"):
        g = load_golden(case)
        _, w = weight_files(str(g["recipe"]), int(g["weight_seed"]))
        tok = W.synth_tokens(int(g["batch"]), int(g["token_seed"]))
        for mode in worst:
            e = rel_err(lowp_policy.classify_tokens_storage_policy(w, tok, mode), g["logits_f64"])
            print(f"storage-policy floor {case} {mode}: {e:.3e}")
            worst[mode] = max(worst[mode], e)
    assert 1e-2 < worst["bf16"] < 4e-2          # the policy alone is of the order of the budget in bf16
    assert worst["fp16"] < 5e-3                 # and an order of magnitude below it in fp16
