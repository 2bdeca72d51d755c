"""TEST INFRASTRUCTURE ONLY -- what the reference's 16-bit STORAGE POLICY alone costs in accuracy.

The reference's bf16 / fp16 modes keep the residual stream, the projections, the delta rule and the readout row in
float32 and store four things in the mode's 16-bit type: the normalised rows xn, the all-row weights, the gated
delta-rule output `on` and the SwiGLU product `hid` (engine/cuda/engine.cu:150-164,213-219).  This module evaluates the
numpy oracle in float64 with exactly those four roundings and nothing else, so the distance of its logits from the
float64 oracle is a floor: no implementation that follows the policy can be expected to come closer than that, however
exact its own arithmetic.  tests/ use it to put the 16-bit modes' tolerance into perspective on small golden sets.
"""
from __future__ import annotations

import math

import numpy as np

from oracle import seq_oracle as O


def _round_to(a, mode: str):
    import torch                              # only for its bf16 / fp16 rounding

    dt = torch.bfloat16 if mode == "bf16" else torch.float16
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dt).float().numpy().astype(np.float64)


def classify_tokens_storage_policy(w, tokens, mode: str):
    """Logits [B] of the float64 oracle with xn, the all-row weights, on and hid rounded to `mode` ("bf16" / "fp16")."""
    f = np.float64
    q = lambda name: _round_to(w[name], mode)  # noqa: E731
    b = tokens.shape[0]
    h = np.empty((b, O.NTOK, O.D), f)
    h[:, :320] = tokens.astype(np.float32).reshape(b, 320, O.D) + O.positions(w, np.dtype(np.float32))
    h[:, 320] = w["readout"].reshape(O.D)
    for name, reps in (("gdn_a", 1), ("gdn_b", 2)):
        p = f"{name}.mixer"
        gw = lambda n: w[f"{p}.{n}"].astype(f)  # noqa: E731
        for _ in range(reps):
            x = _round_to(O.rms_norm(h, w[f"{name}.norm.weight"].astype(f)), mode)
            t = x.shape[1]
            qq = O.short_conv_silu(x @ q(f"{p}.q_proj.weight").T, gw("q_conv1d.weight"), gw("q_conv1d.bias")).reshape(b, t, O.H, O.DK)
            kk = O.short_conv_silu(x @ q(f"{p}.k_proj.weight").T, gw("k_conv1d.weight"), gw("k_conv1d.bias")).reshape(b, t, O.H, O.DK)
            vv = O.short_conv_silu(x @ q(f"{p}.v_proj.weight").T, gw("v_conv1d.weight"), gw("v_conv1d.bias")).reshape(b, t, O.H, O.DV)
            logdecay = -np.exp(gw("A_log")) * O.softplus(x @ q(f"{p}.a_proj.weight").T + gw("dt_bias"))
            beta = O.sigmoid(x @ q(f"{p}.b_proj.weight").T)
            o = O.gated_delta_rule_recurrent(O.l2norm(qq), O.l2norm(kk), vv, logdecay, beta, O.DK ** -0.5)
            gate = (x @ q(f"{p}.g_proj.weight").T).reshape(b, t, O.H, O.DV)
            rstd = 1.0 / np.sqrt((o * o).mean(-1, keepdims=True) + O.NORM_EPS)
            on = _round_to(((o * rstd) * gw("o_norm.weight") * O.silu(gate)).reshape(b, t, O.H * O.DV), mode)
            h = h + (on @ q(f"{p}.o_proj.weight").T) / math.sqrt(reps)
        hn = _round_to(O.rms_norm(h, w[f"{name}.ffn_norm.weight"].astype(f)), mode)
        hid = _round_to(O.silu(hn @ q(f"{name}.ffn.gate.weight").T) * (hn @ q(f"{name}.ffn.up.weight").T), mode)
        h = h + hid @ q(f"{name}.ffn.down.weight").T
    # SISA: the all-row projections use rounded weights (their rounded input rows are not emulated: a smaller term of
    # the same kind); the readout row is float32 in every mode
    w_sisa = dict(w)
    for n in ("W_K", "W_V", "W_B", "theta_proj", "alpha_proj", "forget_proj"):
        w_sisa[f"sisa.attn.{n}.weight"] = q(f"sisa.attn.{n}.weight").astype(np.float32)
    x2 = O.sisa_last_row(w_sisa, h, None)
    z = O.rms_norm(x2, w["final_norm.weight"].astype(f))
    hid = O.silu(z @ w["head.0.weight"].astype(f).T + w["head.0.bias"].astype(f))
    return (hid @ w["head.2.weight"].astype(f).T + w["head.2.bias"].astype(f)).reshape(b)
