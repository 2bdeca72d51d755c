"""TEST INFRASTRUCTURE ONLY -- CPU restatement (numpy) of the SHIELD-V sequence path.

This module is the checker for the CUDA engine: only tests/, the smoke test and the benchmark's CPU-baseline leg may
import it.  Nothing in the shipped engine calls it.

It restates, in float32 or float64 numpy, the function that the reference defines three times:
  * PyTorch oracle        oracle/shieldv_ref.py:111-163 (norms, short conv, recurrence), :186-202 (GatedDeltaNet),
                          :218-242 (GDN stage), :245-313 (SISA attention), :346-356 (SISA block), :398-422 (classify)
  * CPU engine            engine/model/isa_impl.hpp:854-860 (rms), :866-961 (GDN head), :964-994 (stage),
                          :996-1069 (SISA head, last row), :1071-1140 (window)
  * CUDA engine           engine/cuda/seq.cu:27-336, engine/cuda/engine.cu:406-470
Parity of this restatement is pinned in tests/ against (a) golden vectors produced by importing the reference's own
PyTorch oracle (tests/golden/make_golden.py) and (b) the reference's CPU engine compiled by oracle/Makefile.

Input: `w` is the {name: array} dict of a SHLDV001 weight file, `tokens` is [B, 20, 16, 384] (frame embeddings before
positions).  Output: logits [B]; pass `trace={}` to collect intermediates under the reference's trace names.
"""
from __future__ import annotations

import math

import numpy as np

D, H, DK, DV, DFF, DSTATE, NTOK = 384, 6, 64, 128, 960, 32, 321
NORM_EPS = 1e-6
L2_EPS = 1e-6


# ---------------------------------------------------------------------------------------------- scalar functions
def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x / (1.0 + np.exp(-x))


def softplus(x):
    """torch softplus, threshold 20 (shieldv_ref.py:192; common.cuh:76)."""
    with np.errstate(over="ignore"):
        return np.where(x > 20.0, x, np.log1p(np.exp(np.minimum(x, 20.0))))


def logsigmoid(x):
    """min(x, 0) - log1p(exp(-|x|)) (common.cuh:78)."""
    return np.minimum(x, 0.0) - np.log1p(np.exp(-np.abs(x)))


def rms_norm(x, weight, eps=NORM_EPS):
    """(x * (1 / sqrt(mean(x^2) + eps))) * w (seq.cu:44-69; isa_impl.hpp:854-860)."""
    dt = x.dtype
    ms = (x * x).mean(-1, keepdims=True, dtype=dt)
    return (x * (dt.type(1.0) / np.sqrt(ms + dt.type(eps)))) * weight


def l2norm(x, eps=L2_EPS):
    dt = x.dtype
    return x * (dt.type(1.0) / np.sqrt((x * x).sum(-1, keepdims=True, dtype=dt) + dt.type(eps)))


def short_conv_silu(x, weight, bias):
    """Causal depthwise conv, kernel 4, bias, SiLU.  x [B,T,C]; weight [C,1,4]: tap j multiplies x[t-3+j]
    (shieldv_ref.py:142-150; seq.cu:77-86)."""
    b, t, c = x.shape
    acc = np.zeros_like(x)
    for j in range(4):
        shift = 3 - j
        if shift == 0:
            acc += weight[:, 0, j] * x
        else:
            acc[:, shift:] += weight[:, 0, j] * x[:, : t - shift]
    return silu(acc + bias)


# ---------------------------------------------------------------------------------------------- gated delta rule
def gated_delta_rule_recurrent(q, k, v, g, beta, scale):
    """Token-by-token gated delta rule from a zero state (shieldv_ref.py:121-139).

    q, k [B,T,H,K] (L2-normalised), v [B,T,H,V], g (log decay) and beta [B,T,H].  Returns o [B,T,H,V].
    """
    b, t, h, dk = q.shape
    dv = v.shape[-1]
    q = q * q.dtype.type(scale)
    decay = np.exp(g)
    state = np.zeros((b, h, dk, dv), q.dtype)
    out = np.empty((b, t, h, dv), q.dtype)
    for i in range(t):
        state = state * decay[:, i, :, None, None]
        kt = k[:, i]
        pred = np.einsum("bhk,bhkv->bhv", kt, state)
        u = (v[:, i] - pred) * beta[:, i, :, None]
        state = state + kt[..., None] * u[..., None, :]
        out[:, i] = np.einsum("bhk,bhkv->bhv", q[:, i], state)
    return out


def gated_delta_rule_chunked(q, k, v, g, beta, scale, chunk=64):
    """Chunked (WY / UT-transform) form of the same recurrence; algebraically identical, used to validate the
    tensor-core kernel's algorithm.  Per chunk with in-chunk cumulative log decay c_i:
        L_ij = beta_i exp(c_i - c_j) (k_i . k_j)   (j < i),   T = (I + L)^-1
        W = T diag(beta exp(c)) K,  U0 = T diag(beta) V,  U = U0 - W S0
        O = diag(exp(c)) Q S0 + (M o Q K^T) U,  M_ij = exp(c_i - c_j) (j <= i)
        S' = exp(c_C) S0 + (diag(exp(c_C - c)) K)^T U
    """
    b, t, h, dk = q.shape
    dv = v.shape[-1]
    dt = q.dtype
    q = q * dt.type(scale)
    out = np.empty((b, t, h, dv), dt)
    state = np.zeros((b, h, dk, dv), dt)
    for s0 in range(0, t, chunk):
        s1 = min(t, s0 + chunk)
        n = s1 - s0
        qc, kc, vc = (x[:, s0:s1].transpose(0, 2, 1, 3) for x in (q, k, v))          # [B,H,n,*]
        gc = np.cumsum(g[:, s0:s1].transpose(0, 2, 1), axis=-1, dtype=dt)               # [B,H,n]
        bc = beta[:, s0:s1].transpose(0, 2, 1)
        diff = gc[..., :, None] - gc[..., None, :]                                      # c_i - c_j
        tri = np.tril(np.ones((n, n), bool))
        m = np.where(tri, np.exp(np.where(tri, diff, 0.0)), 0.0).astype(dt)
        kk = kc @ kc.transpose(0, 1, 3, 2)
        lmat = np.tril(bc[..., :, None] * m * kk, -1)
        tinv = np.linalg.inv(np.eye(n, dtype=dt) + lmat)
        wmat = tinv @ ((bc * np.exp(gc))[..., None] * kc)
        u0 = tinv @ (bc[..., None] * vc)
        u = u0 - wmat @ state
        o = np.exp(gc)[..., None] * (qc @ state) + (m * (qc @ kc.transpose(0, 1, 3, 2))) @ u
        out[:, s0:s1] = o.transpose(0, 2, 1, 3)
        last = gc[..., -1]
        state = np.exp(last)[..., None, None] * state + (np.exp(last[..., None] - gc)[..., None] * kc).transpose(0, 1, 3, 2) @ u
    return out


# ---------------------------------------------------------------------------------------------- model blocks
def positions(w, dtype):
    """[320, 384]: (time[t] + row[r]) + col[c], token t*16 + r*4 + c, each sum rounded in float32 when dtype is
    float32 (engine/cuda/model.cpp:216-227)."""
    te, re, ce = (w[n].astype(dtype) for n in ("time_embedding", "row_embedding", "col_embedding"))
    return ((te[:, None, None, :] + re[None, :, None, :]) + ce[None, None, :, :]).reshape(320, D)


def gdn_mixer(w, p, x, trace, tag):
    dt = x.dtype
    g = lambda n: w[f"{p}.{n}"].astype(dt)  # noqa: E731
    b, t, _ = x.shape
    q = short_conv_silu(x @ g("q_proj.weight").T, g("q_conv1d.weight"), g("q_conv1d.bias")).reshape(b, t, H, DK)
    k = short_conv_silu(x @ g("k_proj.weight").T, g("k_conv1d.weight"), g("k_conv1d.bias")).reshape(b, t, H, DK)
    v = short_conv_silu(x @ g("v_proj.weight").T, g("v_conv1d.weight"), g("v_conv1d.bias")).reshape(b, t, H, DV)
    qn, kn = l2norm(q), l2norm(k)
    logdecay = -np.exp(g("A_log")) * softplus(x @ g("a_proj.weight").T + g("dt_bias"))
    beta = sigmoid(x @ g("b_proj.weight").T)
    o = gated_delta_rule_recurrent(qn, kn, v, logdecay.astype(dt), beta.astype(dt), DK ** -0.5)
    gate = (x @ g("g_proj.weight").T).reshape(b, t, H, DV)
    rstd = dt.type(1.0) / np.sqrt((o * o).mean(-1, keepdims=True, dtype=dt) + dt.type(NORM_EPS))
    on = (o * rstd) * g("o_norm.weight") * silu(gate)
    out = on.reshape(b, t, H * DV) @ g("o_proj.weight").T
    if trace is not None:
        for name, val in (("q_conv", q), ("k_conv", k), ("v_conv", v), ("q_l2", qn), ("k_l2", kn), ("g", logdecay),
                          ("beta", beta), ("o_core", o), ("gate", gate), ("o_gated", on), ("out", out)):
            trace[f"{tag}.{name}"] = val
    return out


def gdn_stage(w, name, repeats, h, trace):
    dt = h.dtype
    for r in range(repeats):
        hn = rms_norm(h, w[f"{name}.norm.weight"].astype(dt))
        delta = gdn_mixer(w, f"{name}.mixer", hn, trace, f"{name}.rep{r}")
        h = h + delta / dt.type(math.sqrt(repeats))
        if trace is not None:
            trace[f"{name}.rep{r}.h"] = h
    hn = rms_norm(h, w[f"{name}.ffn_norm.weight"].astype(dt))
    f = (silu(hn @ w[f"{name}.ffn.gate.weight"].astype(dt).T) * (hn @ w[f"{name}.ffn.up.weight"].astype(dt).T)) \
        @ w[f"{name}.ffn.down.weight"].astype(dt).T
    return h + f


def _cumsum_double(x, dt):
    """torch CPU cumsum semantics kept by both native engines: accumulate in double, round each prefix to the
    working type (seq.cu:249-258; isa_impl.hpp:1001-1009)."""
    return np.cumsum(x.astype(np.float64), axis=1).astype(dt)


def sisa_last_row(w, h, trace):
    """SISA block evaluated for the readout row only (engine.cu:445-467; isa_impl.hpp:1092-1126): K, V, B, theta,
    alpha and forget for all 321 rows, Q, C, attention, W_O and the FFN for row 320."""
    dt = h.dtype
    a = "sisa.attn"
    g = lambda n: w[n].astype(dt)  # noqa: E731
    b = h.shape[0]
    xn = rms_norm(h, g("sisa.attn_norm.weight"))
    k = (xn @ g(f"{a}.W_K.weight").T).reshape(b, NTOK, H, DK)
    v = (xn @ g(f"{a}.W_V.weight").T).reshape(b, NTOK, H, DK)
    bb = (xn @ g(f"{a}.W_B.weight").T).reshape(b, NTOK, H, DSTATE)
    theta = (xn @ g(f"{a}.theta_proj.weight").T).reshape(b, NTOK, H, DSTATE // 2)
    alpha = xn @ g(f"{a}.alpha_proj.weight").T + g(f"{a}.alpha_proj.bias")
    z = xn @ g(f"{a}.forget_proj.weight").T + g(f"{a}.forget_proj.bias")
    gcum = _cumsum_double(-softplus(alpha), dt)                              # [B,T,H]
    fcum = _cumsum_double(logsigmoid(z), dt)
    phi = _cumsum_double(theta, dt)                                           # [B,T,H,16]
    xl = xn[:, NTOK - 1]
    q = (xl @ g(f"{a}.W_Q.weight").T).reshape(b, H, DK)
    c = (xl @ g(f"{a}.W_C.weight").T).reshape(b, H, DSTATE)

    def rotate(zz, ph):
        ze, zo = zz[..., 0::2], zz[..., 1::2]
        co, si = np.cos(ph), np.sin(ph)
        return np.stack([ze * co - zo * si, ze * si + zo * co], axis=-1).reshape(zz.shape)

    b_rot = rotate(bb, phi)
    c_rot = rotate(c, phi[:, NTOK - 1])
    lam = softplus(g(f"{a}.lambda_raw"))
    content = np.einsum("bhd,bthd->bth", q, k) * dt.type(1.0 / math.sqrt(DK))
    ssm = np.einsum("bhs,bths->bth", c_rot, b_rot)
    score = content + (lam * np.exp(gcum[:, NTOK - 1:NTOK] - gcum)) * ssm
    score = score + (fcum[:, NTOK - 1:NTOK] - fcum)
    score = score - score.max(axis=1, keepdims=True)
    e = np.exp(score)
    p = e / e.sum(axis=1, keepdims=True, dtype=dt)
    y = np.einsum("bth,bthd->bhd", p, v).reshape(b, D)
    x1 = h[:, NTOK - 1] + y @ g(f"{a}.W_O.weight").T
    xf = rms_norm(x1, g("sisa.ffn_norm.weight"))
    f = (silu(xf @ g("sisa.ffn.w_gate.weight").T) * (xf @ g("sisa.ffn.w_up.weight").T)) @ g("sisa.ffn.w_down.weight").T
    if trace is not None:
        trace["sisa.g"], trace["sisa.fgate"], trace["sisa.phi"] = gcum, fcum, phi
        trace["sisa.attn_y_last"] = y
    return x1 + f


def classify_tokens(w, tokens, dtype=np.float32, trace=None):
    """tokens [B,20,16,384] -> logits [B] (shieldv_ref.py:398-422)."""
    dt = np.dtype(dtype)
    tokens = np.asarray(tokens)
    if tokens.ndim != 4 or tokens.shape[1:] != (20, 16, D):
        raise ValueError("expected [B,20,16,384] tokens")
    b = tokens.shape[0]
    h = np.empty((b, NTOK, D), dt)
    h[:, :320] = tokens.astype(dt).reshape(b, 320, D) + positions(w, dt)
    h[:, 320] = w["readout"].astype(dt).reshape(D)
    if trace is not None:
        trace["h0"] = h.copy()
    h = gdn_stage(w, "gdn_a", 1, h, trace)
    if trace is not None:
        trace["after_gdn_a"] = h
    h = gdn_stage(w, "gdn_b", 2, h, trace)
    if trace is not None:
        trace["after_gdn_b"] = h
    x2 = sisa_last_row(w, h, trace)
    z = rms_norm(x2, w["final_norm.weight"].astype(dt))
    hid = silu(z @ w["head.0.weight"].astype(dt).T + w["head.0.bias"].astype(dt))
    logit = (hid @ w["head.2.weight"].astype(dt).T + w["head.2.bias"].astype(dt)).reshape(b)
    if trace is not None:
        trace["after_sisa_last"] = x2
        trace["final_norm_row"] = z
        trace["head_hidden"] = hid
        trace["logit"] = logit
    return logit
