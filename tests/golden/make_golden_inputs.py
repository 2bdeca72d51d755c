"""Seeded inputs shared by the golden-vector generator and the tests that replay it."""
import numpy as np


def delta_inputs(b, t, h, dk, dv, seed):
    """float64 q, k (L2-normalised), v, log decay g = logsigmoid(n), beta = sigmoid(n) from one seeded stream."""
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((b, t, h, dk))
    k = rng.standard_normal((b, t, h, dk))
    v = rng.standard_normal((b, t, h, dv))
    q /= np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6)
    k /= np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    g = -np.log1p(np.exp(-rng.standard_normal((b, t, h))))
    beta = 1.0 / (1.0 + np.exp(-rng.standard_normal((b, t, h))))
    return q, k, v, g, beta
