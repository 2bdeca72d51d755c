"""Shared helpers of the test suite."""
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]
GOLDEN = ROOT / "tests" / "golden"


def load_golden(name):
    with np.load(GOLDEN / f"{name}.npz", allow_pickle=False) as z:
        return {k: z[k] for k in z.files}


# ---------------------------------------------------------------------------------------------- GPU helpers
def dev(array, dtype=None):
    """numpy -> contiguous CUDA tensor (torch is only the device-memory plumbing of the tests)."""
    import torch

    t = torch.from_numpy(np.ascontiguousarray(array))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda().contiguous()


def stream_ptr():
    import torch

    return torch.cuda.current_stream().cuda_stream


def sync():
    import torch

    torch.cuda.synchronize()


def rel_err(got, ref):
    """max |got - ref| / max |ref|: the normalised error the 16-bit modes are judged by."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))
