"""Loader for the fixtures in tests/golden/ (written by tests/golden/make_golden.py)."""
import glob
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
PER_THREAD_CONFIGS = [(128, 64, 32, 64), (64, 64, 32, 64), (128, 64, 16, 64), (128, 32, 32, 32)]


def names():
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def from_bits(a: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(dtype)


def load(name: str) -> dict:
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    d = {k: z[k] for k in z.files}
    dt = getattr(torch, str(d["dtype"]))
    out = dict(raw=d, dtype=dt, layout=str(d["layout"]), smooth_k=bool(d["smooth_k"]))
    for t in ("q", "k", "v", "km"):
        if t + "_bits" in d:
            out[t] = from_bits(d[t + "_bits"], dt)
    out.setdefault("km", None)
    return out
