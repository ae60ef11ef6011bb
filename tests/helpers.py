"""Shared helpers for the GPU parity tests."""
from __future__ import annotations

import numpy as np

from trigrad_b200.stages import *  # noqa: F401,F403  (stage wrappers over the C ABI)


def rel_err(a, b):
    """max |a-b| / max |b| (tensor-relative maximum error)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    denom = np.abs(b).max()
    return float(np.abs(a - b).max() / (denom if denom > 0 else 1.0))


def rel_l2(a, b):
    """||a-b||_2 / ||b||_2."""
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    denom = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / (denom if denom > 0 else 1.0))
