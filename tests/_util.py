"""Shared helpers of the test-suite."""
import glob
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# fp32 parity bar for the default (fp32x3) and fp32 modes: the tolerance the specification states.
RTOL, ATOL = 1e-4, 1e-5
# The reference's own comparator (daceml/testing/utils.py:6).
REF_RTOL, REF_ATOL = 1e-5, 1e-4
# Single-pass TF32: operands cut to a 10-bit mantissa by the tensor core; stated wider tolerance.
TF32_RTOL, TF32_ATOL = 2e-2, 1e-2
# BF16 operands (8-bit mantissa, round-to-nearest-even), fp32 accumulate; stated wider tolerance.
BF16_RTOL, BF16_ATOL = 5e-2, 3e-2


def golden(name):
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        return {k: z[k] for k in z.files}


def golden_names(prefix):
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, prefix + "*.npz")))


def dev(x, device="cuda:0"):
    return torch.as_tensor(np.ascontiguousarray(x), dtype=torch.float32).to(device)


def close(actual, expected, rtol=RTOL, atol=ATOL):
    a = actual.detach().cpu().numpy() if isinstance(actual, torch.Tensor) else np.asarray(actual)
    e = expected.detach().cpu().numpy() if isinstance(expected, torch.Tensor) else np.asarray(expected)
    assert a.shape == e.shape, (a.shape, e.shape)
    err = np.abs(a.astype(np.float64) - e.astype(np.float64))
    bound = atol + rtol * np.abs(e.astype(np.float64))
    bad = err > bound
    assert not bad.any(), "%d / %d elements out of tolerance; max err %.3e (|ref| there %.3e)" % (
        bad.sum(), bad.size, err.max(), np.abs(e.ravel()[err.argmax()]))
