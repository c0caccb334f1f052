"""Helpers shared by the GPU parity tests."""
import os

import numpy as np
import torch

from conftest import ROOT

REPORT = os.path.join(ROOT, "gpurun_out", "parity_report.txt")


def report(name, got, want, tol, rel=False):
    """Compare, append a line to the parity report and assert.  The bound is
    ``tol * max(1, max|ref|)`` (absolute for small values, relative for large), or purely relative with rel=True."""
    got = np.asarray(got.detach().cpu().double() if torch.is_tensor(got) else got, dtype=np.float64)
    want = np.asarray(want.detach().cpu().double() if torch.is_tensor(want) else want, dtype=np.float64)
    assert got.shape == want.shape, (name, got.shape, want.shape)
    err = float(np.abs(got - want).max()) if got.size else 0.0
    scale = float(np.abs(want).max()) if want.size else 0.0
    bad = not np.isfinite(got).all()
    line = f"{name:58s} max|err|={err:.3e} max|ref|={scale:.3e} rel={err / (scale + 1e-30):.3e} tol={tol:.1e}"
    try:
        os.makedirs(os.path.dirname(REPORT), exist_ok=True)
        with open(REPORT, "a") as f:
            f.write(line + ("  NONFINITE" if bad else "") + "\n")
    except OSError:
        pass
    print(line)
    assert not bad, f"{name}: non-finite values"
    bound = tol * max(scale, 1e-30) if rel else tol * max(scale, 1.0)
    assert err <= bound, line
    return err


def dev(x, dtype=None):
    t = torch.as_tensor(x)
    if dtype is not None:
        t = t.to(dtype)
    return t.contiguous().cuda()
