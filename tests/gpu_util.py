"""Helpers shared by the GPU parity tests."""
import os

import numpy as np
import torch

# a line per comparison is appended to this file when the environment names one
REPORT = os.environ.get("MATRIS_PARITY_REPORT")


def report(name, got, want, tol, rel=False, scaled=False):
    """Compare, log a line and assert.  The bound is ABSOLUTE (``tol``) by default - the gates on energy, force,
    stress and magnetic moment are absolute numbers; ``rel=True`` makes it ``tol * max|ref|``; ``scaled=True``
    makes it ``tol * max(1, max|ref|)`` (for feature tensors whose magnitude is not fixed by the problem)."""
    got = np.asarray(got.detach().cpu().double() if torch.is_tensor(got) else got, dtype=np.float64)
    want = np.asarray(want.detach().cpu().double() if torch.is_tensor(want) else want, dtype=np.float64)
    assert got.shape == want.shape, (name, got.shape, want.shape)
    err = float(np.abs(got - want).max()) if got.size else 0.0
    scale = float(np.abs(want).max()) if want.size else 0.0
    bad = not np.isfinite(got).all()
    line = f"{name:58s} max|err|={err:.3e} max|ref|={scale:.3e} rel={err / (scale + 1e-30):.3e} tol={tol:.1e}"
    if REPORT:
        try:
            with open(REPORT, "a") as f:
                f.write(line + ("  NONFINITE" if bad else "") + "\n")
        except OSError:
            pass
    print(line)
    assert not bad, f"{name}: non-finite values"
    bound = tol * max(scale, 1e-30) if rel else (tol * max(scale, 1.0) if scaled else tol)
    assert err <= bound, line
    return err


def dev(x, dtype=None):
    t = torch.as_tensor(x)
    if dtype is not None:
        t = t.to(dtype)
    return t.contiguous().cuda()
