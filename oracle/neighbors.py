"""Brute-force float64 periodic neighbour list (test infrastructure only).

Stands in for ``pymatgen.core.Structure.get_neighbor_list(r, numerical_tol=1e-8)``,
the single third-party call of the reference's graph path
(matris/graph/converter.py:85-87; pymatgen pinned ==2025.10.07 in the
reference's requirements.txt).  pymatgen is neither vendored nor installed and
no reference test pins its output, so this function is DEFINITIONAL:
PARITY UNPINNED at that boundary.

Definition: all ordered triples (i, j, n), n an integer lattice translation,
with ``tol < d <= r`` where, in IEEE float64 with NO fused multiply-add and in
exactly this operation order,

    s   = (n0*L[0] + n1*L[1]) + n2*L[2]          (per Cartesian component)
    dx  = (x_j + s) - x_i
    d2  = (dx0*dx0 + dx1*dx1) + dx2*dx2
    d   = sqrt(d2)

Coordinates are NOT wrapped into the cell: images are relative to the
coordinates as given (as pymatgen reports them).  The inclusive ``<= r`` at the
boundary cannot be verified against pymatgen here; it is measure-zero for all
perturbed benchmark structures.
"""
from __future__ import annotations

import numpy as np


def perpendicular_widths(lattice: np.ndarray) -> np.ndarray:
    """Distance between opposite cell faces along each lattice axis."""
    L = np.asarray(lattice, dtype=np.float64)
    vol = abs(np.dot(L[0], np.cross(L[1], L[2])))
    w = np.empty(3)
    for k in range(3):
        c = np.cross(L[(k + 1) % 3], L[(k + 2) % 3])
        w[k] = vol / np.linalg.norm(c)
    return w


def neighbor_list(cart: np.ndarray, lattice: np.ndarray, r: float, tol: float = 1e-8,
                  chunk: int = 4096):
    """Return (center[int64], neighbor[int64], image[int64,3], distance[float64]).

    Output is sorted by (center, neighbor, n0, n1, n2).
    """
    x = np.ascontiguousarray(cart, dtype=np.float64)
    L = np.ascontiguousarray(lattice, dtype=np.float64)
    n_atoms = x.shape[0]
    frac = x @ np.linalg.inv(L)
    spread = frac.max(axis=0) - frac.min(axis=0) if n_atoms else np.zeros(3)
    w = perpendicular_widths(L)
    nmax = np.ceil(r / w + spread + 1e-9).astype(int)
    cs, ns, ims, ds = [], [], [], []
    for n0 in range(-nmax[0], nmax[0] + 1):
        for n1 in range(-nmax[1], nmax[1] + 1):
            for n2 in range(-nmax[2], nmax[2] + 1):
                s = (float(n0) * L[0] + float(n1) * L[1]) + float(n2) * L[2]
                xs = x + s  # x_j + s
                for i0 in range(0, n_atoms, chunk):
                    xi = x[i0:i0 + chunk]
                    dx = xs[None, :, :] - xi[:, None, :]
                    d2 = (dx[..., 0] * dx[..., 0] + dx[..., 1] * dx[..., 1]) + dx[..., 2] * dx[..., 2]
                    d = np.sqrt(d2)
                    ii, jj = np.nonzero((d > tol) & (d <= r))
                    if ii.size:
                        cs.append(ii + i0)
                        ns.append(jj)
                        ims.append(np.broadcast_to(np.array([n0, n1, n2], dtype=np.int64), (ii.size, 3)))
                        ds.append(d[ii, jj])
    if not cs:
        z = np.zeros(0, dtype=np.int64)
        return z, z.copy(), np.zeros((0, 3), dtype=np.int64), np.zeros(0)
    c = np.concatenate(cs).astype(np.int64)
    n = np.concatenate(ns).astype(np.int64)
    im = np.concatenate(ims).astype(np.int64)
    d = np.concatenate(ds)
    order = np.lexsort((im[:, 2], im[:, 1], im[:, 0], n, c))
    return c[order], n[order], np.ascontiguousarray(im[order]), d[order]
