"""Seeded synthetic structures for the benchmark configurations.

No public dataset is involved: every configuration is generated from a NumPy
``default_rng`` seed and returned as plain arrays ``(numbers, cart, lattice)``
(atomic numbers int64 [N], Cartesian positions float64 [N,3] in Angstrom,
lattice rows float64 [3,3]).
"""
from __future__ import annotations

from typing import NamedTuple

import numpy as np


class Crystal(NamedTuple):
    numbers: np.ndarray   # int64 [N]
    cart: np.ndarray      # float64 [N,3], Angstrom, not necessarily wrapped
    lattice: np.ndarray   # float64 [3,3], rows are the cell vectors

    @property
    def frac(self) -> np.ndarray:
        return self.cart @ np.linalg.inv(self.lattice)


# IUPAC standard atomic weights (abridged; mass number of the longest-lived isotope for Tc, Pm), Z = 1..83
ATOMIC_WEIGHT = np.array([
    0.0, 1.008, 4.0026, 6.94, 9.0122, 10.81, 12.011, 14.007, 15.999, 18.998, 20.180,
    22.990, 24.305, 26.982, 28.085, 30.974, 32.06, 35.45, 39.948, 39.098, 40.078,
    44.956, 47.867, 50.942, 51.996, 54.938, 55.845, 58.933, 58.693, 63.546, 65.38,
    69.723, 72.630, 74.922, 78.971, 79.904, 83.798, 85.468, 87.62, 88.906, 91.224,
    92.906, 95.95, 98.0, 101.07, 102.91, 106.42, 107.87, 112.41, 114.82, 118.71,
    121.76, 127.60, 126.90, 131.29, 132.91, 137.33, 138.91, 140.12, 140.91, 144.24,
    145.0, 150.36, 151.96, 157.25, 158.93, 162.50, 164.93, 167.26, 168.93, 173.05,
    174.97, 178.49, 180.95, 183.84, 186.21, 190.23, 192.22, 195.08, 196.97, 200.59,
    204.38, 207.2, 208.98])
AMU_PER_A3_TO_G_PER_CM3 = 1.66053906660


def _supercell(basis_frac, cell, reps):
    r = np.array([[i, j, k] for i in range(reps[0]) for j in range(reps[1]) for k in range(reps[2])], float)
    frac = (r[:, None, :] + np.asarray(basis_frac)[None, :, :]).reshape(-1, 3)
    return frac @ np.asarray(cell, float), np.asarray(cell, float) * np.asarray(reps, float)[:, None]


def cu_fcc(reps=(2, 2, 2), a=3.615, sigma=0.02, seed=0) -> Crystal:
    """FCC Cu supercell of the conventional cell, Gaussian-perturbed (32 atoms at 2x2x2)."""
    basis = [[0, 0, 0], [0.5, 0.5, 0], [0.5, 0, 0.5], [0, 0.5, 0.5]]
    cart, lat = _supercell(basis, np.eye(3) * a, reps)
    cart = cart + np.random.default_rng(seed).normal(0.0, sigma, cart.shape)
    return Crystal(np.full(len(cart), 29, dtype=np.int64), cart, lat)


def fe_bcc(reps=(20, 20, 20), a=2.866, sigma=0.05, seed=3) -> Crystal:
    """BCC Fe supercell with Gaussian thermal displacements (16,000 atoms at 20^3)."""
    cart, lat = _supercell([[0, 0, 0], [0.5, 0.5, 0.5]], np.eye(3) * a, reps)
    cart = cart + np.random.default_rng(seed).normal(0.0, sigma, cart.shape)
    return Crystal(np.full(len(cart), 26, dtype=np.int64), cart, lat)


def _min_image_dist2(frac_new, frac_old, lattice):
    d = frac_old - frac_new
    d -= np.round(d)
    # small triclinic cells: the minimum image may be a neighbouring translate
    best = None
    for s in [(i, j, k) for i in (-1, 0, 1) for j in (-1, 0, 1) for k in (-1, 0, 1)]:
        c = (d + np.asarray(s, float)) @ lattice
        d2 = (c * c).sum(axis=1)
        best = d2 if best is None else np.minimum(best, d2)
    return best


def random_crystal(rng: np.random.Generator, min_dist=1.2) -> Crystal:
    noble = {2, 10, 18, 36, 54}
    elements = np.array([z for z in range(1, 84) if z not in noble])
    n = int(rng.integers(8, 65))
    numbers = rng.choice(elements, size=n)
    while True:
        a, b, c = rng.uniform(4.0, 12.0, 3)
        al, be, ga = np.deg2rad(rng.uniform(70.0, 110.0, 3))
        cx = np.cos(be)
        cy = (np.cos(al) - np.cos(be) * np.cos(ga)) / np.sin(ga)
        cz2 = 1.0 - cx * cx - cy * cy
        if cz2 > 1e-3:
            break
    lat = np.array([[a, 0, 0], [b * np.cos(ga), b * np.sin(ga), 0], [c * cx, c * cy, c * np.sqrt(cz2)]])
    rho = rng.uniform(2.0, 8.0)
    mass = ATOMIC_WEIGHT[numbers].sum() * AMU_PER_A3_TO_G_PER_CM3
    vol = abs(np.linalg.det(lat))
    lat = lat * (mass / rho / vol) ** (1.0 / 3.0)
    frac = np.empty((n, 3))
    k = 0
    tries = 0
    while k < n:
        f = rng.uniform(0.0, 1.0, 3)
        tries += 1
        if k == 0 or _min_image_dist2(f, frac[:k], lat).min() >= min_dist ** 2 or tries > 20000:
            frac[k] = f
            k += 1
    return Crystal(numbers.astype(np.int64), frac @ lat, lat)


def random_crystals(count=256, seed=1) -> list[Crystal]:
    """Random triclinic crystals: 8-64 atoms, Z in 1..83 without noble gases, cell lengths
    4-12 A, angles 70-110 deg, rescaled to 2-8 g/cm^3, 1.2 A minimum separation."""
    rng = np.random.default_rng(seed)
    return [random_crystal(rng) for _ in range(count)]


def lipscl(n_atoms=4096, density=1.9, min_dist=1.6, seed=2) -> Crystal:
    """Amorphous Li6PS5Cl-ratio cell: cubic box at ``density`` g/cm^3, uniform positions
    with sequential rejection below ``min_dist``.  Composition: floor(n/13) formula units
    (6 Li, 1 P, 5 S, 1 Cl); any remainder atoms are Li."""
    rng = np.random.default_rng(seed)
    fu = n_atoms // 13
    numbers = np.array([3] * (6 * fu) + [15] * fu + [16] * (5 * fu) + [17] * fu + [3] * (n_atoms - 13 * fu),
                       dtype=np.int64)
    rng.shuffle(numbers)
    mass = ATOMIC_WEIGHT[numbers].sum() * AMU_PER_A3_TO_G_PER_CM3
    box = (mass / density) ** (1.0 / 3.0)
    ncell = max(1, int(box // min_dist))
    cw = box / ncell
    cells: dict[tuple, list] = {}
    pos = np.empty((n_atoms, 3))
    k = 0
    while k < n_atoms:
        p = rng.uniform(0.0, box, 3)
        ci = tuple((p // cw).astype(int) % ncell)
        ok = True
        for dx in (-1, 0, 1):
            for dy in (-1, 0, 1):
                for dz in (-1, 0, 1):
                    for q in cells.get(((ci[0] + dx) % ncell, (ci[1] + dy) % ncell, (ci[2] + dz) % ncell), ()):
                        d = pos[q] - p
                        d -= box * np.round(d / box)
                        if d @ d < min_dist ** 2:
                            ok = False
        if ok:
            pos[k] = p
            cells.setdefault(ci, []).append(k)
            k += 1
    return Crystal(numbers, pos, np.eye(3) * box)


def perovskites(count=4096, seed=4, sigma=0.1) -> list[Crystal]:
    """Random ABX3 2x2x2 supercells (40 atoms): A in {Ca,Sr,Ba,K,Cs}, B in
    {Ti,Zr,Nb,Mn,Fe,Co,Ni}, X in {O,F,Cl}; lattice 3.8-4.2 A; Gaussian noise on all positions."""
    rng = np.random.default_rng(seed)
    A, B, X = [20, 38, 56, 19, 55], [22, 40, 41, 25, 26, 27, 28], [8, 9, 17]
    basis = [[0, 0, 0], [0.5, 0.5, 0.5], [0.5, 0.5, 0], [0.5, 0, 0.5], [0, 0.5, 0.5]]
    out = []
    for _ in range(count):
        za, zb, zx = rng.choice(A), rng.choice(B), rng.choice(X)
        a = rng.uniform(3.8, 4.2)
        cart, lat = _supercell(basis, np.eye(3) * a, (2, 2, 2))
        cart = cart + rng.normal(0.0, sigma, cart.shape)
        out.append(Crystal(np.tile(np.array([za, zb, zx, zx, zx], dtype=np.int64), 8), cart, lat))
    return out


def demo_pu4si6() -> Crystal:
    """A 10-atom P1 cell with the lattice of the reference's example structure
    (a=4.260, b=c=7.167 A): short axis < cutoff, so self-image bonds occur."""
    rng = np.random.default_rng(7)
    lat = np.diag([4.260, 7.167, 7.167])
    frac = np.array([[0.0, 0.0, 0.0], [0.5, 0.5, 0.0], [0.0, 0.5, 0.5], [0.5, 0.0, 0.5],
                     [0.25, 0.2, 0.3], [0.75, 0.8, 0.7], [0.25, 0.7, 0.8], [0.75, 0.3, 0.2],
                     [0.5, 0.25, 0.75], [0.0, 0.75, 0.25]])
    frac = frac + rng.normal(0, 0.01, frac.shape)
    return Crystal(np.array([94] * 4 + [14] * 6, dtype=np.int64), frac @ lat, lat)
