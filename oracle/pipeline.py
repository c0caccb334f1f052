"""Structure -> graph -> E/F/S/M on CPU through the oracle (test infrastructure only).

Restates GraphConverter.forward (matris/graph/converter.py:63-129: float32
casts of fractional coordinates, lattice and images; isolated-atom check) and
the result conversion of MatRISCalculator.calculate
(matris/applications/base.py:108-122).
"""
from __future__ import annotations

import numpy as np
import torch

from . import graph as ograph
from . import model as omodel
from .neighbors import neighbor_list


def graph_from_arrays(numbers, cart, lattice, cutoff=6.0, line_cutoff=4.0, sequential=False):
    cart = np.asarray(cart, dtype=np.float64)
    lattice = np.asarray(lattice, dtype=np.float64)
    c, n, im, d = neighbor_list(cart, lattice, cutoff)
    if len(set(range(len(numbers))) - set(c.tolist())):
        raise ValueError("Error: Detected isolated atom. Calculation stopped")
    if sequential:
        d2u, u2d = ograph.build_graph_sequential(c, n, im)
        lg = ograph.line_graph_sequential(c, n, d, d2u, u2d, line_cutoff)
    else:
        d2u, u2d, rev = ograph.build_graph(c, n, im)
        lg = ograph.line_graph(c, n, d, d2u, u2d, rev, line_cutoff)
    frac = cart @ np.linalg.inv(lattice)
    return dict(
        atomic_number=torch.tensor(np.asarray(numbers), dtype=torch.int32),
        frac=torch.tensor(frac, dtype=torch.float32),
        lattice=torch.tensor(lattice, dtype=torch.float32),
        image=torch.tensor(im, dtype=torch.float32),
        atom_graph=torch.tensor(np.stack([c, n], axis=1), dtype=torch.int32),
        directed2undirected=torch.tensor(d2u, dtype=torch.int32),
        undirected2directed=torch.tensor(u2d, dtype=torch.int32),
        line_graph=torch.tensor(lg, dtype=torch.int32),
        distance=d,
    )


def evaluate(checkpoint, crystals, task="efsm", dtype=torch.float32, graphs=None):
    """Returns dict with e [B] (eV/atom incl. reference energy), f [N,3] eV/A,
    s [B,3,3] GPa, m [N] mu_B as float64 numpy arrays, plus 'graphs'."""
    if graphs is None:
        cfg = checkpoint["config"]
        graphs = [graph_from_arrays(c.numbers, c.cart, c.lattice, float(cfg.get("pairwise_cutoff", 6)),
                                    float(cfg.get("three_body_cutoff", 4))) for c in crystals]
    if dtype == torch.float64:
        graphs = [{**g, "frac": g["frac"].double(), "lattice": g["lattice"].double()} for g in graphs]
    out = omodel.forward(checkpoint["state_dict"], checkpoint["config"], graphs, task, dtype)
    res = {"e": out["e"].double().numpy(), "graphs": graphs,
           "ref_energy": out["ref_energy"].double().numpy() if torch.is_tensor(out["ref_energy"]) else out["ref_energy"]}
    if "f" in out:
        res["f"] = torch.cat(list(out["f"])).double().numpy()
    if "s" in out:
        res["s"] = torch.stack(out["s"]).double().numpy()
    if "m" in out:
        res["m"] = torch.cat(out["m"]).double().numpy()
    return res


def calculator_results(res, n_atoms, index=-1):
    """MatRISCalculator.calculate's conversion for one structure (base.py:108-122):
    total energy = e_per_atom * n_atoms; stress GPa -> eV/A^3."""
    gpa = 1.0 / omodel.GPA_PER_EV_A3
    return dict(energy=res["e"][index] * n_atoms, ref_energy=res["ref_energy"][index] * n_atoms,
                forces=res.get("f"), stress=None if "s" not in res else res["s"][index] * gpa,
                magmoms=res.get("m"))
