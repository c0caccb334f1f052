"""Generate the committed golden vectors by running the REFERENCE ITSELF.

Run where a copy of the reference tree exists (it is imported, never copied):

    MATRIS_REFERENCE_ROOT=<reference tree> python tests/golden/make_golden.py [case ...]

With case names only those cases are regenerated; without, all of them.

For each case the structure comes from matris_b200.workloads (seeded), the
neighbour list from oracle.neighbors (brute-force float64, standing in for
pymatgen), the graph from the reference's own ``Graph`` classes (legacy Python
builder and, when oracle/_ref holds it, the compiled C builder - both must
agree), and E/F/S/M from the reference's ``MatRIS.forward`` on CPU in float32
and float64 with weights from matris_b200.weights.random_state_dict.

Outputs: tests/golden/<case>.npz (inputs, reference graph tensors, reference
results) and tests/golden/schema.json (the reference's state_dict key list).
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from matris_b200 import workloads  # noqa: E402
from matris_b200.weights import random_state_dict  # noqa: E402
from oracle.neighbors import neighbor_list  # noqa: E402
from oracle.refshim import import_reference  # noqa: E402

CASES = {
    # name: (crystal factory, num_layers, task, weight jitter[, extra constructor arguments])
    "cu32_L10": (lambda: workloads.cu_fcc(), 10, "efsm", 0.0),
    "cu32_L2_jit": (lambda: workloads.cu_fcc(), 2, "efsm", 0.1),
    "cu32_ideal_L1": (lambda: workloads.cu_fcc(sigma=0.0), 1, "efsm", 0.1),  # exact 180-degree triplets
    "random2_L2": (lambda: workloads.random_crystals(2, seed=11), 2, "efs", 0.1),
    "pu4si6_L2": (lambda: workloads.demo_pu4si6(), 2, "efsm", 0.1),
    "cu1_L1": (lambda: workloads.cu_fcc(reps=(1, 1, 1), sigma=0.0), 1, "efsm", 0.1),  # self-image bonds only... 4 atoms
    "perov_L3": (lambda: workloads.perovskites(1, seed=5)[0], 3, "efsm", 0.1),
    # 432-atom BCC Fe: ~112k triplets, above the 60,000-triplet switch to torch.utils.checkpoint
    # (matris/model/interaction_block.py:15, 400-403)
    "fe432_L2": (lambda: workloads.fe_bcc(reps=(6, 6, 6)), 2, "efsm", 0.1),
    "lipscl256_L2": (lambda: workloads.lipscl(n_atoms=256), 2, "efsm", 0.1),
    # the first eight structures of the benchmark batch (the generator is sequential in its seed)
    "random8_L2": (lambda: workloads.random_crystals(8, seed=1), 2, "efs", 0.1),
    # the structure file the reference ships (example/cif_file/demo.cif; a copy sits beside this script)
    "democif_L2": (lambda: demo_cif(), 2, "efsm", 0.1),
    # non-default options: biases in the FFN layers, smoothed rows into the atom graph's edge update
    "random2_L2_bias_smoothed": (lambda: workloads.random_crystals(2, seed=11), 2, "efsm", 0.1,
                                 dict(use_bias=True, use_smoothed_for_delta_edge=True)),
    # non-default bases: Gaussian distance expansion, Fourier angle expansion
    "random2_L2_gaussian_fourier": (lambda: workloads.random_crystals(2, seed=11), 2, "efsm", 0.1,
                                    dict(distance_expansion="Gaussian", three_body_expansion="fourier")),
    # the plain-MLP variant of the update blocks, with biases
    "random2_L2_mlp_bias": (lambda: workloads.random_crystals(2, seed=11), 2, "efsm", 0.1,
                            dict(graph_conv_mlp="MLP", use_bias=True)),
}


def demo_cif():
    from matris_b200.io import read_cif
    a = read_cif(os.path.join(HERE, "demo.cif"))
    return workloads.Crystal(np.asarray(a.get_atomic_numbers(), dtype=np.int64), np.asarray(a.get_positions(), float),
                             np.asarray(a.get_cell(), float))


def reference_graph(ns, crystal, cutoff=6.0, line_cutoff=4.0):
    c, n, im, d = neighbor_list(crystal.cart, crystal.lattice, cutoff)
    conv = ns.converter.GraphConverter
    g = conv._create_graph_legacy(len(crystal.numbers), c, n, im, d)
    ag, d2u = g.adjacency_list()
    u2d = g.undirected2directed()
    lg = g.line_graph_adjacency_list(line_cutoff)
    if ns.make_graph is not None:
        g2 = conv._create_graph_fast(len(crystal.numbers), c, n, im, d)
        ag2, d2u2 = g2.adjacency_list()
        assert ag2 == [list(x) for x in ag] or np.array_equal(np.array(ag2), np.array(ag))
        assert d2u2 == d2u and g2.undirected2directed() == u2d
        assert g2.line_graph_adjacency_list(line_cutoff) == lg
    rg = ns.radiusgraph.RadiusGraph(
        graph_id=None, mp_id=None, composition=None,
        atomic_number=torch.tensor(crystal.numbers, dtype=torch.int32),
        atom_frac_coord=torch.tensor(crystal.frac, dtype=torch.float32),
        lattice=torch.tensor(crystal.lattice, dtype=torch.float32),
        neighbor_image=torch.tensor(im, dtype=torch.float32),
        atom_graph=torch.tensor(np.array(ag).reshape(-1, 2), dtype=torch.int32), atom_graph_cutoff=cutoff,
        line_graph=torch.tensor(lg, dtype=torch.int32), line_graph_cutoff=line_cutoff,
        directed2undirected=torch.tensor(d2u, dtype=torch.int32),
        undirected2directed=torch.tensor(u2d, dtype=torch.int32))
    return rg, (c, n, im, d)


def run_reference(ns, graphs, layers, task, jitter, double, extra=None):
    cfg = dict(num_layers=layers, reference_energy="mpa", **(extra or {}))
    model = ns.MatRIS(**cfg)
    model.load_state_dict(random_state_dict(cfg, seed=0, jitter=jitter))
    model.eval()
    if double:
        model = model.double()
        model.reference_energy.float()
        graphs = [ns.radiusgraph.RadiusGraph(**{**g.to_dict(),
                                                "atom_frac_coord": g.atom_frac_coord.double(),
                                                "lattice": g.lattice.double(),
                                                "neighbor_image": g.neighbor_image.double()}) for g in graphs]
    pooled = []  # EnergyHead output: per-structure total energy before the division by atoms and before AtomRef
    hook = model.energy_head.register_forward_hook(lambda m, a, k, o: pooled.append(o.detach()), with_kwargs=True)
    out = model(graphs, task=task)
    hook.remove()
    res = {"e": out["e"].detach().double().numpy(), "ref_energy": out["ref_energy"].detach().double().numpy(),
           "e_model": (pooled[-1] / out["atoms_per_graph"]).double().numpy()}
    if "f" in out:
        res["f"] = torch.cat(list(out["f"])).detach().double().numpy()
    if "s" in out:
        res["s"] = torch.stack(out["s"]).detach().double().numpy()
    if "m" in out:
        res["m"] = torch.cat(out["m"]).detach().double().numpy()
    return res


def main():
    ns = import_reference(os.environ.get("MATRIS_REFERENCE_ROOT"))
    only = set(sys.argv[1:])
    unknown = only - set(CASES)
    if unknown:
        raise SystemExit(f"unknown cases: {sorted(unknown)}")
    torch.set_num_threads(os.cpu_count() or 1)
    ref_model = ns.MatRIS(num_layers=2, reference_energy="mpa")
    with open(os.path.join(HERE, "schema.json"), "w") as f:
        json.dump({"num_layers": 2, "reference_energy": "mpa",
                   "keys": [[k, list(v.shape)] for k, v in ref_model.state_dict().items()]}, f, indent=0)
    for name, case in CASES.items():
        factory, layers, task, jitter = case[:4]
        extra = case[4] if len(case) > 4 else {}
        if only and name not in only:
            continue
        crystals = factory()
        if not isinstance(crystals, list):
            crystals = [crystals]
        graphs, arrays = [], {}
        for b, cr in enumerate(crystals):
            rg, (c, n, im, d) = reference_graph(ns, cr)
            graphs.append(rg)
            arrays.update({f"numbers{b}": cr.numbers, f"cart{b}": cr.cart, f"lattice{b}": cr.lattice,
                           f"nl_center{b}": c.astype(np.int32), f"nl_neighbor{b}": n.astype(np.int32),
                           f"nl_image{b}": im.astype(np.int8), f"nl_distance{b}": d,
                           f"d2u{b}": rg.directed2undirected.numpy(), f"u2d{b}": rg.undirected2directed.numpy(),
                           f"line_graph{b}": rg.line_graph.numpy().reshape(-1, 5).astype(np.int32)})
        r32 = run_reference(ns, graphs, layers, task, jitter, False, extra)
        r64 = run_reference(ns, graphs, layers, task, jitter, True, extra)
        for k, v in r32.items():
            arrays["ref32_" + k] = v
        for k, v in r64.items():
            arrays["ref64_" + k] = v
        arrays["meta"] = np.array(json.dumps(dict(n_structures=len(crystals), num_layers=layers, task=task,
                                                  jitter=jitter, seed=0, reference_energy="mpa", config=extra)))
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **arrays)
        print(name, {k: float(np.abs(r32[k] - r64[k]).max()) for k in r32},
              "Fmax", float(np.abs(r32.get("f", np.zeros(1))).max()))


if __name__ == "__main__":
    main()
