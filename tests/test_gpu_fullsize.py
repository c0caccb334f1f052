"""GPU: BASELINE-size structures checked through size-independent properties (no oracle run at these sizes):
graph counting identities, zero net force, supercell extensivity, permutation and rotation behaviour."""
import numpy as np
import pytest
import torch

from gpu_util import report
from matris_b200 import workloads
from matris_b200.weights import random_checkpoint
from matris_b200.workloads import Crystal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model():
    from matris_b200 import MatRIS
    ck = random_checkpoint(dict(num_layers=2, reference_energy="mpa"), seed=0)
    return MatRIS.from_dict(ck).to("cuda")


def _graph_identities(g):
    """Identities every valid graph satisfies (radiusgraph.py:92-95, 412-487)."""
    assert g.n_edges == 2 * g.n_bonds
    rev = g.rev.long()
    assert torch.equal(rev[rev], torch.arange(g.n_edges, device=rev.device))
    assert torch.equal(g.center[rev], g.neighbor) and torch.equal(g.image[rev], -g.image)
    d = g.dist64
    assert float(d.min()) > 1e-8 and float(d.max()) <= g.cutoff
    # triplets: sum over atoms of n(n-1), n = bonds shorter than the line cutoff at that atom (no ties here)
    short = (d < g.line_cutoff)
    n_short = torch.zeros(g.n_atoms, dtype=torch.long, device=d.device).index_add_(0, g.center.long(), short.long())
    assert g.n_triplets == int((n_short * (n_short - 1)).sum())
    lg = g.line_graph.long()
    assert torch.equal(g.center.long()[lg[:, 2]], lg[:, 0]) and torch.equal(g.center.long()[lg[:, 4]], lg[:, 0])
    assert torch.equal(g.d2u.long()[lg[:, 2]], lg[:, 1]) and torch.equal(g.d2u.long()[lg[:, 4]], lg[:, 3])
    assert bool((lg[:, 2] != lg[:, 4]).all())
    perm = g.trip_src_perm.long()
    assert torch.equal(torch.sort(perm)[0], torch.arange(g.n_triplets, device=perm.device))


def test_fe16k_graph_identities_and_zero_net_force(model):
    cr = workloads.fe_bcc()  # 16,000 atoms
    g = model.graph_converter.batch([cr])
    assert g.n_atoms == 16000 and g.n_edges > 900_000 and g.n_triplets > 3_000_000
    _graph_identities(g)
    out = model(g, task="efs")
    f = out["f"][0]
    assert torch.isfinite(f).all() and torch.isfinite(out["s"][0]).all()
    report("fe16k net force (eV/A)", f.sum(0), torch.zeros(3), 2e-3)
    report("fe16k stress symmetry", out["s"][0], out["s"][0].T, 1e-4)


def test_lipscl_4096_graph_identities_and_magmoms(model):
    cr = workloads.lipscl()  # 4,096 atoms
    g = model.graph_converter.batch([cr])
    assert g.n_atoms == 4096
    _graph_identities(g)
    out = model(g, task="efsm")
    assert out["m"][0].shape == (4096,) and bool((out["m"][0] >= 0).all())
    report("lipscl net force (eV/A)", out["f"][0].sum(0), torch.zeros(3), 2e-3)


def test_supercell_extensivity_permutation_rotation(model):
    cr = workloads.random_crystals(3, seed=12)[2]
    base = model.predict([cr], "efs")
    n = len(cr.numbers)
    # 2x1x1 supercell: same energy per atom, same forces on the images, same stress
    sup = Crystal(np.concatenate([cr.numbers, cr.numbers]), np.concatenate([cr.cart, cr.cart + cr.lattice[0]]),
                  cr.lattice * np.array([[2.0], [1.0], [1.0]]))
    o2 = model.predict([sup], "efs")
    report("supercell E/atom", o2["e"], base["e"], 2e-6)
    report("supercell forces", o2["f"][0][:n], base["f"][0], 5e-6)
    report("supercell stress (GPa)", o2["s"][0], base["s"][0], 2e-4)
    # permutation of the atoms permutes the forces
    p = np.random.default_rng(0).permutation(n)
    op = model.predict([Crystal(cr.numbers[p], cr.cart[p], cr.lattice)], "efs")
    report("permutation E", op["e"], base["e"], 2e-6)
    report("permutation forces", op["f"][0], base["f"][0][torch.as_tensor(p, device="cuda")], 5e-6)
    # rigid rotation: energy invariant, forces rotate, stress transforms as a tensor
    rot, _ = np.linalg.qr(np.random.default_rng(1).normal(size=(3, 3)))
    if np.linalg.det(rot) < 0:
        rot[:, 0] *= -1
    o_r = model.predict([Crystal(cr.numbers, cr.cart @ rot, cr.lattice @ rot)], "efs")
    r = torch.as_tensor(rot, dtype=torch.float32, device="cuda")
    report("rotation E", o_r["e"], base["e"], 2e-6)
    report("rotation forces", o_r["f"][0], base["f"][0] @ r, 1e-5)
    report("rotation stress (GPa)", o_r["s"][0], r.T @ base["s"][0] @ r, 5e-4)


def test_translation_across_cell_boundary(model):
    """Unwrapped coordinates: shifting all atoms by a non-lattice vector changes images, not results."""
    cr = workloads.demo_pu4si6()
    base = model.predict([cr], "ef")
    moved = model.predict([Crystal(cr.numbers, cr.cart + np.array([3.3, -9.1, 12.7]), cr.lattice)], "ef")
    report("translation E", moved["e"], base["e"], 2e-6)
    report("translation forces", moved["f"][0], base["f"][0], 5e-6)
