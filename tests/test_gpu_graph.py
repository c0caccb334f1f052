"""GPU: graph build through the C ABI against the oracle, bit-exact.

The CUDA builder emits directed edges sorted by (centre, neighbour, image) - the
order of the oracle's neighbour list - so every tensor must be IDENTICAL to what
the reference's Graph classes give on that list (and to the committed goldens)."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN_CASES, load_golden
from matris_b200 import workloads
from matris_b200.workloads import Crystal

pytestmark = pytest.mark.gpu


def oracle_graph(cr, cutoff=6.0, lc=4.0):
    from oracle import graph as og
    from oracle.neighbors import neighbor_list
    c, n, im, d = neighbor_list(cr.cart, cr.lattice, cutoff)
    d2u, u2d, rev = og.build_graph(c, n, im)
    lg = og.line_graph(c, n, d, d2u, u2d, rev, lc)
    return dict(center=c, neighbor=n, image=im, dist=d, d2u=d2u, u2d=u2d, rev=rev, line_graph=lg)


def check_batch(crystals, cutoff=6.0, lc=4.0):
    from matris_b200.graph import build_batched_graph, split_batch
    g = build_batched_graph([c.numbers for c in crystals], [c.cart for c in crystals], [c.lattice for c in crystals],
                            cutoff, lc, "cuda")
    ap, ep, bp, tp = g.structure_slices()
    cpu = {k: getattr(g, k).cpu().numpy() for k in ("center", "neighbor", "image", "dist64", "rev", "d2u", "u2d",
                                                    "line_graph", "trip_ptr", "trip_src_ptr", "trip_src_perm",
                                                    "edge_ptr")}
    for b, cr in enumerate(crystals):
        o = oracle_graph(cr, cutoff, lc)
        e0, e1, u0, u1, t0, t1, a0 = ep[b], ep[b + 1], bp[b], bp[b + 1], tp[b], tp[b + 1], ap[b]
        assert e1 - e0 == len(o["center"]), f"structure {b}: {e1 - e0} edges, oracle {len(o['center'])}"
        assert np.array_equal(cpu["center"][e0:e1] - a0, o["center"])
        assert np.array_equal(cpu["neighbor"][e0:e1] - a0, o["neighbor"])
        assert np.array_equal(cpu["image"][e0:e1], o["image"])
        assert np.array_equal(cpu["dist64"][e0:e1], o["dist"]), "float64 bond lengths must be bit-identical"
        assert np.array_equal(cpu["rev"][e0:e1] - e0, o["rev"])
        assert np.array_equal(cpu["d2u"][e0:e1] - u0, o["d2u"])
        assert np.array_equal(cpu["u2d"][u0:u1] - e0, o["u2d"])
        assert t1 - t0 == len(o["line_graph"])
        if t1 > t0:
            lg = cpu["line_graph"][t0:t1] - np.array([a0, u0, e0, u0, e0])
            assert np.array_equal(lg, o["line_graph"])
    # CSR consistency of the whole batch
    lg = cpu["line_graph"]
    T = g.n_triplets
    assert cpu["trip_ptr"][-1] == T and cpu["trip_src_ptr"][-1] == T
    if T:
        assert np.array_equal(np.repeat(np.arange(g.n_bonds), np.diff(cpu["trip_ptr"])), lg[:, 1])
        perm = cpu["trip_src_perm"]
        assert np.array_equal(np.sort(perm), np.arange(T))
        assert np.array_equal(np.repeat(np.arange(g.n_bonds), np.diff(cpu["trip_src_ptr"])), lg[perm, 3])
    assert np.array_equal(np.repeat(np.arange(g.n_atoms), np.diff(cpu["edge_ptr"])), cpu["center"])
    # the reference-layout per-structure views
    for rg, cr in zip(split_batch(g), crystals):
        o = oracle_graph(cr, cutoff, lc)
        assert np.array_equal(rg.atom_graph.cpu().numpy(), np.stack([o["center"], o["neighbor"]], 1))
        assert np.array_equal(rg.neighbor_image.cpu().numpy(), o["image"].astype(np.float32))
        assert len(rg.directed2undirected) == 2 * len(rg.undirected2directed)
    return g


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_graph_matches_golden(case):
    meta, crystals, z = load_golden(case)
    g = check_batch(crystals)
    # and against the tensors the REFERENCE's Graph produced (committed fixtures)
    ap, ep, bp, tp = g.structure_slices()
    for b in range(len(crystals)):
        assert np.array_equal(g.d2u.cpu().numpy()[ep[b]:ep[b + 1]] - bp[b], z[f"d2u{b}"])
        assert np.array_equal(g.u2d.cpu().numpy()[bp[b]:bp[b + 1]] - ep[b], z[f"u2d{b}"])
        lg = g.line_graph.cpu().numpy()[tp[b]:tp[b + 1]] - np.array([ap[b], bp[b], ep[b], bp[b], ep[b]])
        assert np.array_equal(lg, z[f"line_graph{b}"].reshape(-1, 5))


def test_random_crystal_batch():
    check_batch(workloads.random_crystals(24, seed=1))


def test_perovskite_batch():
    check_batch(workloads.perovskites(8, seed=4))


def test_larger_cells_use_cell_list():
    check_batch([workloads.fe_bcc((6, 6, 6)), workloads.lipscl(512)])


def test_unwrapped_coordinates_and_small_cell():
    cr = workloads.cu_fcc(reps=(1, 1, 1), sigma=0.01, seed=3)
    shifted = Crystal(cr.numbers, cr.cart + np.array([2.3, -1.7, 0.4]) @ cr.lattice, cr.lattice)
    check_batch([cr, shifted])


def test_cutoff_ties_follow_reference_rule():
    """Bond lengths exactly on the line-graph cutoff: target side uses <=, source side <."""
    cubic = Crystal(np.array([26]), np.zeros((1, 3)), np.eye(3) * 4.0)
    two = Crystal(np.array([26, 8]), np.array([[0.0, 0, 0], [2.0, 0, 0]]), np.eye(3) * 4.0)
    g = check_batch([cubic, two])
    assert g.n_triplets > 0


def test_isolated_atom_raises_value_error():
    from matris_b200.graph import GraphConverter
    cr = Crystal(np.array([1, 1]), np.array([[0.0, 0, 0], [10.0, 10, 10]]), np.eye(3) * 30.0)
    with pytest.raises(ValueError, match="isolated atom"):
        GraphConverter()(cr)


def test_converter_single_structure_reference_layout():
    from matris_b200.graph import GraphConverter
    cr = workloads.demo_pu4si6()
    rg = GraphConverter(6, 4)(cr, graph_id="x")
    o = oracle_graph(cr)
    assert rg.graph_id == "x" and rg.atomic_number.dtype == torch.int32
    assert rg.atom_frac_coord.dtype == torch.float32 and rg.lattice.shape == (3, 3)
    assert np.array_equal(rg.line_graph.cpu().numpy(), o["line_graph"])
    assert rg.to("cuda").atom_graph.is_cuda


def test_capacity_too_small_is_reported_and_retried():
    """Undersized edge / triplet buffers: the builder reports the sizes it needed in the device status block, the host
    enlarges the buffers and runs it again; the result is the same graph.  Rebuilding after the positions changed on
    the device reuses the buffers."""
    from matris_b200 import graph as G
    crystals = workloads.random_crystals(6, seed=2)
    ref = check_batch(crystals)
    hb = G.HostBatch([c.numbers for c in crystals], [c.cart for c in crystals], [c.lattice for c in crystals], 6.0)
    g = G.upload(hb, 6.0, 4.0, torch.device("cuda"))
    g._buffers = G._GraphBuffers(g, 64, 8, g.cart64.device)  # far too small on purpose
    G.build_on_device(g)
    assert (g.n_edges, g.n_bonds, g.n_triplets) == (ref.n_edges, ref.n_bonds, ref.n_triplets)
    assert g._buffers.cap_e >= g.n_edges and g._buffers.cap_t >= g.n_triplets
    for k in ("center", "neighbor", "image", "rev", "d2u", "u2d", "line_graph", "trip_src_perm", "trip_ptr"):
        assert torch.equal(getattr(g, k), getattr(ref, k)), k
    buffers = g._buffers
    g.cart64 += 0.01
    G.build_on_device(g)
    assert g._buffers is buffers and g.n_edges > 0


def test_periodic_image_beyond_the_packed_range_is_an_error_before_anything_is_paired():
    """An atom that has drifted more than 127 cell lengths away from its neighbours (unwrapped coordinates in a long
    run): the image index does not fit the packed key.  The counting pass reports it and the build stops there."""
    from matris_b200._lib import MbError
    from matris_b200.graph import build_batched_graph
    cr = workloads.cu_fcc(reps=(1, 1, 1), sigma=0.0)
    cart = cr.cart.copy()
    cart[0] += 200 * cr.lattice[0]
    with pytest.raises(MbError, match="out of range"):
        build_batched_graph([cr.numbers], [cart], [cr.lattice])


GRAPH_FIELDS = ("edge_ptr", "center", "neighbor", "image", "dist64", "rev", "d2u", "u2d", "trip_ptr", "trip_src_ptr",
                "line_graph", "trip_src_perm")


def _same_graph(a, b, what):
    assert (a.n_edges, a.n_bonds, a.n_triplets) == (b.n_edges, b.n_bonds, b.n_triplets), what
    for k in GRAPH_FIELDS:
        assert torch.equal(getattr(a, k), getattr(b, k)), f"{what}: {k} differs from the fresh build"


@pytest.mark.parametrize("skin", [0.3, 1.0])
def test_verlet_skin_reuse_gives_the_fresh_graph(skin):
    """A random walk of all atoms: every step's graph from the candidate list must be bit-identical to a full rebuild
    at the same positions, across steps that keep the list and steps that trigger its rebuild; the list must be
    rebuilt when (and only when) an atom has moved half the skin since the last rebuild."""
    from matris_b200.graph import HostBatch, build_on_device, set_positions_on_device, upload
    crystals = workloads.random_crystals(6, seed=11) + [workloads.cu_fcc()]
    args = ([c.numbers for c in crystals], [c.cart for c in crystals], [c.lattice for c in crystals])
    g_skin = upload(HostBatch(*args, 6.0), 6.0, 4.0, torch.device("cuda"))
    g_full = upload(HostBatch(*args, 6.0), 6.0, 4.0, torch.device("cuda"))
    x = g_skin.cart64.clone()
    gen = torch.Generator(device="cuda").manual_seed(3)
    ref = x.clone()
    expected_rebuilds = 0
    for step in range(14):
        if step:
            scale = 0.25 if step == 9 else 0.03   # one large move among small ones
            x = x + scale * torch.randn(x.shape, dtype=torch.float64, device="cuda", generator=gen)
        moved = float((x - ref).norm(dim=1).max())
        if step == 0 or moved >= 0.5 * skin:
            expected_rebuilds += 1
            ref = x.clone()
        for g in (g_skin, g_full):
            set_positions_on_device(g, x)
        build_on_device(g_skin, skin=skin)
        build_on_device(g_full)
        _same_graph(g_skin, g_full, f"skin {skin}, step {step}")
        assert int(g_skin._candidates.flag[1]) == expected_rebuilds, f"step {step}: moved {moved:.3f}"
    assert expected_rebuilds < 14, "the walk never reused a list: the test would show nothing"


def test_verlet_skin_candidate_capacity_grows():
    """A candidate buffer that is too small is enlarged and the build repeated; the result is still the fresh graph."""
    from matris_b200 import graph as G
    crystals = workloads.random_crystals(4, seed=5)
    args = ([c.numbers for c in crystals], [c.cart for c in crystals], [c.lattice for c in crystals])
    g_skin = G.upload(G.HostBatch(*args, 6.0), 6.0, 4.0, torch.device("cuda"))
    g_full = G.upload(G.HostBatch(*args, 6.0), 6.0, 4.0, torch.device("cuda"))
    g_skin._candidates = G._Candidates(g_skin, 0.5, 512, torch.device("cuda"))  # far too few candidates
    G.build_on_device(g_skin, skin=0.5)
    G.build_on_device(g_full)
    assert g_skin._candidates.cap > 512
    _same_graph(g_skin, g_full, "after the candidate buffers grew")


def test_verlet_skin_isolated_atom_is_reported():
    from matris_b200 import graph as G
    from matris_b200._lib import MbError
    lat = np.eye(3) * 30.0
    g = G.upload(G.HostBatch([np.array([29, 29])], [np.array([[0.0, 0, 0], [15.0, 15, 15]])], [lat], 6.0), 6.0, 4.0,
                 torch.device("cuda"))
    with pytest.raises((ValueError, MbError)):
        G.build_on_device(g, skin=0.5)
