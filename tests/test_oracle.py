"""CPU: the oracle against the golden vectors produced by the reference itself."""
import json
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN, GOLDEN_CASES, GPA, TOL, golden_config, load_golden
from matris_b200.weights import random_checkpoint, schema
from oracle import graph as og
from oracle import pipeline
from oracle.neighbors import neighbor_list


def test_schema_matches_reference_state_dict():
    with open(os.path.join(GOLDEN, "schema.json")) as f:
        ref = json.load(f)
    mine = schema(dict(num_layers=ref["num_layers"], reference_energy=ref["reference_energy"]))
    assert [[k, list(v)] for k, v in mine.items()] == ref["keys"]


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_graph_restatement_matches_reference(case):
    meta, crystals, z = load_golden(case)
    for b, cr in enumerate(crystals):
        c, n, im, d = neighbor_list(cr.cart, cr.lattice, 6.0)
        assert np.array_equal(c, z[f"nl_center{b}"]) and np.array_equal(n, z[f"nl_neighbor{b}"])
        assert np.array_equal(im, z[f"nl_image{b}"]) and np.array_equal(d, z[f"nl_distance{b}"])
        d2u, u2d, rev = og.build_graph(c, n, im)
        assert np.array_equal(d2u, z[f"d2u{b}"]) and np.array_equal(u2d, z[f"u2d{b}"])
        lg = og.line_graph(c, n, d, d2u, u2d, rev, 4.0)
        assert np.array_equal(lg, z[f"line_graph{b}"])
        if len(c) < 5000:
            d2u_s, u2d_s = og.build_graph_sequential(c, n, im)
            assert np.array_equal(d2u_s, d2u) and np.array_equal(u2d_s, u2d)
            assert np.array_equal(og.line_graph_sequential(c, n, d, d2u, u2d, 4.0), lg)


def test_graph_restatement_order_independent_semantics():
    """Shuffled input order: sequential and closed-form builders still agree."""
    _, crystals, _ = load_golden("pu4si6_L2")
    c, n, im, d = neighbor_list(crystals[0].cart, crystals[0].lattice, 6.0)
    perm = np.random.default_rng(5).permutation(len(c))
    c, n, im, d = c[perm], n[perm], im[perm], d[perm]
    d2u, u2d, rev = og.build_graph(c, n, im)
    d2u_s, u2d_s = og.build_graph_sequential(c, n, im)
    assert np.array_equal(d2u, d2u_s) and np.array_equal(u2d, u2d_s)
    assert np.array_equal(og.line_graph(c, n, d, d2u, u2d, rev, 4.0),
                          og.line_graph_sequential(c, n, d, d2u, u2d, 4.0))


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_model_restatement_matches_reference(case):
    meta, crystals, z = load_golden(case)
    ckpt = random_checkpoint(golden_config(meta), seed=meta["seed"], jitter=meta["jitter"])
    torch.set_num_threads(min(8, os.cpu_count() or 1))
    res = pipeline.evaluate(ckpt, crystals, meta["task"])
    # same code path as the reference up to summation order: far inside the gates
    assert np.abs(res["e"] - z["ref32_e"]).max() < 2e-6
    assert np.abs(res["f"] - z["ref32_f"]).max() < 2e-6
    assert np.abs(res["s"] - z["ref32_s"]).max() / GPA < 1e-6
    if "m" in meta["task"]:
        assert np.abs(res["m"] - z["ref32_m"]).max() < 1e-5
    assert np.array_equal(res["ref_energy"], z["ref32_ref_energy"])


def test_model_restatement_fp64_matches_reference_fp64():
    meta, crystals, z = load_golden("pu4si6_L2")
    ckpt = random_checkpoint(dict(num_layers=meta["num_layers"], reference_energy="mpa"), seed=0, jitter=meta["jitter"])
    res = pipeline.evaluate(ckpt, crystals, meta["task"], dtype=torch.float64)
    assert np.abs(res["e"] - z["ref64_e"]).max() < 1e-7   # limited by the float32 reference-energy head
    assert np.abs(res["f"] - z["ref64_f"]).max() < 1e-10
    assert np.abs(res["s"] - z["ref64_s"]).max() < 1e-8
    assert np.abs(res["m"] - z["ref64_m"]).max() < 1e-10


def test_isolated_atom_raises():
    from matris_b200.workloads import Crystal
    cr = Crystal(np.array([1, 1]), np.array([[0.0, 0, 0], [10.0, 10, 10]]), np.eye(3) * 30.0)
    with pytest.raises(ValueError):
        pipeline.graph_from_arrays(cr.numbers, cr.cart, cr.lattice)
