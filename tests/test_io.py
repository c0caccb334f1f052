"""CPU: plain-text structure / trajectory files (extended XYZ, POSCAR, P1 CIF) round-trip without ASE or pymatgen."""
import numpy as np
import pytest

from matris_b200 import io as mio
from matris_b200 import workloads
from matris_b200.applications import SimpleAtoms


def _atoms(seed=0):
    cr = workloads.random_crystals(1, seed=seed)[0]
    a = SimpleAtoms(cr.numbers, cr.cart, cr.lattice)
    a.set_momenta(np.random.default_rng(seed).normal(size=a.positions.shape))
    return a


def test_extxyz_round_trip_with_results(tmp_path):
    frames = [_atoms(1), _atoms(2)]
    rng = np.random.default_rng(0)
    results = [dict(energy=-3.25 * (k + 1), forces=rng.normal(size=f.positions.shape), stress=rng.normal(size=(3, 3)),
                    magmoms=rng.normal(size=len(f))) for k, f in enumerate(frames)]
    p = str(tmp_path / "traj.xyz")
    mio.write_extxyz(p, frames[0], results=results[0])
    mio.write_extxyz(p, frames[1:], append=True, results=results[1:])
    back = mio.read_extxyz(p)
    assert len(back) == 2
    for a, b, r in zip(frames, back, results):
        assert np.array_equal(a.numbers, b.numbers) and b.pbc.all()
        np.testing.assert_allclose(b.positions, a.positions, rtol=0, atol=1e-9)
        np.testing.assert_allclose(b.cell, a.cell, rtol=0, atol=1e-9)
        np.testing.assert_allclose(b.momenta, a.momenta, rtol=1e-10)
        np.testing.assert_allclose(b.arrays["forces"], r["forces"], rtol=1e-10)
        np.testing.assert_allclose(b.arrays["magmoms"], r["magmoms"], rtol=1e-10)
        np.testing.assert_allclose(b.info["stress"].reshape(3, 3), r["stress"], rtol=1e-10)
        assert abs(b.info["energy"] - r["energy"]) < 1e-10
    assert np.array_equal(mio.read_extxyz(p, index=-1).numbers, frames[1].numbers)


def test_plain_xyz_and_truncated_file(tmp_path):
    p = tmp_path / "m.xyz"
    p.write_text("3\nwater\nO 0 0 0\nH 0.96 0 0\nH -0.24 0.93 0\n")
    a = mio.read_extxyz(str(p), index=0)
    assert list(a.numbers) == [8, 1, 1] and not a.pbc.any() and a.info.get("water") == "T"
    p.write_text("3\nwater\nO 0 0 0\n")
    with pytest.raises(ValueError):
        mio.read_extxyz(str(p))


def test_poscar_round_trip_groups_species(tmp_path):
    a = _atoms(3)
    p = str(tmp_path / "POSCAR")
    mio.write_poscar(p, a)
    b = mio.read_poscar(p)
    order = np.argsort(a.numbers, kind="stable")
    assert np.array_equal(b.numbers, a.numbers[order])
    np.testing.assert_allclose(b.cell, a.cell, atol=1e-12)
    np.testing.assert_allclose(b.positions, a.positions[order], atol=1e-9)


def test_cif_p1_and_symmetry_rejection(tmp_path):
    p = tmp_path / "nacl.cif"
    p.write_text("""data_x
_cell_length_a 4.0(1)
_cell_length_b 5.0
_cell_length_c 6.0
_cell_angle_alpha 90
_cell_angle_beta 100.0
_cell_angle_gamma 90
loop_
_symmetry_equiv_pos_as_xyz
 'x, y, z'
loop_
_atom_site_label
_atom_site_type_symbol
_atom_site_fract_x
_atom_site_fract_y
_atom_site_fract_z
Na1 Na 0.0 0.0 0.0
Cl1 Cl 0.5 0.5 0.5(2)
""")
    a = mio.read_cif(str(p))
    assert list(a.numbers) == [11, 17]
    lengths = np.linalg.norm(a.cell, axis=1)
    np.testing.assert_allclose(lengths, [4.0, 5.0, 6.0], atol=1e-12)
    cosb = a.cell[0] @ a.cell[2] / (lengths[0] * lengths[2])
    assert abs(np.degrees(np.arccos(cosb)) - 100.0) < 1e-9
    np.testing.assert_allclose(a.positions[1], 0.5 * a.cell.sum(axis=0), atol=1e-12)
    p.write_text(p.read_text().replace(" 'x, y, z'", " 'x, y, z'\n '-x, -y, -z'"))
    with pytest.raises(ValueError):
        mio.read_cif(str(p))


def test_reference_demo_cif_is_read():
    """The structure file the reference ships (example/cif_file/demo.cif, Pu4Si6, P1; a copy sits in tests/golden):
    10 sites, and the same arrays the committed golden case was generated from."""
    import os

    from conftest import GOLDEN, load_golden
    a = mio.read_cif(os.path.join(GOLDEN, "demo.cif"))
    assert list(a.get_atomic_numbers()) == [94] * 4 + [14] * 6
    np.testing.assert_allclose(np.diag(a.get_cell()), [4.26022438, 7.16692875, 7.16692875], atol=1e-12)
    _, crystals, _ = load_golden("democif_L2")
    assert np.array_equal(crystals[0].numbers, a.get_atomic_numbers())
    np.testing.assert_allclose(crystals[0].cart, a.get_positions(), atol=1e-12)
    np.testing.assert_allclose(crystals[0].lattice, a.get_cell(), atol=1e-12)
