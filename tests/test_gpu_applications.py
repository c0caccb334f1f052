"""GPU: the application layer (calculator / relax / MD) on top of the CUDA path, without ASE."""
import numpy as np
import pytest
import torch

from conftest import GPA, load_golden
from gpu_util import report
from matris_b200 import workloads
from matris_b200.weights import random_checkpoint
from matris_b200.workloads import Crystal

pytestmark = pytest.mark.gpu


def _atoms(cr):
    from matris_b200.applications import SimpleAtoms
    return SimpleAtoms(cr.numbers, cr.cart, cr.lattice)


def test_calculator_results_match_reference_conversion():
    """MatRISCalculator.calculate: total energy = e/atom * n, stress GPa -> eV/A^3 (base.py:108-122)."""
    from matris_b200.applications import MatRISCalculator
    meta, crystals, z = load_golden("pu4si6_L2")
    ck = random_checkpoint(dict(num_layers=2, reference_energy="mpa"), seed=0, jitter=meta["jitter"])
    calc = MatRISCalculator(model=ck, task="efsm", device="cuda")
    atoms = _atoms(crystals[0])
    calc.calculate(atoms)
    n = len(crystals[0].numbers)
    r = calc.results
    report("calculator energy (eV)", np.array([r["energy"]]), z["ref32_e"] * n, 1e-5 * n)
    report("calculator ref_energy (eV)", np.array([r["ref_energy"]]), z["ref32_ref_energy"] * n, 1e-5)
    report("calculator forces", r["forces"], z["ref32_f"], 1e-4)
    report("calculator stress (eV/A^3)", r["stress"], z["ref32_s"][0] / GPA, 1e-5)
    report("calculator magmoms", r["magmoms"], z["ref32_m"], 1e-4)
    assert r["stress"].shape == (3, 3) and set(r) >= {"energy", "forces", "stress", "magmoms", "ref_energy"}
    calc2 = MatRISCalculator(model=calc.model, task="e", device="cuda")
    calc2.calculate(atoms)
    assert calc2.results["forces"] is None and calc2.results["stress"] is None


def test_calculator_non_periodic_axis_gets_a_big_box():
    from matris_b200.applications import MatRISCalculator, SimpleAtoms
    ck = random_checkpoint(dict(num_layers=1, reference_energy="mpa"), seed=0)
    cr = workloads.cu_fcc(reps=(2, 2, 1))
    atoms = SimpleAtoms(cr.numbers, cr.cart, cr.lattice, pbc=[True, True, False])
    MatRISCalculator(model=ck, task="ef", device="cuda").calculate(atoms)
    assert atoms.get_cell()[2, 2] > 100.0  # the cell of the caller's object is changed, as in the reference


def test_nve_energy_conservation_and_langevin_runs():
    from matris_b200.applications import MolecularDynamics
    ck = random_checkpoint(dict(num_layers=2, reference_energy="mpa"), seed=0)
    from matris_b200 import MatRIS
    model = MatRIS.from_dict(ck).to("cuda")
    md = MolecularDynamics(_atoms(workloads.cu_fcc()), model=model, ensemble="nve", timestep=1.0,
                           starting_temperature=300, task="ef", device="cuda")
    e0 = md.atoms.get_potential_energy() + md.atoms.get_kinetic_energy()
    md.run(20)
    e1 = md.atoms.get_potential_energy() + md.atoms.get_kinetic_energy()
    assert abs(e1 - e0) < 2e-3 * len(md.atoms), (e0, e1)
    md2 = MolecularDynamics(_atoms(workloads.cu_fcc()), model=model, ensemble="nvt", thermostat="langevin",
                            temperature=600, starting_temperature=600, timestep=1.0, task="efsm", device="cuda")
    md2.run(5)
    assert md2.steps_done == 5 and np.isfinite(md2.atoms.get_temperature())


def test_device_resident_nve_follows_the_host_loop():
    """Velocity Verlet has no noise: the loop with its state on the GPU must retrace the host-driven loop."""
    from matris_b200 import MatRIS
    from matris_b200.applications import MolecularDynamics
    model = MatRIS.from_dict(random_checkpoint(dict(num_layers=2, reference_energy="mpa"), seed=0)).to("cuda")
    runs = []
    for resident in (False, True):
        md = MolecularDynamics(_atoms(workloads.cu_fcc()), model=model, ensemble="nve", timestep=1.0,
                               starting_temperature=300, task="ef", device="cuda", seed=5, device_resident=resident)
        md.run(10)
        md.run(5)  # a second call continues from the stored state
        assert md.steps_done == 15
        runs.append((md.atoms.get_positions(), md.atoms.get_momenta()))
    report("device-resident NVE positions vs host loop", torch.tensor(runs[1][0]), torch.tensor(runs[0][0]), 1e-6)
    report("device-resident NVE momenta vs host loop", torch.tensor(runs[1][1]), torch.tensor(runs[0][1]), 1e-5)


def test_md_with_a_verlet_skin_retraces_the_rebuild_every_step_trajectory():
    """Neighbour-list reuse changes how the graph is found, not the graph: a hot NVE run (atoms move far enough to
    trigger candidate rebuilds) with a skin must retrace the run that rebuilds at every step, up to the summation
    order of the force scatter (float atomics)."""
    from matris_b200 import MatRIS
    from matris_b200.applications import MolecularDynamics
    model = MatRIS.from_dict(random_checkpoint(dict(num_layers=2, reference_energy="mpa"), seed=0)).to("cuda")
    runs = []
    for skin in (0.0, 0.4):
        md = MolecularDynamics(_atoms(workloads.random_crystals(1, seed=3)[0]), model=model, ensemble="nve", timestep=2.0,
                               starting_temperature=3000, task="ef", device="cuda", seed=5, skin=skin)
        md.run(40)
        runs.append((md.atoms.get_positions(), md.atoms.get_momenta()))
    moved = np.abs(runs[0][0] - workloads.random_crystals(1, seed=3)[0].cart).max()
    assert moved > 0.2, f"atoms moved {moved:.3f} A only: no candidate rebuild was exercised"
    # two runs of the SAME loop differ by this much too: the force scatter's float atomics reorder from run to run and a
    # hot trajectory amplifies the last bits (measured 1e-6 A after 40 steps); a wrong graph would show as 1e-2 A
    report("NVE positions with skin 0.4 vs rebuild every step", torch.tensor(runs[1][0]), torch.tensor(runs[0][0]), 2e-5)
    report("NVE momenta with skin 0.4 vs rebuild every step", torch.tensor(runs[1][1]), torch.tensor(runs[0][1]), 2e-4)


def test_device_resident_evaluation_equals_predict_at_the_same_positions():
    """The loops that keep their state on the GPU derive the model's float32 positions from the float64 ones on the
    device; the results stored at the end must be those of a fresh evaluation of the final positions."""
    from matris_b200 import MatRIS
    from matris_b200.applications import MolecularDynamics
    model = MatRIS.from_dict(random_checkpoint(dict(num_layers=2, reference_energy="mpa"), seed=0)).to("cuda")
    cr = workloads.random_crystals(3, seed=14)[1]  # triclinic: the fractional / Cartesian round trip is not trivial
    md = MolecularDynamics(_atoms(cr), model=model, ensemble="nve", timestep=1.0, starting_temperature=500,
                           task="efsm", device="cuda", seed=3, device_resident=True)
    md.run(4)
    stored = dict(md.atoms.calc.results)
    fresh = model.predict([Crystal(cr.numbers, md.atoms.get_positions(), cr.lattice)], "efsm")
    n = len(cr.numbers)
    report("device loop vs predict: energy (eV/atom)", np.array([stored["energy"] / n]), fresh["e"].cpu(), 1e-6)
    report("device loop vs predict: forces", stored["forces"], fresh["f"][0].cpu(), 2e-6)
    report("device loop vs predict: stress (eV/A^3)", stored["stress"], fresh["s"][0].cpu() / GPA, 1e-7)
    report("device loop vs predict: magmoms", stored["magmoms"], fresh["m"][0].cpu(), 2e-6)


def test_langevin_thermostat_holds_the_target_temperature():
    """Statistical check of the device-resident BAOAB loop: the mean kinetic temperature over 3,000 steps of the
    32-atom Cu cell at 600 K.  Samples are taken 75 steps apart (several velocity correlation times at a friction
    of 0.05 / fs); one sample of 32 atoms scatters by sqrt(2 / (3 N)) = 14 %, the mean of 40 by 14 K: the bound is
    3 sigma."""
    from matris_b200 import MatRIS
    from matris_b200.applications import MolecularDynamics
    model = MatRIS.from_dict(random_checkpoint(dict(num_layers=1, reference_energy="mpa"), seed=0)).to("cuda")
    md = MolecularDynamics(_atoms(workloads.cu_fcc()), model=model, ensemble="nvt", thermostat="langevin",
                           temperature=600, starting_temperature=600, timestep=1.0, friction=0.05, task="ef",
                           device="cuda", seed=11)
    md.run(300)  # equilibration
    temps = []
    for _ in range(40):
        md.run(75)
        temps.append(md.atoms.get_temperature())
    mean, sigma = float(np.mean(temps)), 600.0 * np.sqrt(2.0 / (3 * 32)) / np.sqrt(len(temps))
    print(f"Langevin: mean kinetic temperature {mean:.1f} K over {md.steps_done} steps (sigma of the mean {sigma:.1f} K)")
    assert abs(mean - 600.0) < 3 * sigma + 5.0, (mean, sigma)
    assert np.isfinite(md.atoms.get_potential_energy())


def test_md_writes_an_extxyz_trajectory(tmp_path):
    from matris_b200 import MatRIS
    from matris_b200.applications import MolecularDynamics
    from matris_b200.io import read_extxyz
    model = MatRIS.from_dict(random_checkpoint(dict(num_layers=1, reference_energy="mpa"), seed=0)).to("cuda")
    for resident in (True, False):
        path = str(tmp_path / f"traj_{int(resident)}.xyz")
        md = MolecularDynamics(_atoms(workloads.cu_fcc()), model=model, ensemble="nve", timestep=1.0,
                               starting_temperature=300, task="ef", device="cuda", trajectory=path, loginterval=2,
                               device_resident=resident)
        md.run(6)
        frames = read_extxyz(path)
        assert len(frames) == 3 and len(frames[-1]) == 32
        np.testing.assert_allclose(frames[-1].positions, md.atoms.get_positions(), atol=1e-8)
        assert "forces" in frames[-1].arrays and "energy" in frames[-1].info


def test_relax_lowers_the_force():
    from matris_b200.applications import StructOptimizer
    ck = random_checkpoint(dict(num_layers=2, reference_energy="mpa"), seed=0)
    opt = StructOptimizer(model=ck, task="efs", optimizer="FIRE", device="cuda")
    atoms = _atoms(workloads.demo_pu4si6())
    opt.calculator.calculate(atoms)
    f0 = np.abs(opt.calculator.results["forces"]).max()
    out = opt.relax(atoms, fmax=1e-4, steps=15, verbose=False)
    assert set(out) == {"final_structure", "trajectory"} and len(out["trajectory"]) >= 2
    assert out["trajectory"].energies[-1] <= out["trajectory"].energies[0] + 1e-6
    assert np.isfinite(f0)


def test_device_resident_fire_follows_the_host_loop_and_evaluates_once_per_step():
    """FIRE with its state on the GPU retraces the host loop; with result caching one geometry costs one evaluation
    whichever of energy / forces / stress / magmoms the observer asks for."""
    from matris_b200 import MatRIS
    from matris_b200.applications import StructOptimizer
    model = MatRIS.from_dict(random_checkpoint(dict(num_layers=2, reference_energy="mpa"), seed=0)).to("cuda")
    finals = []
    for resident in (False, True):
        opt = StructOptimizer(model=model, task="efsm", optimizer="FIRE", device="cuda")
        calls = {"n": 0}
        inner = model._evaluate

        def counting(g, task, _inner=inner, _calls=calls):
            _calls["n"] += 1
            return _inner(g, task)

        model._evaluate = counting
        try:
            out = opt.relax(_atoms(workloads.demo_pu4si6()), fmax=1e-6, steps=6, verbose=False, device_resident=resident)
        finally:
            model._evaluate = inner
        assert len(out["trajectory"]) == 7 and calls["n"] == 7, (len(out["trajectory"]), calls["n"])
        finals.append((out["final_structure"].get_positions(), np.array(out["trajectory"].energies, dtype=float)))
    report("device-resident FIRE positions vs host loop", torch.tensor(finals[1][0]), torch.tensor(finals[0][0]), 1e-6)
    report("device-resident FIRE energies vs host loop", torch.tensor(finals[1][1]), torch.tensor(finals[0][1]), 1e-5)
