"""Callers of the evaluation path with the reference's application API.

``MatRISCalculator`` / ``StructOptimizer`` / ``MolecularDynamics`` keep the
constructor arguments, method names and result keys of
matris/applications/base.py:24-122, relax.py:22-143 and md.py:31-310.  ASE and
pymatgen are imported lazily: where ASE is installed the classes plug into it
exactly like the reference's (``MatRISCalculator`` then derives from
``ase.calculators.calculator.Calculator``); without ASE the calculator still
works on any object offering ``get_cell / get_positions / get_atomic_numbers /
get_pbc`` (and ``set_cell`` for non-periodic axes), and a small velocity-Verlet /
Langevin integrator stands in for the MD drivers.

Unit conventions of ``results`` (base.py:115-122): ``energy`` total eV,
``forces`` eV/A, ``stress`` 3x3 eV/A^3 (model GPa x units.GPa), ``magmoms`` mu_B,
``None`` for parts the task does not cover.
"""
from __future__ import annotations

import functools
import pickle

import numpy as np

from .graph import as_arrays
from .model import GPA_PER_EV_A3, MatRIS
from .workloads import ATOMIC_WEIGHT, Crystal

EV_A3_PER_GPA = 1.0 / GPA_PER_EV_A3          # ase.units.GPa
FS = 0.09822694788464063                      # ase.units.fs  (sqrt(amu A^2 / eV) per fs)^-1
KB = 8.617330337217213e-05                    # ase.units.kB, eV/K

try:  # ASE is optional
    from ase.calculators.calculator import Calculator as _AseCalculator
    from ase.calculators.calculator import all_changes as _all_changes
    from ase.calculators.calculator import all_properties as _all_properties
    HAVE_ASE = True
except Exception:  # pragma: no cover - depends on the environment
    HAVE_ASE = False

    class _AseCalculator:  # minimal stand-in with the attributes the code below relies on
        def __init__(self, **kwargs):
            self.results, self.atoms = {}, None

        def calculate(self, atoms=None, properties=None, system_changes=None):
            self.atoms = atoms

    _all_changes, _all_properties = [], []


def _resolve_model(model, device):
    if isinstance(model, MatRIS):
        return model.to(device) if device is not None else model
    if isinstance(model, dict):
        return MatRIS.from_dict(model).to(device or "cuda")
    return MatRIS.load(model_name=model, device=device)


class MatRISCalculator(_AseCalculator):
    """MatRIS calculator (matris/applications/base.py:24-122).  ``model`` is a checkpoint
    name as in the reference, or (extension) a path, a checkpoint dict or a ``MatRIS`` instance."""

    implemented_properties = ("energy", "forces", "stress", "magmoms")

    def __init__(self, model="matris_10m_oam", task: str = "efs", device: str = "cuda", **kwargs) -> None:
        super().__init__(**kwargs)
        self.task, self.device = task, device
        self.model = _resolve_model(model, device)
        self.stress_unit = EV_A3_PER_GPA
        self.key = {"atoms_per_graph", "ref_energy", *task}
        if not hasattr(self, "results") or self.results is None:
            self.results = {}

    def calculate(self, atoms=None, properties=None, system_changes=None) -> None:
        properties = properties or _all_properties
        system_changes = system_changes or _all_changes
        super().calculate(atoms=atoms, properties=properties, system_changes=system_changes)
        pbc = np.asarray(atoms.get_pbc(), dtype=bool) if hasattr(atoms, "get_pbc") else np.array([True] * 3)
        if not pbc.all():
            # non-periodic axes get a box large enough that no image is inside the receptive field
            # (same rule, and the same in-place change of the cell, as base.py:70-93)
            pos = atoms.get_positions()
            cell = np.array(atoms.get_cell(), dtype=float)
            big = (np.max(np.abs(pos)) + 1) * max(5, self.model.config["num_layers"]) * self.model.config["pairwise_cutoff"]
            for k in range(3):
                if not pbc[k]:
                    cell[k, :] = big * np.identity(3)[k, :]
            atoms.set_cell(cell, scale_atoms=False)
        numbers, cart, lattice = as_arrays(atoms)
        out = self.model.predict([Crystal(numbers, cart, lattice)], task=self.task)
        self.store_output(out, len(numbers))

    def store_output(self, out: dict, n_atoms_in_structure: int) -> None:
        """Fill ``results`` from a model output dictionary (the last structure of the batch), with the reference's
        unit conversions (base.py:115-122)."""
        n_atoms = n_atoms_in_structure if self.model.is_intensive else 1
        get = lambda k: out[k][-1].detach().cpu().numpy() if k in out else None  # noqa: E731  (last structure)
        ref = out["ref_energy"]
        ref = ref[-1].detach().cpu().numpy() if hasattr(ref, "detach") else np.float32(ref)
        stress = get("s")
        self.results.update(
            ref_energy=ref * n_atoms,
            energy=out["e"][-1].detach().cpu().numpy() * n_atoms,
            forces=get("f"),
            stress=None if stress is None else stress * self.stress_unit,
            magmoms=get("m"),
        )
        # the copies above synchronised the stream: a bounded wait that expired in this evaluation is known now
        self.model.check_status()

    # convenience for ASE-free use
    def get_property_dict(self, atoms) -> dict:
        self.calculate(atoms)
        return dict(self.results)


class TrajectoryObserver:
    """Records energies, forces, stresses, magmoms, positions and cells (base.py:128-175)."""

    def __init__(self, atoms) -> None:
        self.atoms = atoms
        self.energies, self.forces, self.stresses, self.magmoms = [], [], [], []
        self.atom_positions, self.cells = [], []

    def __call__(self) -> None:
        self.energies.append(self.compute_energy())
        self.forces.append(self.atoms.get_forces())
        self.stresses.append(self.atoms.get_stress())
        self.magmoms.append(self.atoms.get_magnetic_moments())
        self.atom_positions.append(self.atoms.get_positions())
        self.cells.append(self.atoms.get_cell()[:])

    def __len__(self) -> int:
        return len(self.energies)

    def compute_energy(self) -> float:
        return self.atoms.get_potential_energy()

    def save(self, filename: str) -> None:
        """Pickle of the recorded lists (base.py:163-175); a name ending in ``.xyz`` / ``.extxyz`` writes the frames
        as extended XYZ instead (an extension)."""
        if str(filename).endswith((".xyz", ".extxyz")):
            from .io import write_extxyz
            numbers = self.atoms.get_atomic_numbers()
            frames = [SimpleAtoms(numbers, p, c) for p, c in zip(self.atom_positions, self.cells)]
            results = [dict(energy=e, forces=f, stress=s, magmoms=m)
                       for e, f, s, m in zip(self.energies, self.forces, self.stresses, self.magmoms)]
            write_extxyz(filename, frames, results=results)
            return
        out = {"energy": self.energies, "forces": self.forces, "stresses": self.stresses, "magmoms": self.magmoms,
               "atom_positions": self.atom_positions, "cell": self.cells,
               "atomic_number": self.atoms.get_atomic_numbers()}
        with open(filename, "wb") as f:
            pickle.dump(out, f)


class CrystalFeasObserver:
    """Records ``results['crystal_fea']`` after each step (base.py:178-198)."""

    def __init__(self, atoms) -> None:
        self.atoms, self.crystal_feature_vectors = atoms, []

    def __call__(self) -> None:
        self.crystal_feature_vectors.append(self.atoms._calc.results["crystal_fea"])

    def __len__(self) -> int:
        return len(self.crystal_feature_vectors)

    def save(self, filename: str) -> None:
        with open(filename, "wb") as f:
            pickle.dump({"crystal_feas": self.crystal_feature_vectors}, f)


def _ase_optimizers():
    from ase.optimize import BFGS, FIRE, LBFGS, BFGSLineSearch, LBFGSLineSearch, MDMin
    return {"BFGS": BFGS, "BFGSLineSearch": BFGSLineSearch, "FIRE": FIRE, "LBFGS": LBFGS,
            "LBFGSLineSearch": LBFGSLineSearch, "MDMin": MDMin}


OPTIMIZER_NAMES = ["BFGS", "BFGSLineSearch", "FIRE", "LBFGS", "LBFGSLineSearch", "MDMin"]


class SimpleAtoms:
    """Minimal ASE-``Atoms``-like container for use without ASE (positions A, cell rows A, masses amu)."""

    def __init__(self, numbers, positions, cell, pbc=True, momenta=None):
        self.numbers = np.asarray(numbers, dtype=np.int64)
        self.positions = np.array(positions, dtype=float)
        self.cell = np.array(cell, dtype=float).reshape(3, 3)
        self.pbc = np.array([pbc] * 3 if isinstance(pbc, bool) else pbc, dtype=bool)
        self.masses = ATOMIC_WEIGHT[np.minimum(self.numbers, len(ATOMIC_WEIGHT) - 1)]
        self.momenta = np.zeros_like(self.positions) if momenta is None else np.array(momenta, dtype=float)
        self.calc = None

    def get_positions(self): return self.positions.copy()
    def set_positions(self, p): self.positions = np.array(p, dtype=float)
    def get_cell(self): return self.cell.copy()
    def set_cell(self, c, scale_atoms=False): self.cell = np.array(c, dtype=float).reshape(3, 3)
    def get_atomic_numbers(self): return self.numbers.copy()
    def get_pbc(self): return self.pbc.copy()
    def get_masses(self): return self.masses.copy()
    def get_momenta(self): return self.momenta.copy()
    def set_momenta(self, m): self.momenta = np.array(m, dtype=float)
    def get_velocities(self): return self.momenta / self.masses[:, None]
    def __len__(self): return len(self.numbers)

    def _state_key(self):
        return (self.positions.tobytes(), self.cell.tobytes(), self.numbers.tobytes(), self.pbc.tobytes())

    def mark_results_current(self) -> None:
        """Declare ``calc.results`` valid for the present positions / cell (used by the device-resident drivers)."""
        self._cache_key, self._cache_calc = self._state_key(), self.calc

    def _results(self):
        # one evaluation per geometry: energy, forces, stress and magmoms of the same state share it
        if getattr(self, "_cache_calc", None) is not self.calc or getattr(self, "_cache_key", None) != self._state_key():
            self.calc.calculate(self)
            self.mark_results_current()  # after calculate(): it may have enlarged the cell of a non-periodic axis
        return self.calc.results

    def get_potential_energy(self): return float(self._results()["energy"])
    def get_forces(self): return self._results()["forces"]
    def get_stress(self): return self._results()["stress"]
    def get_magnetic_moments(self): return self._results()["magmoms"]
    def get_kinetic_energy(self): return float(0.5 * (self.momenta ** 2 / self.masses[:, None]).sum())
    def get_temperature(self): return 2.0 * self.get_kinetic_energy() / (3.0 * len(self) * KB)


class StructOptimizer:
    """Structure relaxation (matris/applications/relax.py:22-143).  With ASE: any ASE optimizer and cell
    filter, as in the reference.  Without ASE: a built-in FIRE on the atomic positions (no cell relaxation)."""

    def __init__(self, model="matris_10m_oam", task: str = "efs", optimizer: str = "FIRE", device: str = "cuda"):
        if optimizer not in OPTIMIZER_NAMES:
            raise ValueError(f"Optimizer {optimizer} not found. Select from {OPTIMIZER_NAMES}")
        self.optimizer_name = optimizer
        self.optimizer = _ase_optimizers()[optimizer] if HAVE_ASE else None
        self.calculator = MatRISCalculator(model=model, task=task, device=device)

    def relax(self, atoms, fmax: float = 0.05, steps: int = 500, relax_cell: bool = True,
              ase_filter: str = "FrechetCellFilter", save_path: str = None, loginterval: int = 1,
              crystal_feas_save_path: str = None, verbose: bool = True, assign_magmoms: bool = True, **kwargs):
        if HAVE_ASE:
            return self._relax_ase(atoms, fmax, steps, relax_cell, ase_filter, save_path, loginterval,
                                   crystal_feas_save_path, verbose, assign_magmoms, **kwargs)
        if not hasattr(atoms, "set_positions"):
            numbers, cart, lattice = as_arrays(atoms)
            atoms = SimpleAtoms(numbers, cart, lattice)
        atoms.calc = self.calculator
        obs = TrajectoryObserver(atoms)
        relax_fn = fire_relax
        if kwargs.get("device_resident", True) and isinstance(atoms, SimpleAtoms) and bool(np.all(atoms.get_pbc())):
            relax_fn = functools.partial(fire_relax_device, skin=float(kwargs.get("skin", 0.0)))
        relax_fn(atoms, fmax=fmax, steps=steps, observer=obs, interval=loginterval, verbose=verbose)
        obs()
        if save_path is not None:
            obs.save(save_path)
        return {"final_structure": atoms, "trajectory": obs}

    def _relax_ase(self, atoms, fmax, steps, relax_cell, ase_filter, save_path, loginterval, crystal_feas_save_path,
                   verbose, assign_magmoms, **kwargs):  # pragma: no cover - needs ASE
        import contextlib
        import inspect
        import io
        import sys

        import ase.filters as filter_classes
        from ase.filters import Filter
        valid = [n for n, c in inspect.getmembers(filter_classes, inspect.isclass) if issubclass(c, Filter)]
        if isinstance(ase_filter, str):
            if ase_filter not in valid:
                raise ValueError(f"Invalid {ase_filter=}, must be one of {valid}. ")
            ase_filter = getattr(filter_classes, ase_filter)
        if not hasattr(atoms, "get_positions"):
            from pymatgen.io.ase import AseAtomsAdaptor
            atoms = AseAtomsAdaptor().get_atoms(atoms)
        atoms.calc = self.calculator
        stream = sys.stdout if verbose else io.StringIO()
        with contextlib.redirect_stdout(stream):
            obs = TrajectoryObserver(atoms)
            cry_obs = CrystalFeasObserver(atoms) if crystal_feas_save_path else None
            target = ase_filter(atoms) if relax_cell else atoms
            opt = self.optimizer(target, **kwargs)
            opt.attach(obs, interval=loginterval)
            if cry_obs is not None:
                opt.attach(cry_obs, interval=loginterval)
            opt.run(fmax=fmax, steps=steps)
            obs()
        if save_path is not None:
            obs.save(save_path)
        if cry_obs is not None:
            cry_obs.save(crystal_feas_save_path)
        final = atoms
        try:
            from pymatgen.io.ase import AseAtomsAdaptor
            final = AseAtomsAdaptor.get_structure(atoms)
            if assign_magmoms and atoms.get_magnetic_moments() is not None:
                for key in list(final.site_properties):
                    final.remove_site_property(property_name=key)
                final.add_site_property("magmom", [float(m) for m in atoms.get_magnetic_moments()])
        except ImportError:
            pass
        return {"final_structure": final, "trajectory": obs}


def fire_relax(atoms, fmax=0.05, steps=500, dt=0.1, dt_max=1.0, n_min=5, f_inc=1.1, f_dec=0.5, alpha0=0.1,
               f_alpha=0.99, max_step=0.2, observer=None, interval=1, verbose=False):
    """FIRE (Bitzek et al. 2006) on the positions; returns the number of steps taken."""
    v = np.zeros_like(atoms.get_positions())
    alpha, n_pos = alpha0, 0
    for it in range(steps):
        f = atoms.get_forces()
        if observer is not None and it % interval == 0:
            observer()
        fnorm = np.sqrt((f ** 2).sum(axis=1).max())
        if verbose:
            print(f"FIRE {it:4d}  E={atoms.get_potential_energy():.6f}  fmax={fnorm:.5f}")
        if fnorm < fmax:
            return it
        p = float((f * v).sum())
        if p > 0:
            v = (1 - alpha) * v + alpha * f / max(np.linalg.norm(f), 1e-30) * np.linalg.norm(v)
            if n_pos > n_min:
                dt, alpha = min(dt * f_inc, dt_max), alpha * f_alpha
            n_pos += 1
        else:
            v[:], alpha, dt, n_pos = 0.0, alpha0, dt * f_dec, 0
        v = v + dt * f
        step = dt * v
        norm = np.sqrt((step ** 2).sum(axis=1).max())
        if norm > max_step:
            step *= max_step / norm
        atoms.set_positions(atoms.get_positions() + step)
    return steps


def fire_relax_device(atoms, fmax=0.05, steps=500, dt=0.1, dt_max=1.0, n_min=5, f_inc=1.1, f_dec=0.5, alpha0=0.1,
                      f_alpha=0.99, max_step=0.2, observer=None, interval=1, verbose=False, skin=0.0):
    """``fire_relax`` with positions, velocities and forces kept on the GPU (an extension; the reference's loop,
    relax.py:116-123, goes through ASE on the host).  Per step the positions of the device-resident batch are updated
    in place, the graph is rebuilt on the device and the model evaluated; three scalars (max force, F.v and the
    norms) come back to the host for the FIRE decisions, and the full state only when the observer logs.
    ``skin`` > 0 (Angstrom) reuses the neighbour search between steps (graph.build_on_device); the graphs, and so
    the trajectory, are the same as with a rebuild at every step."""
    import torch

    from .graph import build_on_device, set_positions_on_device

    calc = atoms.calc
    model, task = calc.model, calc.task
    numbers, cart, lattice = as_arrays(atoms)
    g = model.graph_converter.batch([Crystal(numbers, cart, lattice)])
    x = g.cart64.clone()
    v = torch.zeros_like(x)
    alpha, n_pos = alpha0, 0

    def push_state(out):
        atoms.set_positions(x.cpu().numpy())
        calc.store_output(out, len(numbers))
        atoms.mark_results_current()

    it, out = 0, None
    for it in range(steps):
        if it > 0:
            set_positions_on_device(g, x)
            build_on_device(g, skin=skin)
        out = model(g, task=task)
        f = out["f"][0].to(torch.float64)
        stats = torch.stack([(f * f).sum(dim=1).max().sqrt(), (f * v).sum(), f.norm(), v.norm()]).tolist()
        fnorm, p, f_len, v_len = stats
        if observer is not None and it % interval == 0:
            push_state(out)
            observer()
        if verbose:
            print(f"FIRE {it:4d}  E={float(out['e'][0]) * (len(numbers) if model.is_intensive else 1):.6f}  fmax={fnorm:.5f}")
        if fnorm < fmax:
            push_state(out)
            return it
        if p > 0:
            v = (1 - alpha) * v + (alpha * v_len / max(f_len, 1e-30)) * f
            if n_pos > n_min:
                dt, alpha = min(dt * f_inc, dt_max), alpha * f_alpha
            n_pos += 1
        else:
            v = torch.zeros_like(v)
            alpha, dt, n_pos = alpha0, dt * f_dec, 0
        v = v + dt * f
        step = dt * v
        norm = float((step * step).sum(dim=1).max().sqrt())
        if norm > max_step:
            step = step * (max_step / norm)
        x = x + step
    # the loop ended on the step limit: evaluate the final positions so that the stored results match them
    set_positions_on_device(g, x)
    build_on_device(g, skin=skin)
    push_state(model(g, task=task))
    return steps


class MolecularDynamics:
    """Molecular dynamics (matris/applications/md.py:31-310).  With ASE the same ensembles / thermostats as the
    reference are built on ASE's integrators; ``thermostat='langevin'`` (NVT) is an extension.  Without ASE:
    ``nve`` (velocity Verlet) and ``nvt`` with ``thermostat='langevin'`` run on the built-in integrator."""

    def __init__(self, atoms, model="matris_10m_oam", ensemble: str = "nvt",
                 thermostat: str = "Berendsen_inhomogeneous", temperature: int = 300,
                 starting_temperature: int | None = None, timestep: float = 2.0, pressure: float = 1.01325e-4,
                 taut: float | None = None, taup: float | None = None, bulk_modulus: float | None = None,
                 trajectory=None, logfile: str | None = None, loginterval: int = 1,
                 crystal_feas_logfile: str | None = None, append_trajectory: bool = False, task: str = "efs",
                 device: str | None = "cuda", friction: float = 0.01, seed: int = 0,
                 device_resident: bool = True, skin: float = 0.0) -> None:
        self.ensemble, self.thermostat = ensemble, thermostat
        self.device_resident, self.seed, self.skin = bool(device_resident), int(seed), float(skin)
        self.temperature, self.timestep, self.friction = temperature, timestep, friction
        self.trajectory, self.logfile, self.loginterval = trajectory, logfile, loginterval
        self.crystal_feas_logfile = crystal_feas_logfile
        self.rng = np.random.default_rng(seed)
        if not hasattr(atoms, "get_positions"):
            numbers, cart, lattice = as_arrays(atoms)
            atoms = SimpleAtoms(numbers, cart, lattice)
        if starting_temperature is not None:
            if HAVE_ASE and not isinstance(atoms, SimpleAtoms):
                from ase.md.velocitydistribution import MaxwellBoltzmannDistribution, Stationary
                MaxwellBoltzmannDistribution(atoms, temperature_K=starting_temperature, force_temp=True)
                Stationary(atoms)
            else:
                maxwell_boltzmann(atoms, starting_temperature, self.rng)
        self.atoms = atoms
        self.atoms.calc = MatRISCalculator(model=model, device=device, task=task)
        taut = 100 * timestep if taut is None else taut
        taup = 1000 * timestep if taup is None else taup
        self.dyn = None
        if HAVE_ASE and not isinstance(atoms, SimpleAtoms):
            self.dyn = self._ase_dynamics(ensemble, thermostat, temperature, timestep, pressure, taut, taup,
                                          bulk_modulus, trajectory, logfile, loginterval, append_trajectory)
        else:
            ens, th = ensemble.lower(), thermostat.lower()
            if ens == "nve":
                self._mode = "nve"
            elif ens == "nvt" and th == "langevin":
                self._mode = "langevin"
            else:
                raise ValueError("without ASE only ensemble='nve' and ensemble='nvt' with thermostat='langevin' "
                                 "are available")
        self.steps_done = 0

    def _ase_dynamics(self, ensemble, thermostat, temperature, timestep, pressure, taut, taup, bulk_modulus,
                      trajectory, logfile, loginterval, append_trajectory):  # pragma: no cover - needs ASE
        from ase import units
        common = dict(trajectory=trajectory, logfile=logfile, loginterval=loginterval)
        ens, th = ensemble.lower(), thermostat.lower()
        if ens == "nve":
            from ase.md.verlet import VelocityVerlet
            return VelocityVerlet(atoms=self.atoms, timestep=timestep * units.fs, append_trajectory=append_trajectory,
                                  **common)
        if ens == "nvt":
            if th == "langevin":
                from ase.md.langevin import Langevin
                return Langevin(self.atoms, timestep=timestep * units.fs, temperature_K=temperature,
                                friction=self.friction / units.fs, append_trajectory=append_trajectory, **common)
            if th == "nose-hoover":
                from ase.md.npt import NPT
                self.upper_triangular_cell()
                return NPT(atoms=self.atoms, timestep=timestep * units.fs, temperature_K=temperature,
                           externalstress=pressure * units.GPa, ttime=taut * units.fs, pfactor=None,
                           append_trajectory=append_trajectory, **common)
            if th.startswith("berendsen"):
                from ase.md.nvtberendsen import NVTBerendsen
                return NVTBerendsen(atoms=self.atoms, timestep=timestep * units.fs, temperature_K=temperature,
                                    taut=taut * units.fs, append_trajectory=append_trajectory, **common)
            raise ValueError("Thermostat not supported, choose in 'Nose-Hoover', 'Berendsen', "
                             "'Berendsen_inhomogeneous', 'Langevin'")
        if ens == "npt":
            if bulk_modulus is None:
                print("Warning!!! no bulk modulus given, setting bulk modulus to 2 GPa. NPT simulation can proceed "
                      "with incorrect pressure relaxation time. User input for bulk modulus is recommended.")
                bulk_modulus = 2.0
            self.bulk_modulus = bulk_modulus
            compressibility_au = 1.0 / (bulk_modulus * units.GPa)
            if th == "nose-hoover":
                from ase.md.npt import NPT
                self.upper_triangular_cell()
                ptime = taup * units.fs
                return NPT(atoms=self.atoms, timestep=timestep * units.fs, temperature_K=temperature,
                           externalstress=pressure * units.GPa, ttime=taut * units.fs,
                           pfactor=bulk_modulus * units.GPa * ptime * ptime, append_trajectory=append_trajectory,
                           **common)
            if th == "berendsen_inhomogeneous":
                from ase.md.nptberendsen import Inhomogeneous_NPTBerendsen
                return Inhomogeneous_NPTBerendsen(atoms=self.atoms, timestep=timestep * units.fs,
                                                  temperature_K=temperature, pressure_au=pressure * units.GPa,
                                                  taut=taut * units.fs, taup=taup * units.fs,
                                                  compressibility_au=compressibility_au, **common)
            if th == "npt_berendsen":
                from ase.md.nptberendsen import NPTBerendsen
                return NPTBerendsen(atoms=self.atoms, timestep=timestep * units.fs, temperature_K=temperature,
                                    pressure_au=pressure * units.GPa, taut=taut * units.fs, taup=taup * units.fs,
                                    compressibility_au=compressibility_au, append_trajectory=append_trajectory,
                                    **common)
            raise ValueError("Thermostat not supported, choose in 'Nose-Hoover', 'Berendsen', "
                             "'Berendsen_inhomogeneous'")
        raise ValueError(f"unknown ensemble {ensemble!r}")

    def run(self, steps: int) -> None:
        """Run ``steps`` MD steps (thin wrapper of the ASE run; built-in integrator without ASE)."""
        if self.dyn is not None:  # pragma: no cover - needs ASE
            obs = None
            if self.crystal_feas_logfile:
                obs = CrystalFeasObserver(self.atoms)
                self.dyn.attach(obs, interval=self.loginterval)
            self.dyn.run(steps)
            if obs is not None:
                obs.save(self.crystal_feas_logfile)
            return
        if self.device_resident and bool(np.all(self.atoms.get_pbc())):
            self._run_on_device(steps)
            return
        a = self.atoms
        dt = self.timestep * FS
        m = a.get_masses()[:, None]
        f = a.get_forces()
        if self._mode == "langevin":
            # BAOAB splitting; friction is given per fs
            c1 = np.exp(-self.friction * self.timestep)
            c2 = np.sqrt((1.0 - c1 * c1) * KB * self.temperature) * np.sqrt(m)
        for _ in range(steps):
            p = a.get_momenta() + 0.5 * dt * f
            if self._mode == "langevin":
                a.set_positions(a.get_positions() + 0.5 * dt * p / m)
                p = c1 * p + c2 * self.rng.standard_normal(p.shape)
                a.set_positions(a.get_positions() + 0.5 * dt * p / m)
            else:
                a.set_positions(a.get_positions() + dt * p / m)
            f = a.get_forces()
            a.set_momenta(p + 0.5 * dt * f)
            self.steps_done += 1
            if self._logs_now():
                self._log_frame(a, dict(a.calc.results))

    def _run_on_device(self, steps: int) -> None:
        """The built-in integrators with the whole state on the GPU (an extension: the reference's loop,
        md.py:297-310, goes through the host every step).  Positions (fp64), momenta and forces stay in device
        memory; each step updates the batch's positions in place, rebuilds the graph there and evaluates the
        model; nothing is copied to the host until the run ends.  The thermostat noise comes from a torch CUDA
        generator seeded with ``seed + steps_done``, so a trajectory differs from the host loop's in its noise
        only.  ``skin`` > 0 (constructor argument, Angstrom) reuses the neighbour search between steps: the
        reference rebuilds its neighbour list at every step (base.py:96-97); here a candidate list with the cut-off
        enlarged by the skin is rebuilt only when an atom has moved by half the skin, and every step's graph is
        identical to the one a full rebuild gives."""
        import torch

        from .graph import build_on_device, set_positions_on_device

        a, calc = self.atoms, self.atoms.calc
        model, task = calc.model, calc.task
        if "f" not in task:
            raise ValueError("molecular dynamics needs forces: the task must contain 'f'")
        numbers, cart, lattice = as_arrays(a)
        g = model.graph_converter.batch([Crystal(numbers, cart, lattice)])
        dev = g.cart64.device
        dt = self.timestep * FS
        x = g.cart64.clone()
        p = torch.as_tensor(a.get_momenta(), dtype=torch.float64, device=dev)
        m = torch.as_tensor(a.get_masses(), dtype=torch.float64, device=dev)[:, None]
        gen = torch.Generator(device=dev)
        gen.manual_seed(self.seed + self.steps_done)
        if self._mode == "langevin":  # BAOAB splitting; friction is given per fs
            c1 = float(np.exp(-self.friction * self.timestep))
            c2 = torch.sqrt((1.0 - c1 * c1) * KB * self.temperature * m)
        out = model(g, task=task)
        f = out["f"][0].to(torch.float64)
        for _ in range(steps):
            p = p + 0.5 * dt * f
            if self._mode == "langevin":
                x = x + 0.5 * dt * p / m
                p = c1 * p + c2 * torch.randn(p.shape, dtype=torch.float64, device=dev, generator=gen)
                x = x + 0.5 * dt * p / m
            else:
                x = x + dt * p / m
            set_positions_on_device(g, x)
            build_on_device(g, skin=self.skin)
            out = model(g, task=task)
            f = out["f"][0].to(torch.float64)
            p = p + 0.5 * dt * f
            self.steps_done += 1
            if self._logs_now():  # the only host copies inside the loop, every ``loginterval`` steps
                frame = SimpleAtoms(numbers, x.cpu().numpy(), lattice, momenta=p.cpu().numpy())
                calc.store_output(out, len(numbers))
                self._log_frame(frame, dict(calc.results))
        a.set_positions(x.cpu().numpy())
        a.set_momenta(p.cpu().numpy())
        calc.store_output(out, len(numbers))
        if hasattr(a, "mark_results_current"):
            a.mark_results_current()

    def _logs_now(self) -> bool:
        return (self.dyn is None and isinstance(self.trajectory, str) and self.loginterval > 0
                and self.steps_done % self.loginterval == 0)

    def _log_frame(self, atoms, results) -> None:
        """Built-in integrators: append a frame to the extended-XYZ file named by ``trajectory``."""
        from .io import write_extxyz
        write_extxyz(self.trajectory, atoms, append=True, results=results)

    def set_atoms(self, atoms) -> None:
        calculator = self.atoms.calc
        self.atoms = atoms
        if self.dyn is not None:
            self.dyn.atoms = atoms
        self.atoms.calc = calculator

    def upper_triangular_cell(self, verbose: bool | None = False) -> None:  # pragma: no cover - needs ASE
        """ASE's Nose-Hoover NPT needs an upper-triangular cell (md.py:320-349)."""
        from ase.md.npt import NPT
        if not NPT._isuppertriangular(self.atoms.get_cell()):
            a, b, c, alpha, beta, gamma = self.atoms.cell.cellpar()
            angles = np.radians((alpha, beta, gamma))
            sin_a, sin_b, _ = np.sin(angles)
            cos_a, cos_b, cos_g = np.cos(angles)
            cos_p = np.clip((cos_g - cos_a * cos_b) / (sin_a * sin_b), -1, 1)
            sin_p = (1 - cos_p ** 2) ** 0.5
            self.atoms.set_cell([(a * sin_b * sin_p, a * sin_b * cos_p, a * cos_b), (0, b * sin_a, b * cos_a),
                                 (0, 0, c)], scale_atoms=True)
            if verbose:
                print("Transformed to upper triangular unit cell.", flush=True)


def maxwell_boltzmann(atoms, temperature_K: float, rng) -> None:
    """Draw momenta at ``temperature_K``, remove the centre-of-mass motion and rescale to the exact temperature."""
    m = atoms.get_masses()[:, None]
    p = rng.standard_normal((len(atoms), 3)) * np.sqrt(m * KB * temperature_K)
    p -= m * (p.sum(axis=0) / m.sum())
    atoms.set_momenta(p)
    t = atoms.get_temperature()
    if t > 0:
        atoms.set_momenta(p * np.sqrt(temperature_K / t))
