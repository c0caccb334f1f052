import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def load_golden(name):
    """Return (meta, crystals, arrays) for a committed golden case."""
    from matris_b200.workloads import Crystal
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    meta = json.loads(str(z["meta"]))
    crystals = [Crystal(z[f"numbers{b}"], z[f"cart{b}"], z[f"lattice{b}"]) for b in range(meta["n_structures"])]
    return meta, crystals, z


GOLDEN_CASES = ["cu32_L10", "cu32_L2_jit", "cu32_ideal_L1", "random2_L2", "pu4si6_L2", "cu1_L1", "perov_L3",
                "fe432_L2", "lipscl256_L2", "random8_L2", "democif_L2", "random2_L2_bias_smoothed",
                "random2_L2_gaussian_fourier", "random2_L2_mlp_bias"]


def golden_config(meta):
    """Constructor arguments of a golden case: layers, reference energy and any non-default options."""
    return dict(num_layers=meta["num_layers"], reference_energy=meta["reference_energy"], **meta.get("config", {}))

# tolerances of the evaluation path (energy eV/atom, force eV/A, stress eV/A^3, magmom mu_B)
TOL = dict(e=1e-5, f=1e-4, s=1e-5, m=1e-4)
GPA = 160.21766208


@pytest.fixture(scope="session")
def golden_loader():
    return load_golden
