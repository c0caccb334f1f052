"""Regenerate matris_b200/data/atomref.json: the three per-element reference-energy tables that
the reference hard-codes (matris/model/reference_energy.py:116-207) and ships
inside every checkpoint as ``reference_energy.fc.weight``.  They are read out of
the reference's own ``AtomRef`` module so that ``MatRIS(reference_energy=...)``
built here starts from bit-identical values.

Run where a copy of the reference tree exists:
    MATRIS_REFERENCE_ROOT=<reference tree> python tests/golden/make_atomref.py
"""
import json
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from oracle.refshim import import_reference  # noqa: E402


def main():
    import_reference(os.environ.get("MATRIS_REFERENCE_ROOT"))
    import importlib
    AtomRef = importlib.import_module("matris.model.reference_energy").AtomRef
    out = {}
    for name in ("mptrj", "omat", "mpa"):
        w = AtomRef(reference_energy=name).fc.weight.detach().view(-1)
        out[name] = [float.hex(float(v)) for v in w]  # exact float32 values
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "matris_b200", "data", "atomref.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=0)
    print("wrote", path)


if __name__ == "__main__":
    main()
