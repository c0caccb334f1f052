"""Import the real reference implementation (test infrastructure only).

The reference imports ``pymatgen.core.Structure`` purely as a type
(matris/graph/converter.py:13, matris/model/reference_energy.py:7) and ``ase``
only in matris/applications.  Neither is installed, so stub modules are placed
in ``sys.modules`` before ``matris.graph`` / ``matris.model`` are imported.
Works only where the reference tree is present; callers treat ``ImportError``
as "reference unavailable".
"""
from __future__ import annotations

import importlib
import os
import sys
import types

_HERE = os.path.dirname(os.path.abspath(__file__))


def _install_stubs() -> None:
    try:
        import pymatgen.core  # noqa: F401  (a real install wins)
        return
    except Exception:
        pass
    pmg = types.ModuleType("pymatgen")
    core = types.ModuleType("pymatgen.core")

    class Structure:  # used by the reference only for isinstance / annotations
        pass

    core.Structure = Structure
    pmg.core = core
    sys.modules["pymatgen"] = pmg
    sys.modules["pymatgen.core"] = core


def import_reference(root: str | None = None):
    """Return a namespace with the reference's graph and model modules.

    When ``oracle/_ref`` holds the compiled ``cygraph`` extension (built by
    oracle/build_ref.sh from the reference's own C sources) it is attached as
    ``matris.graph.cygraph`` and ``ns.make_graph`` is the reference's C builder;
    otherwise ``ns.make_graph`` is None and only the legacy Python builder exists.
    """
    root = root or os.environ.get("MATRIS_REFERENCE_ROOT")
    if not root:
        raise ImportError("set MATRIS_REFERENCE_ROOT to a copy of the reference tree")
    if not os.path.isdir(os.path.join(root, "matris")):
        raise ImportError(f"reference tree not found under {root}")
    _install_stubs()
    if root not in sys.path:
        sys.path.insert(0, root)
    graph = importlib.import_module("matris.graph")
    converter = importlib.import_module("matris.graph.converter")
    make_graph = getattr(converter, "make_graph", None)
    so_dir = os.path.join(_HERE, "_ref")
    if make_graph is None and os.path.isdir(so_dir):
        if so_dir not in graph.__path__:
            graph.__path__.append(so_dir)
        try:
            cyg = importlib.import_module("matris.graph.cygraph")
            make_graph = cyg.make_graph
            converter.make_graph = make_graph
        except ImportError:
            make_graph = None
    model = importlib.import_module("matris.model.model")
    return types.SimpleNamespace(
        graph=graph,
        converter=converter,
        radiusgraph=importlib.import_module("matris.graph.radiusgraph"),
        processgraph=importlib.import_module("matris.model.processgraph"),
        model=model,
        MatRIS=model.MatRIS,
        make_graph=make_graph,
    )
