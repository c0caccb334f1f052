"""matris_b200: B200-native (sm_100a) evaluation path for the MatRIS interatomic potential.

Public surface mirrors the reference package: ``MatRIS`` (model and checkpoint
interface), ``GraphConverter`` / ``RadiusGraph`` (graph package), and
``MatRISCalculator`` / ``StructOptimizer`` / ``MolecularDynamics`` (applications).
"""
from .graph import GraphConverter, RadiusGraph, datatype  # noqa: F401
from .model import MatRIS  # noqa: F401

__version__ = "0.1.0"


def __getattr__(name):
    if name in ("MatRISCalculator", "StructOptimizer", "MolecularDynamics"):
        from . import applications
        return getattr(applications, name)
    raise AttributeError(name)
