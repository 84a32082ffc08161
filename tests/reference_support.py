"""Access to the reference package for the tests that drive it (the planner registration and FastMACE's own
``GraphEngine`` over the CUDA force field). It is looked for on ``sys.path`` first, then in ``baseline/_ref`` (an
install made with ``pip install --no-deps --target baseline/_ref <reference tree>``; not part of the repository), then
in the directory ``FASTMACE_REFERENCE`` names. Tests skip when it is nowhere."""
import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def require_fastmace():
    candidates = [None, os.path.join(ROOT, "baseline", "_ref"), os.environ.get("FASTMACE_REFERENCE")]
    for path in candidates:
        if path is not None:
            if not os.path.isdir(os.path.join(path, "fastmace")):
                continue
            if path not in sys.path:
                sys.path.insert(0, path)
        try:
            return importlib.import_module("fastmace")
        except ImportError:
            continue
    pytest.skip("the fastmace package is not importable here (no install under baseline/_ref)")


class AtomsView:
    """The few ``ase.Atoms`` members ``SimulationState.from_atoms`` and the planner hook read, over a structure of
    this package (ASE itself is not a dependency)."""

    def __init__(self, structure):
        import numpy as np
        self.s = structure
        self.constraints = []
        self.pbc = np.array([True, True, True])
        self.numbers = np.asarray(structure.numbers)

        class _Cell:
            array = np.asarray(structure.cell)
        self.cell = _Cell()

    def __len__(self):
        return self.s.natoms

    def get_positions(self):
        return self.s.positions

    def get_velocities(self):
        return self.s.velocities

    def get_masses(self):
        return self.s.masses

    def get_atomic_numbers(self):
        return self.numbers
