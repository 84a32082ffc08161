"""MD state and noise stream: the data contract of FastMACE's ``SimulationState`` / ``RandomStream``
(``fastmace/state.py:274-394``) with the fields the NVT Langevin path uses.

All tensors are float64 on the device except ``species``; velocities (not momenta) are stored; ``masses`` is
``(N, 1)``; tensors keep fixed addresses and are updated in place (``state.py:3-7``).
"""

from __future__ import annotations

import dataclasses
from types import SimpleNamespace
from typing import Any

import numpy as np
import torch


class RandomStream:
    """Host NumPy generator plus the drawn-ahead device batch and its cursor (``state.py`` ``RandomStream``)."""

    def __init__(self, generator: np.random.Generator):
        self.generator = generator
        self.batch: torch.Tensor | None = None     # (k, 2, N, 3) float64 on the device
        self.cursor: int = 0                       # host mirror of the device cursor


@dataclasses.dataclass
class SimulationState:
    positions: torch.Tensor
    velocities: torch.Tensor
    masses: torch.Tensor
    cell: torch.Tensor
    species: torch.Tensor
    forces: torch.Tensor
    energy: torch.Tensor
    stress: torch.Tensor | None
    rng: RandomStream
    step: int = 0

    @classmethod
    def from_structure(cls, structure: Any, device, seed: int, compute_stress: bool = False) -> "SimulationState":
        """From an object with ``positions``, ``velocities`` (or None), ``masses``, ``cell``, ``numbers``
        (``SimulationState.from_atoms``, ``state.py:340-378``)."""
        f64 = dict(dtype=torch.float64, device=device)
        positions = torch.tensor(np.asarray(structure.positions), **f64)
        velocities = structure.velocities if getattr(structure, "velocities", None) is not None else \
            np.zeros_like(structure.positions)
        return cls(positions=positions, velocities=torch.tensor(np.asarray(velocities), **f64),
                   masses=torch.tensor(np.asarray(structure.masses)[:, None], **f64),
                   cell=torch.tensor(np.asarray(structure.cell), **f64),
                   species=torch.tensor(np.asarray(structure.numbers), dtype=torch.int64, device=device),
                   forces=torch.zeros_like(positions), energy=torch.zeros(1, **f64),
                   stress=torch.zeros((3, 3), **f64) if compute_stress else None,
                   rng=RandomStream(np.random.default_rng(seed)))

    @classmethod
    def from_atoms(cls, atoms: Any, device, seed: int, compute_stress: bool = False) -> "SimulationState":
        """From an ASE-style object (``get_positions``, ``get_velocities``, ``get_masses``, ``get_cell``,
        ``get_atomic_numbers``; ``state.py:340-378``). Constraints are outside this path and raise."""
        if getattr(atoms, "constraints", None):
            raise ValueError("constraints are not supported on this path")
        velocities = atoms.get_velocities()
        structure = SimpleNamespace(positions=np.asarray(atoms.get_positions()),
                                    velocities=None if velocities is None else np.asarray(velocities),
                                    masses=np.asarray(atoms.get_masses()), cell=np.asarray(atoms.get_cell()),
                                    numbers=np.asarray(atoms.get_atomic_numbers()))
        return cls.from_structure(structure, device, seed, compute_stress)

    @property
    def natoms(self) -> int:
        return self.positions.shape[0]

    @property
    def momenta(self) -> torch.Tensor:
        return self.velocities * self.masses


__all__ = ["SimulationState", "RandomStream"]
