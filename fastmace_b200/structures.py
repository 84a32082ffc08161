"""Seeded synthetic structures of the benchmark configurations and the unit constants the MD path needs.

The reference builds its NaCl test cells with ASE (``tests/_support/structures.py:56-59``:
``bulk("NaCl", "rocksalt", a=5.64, cubic=True).repeat(...)`` then ``rattle``); ASE is not a dependency here, so the
lattices are written out and the jitter is defined explicitly as ``default_rng(seed).normal(0, sigma, (N, 3))``.
Velocities follow ``MaxwellBoltzmannDistribution``'s definition (``fastmace/quick.py:350-361``):
``v_i ~ N(0, kT / m_i)`` per component.

Unit constants are ASE's (CODATA 2014): time unit Å sqrt(amu/eV), ``FS`` = one femtosecond, ``KB`` in eV/K.
"""

from __future__ import annotations

import dataclasses
import math

import numpy as np

_E = 1.6021766208e-19
_AMU = 1.660539040e-27
_K = 1.38064852e-23
FS = 1.0e-5 * math.sqrt(_E / _AMU)       # one femtosecond in ASE time units (0.0982269...)
KB = _K / _E                              # Boltzmann constant, eV/K

ATOMIC_MASSES = {8: 15.999, 11: 22.98976928, 13: 26.9815385, 14: 28.085, 17: 35.45, 24: 51.9961, 26: 55.845,
                 27: 58.933194, 28: 58.6934, 18: 39.948}


@dataclasses.dataclass
class Structure:
    positions: np.ndarray        # [N, 3] float64, Å
    cell: np.ndarray             # [3, 3] float64, rows are lattice vectors
    numbers: np.ndarray          # [N] int64 atomic numbers
    velocities: np.ndarray | None = None   # [N, 3] float64, ASE units

    @property
    def natoms(self) -> int:
        return int(self.positions.shape[0])

    @property
    def masses(self) -> np.ndarray:
        return np.array([ATOMIC_MASSES[int(z)] for z in self.numbers], dtype=np.float64)

    def get_positions(self):
        return self.positions

    def with_velocities(self, temperature_K: float, seed: int) -> "Structure":
        rng = np.random.default_rng(seed)
        sigma = np.sqrt(KB * temperature_K / self.masses)[:, None]
        self.velocities = rng.normal(size=(self.natoms, 3)) * sigma
        return self


def _repeat(basis_frac, basis_numbers, cell, repeat):
    rx, ry, rz = repeat
    grid = np.stack(np.meshgrid(np.arange(rx), np.arange(ry), np.arange(rz), indexing="ij"), -1).reshape(-1, 3)
    frac = (grid[:, None, :] + np.asarray(basis_frac)[None, :, :]).reshape(-1, 3)
    numbers = np.tile(np.asarray(basis_numbers, dtype=np.int64), len(grid))
    return frac @ np.asarray(cell, dtype=np.float64), numbers, np.asarray(cell) * np.array(repeat)[:, None]


def nacl(repeat=(3, 3, 3), sigma: float = 0.05, seed: int = 0, a: float = 5.64) -> Structure:
    """Rock-salt NaCl, conventional 8-atom cubic cell repeated; positions jittered by N(0, sigma) per coordinate."""
    basis = [(0, 0, 0), (0, .5, .5), (.5, 0, .5), (.5, .5, 0), (.5, 0, 0), (.5, .5, .5), (0, 0, .5), (0, .5, 0)]
    numbers = [11, 11, 11, 11, 17, 17, 17, 17]
    positions, z, cell = _repeat(basis, numbers, a * np.eye(3), repeat)
    if sigma:
        positions = positions + np.random.default_rng(seed).normal(0.0, sigma, positions.shape)
    return Structure(positions, cell, z)


def fcc_alloy(repeat=(24, 24, 24), sigma: float = 0.1, seed: int = 2, a: float = 4.0,
              species=(13, 24, 26, 27, 28)) -> Structure:
    """Random alloy on the primitive FCC lattice (one site per cell, triclinic supercell)."""
    prim = 0.5 * a * np.array([[0.0, 1.0, 1.0], [1.0, 0.0, 1.0], [1.0, 1.0, 0.0]])
    positions, _, cell = _repeat([(0, 0, 0)], [0], prim, repeat)
    rng = np.random.default_rng(seed)
    z = rng.choice(np.asarray(species, dtype=np.int64), size=len(positions))
    positions = positions + rng.normal(0.0, sigma, positions.shape)
    return Structure(positions, cell, z)


def silica(n_si: int = 36864, density: float = 2.2, seed: int = 1, min_distance: float = 1.4) -> Structure:
    """Amorphous Si-O box: n_si Si + 2 n_si O placed one after the other uniformly at random in a cubic periodic cell
    at ``density`` g/cm^3; a trial position closer than ``min_distance`` (minimum image) to an accepted one is
    rejected. Trials are drawn in batches; inside a batch they are accepted in order, so the result is that of the
    sequential procedure."""
    from scipy.spatial import cKDTree

    n = 3 * n_si
    mass_g = (n_si * ATOMIC_MASSES[14] + 2 * n_si * ATOMIC_MASSES[8]) * _AMU * 1e3
    length = (mass_g / density) ** (1.0 / 3.0) * 1e8  # cm -> Å
    rng = np.random.default_rng(seed)
    accepted = np.empty((0, 3))
    while len(accepted) < n:
        trial = rng.uniform(0.0, length, size=(min(8192, 2 * (n - len(accepted)) + 64), 3))
        ok = np.ones(len(trial), dtype=bool)
        if len(accepted):
            dist, _ = cKDTree(accepted, boxsize=length).query(trial, k=1, distance_upper_bound=min_distance)
            ok &= ~np.isfinite(dist)
        pairs = cKDTree(trial, boxsize=length).query_pairs(min_distance, output_type="ndarray")
        for i, j in pairs[np.lexsort((pairs[:, 0], pairs[:, 1]))] if len(pairs) else ():
            # j > i: the later trial is rejected if the earlier one stands
            if ok[i] and ok[j]:
                ok[j] = False
        accepted = np.concatenate([accepted, trial[ok]])[:n]
    numbers = np.where(rng.permutation(n) < n_si, 14, 8).astype(np.int64)
    return Structure(accepted, length * np.eye(3), numbers)


__all__ = ["Structure", "nacl", "fcc_alloy", "silica", "FS", "KB", "ATOMIC_MASSES"]
