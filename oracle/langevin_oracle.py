"""TEST INFRASTRUCTURE ONLY -- NumPy float64 restatement of FastMACE's Langevin half steps.

Follows ``fastmace/integrators/langevin.py``: coefficients ``:184-198``, ``first_half`` ``:233-257`` (random terms,
centre-of-mass projection "ase" or "mass_weighted", half kick, drift, velocity from the displacement),
``second_half`` ``:259-263``. Unit constants are ASE's (CODATA 2014), restated in ``fastmace_b200.structures``
because ASE is not installed here. Pinned: ``tests/test_oracle_langevin.py`` compares it with trajectories of the
reference's own ``Langevin`` (three cases: ASE projection, mass-weighted projection, no centre-of-mass constraint),
written by ``tests/golden/make_langevin_golden.py``, which imports the reference module unchanged behind a stand-in for
the two ``ase.units`` constants it reads.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs may import this module.
"""

from __future__ import annotations

import math

import numpy as np


class LangevinOracle:
    def __init__(self, masses, dt, friction, temperature_K, kB, fixcm=True, projection="mass_weighted"):
        self.m = np.asarray(masses, dtype=np.float64).reshape(-1, 1)
        self.dt, self.fr = dt, friction
        self.c1 = dt / 2.0 - dt * dt * friction / 8.0
        self.c2 = dt * friction / 2 - dt * dt * friction * friction / 8.0
        sigma_unit = np.sqrt(2 * friction / self.m)
        self.c3 = math.sqrt(dt) * sigma_unit / 2.0 - dt ** 1.5 * friction * sigma_unit / 8.0
        self.c5 = dt ** 1.5 * sigma_unit / (2 * math.sqrt(3))
        self.c4 = friction / 2.0 * self.c5
        self.sqrt_kT = math.sqrt(kB * temperature_K)
        self.fixcm, self.projection = fixcm, projection

    def first_half(self, x, v, f, xi, eta):
        m, n = self.m, len(x)
        rnd_pos = (self.c5 * self.sqrt_kT) * eta
        rnd_vel = (self.c3 * self.sqrt_kT) * xi - (self.c4 * self.sqrt_kT) * eta
        if self.fixcm and self.projection == "mass_weighted":
            total = m.sum()
            rnd_pos = rnd_pos - (rnd_pos * m).sum(axis=0) / total
            rnd_vel = rnd_vel - (rnd_vel * m).sum(axis=0) / total
        elif self.fixcm:
            factor = math.sqrt(n / (n - 1.0))
            rnd_pos = (rnd_pos - rnd_pos.sum(axis=0) / n) * factor
            rnd_vel = (rnd_vel - (rnd_vel * m).sum(axis=0) / (m * n)) * factor
        v = v + (self.c1 * f / m - self.c2 * v + rnd_vel)
        x_old = x
        x = x + (self.dt * v + rnd_pos)
        v = (x - x_old - rnd_pos) / self.dt
        self.rnd_vel = rnd_vel
        return x, v

    def second_half(self, v, f):
        return v + (self.c1 * f / self.m - self.c2 * v + self.rnd_vel)


__all__ = ["LangevinOracle"]
