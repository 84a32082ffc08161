"""The Langevin oracle against trajectories of the reference's own integrator (``tests/golden/langevin.npz``, written
by ``tests/golden/make_langevin_golden.py`` from ``fastmace.integrators.langevin.Langevin`` on CPU float64)."""
import os

import numpy as np
import pytest

from oracle.langevin_oracle import LangevinOracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "langevin.npz")
_E, _AMU, _K = 1.6021766208e-19, 1.660539040e-27, 1.38064852e-23
KB = _K / _E


@pytest.mark.parametrize("name", ["ase", "mass", "free"])
def test_oracle_reproduces_the_reference_trajectory(name):
    g = np.load(GOLDEN)
    temperature, friction_per_fs, fixcm, mass_weighted, dt = g[f"{name}.params"]
    from fastmace_b200.structures import FS
    assert dt == FS                                        # one femtosecond in ASE time units, same constants
    oracle = LangevinOracle(g[f"{name}.masses"], dt, friction_per_fs / FS, temperature, KB, fixcm=bool(fixcm),
                            projection="mass_weighted" if mass_weighted else "ase")
    x, v, f = g[f"{name}.x0"].copy(), g[f"{name}.v0"].copy(), g[f"{name}.f0"].copy()
    anchor = g[f"{name}.anchor"]
    for step in range(len(g[f"{name}.x"])):
        x, v = oracle.first_half(x, v, f, g[f"{name}.xi"][step], g[f"{name}.eta"][step])
        # float64 on both sides, same expressions: agreement to rounding of differently grouped sums
        np.testing.assert_allclose(v, g[f"{name}.v_mid"][step], rtol=1e-12, atol=1e-15)
        f = -1.5 * (x - anchor)
        v = oracle.second_half(v, f)
        np.testing.assert_allclose(x, g[f"{name}.x"][step], rtol=1e-13, atol=1e-13)
        np.testing.assert_allclose(v, g[f"{name}.v"][step], rtol=1e-12, atol=1e-15)
