"""Writes ``tests/golden/langevin.npz``: trajectories of the reference's own Langevin integrator.

Run where the reference tree is present (``python tests/golden/make_langevin_golden.py <reference root>``). It imports
``fastmace.integrators.langevin.Langevin`` and ``fastmace.state.SimulationState`` unchanged and steps them on CPU
float64 tensors with a harmonic force. The reference module imports ``ase.units`` for two constants only (``fs`` and
``kB``); ASE is not installed here, so a two-attribute stand-in carrying ASE's CODATA 2014 values is registered before
the import. Everything else -- coefficients, noise layout, order of operations, centre-of-mass projections -- is the
reference's code. The test ``tests/test_oracle_langevin.py`` compares ``oracle/langevin_oracle.py`` with these files.
"""

from __future__ import annotations

import math
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

_E, _AMU, _K = 1.6021766208e-19, 1.660539040e-27, 1.38064852e-23
FS = 1.0e-5 * math.sqrt(_E / _AMU)
KB = _K / _E


def _stub_ase() -> None:
    ase = types.ModuleType("ase")
    units = types.ModuleType("ase.units")
    units.fs, units.kB = FS, KB
    ase.units = units
    sys.modules.setdefault("ase", ase)
    sys.modules.setdefault("ase.units", units)


def harmonic_force(x: torch.Tensor, x0: torch.Tensor, k: float) -> torch.Tensor:
    return -k * (x - x0)


def run_case(name: str, n: int, steps: int, *, fixcm: bool, projection: str, temperature: float, friction_per_fs: float,
             seed: int):
    from fastmace.config import IntegratorConfig
    from fastmace.integrators.langevin import Langevin
    from fastmace.state import RandomStream, SimulationState

    rng = np.random.default_rng(seed)
    x0 = rng.uniform(0.0, 8.0, (n, 3))
    masses = rng.choice([22.98976928, 35.45, 15.999, 28.085], size=n)
    v0 = rng.normal(size=(n, 3)) * np.sqrt(KB * temperature / masses)[:, None]
    f64 = dict(dtype=torch.float64)
    state = SimulationState(positions=torch.tensor(x0 + rng.normal(0, 0.05, (n, 3)), **f64),
                            velocities=torch.tensor(v0, **f64), masses=torch.tensor(masses, **f64).reshape(n, 1),
                            cell=torch.eye(3, **f64) * 8.0, species=torch.zeros(n, dtype=torch.int64),
                            forces=torch.zeros(n, 3, **f64), energy=torch.zeros(1, **f64), stress=None,
                            rng=RandomStream(np.random.default_rng(seed + 1)))
    config = IntegratorConfig(timestep_fs=1.0, friction=friction_per_fs / FS, fixcm=fixcm, fixcm_projection=projection,
                              noise_batch=4)
    integrator = Langevin(state, config, temperature_K=temperature)
    anchor = torch.tensor(x0, **f64)
    state.forces.copy_(harmonic_force(state.positions, anchor, 1.5))
    out = {f"{name}.x0": state.positions.numpy().copy(), f"{name}.v0": state.velocities.numpy().copy(),
           f"{name}.f0": state.forces.numpy().copy(), f"{name}.masses": masses, f"{name}.anchor": x0}
    xi, eta, xs, vs, mids = [], [], [], [], []
    for _ in range(steps):
        integrator.prepare_step(state)
        xi.append(integrator.xi.numpy().copy())
        eta.append(integrator.eta.numpy().copy())
        integrator.first_half(state)
        mids.append(state.velocities.numpy().copy())
        state.forces.copy_(harmonic_force(state.positions, anchor, 1.5))
        integrator.second_half(state)
        xs.append(state.positions.numpy().copy())
        vs.append(state.velocities.numpy().copy())
    out.update({f"{name}.xi": np.stack(xi), f"{name}.eta": np.stack(eta), f"{name}.x": np.stack(xs),
                f"{name}.v": np.stack(vs), f"{name}.v_mid": np.stack(mids),
                f"{name}.params": np.array([temperature, friction_per_fs, float(fixcm),
                                            float(projection == "mass_weighted"), integrator.dt])})
    return out


def main() -> None:
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_langevin_golden.py <root of the reference tree>")
    sys.path.insert(0, sys.argv[1])
    _stub_ase()
    data = {}
    data.update(run_case("ase", 17, 9, fixcm=True, projection="ase", temperature=300.0, friction_per_fs=0.01, seed=3))
    data.update(run_case("mass", 23, 9, fixcm=True, projection="mass_weighted", temperature=450.0, friction_per_fs=0.02,
                         seed=5))
    data.update(run_case("free", 11, 6, fixcm=False, projection="ase", temperature=1000.0, friction_per_fs=0.005, seed=7))
    np.savez_compressed(os.path.join(HERE, "langevin.npz"), **data)
    print("wrote", os.path.join(HERE, "langevin.npz"), sorted({k.split(".")[0] for k in data}))


if __name__ == "__main__":
    main()
