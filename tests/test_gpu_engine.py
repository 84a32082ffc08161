"""Langevin stages and the whole-step engine on the device against the NumPy restatement and the model oracle."""
import numpy as np
import pytest
import torch

from oracle import mace_oracle as mo
from oracle import neighbours_oracle as nlo
from oracle.langevin_oracle import LangevinOracle

pytestmark = pytest.mark.gpu


def _setup(spec_name="small", repeat=(2, 2, 2), temperature=300.0, seed=0, projection="mass_weighted", fixcm=True):
    from fastmace_b200.forcefield import B200ForceField
    from fastmace_b200.langevin import IntegratorConfig, Langevin
    from fastmace_b200.model import SPECS, init_weights
    from fastmace_b200.state import SimulationState
    from fastmace_b200.structures import nacl
    spec = SPECS[spec_name]
    weights = init_weights(spec, seed)
    s = nacl(repeat, 0.05, seed).with_velocities(temperature, seed + 1)
    ff = B200ForceField(spec, weights, s.numbers, s.cell, compute_stress=True)
    state = SimulationState.from_structure(s, ff.device, seed=seed + 2, compute_stress=True)
    config = IntegratorConfig(fixcm=fixcm, fixcm_projection=projection)
    integrator = Langevin(state, config, temperature_K=temperature)
    return spec, weights, s, ff, state, integrator


@pytest.mark.parametrize("projection,fixcm", [("mass_weighted", True), ("ase", True), ("ase", False)])
def test_half_steps_against_numpy(projection, fixcm):
    from fastmace_b200.structures import FS, KB
    spec, weights, s, ff, state, it = _setup(projection=projection, fixcm=fixcm)
    rng = np.random.default_rng(9)
    noise = rng.standard_normal((2, 2, s.natoms, 3))
    f = rng.normal(size=(s.natoms, 3)) * 0.1
    state.forces.copy_(torch.tensor(f))
    it.upload_noise(state, noise)
    ref = LangevinOracle(s.masses, 1.0 * FS, 0.01 / FS, 300.0, KB, fixcm, projection)
    x, v = s.positions.copy(), s.velocities.copy()
    for step in range(2):
        it.first_half(state)
        x, v = ref.first_half(x, v, f, noise[step, 0], noise[step, 1])
        assert np.abs(state.positions.cpu().numpy() - x).max() < 1e-13
        assert np.abs(state.velocities.cpu().numpy() - v).max() < 1e-12
        it.second_half(state)
        v = ref.second_half(v, f)
        assert np.abs(state.velocities.cpu().numpy() - v).max() < 1e-12
    assert int(it.cursor_dev.item()) == 2


def test_trajectory_against_oracle_model():
    """8 checked steps of the small model on 64 atoms against NumPy Langevin + the CPU model oracle."""
    from fastmace_b200.engine import B200Engine
    from fastmace_b200.structures import FS, KB
    spec, weights, s, ff, state, it = _setup()
    engine = B200Engine(ff, it, state, mode="checked")
    gen = np.random.default_rng(2)           # the state's seed
    noise = gen.standard_normal((it.noise_batch, 2, s.natoms, 3))
    ref = LangevinOracle(s.masses, 1.0 * FS, 0.01 / FS, 300.0, KB)

    def forces(x):
        snd, rcv, u = nlo.build(x, s.cell, spec.r_cut, 0.0)
        e, f, _ = mo.evaluate(spec, weights, x, s.cell, s.numbers, snd, rcv, u, compute_stress=False)
        return float(e), f.numpy()

    x, v = s.positions.copy(), s.velocities.copy()
    e, f = forces(x)
    assert abs(engine.potential_energy() - e) < 1e-6
    for step in range(8):
        engine.step()
        x, v = ref.first_half(x, v, f, noise[step, 0], noise[step, 1])
        e, f = forces(x)
        v = ref.second_half(v, f)
    engine.flush()
    assert np.abs(state.positions.cpu().numpy() - x).max() < 1e-9
    assert np.abs(state.velocities.cpu().numpy() - v).max() < 1e-8
    assert abs(engine.potential_energy() - e) < 1e-6


def test_captured_step_equals_checked_step_bitwise():
    """The one-graph step (device-gated rebuilds) against stage-by-stage stepping, 300 steps at 2,000 K so that the
    list is rebuilt several times (the reference's own engine test: captured replay == eager bitwise)."""
    from fastmace_b200.engine import B200Engine
    out = {}
    for mode in ("checked", "graph"):
        spec, weights, s, ff, state, it = _setup("medium", temperature=2000.0, seed=3)
        engine = B200Engine(ff, it, state, mode=mode)
        engine.run(300)
        out[mode] = (state.positions.clone(), state.velocities.clone(), state.energy.clone(), state.forces.clone(),
                     engine.info())
    a, b = out["checked"], out["graph"]
    assert a[4]["neighbour_rebuilds"] > 1
    for k in range(4):
        assert torch.equal(a[k], b[k]), k
    assert b[4]["captures"] == 1
