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


def test_overflow_in_graph_mode_is_restored_grown_and_redone():
    """The candidate buffers are sized with no headroom at all, so a later rebuild of the hot crystal finds more
    pairs than they hold. The captured step can only raise the device flag; the engine goes back to its last check
    point, rebuilds host-driven, redoes the lost steps and captures again. The result equals the stage-by-stage
    engine, whose rebuilds grow the buffers on the spot (reference: overflow before commit with redo,
    fastmace/engine/graph.py:605-660,921-966; tested there by shrinking capacities on the host,
    tests/cpu/test_overflow_commit.py:10-13)."""
    from fastmace_b200.engine import B200Engine
    from fastmace_b200.forcefield import B200ForceField
    from fastmace_b200.langevin import IntegratorConfig, Langevin
    from fastmace_b200.model import SMALL, init_weights
    from fastmace_b200.neighbours import NeighbourConfig
    from fastmace_b200.state import SimulationState
    from fastmace_b200.structures import nacl
    tight = NeighbourConfig(skin=0.2, capacity_headroom=1.0, edge_multiple=1)
    weights = init_weights(SMALL, 0)

    def run(mode):
        s = nacl((3, 3, 3), 0.02, 3).with_velocities(2500.0, 4)
        ff = B200ForceField(SMALL, weights, s.numbers, s.cell, compute_stress=True, neighbours=tight)
        state = SimulationState.from_structure(s, ff.device, seed=5, compute_stress=True)
        engine = B200Engine(ff, Langevin(state, IntegratorConfig(), temperature_K=2500.0), state, mode=mode,
                            check_every=16)
        engine.run(160)
        return engine, state, ff

    graph_engine, graph_state, graph_ff = run("graph")
    checked_engine, checked_state, checked_ff = run("checked")
    info = graph_engine.info()
    print(f"overflows redone {info['overflows_redone']}, log {info['overflow_log'][:3]}, captures {info['captures']}, "
          f"capacity {graph_ff.edge_capacity} vs {checked_ff.edge_capacity}, rebuilds {graph_ff.neighbours.rebuilds}")
    assert info["overflows_redone"] >= 1 and info["captures"] >= 2
    assert graph_state.step == checked_state.step == 160
    assert torch.equal(graph_state.positions, checked_state.positions)
    assert torch.equal(graph_state.velocities, checked_state.velocities)
    assert torch.equal(graph_state.energy, checked_state.energy)


def test_headline_run_survives_its_own_edge_growth():
    """5,000 steps of the headline configuration (1,944-atom NaCl, medium model, 300 K): the random-init model pulls
    the crystal together, so the edge count grows by a quarter over the run (62 k -> 78 k). The captured engine must
    come through -- inside the headroom of its buffers or, where that runs out, through check points, host-driven
    growth and redo -- with the state of the stage-by-stage engine, bit for bit."""
    from fastmace_b200.engine import B200Engine
    out = {}
    for mode in ("graph", "checked"):
        spec, weights, s, ff, state, it = _setup("medium", repeat=(9, 9, 3), temperature=300.0, seed=1)
        first_edges = None
        engine = B200Engine(ff, it, state, mode=mode)
        engine.run(1)
        first_edges = int(ff.neighbours.count.item())
        engine.run(4999)
        engine.flush()
        out[mode] = (state.positions.clone(), state.velocities.clone(), state.energy.clone(), state.forces.clone(),
                     engine.info(), first_edges, int(ff.neighbours.count.item()))
    g, c = out["graph"], out["checked"]
    print(f"edges {g[5]} -> {g[6]}, overflows redone {g[4]['overflows_redone']}, captures {g[4]['captures']}, "
          f"rebuilds {g[4]['neighbour_rebuilds']}")
    assert g[6] > 1.2 * g[5]
    assert bool(torch.isfinite(g[2]).all())
    for k in range(4):
        assert torch.equal(g[k], c[k]), k


def test_status_words_are_cleared_once_reported():
    from fastmace_b200 import _lib
    spec, weights, s, ff, state, it = _setup()
    from fastmace_b200.engine import B200Engine
    engine = B200Engine(ff, it, state, mode="graph", check_every=4)
    engine.run(2)
    ff.status.fill_(_lib.STATUS_NONFINITE)
    engine.step()
    with pytest.raises(_lib.Fmb200Error):
        engine.flush()
    assert int(ff.status.item()) == 0
    engine.run(3)                                   # the run goes on and the next check is clean


@pytest.mark.parametrize("mode", ["graph", "checked"])
def test_resumed_run_continues_bit_for_bit(mode, tmp_path):
    """Restart at a canonical point (fastmace/engine/graph.py:739-782, fastmace/io/restart.py:1-20): 30 steps, a
    restart file, 40 more steps -- against a fresh engine that loads the file and runs the 40 steps."""
    from fastmace_b200.engine import B200Engine
    spec, weights, s, ff, state, it = _setup("small", temperature=1200.0, seed=6)
    engine = B200Engine(ff, it, state, mode=mode, check_every=16)
    engine.run(30)
    path = str(tmp_path / "restart.npz")
    engine.save_restart(path)
    engine.run(40)
    spec2, weights2, s2, ff2, state2, it2 = _setup("small", temperature=1200.0, seed=6)
    resumed = B200Engine(ff2, it2, state2, mode=mode, check_every=16)
    resumed.load_restart(path)
    assert state2.step == 30
    resumed.run(40)
    assert state2.step == state.step == 70
    assert torch.equal(state.positions, state2.positions) and torch.equal(state.velocities, state2.velocities)
    assert torch.equal(state.energy, state2.energy) and torch.equal(state.forces, state2.forces)
    record = dict(np.load(path))
    assert {"positions", "momenta", "velocities", "cell", "rng_state", "noise", "noise_next", "forces", "energy",
            "step", "masses", "species", "fastmace_restart", "plan"} <= set(record)
