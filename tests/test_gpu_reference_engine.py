"""The reference's own ``GraphEngine`` (``fastmace/engine/graph.py:167-345``) stepping ``B200ForceField`` and the CUDA
Langevin stages: its process-constraint checks, registry policies, flag protocol, graph captures (AC and B) and rebuild
path act on the drop-in unchanged. Skipped where the reference package is not importable."""
import importlib.util

import numpy as np
import pytest
import torch

from reference_support import AtomsView, require_fastmace

pytestmark = pytest.mark.gpu


def _parts(temperature=1500.0, seed=4, cursor="host"):
    from fastmace_b200.forcefield import B200ForceField
    from fastmace_b200.langevin import IntegratorConfig, Langevin
    from fastmace_b200.model import SMALL, init_weights
    from fastmace_b200.neighbours import NeighbourConfig
    from fastmace_b200.structures import nacl
    s = nacl((3, 3, 3), 0.05, seed).with_velocities(temperature, seed + 1)
    ff = B200ForceField(SMALL, init_weights(SMALL, 0), s.numbers, s.cell, compute_stress=True,
                        neighbours=NeighbourConfig(skin=0.2))
    return s, ff, IntegratorConfig, Langevin, temperature, cursor


def test_reference_graph_engine_steps_the_drop_in():
    require_fastmace()
    from fastmace.config import EngineConfig
    from fastmace.engine.constraints import ProcessRecord
    from fastmace.engine.graph import GraphEngine
    from fastmace_b200.engine import B200Engine
    from fastmace_b200.planner_hook import state_from_atoms
    from fastmace_b200.state import SimulationState as OwnState

    s, ff, IntegratorConfig, Langevin, temperature, cursor = _parts()
    state = state_from_atoms(AtomsView(s), ff.device, 11, True)
    ff.rebuild(state.positions)
    integrator = Langevin(state, IntegratorConfig(), temperature_K=temperature, cursor=cursor)
    config = EngineConfig(device=str(ff.device), pipelined="off", async_output="off", compile_mode="none",
                          expandable_segments="off", fused_integrator=False)
    # the reference's capture path imports mace-torch (fastmace/_patches.py, called from graph.py:1331): where that
    # package is absent the same stages run uncaptured, as they do on its reference tier
    capture = importlib.util.find_spec("mace") is not None
    engine = GraphEngine(config, ff, integrator, state, constraints=ProcessRecord(), capture=capture, pad_edges=True)
    assert engine.pad_edges                                          # padded edge counts either way
    names = set(engine.registry.entries())                           # every published buffer has a policy
    assert {"force_field.neighbours.edge_index", "force_field.neighbours.candidate_index",
            "force_field.neighbours.build_cell", "force_field.neighbours.status"} <= {str(n) for n in names}
    steps = 60
    for _ in range(steps):
        engine.step()
    engine.flush()
    torch.cuda.synchronize()
    ff.check_status()
    assert state.step == steps and engine.rebuilds >= 1
    if capture:
        assert len(engine._graphs) >= 2                              # AC and at least one padded B graph
    got_x, got_v = state.positions.cpu().numpy(), state.velocities.cpu().numpy()
    got_e = float(state.energy.item())

    # the same run through this package's own checked engine: same kernels, same noise stream, same bits
    s2, ff2, _, _, _, _ = _parts()
    own = OwnState.from_structure(s2, ff2.device, seed=11, compute_stress=True)
    own_engine = B200Engine(ff2, Langevin(own, IntegratorConfig(), temperature_K=temperature), own, mode="checked")
    own_engine.run(steps)
    assert np.array_equal(got_x, own.positions.cpu().numpy())
    assert np.array_equal(got_v, own.velocities.cpu().numpy())
    assert got_e == float(own.energy.item())
    info = engine.info()
    assert info.get("neighbour_rebuilds", ff.neighbours.rebuilds) >= 1


def test_planner_hook_builds_the_reference_engine_over_the_drop_in():
    """``build_b200`` from a ``tier="b200"`` plan: the assembly a registered planner hands to ``Simulation``."""
    require_fastmace()
    from types import SimpleNamespace
    from fastmace.config import EngineConfig, IntegratorConfig as RefIntegratorConfig, NeighbourConfig as RefNeighbours
    from fastmace.engine.constraints import ProcessRecord
    from fastmace.planner.plan import Plan
    from fastmace_b200 import planner_hook
    from fastmace_b200.model import SMALL, init_weights
    from fastmace_b200.structures import FS, nacl
    planner_hook.register()
    try:
        s = nacl((3, 3, 3), 0.05, 2).with_velocities(300.0, 3)
        plan = Plan(tier="b200",
                    engine=EngineConfig(backend="b200", device="cuda:0", pipelined="off", async_output="off",
                                        compile_mode="none", expandable_segments="off", fused_integrator=False),
                    neighbours=RefNeighbours(skin=0.3),
                    integrator=RefIntegratorConfig(timestep_fs=1.0, friction=0.01 / FS, seed=5, temperature_K=300.0))
        container = SimpleNamespace(spec=SMALL, weights=init_weights(SMALL, 0))
        engine = planner_hook.build_b200(SimpleNamespace(process=ProcessRecord()), plan, container, AtomsView(s))
        e0 = float(engine.state.energy.item())
        for _ in range(10):
            engine.step()
        engine.flush()
        torch.cuda.synchronize()
        assert engine.state.step == 10 and np.isfinite(float(engine.state.energy.item())) and np.isfinite(e0)
        assert engine.plan.tier == "b200"
    finally:
        planner_hook.unregister()
