"""The halo-exchange decomposition on the device. One process plays every rank in turn on one GPU (the exchanges are
copies), so 2, 4 and 8 bricks are checked against the single-domain call on any box; the NCCL transport runs in child
processes when the box has at least two GPUs. Everything goes through the C ABI."""
import dataclasses
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL_E, TOL_F, TOL_S = 1e-5, 1e-4, 1e-6     # eV/atom, eV/Å, eV/Å³


def _medium(repeat=(9, 9, 3), seed=1):
    from fastmace_b200.model import MEDIUM, init_weights
    from fastmace_b200.structures import nacl
    spec = MEDIUM
    return spec, init_weights(spec, seed), nacl(repeat, 0.05, seed).with_velocities(300.0, seed + 100)


@pytest.fixture(scope="module")
def single_domain():
    from fastmace_b200.forcefield import B200ForceField
    spec, weights, s = _medium()
    ff = B200ForceField(spec, weights, s.numbers, s.cell, compute_stress=True)
    return spec, weights, s, ff.evaluate(s, stress=True)


@pytest.mark.parametrize("n_ranks", [1, 2, 4, 8])
def test_forces_of_the_bricks_equal_the_single_domain_call(single_domain, n_ranks):
    """1,944-atom NaCl, medium model: bricks of 25 x 25 x 17 Å at 8 ranks, i.e. most atoms are someone's halo atom."""
    from fastmace_b200.halo import DomainSimulation
    spec, weights, s, (e, f, st) = single_domain
    sim = DomainSimulation(spec, weights, s, n_ranks, temperature_K=300.0, seed=3)
    _, _, forces = sim.gather()
    energy, stress = sim.potential_energy(), sim.stress.cpu().numpy()
    info = sim.info()
    print(f"{n_ranks} ranks {info['bricks']}: owned {info['owned_all']}, local {info['local_all']}; "
          f"|dE|/atom {abs(energy - e) / s.natoms:.2e}  max|dF| {np.abs(forces - f).max():.2e}  "
          f"max|dS| {np.abs(stress - st).max():.2e}")
    assert sum(info["owned_all"]) == s.natoms
    assert abs(energy - e) / s.natoms <= TOL_E and np.abs(forces - f).max() <= TOL_F and np.abs(stress - st).max() <= TOL_S
    assert np.abs(forces - f).max() <= 2e-4 * np.abs(f).max() + 1e-7        # the random-init model's forces are small
    assert np.abs(stress - st).max() <= 2e-4 * np.abs(st).max() + 1e-9


def test_trajectory_does_not_depend_on_the_decomposition():
    """40 Langevin steps (a thin skin forces several re-partitions, atoms change owner) on 4 bricks against the
    single-GPU engine with the same counter-based noise: the trajectories differ by fp32 summation order only."""
    from fastmace_b200.engine import B200Engine
    from fastmace_b200.forcefield import B200ForceField
    from fastmace_b200.halo import DomainSimulation
    from fastmace_b200.langevin import IntegratorConfig, Langevin
    from fastmace_b200.neighbours import NeighbourConfig
    from fastmace_b200.state import SimulationState
    spec, weights, s = _medium(repeat=(5, 5, 3), seed=2)
    config = NeighbourConfig(skin=0.06)
    sim = DomainSimulation(spec, weights, s, 4, temperature_K=600.0, seed=7, neighbours=config)
    ff = B200ForceField(spec, weights, s.numbers, s.cell, compute_stress=True, neighbours=config)
    state = SimulationState.from_structure(s, ff.device, seed=0, compute_stress=True)
    engine = B200Engine(ff, Langevin(state, IntegratorConfig(), temperature_K=600.0, noise="device", device_seed=7),
                        state, mode="checked")
    owners_before = [r.part.owned.clone() for r in sim.ranks]
    for _ in range(40):
        sim.step()
        engine.step()
    x, v, f = sim.gather()
    engine.flush()
    dx = np.abs(x - state.positions.cpu().numpy()).max()
    dv = np.abs(v - state.velocities.cpu().numpy()).max()
    de = abs(sim.potential_energy() - engine.potential_energy()) / s.natoms
    moved = sum(int((a.shape != r.part.owned.shape) or not torch.equal(a, r.part.owned))
                for a, r in zip(owners_before, sim.ranks))
    print(f"re-partitions {sim.repartitions}, ranks whose atoms changed {moved}, rebuilds {ff.neighbours.rebuilds}; "
          f"max|dx| {dx:.2e} Å  max|dv| {dv:.2e}  |dE|/atom {de:.2e}")
    assert sim.repartitions >= 3
    assert dx <= 1e-6 and dv <= 1e-5 and de <= TOL_E


def test_empty_brick_in_a_vacuum_slab():
    """A slab with two thirds of the cell empty, cut into 4 bricks along the long axis: some bricks own nothing and
    still take part in the exchanges."""
    from fastmace_b200.forcefield import B200ForceField
    from fastmace_b200.halo import DomainSimulation
    from fastmace_b200.model import SMALL, init_weights
    from fastmace_b200.structures import nacl
    s = nacl((3, 3, 4), 0.05, 1).with_velocities(300.0, 4)
    cell = s.cell.copy()
    cell[2, 2] *= 4.0
    s = dataclasses.replace(s, cell=cell)
    weights = init_weights(SMALL, 0)
    e, f, st = B200ForceField(SMALL, weights, s.numbers, s.cell, compute_stress=True).evaluate(s, stress=True)
    sim = DomainSimulation(SMALL, weights, s, 4, temperature_K=300.0, seed=1)
    info = sim.info()
    assert 0 in info["owned_all"], info
    _, _, forces = sim.gather()
    assert abs(sim.potential_energy() - e) / s.natoms <= TOL_E
    assert np.abs(forces - f).max() <= TOL_F and np.abs(sim.stress.cpu().numpy() - st).max() <= TOL_S
    sim.run(5)
    assert np.isfinite(sim.potential_energy())


_NCCL_SCRIPT = r"""
import json, os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, {root!r})
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
from fastmace_b200.halo import DistributedTransport, DomainSimulation
from fastmace_b200.model import MEDIUM, init_weights
from fastmace_b200.structures import nacl
s = nacl((6, 6, 3), 0.05, 1).with_velocities(300.0, 101)
sim = DomainSimulation(MEDIUM, init_weights(MEDIUM, 1), s, world, temperature_K=300.0, seed=3, device=f"cuda:{{rank}}",
                       ranks=[rank], transport=DistributedTransport())
e0 = sim.potential_energy()
_, _, f0 = sim.gather()
sim.run(10)
x, v, f = sim.gather()
if rank == 0:
    print("RESULT " + json.dumps(dict(e0=e0, f0=f0.tolist(), x=x.tolist(), e=sim.potential_energy())))
dist.barrier()
dist.destroy_process_group()
"""


@pytest.mark.parametrize("world", [2, 4])
def test_ranks_over_nccl(world, tmp_path):
    """One process per GPU over NCCL (NVLS off, plain all_to_all): initial forces against the single-domain call and
    10 steps against the in-process decomposition."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import json
    from fastmace_b200.forcefield import B200ForceField
    from fastmace_b200.halo import DomainSimulation
    from fastmace_b200.model import MEDIUM, init_weights
    from fastmace_b200.structures import nacl
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = {**os.environ, "NCCL_NVLS_ENABLE": "0"}
    script = tmp_path / "halo_ranks.py"
    script.write_text(_NCCL_SCRIPT.format(root=root))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                          "--master-addr", "127.0.0.1", "--master-port", str(29517 + world), str(script)],
                         env=env, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-3000:]
    got = json.loads([l for l in out.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    s = nacl((6, 6, 3), 0.05, 1).with_velocities(300.0, 101)
    weights = init_weights(MEDIUM, 1)
    e, f, _ = B200ForceField(MEDIUM, weights, s.numbers, s.cell, compute_stress=True).evaluate(s, stress=True)
    assert abs(got["e0"] - e) / s.natoms <= TOL_E and np.abs(np.asarray(got["f0"]) - f).max() <= TOL_F
    sim = DomainSimulation(MEDIUM, weights, s, world, temperature_K=300.0, seed=3)
    sim.run(10)
    x, _, _ = sim.gather()
    assert np.abs(np.asarray(got["x"]) - x).max() <= 1e-7
    assert abs(got["e"] - sim.potential_energy()) / s.natoms <= TOL_E
