"""Domain decomposition on the CPU: the brick plan, and the decomposed force call against the undecomposed one with
the oracle standing in for the device path (2 ranks over gloo)."""
import os
import socket

import numpy as np
import pytest
import torch

from fastmace_b200.domain import DomainPlan, brick_grid
from fastmace_b200.structures import fcc_alloy, nacl


def test_brick_grid():
    cube = 10.0 * np.eye(3)
    assert sorted(brick_grid(cube, 8)) == [2, 2, 2]
    assert sorted(brick_grid(cube, 4)) == [1, 2, 2]
    assert brick_grid(np.diag([50.76, 50.76, 16.92]), 2) in ((2, 1, 1), (1, 2, 1))
    assert brick_grid(np.diag([10.0, 10.0, 40.0]), 4) == (1, 1, 4)


@pytest.mark.parametrize("n_ranks", [2, 3, 8])
def test_every_atom_is_owned_once_and_halos_hold_all_neighbours(n_ranks):
    s = nacl((3, 3, 3), 0.05, 2)
    rng = np.random.default_rng(0)
    positions = s.positions + rng.integers(-1, 2, size=s.positions.shape) @ s.cell      # some atoms outside the cell
    plan = DomainPlan(s.cell, n_ranks, inner=6.3, outer=12.6)
    owned_total = np.zeros(s.natoms, dtype=int)
    for rank in range(n_ranks):
        loc = plan.local_atoms(positions, rank)
        owned_total[loc.index[:loc.n_owned]] += 1
        x = plan.local_positions(positions, loc)
        # every image within 6 A of an owned atom is present among the first n_inner local atoms
        d = np.linalg.norm(x[:loc.n_owned, None, :] - x[None, :, :], axis=-1)
        near = d < 6.0
        assert not near[:, loc.n_inner:].any()
        assert np.all(near.sum(axis=1) - 1 == 32)          # rock salt: 32 neighbours within 6 A
        # and every image within 6 A of an inner atom is present at all
        d_in = np.linalg.norm(x[loc.n_owned:loc.n_inner, None, :] - x[None, :, :], axis=-1)
        assert np.all((d_in < 6.0).sum(axis=1) - 1 == 32)
    assert np.all(owned_total == 1)


def _problem():
    """A short-ranged, 16-channel copy of the small model (cutoff 3.2 A) on 64-atom NaCl keeps the halo clusters and
    the oracle's cost small; the decomposition logic does not depend on either."""
    import dataclasses
    from fastmace_b200.model import SMALL, init_weights
    spec = dataclasses.replace(SMALL, r_cut=3.2, avg_num_neighbors=6.0, channels=16)
    return spec, init_weights(spec, 0), nacl((2, 2, 2), 0.05, 2)


def _decomposed(rank, world, spec, weights, s, out):
    from oracle import mace_oracle as mo
    from oracle import neighbours_oracle as nlo
    plan = DomainPlan(s.cell, world, inner=spec.r_cut, outer=2 * spec.r_cut)
    loc = plan.local_atoms(s.positions, rank)
    x = plan.local_positions(s.positions, loc)
    box = (x.max(axis=0) - x.min(axis=0)) + 2 * spec.r_cut + 2.0
    x0 = x - x.min(axis=0) + spec.r_cut + 1.0
    snd, rcv, u = nlo.build(x0, np.diag(box), spec.r_cut, 0.0)
    assert not u.any()
    e, f, st = mo.evaluate(spec, weights, x0, np.diag(box), s.numbers[loc.index], snd, rcv, u, n_energy=loc.n_owned)
    forces = torch.zeros(s.natoms, 3, dtype=torch.float64)
    forces.index_add_(0, torch.as_tensor(loc.index), f)
    virial = st * float(np.prod(box))
    out["energy"], out["forces"], out["virial"] = e.reshape(1).clone(), forces, virial.clone()
    return out


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    from fastmace_b200.model import SMALL, init_weights
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    spec, weights, s = _problem()
    out = _decomposed(rank, world, spec, weights, s, {})
    for key in ("energy", "forces", "virial"):
        dist.all_reduce(out[key])                       # the one data-path collective of the scheme
    if rank == 0:
        ret.update({k: v.numpy() for k, v in out.items()})
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_undecomposed_forces():
    import torch.multiprocessing as mp
    from fastmace_b200.model import SMALL, init_weights
    from oracle import mace_oracle as mo
    from oracle import neighbours_oracle as nlo
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    manager = mp.Manager()
    ret = manager.dict()
    saved = {k: os.environ.get(k) for k in ("OMP_NUM_THREADS", "MKL_NUM_THREADS", "OPENBLAS_NUM_THREADS")}
    os.environ.update(OMP_NUM_THREADS="2", MKL_NUM_THREADS="2", OPENBLAS_NUM_THREADS="2")   # two ranks share the host
    try:
        mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    finally:
        for k, v in saved.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    spec, weights, s = _problem()
    snd, rcv, u = nlo.build(s.positions, s.cell, spec.r_cut, 0.0)
    e, f, st = mo.evaluate(spec, weights, s.positions, s.cell, s.numbers, snd, rcv, u)
    assert abs(float(ret["energy"][0]) - float(e)) < 1e-10
    assert np.abs(ret["forces"] - f.numpy()).max() < 1e-10
    assert np.abs(ret["virial"] / abs(np.linalg.det(s.cell)) - st.numpy()).max() < 1e-12
