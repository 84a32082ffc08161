"""Domain-decomposed force call on the device: the ranks' partial results (emulated in one process on one GPU, no
collective) must add up to the undecomposed result, for 1, 2, 3 and 8 bricks."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(spec, weights, s):
    from fastmace_b200.forcefield import B200ForceField
    ff = B200ForceField(spec, weights, s.numbers, s.cell, compute_stress=True)
    return ff.evaluate(s, stress=True)


def _decomposed(spec, weights, s, n_ranks, moved=None):
    from fastmace_b200.domain import DomainForceField
    x = torch.tensor(s.positions, device="cuda")
    forces = torch.zeros(s.natoms, 3, dtype=torch.float64, device="cuda")
    scalars = torch.zeros(10, dtype=torch.float64, device="cuda")
    owned = 0
    info = []
    for rank in range(n_ranks):
        ff = DomainForceField(spec, weights, s.numbers, s.cell, rank=rank, n_ranks=n_ranks, group=None)
        ff.rebuild(x)
        y = x if moved is None else moved
        ff.compact(y)
        sc, f = ff.partial(y)
        forces += f.double()
        scalars += sc
        owned += ff.local.n_owned
        info.append((ff.local.n_owned, ff.local.n_inner, ff.local.n_local))
        torch.cuda.synchronize()
        ff.check_status()
    assert owned == s.natoms
    volume = abs(np.linalg.det(s.cell))
    return float(scalars[0]), forces.cpu().numpy(), (scalars[1:] / volume).reshape(3, 3).cpu().numpy(), info


@pytest.mark.parametrize("n_ranks", [1, 2, 3, 8])
def test_partial_results_add_up(n_ranks):
    from fastmace_b200.model import MEDIUM, init_weights
    from fastmace_b200.structures import nacl
    spec, weights = MEDIUM, init_weights(MEDIUM, 1)
    s = nacl((3, 3, 3), 0.05, 1)
    e0, f0, s0 = _reference(spec, weights, s)
    e, f, st, info = _decomposed(spec, weights, s, n_ranks)
    print(n_ranks, "ranks: (owned, inner, local) per rank", info[:2], "|dE|", abs(e - e0), "max|dF|", np.abs(f - f0).max())
    assert abs(e - e0) <= 1e-6 * max(1.0, abs(e0))
    assert np.abs(f - f0).max() <= 2e-5 * np.abs(f0).max()
    assert np.abs(st - s0).max() <= 2e-5 * np.abs(s0).max()


def test_positions_moved_within_the_skin_and_atoms_outside_the_cell():
    """Compaction at positions that moved since the partition (inside the skin), with unwrapped atoms."""
    from fastmace_b200.forcefield import B200ForceField
    from fastmace_b200.model import SMALL, init_weights
    from fastmace_b200.structures import nacl
    spec, weights = SMALL, init_weights(SMALL, 0)
    s = nacl((3, 3, 3), 0.05, 3)
    rng = np.random.default_rng(1)
    s.positions = s.positions + rng.integers(-1, 2, size=s.positions.shape) @ s.cell
    moved_np = s.positions + rng.normal(0.0, 0.03, s.positions.shape)
    ff = B200ForceField(spec, weights, s.numbers, s.cell, compute_stress=True)
    x, moved = torch.tensor(s.positions, device="cuda"), torch.tensor(moved_np, device="cuda")
    ff.rebuild(x); ff.compact(moved); ff.use_edges(int(ff.edge_count))
    out = ff(moved)
    e0, f0 = float(out.energy), out.forces.double().cpu().numpy()
    e, f, st, _ = _decomposed(spec, weights, s, 4, moved=moved)
    assert abs(e - e0) <= 1e-6 * max(1.0, abs(e0))
    assert np.abs(f - f0).max() <= 2e-5 * np.abs(f0).max()


def test_device_noise_is_reproducible_and_normal():
    import ctypes
    from fastmace_b200 import _lib
    lib = _lib.load()
    n = 200_000
    row = torch.zeros(2, n, 3, dtype=torch.float64, device="cuda")
    step = torch.tensor(7, dtype=torch.int32, device="cuda")
    _lib.check(lib.fmb_langevin_device_noise(row.data_ptr(), n, 12345, step.data_ptr(), _lib.current_stream()), "noise")
    a = row.clone()
    _lib.check(lib.fmb_langevin_device_noise(row.data_ptr(), n, 12345, step.data_ptr(), _lib.current_stream()), "noise")
    assert torch.equal(a, row)                              # same (seed, step, atom) -> same numbers
    step.fill_(8)
    _lib.check(lib.fmb_langevin_device_noise(row.data_ptr(), n, 12345, step.data_ptr(), _lib.current_stream()), "noise")
    assert not torch.equal(a, row)
    v = torch.cat([a.reshape(-1), row.reshape(-1)])
    assert abs(v.mean().item()) < 5e-3 and abs(v.std().item() - 1.0) < 5e-3
    assert abs((v ** 4).mean().item() - 3.0) < 0.05        # kurtosis of a normal
    assert abs(torch.corrcoef(torch.stack([a[0, :, 0], a[1, :, 0]]))[0, 1].item()) < 0.01


def _nccl_worker(rank, world, port, ret):
    import os
    import torch.distributed as dist
    from fastmace_b200.domain import DomainForceField
    from fastmace_b200.forcefield import B200ForceField
    from fastmace_b200.model import MEDIUM, init_weights
    from fastmace_b200.structures import nacl
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    spec, weights = MEDIUM, init_weights(MEDIUM, 1)
    s = nacl((3, 3, 3), 0.05, 1)
    ff = DomainForceField(spec, weights, s.numbers, s.cell, rank=rank, n_ranks=world, device=f"cuda:{rank}",
                          group=dist.group.WORLD)
    e, f, st = ff.evaluate(s, stress=True)
    if rank == 0:
        e0, f0, s0 = B200ForceField(spec, weights, s.numbers, s.cell, compute_stress=True,
                                    device="cuda:0").evaluate(s, stress=True)
        ret["energy"] = abs(e - e0) / max(1.0, abs(e0))
        ret["forces"] = float(np.abs(f - f0).max() / np.abs(f0).max())
        ret["stress"] = float(np.abs(st - s0).max() / np.abs(s0).max())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_over_nccl():
    """One process per GPU, forces summed by the NCCL all-reduce, against the undecomposed call."""
    import socket
    import torch.multiprocessing as mp
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_nccl_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret["energy"] <= 1e-6 and ret["forces"] <= 2e-5 and ret["stress"] <= 2e-5
