"""Halo partitions of the spatially decomposed run on the CPU: ownership, halo completeness against the neighbour
oracle, matching send / receive lists, the exchange pattern over a 2-rank gloo group."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from fastmace_b200.domain import DomainPlan
from fastmace_b200.halo import LocalTransport, _Geometry, halo_box, partition
from fastmace_b200.structures import fcc_alloy, nacl
from oracle import neighbours_oracle as nlo

CUTOFF, SKIN = 6.0, 0.3


def _cases():
    s = nacl((3, 3, 3), 0.05, 0)
    yield "nacl216", s.positions, s.cell
    s = fcc_alloy((6, 6, 6), 0.1, 2)
    yield "fcc216_triclinic", s.positions, s.cell
    s = nacl((2, 2, 2), 0.05, 5)
    rng = np.random.default_rng(11)
    moved = s.positions + rng.integers(-2, 3, size=s.positions.shape) @ s.cell * 1.0
    yield "nacl64_outside_cell", moved, s.cell
    s = nacl((2, 2, 4), 0.05, 1)
    slab_cell = s.cell.copy()
    slab_cell[2, 2] *= 3.0                          # two thirds of the cell are vacuum: some bricks own nothing
    yield "nacl128_vacuum_slab", s.positions, slab_cell


CASES = list(_cases())


def _parts(positions, cell, n_ranks):
    plan = DomainPlan(cell, n_ranks, inner=CUTOFF + SKIN, outer=CUTOFF + SKIN)
    x = torch.tensor(positions, dtype=torch.float64)
    geometry = _Geometry(plan, x)
    return plan, x, [partition(plan, x, r, geometry) for r in range(n_ranks)]


@pytest.mark.parametrize("name,positions,cell", CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize("n_ranks", [1, 2, 4, 8])
def test_partition_owns_every_atom_once_and_lists_match(name, positions, cell, n_ranks):
    plan, x, parts = _parts(positions, cell, n_ranks)
    owned = torch.cat([p.owned for p in parts])
    assert sorted(owned.tolist()) == list(range(len(positions)))
    for p in parts:
        assert torch.equal(p.owned, torch.sort(p.owned).values)
        assert len(p.send_index) == sum(p.send_counts) and p.n_halo == sum(p.recv_counts)
        assert int(p.add_ptr[-1]) == len(p.send_index)
    for r, mine in enumerate(parts):
        at = 0
        for q, peer in enumerate(parts):
            # what q sends to r is r's block of halo atoms owned by q, atom by atom
            start = sum(peer.send_counts[:r])
            sent = peer.owned[peer.send_index[start:start + peer.send_counts[r]].long()]
            block = mine.halo[at:at + mine.recv_counts[q]]
            assert torch.equal(sent, block), (r, q)
            at += mine.recv_counts[q]


@pytest.mark.parametrize("name,positions,cell", CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize("n_ranks", [2, 8])
def test_local_lists_union_to_the_global_list(name, positions, cell, n_ranks):
    """Every edge into an owned atom is found among the rank's local atoms (non-periodic frame), with the same
    sender and image: the ranks' lists of owned receivers partition the global list."""
    plan, x, parts = _parts(positions, cell, n_ranks)
    snd, rcv, unit = nlo.build_screened(positions, cell, CUTOFF, SKIN)
    want = {}
    for s, r, u in zip(snd, rcv, unit):
        want.setdefault(int(r), []).append(positions[r] - positions[s] + u @ cell)
    total = 0
    for p in parts:
        if p.n_owned == 0:
            continue
        origin, lengths = halo_box(plan, p.rank, 2.0 + SKIN)
        local_ids = torch.cat([p.owned, p.halo]).numpy()
        local = positions[local_ids] + p.shift.numpy() - origin
        assert local.min() >= 0.0 and (local.max(axis=0) <= lengths).all()
        box = np.diag(lengths + 2 * (CUTOFF + SKIN))
        ls, lr, lu = nlo.build_screened(local + (CUTOFF + SKIN), box, CUTOFF, SKIN)
        assert not lu.any()                                   # the frame is not periodic in effect
        keep = lr < p.n_owned
        got = {}
        for s, r in zip(ls[keep], lr[keep]):
            got.setdefault(int(local_ids[r]), []).append(local[r] - local[s])
        for atom in p.owned.tolist():
            a = np.array(sorted(map(tuple, np.round(got.get(atom, []), 9))))
            b = np.array(sorted(map(tuple, np.round(want.get(atom, []), 9))))
            assert a.shape == b.shape and (a.size == 0 or np.abs(a - b).max() < 1e-8), (p.rank, atom)
            total += len(a)
    assert total == len(snd)


def test_rows_travel_out_and_back_in_process():
    """The exchange pattern with every rank in one process: rows keyed by the global atom index go out to the halo
    rows, counts come back and add up to the number of ranks and images that hold each atom."""
    name, positions, cell = CASES[0]
    plan, x, parts = _parts(positions, cell, 4)
    t = LocalTransport()
    send = [p.owned[p.send_index.long()].double().reshape(-1, 1) for p in parts]
    recv = [torch.zeros(p.n_halo, 1, dtype=torch.float64) for p in parts]
    send_counts, recv_counts = [p.send_counts for p in parts], [p.recv_counts for p in parts]
    t.forward(send, send_counts, recv, recv_counts)
    for p, rows in zip(parts, recv):
        assert torch.equal(rows.reshape(-1).long(), p.halo)
    back = [torch.zeros(len(p.send_index), 1, dtype=torch.float64) for p in parts]
    t.reverse([torch.ones(p.n_halo, 1, dtype=torch.float64) for p in parts], recv_counts, back, send_counts)
    held = torch.zeros(len(positions))
    for p in parts:
        held += torch.bincount(p.halo, minlength=len(positions))
    for p, rows in zip(parts, back):
        got = torch.zeros(p.n_owned, dtype=torch.float64)
        for i in range(p.n_owned):
            got[i] = rows[p.add_source[p.add_ptr[i]:p.add_ptr[i + 1]].long()].sum()
        assert torch.equal(got, held[p.owned].double())


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_worker(rank, world, port, positions, cell, out):
    import torch.distributed as dist
    from fastmace_b200.halo import DistributedTransport
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        plan = DomainPlan(cell, world, inner=CUTOFF + SKIN, outer=CUTOFF + SKIN)
        x = torch.tensor(positions, dtype=torch.float64)
        p = partition(plan, x, rank)
        t = DistributedTransport()
        t.check_counts(p.send_counts, p.recv_counts, "cpu")
        send = x[p.owned][p.send_index.long()].contiguous()
        recv = torch.zeros(p.n_halo, 3, dtype=torch.float64)
        t.forward([send], [p.send_counts], [recv], [p.recv_counts])
        assert torch.equal(recv, x[p.halo])                                  # the owners' float64 positions, bit for bit
        back = torch.zeros(len(p.send_index), 3, dtype=torch.float64)
        t.reverse([recv], [p.recv_counts], [back], [p.send_counts])
        assert torch.equal(back, send)
        total = torch.tensor([float(p.n_owned)])
        t.sum_([total])
        out[rank] = int(total.item())
    finally:
        dist.destroy_process_group()


def test_exchange_over_a_two_rank_gloo_group():
    name, positions, cell = CASES[1]
    with mp.Manager() as manager:
        out = manager.dict()
        mp.spawn(_gloo_worker, args=(2, _free_port(), positions, cell, out), nprocs=2, join=True)
        assert dict(out) == {0: len(positions), 1: len(positions)}
