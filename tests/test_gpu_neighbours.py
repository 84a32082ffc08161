"""Device neighbour list against fixtures made by the reference's own build_gpu + compact, and against the oracle."""
import glob
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import neighbours_oracle as nlo

pytestmark = pytest.mark.gpu
CASES = sorted(glob.glob(os.path.join(GOLDEN, "neighbours_*.npz")))


def _list(cell, cutoff, skin):
    from fastmace_b200.neighbours import CellListNeighbours, NeighbourConfig
    return CellListNeighbours(cell, cutoff, "cuda", torch.float32, NeighbourConfig(skin=skin))


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p)[11:-4] for p in CASES])
def test_build_and_compact_bitwise_against_reference(path):
    g = np.load(path)
    nl = _list(g["cell"], float(g["cutoff"]), float(g["skin"]))
    x = torch.tensor(g["positions"], device="cuda")
    grew = nl.build(x)
    assert grew and nl.capacity == int(g["capacity"])          # the reference's capacity rule
    n = nl.num_candidates
    assert n == len(g["cand_sender"])
    ci = nl.candidate_index.cpu().numpy()
    assert np.array_equal(ci[0, :n], g["cand_sender"]) and np.array_equal(ci[1, :n], g["cand_receiver"])
    assert np.array_equal(nl.candidate_unit_shifts.cpu().numpy()[:n], g["cand_unit_shifts"].astype(np.float32))
    assert np.array_equal(nl.reference_positions.cpu().numpy(), g["positions"])
    # padding: atom 0 and its far image
    assert np.all(ci[:, n:] == 0)
    moved = torch.tensor(g["moved"], device="cuda")
    nl.compact(moved)
    count = int(nl.count.item())
    assert count == int(g["count"])
    ei = nl.edge_index.cpu().numpy()
    assert np.array_equal(ei[0, :count], g["edge_sender"]) and np.array_equal(ei[1, :count], g["edge_receiver"])
    assert np.array_equal(nl.unit_shifts.cpu().numpy()[:count], g["edge_unit_shifts"].astype(np.float32))
    assert np.array_equal(nl.shifts.cpu().numpy()[:count], g["edge_shifts"].astype(np.float32))
    # the whole stable partition (outside pairs after the count, in order) equals the oracle's
    s, r, u = nlo.build(g["positions"], g["cell"], float(g["cutoff"]), float(g["skin"]))
    cs, cr, cu, csh, _ = nlo.compact(g["moved"], g["cell"], s, r, u, float(g["cutoff"]))
    assert np.array_equal(ei[0, :n], cs) and np.array_equal(ei[1, :n], cr)
    # CSR row pointers over the compacted edges
    row_ptr = nl.edge_row_ptr.cpu().numpy()
    expected = np.concatenate([[0], np.cumsum(np.bincount(g["edge_receiver"], minlength=len(g["positions"])))])
    assert np.array_equal(row_ptr, expected)
    assert bool(nl.needs_rebuild(moved).item()) == bool(g["needs_rebuild"])
    assert not bool(nl.needs_rebuild(x).item())
    far = moved.clone()
    far[3, 1] += 0.2
    assert bool(nl.needs_rebuild(far).item())
    # fraction scales the threshold (skin.py:685-693): the same test in NumPy float64 decides what to expect
    for fraction in (2.0, 0.5, 1.0):
        disp2 = ((far.cpu().numpy() - g["positions"]) ** 2).sum(axis=1).max()
        threshold = (fraction * float(g["skin"]) / 2.0) ** 2
        assert abs(disp2 - threshold) > 1e-9 * threshold          # not a borderline case
        assert bool(nl.needs_rebuild(far, fraction).item()) == bool(disp2 > threshold)


def _golden_module():
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_neighbour_golden", os.path.join(GOLDEN, "make_neighbour_golden.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


@pytest.mark.parametrize("name", ["fcc10648_triclinic", "silica3456"])
def test_large_shapes_bitwise_against_reference_digests(name):
    """The shapes that are too big to commit as arrays: a 10,648-atom triclinic primitive-FCC alloy cell (several
    cell-list bins per axis, oblique stencil) and a 3,456-atom amorphous Si-O cell (rows of 45-80 pairs). The fixture
    holds SHA-256 digests of the reference's own candidate and edge arrays; equal digests mean equal pairs, shifts and
    order, bit for bit."""
    import json
    from fastmace_b200 import structures
    golden = _golden_module()
    with open(os.path.join(GOLDEN, "neighbours_large.json")) as handle:
        record = json.load(handle)[name]
    s = getattr(structures, record["builder"])(**{k: tuple(v) if isinstance(v, list) else v
                                                  for k, v in record["kwargs"].items()})
    assert s.natoms == record["natoms"]
    assert golden.digest(s.positions) == record["positions"], "the seeded structure differs from the generator's"
    nl = _list(s.cell, record["cutoff"], record["skin"])
    x = torch.tensor(s.positions, device="cuda")
    nl.build(x)
    n = nl.num_candidates
    assert n == record["num_candidates"] and nl.capacity == record["capacity"]
    moved_host = s.positions + np.random.default_rng(1).normal(0, 0.03, s.positions.shape)
    assert golden.digest(moved_host) == record["moved"]
    moved = torch.tensor(moved_host, device="cuda")
    nl.compact(moved)
    nl.check_status()
    count = int(nl.count.item())
    assert count == record["count"]
    got = golden.large_digests(dict(candidate_index=nl.candidate_index[:, :n].cpu().numpy(),
                                    candidate_unit_shifts=nl.candidate_unit_shifts[:n].cpu().numpy(),
                                    edge_index=nl.edge_index[:, :count].cpu().numpy(),
                                    unit_shifts=nl.unit_shifts[:count].cpu().numpy(),
                                    shifts=nl.shifts[:count].cpu().numpy()))
    for key, value in got.items():
        assert value == record[key], key
    rows = np.diff(nl.edge_row_ptr.cpu().numpy())
    assert int(rows.max()) == record["longest_row"] and int(rows.min()) == record["shortest_row"]
    assert bool(nl.needs_rebuild(moved).item()) == record["needs_rebuild"]


def test_second_build_keeps_addresses_and_in_graph_rebuild_is_gated():
    from fastmace_b200.structures import nacl
    s = nacl((3, 3, 3), 0.05, 0)
    nl = _list(s.cell, 6.0, 0.3)
    x = torch.tensor(s.positions, device="cuda")
    nl.build(x)
    ptr = nl.candidate_index.data_ptr()
    before = nl.candidate_index.clone()
    moved = x + 0.01 * torch.randn_like(x)
    assert nl.build(moved) is False and nl.candidate_index.data_ptr() == ptr
    # gated rebuild: the flag is clear, so nothing may change
    snapshot = nl.candidate_index.clone()
    nl.rebuild_flag.zero_()
    nl.build_in_graph(x)
    torch.cuda.synchronize()
    assert torch.equal(nl.candidate_index, snapshot)
    nl.rebuild_flag.fill_(1)
    nl.build_in_graph(x)
    torch.cuda.synchronize()
    assert torch.equal(nl.candidate_index, before)
    assert torch.equal(nl.reference_positions, x)


def test_large_cell_matches_oracle_set():
    """1,000-atom NaCl 5x5x5: the cell list has 4 bins per axis; sets equal the brute-force oracle's."""
    from fastmace_b200.structures import nacl
    s = nacl((5, 5, 5), 0.05, 4)
    nl = _list(s.cell, 6.0, 0.3)
    x = torch.tensor(s.positions, device="cuda")
    nl.build(x)
    nl.compact(x)
    snd, rcv, u = nlo.build(s.positions, s.cell, 6.0, 0.3)
    n = nl.num_candidates
    assert n == len(snd)
    ci = nl.candidate_index.cpu().numpy()
    assert np.array_equal(ci[0, :n], snd) and np.array_equal(ci[1, :n], rcv)
    assert np.array_equal(nl.candidate_unit_shifts.cpu().numpy()[:n], u.astype(np.float32))
    count = int(nl.count.item())
    cs, cr, cu, _, c2 = nlo.compact(s.positions, s.cell, snd, rcv, u, 6.0)
    assert count == c2 == 32 * s.natoms
    got = nlo.edge_set(nl.edge_index[0].cpu().numpy(), nl.edge_index[1].cpu().numpy(), nl.unit_shifts.cpu().numpy(), count)
    assert got == nlo.edge_set(cs, cr, cu, c2)
