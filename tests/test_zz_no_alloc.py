"""fmb_nl_compact_static -- the compaction entry point that keeps its scratch inside the library -- against
fmb_nl_compact, through the C ABI.

It exists for hosts that cannot give the library scratch buffers (a frozen device pool under captured graphs, a
plugin arena that forbids allocation while stepping). The check: the same candidates compacted by both entry points
give identical edges, shifts, count and row pointers, on two calls in a row (the second call finds the first call's
leftovers in the shared scratch), and the caller-provided scratch is really not touched.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _outputs(nl):
    torch.cuda.synchronize()
    return [t.clone() for t in (nl.edge_index, nl.unit_shifts, nl.shifts, nl.count, nl.edge_row_ptr)]


def test_static_scratch_compaction_matches_on_two_calls_in_a_row():
    from fastmace_b200 import _lib
    from fastmace_b200.neighbours import CellListNeighbours, NeighbourConfig
    from fastmace_b200.structures import nacl

    lib = _lib.load()
    s = nacl((3, 3, 3), 0.05, 0)
    nl = CellListNeighbours(s.cell, 6.0, "cuda", torch.float32, NeighbourConfig(skin=0.3))
    x = torch.tensor(s.positions, device="cuda")
    nl.build(x)
    rng = np.random.default_rng(5)
    for call in range(2):
        moved = x + torch.tensor(rng.normal(0.0, 0.04, s.positions.shape), device="cuda")
        nl.compact(moved)                                   # existing entry point, caller-provided scratch
        expected = _outputs(nl)
        for t in (nl.edge_index, nl.unit_shifts, nl.shifts, nl.edge_row_ptr):
            t.zero_()
        nl.count.fill_(-1)
        nl.edge_row_count.fill_(-7)                         # must stay untouched by the static variant
        nl.scan_scratch.fill_(-7)
        _lib.check(lib.fmb_nl_compact_static(ctypes.byref(nl.struct), moved.data_ptr(), _lib.current_stream()),
                   "fmb_nl_compact_static")
        got = _outputs(nl)
        n = nl.num_candidates
        assert int(got[3]) == int(expected[3]) > 0
        assert torch.equal(got[0][:, :n], expected[0][:, :n])
        assert torch.equal(got[1][:n], expected[1][:n]) and torch.equal(got[2][:n], expected[2][:n])
        assert torch.equal(got[4], expected[4])
        assert bool((nl.edge_row_count == -7).all()) and bool((nl.scan_scratch == -7).all())


def test_static_scratch_refuses_lists_beyond_its_maximum():
    from fastmace_b200 import _lib
    lib = _lib.load()
    big = _lib.NlStruct()
    big.n_atoms = 262144 + 1
    x = torch.zeros(3, dtype=torch.float64, device="cuda")
    status = lib.fmb_nl_compact_static(ctypes.byref(big), x.data_ptr(), _lib.current_stream())
    assert status == 1
    assert b"FMB_STATIC_COMPACT_MAX_ATOMS" in lib.fmb_last_error()
    empty = _lib.NlStruct()
    empty.n_atoms = 0
    assert lib.fmb_nl_compact_static(ctypes.byref(empty), x.data_ptr(), _lib.current_stream()) == 1
    assert b"no atoms" in lib.fmb_last_error()
