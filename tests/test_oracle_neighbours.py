"""The neighbour-list oracle against fixtures produced by the reference's own ``build_gpu`` + ``compact``."""
import glob
import os

import numpy as np
import pytest

from conftest import GOLDEN
from oracle import neighbours_oracle as nlo

CASES = sorted(glob.glob(os.path.join(GOLDEN, "neighbours_*.npz")))


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p)[11:-4] for p in CASES])
def test_build_and_compact_match_reference(path):
    g = np.load(path)
    s, r, u = nlo.build(g["positions"], g["cell"], float(g["cutoff"]), float(g["skin"]))
    # same pairs in the same order (receiver, sender, image)
    assert np.array_equal(s, g["cand_sender"]) and np.array_equal(r, g["cand_receiver"])
    assert np.array_equal(u, g["cand_unit_shifts"])
    cs, cr, cu, csh, count = nlo.compact(g["moved"], g["cell"], s, r, u, float(g["cutoff"]))
    assert count == int(g["count"])
    assert np.array_equal(cs[:count], g["edge_sender"]) and np.array_equal(cr[:count], g["edge_receiver"])
    assert np.array_equal(cu[:count], g["edge_unit_shifts"])
    assert np.array_equal(csh[:count], g["edge_shifts"])  # bitwise: same float64 expression
    assert nlo.needs_rebuild(g["moved"], g["positions"], float(g["skin"])) == bool(g["needs_rebuild"])


def test_large_amorphous_cell_matches_reference_digests():
    """3,456-atom amorphous Si-O cell (rows of 45-80 pairs): digests of the reference's own lists
    (``tests/golden/neighbours_large.json``, written by ``make_neighbour_golden.py``)."""
    import json

    from fastmace_b200 import structures
    sys_path_golden = os.path.join(GOLDEN, "make_neighbour_golden.py")
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_neighbour_golden", sys_path_golden)
    golden = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(golden)
    with open(os.path.join(GOLDEN, "neighbours_large.json")) as handle:
        record = json.load(handle)["silica3456"]
    s = getattr(structures, record["builder"])(**record["kwargs"])
    assert golden.digest(s.positions) == record["positions"], "the seeded structure differs from the generator's"
    snd, rcv, u = nlo.build(s.positions, s.cell, record["cutoff"], record["skin"])
    assert len(snd) == record["num_candidates"]
    moved = s.positions + np.random.default_rng(1).normal(0, 0.03, s.positions.shape)
    assert golden.digest(moved) == record["moved"]
    cs, cr, cu, csh, count = nlo.compact(moved, s.cell, snd, rcv, u, record["cutoff"])
    assert count == record["count"]
    got = golden.large_digests(dict(candidate_index=np.stack([snd, rcv]), candidate_unit_shifts=u,
                                    edge_index=np.stack([cs[:count], cr[:count]]), unit_shifts=cu[:count],
                                    shifts=csh[:count]))
    for name, value in got.items():
        assert value == record[name], name


def test_edge_set_is_symmetric():
    g = np.load(os.path.join(GOLDEN, "neighbours_nacl216.npz"))
    edges = nlo.edge_set(g["edge_sender"], g["edge_receiver"], g["edge_unit_shifts"])
    assert all((r, s, -a, -b, -c) in edges for s, r, a, b, c in edges)


def test_times_3x3_is_the_row_by_matrix_product():
    """The reference checks its element-wise ``rows @ matrix`` against the library product at 1e-14
    (``tests/cpu/test_neighbors.py:427-433``); the restatement meets the same bound on the same kind of input."""
    rng = np.random.default_rng(0)
    m = rng.normal(size=(3, 3)) + 3 * np.eye(3)
    rows = rng.normal(size=(5, 3))
    np.testing.assert_allclose(nlo.times_3x3(rows, m), rows @ m, rtol=1e-14, atol=1e-14)
