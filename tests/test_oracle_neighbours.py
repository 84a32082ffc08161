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
