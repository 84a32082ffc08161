"""The ratio rule of the accuracy gate on known numbers (fastmace/planner/selfcheck.py:242-274)."""
import numpy as np

from fastmace_b200 import gate


def _row(p, y):
    names = gate.QUANTITIES
    return {"production": dict(zip(names, p)), "yardstick": dict(zip(names, y))}


def test_ratio_floors_and_nonfinite():
    ok = gate.verdict([_row((0.02, 2e-5, 2e-7), (0.01, 1e-5, 1e-7)), _row((0.001, 1e-6, None), (0.002, 5e-6, None))])
    assert ok["passed"]
    assert abs(ok["quantities"]["force_eV_per_A"]["limit"] - 3e-5) < 1e-18 and ok["quantities"]["force_eV_per_A"]["ratio"] == 2.0
    # above three times the yardstick and above the floor: fails on that quantity only
    bad = gate.verdict([_row((0.05, 1e-6, 1e-9), (0.01, 1e-5, 1e-7))])
    assert not bad["passed"] and not bad["quantities"]["energy_meV_per_atom"]["passed"]
    assert bad["quantities"]["force_eV_per_A"]["passed"]
    # a yardstick that happens to be exact: the floor decides
    floor = gate.verdict([_row((0.009, 9e-6, 9e-8), (0.0, 0.0, 0.0))])
    assert floor["passed"] and floor["quantities"]["energy_meV_per_atom"]["limit"] == 0.01
    assert not gate.verdict([_row((0.011, 0.0, 0.0), (0.0, 0.0, 0.0))])["passed"]
    nan = gate.verdict([_row((float("nan"), 0.0, 0.0), (0.0, 0.0, 0.0))])
    assert not nan["passed"] and nan["nonfinite"]
    none = gate.verdict([_row((0.0, 0.0, None), (0.0, 0.0, None))])
    assert none["passed"] and "note" in none["quantities"]["stress_eV_per_A3"]


def test_copies_and_record():
    x = np.random.default_rng(0).uniform(0, 10, (20, 3))
    cell = np.eye(3) * 10
    copies = gate.make_copies(x, cell, 5, stress=True)
    assert len(copies) == 4 and np.allclose(copies[0].cell, cell) and not np.allclose(copies[2].cell, cell)
    assert np.allclose(copies[2].cell, copies[2].cell.T) and abs((copies[0].positions - x).std() - 0.05) < 0.02
    again = gate.make_copies(x, cell, 5, stress=True)
    assert all(np.array_equal(a.positions, b.positions) for a, b in zip(copies, again))
    exact = lambda p, c: (float(p.sum()), p * 2.0, np.eye(3) * c[0, 0])
    off = lambda scale: (lambda p, c: (float(p.sum()) + scale * len(p) * 1e-3, p * 2.0 + scale, np.eye(3) * c[0, 0] + scale))
    record = gate.run_gate(off(2e-6), exact, off(1e-6), x, cell, len(x), seed=1)
    assert record["status"] == "passed" and record["tier"] == "b200" and len(record["rows"]) == 4
    assert abs(record["verdict"]["quantities"]["force_eV_per_A"]["ratio"] - 2.0) < 1e-6
    assert gate.run_gate(off(1e-3), exact, off(1e-6), x, cell, len(x), seed=1)["status"] == "failed"
