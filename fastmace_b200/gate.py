"""The accuracy gate on the user's structure and its provenance record.

FastMACE accepts a production path by a ratio rule (``SPEC.md:2038,2051-2066``; ``fastmace/planner/selfcheck.py``,
``RATIO`` and ``FLOORS`` at ``:83-88``, ``copy_errors`` ``:201-212``, ``verdict`` ``:242-274``): on a few rattled
(0.05 Å) and, when stress is in the plan, strained (±2 %) copies of the structure, the production path's largest error
against the float64 reference must not exceed three times the float32 calculator's largest error, per quantity
(energy per atom, largest force component, largest stress component), with absolute floors of 0.01 meV/atom,
1e-5 eV/Å and 1e-7 eV/Å³ where the float32 yardstick happens to be nearly exact.

This module states that rule for the CUDA path: ``run_gate`` evaluates the copies with the force field and with two
reference callables the caller supplies (the planner's float64 reference and float32 yardstick calculators in a
FastMACE run; the CPU oracle in this repository's tests) and returns the record a run's ``metadata.json`` keeps
(``fastmace/provenance.py``): status, per-quantity errors, ratios and limits, the copies' description, the tier.
Nothing here evaluates a model itself.
"""

from __future__ import annotations

import dataclasses
import math
from typing import Any, Callable

import numpy as np

RATIO = 3.0
QUANTITIES = ("energy_meV_per_atom", "force_eV_per_A", "stress_eV_per_A3")
FLOORS = {"energy_meV_per_atom": 0.01, "force_eV_per_A": 1e-5, "stress_eV_per_A3": 1e-7}
RATTLE_A = 0.05
STRAIN = 0.02
COPIES = 2


def copy_errors(reference, candidate, natoms: int) -> dict:
    """Errors of one copy: |dE| per atom in meV, largest force component, largest stress component (None if either
    side has no stress). ``reference`` and ``candidate`` are ``(energy, forces, stress)``."""
    out = {"energy_meV_per_atom": abs(float(candidate[0]) - float(reference[0])) / natoms * 1e3,
           "force_eV_per_A": float(np.abs(np.asarray(candidate[1], float) - np.asarray(reference[1], float)).max()),
           "stress_eV_per_A3": None}
    if candidate[2] is not None and reference[2] is not None:
        out["stress_eV_per_A3"] = float(np.abs(np.asarray(candidate[2], float) - np.asarray(reference[2], float)).max())
    return out


def verdict(rows, ratio: float = RATIO, floors=None) -> dict:
    """The ratio rule over the copies: ``rows`` is a list of ``{"production": errors, "yardstick": errors}``. A
    quantity passes when the production path's largest error is at most ``max(ratio * yardstick's largest error,
    floor)``; a non-finite error fails the gate outright; an unmeasured stress passes with a note."""
    floors = dict(FLOORS if floors is None else floors)
    bad = [f"{i}/{path}/{q}" for i, row in enumerate(rows) for path in ("production", "yardstick") for q in QUANTITIES
           if row[path][q] is not None and not math.isfinite(row[path][q])]
    if bad:
        return {"passed": False, "nonfinite": bad, "quantities": {}}
    quantities = {}
    for q in QUANTITIES:
        production = [row["production"][q] for row in rows if row["production"][q] is not None]
        if not production:
            quantities[q] = {"passed": True, "note": "stress: not in plan"}
            continue
        worst = max(production)
        yardstick = max(row["yardstick"][q] for row in rows if row["yardstick"][q] is not None)
        limit = max(ratio * yardstick, floors[q])
        quantities[q] = {"production": worst, "yardstick": yardstick, "ratio": worst / yardstick if yardstick else None,
                         "floor": floors[q], "limit": limit, "passed": bool(worst <= limit)}
    return {"passed": all(v["passed"] for v in quantities.values()), "nonfinite": [], "quantities": quantities}


@dataclasses.dataclass(frozen=True)
class GateCopy:
    positions: np.ndarray
    cell: np.ndarray
    what: str


def make_copies(positions, cell, seed: int, *, stress: bool, count: int = COPIES) -> list:
    """``count`` rattled copies (N(0, 0.05 Å) per coordinate) and, with ``stress``, ``count`` copies under a random
    symmetric strain of ±2 % amplitude (positions and cell together), from a generator of their own."""
    rng = np.random.default_rng((int(seed) << 16) ^ 0x6A7E)
    positions, cell = np.asarray(positions, float), np.asarray(cell, float)
    copies = [GateCopy(positions + rng.normal(0.0, RATTLE_A, positions.shape), cell.copy(), f"rattled {RATTLE_A} A")
              for _ in range(count)]
    if stress:
        for k in range(count):
            eps = rng.uniform(-STRAIN, STRAIN, (3, 3))
            deform = np.eye(3) + 0.5 * (eps + eps.T)
            copies.append(GateCopy((positions + rng.normal(0.0, RATTLE_A, positions.shape)) @ deform, cell @ deform,
                                   f"rattled and strained {STRAIN:.0%}"))
    return copies


Evaluate = Callable[[np.ndarray, np.ndarray], tuple]


def run_gate(production: Evaluate, reference64: Evaluate, yardstick32: Evaluate, positions, cell, natoms: int, *,
             seed: int = 0, stress: bool = True, ratio: float = RATIO, floors=None, tier: str = "b200") -> dict:
    """Evaluate the copies three ways -- each callable maps ``(positions, cell)`` to ``(energy, forces, stress or
    None)`` -- and judge them. Returns the provenance record: ``status`` ("passed" / "failed"), the verdict, the
    per-copy errors and what was compared."""
    copies = make_copies(positions, cell, seed, stress=stress)
    rows = []
    for copy in copies:
        ref = reference64(copy.positions, copy.cell)
        rows.append({"what": copy.what,
                     "production": copy_errors(ref, production(copy.positions, copy.cell), natoms),
                     "yardstick": copy_errors(ref, yardstick32(copy.positions, copy.cell), natoms)})
    result = verdict(rows, ratio, floors)
    return {"schema": "fmb200.gate/1", "tier": tier, "status": "passed" if result["passed"] else "failed",
            "rule": f"production error <= max({ratio:g} x float32 yardstick error, floor) per quantity, against float64",
            "ratio": ratio, "copies": [row["what"] for row in rows], "atoms": int(natoms), "verdict": result,
            "rows": rows}


def force_field_evaluator(force_field_factory: Callable[[np.ndarray], Any], numbers, *, stress: bool = True) -> Evaluate:
    """``(positions, cell) -> (E, F, S)`` through ``B200ForceField.evaluate``; ``force_field_factory(cell)`` builds (or
    returns a cached) force field for a cell, since a strained copy has a cell of its own."""
    from types import SimpleNamespace

    def evaluate(positions, cell):
        ff = force_field_factory(np.asarray(cell, float))
        atoms = SimpleNamespace(get_positions=lambda: np.asarray(positions, float))
        return ff.evaluate(atoms, stress=stress)

    return evaluate


__all__ = ["RATIO", "FLOORS", "QUANTITIES", "copy_errors", "verdict", "make_copies", "run_gate", "GateCopy",
           "force_field_evaluator"]
