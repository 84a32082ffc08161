"""Names and signatures of the classes that stand in for the reference's interfaces on this path.

The reference pins, member by member, the cut between integrator, force field and engine
(``tests/cpu/test_interfaces.py:21-62``). The rows below are the rows of that table for the three interfaces and the
state that this package mirrors; a caller written against the reference's protocol finds every member here under the
same name with the same parameter names.
"""

import inspect

import pytest

from fastmace_b200.engine import B200Engine
from fastmace_b200.forcefield import B200ForceField
from fastmace_b200.langevin import Langevin
from fastmace_b200.state import SimulationState

# (class, member) -> parameter names after ``self`` (or ``cls``), or None for a property / attribute.
SIGNATURES = {
    (B200ForceField, "device"): None,
    (B200ForceField, "dtype"): None,
    (B200ForceField, "compute_stress"): None,
    (B200ForceField, "padding_exact"): None,
    (B200ForceField, "__call__"): ("positions",),
    (B200ForceField, "evaluate"): ("atoms", "stress"),
    (B200ForceField, "set_cell"): ("cell",),
    (B200ForceField, "needs_rebuild"): ("positions", "fraction"),
    (B200ForceField, "compact"): ("positions",),
    (B200ForceField, "rebuild"): ("positions",),
    (B200ForceField, "use_edges"): ("num_edges",),
    (B200ForceField, "edge_count"): None,
    (B200ForceField, "edge_capacity"): None,
    (B200ForceField, "buffers"): (),
    (B200ForceField, "info"): (),
    (Langevin, "variable_cell"): None,
    (Langevin, "set_temperature"): ("temperature_K",),
    (Langevin, "prepare_step"): ("state",),
    (Langevin, "first_half"): ("state",),
    (Langevin, "second_half"): ("state",),
    (Langevin, "start"): ("state",),
    (Langevin, "mid_step_tensors"): ("state",),
    (Langevin, "buffers"): ("state",),
    (Langevin, "output_values"): ("state",),
    (Langevin, "state_dict"): (),
    (Langevin, "load_state_dict"): ("state_dict",),
    (SimulationState, "from_atoms"): ("atoms", "device", "seed", "compute_stress"),
    (SimulationState, "natoms"): None,
    (SimulationState, "momenta"): None,
    (B200Engine, "step"): (),
    (B200Engine, "run"): ("steps",),
    (B200Engine, "flush"): (),
    (B200Engine, "snapshot"): (),
    (B200Engine, "sync"): (),
    (B200Engine, "potential_energy"): (),
    (B200Engine, "info"): (),
}


@pytest.mark.parametrize("key", SIGNATURES, ids=lambda k: f"{k[0].__name__}.{k[1]}")
def test_member_matches_the_reference_table(key):
    cls, member = key
    assert cls.__doc__ and cls.__doc__.strip()
    raw = inspect.getattr_static(cls, member)
    expected = SIGNATURES[key]
    if expected is None:
        assert not inspect.isfunction(raw), f"{cls.__name__}.{member} is a method, the reference has a property"
        return
    function = raw.__func__ if isinstance(raw, (classmethod, staticmethod)) else raw
    names = tuple(inspect.signature(function).parameters)[1:]
    assert names == expected


def test_langevin_has_no_internal_state_to_restore():
    """``state_dict`` is empty and ``load_state_dict`` refuses anything else
    (``fastmace/integrators/langevin.py:275-280``)."""
    assert Langevin.state_dict(object()) == {}
    Langevin.load_state_dict(object(), {})
    with pytest.raises(ValueError):
        Langevin.load_state_dict(object(), {"p_eps": 1.0})


class _Atoms:
    constraints = []

    def __init__(self):
        import numpy as np
        self._x = np.arange(12, dtype=float).reshape(4, 3)

    def get_positions(self):
        return self._x

    def get_velocities(self):
        return self._x * 0.5

    def get_masses(self):
        import numpy as np
        return np.array([1.0, 2.0, 3.0, 4.0])

    def get_cell(self):
        import numpy as np
        return np.eye(3) * 9.0

    def get_atomic_numbers(self):
        import numpy as np
        return np.array([11, 17, 11, 17])


def test_from_atoms_builds_the_float64_state():
    """Velocities are stored, masses are (N, 1), forces and energy start as zeros, stress exists only on request
    (``fastmace/state.py:340-378``)."""
    import torch
    state = SimulationState.from_atoms(_Atoms(), "cpu", 3, compute_stress=True)
    assert state.natoms == 4 and state.masses.shape == (4, 1)
    assert state.positions.dtype == torch.float64 and state.species.dtype == torch.int64
    assert torch.equal(state.momenta, state.velocities * state.masses)
    assert float(state.forces.abs().sum()) == 0.0 and state.stress.shape == (3, 3)
    assert SimulationState.from_atoms(_Atoms(), "cpu", 3).stress is None
    constrained = _Atoms()
    constrained.constraints = ["FixAtoms"]
    with pytest.raises(ValueError):
        SimulationState.from_atoms(constrained, "cpu", 3)
