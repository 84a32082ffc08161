"""Registration of the B200 force path behind FastMACE's planner, so that ``fm.md``, ``Simulation`` and the ASE
calculator reach it without a change at their call sites.

FastMACE has no plugin registry for engines: ``Simulation`` and ``FastMACECalculator`` take their planner from the
module attribute ``fastmace.planner.minimal.default_planner`` (``simulation.py:549``, ``ase/calculator.py:93``), the
planner checks ``mode`` against ``minimal.MODES`` (``planner/minimal.py:70,761-771``) and ``MinimalPlanner.build``
dispatches on ``plan.tier`` (``:1204-1236``; the reference tier's ``build_reference``, ``:1260-1286``, is the model
for ``build_b200``). ``config.Mode`` and ``EngineConfig.backend`` are ``Literal`` types checked at construction
(``config.py:43,57-68,271``). ``register()`` does the four things a maintainer would otherwise write into those files:

* adds ``"b200"`` to ``config.Mode`` / ``config.MODES`` and to ``EngineConfig.backend``'s choices;
* adds the mode and its tier reason to ``minimal.MODES`` / ``minimal.MODE_TIERS``;
* replaces ``minimal.default_planner`` by one that returns a ``B200Planner`` on a CUDA device;
* ``B200Planner.plan_traits`` plans like the reference tier (no rewrites, no compilation: there is no third-party
  graph to rewrite) and stamps the plan ``tier="b200"``; ``B200Planner.build`` sends such plans to ``build_b200``,
  which assembles ``B200ForceField`` + the reference's ``SimulationState`` + the CUDA Langevin stages + the
  reference's own ``GraphEngine`` (its registry, capture and flag protocol drive the force field unchanged).

``fastmace`` is imported lazily: this module imports without it, and ``register()`` raises a clear error when the
package is absent.
"""

from __future__ import annotations

import dataclasses
import typing
from typing import Literal

TIER = "b200"
MODE = "b200"
_registered = {}


def _fastmace():
    try:
        import fastmace.config as config
        import fastmace.planner.minimal as minimal
    except ImportError as error:           # pragma: no cover - depends on the environment
        raise RuntimeError("fastmace is not importable: the B200 path registers itself behind FastMACE's planner "
                           f"and needs the package ({error})") from error
    return config, minimal


def extend_literals(config) -> None:
    """``"b200"`` as a legal ``Mode`` and ``EngineConfig.backend`` (``config.py:43,271``; checked by
    ``_check_choices``, ``:57-68``, which reads the annotations when an instance is built)."""
    modes = typing.get_args(config.Mode)
    if MODE not in modes:
        config.Mode = Literal[(*modes, MODE)]
        config.MODES = typing.get_args(config.Mode)
    hints = typing.get_type_hints(config.EngineConfig)
    backends = typing.get_args(hints["backend"])
    if TIER not in backends:
        config.EngineConfig.__annotations__["backend"] = Literal[(*backends, TIER)]


def spec_of(model):
    """``MaceSpec`` of a loaded model that carries it (this package's container: ``.spec`` and ``.weights``). A
    mace-torch ``ScaleShiftMACE`` is not read here: its attribute layout belongs to a package that was not available
    where this was written, and a guessed reader would be worse than a clear refusal."""
    if hasattr(model, "spec"):
        return model.spec
    raise NotImplementedError("reading the hyper-parameters of a mace-torch module is not implemented: pass a model "
                              "container with .spec and .weights")


def weights_of(model):
    """The weight dictionary of ``fastmace_b200.model.init_weights`` from a loaded model: its own ``weights`` when
    it carries them; a mace-torch module is not converted here (its parameter layout belongs to a package that is not
    available where this was written) and raises with that reason."""
    if hasattr(model, "weights"):
        return model.weights
    raise NotImplementedError("conversion of a mace-torch ScaleShiftMACE state_dict to the fmb200 weight layout is "
                              "not implemented: pass a model container with .spec and .weights")


def _numbers_cell(atoms):
    import numpy as np
    numbers = np.asarray(atoms.get_atomic_numbers() if hasattr(atoms, "get_atomic_numbers") else atoms.numbers)
    cell = np.asarray(getattr(atoms.cell, "array", atoms.cell), dtype=np.float64).reshape(3, 3)
    return numbers, cell


def state_from_atoms(atoms, device, seed: int, compute_stress: bool):
    """FastMACE's ``SimulationState`` for ``atoms``: ``SimulationState.from_atoms`` (``fastmace/state.py:340-378``)
    where ASE is installed (it reads the constraints through ``ase.constraints``); without ASE the same fields from the
    same accessors, for atoms objects without constraints."""
    import numpy as np
    import torch
    from fastmace.state import RandomStream, SimulationState
    try:
        return SimulationState.from_atoms(atoms, device, seed, compute_stress=compute_stress)
    except ModuleNotFoundError as error:
        if error.name != "ase" and not str(error.name).startswith("ase."):
            raise
    if getattr(atoms, "constraints", None):
        raise ValueError("constraints need ASE (SimulationState.from_atoms reads them through ase.constraints)")
    f64 = dict(dtype=torch.float64, device=device)
    positions = torch.tensor(np.asarray(atoms.get_positions()), **f64)
    numbers, cell = _numbers_cell(atoms)
    return SimulationState(
        positions=positions, velocities=torch.tensor(np.asarray(atoms.get_velocities()), **f64),
        masses=torch.tensor(np.asarray(atoms.get_masses())[:, None], **f64), cell=torch.tensor(cell, **f64),
        species=torch.tensor(numbers, dtype=torch.int64, device=device), forces=torch.zeros_like(positions),
        energy=torch.zeros(1, **f64), stress=torch.zeros((3, 3), **f64) if compute_stress else None,
        rng=RandomStream(np.random.default_rng(seed)), pbc=tuple(bool(p) for p in getattr(atoms, "pbc", (True,) * 3)))


def build_b200(planner, plan, force_field, atoms, *, temperature_K=None):
    """The engine of a ``tier="b200"`` plan, modelled on ``MinimalPlanner.build_reference``
    (``planner/minimal.py:1260-1286``): the CUDA force field and Langevin stages of this package on FastMACE's own
    ``SimulationState`` and ``GraphEngine``."""
    from fastmace.engine.graph import GraphEngine

    from .forcefield import B200ForceField
    from .langevin import IntegratorConfig, Langevin
    from .neighbours import NeighbourConfig

    if plan.tier != TIER:
        raise ValueError(f"build_b200 builds {TIER!r} plans, not tier {plan.tier!r}")
    if plan.integrator is not None and getattr(plan.integrator, "ensemble", "nvt") != "nvt":
        raise ValueError("the b200 tier integrates NVT Langevin only")
    model = getattr(force_field, "model", force_field)
    spec, weights = spec_of(model), weights_of(model)
    numbers, cell = _numbers_cell(atoms)
    if temperature_K is None:
        temperature_K = getattr(plan.integrator, "temperature_K", None) or 0.0
    nb = plan.neighbours
    neighbours = NeighbourConfig() if nb is None else NeighbourConfig(
        skin=float(nb.skin), edge_multiple=int(nb.edge_multiple), edge_bucket_fraction=float(nb.edge_bucket_fraction),
        capacity_headroom=float(nb.capacity_headroom))
    stress = bool(getattr(plan.workload, "stress", False)) if plan.workload is not None else False
    field = B200ForceField(spec, weights, numbers, cell, compute_stress=stress, device=plan.engine.device,
                           neighbours=neighbours)
    seed = int(getattr(plan.integrator, "seed", 0) or 0)
    state = state_from_atoms(atoms, field.device, seed, stress)
    field.rebuild(state.positions)
    it = plan.integrator
    config = IntegratorConfig() if it is None else IntegratorConfig(
        timestep_fs=float(it.timestep_fs), friction=float(it.friction), fixcm=bool(it.fixcm),
        fixcm_projection=str(getattr(it, "fixcm_projection", "mass_weighted") or "mass_weighted"),
        noise_batch=int(it.noise_batch))
    integrator = Langevin(state, config, temperature_K=float(temperature_K), cursor="host")
    # GraphEngine's capture path prepares mace-torch's modules for capture (fastmace/_patches.py, from graph.py:1331);
    # in an installation without that package the stages run uncaptured on padded edge counts
    import importlib.util
    capture = None if importlib.util.find_spec("mace") is not None else False
    engine = GraphEngine(plan.engine, field, integrator, state, neighbours=plan.neighbours, capture=capture,
                         pad_edges=True, constraints=planner.process if planner is not None else None)
    engine.plan = plan
    return engine


def make_planner_class(minimal):
    """``MinimalPlanner`` with the b200 tier: built at registration because its base class lives in ``fastmace``."""

    class B200Planner(minimal.MinimalPlanner):
        def plan_traits(self, traits, atoms, integrator, workload, hardware, *, mode=None, allow_reference=False,
                        **options):
            if mode not in (None, MODE):
                return super().plan_traits(traits, atoms, integrator, workload, hardware, mode=mode,
                                           allow_reference=allow_reference, **options)
            # the reference tier's plan has what this tier needs: no rewrites, no compilation, resolved engine,
            # neighbour and integrator options
            plan = super().plan_traits(traits, atoms, integrator, workload, hardware, mode="reference",
                                       allow_reference=True, **options)
            engine = dataclasses.replace(plan.engine, backend=TIER, compile_mode="none", pipelined="off",
                                         speculative_graph=False, fused_integrator=False, expandable_segments="off")
            reason = minimal.MODE_TIERS[MODE]
            decisions = tuple(d for d in plan.decisions if d[0] != "mode") + (("mode", MODE, str(reason)),)
            return dataclasses.replace(plan, tier=TIER, engine=engine, decisions=decisions)

        def build(self, plan, force_field, atoms, **options):
            if plan.tier == TIER:
                return build_b200(self, plan, force_field, atoms, temperature_K=options.get("temperature_K"))
            return super().build(plan, force_field, atoms, **options)

        def build_b200(self, plan, force_field, atoms, *, temperature_K=None):
            return build_b200(self, plan, force_field, atoms, temperature_K=temperature_K)

    return B200Planner


def register():
    """Install the b200 tier behind ``fastmace.planner.minimal`` (idempotent). Returns the planner class."""
    config, minimal = _fastmace()
    if "planner" in _registered:
        return _registered["planner"]
    extend_literals(config)
    if MODE not in minimal.MODES:
        minimal.MODES = (*minimal.MODES, MODE)
        minimal.MODE_TIERS[MODE] = minimal.Reason(
            "molecular dynamics on the b200 tier: neighbour list, model, analytic forces and Langevin stages in the "
            "fmb200 CUDA library for sm_100a, on FastMACE's state, engine, output and restart", code="mode-b200")
    planner_class = make_planner_class(minimal)
    original = minimal.default_planner

    def default_planner(force_field):
        import torch
        base = original(force_field)
        if not torch.cuda.is_available():
            return base                      # the CUDA path has no CPU fallback: FastMACE's own tiers serve the CPU
        return planner_class(engine=base.engine, polar=getattr(base, "polar", None))

    default_planner.__doc__ = original.__doc__
    default_planner.original = original
    minimal.default_planner = default_planner
    _registered.update(planner=planner_class, original=original)
    return planner_class


def unregister() -> None:
    """Undo ``register()``'s replacement of ``default_planner`` (tests)."""
    if "original" in _registered:
        _, minimal = _fastmace()
        minimal.default_planner = _registered["original"]
        _registered.clear()


__all__ = ["TIER", "MODE", "register", "unregister", "build_b200", "state_from_atoms", "extend_literals", "spec_of", "weights_of",
           "make_planner_class"]
