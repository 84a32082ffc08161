"""``B200Engine``: steps a ``SimulationState`` with a Langevin integrator and a ``B200ForceField``.

The interface is FastMACE's ``Engine`` (``fastmace/engine/base.py:91-142``: ``step / run / flush / snapshot / sync /
potential_energy / info``); the step is the reference's checked step (``fastmace/engine/graph.py:968-998``):

    prepare_step (host noise refill) -> first half kick + drift -> rebuild test -> [rebuild] -> compact ->
    forces -> state.forces/energy/stress <- output -> second half kick

Two modes:

* ``mode="checked"``: stages launched one by one with the reference's single host read per step (the rebuild flag);
  a rebuild is host-driven and may grow the buffers.
* ``mode="graph"`` (default): the WHOLE step, including a device-gated neighbour rebuild, is captured once in one
  CUDA graph and replayed with no host synchronisation. The reference instead keeps stages A/C and B in separate
  graphs with a flag read in between (``graph.py:974-991``). Capacity is fixed while the graph lives, so a rebuild
  that finds more candidate pairs than the buffers hold can only set a status bit on the device. That bit is the
  reference's overflow flag, checked before commit (``graph.py:44-56,586-595``), with the commit moved to a check
  point: every ``check_every`` steps and before every noise refill the engine synchronises, reads the word, and
  either keeps a device snapshot of the state (positions, velocities, forces, energy, stress, noise cursor) as the
  new committed point or -- on overflow -- goes back to the last one, rebuilds host-driven (the buffers grow), drops
  the graph, and steps the lost stretch again with the same noise rows before it captures anew (the reference's
  restore, grow, redo: ``graph.py:605-660,921-966``). Captured and stage-by-stage steps give the same bits, so the
  trajectory is that of a run whose buffers were large enough from the start.
"""

from __future__ import annotations

import ctypes
from typing import Any, Mapping

import torch

from . import _lib
from .forcefield import B200ForceField
from .langevin import Langevin
from .state import SimulationState


class B200Engine:
    """Runs MD steps of one force field, integrator and state: the members of the reference's ``Engine``
    (``fastmace/engine/base.py``). ``mode="graph"`` replays one captured CUDA graph per step; ``"checked"`` launches
    the stages one by one and reads the status word every step."""

    def __init__(self, force_field: B200ForceField, integrator: Langevin, state: SimulationState, *,
                 mode: str = "graph", check_every: int = 64, warmup_steps: int = 3):
        if mode not in ("graph", "checked"):
            raise ValueError("mode is 'graph' or 'checked'")
        self.force_field, self.integrator, self.state = force_field, integrator, state
        self.mode = mode
        self.check_every = int(check_every)
        self.warmup_steps = int(warmup_steps)
        self.lib = _lib.load()
        self.graph: torch.cuda.CUDAGraph | None = None
        self.captures = 0
        self.steps_since_check = 0
        self.overflows_redone = 0
        self.overflow_log = []
        self._committed = None
        self._commit_pending = False
        self.stream = torch.cuda.Stream(device=force_field.device)
        ff = force_field
        x = state.positions
        ff.rebuild(x)
        ff.compact(x)
        ff.use_edges(int(ff.edge_count))
        self._force_stage()
        torch.cuda.synchronize(ff.device)
        ff.check_status()

    # ------------------------------------------------------------------ committed point, overflow redo
    def _commit(self) -> None:
        """The state as it is now becomes the point an overflow goes back to (device copies, stream-ordered). Taken
        after ``prepare_step`` of the step about to run, so that a noise refill at this step is part of the point: the
        redo finds the rows of the stretch still in the batch and the cursors where they were."""
        st, it = self.state, self.integrator
        tensors = dict(x=st.positions, v=st.velocities, f=st.forces, e=st.energy, cursor=it.cursor_dev)
        if st.stress is not None:
            tensors["s"] = st.stress
        if self._committed is None:
            self._committed = {k: v.clone() for k, v in tensors.items()}
        else:
            for k, v in tensors.items():
                self._committed[k].copy_(v)
        self._committed_host = (st.step, st.rng.cursor - 1)      # prepare_step has counted the step about to run
        self.steps_since_check = 0
        self._commit_pending = False

    def _check(self) -> None:
        """Check point of graph mode: synchronise, read the status words, commit or redo."""
        ff = self.force_field
        torch.cuda.synchronize(ff.device)
        overflow = _lib.STATUS_CAND_OVERFLOW
        word = int(ff.neighbours.status.item())
        if word & overflow and not word & ~overflow and self._committed is not None:
            self._redo_from_committed()
            return
        try:
            ff.check_status()
        finally:
            ff.status.zero_()                # reported once: a later check reads what happened after this one
            ff.neighbours.status.zero_()
        self.steps_since_check = 0
        self._commit_pending = True          # the next step commits, behind its prepare_step

    def _redo_from_committed(self) -> None:
        st, it, ff = self.state, self.integrator, self.force_field
        lost = self.steps_since_check
        saved = self._committed
        st.positions.copy_(saved["x"]); st.velocities.copy_(saved["v"]); st.forces.copy_(saved["f"])
        st.energy.copy_(saved["e"])
        if "s" in saved:
            st.stress.copy_(saved["s"])
        it.cursor_dev.copy_(saved["cursor"])
        st.step, st.rng.cursor = self._committed_host
        ff.status.zero_()
        ff.neighbours.status.zero_()
        self.graph = None                    # the buffers are about to move
        before = ff.edge_capacity
        ff.rebuild(st.positions)             # host-driven: grows the buffers where the captured rebuild could not
        ff.compact(st.positions)
        self.overflows_redone += 1
        self.overflow_log.append(dict(step=st.step, lost_steps=lost, capacity=(before, ff.edge_capacity)))
        del self.overflow_log[:-64]
        for _ in range(lost):                # the same noise rows: no refill happened since the committed point
            self._checked_step()
        torch.cuda.synchronize(ff.device)
        ff.check_status()
        self.steps_since_check = 0
        self._commit_pending = True

    # ------------------------------------------------------------------ stages
    def _force_stage(self) -> None:
        ff, st = self.force_field, self.state
        ff(st.positions)
        _lib.check(self.lib.fmb_commit_forces(ctypes.byref(ff.work), st.forces.data_ptr(), st.energy.data_ptr(),
                                              st.stress.data_ptr() if st.stress is not None else None,
                                              _lib.current_stream()), "fmb_commit_forces")

    def _device_step(self) -> None:
        """Everything of one step that runs on the device, with the rebuild gated on the device flag."""
        ff, st, it = self.force_field, self.state, self.integrator
        it.first_half(st)
        ff.neighbours.needs_rebuild(st.positions, 1.0)
        ff.neighbours.build_in_graph(st.positions)
        ff.compact(st.positions)
        self._force_stage()
        it.second_half(st)

    def _capture(self) -> None:
        """Capture the whole step: a few eager warm-ups on the side stream, the state restored and the neighbour
        list rebuilt for it (``graph.py:1328-1397``: warm-ups leave no trace), then one ``torch.cuda.graph``."""
        st, it, ff = self.state, self.integrator, self.force_field
        saved = {k: v.clone() for k, v in dict(x=st.positions, v=st.velocities, f=st.forces, e=st.energy).items()}
        stress = st.stress.clone() if st.stress is not None else None
        cursor = it.cursor_dev.clone()
        while True:
            torch.cuda.synchronize()
            with torch.cuda.stream(self.stream):
                for _ in range(self.warmup_steps):
                    it.cursor_dev.zero_()          # warm-ups re-read row 0: the batch may hold a single step
                    self._device_step()
            self.stream.synchronize()
            st.positions.copy_(saved["x"]); st.velocities.copy_(saved["v"]); st.forces.copy_(saved["f"])
            st.energy.copy_(saved["e"])
            if stress is not None:
                st.stress.copy_(stress)
            it.cursor_dev.copy_(cursor)
            grew = ff.rebuild(st.positions)
            ff.compact(st.positions)
            torch.cuda.synchronize()
            if not grew:
                break
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=self.stream):
            self._device_step()
        self.graph = graph
        self.captures += 1

    # ------------------------------------------------------------------ Engine interface
    def _checked_step(self) -> None:
        st, it, ff = self.state, self.integrator, self.force_field
        it.prepare_step(st)
        it.first_half(st)
        flag = ff.neighbours.needs_rebuild(st.positions, 1.0)
        if int(flag.item()):                      # the one host read per step (graph.py:974-978)
            ff.rebuild(st.positions)
        ff.compact(st.positions)
        self._force_stage()
        it.second_half(st)
        st.step += 1

    def step(self) -> None:
        st, it = self.state, self.integrator
        if self.mode != "graph":
            self._checked_step()
            return
        refill_due = it.noise_mode == "host" and st.rng.cursor >= it.rows
        if self.check_every and self.steps_since_check and (refill_due or self.steps_since_check >= self.check_every):
            self._check()                    # before the rows of the stretch since the last check point are replaced
        if self.graph is None:
            self._capture()
        it.prepare_step(st)
        if self.check_every and (self._commit_pending or self._committed is None):
            self._commit()
        self.graph.replay()
        self.steps_since_check += 1
        st.step += 1

    def run(self, steps: int) -> None:
        for _ in range(steps):
            self.step()
        self.flush()

    def flush(self) -> None:
        """Synchronise; in graph mode this is a check point (an overflow since the last one is redone here), and a
        status bit that cannot be repaired (non-finite energy, a row beyond the sort buffer) becomes an error."""
        if self.mode == "graph" and self.check_every and self.steps_since_check:
            self._check()
            return
        torch.cuda.synchronize(self.force_field.device)
        self.force_field.check_status()

    # ------------------------------------------------------------------ canonical points and restart
    def canonicalise(self, *, reevaluate: bool = False) -> None:
        """Put the engine into the state a fresh build at the current positions has (``graph.py:739-782``): check
        point, neighbour list rebuilt from the current positions and compacted, status words cleared. Every restart
        write calls it, in interrupted and uninterrupted runs alike, so that a resumed run continues bit for bit."""
        self.flush()
        st, ff = self.state, self.force_field
        if ff.rebuild(st.positions):
            self.graph = None                # the buffers moved
        ff.compact(st.positions)
        ff.use_edges(int(ff.edge_count))
        ff.status.zero_()
        ff.neighbours.status.zero_()
        if reevaluate:
            self._force_stage()
            self.integrator.start(st)
        torch.cuda.synchronize(ff.device)
        self._commit_pending = True
        self.canonical_points = getattr(self, "canonical_points", 0) + 1

    def restart_record(self) -> dict:
        """The restart file's arrays under the reference's key names (format 4, ``fastmace/io/restart.py:1-20``):
        step, positions, velocities and momenta, cell, masses, species, forces, energy, stress, the noise stream
        (``rng_state``, ``noise``, ``noise_next``) and the plan's edge bucket and neighbour capacity. Canonicalises
        first, like every restart write of the reference."""
        import json

        from .neighbours import edge_bucket
        self.canonicalise()
        st, ff = self.state, self.force_field
        config = ff.neighbours.config
        record = dict(fastmace_restart=4, engine="fmb200", step=st.step,
                      positions=st.positions.cpu().numpy(), velocities=st.velocities.cpu().numpy(),
                      momenta=(st.velocities * st.masses).cpu().numpy(), cell=st.cell.cpu().numpy(),
                      masses=st.masses.cpu().numpy(), species=st.species.cpu().numpy(),
                      forces=st.forces.cpu().numpy(), energy=st.energy.cpu().numpy(),
                      plan=json.dumps(dict(tier="b200", edge_bucket=edge_bucket(int(ff.edge_count), config.edge_bucket_fraction,
                                                                             config.edge_multiple),
                                           neighbour_capacity=int(ff.edge_capacity))))
        if st.stress is not None:
            record["stress"] = st.stress.cpu().numpy()
        record.update(self.integrator.noise_record(st))
        return record

    def save_restart(self, path: str) -> None:
        import numpy as np
        np.savez(path, **self.restart_record())

    def load_restart(self, record) -> None:
        """Resume on a freshly built engine of the same system: state, noise stream and neighbour capacity of
        ``record`` (a mapping or an ``.npz`` path), then ``canonicalise`` (``restore_restart_point``,
        ``graph.py:810-829``)."""
        import json

        import numpy as np
        if isinstance(record, str):
            record = dict(np.load(record, allow_pickle=False))
        if str(record["engine"]) != "fmb200" or int(record["fastmace_restart"]) != 4:
            raise ValueError("not a format-4 restart of this engine")
        st, ff = self.state, self.force_field
        if not np.array_equal(np.asarray(record["species"]), st.species.cpu().numpy()):
            raise ValueError("the restart holds another composition")
        dev = st.positions.device
        for name in ("positions", "velocities", "forces", "energy"):
            getattr(st, name).copy_(torch.as_tensor(np.asarray(record[name]), device=dev))
        if st.stress is not None and "stress" in record:
            st.stress.copy_(torch.as_tensor(np.asarray(record["stress"]), device=dev))
        st.step = int(record["step"])
        self.integrator.load_noise_record(st, record)
        capacity = int(json.loads(str(record["plan"]))["neighbour_capacity"])
        self.graph = None
        self._committed = None
        self.steps_since_check = 0
        if capacity > ff.edge_capacity and ff.neighbours.set_capacity(capacity):
            ff._allocate_work()
        self.canonicalise()

    def snapshot(self):
        self.flush()
        return {k: v.detach().clone() for k, v in self.integrator.output_values(self.state).items()}

    def sync(self) -> Mapping[str, Any]:
        self.flush()
        return {k: v.detach().cpu().numpy() for k, v in self.integrator.output_values(self.state).items()}

    def potential_energy(self) -> float:
        self.flush()
        return float(self.state.energy.item())

    def info(self) -> Mapping[str, Any]:
        return {"mode": self.mode, "captures": self.captures, "steps": self.state.step,
                "overflows_redone": self.overflows_redone, "overflow_log": list(self.overflow_log),
                **self.force_field.info()}


__all__ = ["B200Engine"]
