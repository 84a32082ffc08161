"""``B200Engine``: steps a ``SimulationState`` with a Langevin integrator and a ``B200ForceField``.

The interface is FastMACE's ``Engine`` (``fastmace/engine/base.py:91-142``: ``step / run / flush / snapshot / sync /
potential_energy / info``); the step is the reference's checked step (``fastmace/engine/graph.py:968-998``):

    prepare_step (host noise refill) -> first half kick + drift -> rebuild test -> [rebuild] -> compact ->
    forces -> state.forces/energy/stress <- output -> second half kick

Two modes:

* ``mode="checked"``: stages launched one by one with the reference's single host read per step (the rebuild flag);
  a rebuild is host-driven and may grow the buffers.
* ``mode="graph"`` (default): the WHOLE step, including a device-gated neighbour rebuild, is captured once in one
  CUDA graph and replayed with no host synchronisation. Capacity is fixed while the graph lives; an overflow sets the
  status word, which ``flush`` (and every ``check_every`` steps) turns into an error. The reference instead keeps
  stages A/C and B in separate graphs with a flag read in between (``graph.py:974-991``).
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
                 mode: str = "graph", check_every: int = 256, warmup_steps: int = 3):
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
        self.stream = torch.cuda.Stream(device=force_field.device)
        ff = force_field
        x = state.positions
        ff.rebuild(x)
        ff.compact(x)
        ff.use_edges(int(ff.edge_count))
        self._force_stage()
        torch.cuda.synchronize(ff.device)
        ff.check_status()

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
    def step(self) -> None:
        st, it, ff = self.state, self.integrator, self.force_field
        if self.mode == "graph":
            if self.graph is None:
                self._capture()
            it.prepare_step(st)
            self.graph.replay()
            self.steps_since_check += 1
            if self.check_every and self.steps_since_check >= self.check_every:
                self.flush()
        else:
            it.prepare_step(st)
            it.first_half(st)
            flag = ff.neighbours.needs_rebuild(st.positions, 1.0)
            if int(flag.item()):                      # the one host read per step (graph.py:974-978)
                ff.rebuild(st.positions)
            ff.compact(st.positions)
            self._force_stage()
            it.second_half(st)
        st.step += 1

    def run(self, steps: int) -> None:
        for _ in range(steps):
            self.step()
        self.flush()

    def flush(self) -> None:
        """Synchronise and turn a device status bit (capacity overflow, non-finite energy) into an error."""
        torch.cuda.synchronize(self.force_field.device)
        self.steps_since_check = 0
        self.force_field.check_status()

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
                **self.force_field.info()}


__all__ = ["B200Engine"]
