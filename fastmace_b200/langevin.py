"""ASE's ``Langevin`` (NVT, fixed cell) as two device stages: the interface of FastMACE's integrator
(``fastmace/integrators/langevin.py:157-263``; ``Integrator`` ABC ``fastmace/integrators/base.py:48-178``) over
``fmb_langevin_first_half`` / ``fmb_langevin_second_half``.

Same coefficients (``langevin.py:184-198``), same noise source and order: NumPy ``default_rng(seed)`` on the host,
``standard_normal((k, 2, N, 3))`` per batch (per step ``xi`` then ``eta``), uploaded ``noise_batch`` steps at a time
and capped at 64 MiB (``langevin.py:31-45``). The kernels pick the step's row through a device-side cursor, so a
captured step needs no per-step host copy; the next batch is drawn on a background thread into pinned memory while
the current one is consumed (``langevin.py:67-89``). The first batches are short (8, 16, 32 ... steps up to
``noise_batch``) so that a run of a few steps does not wait for 256 steps of normals it never reads; NumPy fills the
array in order, so the stream of numbers is the same for any split into batches.
"""

from __future__ import annotations

import ctypes
import dataclasses
import math
import threading

import numpy as np
import torch

from . import _lib
from .state import SimulationState
from .structures import FS, KB

NOISE_BATCH_BYTES = 64 * 2 ** 20
FIRST_NOISE_ROWS = 8


@dataclasses.dataclass(frozen=True)
class IntegratorConfig:
    """The fields of the reference's ``IntegratorConfig`` the Langevin path reads (``fastmace/config.py:471-512``).
    ``friction`` is in inverse ASE time units (0.01 / fs = 0.01 / FS)."""
    timestep_fs: float = 1.0
    friction: float = 0.01 / FS
    fixcm: bool = True
    fixcm_projection: str = "mass_weighted"      # or "ase"
    noise_batch: int = 256
    ensemble: str = "nvt"


def noise_steps(limit: int, numbers: int) -> int:
    """Steps per drawn-ahead batch (``langevin.py:41-45``)."""
    return max(1, min(limit, NOISE_BATCH_BYTES // (8 * numbers)))


class Langevin:
    """NVT Langevin step in the reference's split (``prepare_step`` / ``first_half`` / forces / ``second_half``,
    ``fastmace/integrators/langevin.py``), each half one CUDA kernel on float64 state that stays on the device."""

    def __init__(self, state: SimulationState, config: IntegratorConfig | None = None, *, temperature_K: float = 0.0,
                 force_buffer: torch.Tensor | None = None, noise: str = "host", device_seed: int = 0,
                 atom_ids: torch.Tensor | None = None, n_global: int = 0, cursor: str = "device"):
        """``noise="host"``: the reference's NumPy stream, uploaded in batches. ``noise="device"``: counter-based
        normals generated on the GPU per step (``fmb_langevin_device_noise``): not the reference's numbers, but
        identical on every rank of a domain-decomposed run and free of the host draw that limits large systems."""
        self.lib = _lib.load()
        config = config or IntegratorConfig()
        if config.ensemble != "nvt":
            raise ValueError("Langevin integrates the 'nvt' ensemble")
        self.config = config
        self.dt = config.timestep_fs * FS
        self.natoms = state.natoms
        if noise not in ("host", "device"):
            raise ValueError("noise is 'host' or 'device'")
        self.noise_mode, self.device_seed = noise, int(device_seed)
        # ``cursor="device"``: the second half advances the row counter on the device, so a captured whole step needs
        # no host write (B200Engine). ``cursor="host"``: ``prepare_step`` writes the row index before every step and
        # the kernels leave it alone -- for engines that replay a stage several times while they capture it (the
        # reference's GraphEngine warms a stage up three times, fastmace/engine/graph.py:1328-1397) and would
        # otherwise run the counter ahead
        if cursor not in ("device", "host"):
            raise ValueError("cursor is 'device' or 'host'")
        self.cursor_mode = cursor
        # a rank of a spatially decomposed run integrates ``state``'s atoms out of ``n_global``: the device noise is
        # keyed by ``atom_ids`` (int32 indices in the whole system) and the centre-of-mass projection uses the sums
        # over all ranks (``noise_sums`` / ``first_half_global``)
        self.atom_ids = None if atom_ids is None else atom_ids.to(torch.int32).contiguous()
        self.n_global = int(n_global)
        if self.atom_ids is not None and noise != "device":
            raise ValueError("atom_ids key the device noise generator: pass noise='device'")
        self.noise_batch = 1 if noise == "device" else noise_steps(config.noise_batch, 6 * self.natoms)
        dev = state.positions.device
        f64 = dict(dtype=torch.float64, device=dev)
        dt, fr = self.dt, config.friction
        self.fr = fr
        self.c1 = dt / 2.0 - dt * dt * fr / 8.0
        self.c2 = dt * fr / 2 - dt * dt * fr * fr / 8.0
        masses = state.masses.reshape(-1)
        sigma_unit = torch.sqrt(2 * fr / masses)
        self.c3_unit = (math.sqrt(dt) * sigma_unit / 2.0 - dt ** 1.5 * fr * sigma_unit / 8.0).contiguous()
        self.c5_unit = (dt ** 1.5 * sigma_unit / (2 * math.sqrt(3))).contiguous()
        self.c4_unit = (fr / 2.0 * self.c5_unit).contiguous()
        self.masses = masses.contiguous()
        self.x_old = torch.zeros_like(state.positions)
        self.rnd_pos = torch.zeros_like(state.positions)
        self.rnd_vel = torch.zeros_like(state.positions)
        self.partial = torch.zeros(128 * 16, **f64)
        self.sqrt_kT = torch.zeros((), **f64)
        self.cursor_dev = torch.zeros((), dtype=torch.int32, device=dev)
        shape = (self.noise_batch, 2, self.natoms, 3)
        state.rng.batch = torch.zeros(shape, **f64)
        self.rows = self.noise_batch               # steps the batch on the device holds
        self._draw_rows = [min(FIRST_NOISE_ROWS, self.noise_batch)] * 2     # rows drawn into each staging buffer
        state.rng.cursor = self.rows               # used up: the first step refills
        self.zero_cursor = torch.zeros((), dtype=torch.int32, device=dev)
        self._staging = [] if noise == "device" else \
            [torch.empty(shape, dtype=torch.float64).pin_memory() if dev.type == "cuda"
             else torch.empty(shape, dtype=torch.float64) for _ in range(2)]
        self._staging_events = [torch.cuda.Event() if dev.type == "cuda" else None for _ in range(2)]
        self._next = 0
        self._ahead: threading.Thread | None = None
        self._queued: np.ndarray | None = None     # drawn rows that come before the generator's next draw (a resume)
        self.set_temperature(temperature_K)
        self.struct = _lib.LangevinStruct()
        s = self.struct
        s.n_atoms = self.natoms
        s.fix_com = 0 if not config.fixcm else (2 if config.fixcm_projection == "mass_weighted" else 1)
        s.dt, s.c1, s.c2 = self.dt, self.c1, self.c2
        s.positions, s.velocities = state.positions.data_ptr(), state.velocities.data_ptr()
        s.forces = (force_buffer if force_buffer is not None else state.forces).data_ptr()
        s.masses = self.masses.data_ptr()
        s.c3_unit, s.c4_unit, s.c5_unit = self.c3_unit.data_ptr(), self.c4_unit.data_ptr(), self.c5_unit.data_ptr()
        s.sqrt_kT = self.sqrt_kT.data_ptr()
        s.noise = state.rng.batch.data_ptr()
        # device noise: the batch holds the current step only (row 0) and the counter the second half advances is
        # the step index the generator is keyed with
        s.noise_cursor = (self.zero_cursor if noise == "device" else self.cursor_dev).data_ptr()
        self._idle_cursor = torch.zeros((), dtype=torch.int32, device=dev)
        s.noise_cursor_rw = (self.cursor_dev if cursor == "device" else self._idle_cursor).data_ptr()
        s.x_old, s.rnd_pos, s.rnd_vel = self.x_old.data_ptr(), self.rnd_pos.data_ptr(), self.rnd_vel.data_ptr()
        s.partial = self.partial.data_ptr()

    @property
    def variable_cell(self) -> bool:
        return False

    def set_temperature(self, temperature_K: float) -> None:
        self.temperature_K = float(temperature_K)
        self.sqrt_kT.fill_(math.sqrt(KB * temperature_K))

    # ------------------------------------------------------------------ noise
    def _draw_into(self, generator: np.random.Generator, slot: int) -> None:
        rows = self._draw_rows[slot]
        out = self._staging[slot].numpy()[:rows]
        taken = 0
        if self._queued is not None:
            taken = min(rows, len(self._queued))
            out[:taken] = self._queued[:taken]
            self._queued = self._queued[taken:] if taken < len(self._queued) else None
        if taken < rows:
            generator.standard_normal(out=out[taken:])        # straight into the pinned buffer

    def _start_draw_ahead(self, state: SimulationState) -> None:
        slot = self._next
        event = self._staging_events[slot]
        if event is not None:
            event.synchronize()       # the copy that last read this buffer has finished
        self._ahead = threading.Thread(target=self._draw_into, args=(state.rng.generator, slot), daemon=True)
        self._ahead.start()

    def refill(self, state: SimulationState) -> None:
        """Upload the next drawn-ahead batch (drawing it now if no draw is in flight), rewind the cursors and start
        drawing the batch after it on the background thread."""
        rng = state.rng
        if self._ahead is None:
            self._draw_into(rng.generator, self._next)
        else:
            self._ahead.join()
        slot = self._next
        rows = self._draw_rows[slot]
        rng.batch[:rows].copy_(self._staging[slot][:rows], non_blocking=True)
        if self._staging_events[slot] is not None:
            self._staging_events[slot].record()
        self.cursor_dev.zero_()
        rng.cursor = 0
        self.rows = rows
        self._next = 1 - slot
        self._draw_rows[self._next] = min(2 * rows, self.noise_batch)
        self._start_draw_ahead(state)

    def prepare_step(self, state: SimulationState) -> None:
        """Refill the noise batch when it is used up (host; between replays) and advance the host cursor."""
        if self.noise_mode == "device":
            return
        if state.rng.cursor >= self.rows:
            self.refill(state)
        if self.cursor_mode == "host":
            self.cursor_dev.fill_(int(state.rng.cursor))
        state.rng.cursor += 1

    def noise_record(self, state: SimulationState) -> dict:
        """The noise stream for a restart file (``fastmace/io/restart.py:1-20``: ``rng_state``, ``noise``,
        ``noise_next``): every drawn row that no step has used yet -- the rest of the batch on the device, then the
        batch drawn ahead on the host -- and the generator's state behind them, so that a resumed run reads the same
        numbers in the same order. Device noise has no stream: the step counter is its whole state."""
        if self.noise_mode == "device":
            return dict(noise=np.zeros((0, 2, self.natoms, 3)), noise_next=0, rng_state="{}",
                        noise_step=int(self.cursor_dev.item()))
        import json
        rows = [state.rng.batch[state.rng.cursor:self.rows].cpu().numpy()]
        if self._ahead is not None:
            self._ahead.join()
            rows.append(self._staging[self._next].numpy()[:self._draw_rows[self._next]].copy())
        if self._queued is not None:
            rows.append(self._queued)
        bit_state = state.rng.generator.bit_generator.state
        return dict(noise=np.concatenate(rows), noise_next=0, rng_state=json.dumps(bit_state, default=int),
                    noise_step=int(self.cursor_dev.item()))

    def load_noise_record(self, state: SimulationState, record) -> None:
        """Resume the stream of ``noise_record``: its rows are served first, then the generator continues."""
        if self.noise_mode == "device":
            self.cursor_dev.fill_(int(record["noise_step"]))
            return
        import json
        if self._ahead is not None:
            self._ahead.join()
            self._ahead = None
        bit_state = json.loads(str(record["rng_state"]))
        generator = np.random.Generator(getattr(np.random, bit_state["bit_generator"])())
        generator.bit_generator.state = bit_state
        state.rng.generator = generator
        rows = np.asarray(record["noise"], dtype=np.float64)[int(record["noise_next"]):]
        self._queued = rows if len(rows) else None
        self.rows = 0
        state.rng.cursor = 0                         # used up: the next step refills, queued rows first
        self._draw_rows = [min(FIRST_NOISE_ROWS, self.noise_batch)] * 2

    def upload_noise(self, state: SimulationState, rows: np.ndarray) -> None:
        """Replace the batch by ``rows`` (k <= noise_batch steps) and rewind the cursor: for tests and for
        runs whose noise is resident before the timed region."""
        k = rows.shape[0]
        state.rng.batch[:k].copy_(torch.from_numpy(np.ascontiguousarray(rows)))
        self.cursor_dev.zero_()
        state.rng.cursor = 0
        self.rows = k

    # ------------------------------------------------------------------ stages (graph-capturable)
    def _device_noise(self, state: SimulationState) -> None:
        if self.noise_mode != "device":
            return
        if self.atom_ids is not None:
            _lib.check(self.lib.fmb_langevin_device_noise_ids(state.rng.batch.data_ptr(), self.natoms,
                                                              self.atom_ids.data_ptr(), self.device_seed,
                                                              self.cursor_dev.data_ptr(), _lib.current_stream()),
                       "fmb_langevin_device_noise_ids")
        else:
            _lib.check(self.lib.fmb_langevin_device_noise(state.rng.batch.data_ptr(), self.natoms, self.device_seed,
                                                          self.cursor_dev.data_ptr(), _lib.current_stream()),
                       "fmb_langevin_device_noise")

    def first_half(self, state: SimulationState) -> None:
        self._device_noise(state)
        _lib.check(self.lib.fmb_langevin_first_half(ctypes.byref(self.struct), _lib.current_stream()),
                   "fmb_langevin_first_half")

    def noise_sums(self, state: SimulationState, sums: torch.Tensor) -> None:
        """First part of the first half on a rank that integrates a part of the system: the random terms of its
        atoms and, in ``sums`` (10 float64), its share of the sums the centre-of-mass projection needs."""
        self._device_noise(state)
        _lib.check(self.lib.fmb_langevin_noise_sums(ctypes.byref(self.struct), sums.data_ptr(), _lib.current_stream()),
                   "fmb_langevin_noise_sums")

    def first_half_global(self, state: SimulationState, sums: torch.Tensor) -> None:
        """Second part: projection with the sums over all ranks, half kick, drift."""
        _lib.check(self.lib.fmb_langevin_first_half_global(ctypes.byref(self.struct), sums.data_ptr(), self.n_global,
                                                           _lib.current_stream()), "fmb_langevin_first_half_global")

    def second_half(self, state: SimulationState) -> None:
        _lib.check(self.lib.fmb_langevin_second_half(ctypes.byref(self.struct), _lib.current_stream()),
                   "fmb_langevin_second_half")

    def start(self, state: SimulationState) -> None:
        """Called once after the initial force evaluation; Langevin has nothing to prepare
        (``integrators/base.py:123-128``)."""

    def register_derived(self, registry, state: SimulationState) -> None:
        """Nothing here is derived from state an event may change (``integrators/base.py``: default none)."""

    def mid_step_tensors(self, state: SimulationState):
        return (state.velocities,)

    def buffers(self, state: SimulationState):
        return dict(positions=state.positions, velocities=state.velocities, x_old=self.x_old, rnd_pos=self.rnd_pos,
                    rnd_vel=self.rnd_vel)

    def output_values(self, state: SimulationState):
        kinetic = (0.5 * (state.masses * state.velocities ** 2).sum()).reshape(1)
        return dict(positions=state.positions, momenta=state.velocities * state.masses, forces=state.forces,
                    energy=state.energy.reshape(-1)[:1], kinetic=kinetic)

    def state_dict(self) -> dict:
        """Langevin carries no state of its own between steps: the noise stream lives in ``state.rng``
        (``integrators/langevin.py:275-280``)."""
        return {}

    def load_state_dict(self, state_dict) -> None:
        if state_dict:
            raise ValueError(f"Langevin has no internal state, got {sorted(state_dict)}")


__all__ = ["Langevin", "IntegratorConfig", "noise_steps", "NOISE_BATCH_BYTES"]
