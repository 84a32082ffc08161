"""Spatially decomposed MD with per-layer halo exchange: one rank per GPU, every rank owns the atoms of one brick of
the periodic cell, integrates them, and evaluates both interactions for them alone.

The reference runs one structure on one GPU (a stated non-goal, ``SPEC.md:70-74``); the structural precedent is its
tiled backend, where a tile is "receivers + their edges + halo senders" and only the first interaction's output and
its adjoint cross tile borders (``fastmace/model/tiled.py:1-26,98-101``, ``docs/design/tiled-backend.md:74-90``).
Here the tiles are ranks:

* a rank's local atoms are ``owned | halo``: the halo holds every atom (periodic images included) within
  ``cutoff + skin`` of the brick, ordered by owner rank, so that whatever one peer sends is one contiguous block of rows;
* per step four exchanges run between an atom's owner and the ranks that hold it as a halo atom: float64 positions
  and ``x = linear_up(h1)`` (2 KiB per atom for the medium model) outwards; the gradient of ``x`` and the partial forces
  back (the reverse accumulation). Receives land in place, sends out of the halo rows need no packing; the other two
  ends are one gather and one ordered add kernel (``csrc/halo.cu``). One small all-reduce carries energy and virial,
  one the ten sums of the centre-of-mass projection, one the rebuild flag;
* the MD state is partitioned: a rank holds positions, velocities and forces of its owned atoms only. When the
  displacement test fires (on any rank) the ranks put their atoms into a global array (one all-reduce of zero-padded
  rows), every rank selects the atoms of its brick again (atoms migrate between ranks here) and rebuilds its
  neighbour list; the noise generator is keyed by the atom's global index, so a trajectory does not depend on the
  decomposition beyond floating-point summation order.

``HaloPartition`` and ``partition`` are plain tensor code (CPU or CUDA) and are tested on the CPU; ``Transport`` has an
in-process implementation (all ranks in one process, one after the other on one GPU: tests and single-GPU runs) and a
``torch.distributed`` one (NCCL ``all_to_all_single`` = grouped send / receive, or gloo on the CPU).
"""

from __future__ import annotations

import ctypes
import dataclasses
import math

import numpy as np
import torch

from .domain import DomainPlan


def _times_3x3(rows: torch.Tensor, matrix: torch.Tensor) -> torch.Tensor:
    """rows @ matrix as element-wise products summed left to right: the same bits for any number of rows."""
    return rows[:, 0:1] * matrix[0] + rows[:, 1:2] * matrix[1] + rows[:, 2:3] * matrix[2]


@dataclasses.dataclass
class HaloPartition:
    """One rank's share of a partition of the global atoms."""
    rank: int
    owned: torch.Tensor          # [n_owned] int64 global indices of the owned atoms, ascending
    halo: torch.Tensor           # [n_halo] int64 global indices of the halo atoms, ordered by (owner, image, index)
    shift: torch.Tensor          # [n_owned + n_halo, 3] float64 whole cell vectors: an owned atom's position may lie
                                 # outside the cell, its shift brings it into the brick; a halo atom's takes it to its image
    recv_counts: list            # [n_ranks] halo atoms owned by each rank (blocks of ``halo`` in rank order)
    send_index: torch.Tensor     # [n_send] int32 positions in ``owned`` of the atoms peers hold as halo atoms,
    send_counts: list            # ordered by (peer, image, index); [n_ranks] rows per peer
    add_ptr: torch.Tensor        # [n_owned + 1] int32 CSR over the owned atoms into ``add_source``
    add_source: torch.Tensor     # [n_send] int32 rows of a received buffer (ordered like ``send_index``) per owned atom

    @property
    def n_owned(self) -> int:
        return int(self.owned.shape[0])

    @property
    def n_halo(self) -> int:
        return int(self.halo.shape[0])

    @property
    def n_local(self) -> int:
        return self.n_owned + self.n_halo


class _Geometry:
    """Wrapped fractional coordinates and owners of all atoms, shared by the partitions of every rank."""

    def __init__(self, plan: DomainPlan, positions: torch.Tensor):
        dev = positions.device
        self.plan = plan
        inverse = torch.as_tensor(plan.inverse, dtype=torch.float64, device=dev)
        frac = _times_3x3(positions, inverse)
        self.base = torch.floor(frac)
        self.f = frac - self.base
        grid = torch.tensor(plan.grid, device=dev)
        b = torch.minimum((self.f * grid).to(torch.int64), grid - 1)
        self.owner = (b[:, 0] * plan.grid[1] + b[:, 1]) * plan.grid[2] + b[:, 2]
        self.cell = torch.as_tensor(plan.cell, dtype=torch.float64, device=dev)

    def images_of(self, rank: int):
        """(lo, hi, margin, images [k, 3]) of a rank's halo box: the brick widened by ``inner`` in every direction,
        in fractional coordinates, and the periodic images that can reach it, in lexicographic order."""
        plan = self.plan
        lo, hi = plan.brick(rank)
        margin = plan.inner / plan.widths
        reach = [int(math.floor(m + (h - l))) + 1 for m, l, h in zip(margin, lo, hi)]
        axes = [torch.arange(-r, r + 1, dtype=torch.float64) for r in reach]
        images = torch.stack(torch.meshgrid(*axes, indexing="ij"), dim=-1).reshape(-1, 3)
        return lo, hi, margin, images

    def in_halo(self, rank: int, atoms: torch.Tensor, chunk: int = 1 << 18):
        """(image row, atom) pairs, in (image, atom) order, of the atoms of ``atoms`` (ascending global indices) whose
        periodic image lies in ``rank``'s halo box, the rank's own unshifted atoms excepted. Returns
        (image index [m], global atom index [m])."""
        lo, hi, margin, images = self.images_of(rank)
        dev = self.f.device
        images = images.to(dev)
        low = torch.as_tensor(lo - margin, dtype=torch.float64, device=dev)
        high = torch.as_tensor(hi + margin, dtype=torch.float64, device=dev)
        zero = int(torch.nonzero((images == 0).all(dim=1))[0])
        found_image, found_atom = [], []
        for start in range(0, len(atoms), chunk):
            part = atoms[start:start + chunk]
            f3 = self.f[part][None, :, :] + images[:, None, :]                   # [images, atoms, 3]
            inside = ((f3 >= low) & (f3 < high)).all(dim=-1)
            inside[zero] &= self.owner[part] != rank
            pair = torch.nonzero(inside)                                          # sorted by (image, atom)
            found_image.append(pair[:, 0])
            found_atom.append(part[pair[:, 1]])
        image = torch.cat(found_image) if found_image else torch.zeros(0, dtype=torch.int64, device=dev)
        atom = torch.cat(found_atom) if found_atom else torch.zeros(0, dtype=torch.int64, device=dev)
        if len(atoms) > chunk:                                                    # chunks broke the (image, atom) order
            order = torch.argsort(image * (int(self.f.shape[0]) + 1) + atom)
            image, atom = image[order], atom[order]
        return image, atom, images


def partition(plan: DomainPlan, positions: torch.Tensor, rank: int, geometry: _Geometry | None = None) -> HaloPartition:
    """The share of ``rank``: its owned atoms, its halo (ordered by owner) and, for every peer, which of its owned
    atoms the peer holds as halo atoms, in the peer's order. Pure tensor code on the positions' device; every rank runs
    it on the same global positions and gets lists that match its peers' without talking to them."""
    g = geometry or _Geometry(plan, positions)
    dev = positions.device
    n_ranks = plan.n_ranks
    everyone = torch.arange(positions.shape[0], device=dev)
    owned = everyone[g.owner == rank]
    # my halo: every atom, every image
    image, atom, images = g.in_halo(rank, everyone)
    order = torch.argsort(g.owner[atom], stable=True)
    image, atom = image[order], atom[order]
    shift = torch.cat([_times_3x3(-g.base[owned], g.cell), _times_3x3(images[image] - g.base[atom], g.cell)])
    recv_counts = torch.bincount(g.owner[atom], minlength=n_ranks).tolist()
    # what the peers hold of mine: their halo boxes tested on my atoms only (the same comparisons on the same numbers)
    local_of = torch.full((positions.shape[0],), -1, dtype=torch.int64, device=dev)
    local_of[owned] = torch.arange(len(owned), device=dev)
    send, send_counts = [], []
    for peer in range(n_ranks):
        _, mine, _ = g.in_halo(peer, owned)
        send.append(local_of[mine])
        send_counts.append(int(mine.shape[0]))
    send_index = torch.cat(send) if send else torch.zeros(0, dtype=torch.int64, device=dev)
    add_source = torch.argsort(send_index, stable=True)
    add_ptr = torch.zeros(len(owned) + 1, dtype=torch.int64, device=dev)
    add_ptr[1:] = torch.cumsum(torch.bincount(send_index, minlength=len(owned)), dim=0)
    return HaloPartition(rank=rank, owned=owned, halo=atom, shift=shift.contiguous(), recv_counts=recv_counts,
                         send_index=send_index.to(torch.int32).contiguous(), send_counts=send_counts,
                         add_ptr=add_ptr.to(torch.int32).contiguous(), add_source=add_source.to(torch.int32).contiguous())


def halo_box(plan: DomainPlan, rank: int, slack: float):
    """(origin [3], lengths [3]) of an axis-aligned box around ``rank``'s halo box with ``slack`` to spare: the
    non-periodic frame the rank's neighbour list lives in (no periodic image of it is within reach of itself)."""
    lo, hi = plan.brick(rank)
    margin = plan.inner / plan.widths
    corners = np.array([[(lo - margin)[a] if (k >> a) & 1 == 0 else (hi + margin)[a] for a in range(3)]
                        for k in range(8)]) @ plan.cell
    low, high = corners.min(axis=0) - slack, corners.max(axis=0) + slack
    return low, high - low


# --------------------------------------------------------------------------------------------------- transports


class LocalTransport:
    """All ranks live in this process (one after the other on one device): exchanges are copies."""

    world = None

    def forward(self, send, send_counts, recv, recv_counts):
        """recv[r] block of owner p  <-  send[p] block of peer r (lists indexed by rank; counts[r][p])."""
        n = len(send)
        for r in range(n):
            at = 0
            for p in range(n):
                count = recv_counts[r][p]
                start = sum(send_counts[p][:r])
                assert send_counts[p][r] == count, "the partitions of two ranks disagree"
                if count:
                    recv[r][at:at + count].copy_(send[p][start:start + count])
                at += count

    def reverse(self, halo_rows, recv_counts, back, send_counts):
        """back[p] block of peer r  <-  halo_rows[r] block of owner p."""
        n = len(back)
        for r in range(n):
            at = 0
            for p in range(n):
                count = recv_counts[r][p]
                start = sum(send_counts[p][:r])
                if count:
                    back[p][start:start + count].copy_(halo_rows[r][at:at + count])
                at += count

    def sum_(self, tensors):
        total = torch.stack(list(tensors)).sum(dim=0)
        for t in tensors:
            t.copy_(total)

    def max_(self, tensors):
        top = torch.stack(list(tensors)).max(dim=0).values
        for t in tensors:
            t.copy_(top)


class DistributedTransport:
    """One rank per process: ``torch.distributed`` over NCCL (GPUs) or gloo (CPU tests). An exchange is one
    ``all_to_all_single`` with per-peer row counts, i.e. grouped sends and receives into and out of local buffers."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.world = dist.get_world_size(group)

    def forward(self, send, send_counts, recv, recv_counts):
        self.dist.all_to_all_single(recv[0], send[0], output_split_sizes=list(recv_counts[0]),
                                    input_split_sizes=list(send_counts[0]), group=self.group)

    def reverse(self, halo_rows, recv_counts, back, send_counts):
        self.dist.all_to_all_single(back[0], halo_rows[0], output_split_sizes=list(send_counts[0]),
                                    input_split_sizes=list(recv_counts[0]), group=self.group)

    def sum_(self, tensors):
        self.dist.all_reduce(tensors[0], group=self.group)

    def max_(self, tensors):
        self.dist.all_reduce(tensors[0], op=self.dist.ReduceOp.MAX, group=self.group)

    def check_counts(self, send_counts, recv_counts, device):
        """Every peer expects from this rank what this rank is about to send (one small exchange per re-partition)."""
        mine = torch.tensor(send_counts, dtype=torch.int64, device=device)
        theirs = torch.empty_like(mine)
        self.dist.all_to_all_single(theirs, mine, group=self.group)
        if theirs.tolist() != list(recv_counts):
            raise RuntimeError(f"halo partitions disagree: peers send {theirs.tolist()}, expected {list(recv_counts)}")


# --------------------------------------------------------------------------------------------------- one rank


class HaloRank:
    """State, force field and exchange buffers of one rank."""

    def __init__(self, sim: "DomainSimulation", rank: int):
        from .forcefield import B200ForceField
        self.sim, self.rank = sim, rank
        self.lib, self._lib = sim.lib, sim._lib
        dev = sim.device
        self.part: HaloPartition | None = None
        slack = 2.0 + float(sim.config.skin)
        self.origin, lengths = halo_box(sim.plan, rank, slack)
        reach = sim.spec.r_cut + float(sim.config.skin)
        self.box = np.diag(lengths + 2.0 * reach)          # wide enough that no periodic image of the frame is in range
        self.origin = self.origin - reach
        self.origin_c = (ctypes.c_double * 3)(*self.origin)
        self.box_volume = float(np.prod(np.diag(self.box)))
        self.ff: B200ForceField | None = None
        self.sums = torch.zeros(10, dtype=torch.float64, device=dev)
        self.scalars = torch.zeros(10, dtype=torch.float64, device=dev)
        self.flag = torch.zeros((), dtype=torch.int32, device=dev)
        self.max_disp2 = torch.zeros((), dtype=torch.float64, device=dev)
        self.test = self._lib.NlStruct()

    # ------------------------------------------------------------------ partition
    def set_partition(self, part: HaloPartition, positions: torch.Tensor, velocities: torch.Tensor,
                      random_kick: torch.Tensor | None = None) -> None:
        """Take over the owned atoms of ``part`` from the global arrays and (re)build everything that depends on the
        atom set: state, integrator, local frame, neighbour list, exchange buffers."""
        from .forcefield import B200ForceField
        from .langevin import Langevin
        from .state import RandomStream, SimulationState
        sim, dev = self.sim, self.sim.device
        self.part = part
        n_own, n_loc = part.n_owned, part.n_local
        f64 = dict(dtype=torch.float64, device=dev)
        self.active = n_own > 0
        self._send_x = self._back_x = self._back_f = None
        if not self.active:
            # an empty brick (vacuum, more ranks than occupied bricks): nothing to integrate or evaluate; the rank
            # still takes part in the exchanges with rows of zeros for whatever halo atoms it holds
            width = (sim.spec.hidden_lmax + 1) ** 2 * sim.spec.channels
            self.halo_positions = torch.zeros(part.n_halo, 3, **f64)
            self.send_positions = torch.zeros(0, 3, **f64)
            self._idle_rows = torch.zeros(part.n_halo, width, dtype=torch.float32, device=dev)
            self._idle_forces = torch.zeros(part.n_halo, 3, dtype=torch.float32, device=dev)
            self._send_x = self._back_x = torch.zeros(0, width, dtype=torch.float32, device=dev)
            self._back_f = torch.zeros(0, 3, dtype=torch.float32, device=dev)
            self.sums.zero_(); self.scalars.zero_(); self.flag.zero_()
            self.state = None
            return
        local_ids = torch.cat([part.owned, part.halo])
        numbers = sim.numbers_t[local_ids].cpu().numpy()
        step = sim.step_count
        cursor = torch.full((), sim.step_count, dtype=torch.int32, device=dev)   # the step index keys the noise generator
        self.state = SimulationState(
            positions=positions[part.owned].contiguous(), velocities=velocities[part.owned].contiguous(),
            masses=sim.masses_t[part.owned].reshape(-1, 1).contiguous(), cell=sim.cell_t, species=sim.numbers_t[part.owned],
            forces=torch.zeros(n_own, 3, **f64), energy=torch.zeros(1, **f64), stress=torch.zeros(3, 3, **f64),
            rng=RandomStream(np.random.default_rng(0)), step=step)
        self.integrator = Langevin(self.state, sim.integrator_config, temperature_K=sim.temperature_K, noise="device",
                                   device_seed=sim.seed, atom_ids=part.owned, n_global=sim.natoms)
        self.integrator.cursor_dev.copy_(cursor)
        if random_kick is not None:
            # a re-partition falls between the two half steps: the second half adds the same random velocity term as
            # the first (langevin.py:259-263), so it moves with the atom
            self.integrator.rnd_vel.copy_(random_kick[part.owned])
        if self.ff is None:
            self.ff = B200ForceField(sim.spec, sim.weights, numbers, self.box, compute_stress=True, device=dev,
                                     neighbours=sim.config, chunk_edges=sim.chunk_edges, packed=sim.packed,
                                     n_owned=n_own, n_inner=n_own, halo_exchange=True,
                                     atom_capacity=int(n_loc * sim.atom_headroom) + 64)
        else:
            self.ff.set_atoms(numbers, n_own, n_own)
        self.x_local = torch.zeros(n_loc, 3, **f64)
        self.halo_positions = torch.zeros(part.n_halo, 3, **f64)
        self.halo_positions.copy_(positions[part.halo])
        self.send_positions = torch.zeros(len(part.send_index), 3, **f64)
        self.reference = self.state.positions.clone()
        t = self.test
        t.n_atoms, t.skin = n_own, float(sim.config.skin)
        t.reference_positions = self.reference.data_ptr()
        t.rebuild_flag, t.max_disp2_bits = self.flag.data_ptr(), self.max_disp2.data_ptr()
        self.local_positions()
        self.ff.rebuild(self.x_local)

    def _row_buffers(self):
        """Send / receive staging for the feature rows (allocated once the force field's buffers exist)."""
        if self._send_x is None:
            dev, width = self.sim.device, self.ff.buf["x"].shape[1] * self.ff.buf["x"].shape[2]
            n_send = len(self.part.send_index)
            self._send_x = torch.zeros(n_send, width, dtype=torch.float32, device=dev)
            self._back_x = torch.zeros(n_send, width, dtype=torch.float32, device=dev)
            self._back_f = torch.zeros(n_send, 3, dtype=torch.float32, device=dev)
        return self._send_x, self._back_x, self._back_f

    # ------------------------------------------------------------------ kernels around the exchanges
    def _check(self, status, what):
        self._lib.check(status, what)

    def local_positions(self) -> None:
        p = self.part
        if not self.active:
            return
        self._check(self.lib.fmb_halo_local_positions(self.state.positions.data_ptr(), p.n_owned,
                                                      self.halo_positions.data_ptr(), p.shift.data_ptr(), p.n_halo,
                                                      ctypes.byref(self.origin_c), self.x_local.data_ptr(),
                                                      self._lib.current_stream()), "fmb_halo_local_positions")

    def pack_positions(self) -> None:
        p = self.part
        if not self.active:
            return
        self._check(self.lib.fmb_halo_gather_rows(self.state.positions.data_ptr(), p.send_index.data_ptr(),
                                                  self.send_positions.data_ptr(), len(p.send_index), 24,
                                                  self._lib.current_stream()), "fmb_halo_gather_rows")

    def pack_x(self):
        p, (send, _, _) = self.part, self._row_buffers()
        if not self.active:
            return send
        self._check(self.lib.fmb_halo_gather_rows(self.ff.buf["x"].data_ptr(), p.send_index.data_ptr(), send.data_ptr(),
                                                  len(p.send_index), send.shape[1] * 4, self._lib.current_stream()),
                    "fmb_halo_gather_rows")
        return send

    def x_halo_rows(self):
        p = self.part
        if not self.active:
            return self._idle_rows
        return self.ff.buf["x"].reshape(self.ff.buf["x"].shape[0], -1)[p.n_owned:p.n_local]

    def dx_halo_rows(self):
        p = self.part
        if not self.active:
            return self._idle_rows.zero_()
        return self.ff.buf["d_x"].reshape(self.ff.buf["d_x"].shape[0], -1)[p.n_owned:p.n_local]

    def add_dx(self) -> None:
        p, (_, back, _) = self.part, self._row_buffers()
        if not self.active:
            return
        self._check(self.lib.fmb_halo_add_rows(back.data_ptr(), p.add_ptr.data_ptr(), p.add_source.data_ptr(), None,
                                               self.ff.buf["d_x"].data_ptr(), p.n_owned, back.shape[1],
                                               self._lib.current_stream()), "fmb_halo_add_rows")

    def force_halo_rows(self):
        p = self.part
        if not self.active:
            return self._idle_forces
        return self.ff.forces[p.n_owned:p.n_local]

    def owned_forces(self) -> None:
        p, (_, _, back) = self.part, self._row_buffers()
        if not self.active:
            return
        self._check(self.lib.fmb_halo_owned_forces(self.ff.forces.data_ptr(), back.data_ptr(), p.add_ptr.data_ptr(),
                                                   p.add_source.data_ptr(), p.n_owned, self.state.forces.data_ptr(),
                                                   self._lib.current_stream()), "fmb_halo_owned_forces")
        self.scalars[0:1].copy_(self.ff.energy)
        self.scalars[1:10].copy_((self.ff.stress.double() * self.box_volume).reshape(9))

    def displacement_flag(self) -> None:
        if not self.active:
            return
        self._check(self.lib.fmb_nl_needs_rebuild(ctypes.byref(self.test), self.state.positions.data_ptr(), 1.0,
                                                  self._lib.current_stream()), "fmb_nl_needs_rebuild")


# --------------------------------------------------------------------------------------------------- the run


class DomainSimulation:
    """Langevin NVT MD of one structure over ``n_ranks`` bricks.

    ``ranks=None`` with ``transport=None``: every rank lives in this process (``LocalTransport``), which is how one GPU
    emulates the decomposition in tests and how the single-GPU point of a scaling run is taken with the same code.
    Under ``torch.distributed`` pass ``ranks=[rank]`` and a ``DistributedTransport``. The interface follows the
    reference's ``Engine`` (``fastmace/engine/base.py:91-142``: ``step / run / flush / potential_energy / info``); the
    step is its checked step (``fastmace/engine/graph.py:968-998``) with the exchanges between the stages.
    """

    def __init__(self, spec, weights, structure, n_ranks: int, *, temperature_K: float, seed: int = 0, device="cuda",
                 ranks=None, transport=None, neighbours=None, integrator_config=None, chunk_edges: int | None = None,
                 atom_headroom: float = 1.08):
        from . import _lib
        from .forcefield import DEFAULT_CHUNK_EDGES
        from .langevin import IntegratorConfig
        from .neighbours import NeighbourConfig
        from .packing import PackedModel
        self._lib, self.lib = _lib, _lib.load()
        self.spec, self.weights = spec, weights
        self.device = torch.device(device)
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.config = neighbours or NeighbourConfig()
        self.integrator_config = integrator_config or IntegratorConfig()
        self.temperature_K, self.seed = float(temperature_K), int(seed)
        self.chunk_edges = chunk_edges          # None: B200ForceField decides from the free memory
        self.atom_headroom = float(atom_headroom)
        self.cell = np.asarray(structure.cell, dtype=np.float64).reshape(3, 3)
        self.natoms = int(structure.natoms)
        self.volume = abs(float(np.linalg.det(self.cell)))
        dev, f64 = self.device, dict(dtype=torch.float64, device=self.device)
        self.numbers_t = torch.tensor(np.asarray(structure.numbers), dtype=torch.int64, device=dev)
        self.masses_t = torch.tensor(np.asarray(structure.masses), **f64)
        self.cell_t = torch.tensor(self.cell, **f64)
        self.plan = DomainPlan(self.cell, n_ranks, inner=spec.r_cut + float(self.config.skin),
                               outer=spec.r_cut + float(self.config.skin))
        self.packed = PackedModel(spec, weights, sorted(set(int(z) for z in structure.numbers)), dev)
        self.transport = transport or LocalTransport()
        self.rank_ids = list(range(n_ranks)) if ranks is None else list(ranks)
        self.ranks = [HaloRank(self, r) for r in self.rank_ids]
        self.step_count = 0
        self.repartitions = 0
        self.repartition_seconds = 0.0
        self.repartition_log: list[float] = []      # seconds of each re-partition (the first one sets the buffers up)
        self.energy = torch.zeros(1, **f64)
        self.stress = torch.zeros(3, 3, **f64)
        positions = torch.tensor(np.asarray(structure.positions), **f64)
        velocities = torch.tensor(np.asarray(structure.velocities if structure.velocities is not None
                                             else np.zeros_like(structure.positions)), **f64)
        self._repartition(positions, velocities)
        self._forces()
        self.flush()

    # ------------------------------------------------------------------ partition
    def global_state(self):
        """(positions, velocities, random velocity term of the step in flight) of all atoms, [N, 3] float64 each,
        identical on every rank: each rank writes its owned rows into zeros and the ranks' arrays are added
        (x + 0 = x exactly)."""
        rows = torch.zeros(self.natoms, 9, dtype=torch.float64, device=self.device)
        for r in self.ranks:
            if r.active:
                rows[r.part.owned, 0:3] = r.state.positions
                rows[r.part.owned, 3:6] = r.state.velocities
                rows[r.part.owned, 6:9] = r.integrator.rnd_vel
        if self.transport.world is not None:
            self.transport.sum_([rows])
        return rows[:, 0:3].contiguous(), rows[:, 3:6].contiguous(), rows[:, 6:9].contiguous()

    def _repartition(self, positions: torch.Tensor, velocities: torch.Tensor, random_kick=None) -> None:
        import time
        torch.cuda.synchronize(self.device)
        t0 = time.perf_counter()
        geometry = _Geometry(self.plan, positions)
        for r in self.ranks:
            part = partition(self.plan, positions, r.rank, geometry)
            if isinstance(self.transport, DistributedTransport):
                self.transport.check_counts(part.send_counts, part.recv_counts, self.device)
            r.set_partition(part, positions, velocities, random_kick)
        torch.cuda.synchronize(self.device)
        self.repartition_seconds += time.perf_counter() - t0
        self.repartition_log.append(round(time.perf_counter() - t0, 4))
        self.repartitions += 1

    # ------------------------------------------------------------------ exchanges
    def _counts(self):
        return [r.part.send_counts for r in self.ranks], [r.part.recv_counts for r in self.ranks]

    def _exchange_positions(self) -> None:
        send_counts, recv_counts = self._counts()
        for r in self.ranks:
            r.pack_positions()
        self.transport.forward([r.send_positions for r in self.ranks], send_counts,
                               [r.halo_positions for r in self.ranks], recv_counts)
        for r in self.ranks:
            r.local_positions()

    def _forces(self) -> None:
        t, ranks = self.transport, self.ranks
        send_counts, recv_counts = self._counts()
        for r in ranks:
            if r.active:
                r.ff.compact(r.x_local)
                r.ff.phase(0, r.x_local)
        t.forward([r.pack_x() for r in ranks], send_counts, [r.x_halo_rows() for r in ranks], recv_counts)
        for r in ranks:
            if r.active:
                r.ff.phase(1)
        t.reverse([r.dx_halo_rows() for r in ranks], recv_counts, [r._row_buffers()[1] for r in ranks], send_counts)
        for r in ranks:
            if r.active:
                r.add_dx()
                r.ff.phase(2)
        t.reverse([r.force_halo_rows() for r in ranks], recv_counts, [r._row_buffers()[2] for r in ranks], send_counts)
        for r in ranks:
            r.owned_forces()
        t.sum_([r.scalars for r in ranks])
        s = ranks[0].scalars
        self.energy.copy_(s[0:1])
        self.stress.copy_((s[1:10] / self.volume).reshape(3, 3))
        for r in ranks:
            if r.active:
                r.state.energy.copy_(self.energy)

    # ------------------------------------------------------------------ Engine interface
    def step(self) -> None:
        t, ranks = self.transport, self.ranks
        for r in ranks:
            if r.active:
                r.integrator.noise_sums(r.state, r.sums)
        t.sum_([r.sums for r in ranks])
        for r in ranks:
            if r.active:
                r.integrator.first_half_global(r.state, r.sums)
                r.displacement_flag()
        t.max_([r.flag for r in ranks])
        if int(ranks[0].flag.item()):                      # the one host read per step (graph.py:974-978)
            self._repartition(*self.global_state())
        else:
            self._exchange_positions()
        self._forces()
        for r in ranks:
            if r.active:
                r.integrator.second_half(r.state)
                r.state.step += 1
        self.step_count += 1

    def run(self, steps: int) -> None:
        for _ in range(steps):
            self.step()
        self.flush()

    def flush(self) -> None:
        torch.cuda.synchronize(self.device)
        for r in self.ranks:
            if r.active:
                r.ff.check_status()

    def potential_energy(self) -> float:
        self.flush()
        return float(self.energy.item())

    def gather(self):
        """Global (positions, velocities, forces) as float64 NumPy arrays (synchronises; for tests and output)."""
        positions, velocities, _ = self.global_state()
        forces = torch.zeros(self.natoms, 3, dtype=torch.float64, device=self.device)
        for r in self.ranks:
            if r.active:
                forces[r.part.owned] = r.state.forces
        if self.transport.world is not None:
            self.transport.sum_([forces])
        return positions.cpu().numpy(), velocities.cpu().numpy(), forces.cpu().numpy()

    def info(self):
        r = self.ranks[0]
        return {"engine": "fmb200-halo", "ranks": self.plan.n_ranks, "bricks": self.plan.grid, "rank": r.rank,
                "owned_atoms": r.part.n_owned, "local_atoms": r.part.n_local, "halo_rows_sent": len(r.part.send_index),
                "repartitions": self.repartitions, "repartition_seconds": round(self.repartition_seconds, 4),
                "repartition_log": list(self.repartition_log),
                "steps": self.step_count,
                "local_edges": int(r.ff.edge_count.item()) if r.active else 0,
                "streaming_interactions": self.spec.num_interactions, "sort_receivers": True,
                "owned_all": [x.part.n_owned for x in self.ranks], "local_all": [x.part.n_local for x in self.ranks]}


__all__ = ["HaloPartition", "partition", "halo_box", "LocalTransport", "DistributedTransport", "HaloRank",
           "DomainSimulation"]
