"""Spatial domain decomposition of the force call over the GPUs of one node.

The reference runs one structure on one GPU (multi-GPU decomposition is a stated non-goal, ``SPEC.md:70-74``); its
only structural precedent is the tiled path, where a tile is "receivers + their edges + halo senders laid out like
LAMMPS ghosts" (``fastmace/model/tiled.py:1-26``, ``docs/design/tiled-backend.md:54-110``). The scheme here:

* the periodic cell is cut into bricks in fractional coordinates, one per rank; a rank *owns* the atoms inside its
  brick and imports two halo shells as ghost atoms (explicit periodic images): the inner shell (within cutoff + skin)
  holds every sender of an owned receiver, the outer shell (twice that) every sender of an inner-shell atom. Layer 0's
  senders are species-only (``tiled-backend.md:84-90``), so the outer shell needs no features of its own;
* local atoms are ordered owned | inner | outer; the force kernels compute first-layer rows for owned + inner atoms,
  last-layer rows and energies for owned atoms only, and forces (partial sums) for every local atom;
* the MD state is replicated: every rank holds all positions and integrates all atoms with the same noise, so ghost
  positions need no exchange; the ONE data-path collective per step is the all-reduce that sums the ranks' partial
  forces (the "reverse force accumulation"), together with the energy and the virial.

``DomainPlan`` is pure NumPy (tested on CPU, also under a 2-rank gloo group); ``DomainForceField`` runs the device path.
"""

from __future__ import annotations

import dataclasses
import math

import numpy as np


def brick_grid(cell: np.ndarray, n_ranks: int) -> tuple[int, int, int]:
    """Bricks per axis (px, py, pz) with px * py * pz = n_ranks, the most cubic bricks for this cell."""
    widths = 1.0 / np.linalg.norm(np.linalg.inv(cell), axis=0)
    best, best_score = (n_ranks, 1, 1), None
    for px in range(1, n_ranks + 1):
        if n_ranks % px:
            continue
        for py in range(1, n_ranks // px + 1):
            if (n_ranks // px) % py:
                continue
            pz = n_ranks // (px * py)
            sides = sorted([widths[0] / px, widths[1] / py, widths[2] / pz])
            score = sides[2] / sides[0]
            if best_score is None or score < best_score - 1e-12:
                best, best_score = (px, py, pz), score
    return best


@dataclasses.dataclass
class LocalAtoms:
    index: np.ndarray        # [n_local] global atom index of every local atom (owned | inner | outer)
    image: np.ndarray        # [n_local, 3] integer cell shift added to the global position
    n_owned: int
    n_inner: int             # owned + inner shell

    @property
    def n_local(self) -> int:
        return int(len(self.index))


class DomainPlan:
    """Brick decomposition of a periodic cell and the ghost shells of each brick."""

    def __init__(self, cell, n_ranks: int, inner: float, outer: float):
        self.cell = np.asarray(cell, dtype=np.float64).reshape(3, 3)
        self.inverse = np.linalg.inv(self.cell)
        self.n_ranks = int(n_ranks)
        self.grid = brick_grid(self.cell, self.n_ranks)
        self.widths = 1.0 / np.linalg.norm(self.inverse, axis=0)   # distance between opposite cell faces
        self.inner, self.outer = float(inner), float(outer)
        if outer < inner:
            raise ValueError("the outer shell must contain the inner one")

    def brick(self, rank: int):
        px, py, pz = self.grid
        b = (rank // (py * pz), (rank // pz) % py, rank % pz)
        lo = np.array([b[0] / px, b[1] / py, b[2] / pz])
        hi = np.array([(b[0] + 1) / px, (b[1] + 1) / py, (b[2] + 1) / pz])
        return lo, hi

    def fractional(self, positions: np.ndarray):
        frac = positions @ self.inverse
        base = np.floor(frac)
        return frac - base, base.astype(np.int64)

    def owner(self, positions: np.ndarray) -> np.ndarray:
        """Rank that owns each atom."""
        f, _ = self.fractional(np.asarray(positions, dtype=np.float64))
        px, py, pz = self.grid
        b = np.minimum((f * np.array([px, py, pz])).astype(np.int64), np.array([px, py, pz]) - 1)
        return (b[:, 0] * py + b[:, 1]) * pz + b[:, 2]

    def local_atoms(self, positions: np.ndarray, rank: int) -> LocalAtoms:
        """Owned atoms of ``rank`` and the periodic images inside its two halo shells. A shell of width h is the
        box that extends the brick by h / (face distance) in fractional coordinates: a superset of every point
        within h of the brick, for any cell shape."""
        positions = np.asarray(positions, dtype=np.float64)
        f, base = self.fractional(positions)
        lo, hi = self.brick(rank)
        own_rank = self.owner(positions)
        margin_in, margin_out = self.inner / self.widths, self.outer / self.widths
        reach = [int(math.floor(m + (h - l))) + 1 for m, l, h in zip(margin_out, lo, hi)]
        owned_mask = own_rank == rank
        owned = np.flatnonzero(owned_mask)
        # per axis and image: is the shifted coordinate inside the inner / outer box? (27 cheap boolean ANDs follow)
        out_ax = [{n: (f[:, a] + n >= lo[a] - margin_out[a]) & (f[:, a] + n < hi[a] + margin_out[a])
                   for n in range(-reach[a], reach[a] + 1)} for a in range(3)]
        in_ax = [{n: (f[:, a] + n >= lo[a] - margin_in[a]) & (f[:, a] + n < hi[a] + margin_in[a])
                  for n in range(-reach[a], reach[a] + 1)} for a in range(3)]
        inner_idx, inner_img, outer_idx, outer_img = [], [], [], []
        for n0 in range(-reach[0], reach[0] + 1):
            if not out_ax[0][n0].any():
                continue
            for n1 in range(-reach[1], reach[1] + 1):
                o01 = out_ax[0][n0] & out_ax[1][n1]
                if not o01.any():
                    continue
                i01 = in_ax[0][n0] & in_ax[1][n1]
                for n2 in range(-reach[2], reach[2] + 1):
                    in_outer = o01 & out_ax[2][n2]
                    if not in_outer.any():
                        continue
                    n = np.array([n0, n1, n2])
                    in_inner = i01 & in_ax[2][n2]
                    pick_in = np.flatnonzero(in_inner & ~owned_mask) if not n.any() else np.flatnonzero(in_inner)
                    pick_out = np.flatnonzero(in_outer & ~in_inner)
                    inner_idx.append(pick_in)
                    inner_img.append(np.broadcast_to(n, (len(pick_in), 3)))
                    outer_idx.append(pick_out)
                    outer_img.append(np.broadcast_to(n, (len(pick_out), 3)))
        index = np.concatenate([owned, *inner_idx, *outer_idx]).astype(np.int64)
        image = np.concatenate([np.zeros((len(owned), 3), dtype=np.int64), *inner_img, *outer_img]).astype(np.int64)
        image = image - base[index]          # relative to the (possibly unwrapped) global position
        n_inner = len(owned) + sum(len(k) for k in inner_idx)
        return LocalAtoms(index, image, int(len(owned)), int(n_inner))

    def local_atoms_device(self, positions, rank: int):
        """``local_atoms`` with torch tensors on the positions' device (the same boolean algebra; a re-partition of
        10^6 atoms takes milliseconds there instead of most of a second on the host). Returns
        (index int64 [n_local], image int64 [n_local, 3], n_owned, n_inner) as device tensors and ints."""
        import torch
        dev = positions.device
        inverse = torch.as_tensor(self.inverse, dtype=torch.float64, device=dev)
        frac = positions @ inverse
        base = torch.floor(frac)
        f = frac - base
        base = base.to(torch.int64)
        px, py, pz = self.grid
        grid = torch.tensor([px, py, pz], device=dev)
        b = torch.minimum((f * grid).to(torch.int64), grid - 1)
        own_rank = (b[:, 0] * py + b[:, 1]) * pz + b[:, 2]
        lo, hi = self.brick(rank)
        margin_in, margin_out = self.inner / self.widths, self.outer / self.widths
        reach = [int(math.floor(m + (h - l))) + 1 for m, l, h in zip(margin_out, lo, hi)]
        owned_mask = own_rank == rank
        owned = torch.nonzero(owned_mask).reshape(-1)
        out_ax = [{n: (f[:, a] + n >= lo[a] - margin_out[a]) & (f[:, a] + n < hi[a] + margin_out[a])
                   for n in range(-reach[a], reach[a] + 1)} for a in range(3)]
        in_ax = [{n: (f[:, a] + n >= lo[a] - margin_in[a]) & (f[:, a] + n < hi[a] + margin_in[a])
                  for n in range(-reach[a], reach[a] + 1)} for a in range(3)]
        inner_idx, inner_img, outer_idx, outer_img = [], [], [], []
        for n0 in range(-reach[0], reach[0] + 1):
            for n1 in range(-reach[1], reach[1] + 1):
                o01 = out_ax[0][n0] & out_ax[1][n1]
                i01 = in_ax[0][n0] & in_ax[1][n1]
                for n2 in range(-reach[2], reach[2] + 1):
                    in_outer = o01 & out_ax[2][n2]
                    in_inner = i01 & in_ax[2][n2]
                    zero = n0 == 0 and n1 == 0 and n2 == 0
                    pick_in = torch.nonzero(in_inner & ~owned_mask if zero else in_inner).reshape(-1)
                    pick_out = torch.nonzero(in_outer & ~in_inner).reshape(-1)
                    n = torch.tensor([n0, n1, n2], device=dev)
                    inner_idx.append(pick_in)
                    inner_img.append(n.expand(len(pick_in), 3))
                    outer_idx.append(pick_out)
                    outer_img.append(n.expand(len(pick_out), 3))
        index = torch.cat([owned, *inner_idx, *outer_idx])
        image = torch.cat([torch.zeros(len(owned), 3, dtype=torch.int64, device=dev), *inner_img, *outer_img])
        image = image - base[index]
        n_inner = len(owned) + sum(len(k) for k in inner_idx)
        return index, image, int(len(owned)), int(n_inner)

    def local_positions(self, positions: np.ndarray, local: LocalAtoms) -> np.ndarray:
        return positions[local.index] + local.image.astype(np.float64) @ self.cell


__all__ = ["DomainPlan", "LocalAtoms", "brick_grid"]


class _GlobalRebuildTest:
    """``needs_rebuild`` over the replicated global positions (every rank takes the same decision without
    communicating), through the same kernel as the single-GPU list."""

    def __init__(self, natoms: int, skin: float, device):
        import torch

        from . import _lib
        self.lib, self._lib = _lib.load(), _lib
        self.rebuilds = 0
        self.skin = float(skin)
        self.reference_positions = torch.zeros(natoms, 3, dtype=torch.float64, device=device)
        self.rebuild_flag = torch.zeros((), dtype=torch.int32, device=device)
        self.max_disp2 = torch.zeros((), dtype=torch.float64, device=device)
        self.struct = _lib.NlStruct()
        self.struct.n_atoms, self.struct.skin = natoms, self.skin
        self.struct.reference_positions = self.reference_positions.data_ptr()
        self.struct.rebuild_flag = self.rebuild_flag.data_ptr()
        self.struct.max_disp2_bits = self.max_disp2.data_ptr()

    def needs_rebuild(self, positions, fraction: float = 1.0):
        import ctypes
        self._lib.check(self.lib.fmb_nl_needs_rebuild(ctypes.byref(self.struct), positions.data_ptr(), float(fraction),
                                                      self._lib.current_stream()), "fmb_nl_needs_rebuild")
        return self.rebuild_flag


class DomainForceField:
    """The ``ForceField`` protocol (``fastmace/model/forces.py:63-161``) for one rank of a domain-decomposed run.

    Takes and returns GLOBAL arrays: ``__call__(positions [N, 3] float64)`` gathers this rank's local atoms, runs
    the device force path on them (``B200ForceField`` with the owned | inner | outer ordering) and sums the ranks'
    partial forces, energies and virials with one all-reduce each. ``group`` is a ``torch.distributed`` process group
    (NCCL); with ``group=None`` the object covers rank ``rank`` of ``n_ranks`` without communicating, which is how one
    process emulates all ranks in the single-GPU tests.
    """

    dtype = None
    padding_exact = True
    compile_mode = "none"

    def __init__(self, spec, weights, numbers, cell, *, rank: int, n_ranks: int, device="cuda", group=None,
                 compute_stress: bool = True, neighbours=None, chunk_edges: int | None = None):
        import torch

        from . import _lib
        from .forcefield import DEFAULT_CHUNK_EDGES
        from .neighbours import NeighbourConfig
        from .packing import PackedModel
        self.torch, self._lib = torch, _lib
        self.spec, self.weights = spec, weights
        self.numbers = np.asarray(numbers, dtype=np.int64)
        self.cell = np.asarray(cell, dtype=np.float64).reshape(3, 3)
        self.rank, self.n_ranks, self.group = int(rank), int(n_ranks), group
        self._device = torch.device(device)
        if self._device.index is None:
            self._device = torch.device("cuda", torch.cuda.current_device())
        self._compute_stress = bool(compute_stress)
        self.config = neighbours or NeighbourConfig()
        self.chunk_edges = chunk_edges or DEFAULT_CHUNK_EDGES
        skin = float(self.config.skin)
        # an atom moves at most skin / 2 between rebuilds, so shells wider by one skin hold their atoms until then
        self.plan = DomainPlan(self.cell, n_ranks, inner=spec.r_cut + skin, outer=2.0 * (spec.r_cut + skin))
        self.packed = PackedModel(spec, weights, sorted(set(int(z) for z in self.numbers)), self._device)
        self.natoms = len(self.numbers)
        self.volume = abs(float(np.linalg.det(self.cell)))
        self.neighbours = _GlobalRebuildTest(self.natoms, skin, self._device)
        f64 = dict(dtype=torch.float64, device=self._device)
        self.energy = torch.zeros(1, **f64)
        self.forces = torch.zeros(self.natoms, 3, dtype=torch.float32, device=self._device)
        self.stress = torch.zeros(3, 3, dtype=torch.float32, device=self._device)
        self.scalars = torch.zeros(10, **f64)                 # energy + virial, reduced together
        self.cell_t = torch.tensor(self.cell, **f64)
        self.local = None
        self.local_ff = None
        self.calls = 0
        self.work = _lib.WorkStruct()                         # the global outputs, for fmb_commit_forces
        self.work.n_atoms, self.work.compute_stress = self.natoms, int(self._compute_stress)
        self.work.forces, self.work.energy = self.forces.data_ptr(), self.energy.data_ptr()
        self.work.stress = self.stress.data_ptr()

    @property
    def device(self):
        return self._device

    @property
    def compute_stress(self) -> bool:
        return self._compute_stress

    @property
    def edge_count(self):
        return self.local_ff.edge_count

    @property
    def edge_capacity(self) -> int:
        return self.local_ff.edge_capacity

    # ------------------------------------------------------------------ partition (host, at rebuilds)
    def _local_positions(self, positions):
        return positions.index_select(0, self.local_index) + self.local_shift

    def rebuild(self, positions) -> bool:
        """Re-partition from the global positions and rebuild this rank's neighbour list. Always returns True: the
        local atom set changes, so every local buffer is new."""
        torch = self.torch
        from .forcefield import B200ForceField
        index, image, n_owned, n_inner = self.plan.local_atoms_device(positions, self.rank)
        local = LocalAtoms(index.cpu().numpy(), image.cpu().numpy(), n_owned, n_inner)
        reach = self.spec.r_cut + float(self.config.skin)
        shift = image.to(torch.float64) @ self.cell_t
        x = positions.index_select(0, index) + shift
        lo_t, hi_t = x.min(dim=0).values, x.max(dim=0).values
        lo = lo_t.cpu().numpy() - (reach + 2.0)
        box = np.diag(hi_t.cpu().numpy() - lo_t.cpu().numpy() + 2.0 * (reach + 2.0))   # no periodic image is in range
        self.local = local
        self.local_index = index
        self.local_shift = shift - torch.as_tensor(lo, dtype=torch.float64, device=self._device)
        self.local_ff = B200ForceField(self.spec, self.weights, self.numbers[local.index], box,
                                       compute_stress=True, device=self._device, neighbours=self.config,
                                       chunk_edges=self.chunk_edges, packed=self.packed, n_owned=local.n_owned,
                                       n_inner=local.n_inner)
        self.local_box_volume = float(np.prod(np.diag(box)))
        if local.n_owned > 0:
            self.local_ff.rebuild(self._local_positions(positions))
        self.neighbours.reference_positions.copy_(positions)
        self.neighbours.rebuilds += 1
        return True

    def compact(self, positions) -> None:
        if self.local.n_owned > 0:
            self.local_ff.compact(self._local_positions(positions))

    def needs_rebuild(self, positions, fraction: float = 1.0):
        return self.neighbours.needs_rebuild(positions, fraction) != 0

    def use_edges(self, num_edges: int) -> None:
        self.local_ff.use_edges(num_edges)

    # ------------------------------------------------------------------ force call
    def partial(self, positions):
        """This rank's contribution before the reduction: (energy+virial scalars [10], forces [N, 3])."""
        self.forces.zero_()
        if self.local.n_owned == 0:
            # an empty brick (vacuum slab, more ranks than occupied bricks): nothing to evaluate, zeros to the sums
            self.scalars.zero_()
            return self.scalars, self.forces
        out = self.local_ff(self._local_positions(positions))
        self.forces.index_add_(0, self.local_index, out.forces)
        self.scalars[0:1].copy_(out.energy)
        self.scalars[1:10].copy_((out.stress.double() * self.local_box_volume).reshape(9))
        return self.scalars, self.forces

    def finish(self) -> None:
        """Global energy and stress from the (reduced) scalars."""
        self.energy.copy_(self.scalars[0:1])
        self.stress.copy_((self.scalars[1:10] / self.volume).reshape(3, 3))

    def __call__(self, positions):
        from .forcefield import ForceOutput
        self.calls += 1
        self.partial(positions)
        if self.group is not None:
            import torch.distributed as dist
            dist.all_reduce(self.forces, group=self.group)         # the reverse force accumulation
            dist.all_reduce(self.scalars, group=self.group)
        self.finish()
        return ForceOutput(self.energy, self.forces, self.stress if self._compute_stress else None)

    def evaluate(self, atoms, stress: bool = False):
        torch = self.torch
        x = torch.as_tensor(np.asarray(atoms.get_positions(), dtype=np.float64), device=self._device)
        self.rebuild(x)
        self.compact(x)
        out = self(x)
        torch.cuda.synchronize(self._device)
        self.check_status()
        return (float(out.energy.item()), out.forces.double().cpu().numpy(),
                out.stress.double().cpu().numpy() if stress else None)

    def check_status(self) -> None:
        if self.local.n_owned > 0:
            self.local_ff.check_status()

    def buffers(self):
        return {f"neighbours.{k}": v for k, v in self.local_ff.neighbours.buffers().items()}

    def info(self):
        return {"streaming_interactions": self.spec.num_interactions, "sort_receivers": True,
                "neighbour_rebuilds": self.neighbours.rebuilds, "engine": "fmb200-domain", "rank": self.rank,
                "ranks": self.n_ranks, "bricks": self.plan.grid, "local_atoms": self.local.n_local if self.local else 0,
                "owned_atoms": self.local.n_owned if self.local else 0, "force_calls": self.calls}


__all__ += ["DomainForceField"]
