"""Host side of the device neighbour list: the interface of FastMACE's ``SkinNeighbourList``
(``fastmace/neighbors/skin.py:164-747``) over the cell-list kernels of ``csrc/neighbours.cu``.

Same members and buffer names as the reference (``candidate_index``, ``candidate_unit_shifts``, ``edge_index``,
``unit_shifts``, ``shifts``, ``count``, ``reference_positions``, ``build_cell``; ``skin.py:606-621``), always
receiver-sorted, with CSR row pointers over the compacted edges (``edge_row_ptr``) in addition. The padded-size helpers
are those of ``fastmace/neighbors/buckets.py:19-34``.
"""

from __future__ import annotations

import ctypes
import dataclasses
import math

import numpy as np
import torch

from . import _lib

DEFAULT_SKIN_A = 0.3   # fastmace/config.py:49


def edge_bucket(reference_count: int, fraction: float, multiple: int) -> int:
    """Step between padded edge counts (buckets.py:19-24)."""
    return multiple * max(1, math.ceil(fraction * reference_count / multiple))


def round_up_edges(count: int, capacity: int, bucket: int) -> int:
    """Padded edge size for ``count`` edges (buckets.py:27-29)."""
    return min(capacity, bucket * max(1, math.ceil(count / bucket)))


def edge_capacity(needed: int, headroom: float, multiple: int) -> int:
    """Buffer size for ``needed`` candidate pairs (buckets.py:32-34)."""
    return multiple * max(1, math.ceil(int(needed * headroom) / multiple))


@dataclasses.dataclass(frozen=True)
class NeighbourConfig:
    """The fields of the reference's ``NeighbourConfig`` this list reads (``fastmace/config.py:400-440``)."""
    skin: float = DEFAULT_SKIN_A
    edge_multiple: int = 256
    edge_bucket_fraction: float = 0.05
    capacity_headroom: float = 1.15
    sort_receivers: str = "on"
    gpu_neighbour_list: str = "on"
    edge_index_int32: str = "on"


def cell_list_plan(cell: np.ndarray, reach: float):
    """(nbins[3], reach_bins[3]) of the fractional cell list: slabs at least ``reach`` thick along every axis."""
    widths = 1.0 / np.linalg.norm(np.linalg.inv(cell), axis=0)
    nbins = [max(1, int(math.floor(w / reach))) for w in widths]
    reach_bins = [int(math.floor(reach * nb / w)) + 1 for nb, w in zip(nbins, widths)]
    return nbins, reach_bins


class CellListNeighbours:
    """Periodic pairs within cutoff + skin built on the device, compacted to the cutoff each step."""

    def __init__(self, cell, cutoff: float, device, float_dtype=torch.float32, config: NeighbourConfig | None = None,
                 atom_capacity: int = 0):
        self.lib = _lib.load()
        self.config = config or NeighbourConfig()
        self.cell = np.asarray(cell, dtype=np.float64).reshape(3, 3).copy()
        self.cutoff = float(cutoff)
        self.skin = float(self.config.skin)
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise _lib.Fmb200Error("the neighbour list runs on a CUDA device only (no CPU path)")
        if float_dtype != torch.float32:
            raise ValueError("unit shifts and shifts are float32 (the model precision)")
        self.float_dtype = float_dtype
        self.edge_multiple = self.config.edge_multiple
        self.headroom = self.config.capacity_headroom
        self.sort_receivers = True
        self.capacity = 0
        self.num_candidates = 0
        self.rebuilds = 0
        self.variable_cell = False
        self.reader_stream = None
        self.natoms = None
        self.atom_capacity = int(atom_capacity)      # rows of the per-atom buffers (0: the atoms of the first build)
        self.struct = _lib.NlStruct()
        self._set_cell_constants()
        dev = self.device
        self.count = torch.zeros((), dtype=torch.int64, device=dev)
        self.num_candidates_dev = torch.zeros((), dtype=torch.int64, device=dev)
        self.status = torch.zeros((), dtype=torch.int32, device=dev)
        self.rebuild_flag = torch.zeros((), dtype=torch.int32, device=dev)
        self.max_disp2 = torch.zeros((), dtype=torch.float64, device=dev)
        self.build_cell = torch.tensor(self.cell, dtype=torch.float64, device=dev)
        self._reference_all = None

    @property
    def reference_positions(self):
        return None if self._reference_all is None else self._reference_all[:self.natoms]

    # ------------------------------------------------------------------ set-up
    def _set_cell_constants(self):
        reach = self.cutoff + self.skin
        lengths = np.linalg.norm(self.cell, axis=1)
        axis = int(np.argmax(lengths))
        self._pad_unit_shift = np.zeros(3)
        self._pad_unit_shift[axis] = math.ceil(2 * reach / lengths[axis]) + 1   # skin.py:247-252
        self.nbins, self.reach_bins = cell_list_plan(self.cell, reach)
        if max(self.reach_bins) > 100:
            raise ValueError("cell far smaller than the cutoff: more than 100 periodic images per axis")
        s = self.struct
        s.cutoff, s.skin = self.cutoff, self.skin
        inverse = np.linalg.inv(self.cell)
        for k in range(9):
            s.cell[k] = float(self.cell.reshape(-1)[k])
            s.inverse[k] = float(inverse.reshape(-1)[k])
        for a in range(3):
            s.nbins[a] = self.nbins[a]
            s.reach_bins[a] = self.reach_bins[a]
            s.pad_unit_shift[a] = float(self._pad_unit_shift[a])

    def set_natoms(self, natoms: int) -> None:
        """Another number of atoms in the same buffers (a re-partition); the list must be rebuilt afterwards."""
        if self.natoms is None:
            return
        if natoms > self.atom_capacity:
            raise ValueError(f"{natoms} atoms exceed the list's capacity of {self.atom_capacity}")
        self.natoms = int(natoms)
        self.struct.n_atoms = int(natoms)
        self.num_candidates = 0

    def set_atom_capacity(self, capacity: int) -> None:
        self.atom_capacity = int(capacity)
        if self.natoms is not None:
            self._allocate_atoms(min(self.natoms, self.atom_capacity))

    def _allocate_atoms(self, live: int):
        dev, i32, f64 = self.device, torch.int32, torch.float64
        self.atom_capacity = max(self.atom_capacity, live)
        natoms = self.atom_capacity
        self.natoms = live
        total_bins = int(np.prod(self.nbins))
        self._bins_allocated = total_bins
        self.wrapped = torch.zeros(natoms, 3, dtype=f64, device=dev)
        self.offsets = torch.zeros(natoms, 3, dtype=f64, device=dev)
        self.atom_bin = torch.zeros(natoms, dtype=i32, device=dev)
        self.bin_count = torch.zeros(total_bins + 1, dtype=i32, device=dev)
        self.bin_start = torch.zeros(total_bins + 1, dtype=i32, device=dev)
        self.bin_fill = torch.zeros(total_bins + 1, dtype=i32, device=dev)
        self.bin_atoms = torch.zeros(natoms, dtype=i32, device=dev)
        self.cand_row_count = torch.zeros(natoms + 1, dtype=i32, device=dev)
        self.cand_row_ptr = torch.zeros(natoms + 1, dtype=i32, device=dev)
        self.edge_row_count = torch.zeros(natoms + 1, dtype=i32, device=dev)
        self.edge_row_ptr = torch.zeros(natoms + 1, dtype=i32, device=dev)
        self.scan_scratch = torch.zeros(2 * (max(natoms, total_bins) // 4096 + 2) + 8, dtype=i32, device=dev)
        self._reference_all = torch.zeros(natoms, 3, dtype=f64, device=dev)
        s = self.struct
        s.n_atoms = live
        for name in ("wrapped", "offsets", "atom_bin", "bin_count", "bin_start", "bin_fill", "bin_atoms",
                     "cand_row_count", "cand_row_ptr", "edge_row_count", "edge_row_ptr", "scan_scratch",
                     "build_cell", "count", "status", "rebuild_flag"):
            setattr(s, name, getattr(self, name).data_ptr())
        s.reference_positions = self._reference_all.data_ptr()
        s.num_candidates = self.num_candidates_dev.data_ptr()
        s.max_disp2_bits = self.max_disp2.data_ptr()

    def _allocate(self, needed: int, exact: bool = False):
        capacity = int(needed) if exact else edge_capacity(needed, self.headroom, self.edge_multiple)
        self.capacity = capacity
        dev = self.device
        self.candidate_index = torch.zeros(2, capacity, dtype=torch.int32, device=dev)
        self.candidate_unit_shifts = torch.zeros(capacity, 3, dtype=self.float_dtype, device=dev)
        self.edge_index = torch.zeros(2, capacity, dtype=torch.int32, device=dev)
        self.unit_shifts = torch.zeros(capacity, 3, dtype=self.float_dtype, device=dev)
        self.shifts = torch.zeros(capacity, 3, dtype=self.float_dtype, device=dev)
        s = self.struct
        s.capacity = capacity
        for name in ("candidate_index", "candidate_unit_shifts", "edge_index", "unit_shifts", "shifts"):
            setattr(s, name, getattr(self, name).data_ptr())

    def set_capacity(self, capacity: int) -> bool:
        """Reallocate the edge buffers to exactly ``capacity`` (skin.py:281-296). True if they moved."""
        capacity = int(capacity)
        if capacity < max(self.num_candidates, 1):
            raise ValueError(f"neighbour capacity {capacity} is below the {self.num_candidates} candidates of the "
                             "last build")
        if capacity == self.capacity:
            return False
        self._allocate(capacity, exact=True)
        return True

    def _estimate(self, natoms: int) -> int:
        volume = abs(np.linalg.det(self.cell))
        reach = self.cutoff + self.skin
        return int(natoms * (natoms / volume) * 4.0 / 3.0 * math.pi * reach ** 3 * 1.3) + 1024

    # ------------------------------------------------------------------ host-driven build
    def _launch_build(self, positions: torch.Tensor, only_if_flag: bool = False):
        _lib.check(self.lib.fmb_nl_build(ctypes.byref(self.struct), positions.data_ptr(), int(only_if_flag),
                                         _lib.current_stream()), "fmb_nl_build")

    def build(self, positions) -> bool:
        """Rebuild from (N, 3) float64 positions on the device. Returns True if the capacity grew (buffers moved).

        Synchronises once to read the candidate count (the reference's build does too, skin.py:466)."""
        positions = torch.as_tensor(positions, dtype=torch.float64, device=self.device).contiguous()
        if self.variable_cell:
            self._set_cell_constants()                # bins and padding pair of the cell as it is now
            self.build_cell.copy_(self._cell_t.reshape(self.build_cell.shape))
            if self.natoms is not None and int(np.prod(self.nbins)) > self._bins_allocated:
                self._allocate_atoms(self.natoms)     # the cell grew by a bin
        if self.natoms is None:
            self._allocate_atoms(positions.shape[0])
        elif positions.shape[0] != self.natoms:
            raise ValueError("the number of atoms changed")
        grew = False
        if self.capacity == 0:
            self._allocate(self._estimate(self.natoms), exact=True)
            self._launch_build(positions)
            n = int(self.num_candidates_dev.item())
            self._allocate(n)                         # the reference's capacity rule: headroom over the first build
            grew = True
        self.status.zero_()
        self._launch_build(positions)
        n = int(self.num_candidates_dev.item())
        if n > self.capacity:
            self._allocate(n)
            grew = True
            self.status.zero_()
            self._launch_build(positions)
            n = int(self.num_candidates_dev.item())
        self.check_status()
        self.num_candidates = n
        self.rebuilds += 1
        return grew

    build_gpu = build

    def build_in_graph(self, positions: torch.Tensor) -> None:
        """Queue a rebuild that runs only if the device rebuild flag is set (no host synchronisation, fixed
        capacity: an overflow sets the status word instead of growing)."""
        self._launch_build(positions, only_if_flag=True)

    def check_status(self) -> None:
        status = int(self.status.item())
        if status & _lib.STATUS_ROW_OVERFLOW:
            raise _lib.Fmb200Error(f"a receiver has more than {_lib.MAX_ROW} candidate pairs")
        if status & _lib.STATUS_CAND_OVERFLOW:
            raise _lib.Fmb200Error("more candidate pairs than the neighbour capacity")

    # ------------------------------------------------------------------ graph-capturable
    def compact(self, positions: torch.Tensor) -> None:
        """Move pairs within the cutoff to the front (stable order); set ``count`` and the CSR row pointers."""
        _lib.check(self.lib.fmb_nl_compact(ctypes.byref(self.struct), positions.data_ptr(), _lib.current_stream()),
                   "fmb_nl_compact")

    def set_cell(self, cell) -> None:
        """The current cell of a variable-cell run (``skin.py:679-683``): compaction, shifts and edge vectors follow
        it at once, the candidates stay those of the build cell until the deformation-aware test asks for a rebuild.
        Host-side here: the kernels take the cell by value, so a captured graph keeps the cell it was captured with
        and an engine that captures must drop its graphs when the cell changes."""
        cell = torch.as_tensor(cell, dtype=torch.float64).detach().cpu().numpy().reshape(3, 3)
        self.variable_cell = True
        self.cell = cell.copy()
        inverse = np.linalg.inv(self.cell)
        for k in range(9):
            self.struct.cell[k] = float(self.cell.reshape(-1)[k])
            self.struct.inverse[k] = float(inverse.reshape(-1)[k])
        self._cell_t = torch.as_tensor(self.cell, dtype=torch.float64, device=self.device)

    def _needs_rebuild_deformed(self, positions: torch.Tensor, fraction: float) -> torch.Tensor:
        """The deformation-aware test (``skin.py:694-700``): displacements are measured in the build cell's
        coordinates and the allowance shrinks with the smallest singular value of the deformation."""
        build = self.build_cell.reshape(3, 3)
        to_build = torch.linalg.solve(self._cell_t, build)                   # inverse(cell) @ build_cell
        squared = ((positions @ to_build - self.reference_positions) ** 2).sum(dim=1)
        strain = torch.linalg.solve(build, self._cell_t) - torch.eye(3, dtype=torch.float64, device=self.device)
        lower = 1.0 - torch.sqrt((strain * strain).sum())
        allowed = self.cutoff + self.skin - self.cutoff / torch.clamp(lower, min=1e-6)
        flag = (2 * torch.sqrt(squared.max()) > fraction * allowed) | (lower <= 0)
        self.rebuild_flag.copy_(flag.to(torch.int32))
        return self.rebuild_flag

    def needs_rebuild(self, positions: torch.Tensor, fraction: float = 1.0) -> torch.Tensor:
        """Device flag (int32 scalar, nonzero = rebuild): has any atom moved more than fraction * skin / 2?
        After ``set_cell`` the deformation-aware form of the test applies."""
        if self.variable_cell:
            return self._needs_rebuild_deformed(positions, fraction)
        _lib.check(self.lib.fmb_nl_needs_rebuild(ctypes.byref(self.struct), positions.data_ptr(), float(fraction),
                                                 _lib.current_stream()), "fmb_nl_needs_rebuild")
        return self.rebuild_flag

    def edges(self, num_edges: int):
        """Views of the first ``num_edges`` compacted edges: (edge_index, shifts, unit_shifts); no copy."""
        return self.edge_index[:, :num_edges], self.shifts[:num_edges], self.unit_shifts[:num_edges]

    def buffers(self):
        names = ["candidate_index", "candidate_unit_shifts", "edge_index", "unit_shifts", "shifts", "count",
                 "reference_positions", "build_cell", "edge_row_ptr", "cand_row_ptr"]
        return {name: getattr(self, name) for name in names if getattr(self, name, None) is not None}

    def pointer(self):
        return ctypes.byref(self.struct)


__all__ = ["CellListNeighbours", "NeighbourConfig", "edge_bucket", "round_up_edges", "edge_capacity",
           "cell_list_plan", "DEFAULT_SKIN_A"]
