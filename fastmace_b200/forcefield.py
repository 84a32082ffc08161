"""``B200ForceField``: FastMACE's ``ForceField`` protocol (``fastmace/model/forces.py:63-161``) over the C ABI.

Same members, argument meaning and ownership rules as the reference's ``MACEForceField`` (``forces.py:382``) and its
minimal worked example ``TorchLJ`` (``tests/cpu/test_engine.py:40-114``): the force field owns the model, the
neighbour list and every persistent device buffer at a fixed address; ``__call__`` is graph-capturable and returns
views it owns; ``rebuild`` is host-driven and returns True when the edge buffers moved.

Differences that follow from the device design: the kernels read the edge count and CSR row pointers on the device,
so ``use_edges`` only records the padded size the caller asked for (``padding_exact`` stays True: edges past the count
are simply never read), and forces come from analytic backward kernels, not autograd.
"""

from __future__ import annotations

import ctypes
from typing import NamedTuple

import numpy as np
import torch

from . import _lib
from .model import MaceSpec
from .neighbours import CellListNeighbours, NeighbourConfig
from .packing import PackedModel

DEFAULT_CHUNK_EDGES = 1 << 19


class ForceOutput(NamedTuple):
    """``energy`` (1,) float64 eV, ``forces`` (N, 3) float32 eV/Å, ``stress`` (3, 3) float32 eV/Å³ or None
    (ASE sign, no kinetic part): ``fastmace/model/forces.py:35-47``."""
    energy: torch.Tensor
    forces: torch.Tensor
    stress: torch.Tensor | None


class B200ForceField:
    """Energy, forces and (optionally) stress of one configuration through the CUDA library, with the neighbour list
    it owns: the members of the reference's ``ForceField`` protocol (``fastmace/model/forces.py``) under the same names.
    There is no CPU path: construction fails without a CUDA device or without the built library."""

    def __init__(self, spec: MaceSpec, weights, numbers, cell, *, compute_stress: bool = False, device="cuda",
                 neighbours: NeighbourConfig | None = None, chunk_edges: int | None = None,
                 positions=None, packed: PackedModel | None = None, n_owned: int = -1, n_inner: int = -1,
                 halo_exchange: bool = False, atom_capacity: int | None = None, edge_adjoint: bool | None = None):
        if not torch.cuda.is_available():
            raise _lib.Fmb200Error("B200ForceField needs a CUDA device: there is no CPU path")
        self.lib = _lib.load()
        self.spec = spec
        self._device = torch.device(device)
        if self._device.index is None:
            self._device = torch.device("cuda", torch.cuda.current_device())
        self._compute_stress = bool(compute_stress)
        self.numbers = np.asarray(numbers, dtype=np.int64)
        self.natoms = len(self.numbers)
        # ``atom_capacity``: rows every per-atom buffer is allocated for; ``set_atoms`` may then change the atoms (a
        # re-partition of a spatially decomposed run) without moving a buffer as long as they fit
        self.atom_capacity = max(self.natoms, int(atom_capacity or 0))
        self.cell = np.asarray(cell, dtype=np.float64).reshape(3, 3)
        # ``packed``: a model already packed for a superset of these species (the ranks of a decomposed run share
        # one); ``n_owned`` / ``n_inner``: the atoms are ordered owned | inner halo | outer halo (negative = every atom is
        # owned, the default); ``halo_exchange``: the atoms beyond the owned ones belong to other ranks and the call runs in
        # three phases (``phase``) between which the caller moves the halo rows of ``x`` and ``d_x``
        self.packed = packed if packed is not None else \
            PackedModel(spec, weights, sorted(set(int(z) for z in self.numbers)), self._device)
        self.n_owned, self.n_inner = int(n_owned), int(n_inner)
        self.halo_exchange = bool(halo_exchange)
        if self.halo_exchange and self.n_inner != self.n_owned:
            raise ValueError("halo-exchange mode evaluates both interactions for the owned atoms: n_inner == n_owned")
        self.species = torch.zeros(self.atom_capacity, dtype=torch.int32, device=self._device)
        self.symcon_groups = torch.full((self.atom_capacity // 4 + len(self.packed.species_z) + 1, 4), -1,
                                        dtype=torch.int32, device=self._device)
        self.n_symcon_groups = 0
        self._upload_atoms()
        self.neighbours = CellListNeighbours(self.cell, spec.r_cut, self._device, torch.float32, neighbours,
                                             atom_capacity=self.atom_capacity)
        # ``chunk_edges``: None = the whole edge list as one chunk (per-edge radial weights kept between the forward pass
        # and the adjoint, streamed kernels) whenever its buffers fit in the free device memory, else chunks of
        # DEFAULT_CHUNK_EDGES with the weights recomputed per chunk; a number sets the chunk size by hand
        self.chunk_edges = None if chunk_edges is None else int(chunk_edges)
        # ``edge_adjoint``: None = the per-edge hand-over adjoint whenever its buffers fit in the free device memory,
        # else the mirror evaluation; False = the mirror evaluation regardless (the path of lists too large for the
        # buffers, selectable so that tests reach it on small cells); True = refuse to fall back
        self.edge_adjoint = edge_adjoint
        self.num_edges = 0
        self.calls = 0
        self.data = {}
        self.work = None
        self._outputs()
        if positions is not None:
            x = torch.as_tensor(positions, dtype=torch.float64, device=self._device)
            self.rebuild(x)
            self.compact(x)
            self.use_edges(int(self.edge_count))

    # ------------------------------------------------------------------ protocol properties
    @property
    def device(self) -> torch.device:
        return self._device

    dtype = torch.float32
    padding_exact = True
    compile_mode = "none"

    @property
    def compute_stress(self) -> bool:
        return self._compute_stress

    @property
    def forces(self) -> torch.Tensor:
        return self._forces_all[:self.natoms]

    @property
    def edge_count(self) -> torch.Tensor:
        return self.neighbours.count

    @property
    def edge_capacity(self) -> int:
        return self.neighbours.capacity

    @staticmethod
    def _species_groups(species: np.ndarray, size: int) -> torch.Tensor:
        """[n_groups, size] int32 atom indices, same species within a group, -1 in unused slots (in index order, so that
        the atoms below a row limit fill the first groups of their species)."""
        rows = []
        for z in np.unique(species):
            atoms = np.nonzero(species == z)[0].astype(np.int32)
            padded = np.full(-(-len(atoms) // size) * size, -1, dtype=np.int32)
            padded[:len(atoms)] = atoms
            rows.append(padded.reshape(-1, size))
        groups = np.concatenate(rows) if rows else np.zeros((0, size), dtype=np.int32)
        return torch.from_numpy(np.ascontiguousarray(groups))

    def _upload_atoms(self) -> None:
        """Species indices and contraction groups of the current atoms into their (capacity-sized) device buffers."""
        species = self.packed.species_index(self.numbers)
        self.species[:self.natoms].copy_(species)
        # only the rows the interactions are evaluated for need a group
        rows = self.n_inner if self.n_inner >= 0 else self.natoms
        groups = self._species_groups(species[:rows].cpu().numpy(), 4)
        self.n_symcon_groups = int(groups.shape[0])
        self.symcon_groups[:self.n_symcon_groups].copy_(groups)

    def set_atoms(self, numbers, n_owned: int = -1, n_inner: int = -1) -> bool:
        """Replace the atoms (a re-partition of a spatially decomposed run): same model, same box, another set of
        atomic numbers and owned / halo counts. The per-atom buffers stay where they are while the new atoms fit the
        capacity; returns True if they had to be reallocated (every buffer moved). The neighbour list must be rebuilt
        (``rebuild``) before the next call."""
        self.numbers = np.asarray(numbers, dtype=np.int64)
        self.natoms = len(self.numbers)
        self.n_owned, self.n_inner = int(n_owned), int(n_inner)
        if self.halo_exchange and self.n_inner != self.n_owned:
            raise ValueError("halo-exchange mode: n_inner == n_owned")
        moved = False
        if self.natoms > self.atom_capacity:
            self.atom_capacity = int(self.natoms * 1.1) + 16
            self.species = torch.zeros(self.atom_capacity, dtype=torch.int32, device=self._device)
            self.symcon_groups = torch.full((self.atom_capacity // 4 + len(self.packed.species_z) + 1, 4), -1,
                                            dtype=torch.int32, device=self._device)
            self.neighbours.set_atom_capacity(self.atom_capacity)
            self._outputs()
            self.work, self.buf = None, None
            moved = True
        self._upload_atoms()
        self.neighbours.set_natoms(self.natoms)
        if self.work is not None:
            self._fill_counts(self.work)
        return moved

    def _fill_counts(self, w) -> None:
        w.n_atoms = self.natoms
        w.n_energy_atoms, w.n_inner_atoms = self.n_owned, self.n_inner
        w.halo_exchange = int(self.halo_exchange)
        w.species = self.species.data_ptr()
        w.symcon_groups, w.n_symcon_groups = self.symcon_groups.data_ptr(), self.n_symcon_groups

    # ------------------------------------------------------------------ buffers
    def _outputs(self):
        dev = self._device
        self.energy = torch.zeros(1, dtype=torch.float64, device=dev)
        self._forces_all = torch.zeros(self.atom_capacity, 3, dtype=torch.float32, device=dev)
        self.stress = torch.zeros(3, 3, dtype=torch.float32, device=dev)
        self.status = torch.zeros((), dtype=torch.int32, device=dev)

    def _allocate_work(self):
        spec, n, cap, dev = self.spec, self.atom_capacity, self.neighbours.capacity, self._device
        if getattr(self, "buf", None) is not None:
            # the edge capacity grew: give the old buffers back to the device before the new ones are sized, so that the
            # two sets never exist side by side (the per-edge buffers of a large brick are tens of GB each)
            self.work, self.buf = None, None
            torch.cuda.empty_cache()
        c = spec.channels
        max_paths = max(len(spec.paths(t)) for t in range(spec.num_interactions))
        hid = (spec.hidden_lmax + 1) ** 2
        pair_capacity = 0
        if self.chunk_edges is not None:
            chunk = min(self.chunk_edges, cap)
        elif cap <= DEFAULT_CHUNK_EDGES:
            chunk = cap
        elif getattr(self, "_chunked_only", False):
            chunk = DEFAULT_CHUNK_EDGES
        else:
            # what this function allocates per edge with the whole list as one chunk: vector, harmonics, hidden
            # features, hand-over buffers with the pair map -- and the weights with their d/dr, one row per edge or,
            # where the kernels that read one row per pair of opposite edges apply, a little over half a row
            free, _ = torch.cuda.mem_get_info(dev)
            free += torch.cuda.memory_reserved(dev) - torch.cuda.memory_allocated(dev)
            others = 16 + 64 + spec.num_interactions * 2 * 64 * 4 + hid * c * 4 + 28
            row = 2 * max_paths * c * 4
            layers = self.packed.struct.layer
            pair_rows = (self.edge_adjoint is not False and spec.num_interactions == 2 and spec.l_in_max(1) == 1
                         and bool(layers[1].rad_img) and bool(layers[0].first[0]))
            pairs = cap // 2 + cap // 16
            if pair_rows and cap * others + pairs * row <= 0.85 * free:
                chunk, pair_capacity = cap, pairs
            elif cap * (others + row) <= 0.85 * free:
                chunk = cap
            else:
                chunk = DEFAULT_CHUNK_EDGES
        max_mid = max(self.packed.struct.layer[t].mid_dim for t in range(spec.num_interactions))
        # the reassociated first layer keeps its per-species outer-product sums [16][n_species][64] in `mid` / `d_mid`
        mid_floats = max(max_mid * c, 16 * len(self.packed.species_z) * 64)
        f32 = dict(dtype=torch.float32, device=dev)
        buf = {
            "edge_vec": torch.zeros(cap, 4, **f32),
            "edge_sh": torch.zeros(cap, 16, **f32),
            "edge_hidden": torch.zeros(spec.num_interactions, 2, cap, 64, **f32),
            "tp_w": torch.zeros(2 * (pair_capacity or chunk), max_paths * c, **f32),
            "x": torch.zeros(n, hid, c, **f32),
            "mid": torch.zeros(n, mid_floats, **f32),
            "msg": torch.zeros(spec.num_interactions, n, 16, c, **f32),
            "basis": torch.zeros(n, hid, c, **f32),
            "h": torch.zeros(n * (hid + 1), c, **f32),
            "d_h": torch.zeros(n, hid, c, **f32),
            "d_basis": torch.zeros(n, hid, c, **f32),
            "d_msg": torch.zeros(n, 16, c, **f32),
            "d_mid": torch.zeros(n, mid_floats, **f32),
            "d_x": torch.zeros(n, hid, c, **f32),
            "node_energy": torch.zeros(n, **f32),
            "atom_virial": torch.zeros(n, 6, **f32),
            "force_acc": torch.zeros(n, 3, **f32),
            "partial": torch.zeros(1024 * 8, dtype=torch.float64, device=dev),
        }
        # per-edge hand-over buffers of the adjoint (2 KB per edge for the medium model): when they fit in the memory
        # that is free now with a tenth of the device kept back, else the mirror-evaluation kernels run
        free, total = torch.cuda.mem_get_info(dev)
        free += torch.cuda.memory_reserved(dev) - torch.cuda.memory_allocated(dev)   # blocks torch holds but does not use
        need = cap * (hid * c * 4 + 20)
        self.edge_local = need <= free - total // 10 and self.edge_adjoint is not False
        if (self.halo_exchange or self.edge_adjoint) and not self.edge_local:
            raise _lib.Fmb200Error(f"halo-exchange mode needs {need / 2 ** 30:.1f} GiB for the per-edge hand-over "
                                   f"buffers, {max(0, free - total // 10) / 2 ** 30:.1f} GiB are free: use more ranks")
        if self.edge_local:
            try:
                buf["mirror"] = torch.zeros(cap, dtype=torch.int32, device=dev)
                buf["edge_q"] = torch.zeros(cap, 4, **f32)
                buf["edge_dx"] = torch.zeros(cap, hid, c, **f32)
                buf["edge_slot"] = torch.zeros(cap, dtype=torch.int32, device=dev)
                buf["canon_list"] = torch.zeros(cap, dtype=torch.int32, device=dev)
                buf["canon_count"] = torch.zeros(1, dtype=torch.int64, device=dev)
            except torch.OutOfMemoryError:
                # the free memory was there but not in one piece: run the mirror-evaluation adjoint instead
                for name in ("mirror", "edge_q", "edge_dx", "edge_slot", "canon_list", "canon_count"):
                    buf.pop(name, None)
                torch.cuda.empty_cache()
                self.edge_local = False
                if pair_capacity:
                    # the weight buffer was sized for the pair map that now does not exist: size everything again,
                    # in chunks
                    del buf
                    torch.cuda.empty_cache()
                    self._chunked_only = True
                    return self._allocate_work()
        self.buf = buf
        w = _lib.WorkStruct()
        w.edge_capacity, w.chunk_edges, w.compute_stress = cap, chunk, int(self._compute_stress)
        w.pair_capacity = pair_capacity
        for name, tensor in buf.items():
            setattr(w, name, tensor.data_ptr())
        w.energy, w.forces, w.stress = self.energy.data_ptr(), self._forces_all.data_ptr(), self.stress.data_ptr()
        w.status = self.status.data_ptr()
        self._fill_counts(w)
        self.work = w

    # ------------------------------------------------------------------ protocol methods
    def rebuild(self, positions: torch.Tensor) -> bool:
        """Rebuild the candidate pairs (host-driven, synchronises). True if the edge capacity grew."""
        grew = self.neighbours.build(positions)
        if grew or self.work is None:
            self._allocate_work()
        return grew

    def compact(self, positions: torch.Tensor) -> None:
        self.neighbours.compact(positions)

    def needs_rebuild(self, positions: torch.Tensor, fraction: float = 1.0) -> torch.Tensor:
        return self.neighbours.needs_rebuild(positions, fraction) != 0

    def use_edges(self, num_edges: int) -> None:
        self.num_edges = int(num_edges)
        self.data["edge_index"] = self.neighbours.edge_index[:, :self.num_edges]

    def set_cell(self, cell: torch.Tensor) -> None:
        """The current float64 cell of a variable-cell run (``fastmace/model/forces.py:1351-1356``): the neighbour
        list's shifts, the edge vectors and the volume the stress is divided by follow it from the next call on; the
        candidates are rebuilt when the deformation-aware test fires (``needs_rebuild``). Needs ``compute_stress``
        like the reference's. Host-side (the kernels take the cell by value): not for use inside a captured step."""
        if not self._compute_stress:
            raise RuntimeError("set_cell needs a force field built with compute_stress=True")
        self.neighbours.set_cell(cell)
        self.cell = self.neighbours.cell.copy()

    reset_cell = set_cell

    def __call__(self, positions: torch.Tensor) -> ForceOutput:
        """Energy, forces (and stress) at float64 ``positions`` (N, 3) on the compacted edges. Graph-capturable."""
        if self.work is None:
            raise _lib.Fmb200Error("call rebuild() and compact() before the first force call")
        if positions.dtype != torch.float64 or not positions.is_cuda:
            raise ValueError("positions must be a float64 CUDA tensor")
        self.calls += 1
        _lib.check(self.lib.fmb_forces(self.packed.pointer(), self.neighbours.pointer(), ctypes.byref(self.work),
                                       positions.data_ptr(), _lib.current_stream()), "fmb_forces")
        return ForceOutput(self.energy, self.forces, self.stress if self._compute_stress else None)

    def phase(self, index: int, positions: torch.Tensor | None = None) -> None:
        """One of the three phases of a halo-exchange call (``fmb_forces_phase``): 0 reads ``positions`` and ends
        with ``x`` of the owned atoms, 1 ends with ``d_x`` of every local atom, 2 ends with the outputs."""
        if self.work is None:
            raise _lib.Fmb200Error("call rebuild() and compact() before the first force call")
        if index == 0:
            self.calls += 1
        _lib.check(self.lib.fmb_forces_phase(self.packed.pointer(), self.neighbours.pointer(), ctypes.byref(self.work),
                                             positions.data_ptr() if positions is not None else None, int(index),
                                             _lib.current_stream()), "fmb_forces_phase")

    def evaluate(self, atoms, stress: bool = False):
        """One-off evaluation (``ForceField.evaluate``): rebuilds the list, synchronises, returns host values:
        (energy float eV, forces (N, 3) float64 ndarray, stress (3, 3) ndarray or None)."""
        if stress and not self._compute_stress:
            raise ValueError("built without compute_stress")
        x = torch.as_tensor(np.asarray(atoms.get_positions(), dtype=np.float64), device=self._device)
        self.rebuild(x)
        self.compact(x)
        self.use_edges(int(self.edge_count))
        out = self(x)
        torch.cuda.synchronize(self._device)
        self.check_status()
        return (float(out.energy.item()), out.forces.double().cpu().numpy(),
                out.stress.double().cpu().numpy() if stress else None)

    def check_status(self) -> None:
        self.neighbours.check_status()
        status = int(self.status.item())
        if status & _lib.STATUS_NONFINITE:
            raise _lib.Fmb200Error("the force call produced a non-finite energy")
        if status & _lib.STATUS_NO_MIRROR:
            raise _lib.Fmb200Error("an edge has no opposite edge: the neighbour list is not full")
        if status & _lib.STATUS_TENSOR_TIMEOUT:
            raise _lib.Fmb200Error("a tensor-core kernel gave up waiting (FMB_STATUS_TENSOR_TIMEOUT)")
        if status & _lib.STATUS_PAIR_OVERFLOW:
            raise _lib.Fmb200Error("more pairs of opposite edges than the radial-weight buffer has rows")

    def per_atom_energies(self):
        return self.buf["node_energy"][:self.natoms].double().cpu().numpy()

    def buffers(self):
        """Persistent device buffers under the names the reference's registry has policies for
        (``fastmace/engine/registry.py:91-139``): everything a rebuild makes as ``neighbours.*`` (the status words
        included: they are sticky until a rebuild clears them; the cell is ``neighbours.build_cell``). The work buffers
        of a force call are written before they are read in every call and carry nothing across steps."""
        out = {f"neighbours.{name}": value for name, value in self.neighbours.buffers().items()}
        out["neighbours.status"] = self.neighbours.status
        out["neighbours.force_status"] = self.status
        return out

    def info(self):
        return {"streaming_interactions": self.spec.num_interactions, "sort_receivers": True,
                "neighbour_rebuilds": self.neighbours.rebuilds, "edge_capacity": self.neighbours.capacity,
                "engine": "fmb200", "force_calls": self.calls}


__all__ = ["B200ForceField", "ForceOutput", "DEFAULT_CHUNK_EDGES"]
