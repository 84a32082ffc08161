"""ctypes binding of ``libfmb200.so`` (the C ABI declared in ``include/fmb200.h``).

The library is the only compute path: there is no PyTorch or CPU fallback. ``load()`` raises ``Fmb200Error`` with the
build command when the shared object is missing, and every wrapper raises when a call returns a non-zero status.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_float, c_int, c_int32, c_int64, c_uint32, c_uint64, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libfmb200.so")

MAX_ROW = 1024
MAX_LAYERS = 2
MAX_SPECIES = 8

STATUS_CAND_OVERFLOW = 1
STATUS_ROW_OVERFLOW = 2
STATUS_BIN_OVERFLOW = 4
STATUS_NONFINITE = 8
STATUS_TENSOR_TIMEOUT = 16
STATUS_NO_MIRROR = 32
STATUS_PAIR_OVERFLOW = 64

EXPORTS = ("fmb_version", "fmb_last_error", "fmb_sizeof", "fmb_launch_count", "fmb_nl_build", "fmb_nl_compact", "fmb_nl_compact_static",
           "fmb_nl_needs_rebuild",
           "fmb_forces", "fmb_forces_phase", "fmb_halo_gather_rows", "fmb_halo_add_rows", "fmb_halo_local_positions",
           "fmb_halo_owned_forces", "fmb_edge_features", "fmb_harmonics_probe", "fmb_forward", "fmb_backward", "fmb_gemm", "fmb_langevin_first_half",
           "fmb_langevin_second_half", "fmb_langevin_device_noise", "fmb_langevin_device_noise_ids",
           "fmb_langevin_noise_sums", "fmb_langevin_first_half_global", "fmb_commit_forces", "fmb_profile_enable", "fmb_profile_read")


class Fmb200Error(RuntimeError):
    pass


class NlStruct(ctypes.Structure):
    _fields_ = [
        ("n_atoms", c_int32), ("capacity", c_int32), ("cutoff", c_double), ("skin", c_double),
        ("cell", c_double * 9), ("inverse", c_double * 9), ("nbins", c_int32 * 3), ("reach_bins", c_int32 * 3),
        ("pad_unit_shift", c_float * 3), ("max_bin_atoms", c_int32),
        ("wrapped", c_void_p), ("offsets", c_void_p), ("atom_bin", c_void_p), ("bin_count", c_void_p),
        ("bin_start", c_void_p), ("bin_fill", c_void_p), ("bin_atoms", c_void_p), ("cand_row_count", c_void_p),
        ("cand_row_ptr", c_void_p), ("candidate_index", c_void_p), ("candidate_unit_shifts", c_void_p),
        ("edge_row_count", c_void_p), ("edge_row_ptr", c_void_p), ("edge_index", c_void_p), ("unit_shifts", c_void_p),
        ("shifts", c_void_p), ("count", c_void_p), ("num_candidates", c_void_p), ("reference_positions", c_void_p),
        ("build_cell", c_void_p), ("scan_scratch", c_void_p), ("max_disp2_bits", c_void_p),
        ("rebuild_flag", c_void_p), ("status", c_void_p),
    ]


class LayerStruct(ctypes.Structure):
    _fields_ = [
        ("l_in_max", c_int32), ("l_out_max", c_int32), ("n_paths", c_int32), ("mid_dim", c_int32),
        ("n_sc_terms", c_int32), ("skip_lmax", c_int32), ("is_last", c_int32), ("pad_", c_int32),
        ("rad_w", c_void_p * 4), ("x_species", c_void_p), ("sc_species", c_void_p), ("w_up", c_void_p),
        ("w_up_t", c_void_p), ("w_skip", c_void_p), ("w_skip_t", c_void_p), ("w_lin", c_void_p),
        ("w_lin_t", c_void_p), ("w_prod", c_void_p), ("w_prod_t", c_void_p), ("sc_terms", c_void_p),
        ("sc_coef", c_void_p), ("w_readout", c_void_p), ("tc", c_void_p * 9), ("first", c_void_p * 4),
        ("rad_img", c_void_p), ("tc_img", c_void_p * 9), ("first_img", c_void_p * 2),
        ("mlp_img", c_void_p),
    ]


class ModelStruct(ctypes.Structure):
    _fields_ = [
        ("n_species", c_int32), ("channels", c_int32), ("hidden_lmax", c_int32), ("n_layers", c_int32),
        ("n_bessel", c_int32), ("cutoff_p", c_int32), ("radial_width", c_int32), ("mlp_hidden", c_int32),
        ("r_cut", c_float), ("scale", c_float), ("shift", c_float), ("silu_norm", c_float),
        ("e0", c_double * MAX_SPECIES), ("layer", LayerStruct * MAX_LAYERS),
    ]


class WorkStruct(ctypes.Structure):
    _fields_ = [
        ("n_atoms", c_int32), ("edge_capacity", c_int32), ("chunk_edges", c_int32), ("compute_stress", c_int32),
        ("species", c_void_p), ("edge_vec", c_void_p), ("edge_sh", c_void_p), ("edge_hidden", c_void_p),
        ("tp_w", c_void_p), ("x", c_void_p), ("mid", c_void_p), ("msg", c_void_p), ("basis", c_void_p),
        ("h", c_void_p), ("d_h", c_void_p), ("d_basis", c_void_p), ("d_msg", c_void_p), ("d_mid", c_void_p),
        ("d_x", c_void_p), ("node_energy", c_void_p), ("atom_virial", c_void_p), ("force_acc", c_void_p),
        ("partial", c_void_p), ("energy", c_void_p), ("forces", c_void_p), ("stress", c_void_p), ("status", c_void_p),
        ("n_energy_atoms", c_int32), ("n_inner_atoms", c_int32),
        ("mirror", c_void_p), ("edge_q", c_void_p), ("edge_dx", c_void_p),
        ("edge_slot", c_void_p), ("canon_list", c_void_p), ("canon_count", c_void_p),
        ("symcon_groups", c_void_p), ("n_symcon_groups", c_int32), ("halo_exchange", c_int32),
        ("pair_capacity", c_int32), ("pad_", c_int32),
    ]


class LangevinStruct(ctypes.Structure):
    _fields_ = [
        ("n_atoms", c_int32), ("fix_com", c_int32), ("dt", c_double), ("c1", c_double), ("c2", c_double),
        ("positions", c_void_p), ("velocities", c_void_p), ("forces", c_void_p), ("masses", c_void_p),
        ("c3_unit", c_void_p), ("c4_unit", c_void_p), ("c5_unit", c_void_p), ("sqrt_kT", c_void_p),
        ("noise", c_void_p), ("noise_cursor", c_void_p), ("x_old", c_void_p), ("rnd_pos", c_void_p),
        ("rnd_vel", c_void_p), ("partial", c_void_p), ("noise_cursor_rw", c_void_p),
    ]


STAGES = ("edge_features", "radial_gemm", "tp_forward_l0", "tp_forward_l1", "node_linears", "symcon_forward",
          "symcon_backward", "tp_backward_l1", "tp_backward_l0", "readout_reduce")

_LIB = None


def load() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(LIB_PATH):
        raise Fmb200Error(f"{LIB_PATH} is missing: build it with `python -m fastmace_b200.build` (needs nvcc, sm_100a). "
                          "There is no fallback path.")
    lib = ctypes.CDLL(LIB_PATH)
    lib.fmb_last_error.restype = c_char_p
    lib.fmb_sizeof.argtypes = [c_int]
    lib.fmb_launch_count.restype = ctypes.c_longlong
    for which, struct in enumerate((NlStruct, ModelStruct, WorkStruct, LangevinStruct)):
        if lib.fmb_sizeof(which) != ctypes.sizeof(struct):
            raise Fmb200Error(f"struct {struct.__name__} is {ctypes.sizeof(struct)} bytes here, "
                              f"{lib.fmb_sizeof(which)} in the library: rebuild the library")
    P = c_void_p
    lib.fmb_nl_build.argtypes = [POINTER(NlStruct), P, c_int, P]
    lib.fmb_nl_compact.argtypes = [POINTER(NlStruct), P, P]
    lib.fmb_nl_compact_static.argtypes = [POINTER(NlStruct), P, P]
    lib.fmb_nl_needs_rebuild.argtypes = [POINTER(NlStruct), P, c_double, P]
    lib.fmb_forces.argtypes = [POINTER(ModelStruct), POINTER(NlStruct), POINTER(WorkStruct), P, P]
    lib.fmb_edge_features.argtypes = [POINTER(ModelStruct), POINTER(NlStruct), POINTER(WorkStruct), P, P]
    lib.fmb_forces_phase.argtypes = [POINTER(ModelStruct), POINTER(NlStruct), POINTER(WorkStruct), P, c_int, P]
    lib.fmb_halo_gather_rows.argtypes = [P, P, P, c_int, c_int, P]
    lib.fmb_halo_add_rows.argtypes = [P, P, P, P, P, c_int, c_int, P]
    lib.fmb_halo_local_positions.argtypes = [P, c_int, P, P, c_int, POINTER(c_double * 3), P, P]
    lib.fmb_halo_owned_forces.argtypes = [P, P, P, P, c_int, P, P]
    lib.fmb_harmonics_probe.argtypes = [P, P, P, P, c_int, P]
    lib.fmb_forward.argtypes = [POINTER(ModelStruct), POINTER(NlStruct), POINTER(WorkStruct), P]
    lib.fmb_backward.argtypes = [POINTER(ModelStruct), POINTER(NlStruct), POINTER(WorkStruct), P]
    lib.fmb_gemm.argtypes = [P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, P, P]
    lib.fmb_langevin_first_half.argtypes = [POINTER(LangevinStruct), P]
    lib.fmb_langevin_second_half.argtypes = [POINTER(LangevinStruct), P]
    lib.fmb_langevin_device_noise.argtypes = [P, c_int, ctypes.c_ulonglong, P, P]
    lib.fmb_langevin_device_noise_ids.argtypes = [P, c_int, P, ctypes.c_ulonglong, P, P]
    lib.fmb_langevin_noise_sums.argtypes = [POINTER(LangevinStruct), P, P]
    lib.fmb_langevin_first_half_global.argtypes = [POINTER(LangevinStruct), P, ctypes.c_longlong, P]
    lib.fmb_commit_forces.argtypes = [POINTER(WorkStruct), P, P, P, P]
    lib.fmb_profile_enable.argtypes = [c_int]
    lib.fmb_profile_read.argtypes = [POINTER(c_float), POINTER(c_int), c_int]
    _LIB = lib
    return lib


def check(status: int, what: str) -> None:
    if status != 0:
        text = load().fmb_last_error()
        raise Fmb200Error(f"{what} failed with status {status}: {text.decode() if text else ''}")


def profile_read() -> dict:
    """{stage: (milliseconds, spans)} accumulated since the last read (needs fmb_profile_enable(1))."""
    lib = load()
    ms = (c_float * len(STAGES))()
    spans = (c_int * len(STAGES))()
    n = lib.fmb_profile_read(ms, spans, len(STAGES))
    if n != len(STAGES):
        raise Fmb200Error(f"fmb_profile_read returned {n}")
    return {name: (float(ms[k]), int(spans[k])) for k, name in enumerate(STAGES)}


def current_stream() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream


__all__ = ["load", "check", "current_stream", "Fmb200Error", "NlStruct", "LayerStruct", "ModelStruct", "WorkStruct",
           "LangevinStruct", "EXPORTS", "LIB_PATH", "MAX_ROW", "MAX_SPECIES"]
