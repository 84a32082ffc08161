"""TEST INFRASTRUCTURE ONLY -- SO(3) tables of the CPU oracle, derived without the product's tables.

The CUDA path takes its Wigner tensors from ``fastmace_b200/so3.py`` (null space of ``D x D x D - 1`` found by SVD).
This module computes the same objects another way, so that a wrong table on either side shows up as a disagreement
instead of cancelling in every GPU-versus-oracle comparison:

* real spherical harmonics l <= 3: the polynomials, constants and component order of the reference's own kernel
  (``fastmace/kernels/triton/edge_sh.py:22-78``), pinned by ``tests/golden/edge_sh.npz``;
* Wigner-3j symbols in the complex basis: Racah's closed form, exact rational arithmetic under the square root;
* complex -> real change of basis: for l <= 3 fitted to those polynomials against SciPy's complex harmonics
  (``scipy.special.sph_harm_y``); for l > 3 (intermediate irreps of the symmetric contraction only) the textbook
  real harmonics ``sqrt(2) Re / Im`` with the Condon-Shortley phase removed;
* real Wigner tensor = complex symbol contracted with the three basis changes, unit Frobenius norm, first non-zero
  entry positive (a global sign per tensor is a reparametrisation w -> -w of a randomly initialised model);
* tensor-product paths and the coupling trees of the symmetric contraction in the order mace-torch 0.3.16 builds
  them (``tp_out_irreps_with_instructions``; ``U_matrix_real``), restated from the published algorithm: the
  third-party packages are not vendored in the reference tree (call sites:
  ``fastmace/rewrites/generic/modules.py:485``, ``fastmace/kernels/oeq_streaming/schedule.py:318-339``,
  ``fastmace/kernels/cuda/sc_generated.py:1-20``).

PARITY UNPINNED against e3nn 0.4.4 for everything except the l <= 3 harmonics: e3nn cannot be imported here.
Nothing under ``fastmace_b200`` is imported; only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU legs
may import this module.
"""

from __future__ import annotations

import functools
import math
from fractions import Fraction

import numpy as np
from scipy import integrate, special

L_SH = 3
N_SH = (L_SH + 1) ** 2

ROOT3, ROOT5, ROOT7 = math.sqrt(3.0), math.sqrt(5.0), math.sqrt(7.0)
ROOT_5_6 = math.sqrt(5.0 / 6.0)
ROOT_3_8 = math.sqrt(3.0 / 8.0)


def harmonics_of_unit(x, y, z):
    """The 16 polynomials of ``edge_sh.py:40-78`` on unit-vector components (works for NumPy arrays and torch
    tensors alike); returns them as a list in component order."""
    xz = ROOT3 * x * z
    xy = ROOT3 * x * y
    yy = y * y
    rr = x * x + z * z
    d22 = yy - 0.5 * rr
    yz = ROOT3 * y * z
    zx = ROOT3 / 2.0 * (z * z - x * x)
    f0 = ROOT_5_6 * (xz * z + zx * x)
    f1 = ROOT5 * xz * y
    f2 = ROOT_3_8 * (4.0 * yy - rr) * x
    f3 = 0.5 * y * (2.0 * yy - 3.0 * rr)
    f4 = ROOT_3_8 * z * (4.0 * yy - rr)
    f5 = ROOT5 * zx * y
    f6 = ROOT_5_6 * (zx * z - xz * x)
    one = x * 0.0 + 1.0
    return [one, ROOT3 * x, ROOT3 * y, ROOT3 * z, ROOT5 * xz, ROOT5 * xy, ROOT5 * d22, ROOT5 * yz, ROOT5 * zx,
            ROOT7 * f0, ROOT7 * f1, ROOT7 * f2, ROOT7 * f3, ROOT7 * f4, ROOT7 * f5, ROOT7 * f6]


def real_sh(vectors: np.ndarray) -> np.ndarray:
    """[n, 3] -> [n, 16]: component-normalised harmonics of ``v / max(|v|, 1e-12)`` (``edge_sh.py:30-37``)."""
    v = np.asarray(vectors, dtype=np.float64)
    u = v / np.maximum(np.sqrt((v * v).sum(axis=1, keepdims=True)), 1e-12)
    return np.stack(harmonics_of_unit(u[:, 0], u[:, 1], u[:, 2]), axis=1)


# ------------------------------------------------------------------------------------------ complex side


def _complex_sh(l: int, unit: np.ndarray) -> np.ndarray:
    """[n, 2l+1] complex harmonics Y_l^m, m = -l..l, times sqrt(4 pi) (component normalisation)."""
    theta = np.arccos(np.clip(unit[:, 2], -1.0, 1.0))
    phi = np.arctan2(unit[:, 1], unit[:, 0])
    cols = [special.sph_harm_y(l, m, theta, phi) for m in range(-l, l + 1)]
    return math.sqrt(4.0 * math.pi) * np.stack(cols, axis=1)


def _sample_points(count: int = 64) -> np.ndarray:
    rng = np.random.default_rng(991)
    p = rng.normal(size=(count, 3))
    return p / np.linalg.norm(p, axis=1, keepdims=True)


def _textbook_basis(l: int) -> np.ndarray:
    """Q [2l+1, 2l+1] complex with R_a = sum_m Q[a, m] Y_l^m for the real harmonics
    sqrt(2) k P_l^|m|(z) sin(|m| phi) (a < l), k P_l^0 (a = l), sqrt(2) k P_l^m(z) cos(m phi) (a > l), Legendre functions
    without the Condon-Shortley phase."""
    q = np.zeros((2 * l + 1, 2 * l + 1), dtype=np.complex128)
    q[l, l] = 1.0
    for m in range(1, l + 1):
        sign = (-1.0) ** m
        # Y_l^m = (-1)^m k P e^{i m phi}, Y_l^{-m} = k P e^{-i m phi}
        q[l + m, l + m] = sign / math.sqrt(2.0)
        q[l + m, l - m] = 1.0 / math.sqrt(2.0)
        q[l - m, l + m] = -1j * sign / math.sqrt(2.0)
        q[l - m, l - m] = 1j / math.sqrt(2.0)
    return q


@functools.lru_cache(maxsize=None)
def real_basis(l: int) -> np.ndarray:
    """Q with ``R_l(u) = Q Y_l(u)`` for this oracle's real basis of irrep l (unitary)."""
    if l > L_SH:
        return _textbook_basis(l)
    pts = _sample_points()
    target = real_sh(pts)[:, l * l:(l + 1) ** 2]
    q_t, residual, *_ = np.linalg.lstsq(_complex_sh(l, pts), target.astype(np.complex128), rcond=None)
    q = q_t.T
    if not np.allclose(q @ q.conj().T, np.eye(2 * l + 1), atol=1e-10):
        raise RuntimeError(f"real basis of l = {l} is not unitary")
    return q


def real_sh_l(l: int, vectors: np.ndarray) -> np.ndarray:
    """[n, 2l+1] harmonics of degree l in this oracle's real basis (any l)."""
    v = np.asarray(vectors, dtype=np.float64)
    u = v / np.linalg.norm(v, axis=1, keepdims=True)
    if l <= L_SH:
        return real_sh(u)[:, l * l:(l + 1) ** 2]
    values = _complex_sh(l, u) @ real_basis(l).T
    return values.real


def _factorial_ratio_sqrt(num, den) -> float:
    value = Fraction(1)
    for n in num:
        value *= math.factorial(n)
    for n in den:
        value /= math.factorial(n)
    return math.sqrt(value)


def racah_3j(j1: int, m1: int, j2: int, m2: int, j3: int, m3: int) -> float:
    """Wigner 3j symbol (j1 j2 j3; m1 m2 m3) for integer arguments, Racah's formula."""
    if m1 + m2 + m3 != 0 or not abs(j1 - j2) <= j3 <= j1 + j2:
        return 0.0
    if abs(m1) > j1 or abs(m2) > j2 or abs(m3) > j3:
        return 0.0
    pref = _factorial_ratio_sqrt(
        [j1 + j2 - j3, j1 - j2 + j3, -j1 + j2 + j3, j1 + m1, j1 - m1, j2 + m2, j2 - m2, j3 + m3, j3 - m3],
        [j1 + j2 + j3 + 1])
    total = Fraction(0)
    for k in range(0, j1 + j2 + j3 + 1):
        terms = [k, j1 + j2 - j3 - k, j1 - m1 - k, j2 + m2 - k, j3 - j2 + m1 + k, j3 - j1 - m2 + k]
        if min(terms) < 0:
            continue
        den = 1
        for t in terms:
            den *= math.factorial(t)
        total += Fraction((-1) ** k, den)
    return (-1.0) ** (j1 - j2 - m3) * pref * float(total)


@functools.lru_cache(maxsize=None)
def wigner_3j(l1: int, l2: int, l3: int) -> np.ndarray:
    """Real invariant tensor of l1 x l2 x l3 in this oracle's bases, [2l1+1, 2l2+1, 2l3+1], unit Frobenius norm,
    first entry (row-major) above 1e-9 in magnitude positive."""
    if not abs(l1 - l2) <= l3 <= l1 + l2:
        raise ValueError(f"no coupling {l1} x {l2} -> {l3}")
    symbol = np.zeros((2 * l1 + 1, 2 * l2 + 1, 2 * l3 + 1))
    for m1 in range(-l1, l1 + 1):
        for m2 in range(-l2, l2 + 1):
            m3 = -m1 - m2
            if abs(m3) <= l3:
                symbol[l1 + m1, l2 + m2, l3 + m3] = racah_3j(l1, m1, l2, m2, l3, m3)
    # sum_m symbol Y Y Y is invariant and Y_m = sum_a conj(Q[a, m]) R_a
    t = np.einsum("ijk,ai,bj,ck->abc", symbol.astype(np.complex128), real_basis(l1).conj(), real_basis(l2).conj(),
                  real_basis(l3).conj())
    re, im = np.linalg.norm(t.real), np.linalg.norm(t.imag)
    if min(re, im) > 1e-9 * max(re, im):
        raise RuntimeError(f"wigner_3j({l1},{l2},{l3}) is neither real nor imaginary: {re}, {im}")
    t = t.real if re >= im else t.imag
    t = t / np.linalg.norm(t)
    t[np.abs(t) < 1e-12] = 0.0
    flat = t.reshape(-1)
    if flat[np.flatnonzero(np.abs(flat) > 1e-9)[0]] < 0:
        t = -t
    return t


# ------------------------------------------------------------------------------------------ tensor-product paths


def parity_of(l: int) -> int:
    return -1 if l & 1 else 1


def tp_paths(l_in_max: int):
    """Instructions of the channelwise edge tensor product for node irreps 0..l_in_max, harmonics 0..3 and targets
    0..3, all of natural parity; every instruction owns an output segment and the segments are sorted by target l
    (stable). Each entry: dict(l_in, l_edge, l_out, out_off, cg) with cg = sqrt(2 l_out + 1) * wigner_3j."""
    found = [(a, b, c) for a in range(l_in_max + 1) for b in range(L_SH + 1) for c in range(abs(a - b), a + b + 1)
             if c <= L_SH and parity_of(a) * parity_of(b) == parity_of(c)]
    found = sorted(found, key=lambda abc: abc[2])      # Python's sort is stable
    out, offset = [], 0
    for a, b, c in found:
        out.append(dict(l_in=a, l_edge=b, l_out=c, out_off=offset, cg=math.sqrt(2 * c + 1) * wigner_3j(a, b, c)))
        offset += 2 * c + 1
    return out


def mid_dim(paths) -> int:
    return sum(2 * p["l_out"] + 1 for p in paths)


def paths_into(paths, l_out: int):
    return [k for k, p in enumerate(paths) if p["l_out"] == l_out]


# ------------------------------------------------------------------------------------------ symmetric contraction


@functools.lru_cache(maxsize=None)
def coupling_trees(correlation: int, l_out: int):
    """Dense tensors U[2 l_out + 1, 16, ..., 16] (one axis per factor), one per coupling tree
    ((x (x) x)_{l12} (x) x)_{L} ... of ``correlation`` copies of the 16 harmonics components that ends in
    (l_out, natural parity). Each coupling multiplies by sqrt(2 l + 1) of its result; partial trees are kept sorted by
    (l, natural parity first) with a stable sort after every coupling, and the last coupling keeps only the target."""
    partial = []
    for l in range(L_SH + 1):
        start = np.zeros((2 * l + 1, N_SH))
        for m in range(2 * l + 1):
            start[m, l * l + m] = 1.0
        partial.append((l, parity_of(l), start))
    for step in range(1, correlation):
        final = step == correlation - 1
        grown = []
        for l_left, p_left, tensor in partial:
            for l in range(L_SH + 1):
                p_new = p_left * parity_of(l)
                for l_new in range(abs(l_left - l), l_left + l + 1):
                    if final and not (l_new == l_out and p_new == parity_of(l_out)):
                        continue
                    cg = math.sqrt(2 * l_new + 1) * wigner_3j(l_new, l_left, l)       # [new, left, right]
                    coupled = np.tensordot(cg, tensor, axes=([1], [0]))                # [new, right, 16...]
                    coupled = np.moveaxis(coupled, 1, -1)                              # [new, 16..., right]
                    padded = np.zeros(coupled.shape[:-1] + (N_SH,))
                    padded[..., l * l:(l + 1) ** 2] = coupled
                    grown.append((l_new, p_new, padded))
        grown.sort(key=lambda item: (item[0], 0 if item[1] == parity_of(item[0]) else 1))
        partial = grown
    return [tensor for l, p, tensor in partial if l == l_out and p == parity_of(l_out)]


def num_contraction_weights(correlation: int, l_out: int) -> int:
    return len(coupling_trees(correlation, l_out))


# ------------------------------------------------------------------------------------------ activation constant


@functools.lru_cache(maxsize=None)
def silu_second_moment_norm() -> float:
    """1 / sqrt(E[silu(z)^2]), z ~ N(0, 1): the constant e3nn's ``normalize2mom`` puts in front of SiLU (e3nn draws
    10^6 samples with a fixed seed; this is the integral they estimate)."""
    def integrand(z):
        s = z / (1.0 + math.exp(-z))
        return s * s * math.exp(-0.5 * z * z) / math.sqrt(2.0 * math.pi)
    second, _ = integrate.quad(integrand, -40.0, 40.0, epsabs=1e-14, epsrel=1e-13, limit=400)
    return 1.0 / math.sqrt(second)


__all__ = ["real_sh", "real_sh_l", "harmonics_of_unit", "real_basis", "racah_3j", "wigner_3j", "tp_paths", "mid_dim",
           "paths_into", "coupling_trees", "num_contraction_weights", "silu_second_moment_norm", "parity_of", "L_SH",
           "N_SH"]
