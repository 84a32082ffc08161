"""Real SO(3) tables for the MACE force path: spherical harmonics l <= 3, Wigner-3j tensors, coupling paths of the
channelwise tensor product and the polynomial form of the symmetric contraction.

Everything here is float64 NumPy evaluated once when a model is packed for the device (or when the CUDA sources are
generated); nothing here runs per MD step.

Conventions
-----------
* Real spherical harmonics follow the component order and polynomials that FastMACE's own kernel states for
  ``o3.SphericalHarmonics(lmax=3, normalize=True, normalization="component")``
  (reference: ``fastmace/kernels/triton/edge_sh.py:40-78``): index 0 is ``1``; 1..3 are ``sqrt(3) * (x, y, z)``;
  4..8 and 9..15 the l = 2 and l = 3 polynomials in the same order, on the unit vector.
* The real basis of every irrep l is *defined* by those functions: ``Y_l(R v) = D_l(R) Y_l(v)``.
* ``wigner_3j(l1, l2, l3)`` is the (unique up to sign) tensor invariant under ``D_l1 x D_l2 x D_l3`` with unit
  Frobenius norm. The sign is fixed by making the first entry (row-major) larger than 1e-9 in magnitude positive.
  e3nn fixes its signs through a complex-to-real change of basis instead, so a given path may differ from e3nn's by a
  global sign; with randomly initialised weights this is a reparametrisation (w -> -w), not another model.
* The tensor-product paths, their order and their normalisation follow MACE's ``tp_out_irreps_with_instructions`` +
  e3nn ``TensorProduct("uvu", irrep_normalization="component", path_normalization="element")``: each instruction owns
  its output segment, so the path coefficient is ``sqrt(2 l_out + 1)`` (reference call site:
  ``fastmace/rewrites/generic/modules.py:485``; per-term coefficient ``wigner_3j * path_weight``:
  ``fastmace/kernels/oeq_streaming/schedule.py:318-339``).
* The symmetric contraction follows MACE's ``U_matrix_real`` construction: every coupling tree
  ``((x_l1 (x) x_l2)_l12 (x) x_l3)_L`` with component normalisation ``sqrt(2 l + 1)`` at every coupling is one
  weight; the trees are not orthogonalised. Its polynomial form (one coefficient per sorted monomial, weight and
  output component) is what the reference's generated kernels evaluate
  (``fastmace/kernels/cuda/sc_generated.py:1-20``).
"""

from __future__ import annotations

import functools
import itertools
import math

import numpy as np

S3 = math.sqrt(3.0)
S5 = math.sqrt(5.0)
S56 = math.sqrt(5.0 / 6.0)
S38 = math.sqrt(3.0 / 8.0)
C1, C2, C3 = math.sqrt(3.0), math.sqrt(5.0), math.sqrt(7.0)

LMAX_SH = 3
NSH = 16  # (LMAX_SH + 1) ** 2


def sh_offset(l: int) -> int:
    """First component of irrep l inside a 0..l_max block (l*l)."""
    return l * l


def real_sh(vectors: np.ndarray) -> np.ndarray:
    """[n, 3] vectors -> [n, 16] component-normalised real spherical harmonics of the unit vectors."""
    v = np.asarray(vectors, dtype=np.float64)
    n = np.sqrt((v * v).sum(-1, keepdims=True))
    u = v / np.maximum(n, 1e-12)
    x, y, z = u[:, 0], u[:, 1], u[:, 2]
    s20 = S3 * x * z
    s21 = S3 * x * y
    y2 = y * y
    x2z2 = x * x + z * z
    s22 = y2 - 0.5 * x2z2
    s23 = S3 * y * z
    s24 = S3 / 2.0 * (z * z - x * x)
    s30 = S56 * (s20 * z + s24 * x)
    s31 = S5 * s20 * y
    s32 = S38 * (4.0 * y2 - x2z2) * x
    s33 = 0.5 * y * (2.0 * y2 - 3.0 * x2z2)
    s34 = S38 * z * (4.0 * y2 - x2z2)
    s35 = S5 * s24 * y
    s36 = S56 * (s24 * z - s20 * x)
    one = np.ones_like(x)
    return np.stack([one, C1 * x, C1 * y, C1 * z, C2 * s20, C2 * s21, C2 * s22, C2 * s23, C2 * s24,
                     C3 * s30, C3 * s31, C3 * s32, C3 * s33, C3 * s34, C3 * s35, C3 * s36], axis=1)


# --------------------------------------------------------------------------- general real harmonics (any l)
# The symmetric contraction couples through intermediate irreps up to l = 6, so D-matrices are needed beyond the
# 16 functions above. For l > 3 any real orthonormal basis serves (intermediates are summed over), built here from
# the standard real harmonics; for l <= 3 the basis is the one above.


def _legendre(l: int, m: int, t: np.ndarray) -> np.ndarray:
    """Associated Legendre P_l^m(t) without the Condon-Shortley phase, m >= 0 (stable upward recurrence)."""
    pmm = np.ones_like(t)
    if m > 0:
        somx2 = np.sqrt(np.maximum(0.0, 1.0 - t * t))
        fact = 1.0
        for _ in range(m):
            pmm = pmm * fact * somx2
            fact += 2.0
    if l == m:
        return pmm
    pmmp1 = t * (2 * m + 1) * pmm
    if l == m + 1:
        return pmmp1
    for ll in range(m + 2, l + 1):
        pll = (t * (2 * ll - 1) * pmmp1 - (ll + m - 1) * pmm) / (ll - m)
        pmm, pmmp1 = pmmp1, pll
    return pmmp1


def _generic_real_sh(l: int, u: np.ndarray) -> np.ndarray:
    """[n, 2l+1] orthonormal-on-the-sphere-up-to-a-constant real harmonics of unit vectors (component norm)."""
    x, y, z = u[:, 0], u[:, 1], u[:, 2]
    phi = np.arctan2(y, x)
    out = []
    for m in range(-l, l + 1):
        am = abs(m)
        k = math.sqrt((2 * l + 1) * math.factorial(l - am) / math.factorial(l + am))
        p = _legendre(l, am, z)
        if m == 0:
            out.append(k * p)
        elif m > 0:
            out.append(math.sqrt(2.0) * k * p * np.cos(am * phi))
        else:
            out.append(math.sqrt(2.0) * k * p * np.sin(am * phi))
    return np.stack(out, axis=1)


def sh_l(l: int, vectors: np.ndarray) -> np.ndarray:
    """Component-normalised real harmonics of degree l in this module's basis: [n, 2l+1]."""
    v = np.asarray(vectors, dtype=np.float64)
    u = v / np.sqrt((v * v).sum(-1, keepdims=True))
    if l <= LMAX_SH:
        return real_sh(u)[:, l * l:(l + 1) * (l + 1)]
    return _generic_real_sh(l, u)


_RNG_POINTS = np.random.default_rng(20240607).normal(size=(97, 3))


def wigner_d(l: int, rotation: np.ndarray) -> np.ndarray:
    """D_l(R) with ``Y_l(R v) = D_l(R) Y_l(v)`` (least squares over fixed sample points; exact to rounding)."""
    a = sh_l(l, _RNG_POINTS)                    # [n, 2l+1]
    b = sh_l(l, _RNG_POINTS @ rotation.T)       # Y(R v)
    d_t, *_ = np.linalg.lstsq(a, b, rcond=None)  # a @ d_t = b  =>  d_t = D^T
    return d_t.T


def _rotations(count: int = 4) -> list[np.ndarray]:
    rng = np.random.default_rng(7)
    out = []
    for _ in range(count):
        q, r = np.linalg.qr(rng.normal(size=(3, 3)))
        q = q * np.sign(np.diag(r))
        if np.linalg.det(q) < 0:
            q[:, 0] = -q[:, 0]
        out.append(q)
    return out


@functools.lru_cache(maxsize=None)
def wigner_3j(l1: int, l2: int, l3: int) -> np.ndarray:
    """The invariant tensor of l1 x l2 x l3, shape [2l1+1, 2l2+1, 2l3+1], unit Frobenius norm, fixed sign."""
    if not abs(l1 - l2) <= l3 <= l1 + l2:
        raise ValueError(f"no coupling {l1} x {l2} -> {l3}")
    n1, n2, n3 = 2 * l1 + 1, 2 * l2 + 1, 2 * l3 + 1
    rows = []
    for rot in _rotations():
        d1, d2, d3 = wigner_d(l1, rot), wigner_d(l2, rot), wigner_d(l3, rot)
        rows.append(np.kron(np.kron(d1, d2), d3) - np.eye(n1 * n2 * n3))
    _, s, vt = np.linalg.svd(np.concatenate(rows, axis=0))
    if not (s[-1] < 1e-9 and (len(s) == 1 or s[-2] > 1e-3)):
        raise RuntimeError(f"wigner_3j({l1},{l2},{l3}): invariant subspace is not one-dimensional: {s[-3:]}")
    c = vt[-1]
    c = c / np.linalg.norm(c)
    c[np.abs(c) < 1e-12] = 0.0
    first = c[np.flatnonzero(np.abs(c) > 1e-9)[0]]
    if first < 0:
        c = -c
    return c.reshape(n1, n2, n3)


# --------------------------------------------------------------------------- tensor-product paths (conv_tp)


def natural_parity(l: int) -> int:
    return 1 if l % 2 == 0 else -1


def tp_paths(l_in_max: int, l_edge_max: int = LMAX_SH, l_out_max: int = LMAX_SH):
    """Paths of ``conv_tp`` for node irreps 0..l_in_max (natural parity), edge irreps 0..l_edge_max and targets
    0..l_out_max (natural parity), in the order of the sorted output segments.

    Returns a list of dicts ``{l_in, l_edge, l_out, in_off, edge_off, out_off, terms}`` where ``out_off`` is the
    first component of the path's own output segment inside the scattered message (segments sorted by l_out, stable
    in enumeration order), and ``terms`` is a list ``(m_in, m_edge, m_out, coefficient)`` of the nonzero entries of
    ``sqrt(2 l_out + 1) * wigner_3j(l_in, l_edge, l_out)``.
    """
    raw = []
    for l_in in range(l_in_max + 1):
        for l_edge in range(l_edge_max + 1):
            for l_out in range(abs(l_in - l_edge), l_in + l_edge + 1):
                parity = natural_parity(l_in) * natural_parity(l_edge)
                if l_out <= l_out_max and parity == natural_parity(l_out):
                    raw.append((l_in, l_edge, l_out))
    order = sorted(range(len(raw)), key=lambda k: raw[k][2])  # stable sort of the output segments by irrep
    paths, out_off = [], 0
    for k in order:
        l_in, l_edge, l_out = raw[k]
        c = wigner_3j(l_in, l_edge, l_out) * math.sqrt(2 * l_out + 1)
        terms = [(int(a), int(b), int(d), float(c[a, b, d]))
                 for a, b, d in zip(*np.nonzero(np.abs(c) > 1e-12))]
        paths.append(dict(l_in=l_in, l_edge=l_edge, l_out=l_out, in_off=sh_offset(l_in), edge_off=sh_offset(l_edge),
                          out_off=out_off, terms=terms))
        out_off += 2 * l_out + 1
    return paths


def mid_dim(paths) -> int:
    """Components per channel of the scattered message (sum of the paths' 2 l_out + 1)."""
    return sum(2 * p["l_out"] + 1 for p in paths)


def paths_into(paths, l_out: int) -> list[int]:
    """Indices of the paths whose output irrep is l_out, in segment order (the K blocks of the message linear)."""
    return [k for k, p in enumerate(paths) if p["l_out"] == l_out]


# --------------------------------------------------------------------------- symmetric contraction


def _irrep_sort_key(l: int, parity: int):
    # natural parity first for a given l: 0e, 0o, 1o, 1e, 2e, 2o, 3o, 3e, ...
    return (l, 0 if parity == natural_parity(l) else 1)


@functools.lru_cache(maxsize=None)
def coupling_trees(correlation: int, l_out: int, l_in_max: int = LMAX_SH):
    """Coupling trees of ``correlation`` copies of x (irreps 0..l_in_max, natural parity) ending in irrep
    (l_out, natural parity), in MACE's order: the partial trees are sorted by their irrep (stable) at every level.

    Returns a list of dense tensors ``U[2 l_out + 1, 16, ..., 16]`` (one axis of 16 per copy).
    """
    dim = (l_in_max + 1) ** 2
    level = []
    for l in range(l_in_max + 1):
        e = np.zeros((2 * l + 1, dim))
        e[np.arange(2 * l + 1), l * l + np.arange(2 * l + 1)] = 1.0
        level.append(((l, natural_parity(l)), e))
    for depth in range(correlation - 1):
        last = depth == correlation - 2  # the last coupling keeps only the requested output irrep
        nxt = []
        for (l_left, p_left), c_left in level:
            for l in range(l_in_max + 1):
                p = natural_parity(l)
                for l_new in range(abs(l_left - l), l_left + l + 1):
                    if last and (l_new != l_out or p_left * p != natural_parity(l_out)):
                        continue
                    w = wigner_3j(l_new, l_left, l) * math.sqrt(2 * l_new + 1)  # [new, left, right]
                    c = np.einsum("j...,ijl->i...l", c_left, w)
                    full = np.zeros(c.shape[:-1] + (dim,))
                    full[..., l * l:(l + 1) * (l + 1)] = c
                    nxt.append(((l_new, p_left * p), full))
        nxt.sort(key=lambda item: _irrep_sort_key(*item[0]))
        level = nxt
    return [u for (l, p), u in level if l == l_out and p == natural_parity(l_out)]


@functools.lru_cache(maxsize=None)
def contraction_polynomial(correlation: int, l_out: int, l_in_max: int = LMAX_SH):
    """Polynomial form of one (correlation, l_out) block of the symmetric contraction.

    Returns ``(monomials [T, correlation] int, m_out [T] int, weight [T] int, coefficient [T] float, num_weights)``:
    ``out[m_out] += W[weight] * coefficient * prod_k x[monomials[t, k]]`` with sorted monomials; equal
    (monomial, m_out, weight) entries are merged and zeros dropped.
    """
    trees = coupling_trees(correlation, l_out, l_in_max)
    terms: dict[tuple, float] = {}
    for k, u in enumerate(trees):
        for index in zip(*np.nonzero(np.abs(u) > 1e-12)):
            m_out, mono = int(index[0]), tuple(sorted(int(i) for i in index[1:]))
            key = (mono, m_out, k)
            terms[key] = terms.get(key, 0.0) + float(u[index])
    keys = sorted(key for key, value in terms.items() if abs(value) > 1e-12)
    monomials = np.array([key[0] for key in keys], dtype=np.int64).reshape(len(keys), correlation)
    m_out = np.array([key[1] for key in keys], dtype=np.int64)
    weight = np.array([key[2] for key in keys], dtype=np.int64)
    coefficient = np.array([terms[key] for key in keys], dtype=np.float64)
    return monomials, m_out, weight, coefficient, len(trees)


@functools.lru_cache(maxsize=None)
def contraction_keys(l_out_max: int, correlation: int = 3, l_in_max: int = LMAX_SH):
    """Sorted (output component, degree, sorted monomial) keys of the contraction polynomial for outputs 0..l_out_max:
    the order of the per-(species, channel) coefficient table and of the generated kernels."""
    keys = set()
    for big_l in range(l_out_max + 1):
        for nu in range(1, correlation + 1):
            mono, m_out, _, _, _ = contraction_polynomial(nu, big_l, l_in_max)
            for t in range(len(m_out)):
                keys.add((big_l * big_l + int(m_out[t]), nu, tuple(int(i) for i in mono[t])))
    return tuple(sorted(keys))


def num_contraction_weights(correlation: int, l_out: int, l_in_max: int = LMAX_SH) -> int:
    return len(coupling_trees(correlation, l_out, l_in_max))


def random_rotation(seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    q, r = np.linalg.qr(rng.normal(size=(3, 3)))
    q = q * np.sign(np.diag(r))
    if np.linalg.det(q) < 0:
        q[:, 0] = -q[:, 0]
    return q


__all__ = ["real_sh", "sh_l", "wigner_d", "wigner_3j", "tp_paths", "mid_dim", "paths_into", "coupling_trees",
           "contraction_polynomial", "contraction_keys", "num_contraction_weights", "natural_parity", "sh_offset", "random_rotation",
           "NSH", "LMAX_SH"]
