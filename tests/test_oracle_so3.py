"""Pins of the SO(3) tables on both sides of the GPU-versus-oracle comparison (CPU only).

* the reference-made spherical-harmonics fixture (``tests/golden/edge_sh.npz``: values and the analytic gradient of
  the reference's Triton kernel, ``fastmace/kernels/triton/edge_sh.py:40-126``) against the oracle's harmonics, the
  oracle's autograd gradient and the product's table ``so3.real_sh``;
* the product's Wigner tensors against (a) the oracle's, which come from Racah's formula and SciPy's complex
  harmonics, and (b) a Gaunt quadrature written here that uses neither;
* tensor-product paths, coupling trees of the symmetric contraction (equality of the two derivations, rotation
  invariance, linear independence) and the SiLU constant;
* rotation equivariance and finite-difference forces / stress of the oracle's energy.

Mirrors ``tests/gpu/test_edge_sh_cuda.py:1-17`` of the reference (harmonics against e3nn in float64 within float32
rounding, zero-length rows included).
"""

import dataclasses
import math
import os

import numpy as np
import pytest
import torch

from fastmace_b200 import so3
from fastmace_b200.model import SILU_NORM, SMALL, MEDIUM, init_weights
from fastmace_b200.structures import nacl
from oracle import mace_oracle, neighbours_oracle, so3_oracle

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "edge_sh.npz")


@pytest.fixture(scope="module")
def sh_fixture():
    return dict(np.load(GOLDEN))


def test_oracle_harmonics_match_the_reference_kernel(sh_fixture):
    v = sh_fixture["vectors"].astype(np.float64)
    assert np.abs(so3_oracle.real_sh(v) - sh_fixture["sh"]).max() <= 1e-6          # float32 rounding of the kernel
    got = mace_oracle.spherical_harmonics(torch.tensor(v)).numpy()
    assert np.abs(got - sh_fixture["sh"]).max() <= 1e-6
    assert np.all(got[0, 1:] == 0.0) and got[0, 0] == 1.0                           # the zero-length row


def test_product_harmonics_match_the_reference_kernel(sh_fixture):
    v = sh_fixture["vectors"].astype(np.float64)
    assert np.abs(so3.real_sh(v) - sh_fixture["sh"]).max() <= 1e-6


def test_oracle_gradient_matches_the_reference_backward(sh_fixture):
    """Autograd through the oracle's harmonics against the reference's analytic backward kernel."""
    v = torch.tensor(sh_fixture["vectors"].astype(np.float64), requires_grad=True)
    g = torch.tensor(sh_fixture["grad_out"].astype(np.float64))
    (mace_oracle.spherical_harmonics(v) * g).sum().backward()
    want = sh_fixture["grad_vectors"].astype(np.float64)
    got = v.grad.numpy()
    scale = np.maximum(1.0, np.abs(want).max(axis=1, keepdims=True))
    assert np.abs(got[1:] - want[1:]).max() <= 2e-5 * scale.max()                  # fp32 kernel, regrouped sums
    assert np.all(np.isfinite(got[0]))                                              # zero vector: finite (clamped norm)


TRIPLES_TP = sorted({(p["l_in"], p["l_edge"], p["l_out"]) for lin in (0, 1, 2) for p in so3.tp_paths(lin)})


@pytest.mark.parametrize("triple", TRIPLES_TP)
def test_wigner_tensor_equals_racah_derivation(triple):
    a, b = so3.wigner_3j(*triple), so3_oracle.wigner_3j(*triple)
    assert a.shape == b.shape
    assert np.abs(a - b).max() <= 1e-12


def test_wigner_tensors_of_the_contraction_equal_racah_derivation():
    """Every coupling the symmetric contraction uses, intermediates up to l = 6 and unnatural parities included."""
    for l_left in range(0, 7):
        for l in range(0, 4):
            for l_new in range(abs(l_left - l), min(l_left + l, 6) + 1):
                if l_left > 3 and l_new > 2:
                    continue                     # third factor: only targets 0..2 are ever kept
                a, b = so3.wigner_3j(l_new, l_left, l), so3_oracle.wigner_3j(l_new, l_left, l)
                assert np.abs(a - b).max() <= 1e-12, (l_new, l_left, l)


def _sphere_quadrature(n_theta=24, n_phi=49):
    """Gauss-Legendre in cos(theta) times a uniform grid in phi: exact for polynomials of degree < 48."""
    t, w = np.polynomial.legendre.leggauss(n_theta)
    phi = 2.0 * math.pi * np.arange(n_phi) / n_phi
    ct, ph = np.meshgrid(t, phi, indexing="ij")
    st = np.sqrt(1.0 - ct * ct)
    pts = np.stack([st * np.cos(ph), st * np.sin(ph), ct], axis=-1).reshape(-1, 3)
    weights = np.repeat(w, n_phi) / (2.0 * n_phi)          # sums to 1: the average over the sphere
    return pts, weights


def test_wigner_tensor_against_gaunt_quadrature(sh_fixture):
    """<Y_a Y_b Y_c> over the sphere is proportional to the invariant tensor of (l1, l2, l3) when l1 + l2 + l3 is even.
    The harmonics are evaluated with the polynomials written out below, which are checked against the reference-made
    fixture first; no table of the product or of the oracle enters."""
    def harmonics(p):
        x, y, z = p[:, 0], p[:, 1], p[:, 2]
        r3, r5, r7 = math.sqrt(3), math.sqrt(5), math.sqrt(7)
        r15, r105 = math.sqrt(15), math.sqrt(105)
        cols = [np.ones_like(x), r3 * x, r3 * y, r3 * z,
                r15 * x * z, r15 * x * y, r5 * (y * y - 0.5 * (x * x + z * z)), r15 * y * z, 0.5 * r15 * (z * z - x * x),
                r7 * math.sqrt(5 / 8) * x * (3 * z * z - x * x), r105 * x * y * z,
                r7 * math.sqrt(3 / 8) * x * (4 * y * y - x * x - z * z),
                r7 * 0.5 * y * (2 * y * y - 3 * x * x - 3 * z * z),
                r7 * math.sqrt(3 / 8) * z * (4 * y * y - x * x - z * z), 0.5 * r105 * y * (z * z - x * x),
                r7 * math.sqrt(5 / 8) * z * (z * z - 3 * x * x)]
        return np.stack(cols, axis=1)

    v = sh_fixture["vectors"][1:].astype(np.float64)
    u = v / np.linalg.norm(v, axis=1, keepdims=True)
    assert np.abs(harmonics(u) - sh_fixture["sh"][1:]).max() <= 1e-6
    pts, w = _sphere_quadrature()
    y = harmonics(pts)
    assert np.abs((y * w[:, None]).T @ y - np.eye(16)).max() <= 1e-12             # component normalisation
    for l1, l2, l3 in TRIPLES_TP:
        if l1 > 3:
            continue
        s1, s2, s3 = (slice(l * l, (l + 1) ** 2) for l in (l1, l2, l3))
        gaunt = np.einsum("n,na,nb,nc->abc", w, y[:, s1], y[:, s2], y[:, s3])
        norm = np.linalg.norm(gaunt)
        assert norm > 1e-6, (l1, l2, l3)
        t = so3.wigner_3j(l1, l2, l3)
        cosine = float((gaunt * t).sum() / norm)
        assert abs(abs(cosine) - 1.0) <= 1e-12, (l1, l2, l3, cosine)


def test_tensor_product_paths_agree():
    for lin in (0, 1, 2):
        ours, theirs = so3.tp_paths(lin), so3_oracle.tp_paths(lin)
        assert [(p["l_in"], p["l_edge"], p["l_out"], p["out_off"]) for p in ours] == \
               [(p["l_in"], p["l_edge"], p["l_out"], p["out_off"]) for p in theirs]
        assert so3.mid_dim(ours) == so3_oracle.mid_dim(theirs) == (16, 40, 71)[lin]
        for a, b in zip(ours, theirs):
            dense = np.zeros_like(b["cg"])
            for m_in, m_edge, m_out, coef in a["terms"]:
                dense[m_in, m_edge, m_out] = coef
            assert np.abs(dense - b["cg"]).max() <= 1e-12
            # component normalisation of the path: sum over (m_in, m_edge) of cg^2 is 1 for every output component
            assert np.abs((b["cg"] ** 2).sum(axis=(0, 1)) - 1.0).max() <= 1e-12


def _block_rotation(rot):
    d = np.zeros((16, 16))
    for l in range(4):
        pts = np.random.default_rng(3 + l).normal(size=(40, 3))
        a, b = so3_oracle.real_sh_l(l, pts), so3_oracle.real_sh_l(l, pts @ rot.T)
        d[l * l:(l + 1) ** 2, l * l:(l + 1) ** 2] = np.linalg.lstsq(a, b, rcond=None)[0].T
    return d


@pytest.mark.parametrize("correlation,l_out,count", [(1, 0, 1), (1, 1, 1), (2, 0, 4), (2, 1, 6), (3, 0, 23), (3, 1, 51)])
def test_coupling_trees(correlation, l_out, count):
    ours, theirs = so3.coupling_trees(correlation, l_out), so3_oracle.coupling_trees(correlation, l_out)
    assert len(ours) == len(theirs) == count == so3.num_contraction_weights(correlation, l_out)
    for a, b in zip(ours, theirs):
        assert np.abs(a - b).max() <= 1e-12
    # equivariance: U(D x, ..., D x) = D_L U(x, ..., x) for a random rotation
    rot = so3.random_rotation(11)
    d = _block_rotation(rot)
    d_out = d[l_out * l_out:(l_out + 1) ** 2, l_out * l_out:(l_out + 1) ** 2]
    x = np.random.default_rng(5).normal(size=16)
    for u in theirs[:8]:
        def apply(vec):
            out = u
            for _ in range(correlation):
                out = out @ vec
            return out
        assert np.abs(apply(d @ x) - d_out @ apply(x)).max() <= 1e-10
    # the trees, symmetrised over the factors (the contraction feeds the same x into every slot), span a space of
    # full rank only up to the known redundancy; they must at least be non-zero and finite
    assert all(np.isfinite(u).all() and np.abs(u).max() > 0 for u in theirs)


def test_silu_constant():
    assert abs(SILU_NORM - so3_oracle.silu_second_moment_norm()) <= 1e-9
    z = np.random.default_rng(0).normal(size=2_000_000)
    estimate = 1.0 / math.sqrt(np.mean((z / (1.0 + np.exp(-z))) ** 2))
    assert abs(estimate - SILU_NORM) <= 3e-3


def _evaluate(spec, weights, positions, cell, numbers, stress=True):
    snd, rcv, u = neighbours_oracle.build(positions, cell, spec.r_cut, 0.0)
    return mace_oracle.evaluate(spec, weights, positions, cell, numbers, snd, rcv, u, compute_stress=stress)


@pytest.mark.parametrize("spec", [SMALL, MEDIUM], ids=["small", "medium"])
def test_oracle_energy_is_rotation_equivariant(spec):
    spec = dataclasses.replace(spec, channels=128)
    weights = init_weights(spec, 4, dtype=torch.float64)
    s = nacl((1, 1, 1), 0.08, 2)
    e, f, st = _evaluate(spec, weights, s.positions, s.cell, s.numbers)
    rot = so3.random_rotation(9)
    e2, f2, st2 = _evaluate(spec, weights, s.positions @ rot.T, s.cell @ rot.T, s.numbers)
    r = torch.tensor(rot)
    assert abs(float(e2 - e)) <= 1e-10 * max(1.0, abs(float(e)))
    assert float((f2 - f @ r.T).abs().max()) <= 1e-10
    assert float((st2 - r @ st @ r.T).abs().max()) <= 1e-11
    # a relabelling of the atoms permutes the forces
    perm = np.random.default_rng(1).permutation(s.natoms)
    e3, f3, _ = _evaluate(spec, weights, s.positions[perm], s.cell, s.numbers[perm])
    assert abs(float(e3 - e)) <= 1e-10 * max(1.0, abs(float(e)))
    assert float((f3 - f[perm]).abs().max()) <= 1e-10


def test_oracle_forces_and_stress_are_the_energy_derivatives():
    spec = MEDIUM
    weights = init_weights(spec, 5, dtype=torch.float64)
    s = nacl((1, 1, 1), 0.08, 3)
    snd, rcv, u = neighbours_oracle.build(s.positions, s.cell, spec.r_cut, 0.0)

    def energy(positions, cell):
        return float(mace_oracle.evaluate(spec, weights, positions, cell, s.numbers, snd, rcv, u,
                                          compute_stress=False)[0])

    _, forces, stress = mace_oracle.evaluate(spec, weights, s.positions, s.cell, s.numbers, snd, rcv, u)
    h = 1e-5
    for atom, axis in ((0, 0), (3, 1), (6, 2)):
        plus, minus = s.positions.copy(), s.positions.copy()
        plus[atom, axis] += h
        minus[atom, axis] -= h
        fd = -(energy(plus, s.cell) - energy(minus, s.cell)) / (2 * h)
        assert abs(fd - float(forces[atom, axis])) <= 1e-7 * max(1.0, abs(fd))
    volume = abs(np.linalg.det(s.cell))
    for i, j in ((0, 0), (0, 1), (2, 1)):
        eps = np.zeros((3, 3))
        eps[i, j] += 0.5 * h
        eps[j, i] += 0.5 * h
        deform = lambda sign: (s.positions @ (np.eye(3) + sign * eps), s.cell @ (np.eye(3) + sign * eps))
        fd = (energy(*deform(+1)) - energy(*deform(-1))) / (2 * h) / volume
        assert abs(fd - float(stress[i, j])) <= 1e-8 * max(1.0, abs(fd) * 1e3)
