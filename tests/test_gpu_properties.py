"""Size-independent properties of the force call at the benchmark's size (1,944-atom NaCl and a 10,368-atom amorphous
Si-O cell of the 110,592-atom configuration's density, about 60 neighbours per atom; medium model), where the CPU
oracle is too slow to be the checker: the forces are the gradient of the energy, the stress is its strain derivative,
and the result follows translations, rotations and relabelling of the atoms. Everything goes through the C ABI
(B200ForceField); tolerances are the force / energy / stress tolerances of the path or tighter."""
import dataclasses

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL_E, TOL_F, TOL_S = 1e-5, 1e-4, 1e-6     # eV/atom, eV/Å, eV/Å³


@pytest.fixture(scope="module", params=["nacl1944", "silica10368"])
def bench_case(request):
    from fastmace_b200.forcefield import B200ForceField
    from fastmace_b200.model import MEDIUM, init_weights
    from fastmace_b200.structures import nacl, silica
    if request.param == "nacl1944":
        spec, s = MEDIUM, nacl((9, 9, 3), 0.05, 1)
    else:
        spec, s = dataclasses.replace(MEDIUM, avg_num_neighbors=60.0), silica(n_si=3456, seed=1)
    weights = init_weights(spec, 1)
    ff = B200ForceField(spec, weights, s.numbers, s.cell, compute_stress=True)
    e, f, st = ff.evaluate(s, stress=True)
    return spec, weights, s, ff, e, f, st


def _evaluate(case, positions, cell=None, numbers=None):
    from fastmace_b200.forcefield import B200ForceField
    spec, weights, s, ff = case[:4]
    moved = dataclasses.replace(s, positions=np.asarray(positions), cell=s.cell if cell is None else np.asarray(cell),
                                numbers=s.numbers if numbers is None else np.asarray(numbers))
    if cell is None and numbers is None:
        return ff.evaluate(moved, stress=True)
    other = B200ForceField(spec, weights, moved.numbers, moved.cell, compute_stress=True)
    return other.evaluate(moved, stress=True)


def test_forces_sum_to_zero(bench_case):
    f = bench_case[5]
    print(f"sum of forces {np.abs(f.sum(0)).max():.3e}  max|F| {np.abs(f).max():.3e}")
    assert np.abs(f.sum(0)).max() <= 1e-5 * max(1.0, s_natoms(bench_case) / 1944)


def s_natoms(case):
    return case[2].natoms


def test_forces_are_the_gradient_of_the_energy(bench_case):
    s, f = bench_case[2], bench_case[5]
    rng = np.random.default_rng(11)
    for h in (2e-3,):
        d = rng.normal(size=s.positions.shape)
        d /= np.linalg.norm(d, axis=1, keepdims=True)
        e_plus = _evaluate(bench_case, s.positions + h * d)[0]
        e_minus = _evaluate(bench_case, s.positions - h * d)[0]
        slope, expected = (e_plus - e_minus) / (2 * h), -float((f * d).sum())
        print(f"h {h:g}: dE/dh {slope:.6e}  -F.d {expected:.6e}  difference {abs(slope - expected):.3e}")
        # per-atom share of the difference far inside the force tolerance
        assert abs(slope - expected) <= 2e-3 * abs(expected) + s.natoms * 1e-3 * TOL_F


def test_stress_is_the_strain_derivative_of_the_energy(bench_case):
    s, st = bench_case[2], bench_case[6]
    rng = np.random.default_rng(12)
    direction = rng.normal(size=(3, 3))
    direction = 0.5 * (direction + direction.T)
    direction /= np.linalg.norm(direction)
    h = 1e-4
    energies = []
    for sign in (+1.0, -1.0):
        deform = np.eye(3) + sign * h * direction
        energies.append(_evaluate(bench_case, s.positions @ deform, cell=s.cell @ deform)[0])
    volume = abs(np.linalg.det(s.cell))
    slope, expected = (energies[0] - energies[1]) / (2 * h) / volume, float((st * direction).sum())
    print(f"dE/de / V {slope:.6e}  S:e {expected:.6e}  difference {abs(slope - expected):.3e}")
    assert abs(slope - expected) <= 5e-3 * abs(expected) + TOL_S


def test_translation_by_a_lattice_free_vector(bench_case):
    s, e, f, st = bench_case[2], bench_case[4], bench_case[5], bench_case[6]
    e2, f2, s2 = _evaluate(bench_case, s.positions + np.array([0.37, -1.91, 12.3]))
    print(f"translation: |dE|/atom {abs(e2 - e) / s.natoms:.3e}  max|dF| {np.abs(f2 - f).max():.3e}  "
          f"max|dS| {np.abs(s2 - st).max():.3e}")
    assert abs(e2 - e) / s.natoms <= TOL_E and np.abs(f2 - f).max() <= TOL_F and np.abs(s2 - st).max() <= TOL_S
    assert np.abs(f2 - f).max() <= 2e-4 * np.abs(f).max() + 1e-7      # the random-init model's forces are small


def test_rotation_of_atoms_and_cell(bench_case):
    s, e, f, st = bench_case[2], bench_case[4], bench_case[5], bench_case[6]
    q, _ = np.linalg.qr(np.random.default_rng(13).normal(size=(3, 3)))
    if np.linalg.det(q) < 0:
        q[:, 0] = -q[:, 0]
    e2, f2, s2 = _evaluate(bench_case, s.positions @ q, cell=s.cell @ q)
    print(f"rotation: |dE|/atom {abs(e2 - e) / s.natoms:.3e}  max|dF| {np.abs(f2 - f @ q).max():.3e}  "
          f"max|dS| {np.abs(s2 - q.T @ st @ q).max():.3e}")
    assert abs(e2 - e) / s.natoms <= TOL_E
    assert np.abs(f2 - f @ q).max() <= TOL_F and np.abs(s2 - q.T @ st @ q).max() <= TOL_S
    assert np.abs(f2 - f @ q).max() <= 2e-4 * np.abs(f).max() + 1e-7


def test_relabelling_the_atoms(bench_case):
    s, e, f, st = bench_case[2], bench_case[4], bench_case[5], bench_case[6]
    order = np.random.default_rng(14).permutation(s.natoms)
    e2, f2, s2 = _evaluate(bench_case, s.positions[order], numbers=s.numbers[order])
    print(f"relabelling: |dE|/atom {abs(e2 - e) / s.natoms:.3e}  max|dF| {np.abs(f2 - f[order]).max():.3e}  "
          f"max|dS| {np.abs(s2 - st).max():.3e}")
    assert abs(e2 - e) / s.natoms <= TOL_E
    assert np.abs(f2 - f[order]).max() <= TOL_F and np.abs(s2 - st).max() <= TOL_S
    assert np.abs(f2 - f[order]).max() <= 2e-4 * np.abs(f).max() + 1e-7


def test_large_alloy_forces_sum_to_zero_and_follow_the_energy():
    """The same two checks on the five-species alloy with the large model (1,728 atoms in a triclinic cell)."""
    from fastmace_b200.forcefield import B200ForceField
    from fastmace_b200.model import LARGE, init_weights
    from fastmace_b200.structures import fcc_alloy
    spec = dataclasses.replace(LARGE, avg_num_neighbors=54.0)
    s = fcc_alloy((12, 12, 12), 0.1, 2)
    ff = B200ForceField(spec, init_weights(spec, 2), s.numbers, s.cell, compute_stress=True)
    e, f, st = ff.evaluate(s, stress=True)
    assert np.abs(f.sum(0)).max() <= 1e-4
    rng = np.random.default_rng(15)
    d = rng.normal(size=s.positions.shape)
    d /= np.linalg.norm(d, axis=1, keepdims=True)
    h = 2e-3
    e_plus = ff.evaluate(dataclasses.replace(s, positions=s.positions + h * d))[0]
    e_minus = ff.evaluate(dataclasses.replace(s, positions=s.positions - h * d))[0]
    slope, expected = (e_plus - e_minus) / (2 * h), -float((f * d).sum())
    print(f"alloy: sum F {np.abs(f.sum(0)).max():.3e}  dE/dh {slope:.6e}  -F.d {expected:.6e}")
    assert abs(slope - expected) <= 2e-3 * abs(expected) + s.natoms * 1e-3 * TOL_F
