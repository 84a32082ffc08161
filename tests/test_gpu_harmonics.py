"""The device's spherical harmonics and their analytic gradient against the fixture made by the reference's own Triton
kernels (``fastmace/kernels/triton/edge_sh.py:40-126`` under the interpreter; ``tests/golden/edge_sh.npz``: 257
vectors, the first of zero length), through the C ABI. Mirrors ``tests/gpu/test_edge_sh_cuda.py:1-17``."""
import ctypes
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fixture():
    return dict(np.load(os.path.join(GOLDEN, "edge_sh.npz")))


def test_probe_values_and_gradient(fixture):
    from fastmace_b200 import _lib
    lib = _lib.load()
    v = torch.tensor(fixture["vectors"], device="cuda")
    g = torch.tensor(fixture["grad_out"], device="cuda")
    sh = torch.empty(len(v), 16, device="cuda")
    gv = torch.empty(len(v), 3, device="cuda")
    _lib.check(lib.fmb_harmonics_probe(v.data_ptr(), g.data_ptr(), sh.data_ptr(), gv.data_ptr(), len(v),
                                       _lib.current_stream()), "fmb_harmonics_probe")
    torch.cuda.synchronize()
    sh, gv = sh.cpu().numpy(), gv.cpu().numpy()
    assert np.abs(sh - fixture["sh"]).max() <= 2e-6                       # both fp32, a few ulp of values up to 2.65
    assert sh[0, 0] == 1.0 and np.all(sh[0, 1:] == 0.0)                   # zero-length vector
    want = fixture["grad_vectors"]
    scale = np.abs(want[1:]).max()
    assert np.abs(gv[1:] - want[1:]).max() <= 2e-5 * scale                # regrouped fp32 sums
    # the zero-length row: the reference divides by eps = 1e-12 (values of order 1e12); same expression here
    assert np.all(np.isfinite(gv[0]))
    assert np.abs(gv[0] - want[0]).max() <= 1e-5 * max(1.0, np.abs(want[0]).max())


def test_edge_kernel_harmonics(fixture):
    """The same vectors through ``fmb_edge_features``: atom 0 sits in the middle of a large box, atom i at
    ``0.4 * v_i`` from it (inside the cutoff; the harmonics depend on the direction only), atom 1 on top of atom 0."""
    from fastmace_b200 import _lib
    from fastmace_b200.forcefield import B200ForceField
    from fastmace_b200.model import SMALL, init_weights
    lib = _lib.load()
    v = fixture["vectors"].astype(np.float64)
    scale = 0.4
    assert np.linalg.norm(v, axis=1).max() * scale < 5.9
    box = 80.0
    centre = np.full(3, box / 2)
    positions = np.concatenate([centre[None], centre[None] + scale * v])
    numbers = np.full(len(positions), 11)
    ff = B200ForceField(SMALL, init_weights(SMALL, 0), numbers, np.eye(3) * box, compute_stress=False)
    x = torch.tensor(positions, device="cuda")
    ff.rebuild(x)
    ff.compact(x)
    _lib.check(lib.fmb_edge_features(ff.packed.pointer(), ff.neighbours.pointer(), ctypes.byref(ff.work), x.data_ptr(),
                                     _lib.current_stream()), "fmb_edge_features")
    torch.cuda.synchronize()
    count = int(ff.edge_count.item())
    ei = ff.neighbours.edge_index.cpu().numpy()[:, :count]
    sh = ff.buf["edge_sh"].cpu().numpy()[:count]
    vec = ff.buf["edge_vec"].cpu().numpy()[:count]
    from_centre = np.flatnonzero(ei[0] == 0)                  # edges centre -> atom i: vector x_i - x_0 = scale * v_i
    assert len(from_centre) == len(v)
    receivers = ei[1][from_centre]
    assert np.array_equal(np.sort(receivers), np.arange(1, len(v) + 1))
    got = sh[from_centre]
    want = fixture["sh"][receivers - 1]
    assert np.abs(got - want).max() <= 3e-6                   # direction formed from float64 positions, then fp32
    lengths = vec[from_centre, 3]
    assert np.abs(lengths - scale * np.linalg.norm(v, axis=1)[receivers - 1]).max() <= 1e-5
    zero = from_centre[receivers == 1][0]
    assert sh[zero, 0] == 1.0 and np.all(sh[zero, 1:] == 0.0) and vec[zero, 3] == 0.0
