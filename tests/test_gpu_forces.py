"""Energy / forces / stress of the CUDA path against the CPU oracle, through the C ABI (B200ForceField)."""
import numpy as np
import pytest
import torch

from oracle import mace_oracle as mo
from oracle import neighbours_oracle as nlo

pytestmark = pytest.mark.gpu

# north-star tolerances: energy per atom, force component, stress component
TOL_E, TOL_F, TOL_S = 1e-5, 1e-4, 1e-6


def _case(name):
    from fastmace_b200.model import LARGE, MEDIUM, SMALL, init_weights
    from fastmace_b200.structures import fcc_alloy, nacl, silica
    if name == "small":
        return SMALL, init_weights(SMALL, 0), nacl((2, 2, 2), 0.05, 0)
    if name == "medium":
        return MEDIUM, init_weights(MEDIUM, 1), nacl((2, 2, 2), 0.05, 1)
    if name == "medium216":
        return MEDIUM, init_weights(MEDIUM, 1), nacl((3, 3, 3), 0.05, 1)
    if name == "large":
        import dataclasses
        spec = dataclasses.replace(LARGE, avg_num_neighbors=54.0)
        return spec, init_weights(spec, 2), fcc_alloy((4, 4, 4), 0.1, 2)
    if name == "silica":
        # the amorphous Si-O configuration in small: same density and rejection rule, 300 atoms, rows of 45-75 edges
        import dataclasses
        spec = dataclasses.replace(MEDIUM, avg_num_neighbors=60.0)
        return spec, init_weights(spec, 1), silica(n_si=100, seed=1)
    raise KeyError(name)


def _oracle(spec, weights, s, dtype=torch.float64, keep=None):
    snd, rcv, u = nlo.build(s.positions, s.cell, spec.r_cut, 0.0)
    return mo.evaluate(spec, weights, s.positions, s.cell, s.numbers, snd, rcv, u, dtype=dtype, keep=keep)


def _report(name, e, f, st, e_ref, f_ref, s_ref, natoms):
    de = abs(e - float(e_ref)) / natoms
    df = np.abs(f - f_ref.numpy()).max()
    ds = np.abs(st - s_ref.numpy()).max()
    fscale = np.abs(f_ref.numpy()).max()
    print(f"{name}: |dE|/atom {de:.3e}  max|dF| {df:.3e} (max|F| {fscale:.3e})  max|dS| {ds:.3e}")
    return de, df, ds, fscale


@pytest.mark.parametrize("name", ["small", "medium", "large", "silica"])
def test_energy_forces_stress_against_oracle(name):
    from fastmace_b200.forcefield import B200ForceField
    spec, weights, s = _case(name)
    ff = B200ForceField(spec, weights, s.numbers, s.cell, compute_stress=True)
    e, f, st = ff.evaluate(s, stress=True)
    e_ref, f_ref, s_ref = _oracle(spec, weights, s)
    de, df, ds, fscale = _report(name, e, f, st, e_ref, f_ref, s_ref, s.natoms)
    assert de <= TOL_E and df <= TOL_F and ds <= TOL_S
    # the random-init models give small forces, so also hold a relative bound (fp32 rounding, not a wrong term)
    assert df <= 2e-4 * fscale + 1e-7
    assert ds <= 2e-4 * np.abs(s_ref.numpy()).max() + 1e-9
    assert abs(e - float(e_ref)) <= 2e-5 * abs(float(e_ref)) + 1e-6


def test_stage_intermediates_against_oracle():
    """Each stage of the forward pass against the oracle's tensors (fp32 oracle), to localise a wrong kernel."""
    from fastmace_b200 import so3
    from fastmace_b200.codegen import message_slots
    from fastmace_b200.forcefield import B200ForceField
    spec, weights, s = _case("medium")
    keep = {}
    _oracle(spec, weights, s, dtype=torch.float64, keep=keep)
    ff = B200ForceField(spec, weights, s.numbers, s.cell, compute_stress=True)
    ff.evaluate(s, stress=True)
    nl = ff.neighbours
    count = int(nl.count.item())
    ei = nl.edge_index.cpu().numpy()[:, :count]
    # the oracle's edges are sorted the same way (receiver, sender, image) at skin 0 -> same order as compacted
    snd, rcv, u = nlo.build(s.positions, s.cell, spec.r_cut, 0.0)
    assert count == len(snd) and np.array_equal(ei[0], snd) and np.array_equal(ei[1], rcv)

    def close(a, b, what, rtol=2e-5):
        a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
        scale = np.abs(b).max() + 1e-30
        err = np.abs(a - b).max() / scale
        print(f"{what}: rel err {err:.2e} (scale {scale:.2e})")
        assert err < rtol, what

    vec = ff.buf["edge_vec"].cpu().numpy()[:count]
    close(vec[:, :3] * vec[:, 3:4], keep["vectors"].numpy(), "edge vectors")
    close(ff.buf["edge_sh"].cpu().numpy()[:count], keep["sh"].numpy(), "spherical harmonics")
    n, c = s.natoms, spec.channels
    hid = (spec.hidden_lmax + 1) ** 2
    for t in range(2):
        close(ff.buf["msg"][t].cpu().numpy(), keep[f"l{t}.message"].numpy(), f"layer {t} message")
    h = ff.buf["h"].cpu().numpy()
    close(h[:n * hid].reshape(n, hid, c), keep["l0.h"].numpy(), "layer 0 features")
    close(h[n * hid:].reshape(n, 1, c), keep["l1.h"].numpy(), "layer 1 features")
    close(ff.buf["x"].cpu().numpy(), keep["l1.x"].numpy(), "layer 1 linear_up")
    # the scattered message of the last layer is still in `mid` ... overwritten by the backward? no: d_mid is separate
    paths = spec.paths(1)
    slots, _ = message_slots(paths)
    mid = ff.buf["mid"].cpu().numpy().reshape(n, -1)[:, :so3.mid_dim(paths) * c].reshape(n, -1, c)
    ref = keep["l1.mid"].numpy()
    perm = np.zeros(so3.mid_dim(paths), dtype=np.int64)
    for p, path in enumerate(paths):
        for m in range(2 * path["l_out"] + 1):
            perm[path["out_off"] + m] = slots[(p, m)]
    close(mid[:, perm, :], ref, "layer 1 scattered message")
    close(ff.buf["node_energy"].cpu().numpy(), keep["node_energy"].numpy(), "node energies")


def test_chunked_edges_give_the_same_result():
    from fastmace_b200.forcefield import B200ForceField
    spec, weights, s = _case("medium")
    whole = B200ForceField(spec, weights, s.numbers, s.cell, compute_stress=True)
    e0, f0, s0 = whole.evaluate(s, stress=True)
    chunked = B200ForceField(spec, weights, s.numbers, s.cell, compute_stress=True, chunk_edges=300)
    e1, f1, s1 = chunked.evaluate(s, stress=True)
    # same arithmetic up to the order of the tensor-core accumulation (small chunks take the other operand order)
    assert abs(e0 - e1) <= 1e-6 * max(1.0, abs(e0))
    assert np.abs(f0 - f1).max() <= 2e-5 * np.abs(f0).max() and np.abs(s0 - s1).max() <= 2e-5 * np.abs(s0).max()


def test_repeat_calls_are_bitwise_identical():
    from fastmace_b200.forcefield import B200ForceField
    spec, weights, s = _case("medium")
    ff = B200ForceField(spec, weights, s.numbers, s.cell, compute_stress=True)
    x = torch.tensor(s.positions, device="cuda")
    ff.rebuild(x); ff.compact(x); ff.use_edges(int(ff.edge_count))
    a = ff(x)
    e0, f0, s0 = a.energy.clone(), a.forces.clone(), a.stress.clone()
    b = ff(x)
    assert torch.equal(e0, b.energy) and torch.equal(f0, b.forces) and torch.equal(s0, b.stress)


def test_work_buffers_are_released_before_they_are_reallocated():
    """When the edge capacity grows the old buffers go back to the device first, so that the two sets never coexist;
    the call after the reallocation gives the same bits."""
    from fastmace_b200.forcefield import B200ForceField
    spec, weights, s = _case("medium")
    ff = B200ForceField(spec, weights, s.numbers, s.cell, compute_stress=True)
    e0, f0, s0 = ff.evaluate(s, stress=True)
    torch.cuda.synchronize()
    held = torch.cuda.memory_allocated()
    ff._allocate_work()
    assert torch.cuda.memory_allocated() <= held + (1 << 20)
    e1, f1, s1 = ff.evaluate(s, stress=True)
    assert e1 == e0 and np.array_equal(f1, f0) and np.array_equal(s1, s0)


def test_medium_216_atoms():
    from fastmace_b200.forcefield import B200ForceField
    spec, weights, s = _case("medium216")
    ff = B200ForceField(spec, weights, s.numbers, s.cell, compute_stress=True)
    e, f, st = ff.evaluate(s, stress=True)
    e_ref, f_ref, s_ref = _oracle(spec, weights, s, dtype=torch.float32)
    de, df, ds, fscale = _report("medium216 vs fp32 oracle", e, f, st, e_ref, f_ref, s_ref, s.natoms)
    assert de <= TOL_E and df <= TOL_F and ds <= TOL_S
    assert df <= 5e-4 * fscale + 1e-7


def test_pair_rows_hold_the_radial_weights_of_both_edges_of_a_pair():
    """With the whole list as one chunk an edge and its opposite edge share one row of radial weights (they have the
    same length). After a force call: every pair is listed once, the slots are the rows 0 .. pairs - 1, and the row an
    edge reads -- slot[min(e, mirror e)] -- holds hidden(e) x (last radial layer) for values and for d/dr."""
    from fastmace_b200.forcefield import B200ForceField
    spec, weights, s = _case("medium216")
    ff = B200ForceField(spec, weights, s.numbers, s.cell, compute_stress=True)
    ff.evaluate(s, stress=True)
    torch.cuda.synchronize()
    assert int(ff.work.pair_capacity) == 0 and "edge_slot" in ff.buf
    count = int(ff.neighbours.count.item())
    mirror = ff.buf["mirror"][:count].long()
    edges = torch.arange(count, device=ff.device)
    assert bool((mirror >= 0).all()) and bool((mirror[mirror] == edges).all()) and bool((mirror != edges).all())
    pairs = int(ff.buf["canon_count"].item())
    assert pairs * 2 == count
    listed = edges < mirror
    slots = ff.buf["edge_slot"][:count].long()
    assert torch.equal(torch.sort(slots[listed]).values, torch.arange(pairs, device=ff.device))
    assert torch.equal(ff.buf["canon_list"][:pairs].long()[slots[listed]], edges[listed])
    row = slots[torch.minimum(edges, mirror)]
    last = spec.num_interactions - 1
    rad = ff.packed.tensors[f"l{last}.rad.3"].double()                        # [64][paths * C], scaled
    rows_per_half = ff.buf["tp_w"].shape[0] // 2
    for tangent in (0, 1):
        hidden = ff.buf["edge_hidden"][last, tangent, :count].double()
        want = hidden @ rad
        got = ff.buf["tp_w"][tangent * rows_per_half + row].double()
        scale = float(want.abs().max())
        assert float((got - want).abs().max()) <= 2e-6 * scale, tangent


def test_gemm_kernels_against_torch():
    """SIMT fp32 GEMM and the tcgen05 3xTF32 GEMM against a float64 product."""
    from fastmace_b200 import _lib
    from fastmace_b200.packing import tensor_core_twin
    lib = _lib.load()
    torch.manual_seed(0)
    status = torch.zeros((), dtype=torch.int32, device="cuda")
    for m, n, k in [(1000, 128, 128), (257, 256, 64), (4096, 1280, 64), (77, 128, 384), (128, 64, 64)]:
        a = torch.randn(m, k, device="cuda")
        b = torch.randn(k, n, device="cuda")
        ref = (a.double() @ b.double())
        scale = ref.abs().max().item()
        twin = tensor_core_twin([b.cpu()]).cuda()
        hi, lo = twin[:n * k], twin[n * k:]
        for impl, tol in ((0, 1e-5), (1, 1e-5)):
            if impl == 0 and n % 128:
                continue
            c = torch.zeros(m, n, device="cuda")
            args = (a.data_ptr(), b.data_ptr(), hi.data_ptr(), lo.data_ptr(), c.data_ptr(), m, n, k)
            _lib.check(lib.fmb_gemm(*args, 0, impl, status.data_ptr(), _lib.current_stream()), "gemm")
            err = (c.double() - ref).abs().max().item() / scale
            print(f"gemm impl {impl} {m}x{n}x{k}: rel err {err:.2e}")
            assert err <= tol, (impl, m, n, k, err)
            _lib.check(lib.fmb_gemm(*args, 1, impl, status.data_ptr(), _lib.current_stream()), "gemm")
            assert (c.double() - 2 * ref).abs().max().item() / scale <= 2 * tol
    assert int(status.item()) == 0


def test_warp_specialised_gemm_against_torch():
    """The kernel behind the node linears, called alone through its weight image: launches below one wave use
    128 x 128 tiles, larger ones pair column tiles (128 x 256), with an odd 128-wide tile left where N / 128 is odd."""
    from fastmace_b200 import _lib
    from fastmace_b200.packing import tensor_core_image
    lib = _lib.load()
    torch.manual_seed(1)
    status = torch.zeros((), dtype=torch.int32, device="cuda")
    for m, n, k in [(1000, 128, 128), (257, 256, 64), (4096, 1280, 64), (20000, 384, 128), (31104, 256, 128),
                    (19000, 128, 256), (77, 128, 384)]:
        a = torch.randn(m, k, device="cuda")
        b = torch.randn(k, n, device="cuda")
        ref = a.double() @ b.double()
        scale = ref.abs().max().item()
        image = tensor_core_image([b.cpu()]).cuda()
        c = torch.zeros(m, n, device="cuda")
        args = (a.data_ptr(), b.data_ptr(), image.data_ptr(), None, c.data_ptr(), m, n, k)
        _lib.check(lib.fmb_gemm(*args, 0, 2, status.data_ptr(), _lib.current_stream()), "gemm")
        err = (c.double() - ref).abs().max().item() / scale
        print(f"gemm_ws {m}x{n}x{k}: rel err {err:.2e}")
        assert err <= 1e-5, (m, n, k, err)
        _lib.check(lib.fmb_gemm(*args, 1, 2, status.data_ptr(), _lib.current_stream()), "gemm")
        assert (c.double() - 2 * ref).abs().max().item() / scale <= 2e-5
    assert int(status.item()) == 0


@pytest.mark.parametrize("name,chunk,edge_adjoint", [
    ("medium", 1 << 19, False),      # mirror-evaluation adjoint (the path of lists too large for the per-edge
    ("large", 4096, False),          # hand-over buffers), one chunk and several, node l_max 1 and 2
    ("large", 4096, None),           # several chunks: fused forward (weights only in tensor memory), per-edge adjoint
    ("silica", 2048, None),          # the same on the amorphous cell's long rows
])
def test_paths_of_other_size_regimes_against_oracle(name, chunk, edge_adjoint):
    """The kernels that large systems select by themselves (chunked edge lists, the mirror adjoint), reached here on
    small cells through the constructor arguments that size them, against the oracle like the default path."""
    from fastmace_b200.forcefield import B200ForceField
    spec, weights, s = _case(name)
    ff = B200ForceField(spec, weights, s.numbers, s.cell, compute_stress=True, chunk_edges=chunk,
                        edge_adjoint=edge_adjoint)
    e, f, st = ff.evaluate(s, stress=True)
    assert ff.edge_local == (edge_adjoint is None)
    e_ref, f_ref, s_ref = _oracle(spec, weights, s)
    de, df, ds, fscale = _report(f"{name} chunk {chunk} edge_adjoint {edge_adjoint}", e, f, st, e_ref, f_ref, s_ref,
                                 s.natoms)
    assert de <= TOL_E and df <= TOL_F and ds <= TOL_S
    assert df <= 2e-4 * fscale + 1e-7


def test_set_cell_follows_a_strained_cell():
    """Variable cell (``ForceField.set_cell``, fastmace/model/forces.py:1351-1356): after a homogeneous strain of
    cell and positions the force field gives what a force field built for the strained cell gives, first on the
    candidates of the old cell (small strain, inside the skin), then after the rebuild the deformation-aware test
    (fastmace/neighbors/skin.py:694-700) asks for."""
    from fastmace_b200.forcefield import B200ForceField
    spec, weights, s = _case("medium")
    ff = B200ForceField(spec, weights, s.numbers, s.cell, compute_stress=True)
    x0 = torch.tensor(s.positions, device="cuda")
    ff.rebuild(x0); ff.compact(x0)
    rebuilds = ff.neighbours.rebuilds
    for scale, expect_rebuild in ((1.004, False), (1.03, True)):
        strain = np.eye(3) * scale + np.array([[0, 0.002, 0], [0.002, 0, 0], [0, 0, 0]]) * (scale - 1) * 10
        cell = s.cell @ strain
        x = torch.tensor(s.positions @ strain, device="cuda")
        ff.set_cell(torch.tensor(cell, device="cuda"))
        flag = bool(ff.needs_rebuild(x).item())
        # the reference's formula in NumPy
        f_map = np.linalg.solve(cell, s.cell)
        disp = np.sqrt((((s.positions @ strain) @ f_map - s.positions) ** 2).sum(1).max())
        eps = np.linalg.solve(s.cell, cell) - np.eye(3)
        lower = 1.0 - np.sqrt((eps * eps).sum())
        allowed = spec.r_cut + 0.3 - spec.r_cut / max(lower, 1e-6)
        assert flag == bool(2 * disp > allowed or lower <= 0) == expect_rebuild
        if flag:
            ff.rebuild(x)
        ff.compact(x)
        out = ff(x)
        torch.cuda.synchronize()
        ff.check_status()
        fresh = B200ForceField(spec, weights, s.numbers, cell, compute_stress=True)
        import dataclasses
        e, f, st = fresh.evaluate(dataclasses.replace(s, positions=s.positions @ strain, cell=cell), stress=True)
        assert abs(float(out.energy.item()) - e) / s.natoms <= TOL_E
        assert np.abs(out.forces.double().cpu().numpy() - f).max() <= 2e-4 * np.abs(f).max() + 1e-7
        assert np.abs(out.stress.double().cpu().numpy() - st).max() <= 2e-4 * np.abs(st).max() + 1e-9
    assert ff.neighbours.rebuilds == rebuilds + 1


def test_accuracy_gate_on_rattled_and_strained_copies():
    """The reference's acceptance rule for a production path (SPEC.md:2038,2051-2066; planner/selfcheck.py:242-274):
    error against float64 at most 3 x the float32 calculator's error, with floors. Production = the CUDA path; float64
    reference and float32 yardstick = the CPU oracle in the two precisions."""
    from fastmace_b200 import gate
    from fastmace_b200.forcefield import B200ForceField
    spec, weights, s = _case("medium")
    fields = {}

    def field_for(cell):
        key = cell.tobytes()
        if key not in fields:
            fields[key] = B200ForceField(spec, weights, s.numbers, cell, compute_stress=True)
        return fields[key]

    def oracle(dtype):
        def evaluate(positions, cell):
            snd, rcv, u = nlo.build(positions, cell, spec.r_cut, 0.0)
            e, f, st = mo.evaluate(spec, weights, positions, cell, s.numbers, snd, rcv, u, dtype=dtype)
            return float(e), f.numpy(), st.numpy()
        return evaluate

    record = gate.run_gate(gate.force_field_evaluator(field_for, s.numbers), oracle(torch.float64), oracle(torch.float32),
                           s.positions, s.cell, s.natoms, seed=3, stress=True)
    for name, q in record["verdict"]["quantities"].items():
        print(f"gate {name}: production {q['production']:.3e}  float32 yardstick {q['yardstick']:.3e}  "
              f"ratio {q['ratio']}  limit {q['limit']:.3e}  {'passed' if q['passed'] else 'FAILED'}")
    assert record["status"] == "passed" and len(record["rows"]) == 4
