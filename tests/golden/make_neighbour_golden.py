"""Generates ``tests/golden/neighbours_*.npz`` and ``tests/golden/edge_sh.npz`` from the reference itself.

Run once where the reference tree is available (it is not on the GPU box):

    python tests/golden/make_neighbour_golden.py /path/to/reference

Neighbour fixtures: the reference's ``SkinNeighbourList.build_gpu`` on CPU float64 tensors (its pure-PyTorch path,
``fastmace/neighbors/pair_search.py:242-261`` + ``skin.py:421-497``) followed by ``compact`` (``skin.py:702-729``),
for rattled, sheared and out-of-cell inputs. Spherical-harmonic fixture: the reference's Triton kernels
(``fastmace/kernels/triton/edge_sh.py``) under ``TRITON_INTERPRET=1`` on CPU tensors.
"""

import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))


def neighbour_cases():
    from fastmace_b200.structures import fcc_alloy, nacl

    cases = {}
    s = nacl((3, 3, 3), 0.05, 0)
    cases["nacl216"] = (s.positions, s.cell, 6.0, 0.3)
    s = nacl((2, 2, 2), 0.05, 3)
    shear = np.array([[1.0, 0.0, 0.0], [0.25, 1.0, 0.0], [-0.15, 0.2, 1.0]])
    cases["nacl64_sheared"] = (s.positions @ shear, s.cell @ shear, 6.0, 0.3)
    s = nacl((2, 2, 2), 0.05, 5)
    rng = np.random.default_rng(11)
    moved = s.positions + rng.integers(-2, 3, size=s.positions.shape) @ s.cell * 1.0 + rng.normal(0, 0.02, s.positions.shape)
    cases["nacl64_outside"] = (moved, s.cell, 6.0, 0.3)
    s = fcc_alloy((5, 5, 5), 0.1, 2)
    cases["fcc125_triclinic"] = (s.positions, s.cell, 6.0, 0.3)
    s = nacl((1, 1, 1), 0.05, 7)
    cases["nacl8_small_cell"] = (s.positions, s.cell, 6.0, 0.3)   # cell smaller than the cutoff: many images
    return cases


def main(reference_root):
    sys.path.insert(0, reference_root)
    from fastmace.config import NeighbourConfig
    from fastmace.neighbors.skin import SkinNeighbourList

    for name, (positions, cell, cutoff, skin) in neighbour_cases().items():
        config = NeighbourConfig(skin=skin, sort_receivers="on", gpu_neighbour_list="on")
        nl = SkinNeighbourList(cell, cutoff, "cpu", torch.float64, config)
        x = torch.tensor(positions, dtype=torch.float64)
        nl.build_gpu(x)
        n = nl.num_candidates
        cand_index = nl.candidate_index[:, :n].numpy().copy()
        cand_shift = nl.candidate_unit_shifts[:n].numpy().copy()
        # move the atoms a little (within the skin) and compact at the new positions
        moved = positions + np.random.default_rng(1).normal(0, 0.03, positions.shape)
        nl.compact(torch.tensor(moved))
        count = int(nl.count)
        np.savez_compressed(
            os.path.join(HERE, f"neighbours_{name}.npz"), positions=positions, cell=cell, cutoff=cutoff, skin=skin,
            cand_sender=cand_index[0], cand_receiver=cand_index[1], cand_unit_shifts=cand_shift,
            moved=moved, count=count, capacity=nl.capacity,
            edge_sender=nl.edge_index[0, :count].numpy(), edge_receiver=nl.edge_index[1, :count].numpy(),
            edge_unit_shifts=nl.unit_shifts[:count].numpy(), edge_shifts=nl.shifts[:count].numpy(),
            needs_rebuild=bool(nl.needs_rebuild(torch.tensor(moved))))
        print(name, "candidates", n, "edges", count, "capacity", nl.capacity)

    from fastmace.kernels.triton import edge_sh

    rng = np.random.default_rng(5)
    v = rng.normal(size=(257, 3)).astype(np.float32) * 3.0
    v[0] = 0.0                       # zero-length row: only Y_00 survives
    vt = torch.tensor(v)
    out = torch.empty(len(v), 16)
    grid = (-(-len(v) // edge_sh.BLOCK),)
    consts = dict(BLOCK=edge_sh.BLOCK, eps=edge_sh.EPS, s3=edge_sh.S3, s5=edge_sh.S5, s56=edge_sh.S56,
                  s38=edge_sh.S38, c1=edge_sh.C1, c2=edge_sh.C2, c3=edge_sh.C3)
    edge_sh._forward[grid](vt, out, len(v), **consts)
    g = torch.tensor(rng.normal(size=(len(v), 16)).astype(np.float32))
    gv = torch.empty_like(vt)
    edge_sh._backward[grid](vt, g, gv, len(v), **consts)
    np.savez_compressed(os.path.join(HERE, "edge_sh.npz"), vectors=v, sh=out.numpy(), grad_out=g.numpy(),
                        grad_vectors=gv.numpy())
    print("edge_sh", out.shape)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_neighbour_golden.py <root of the reference tree>")
    main(sys.argv[1])
