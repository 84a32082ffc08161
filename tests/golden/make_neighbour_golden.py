"""Generates ``tests/golden/neighbours_*.npz`` and ``tests/golden/edge_sh.npz`` from the reference itself.

Run once where the reference tree is available (it is not on the GPU box):

    python tests/golden/make_neighbour_golden.py /path/to/reference

``neighbours_large.json`` holds SHA-256 digests instead of arrays for the shapes that are too big to commit (a
10,648-atom triclinic primitive-FCC alloy cell and a 3,456-atom amorphous Si-O cell): the test regenerates the seeded
positions, checks their digest, and compares the digests of its own lists.

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


def large_cases():
    """name -> (builder name, builder kwargs, cutoff, skin): big enough for several cell-list bins per axis, the
    alloy's supercell triclinic, the Si-O box with the long rows (45-80 pairs) of the amorphous configuration."""
    return {
        "fcc10648_triclinic": ("fcc_alloy", dict(repeat=(22, 22, 22), sigma=0.1, seed=2), 6.0, 0.3),
        "silica3456": ("silica", dict(n_si=1152, seed=1), 6.0, 0.3),
    }


def digest(array) -> str:
    import hashlib
    return hashlib.sha256(np.ascontiguousarray(array).tobytes()).hexdigest()


def large_digests(nl_arrays):
    """Digests of one list: ``nl_arrays`` maps the reference's buffer names to NumPy arrays cut to their live part."""
    as_type = dict(candidate_index=np.int32, candidate_unit_shifts=np.int8, edge_index=np.int32, unit_shifts=np.int8,
                   shifts=np.float32)
    return {name: digest(np.asarray(nl_arrays[name]).astype(kind)) for name, kind in as_type.items()}


def main(reference_root):
    import json

    from fastmace_b200 import structures

    sys.path.insert(0, reference_root)
    from fastmace.config import NeighbourConfig
    from fastmace.neighbors.skin import SkinNeighbourList

    record = {}
    for name, (builder, kwargs, cutoff, skin) in large_cases().items():
        s = getattr(structures, builder)(**kwargs)
        config = NeighbourConfig(skin=skin, sort_receivers="on", gpu_neighbour_list="on")
        nl = SkinNeighbourList(s.cell, cutoff, "cpu", torch.float64, config)
        nl.build_gpu(torch.tensor(s.positions, dtype=torch.float64))
        n = nl.num_candidates
        moved = s.positions + np.random.default_rng(1).normal(0, 0.03, s.positions.shape)
        nl.compact(torch.tensor(moved))
        count = int(nl.count)
        arrays = dict(candidate_index=nl.candidate_index[:, :n].numpy(),
                      candidate_unit_shifts=nl.candidate_unit_shifts[:n].numpy(),
                      edge_index=nl.edge_index[:, :count].numpy(), unit_shifts=nl.unit_shifts[:count].numpy(),
                      shifts=nl.shifts[:count].numpy())
        rows = np.bincount(arrays["edge_index"][1], minlength=s.natoms)
        record[name] = dict(builder=builder, kwargs={k: list(v) if isinstance(v, tuple) else v for k, v in kwargs.items()},
                            cutoff=cutoff, skin=skin, natoms=s.natoms, positions=digest(s.positions),
                            moved=digest(moved), num_candidates=int(n), capacity=int(nl.capacity), count=count,
                            longest_row=int(rows.max()), shortest_row=int(rows.min()),
                            needs_rebuild=bool(nl.needs_rebuild(torch.tensor(moved))), **large_digests(arrays))
        print(name, "candidates", n, "edges", count, "capacity", nl.capacity, "rows", rows.min(), rows.max())
    with open(os.path.join(HERE, "neighbours_large.json"), "w") as handle:
        json.dump(record, handle, indent=1, sort_keys=True)

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
