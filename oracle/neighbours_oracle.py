"""TEST INFRASTRUCTURE ONLY -- CPU oracle of the skin neighbour list.

NumPy float64 restatement of ``SkinNeighbourList.build_gpu`` (``fastmace/neighbors/skin.py:421-497``), its sort key
(``skin.py:506-517``) and ``compact`` (``skin.py:702-729``), with ``sort_receivers`` on and no sender groups:

* positions are wrapped into the cell (``offsets = floor(x @ inv(cell))`` with ``times_3x3``'s element-wise sums,
  ``skin.py:100-102,439-440``);
* every periodic image that can reach a wrapped pair is tried (``skin.py:399-405``), the decision is
  ``|wrapped[r] - wrapped[s] + image @ cell|^2 < (cutoff + skin)^2`` in float64 (``skin.py:459-462``), the self pair
  with zero unit shift is dropped;
* unit shifts are ``image - offsets[r] + offsets[s]`` (``skin.py:460``);
* order: receiver, then sender, then image index (``skin.py:514-516``); the image index enumerates
  ``meshgrid(range_a, range_b, range_c, indexing="ij")`` (``skin.py:404``), i.e. lexicographic in the shift;
* ``compact`` keeps the candidates whose current float64 distance is below the cutoff, in order, and counts them.

Pinned against the reference itself: ``tests/golden/make_neighbour_golden.py`` runs the reference's
``build_gpu`` + ``compact`` on CPU tensors and stores the results; ``tests/test_oracle_neighbours.py`` compares.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs may import this module.
"""

from __future__ import annotations

import numpy as np


def times_3x3(rows: np.ndarray, matrix: np.ndarray) -> np.ndarray:
    """rows @ matrix as element-wise products summed left to right (the reference's rounding order)."""
    return rows[:, 0:1] * matrix[0] + rows[:, 1:2] * matrix[1] + rows[:, 2:3] * matrix[2]


def image_grid(cell: np.ndarray, reach: float) -> np.ndarray:
    widths = 1.0 / np.linalg.norm(np.linalg.inv(cell), axis=0)
    ranges = [np.arange(-int(np.floor(reach / w + 1.0)), int(np.floor(reach / w + 1.0)) + 1) for w in widths]
    return np.stack(np.meshgrid(*ranges, indexing="ij"), axis=-1).reshape(-1, 3).astype(np.float64)


def build(positions: np.ndarray, cell: np.ndarray, cutoff: float, skin: float, chunk: int = 256):
    """Candidates within cutoff + skin: (sender [n], receiver [n], unit_shifts [n, 3]) sorted by
    (receiver, sender, image)."""
    positions = np.asarray(positions, dtype=np.float64)
    cell = np.asarray(cell, dtype=np.float64)
    reach = cutoff + skin
    natoms = len(positions)
    inverse = np.linalg.inv(cell)
    offsets = np.floor(times_3x3(positions, inverse))
    wrapped = positions - times_3x3(offsets, cell)
    images = image_grid(cell, reach)
    image_vectors = times_3x3(images, cell)
    senders, receivers, image_ids = [], [], []
    for start in range(0, natoms, chunk):
        stop = min(natoms, start + chunk)
        # [images, receivers-in-chunk, senders]
        v = (wrapped[None, start:stop, None, :] - wrapped[None, None, :, :]) + image_vectors[:, None, None, :]
        length2 = (v * v).sum(-1)
        im, rr, ss = np.nonzero(length2 < reach * reach)
        rr = rr + start
        senders.append(ss)
        receivers.append(rr)
        image_ids.append(im)
    sender = np.concatenate(senders)
    receiver = np.concatenate(receivers)
    image = np.concatenate(image_ids)
    unit_shifts = images[image] - offsets[receiver] + offsets[sender]
    keep = ~((sender == receiver) & (unit_shifts == 0).all(axis=1))
    sender, receiver, image, unit_shifts = sender[keep], receiver[keep], image[keep], unit_shifts[keep]
    order = np.lexsort((image, sender, receiver))
    return sender[order].astype(np.int64), receiver[order].astype(np.int64), unit_shifts[order]


def build_screened(positions: np.ndarray, cell: np.ndarray, cutoff: float, skin: float, margin: float = 0.01):
    """``build`` with a k-d tree screen in front of the float64 decision: the same pairs in the same order, in
    seconds instead of minutes for thousands of atoms. The screen keeps every pair within ``cutoff + skin + margin``
    (the reference screens in float32 with the same 0.01 A margin, ``pair_search.py:28``); the decision below is the
    expression of ``build``."""
    from scipy.spatial import cKDTree

    positions = np.asarray(positions, dtype=np.float64)
    cell = np.asarray(cell, dtype=np.float64)
    reach = cutoff + skin
    inverse = np.linalg.inv(cell)
    offsets = np.floor(times_3x3(positions, inverse))
    wrapped = positions - times_3x3(offsets, cell)
    images = image_grid(cell, reach)
    image_vectors = times_3x3(images, cell)
    tree = cKDTree(wrapped)
    lo, hi = wrapped.min(axis=0) - (reach + margin), wrapped.max(axis=0) + (reach + margin)
    senders, receivers, image_ids = [], [], []
    for k, shift in enumerate(image_vectors):
        # receiver r sees sender s through this image when |wrapped[r] + shift - wrapped[s]| < reach
        moved = wrapped + shift
        inside = np.flatnonzero(((moved >= lo) & (moved <= hi)).all(axis=1))
        if len(inside) == 0:
            continue
        near = cKDTree(moved[inside]).sparse_distance_matrix(tree, reach + margin, output_type="coo_matrix")
        rr, ss = inside[near.row], near.col
        v = (wrapped[rr] - wrapped[ss]) + shift
        keep = (v * v).sum(-1) < reach * reach
        senders.append(ss[keep]); receivers.append(rr[keep]); image_ids.append(np.full(int(keep.sum()), k))
    sender, receiver, image = (np.concatenate(a) for a in (senders, receivers, image_ids))
    unit_shifts = images[image] - offsets[receiver] + offsets[sender]
    keep = ~((sender == receiver) & (unit_shifts == 0).all(axis=1))
    sender, receiver, image, unit_shifts = sender[keep], receiver[keep], image[keep], unit_shifts[keep]
    order = np.lexsort((image, sender, receiver))
    return sender[order].astype(np.int64), receiver[order].astype(np.int64), unit_shifts[order]


def compact(positions, cell, sender, receiver, unit_shifts, cutoff: float):
    """Stable partition: the candidates inside the cutoff at ``positions`` first. Returns
    (sender, receiver, unit_shifts, shifts, count) with all candidates reordered."""
    positions = np.asarray(positions, dtype=np.float64)
    shifts = times_3x3(np.asarray(unit_shifts, dtype=np.float64), np.asarray(cell, dtype=np.float64))
    v = positions[receiver] - positions[sender] + shifts
    inside = (v * v).sum(-1) < cutoff * cutoff
    order = np.concatenate([np.flatnonzero(inside), np.flatnonzero(~inside)])
    return sender[order], receiver[order], unit_shifts[order], shifts[order], int(inside.sum())


def needs_rebuild(positions, reference_positions, skin: float, fraction: float = 1.0) -> bool:
    """``max_i |x_i - x_ref,i|^2 > (fraction * skin / 2)^2`` (``skin.py:685-693``)."""
    d = np.asarray(positions, dtype=np.float64) - np.asarray(reference_positions, dtype=np.float64)
    return bool((d * d).sum(-1).max() > (fraction * skin / 2.0) ** 2)


def edge_set(sender, receiver, unit_shifts, count=None):
    n = len(sender) if count is None else count
    s = np.asarray(unit_shifts)[:n].astype(np.int64)
    return set(zip(np.asarray(sender)[:n].tolist(), np.asarray(receiver)[:n].tolist(),
                   s[:, 0].tolist(), s[:, 1].tolist(), s[:, 2].tolist()))


__all__ = ["build", "build_screened", "compact", "needs_rebuild", "edge_set", "times_3x3", "image_grid"]
