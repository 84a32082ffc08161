"""TEST INFRASTRUCTURE ONLY -- CPU oracle of the MACE energy / forces / stress path.

A plain PyTorch (CPU, autograd) restatement of ``ScaleShiftMACE.forward`` as FastMACE calls it
(``fastmace/model/forces.py:1237-1240``): the third-party model (mace-torch 0.3.16 on e3nn 0.4.4) is NOT vendored in
the reference tree and is not installed here, so this file restates its published algorithm from the places where
the reference itself restates it:

* spherical harmonics: ``fastmace/kernels/triton/edge_sh.py:40-78`` (values, constants, component order);
* interaction block dataflow: ``fastmace/rewrites/generic/modules.py:381-505`` (kind "residual"), e3nn
  ``FullyConnectedNet`` scaling ``fastmace/rewrites/generic/modules.py:148-150``;
* channelwise tensor product indexing: ``fastmace/kernels/oeq_streaming/factorized_projected.cuh:128-186``;
* symmetric contraction as a polynomial in the message components: ``fastmace/kernels/cuda/sc_generated.py:1-20``
  (evaluated here in MACE's Horner order from the dense, non-symmetrised coupling tensors);
* forces, virial, stress, symmetric strain: ``fastmace/rewrites/engine.py:142-192``;
* energy contract (E0 and the reduction in float64): ``fastmace/model/energy.py:92-99,122-133``.

PARITY UNPINNED against mace-torch 0.3.16: the reference holds no golden energies/forces, and mace/e3nn cannot be
imported here. What IS pinned: the spherical harmonics (against the reference kernel run under the Triton
interpreter, fixture ``tests/golden/edge_sh.npz``, checked in ``tests/test_oracle_so3.py``), equivariance /
invariance properties and finite-difference forces and stress (same test file).

The coupling tables (Wigner tensors, tensor-product paths, coupling trees, the SiLU constant) come from
``oracle/so3_oracle.py``, which derives them from Racah's formula and SciPy's complex harmonics; nothing of the
product package ``fastmace_b200`` is imported: the model description is read from plain integer / float attributes
(``channels, hidden_lmax, sh_lmax, correlation, num_interactions, r_cut, num_bessel, cutoff_p, num_elements,
mlp_hidden, avg_num_neighbors, scale, shift``) of whatever object is passed as ``spec``.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs may import this module. The
product path never does.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from . import so3_oracle as so3

SILU_NORM = so3.silu_second_moment_norm()


def l_in_max(spec, layer: int) -> int:
    return 0 if layer == 0 else spec.hidden_lmax


def l_out_max(spec, layer: int) -> int:
    return spec.hidden_lmax if layer < spec.num_interactions - 1 else 0


def out_dim(spec, layer: int) -> int:
    return (l_out_max(spec, layer) + 1) ** 2


def skip_lmax(spec, layer: int) -> int:
    return min(l_in_max(spec, layer), l_out_max(spec, layer))


def paths_of(spec, layer: int):
    return so3.tp_paths(l_in_max(spec, layer))


def spherical_harmonics(vectors: torch.Tensor) -> torch.Tensor:
    """[E, 3] -> [E, 16]; ``v / max(|v|, eps)`` like ``torch.nn.functional.normalize`` (edge_sh.py:30-37)."""
    n = torch.linalg.norm(vectors, dim=1, keepdim=True)
    u = vectors / torch.clamp(n, min=1e-12)
    return torch.stack(so3.harmonics_of_unit(u[:, 0], u[:, 1], u[:, 2]), dim=1)


def bessel_cutoff(r: torch.Tensor, spec) -> torch.Tensor:
    """[E] -> [E, num_bessel]: sqrt(2/rc) sin(n pi r / rc) / r times the polynomial envelope (p = cutoff_p)."""
    rc, p = spec.r_cut, float(spec.cutoff_p)
    n = torch.arange(1, spec.num_bessel + 1, dtype=r.dtype)
    bessel = math.sqrt(2.0 / rc) * torch.sin(n * (math.pi / rc) * r[:, None]) / r[:, None]
    x = r / rc
    env = (1.0 - (p + 1.0) * (p + 2.0) / 2.0 * x ** p + p * (p + 2.0) * x ** (p + 1.0)
           - p * (p + 1.0) / 2.0 * x ** (p + 2.0))
    env = env * (x < 1.0).to(r.dtype)
    return bessel * env[:, None]


def silu_n(x: torch.Tensor) -> torch.Tensor:
    return SILU_NORM * torch.nn.functional.silu(x)


def radial_mlp(edge_feats: torch.Tensor, weights, layer: int, hidden_only: bool = False) -> torch.Tensor:
    x = edge_feats
    count = sum(1 for k in weights if k.startswith(f"l{layer}.rad."))
    for i in range(count):
        w = weights[f"l{layer}.rad.{i}"]
        if hidden_only and i == count - 1:
            return x
        x = x @ (w / math.sqrt(w.shape[0]))
        if i < count - 1:
            x = silu_n(x)
    return x


def interaction(spec, weights, layer, h, species, sender, receiver, sh, edge_feats, keep=None):
    """One residual interaction: returns (message [N, 16, C], sc [N, out_dim, C])."""
    c, dtype, n = spec.channels, h.dtype, h.shape[0]
    n_el = spec.num_elements
    sc = torch.zeros(n, out_dim(spec, layer), c, dtype=dtype)
    for l in range(skip_lmax(spec, layer) + 1):
        w = weights[f"l{layer}.skip.{l}"][:, species, :]  # [C, N, C]
        sl = slice(l * l, (l + 1) ** 2)
        sc[:, sl, :] = torch.einsum("nmc,cnd->nmd", h[:, sl, :], w) / math.sqrt(c * n_el)
    x = torch.zeros_like(h)
    for l in range(l_in_max(spec, layer) + 1):
        sl = slice(l * l, (l + 1) ** 2)
        x[:, sl, :] = h[:, sl, :] @ (weights[f"l{layer}.up.{l}"] / math.sqrt(c))
    paths = paths_of(spec, layer)
    tp_w = radial_mlp(edge_feats, weights, layer).reshape(-1, len(paths), c)
    mid = torch.zeros(n, so3.mid_dim(paths), c, dtype=dtype)
    xs = x[sender]
    for p, path in enumerate(paths):
        li, le, lo = path["l_in"], path["l_edge"], path["l_out"]
        cg = torch.tensor(path["cg"], dtype=dtype)
        coupled = torch.einsum("abd,eb->ead", cg, sh[:, le * le:(le + 1) ** 2])       # harmonics first: [E, in, out]
        t = torch.einsum("ead,eac->edc", coupled, xs[:, li * li:(li + 1) ** 2, :])
        mji = t * tp_w[:, p, None, :]
        seg = slice(path["out_off"], path["out_off"] + 2 * lo + 1)
        mid[:, seg, :] = mid[:, seg, :].index_add(0, receiver, mji)
    message = torch.zeros(n, 16, c, dtype=dtype)
    for lo in range(spec.sh_lmax + 1):
        into = so3.paths_into(paths, lo)
        norm = 1.0 / math.sqrt(len(into) * c)
        acc = 0
        for p in into:
            seg = slice(paths[p]["out_off"], paths[p]["out_off"] + 2 * lo + 1)
            acc = acc + mid[:, seg, :] @ (weights[f"l{layer}.lin.{p}"] * norm)
        message[:, lo * lo:(lo + 1) ** 2, :] = acc
    message = message / spec.avg_num_neighbors
    if keep is not None:
        keep[f"l{layer}.x"] = x
        keep[f"l{layer}.tp_w"] = tp_w
        keep[f"l{layer}.mid"] = mid
        keep[f"l{layer}.message"] = message
        keep[f"l{layer}.sc"] = sc
    return message, sc


def symmetric_contraction(spec, weights, layer, message, species, chunk=128):
    """[N, 16, C] -> [N, out_dim, C]: MACE's Horner evaluation with dense coupling tensors (correlation 3).

    Evaluated per present species (the weights are species-dependent) and in chunks of atoms to bound memory."""
    n, _, c = message.shape
    dtype = message.dtype
    out = torch.zeros(n, out_dim(spec, layer), c, dtype=dtype)
    for z in torch.unique(species).tolist():
        atoms = torch.nonzero(species == z).reshape(-1)
        for big_l in range(l_out_max(spec, layer) + 1):
            uws = {}
            for nu in range(1, spec.correlation + 1):
                u = torch.tensor(np.stack(so3.coupling_trees(nu, big_l), axis=0), dtype=dtype)
                uws[nu] = torch.einsum("k...,kc->...c", u, weights[f"l{layer}.sc.{big_l}.{nu}"][z])  # [M,16^nu,C]
            for start in range(0, len(atoms), chunk):
                idx = atoms[start:start + chunk]
                x = message[idx]                                             # [n, 16, C]
                acc = None
                for nu in range(spec.correlation, 0, -1):
                    u = uws[nu]                                              # [M, 16 (nu times), C]
                    if acc is None:
                        # the weighted coupling tensor has no atom axis yet: one GEMM per channel over all atoms
                        flat = u.reshape(-1, u.shape[-2], c)
                        acc = torch.einsum("kic,nic->nkc", flat, x).reshape(len(idx), *u.shape[:-2], c)
                    else:
                        acc = torch.einsum("n...ic,nic->n...c", acc + u[None], x)
                out[idx, big_l * big_l:(big_l + 1) ** 2, :] = acc
    return out


def product(spec, weights, layer, message, sc, species, keep=None):
    c = spec.channels
    basis = symmetric_contraction(spec, weights, layer, message, species)
    out = torch.zeros_like(basis)
    for big_l in range(l_out_max(spec, layer) + 1):
        sl = slice(big_l * big_l, (big_l + 1) ** 2)
        out[:, sl, :] = basis[:, sl, :] @ (weights[f"l{layer}.prod.{big_l}"] / math.sqrt(c))
    if keep is not None:
        keep[f"l{layer}.basis"] = basis
    return out + sc


def readout(spec, weights, layer, h):
    c = spec.channels
    scalars = h[:, 0, :]
    if layer < spec.num_interactions - 1:
        return scalars @ (weights[f"l{layer}.readout"] / math.sqrt(c))
    hidden = silu_n(scalars @ (weights[f"l{layer}.readout.0"] / math.sqrt(c)))
    return hidden @ (weights[f"l{layer}.readout.1"] / math.sqrt(spec.mlp_hidden))


def evaluate(spec, weights, positions, cell, atomic_numbers, sender, receiver, unit_shifts,
             dtype=torch.float64, compute_stress=True, keep=None, n_energy=None):
    """Energy (float64 scalar), forces [N, 3], stress [3, 3] (ASE sign, dE/d(strain) / |det cell|).

    ``positions`` [N, 3] and ``cell`` [3, 3] float64; ``sender``/``receiver`` int64 [E]; ``unit_shifts`` [E, 3]
    integer-valued; ``atomic_numbers`` [N]. ``dtype`` is the model precision: edge vectors are formed in float64 and
    cast (the reference's large-box path, ``fastmace/model/forces.py:176-186``), per-atom energies are summed in
    float64. ``keep``: optional dict that receives intermediates for kernel-level tests. ``n_energy``: only the first
    ``n_energy`` atoms contribute energy (the owned atoms of one domain; the others are halo atoms).
    """
    weights = {k: v.to(dtype) for k, v in weights.items()}
    positions = torch.as_tensor(positions, dtype=torch.float64).clone().requires_grad_(True)
    cell = torch.as_tensor(cell, dtype=torch.float64)
    species = torch.as_tensor(atomic_numbers, dtype=torch.int64) - 1   # one-hot index of Z = 1..89
    sender = torch.as_tensor(sender, dtype=torch.int64)
    receiver = torch.as_tensor(receiver, dtype=torch.int64)
    unit_shifts = torch.as_tensor(unit_shifts, dtype=torch.float64)
    strain = torch.zeros(3, 3, dtype=torch.float64, requires_grad=True)
    sym = 0.5 * (strain + strain.T)
    pos = positions + positions @ sym
    strained_cell = cell + cell @ sym
    vectors64 = pos[receiver] - pos[sender] + unit_shifts @ strained_cell
    vectors = vectors64.to(dtype)
    r = torch.linalg.norm(vectors, dim=1)
    sh = spherical_harmonics(vectors)
    edge_feats = bessel_cutoff(r, spec)
    c = spec.channels
    n = positions.shape[0]
    h = torch.zeros(n, 1, c, dtype=dtype)
    h[:, 0, :] = weights["emb"][species] / math.sqrt(spec.num_elements)
    node_energy = torch.zeros(n, dtype=dtype)
    if keep is not None:
        keep["vectors"], keep["sh"], keep["edge_feats"] = vectors, sh, edge_feats
    for t in range(spec.num_interactions):
        message, sc = interaction(spec, weights, t, h, species, sender, receiver, sh, edge_feats, keep)
        h = product(spec, weights, t, message, sc, species, keep)
        if keep is not None:
            keep[f"l{t}.h"] = h
        node_energy = node_energy + readout(spec, weights, t, h)
    node_energy = spec.scale * node_energy + spec.shift
    e0 = torch.zeros(spec.num_elements, dtype=torch.float64)[species]    # the benchmark models have zero E0
    if n_energy is not None:
        e0, node_energy = e0[:n_energy], node_energy[:n_energy]
    energy = e0.sum() + node_energy.to(torch.float64).sum()
    if keep is not None:
        keep["node_energy"] = node_energy
    grads = torch.autograd.grad(energy, (positions, strain))
    forces = -grads[0]
    stress = None
    if compute_stress:
        stress = grads[1] / torch.abs(torch.linalg.det(cell))
        stress = 0.5 * (stress + stress.T)
    if keep is not None:
        for k, v in list(keep.items()):
            keep[k] = v.detach()
    return energy.detach(), forces.detach(), None if stress is None else stress.detach()


__all__ = ["evaluate", "spherical_harmonics", "bessel_cutoff", "radial_mlp", "interaction", "symmetric_contraction",
           "product", "readout"]
