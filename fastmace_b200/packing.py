"""Packs a MACE model for the device: folds every normalisation constant into the weights, restricts the
species-dependent tensors to the species that are present, lays the per-irrep linears out as plain [K][N] matrices and
turns the symmetric contraction into per-(species, channel) polynomial coefficients.

These are the exact algebraic rewrites the reference applies once at set-up ("species tables", 1/sqrt(fan_in) folded
into W, species skip restricted to present species: ``fastmace/config.py:208-219``,
``fastmace/rewrites/generic/modules.py:584-593,726-737``); nothing here runs per step.
"""

from __future__ import annotations

import ctypes
import math

import numpy as np
import torch

from . import so3
from ._lib import MAX_SPECIES, LayerStruct, ModelStruct
from .codegen import message_slots
from .model import SILU_NORM, MaceSpec, e0_table


def _f64(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to(torch.float64).cpu()


def tf32_round(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> nearest tf32 (10-bit mantissa, ties away from zero, like cvt.rna.tf32.f32), returned as fp32."""
    bits = x.contiguous().view(torch.int32)
    return ((bits + 0x1000) & ~0x1fff).view(torch.float32)


def tensor_core_twin(blocks) -> torch.Tensor:
    """For a list of fp32 [K][N] weight blocks: the concatenation of, per block, the transposed block [N][K] rounded
    to tf32 followed by the tf32-rounded remainder -- the operands of the 3xTF32 tensor-core GEMM. The twin of a
    block that starts at float offset o of the concatenated weights starts at 2 o."""
    out = []
    for block in blocks:
        bt = block.to(torch.float32).t().contiguous()
        hi = tf32_round(bt)
        lo = tf32_round(bt - hi)
        out += [hi.reshape(-1), lo.reshape(-1)]
    return torch.cat(out)


def _swizzled_tile_index() -> torch.Tensor:
    """Float index inside a [128 rows][32 K] operand tile (K-major, 128-byte rows in 1024-byte groups of 8 rows, the
    16-byte chunk index XORed with row mod 8) of element (row, k), flattened row-major."""
    row = torch.arange(128).view(128, 1)
    kk = torch.arange(32).view(1, 32)
    return ((row >> 3) * 256 + (row & 7) * 32 + ((((kk >> 2) & 7) ^ (row & 7)) << 2) + (kk & 3)).reshape(-1)


def tensor_core_image(blocks) -> torch.Tensor:
    """For a list of fp32 [K][N] weight blocks: per block (at twice its float offset, like ``tensor_core_twin``) the
    pieces the warp-specialised GEMM copies into shared memory -- for column tile nt and K chunk kc the [128][32] tile
    of the transposed block as 4,096 tf32 values followed by their 4,096 remainders, both in the swizzled operand
    layout. Blocks with N % 128 != 0 or K % 32 != 0 stay zero."""
    index = _swizzled_tile_index()
    out = []
    for block in blocks:
        k, n = block.shape
        image = torch.zeros(2 * k * n, dtype=torch.float32)
        if n % 128 == 0 and k % 32 == 0:
            bt = block.to(torch.float32).t().contiguous()
            hi = tf32_round(bt)
            lo = tf32_round(bt - hi)
            view = image.view(n // 128, k // 32, 2, 4096)
            for nt in range(n // 128):
                for kc in range(k // 32):
                    rows, cols = slice(nt * 128, nt * 128 + 128), slice(kc * 32, kc * 32 + 32)
                    view[nt, kc, 0, index] = hi[rows, cols].reshape(-1)
                    view[nt, kc, 1, index] = lo[rows, cols].reshape(-1)
        out.append(image)
    return torch.cat(out)


def radial_image(w4: torch.Tensor, channels: int = 128) -> torch.Tensor:
    """The last radial layer [64][paths * channels] (fp32, already scaled) as the fused tensor-product kernels stream it:
    per path p, K half h and part (0 = tf32 remainder, 1 = tf32 value) one 16 KB tile [128 channels][32 features] of the
    transposed block in the K-major operand layout with 128-byte swizzle (8-row groups of 1024 bytes, the 16-byte
    chunk index XORed with row mod 8), at float offset ((p * 2 + h) * 2 + part) * 4096."""
    k, n = w4.shape
    assert k == 64 and channels == 128 and n % channels == 0
    bt = w4.to(torch.float32).t().contiguous()                      # [paths * 128][64]
    hi = tf32_round(bt)
    lo = tf32_round(bt - hi)
    row = torch.arange(128).view(128, 1)
    kk = torch.arange(32).view(1, 32)
    offset = (row >> 3) * 256 + (row & 7) * 32 + ((((kk >> 2) & 7) ^ (row & 7)) << 2) + (kk & 3)   # float index in a tile
    offset = offset.reshape(-1)
    n_paths = n // channels
    image = torch.zeros(n_paths, 2, 2, 4096, dtype=torch.float32)
    for p in range(n_paths):
        for h in range(2):
            for part, source in enumerate((lo, hi)):
                image[p, h, part, offset] = source[p * 128:(p + 1) * 128, h * 32:(h + 1) * 32].reshape(-1)
    return image.reshape(-1)


def mlp_image(w0: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    """The three hidden layers of a radial MLP ([8][64], [64][64], [64][64], fp32, already scaled) as the operand images
    the tcgen05 edge kernel bulk-copies: a layer [K][64] becomes the tile [64 outputs][K] of its transpose, K-major with
    the 128-byte swizzle in halves of 32 K (2,048 floats each; the first layer fills 8 of the 32 columns of one half),
    tf32 values first, then the tf32 remainders. Float offsets: first layer 0 / 2,048, second 4,096 / 8,192, third
    12,288 / 16,384."""
    assert tuple(w0.shape) == (8, 64) and tuple(w1.shape) == (64, 64) and tuple(w2.shape) == (64, 64)
    row = torch.arange(64).view(64, 1)
    kk = torch.arange(32).view(1, 32)
    index = ((row >> 3) * 256 + (row & 7) * 32 + ((((kk >> 2) & 7) ^ (row & 7)) << 2) + (kk & 3)).reshape(-1)
    image = torch.zeros(20480, dtype=torch.float32)

    def parts(w):
        bt = w.to(torch.float32).t().contiguous()                  # [64 outputs][K]
        hi = tf32_round(bt)
        return hi, tf32_round(bt - hi)

    hi, lo = parts(w0)
    for base, source in ((0, hi), (2048, lo)):
        tile = torch.zeros(64, 32, dtype=torch.float32)
        tile[:, :8] = source
        image[base + index] = tile.reshape(-1)
    for layer, w in enumerate((w1, w2)):
        hi, lo = parts(w)
        for part, source in enumerate((hi, lo)):
            for half in range(2):
                base = 4096 + layer * 8192 + part * 4096 + half * 2048
                image[base + index] = source[:, half * 32:half * 32 + 32].reshape(-1)
    return image


def contraction_terms(spec: MaceSpec, weights, layer: int, species_z):
    """(terms int32 [T, 4], coef float64 [n_species, T, C]) of one layer's symmetric contraction, sorted by output."""
    c = spec.channels
    merged: dict[tuple, np.ndarray] = {}
    for big_l in range(spec.l_out_max(layer) + 1):
        for nu in range(1, spec.correlation + 1):
            mono, m_out, weight, coef, _ = so3.contraction_polynomial(nu, big_l, spec.sh_lmax)
            w = _f64(weights[f"l{layer}.sc.{big_l}.{nu}"]).numpy()[[z - 1 for z in species_z]]  # [nz, k, C]
            for t in range(len(coef)):
                key = (big_l * big_l + int(m_out[t]), nu, tuple(int(i) for i in mono[t]))
                value = coef[t] * w[:, weight[t], :]
                if key in merged:
                    merged[key] = merged[key] + value
                else:
                    merged[key] = value
    keys = sorted(merged)
    if tuple(keys) != so3.contraction_keys(spec.l_out_max(layer), spec.correlation, spec.sh_lmax):
        raise RuntimeError("contraction terms are not in the order the generated kernels expect")
    terms = np.full((len(keys), 4), -1, dtype=np.int32)
    coefs = np.zeros((len(species_z), len(keys), c), dtype=np.float64)
    for t, key in enumerate(keys):
        m_out, _, mono = key
        terms[t, :len(mono)] = mono
        terms[t, 3] = m_out
        coefs[:, t, :] = merged[key]
    return terms, coefs


class PackedModel:
    """Device tensors of a model restricted to ``species_z`` (sorted atomic numbers present) and the ``ModelStruct``
    the C ABI reads. Keeps the tensors alive for as long as the struct is used."""

    def __init__(self, spec: MaceSpec, weights, species_z, device):
        species_z = [int(z) for z in species_z]
        if species_z != sorted(set(species_z)):
            raise ValueError("species_z must be sorted and unique")
        if len(species_z) > MAX_SPECIES:
            raise ValueError(f"at most {MAX_SPECIES} species per structure, got {len(species_z)}")
        if spec.num_interactions != 2 or spec.channels != 128 or spec.correlation != 3:
            raise ValueError("the device path takes 2 interactions, 128 channels, correlation 3")
        self.spec = spec
        self.species_z = species_z
        self.device = torch.device(device)
        self.tensors: dict[str, torch.Tensor] = {}
        c, n_el = spec.channels, spec.num_elements
        idx = [z - 1 for z in species_z]
        w = {k: _f64(v) for k, v in weights.items()}
        struct = ModelStruct()
        struct.n_species = len(species_z)
        struct.channels = c
        struct.hidden_lmax = spec.hidden_lmax
        struct.n_layers = spec.num_interactions
        struct.n_bessel = spec.num_bessel
        struct.cutoff_p = spec.cutoff_p
        struct.radial_width = spec.radial_hidden[-1]
        struct.mlp_hidden = spec.mlp_hidden
        struct.r_cut = spec.r_cut
        struct.scale = spec.scale
        struct.shift = spec.shift
        struct.silu_norm = SILU_NORM
        e0 = e0_table(spec)
        for k, z in enumerate(species_z):
            struct.e0[k] = float(e0[z - 1])
        h0 = w["emb"][idx] / math.sqrt(n_el)                                   # [nz, C]
        for t in range(spec.num_interactions):
            layer = struct.layer[t]
            paths = spec.paths(t)
            slots, blocks = message_slots(paths)
            layer.l_in_max = spec.l_in_max(t)
            layer.l_out_max = spec.l_out_max(t)
            layer.n_paths = len(paths)
            layer.mid_dim = so3.mid_dim(paths)
            layer.skip_lmax = spec.skip_lmax(t)
            layer.is_last = int(t == spec.num_interactions - 1)
            widths = (spec.num_bessel, *spec.radial_hidden, len(paths) * c)
            for i in range(4):
                layer.rad_w[i] = self._put(f"l{t}.rad.{i}", w[f"l{t}.rad.{i}"] / math.sqrt(widths[i]))
            layer.tc[0] = self._twin(f"l{t}.rad.3", [self.tensors[f"l{t}.rad.3"]])
            if t > 0 and c == 128:
                layer.rad_img = self._put(f"l{t}.rad.img", radial_image(self.tensors[f"l{t}.rad.3"].cpu(), c))
            if spec.num_bessel == 8 and tuple(spec.radial_hidden) == (64, 64, 64):
                layer.mlp_img = self._put(f"l{t}.rad.mlp_img",
                                          mlp_image(*(self.tensors[f"l{t}.rad.{i}"].cpu() for i in range(3))))
            if t == 0:
                x_species = h0 @ (w["l0.up.0"] / math.sqrt(c))
                sc = torch.zeros(len(idx), spec.out_dim(0), c, dtype=torch.float64)
                skip = w["l0.skip.0"]                                           # [C, 89, C]
                for k, e in enumerate(idx):
                    sc[k, 0] = h0[k] @ skip[:, e, :] / math.sqrt(c * n_el)
                layer.x_species = self._put("l0.x_species", x_species)
                layer.sc_species = self._put("l0.sc_species", sc)
                # reassociated first layer: message[i, (l, m), :] = sum_z S[i, (l, m), z, :] @ first_l[z], with
                # S[i, lm, z, k] = sum_{e -> i, species(sender) = z} hidden[e, k] * Y[e, lm]  (exact algebra)
                w4 = (w["l0.rad.3"] / math.sqrt(widths[3])).to(torch.float32).to(torch.float64)
                blocks = []
                for l_out in range(spec.sh_lmax + 1):
                    (p0,) = so3.paths_into(paths, l_out)
                    lin_l = w[f"l0.lin.{p0}"] / math.sqrt(c) / spec.avg_num_neighbors
                    per_z = [(w4[:, p0 * c:(p0 + 1) * c] * x_species[z][None, :]) @ lin_l for z in range(len(idx))]
                    blocks.append(torch.cat(per_z, dim=0).to(torch.float32))           # [nz * 64, C]
                layer.first[0] = self._put("l0.first", torch.cat([b.reshape(-1) for b in blocks]))
                layer.first[1] = self._put("l0.first_t", torch.cat([b.t().contiguous().reshape(-1) for b in blocks]))
                layer.first[2] = self._twin("l0.first", blocks)
                layer.first_img[0] = self._image_of("l0.first")
                layer.first[3] = self._twin("l0.first_t", [b.t().contiguous() for b in blocks])
                layer.first_img[1] = self._image_of("l0.first_t")
            else:
                up = torch.stack([w[f"l{t}.up.{l}"] / math.sqrt(c) for l in range(spec.l_in_max(t) + 1)])
                layer.w_up = self._put(f"l{t}.w_up", up)
                layer.w_up_t = self._put(f"l{t}.w_up_t", up.transpose(1, 2))
                layer.tc[1] = self._twin(f"l{t}.w_up", list(self.tensors[f"l{t}.w_up"]))
                layer.tc_img[1] = self._image_of(f"l{t}.w_up")
                layer.tc[2] = self._twin(f"l{t}.w_up_t", list(self.tensors[f"l{t}.w_up_t"]))
                layer.tc_img[2] = self._image_of(f"l{t}.w_up_t")
                skip = torch.stack([w[f"l{t}.skip.{l}"][:, idx, :].permute(1, 0, 2) / math.sqrt(c * n_el)
                                    for l in range(spec.skip_lmax(t) + 1)])     # [L, nz, C, C]
                layer.w_skip = self._put(f"l{t}.w_skip", skip)
                layer.w_skip_t = self._put(f"l{t}.w_skip_t", skip.transpose(2, 3))
                layer.tc[3] = self._twin(f"l{t}.w_skip", list(self.tensors[f"l{t}.w_skip"].reshape(-1, c, c)))
                layer.tc_img[3] = self._image_of(f"l{t}.w_skip")
                layer.tc[4] = self._twin(f"l{t}.w_skip_t", list(self.tensors[f"l{t}.w_skip_t"].reshape(-1, c, c)))
                layer.tc_img[4] = self._image_of(f"l{t}.w_skip_t")
            lin, lin_t, lin_blocks = [], [], []
            for l_out in range(spec.sh_lmax + 1):
                into = so3.paths_into(paths, l_out)
                norm = 1.0 / math.sqrt(len(into) * c) / spec.avg_num_neighbors
                block = torch.cat([w[f"l{t}.lin.{p}"] for p in into], dim=0) * norm   # [n_seg * C, C]
                lin.append(block.reshape(-1))
                lin_t.append(block.t().contiguous().reshape(-1))
                lin_blocks.append(block.to(torch.float32))
            layer.w_lin = self._put(f"l{t}.w_lin", torch.cat(lin))
            layer.w_lin_t = self._put(f"l{t}.w_lin_t", torch.cat(lin_t))
            layer.tc[5] = self._twin(f"l{t}.w_lin", lin_blocks)
            layer.tc_img[5] = self._image_of(f"l{t}.w_lin")
            layer.tc[6] = self._twin(f"l{t}.w_lin_t", [b.t().contiguous() for b in lin_blocks])
            layer.tc_img[6] = self._image_of(f"l{t}.w_lin_t")
            prod = torch.stack([w[f"l{t}.prod.{big_l}"] / math.sqrt(c) for big_l in range(spec.l_out_max(t) + 1)])
            layer.w_prod = self._put(f"l{t}.w_prod", prod)
            layer.w_prod_t = self._put(f"l{t}.w_prod_t", prod.transpose(1, 2))
            layer.tc[7] = self._twin(f"l{t}.w_prod", list(self.tensors[f"l{t}.w_prod"]))
            layer.tc_img[7] = self._image_of(f"l{t}.w_prod")
            layer.tc[8] = self._twin(f"l{t}.w_prod_t", list(self.tensors[f"l{t}.w_prod_t"]))
            layer.tc_img[8] = self._image_of(f"l{t}.w_prod_t")
            terms, coefs = contraction_terms(spec, weights, t, species_z)
            layer.n_sc_terms = len(terms)
            layer.sc_terms = self._put(f"l{t}.sc_terms", torch.from_numpy(terms), dtype=torch.int32)
            layer.sc_coef = self._put(f"l{t}.sc_coef", torch.from_numpy(coefs))
            if t < spec.num_interactions - 1:
                layer.w_readout = self._put(f"l{t}.readout", w[f"l{t}.readout"] / math.sqrt(c))
            else:
                ro = torch.cat([(w[f"l{t}.readout.0"] / math.sqrt(c)).reshape(-1),
                                w[f"l{t}.readout.1"] / math.sqrt(spec.mlp_hidden)])
                layer.w_readout = self._put(f"l{t}.readout", ro)
        self.struct = struct

    def _put(self, name: str, tensor: torch.Tensor, dtype=torch.float32) -> int:
        t = tensor.to(dtype).contiguous().to(self.device)
        self.tensors[name] = t
        return t.data_ptr()

    def _twin(self, name: str, blocks) -> int:
        """Tensor-core twin of fp32 [K][N] blocks that are already on the device (so the split is of the fp32 values
        the SIMT path reads)."""
        host = [b.cpu() for b in blocks]
        twin = tensor_core_twin(host).to(self.device)
        self.tensors[name + ".tc"] = twin
        self.tensors[name + ".img"] = tensor_core_image(host).to(self.device)
        return twin.data_ptr()

    def _image_of(self, name: str) -> int:
        return self.tensors[name + ".img"].data_ptr()

    def species_index(self, numbers) -> torch.Tensor:
        """[N] int32 index of each atom's species among the present ones."""
        table = np.full(128, -1, dtype=np.int32)
        for k, z in enumerate(self.species_z):
            table[z] = k
        index = table[np.asarray(numbers, dtype=np.int64)]
        if (index < 0).any():
            raise ValueError("an atom's species is not among the species the model was packed for")
        return torch.as_tensor(index, dtype=torch.int32, device=self.device)

    def pointer(self):
        return ctypes.byref(self.struct)


__all__ = ["PackedModel", "contraction_terms", "mlp_image", "radial_image", "tensor_core_image", "tensor_core_twin", "tf32_round"]
