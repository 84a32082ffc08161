"""MACE model description and weights for the B200 force path.

``MaceSpec`` holds the hyper-parameters the benchmark configurations name (channels, hidden irreps, l_max of the
spherical harmonics, correlation order, cutoff, Bessel functions, radial MLP widths, 89 elements).
``init_weights`` draws a random-initialised ScaleShiftMACE in the parametrisation of mace-torch 0.3.16 / e3nn 0.4.4
(the third-party model behind FastMACE's ``MACEForceField``; constructor arguments as in the reference fixture
``tests/_support/tiny_models.py:95-113``): every learnable tensor is standard normal (symmetric-contraction weights
divided by their count), and all normalisation (1/sqrt(fan_in), second-moment normalised SiLU, path normalisation,
``avg_num_neighbors``) is applied when the model is evaluated, not stored in the tensors.

The model structure (reference: ``fastmace/rewrites/generic/modules.py:381-505`` for the interaction,
``fastmace/model/energy.py:92-99`` for the energy sum):

    h0 = emb[z] / sqrt(89)
    for each layer t:
        sc      = skip_t(h_t, z)                               species-dependent linear, per irrep
        x       = linear_up_t(h_t)                             per irrep, C x C
        w_e     = radial_mlp_t(bessel(r_e) * cutoff(r_e))      8 -> 64 -> 64 -> 64 -> P*C, SiLU, no bias
        M_i     = sum_{e -> i} conv_tp(x[sender_e], Y_e, w_e)  channelwise ("uvu"), one output segment per path
        m_i     = linear_t(M_i) / avg_num_neighbors            per output irrep, K = (paths into l) * C
        B_i     = symmetric_contraction_t(m_i, z_i)            correlation 3, species-dependent weights
        h_{t+1} = product_linear_t(B_i) + sc
        e_i    += readout_t(h_{t+1})                           linear; last layer 128 -> 16 -> SiLU -> 1
    E = sum_i E0[z_i] (float64) + sum_i (scale * e_i + shift)
"""

from __future__ import annotations

import dataclasses
import math

import numpy as np
import torch

from . import so3


def _silu_second_moment_constant() -> float:
    """1 / sqrt(E[silu(z)^2]) for z ~ N(0, 1): e3nn's ``normalize2mom`` constant, by quadrature (e3nn estimates it
    from 1e6 seeded samples, 1.679...; the exact integral is used here)."""
    z = np.linspace(-12.0, 12.0, 240001)
    silu = z / (1.0 + np.exp(-z))
    pdf = np.exp(-0.5 * z * z) / math.sqrt(2.0 * math.pi)
    f = silu * silu * pdf
    dz = z[1] - z[0]
    second = float((f.sum() - 0.5 * (f[0] + f[-1])) * dz)
    return 1.0 / math.sqrt(second)


SILU_NORM = _silu_second_moment_constant()


@dataclasses.dataclass(frozen=True)
class MaceSpec:
    channels: int = 128
    hidden_lmax: int = 1            # hidden irreps 128x0e [+128x1o [+128x2e]]
    sh_lmax: int = 3
    correlation: int = 3
    num_interactions: int = 2
    r_cut: float = 6.0
    num_bessel: int = 8
    cutoff_p: int = 5
    radial_hidden: tuple = (64, 64, 64)
    num_elements: int = 89          # atomic numbers 1..89, one-hot
    mlp_hidden: int = 16
    avg_num_neighbors: float = 32.0
    scale: float = 1.0
    shift: float = 0.0

    def l_in_max(self, layer: int) -> int:
        return 0 if layer == 0 else self.hidden_lmax

    def l_out_max(self, layer: int) -> int:
        return self.hidden_lmax if layer < self.num_interactions - 1 else 0

    def paths(self, layer: int):
        return so3.tp_paths(self.l_in_max(layer), self.sh_lmax, self.sh_lmax)

    def in_dim(self, layer: int) -> int:
        return (self.l_in_max(layer) + 1) ** 2

    def out_dim(self, layer: int) -> int:
        return (self.l_out_max(layer) + 1) ** 2

    def skip_lmax(self, layer: int) -> int:
        return min(self.l_in_max(layer), self.l_out_max(layer))


SMALL = MaceSpec(hidden_lmax=0)
MEDIUM = MaceSpec(hidden_lmax=1)
LARGE = MaceSpec(hidden_lmax=2)
SPECS = {"small": SMALL, "medium": MEDIUM, "large": LARGE}


def init_weights(spec: MaceSpec, seed: int, dtype=torch.float32) -> dict[str, torch.Tensor]:
    """Random-initialised weights: standard normal draws from ``torch.Generator().manual_seed(seed)`` in float64, in
    the order of the keys below, then cast to ``dtype`` (the model precision)."""
    g = torch.Generator().manual_seed(int(seed))
    c = spec.channels

    def randn(*shape):
        return torch.randn(*shape, generator=g, dtype=torch.float64)

    w: dict[str, torch.Tensor] = {"emb": randn(spec.num_elements, c)}
    for t in range(spec.num_interactions):
        paths = spec.paths(t)
        for l in range(spec.l_in_max(t) + 1):
            w[f"l{t}.up.{l}"] = randn(c, c)
        widths = (spec.num_bessel, *spec.radial_hidden, len(paths) * c)
        for i in range(len(widths) - 1):
            w[f"l{t}.rad.{i}"] = randn(widths[i], widths[i + 1])
        for p in range(len(paths)):
            w[f"l{t}.lin.{p}"] = randn(c, c)
        for l in range(spec.skip_lmax(t) + 1):
            w[f"l{t}.skip.{l}"] = randn(c, spec.num_elements, c)
        for big_l in range(spec.l_out_max(t) + 1):
            for nu in range(1, spec.correlation + 1):
                k = so3.num_contraction_weights(nu, big_l, spec.sh_lmax)
                w[f"l{t}.sc.{big_l}.{nu}"] = randn(spec.num_elements, k, c) / k
            w[f"l{t}.prod.{big_l}"] = randn(c, c)
        if t < spec.num_interactions - 1:
            w[f"l{t}.readout"] = randn(c)
        else:
            w[f"l{t}.readout.0"] = randn(c, spec.mlp_hidden)
            w[f"l{t}.readout.1"] = randn(spec.mlp_hidden)
    return {k: v.to(dtype) for k, v in w.items()}


def e0_table(spec: MaceSpec) -> np.ndarray:
    """Isolated-atom energies per element, float64. The benchmark models are random-initialised with zero E0."""
    return np.zeros(spec.num_elements, dtype=np.float64)


__all__ = ["MaceSpec", "SMALL", "MEDIUM", "LARGE", "SPECS", "init_weights", "e0_table", "SILU_NORM"]
