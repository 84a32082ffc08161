"""Host-side packing of the tensor-core operands (no GPU): the images are permutations of the tf32 value / remainder
parts in the shared-memory operand layout, at the offsets the kernels compute."""
import numpy as np
import torch

from fastmace_b200.packing import mlp_image, radial_image, tensor_core_image, tensor_core_twin, tf32_round


def _tile_offset(row, k):
    """Float offset of (row, k) inside a [128][32] operand tile: 128-byte rows, 1024-byte groups of 8 rows, the 16-byte
    chunk index XORed with row mod 8 (tc_common.cuh: tile_offset)."""
    return (row >> 3) * 256 + (row & 7) * 32 + ((((k >> 2) & 7) ^ (row & 7)) << 2) + (k & 3)


def test_tf32_round_keeps_ten_mantissa_bits():
    x = torch.randn(1000)
    hi = tf32_round(x)
    assert torch.all((hi.view(torch.int32) & 0x1fff) == 0)
    assert torch.all((x - hi).abs() <= x.abs() * 2.0 ** -11 + 1e-30)


def test_image_is_the_twin_in_tile_order():
    torch.manual_seed(0)
    blocks = [torch.randn(64, 128), torch.randn(256, 384), torch.randn(128, 320)]   # the last has N % 128 != 0
    image = tensor_core_image(blocks)
    twin = tensor_core_twin(blocks)
    assert image.numel() == twin.numel() == sum(2 * b.numel() for b in blocks)
    offset = 0
    rng = np.random.default_rng(0)
    for block in blocks:
        k, n = block.shape
        part = image[2 * offset: 2 * offset + 2 * k * n]
        if n % 128:
            assert float(part.abs().max()) == 0.0
        else:
            bt = block.t().contiguous()
            hi = tf32_round(bt)
            lo = tf32_round(bt - hi)
            view = part.view(n // 128, k // 32, 2, 4096)
            for _ in range(200):
                col, row = int(rng.integers(n)), int(rng.integers(k))
                nt, r, kc, kk = col // 128, col % 128, row // 32, row % 32
                assert float(view[nt, kc, 0, _tile_offset(r, kk)]) == float(hi[col, row])
                assert float(view[nt, kc, 1, _tile_offset(r, kk)]) == float(lo[col, row])
        offset += k * n


def test_radial_image_pieces():
    torch.manual_seed(1)
    w4 = torch.randn(64, 3 * 128)
    image = radial_image(w4).view(3, 2, 2, 4096)          # [path][K half][remainder, value][tile]
    bt = w4.t().contiguous()
    hi = tf32_round(bt)
    lo = tf32_round(bt - hi)
    rng = np.random.default_rng(1)
    for _ in range(300):
        p, c, k = int(rng.integers(3)), int(rng.integers(128)), int(rng.integers(64))
        assert float(image[p, k // 32, 1, _tile_offset(c, k % 32)]) == float(hi[p * 128 + c, k])
        assert float(image[p, k // 32, 0, _tile_offset(c, k % 32)]) == float(lo[p * 128 + c, k])


def test_mlp_image_layers_at_the_offsets_the_edge_kernel_copies():
    """The three hidden radial layers as [64 outputs][K] operand tiles (halves of 32 K, 2,048 floats each; the row
    pattern of a 64-row tile is that of the first 64 rows of a 128-row one): first layer at float 0 (values) and 2,048
    (remainders) with K = 8 of the 32 columns filled, the 64 x 64 layers at 4,096 / 8,192 and 12,288 / 16,384."""
    torch.manual_seed(2)
    w0, w1, w2 = torch.randn(8, 64), torch.randn(64, 64), torch.randn(64, 64)
    image = mlp_image(w0, w1, w2)
    assert image.numel() == 20480
    rng = np.random.default_rng(2)
    bt = w0.t().contiguous()
    hi = tf32_round(bt)
    lo = tf32_round(bt - hi)
    for n in range(64):
        for k in range(32):
            want_hi = float(hi[n, k]) if k < 8 else 0.0
            want_lo = float(lo[n, k]) if k < 8 else 0.0
            assert float(image[_tile_offset(n, k)]) == want_hi
            assert float(image[2048 + _tile_offset(n, k)]) == want_lo
    for layer, w in enumerate((w1, w2)):
        bt = w.t().contiguous()
        hi = tf32_round(bt)
        lo = tf32_round(bt - hi)
        base = 4096 + layer * 8192
        for _ in range(300):
            n, k = int(rng.integers(64)), int(rng.integers(64))
            at = (k // 32) * 2048 + _tile_offset(n, k % 32)
            assert float(image[base + at]) == float(hi[n, k])
            assert float(image[base + 4096 + at]) == float(lo[n, k])
    # every float of the image is one of the parts (nothing written twice, nothing left over in the 64 x 64 layers)
    assert int((image[4096:] != 0).sum()) == int((tf32_round(w1) != 0).sum() + (tf32_round(w1 - tf32_round(w1)) != 0).sum()
                                                  + (tf32_round(w2) != 0).sum() + (tf32_round(w2 - tf32_round(w2)) != 0).sum())


def test_species_groups_cover_every_atom_once():
    from fastmace_b200.forcefield import B200ForceField
    species = np.array([0, 1, 1, 0, 2, 1, 0, 0, 0, 1], dtype=np.int32)
    groups = B200ForceField._species_groups(species, 4).numpy()
    atoms = groups[groups >= 0]
    assert sorted(atoms.tolist()) == list(range(len(species)))
    for row in groups:
        live = row[row >= 0]
        assert len(set(species[live].tolist())) == 1          # one species per group
        assert np.all(np.diff(live) > 0)                      # in index order
