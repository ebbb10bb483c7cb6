"""Host-side helpers of the block-scaled FFN: the power-of-two scale rule and the 512-byte scale-factor atoms
(byte (r % 32) * 16 + (r / 32) * 4 + slice of an atom = biased exponent of row r).  No GPU needed."""
import torch

from taac_2026_b200 import ops


def test_scale_is_the_smallest_power_of_two_that_fits():
    amax = torch.tensor([448.0, 448.0001, 449.0, 224.0, 223.9, 1.0, 0.0, 896.0, 3.0e38, 1e-30])
    e = ops.mx_scale_exponents(amax)
    scale = torch.ldexp(torch.ones(amax.shape), e)
    live = amax > 0
    assert bool((amax[live] / scale[live] <= 448.0).all())
    assert bool((amax[live] / (scale[live] / 2) > 448.0).all() | (e[live] == -126).any())
    assert e.tolist()[:8] == [0, 1, 1, -1, -1, -8, 0, 1]


def test_atoms_hold_every_row_at_its_offset():
    rows, k_blocks = 300, 3
    e = torch.randint(-20, 20, (rows, k_blocks), dtype=torch.int32)
    atoms = ops.mx_scale_atoms(e)
    assert atoms.shape == (3, k_blocks, 512) and atoms.dtype == torch.uint8
    for r in (0, 1, 31, 32, 33, 127, 128, 129, 299):
        tile, local = divmod(r, 128)
        off = (local % 32) * 16 + (local // 32) * 4
        for kb in range(k_blocks):
            assert atoms[tile, kb, off:off + 4].tolist() == [int(e[r, kb]) + 127] * 4
    local = 300 - 256                                                   # the first row past the end: its bytes stay zero
    assert atoms[2, :, (local % 32) * 16 + (local // 32) * 4].tolist() == [0] * k_blocks
    assert torch.equal(ops.mx_atoms_to_scales(atoms, rows), torch.ldexp(torch.ones(rows, k_blocks), e))


def test_weight_quantisation_round_trips_within_e4m3():
    g = torch.Generator().manual_seed(0)
    w = torch.randn(256, 384, generator=g) * torch.exp(torch.randn(2, 3, generator=g)).repeat_interleave(128, 0).repeat_interleave(128, 1)
    q, atoms = ops.quantize_weight_mx(w)
    assert q.dtype == torch.float8_e4m3fn and atoms.shape == (2, 3, 512)
    scale = torch.ldexp(torch.ones(2, 3), atoms[:, :, 0].to(torch.int32) - 127)
    back = q.float() * scale.repeat_interleave(128, 0).repeat_interleave(128, 1)
    # e4m3 keeps 3 mantissa bits: relative error at most 2^-4 for normal values
    big = w.abs() > w.abs().amax() * 2 ** -6
    assert bool(((back - w).abs()[big] <= w.abs()[big] * 2 ** -4 + 1e-12).all())
    assert float(q.float().abs().max()) <= 448.0
