"""Grouped bf16 GEMM with fused bias / SiLU / residual (`tb200_gemm_bf16_grouped`) against fp32 torch."""
import pytest
import torch

from taac_2026_b200 import ops

pytestmark = pytest.mark.gpu


def _reference(x, w, bias, silu, residual):
    y = torch.einsum("gmk,gnk->gmn", x.float(), w.float())
    if bias is not None:
        y = y + bias.float()[:, None, :]
    if silu:
        y = torch.nn.functional.silu(y)
    if residual is not None:
        y = y + residual.float()
    return y


def _close(got, want):
    # one rounding to bf16 of an fp32 result: half an ulp relative, plus the tanh-form SiLU (about 2^-11)
    err = (got.float() - want).abs()
    tol = 1e-2 * want.abs() + 1e-2
    assert bool((err <= tol).all()), float((err - tol).max())


@pytest.mark.parametrize("groups,rows,n,k", [(1, 128, 256, 64), (3, 200, 512, 128), (9, 1000, 2048, 512),
                                             (2, 77, 512, 2048), (9, 513, 1536, 512), (1, 5000, 512, 512)])
@pytest.mark.parametrize("silu", [False, True])
@pytest.mark.parametrize("with_bias", [False, True])
def test_grouped_linear(groups, rows, n, k, silu, with_bias):
    g = torch.Generator().manual_seed(groups * 1000 + rows)
    x = torch.randn(groups, rows, k, generator=g).bfloat16().cuda()
    w = (torch.randn(groups, n, k, generator=g) * k ** -0.5).bfloat16().cuda()
    bias = torch.randn(groups, n, generator=g).cuda() if with_bias else None
    got = ops.grouped_linear(x, w, bias, silu=silu, check=True)
    assert got.shape == (groups, rows, n) and got.dtype == torch.bfloat16
    _close(got, _reference(x, w, bias, silu, None))


@pytest.mark.parametrize("in_place", [False, True])
def test_grouped_linear_with_residual(in_place):
    g = torch.Generator().manual_seed(11)
    groups, rows, n, k = 9, 777, 512, 2048
    x = torch.randn(groups, rows, k, generator=g).bfloat16().cuda()
    w = (torch.randn(groups, n, k, generator=g) * k ** -0.5).bfloat16().cuda()
    bias = torch.randn(groups, n, generator=g).cuda()
    res = torch.randn(groups, rows, n, generator=g).bfloat16().cuda()
    want = _reference(x, w, bias, False, res)
    if in_place:
        got = ops.grouped_linear(x, w, bias, residual=res, out=res, check=True)
        assert got.data_ptr() == res.data_ptr()
    else:
        keep = res.clone()
        got = ops.grouped_linear(x, w, bias, residual=res, check=True)
        assert torch.equal(res, keep)
    _close(got, want)


def test_plain_linear_and_repeatability():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(3000, 512, generator=g).bfloat16().cuda()
    w = (torch.randn(1024, 512, generator=g) * 512 ** -0.5).bfloat16().cuda()
    b = torch.randn(1024, generator=g).cuda()
    got = ops.grouped_linear(x, w, b, check=True)
    assert got.shape == (3000, 1024)
    _close(got[None], _reference(x[None], w[None], b[None], False, None))
    assert torch.equal(got, ops.grouped_linear(x, w, b))          # same bits on every run
    # many tiles per CTA: both TMEM buffers and every ring stage wrap around several times
    x = torch.randn(2, 40000, 64, generator=g).bfloat16().cuda()
    w = (torch.randn(2, 256, 64, generator=g) * 0.125).bfloat16().cuda()
    _close(ops.grouped_linear(x, w, check=True), _reference(x, w, None, False, None))


def test_grouped_linear_rejects_unsupported_shapes():
    x = torch.zeros(1, 8, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        ops.grouped_linear(x, torch.zeros(1, 100, 64, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):
        ops.grouped_linear(torch.zeros(1, 8, 48, dtype=torch.bfloat16, device="cuda"),
                           torch.zeros(1, 256, 48, dtype=torch.bfloat16, device="cuda"))
    empty = ops.grouped_linear(torch.zeros(2, 0, 64, dtype=torch.bfloat16, device="cuda"),
                               torch.zeros(2, 256, 64, dtype=torch.bfloat16, device="cuda"))
    assert empty.shape == (2, 0, 256)


@pytest.mark.parametrize("groups,rows,n,k", [(1, 100, 256, 64), (1, 128, 512, 128), (2, 300, 1024, 512), (1, 5000, 4096, 512)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_gated_epilogue(groups, rows, n, k, with_bias):
    """act 2: the weight rows of every 256-column tile are [128 gate rows | 128 value rows]; out = silu(gate) * value.
    Rows up to 128 take the single-CTA kernel, more rows the CTA-pair kernel."""
    g = torch.Generator().manual_seed(groups * 77 + rows)
    x = torch.randn(groups, rows, k, generator=g).bfloat16().cuda()
    w = (torch.randn(groups, n, k, generator=g) * k ** -0.5).bfloat16().cuda()
    bias = torch.randn(groups, n, generator=g).cuda() if with_bias else None
    got = ops.grouped_linear(x, w, bias, gated=True, check=True)
    assert got.shape == (groups, rows, n // 2) and got.dtype == torch.bfloat16
    full = _reference(x, w, bias, False, None).view(groups, rows, n // 256, 2, 128)
    want = (torch.nn.functional.silu(full[:, :, :, 0]) * full[:, :, :, 1]).reshape(groups, rows, n // 2)
    _close(got, want)
    with pytest.raises(ValueError):
        ops.grouped_linear(x, w, bias, gated=True, residual=got)
