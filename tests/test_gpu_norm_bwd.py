"""RMSNorm / LayerNorm backward kernels against torch autograd of the fp32 closed forms, called through the C ABI.
Tolerances follow the reference's own GPU tests of its accelerated norms
(tests/gpu/infrastructure/accelerators/test_tilelang_ops_cuda.py:187-306: 1e-2 for the backward of 16-bit inputs)."""

from __future__ import annotations

import pytest
import torch

from conftest import gpu_ready
from taac_2026_b200 import ops

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_gpu():
    if not gpu_ready():
        pytest.fail("gpu tests need an sm_100 device and a built libtb200.so")


def _inputs(rows, cols, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    x[: max(1, rows // 100)] *= 50.0                      # outlier rows, as in the forward sweep
    w = 1 + 0.1 * torch.randn(cols, generator=g)
    b = 0.1 * torch.randn(cols, generator=g)
    dy = torch.randn(rows, cols, generator=g)
    return x.to(dtype), w.to(dtype), b.to(dtype), dy.to(dtype)


def _close(got, want, tol):
    scale = want.abs().max().clamp_min(1e-6)
    assert ((got.float().cpu() - want).abs().max() / scale).item() <= tol


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 1e-2), (torch.float16, 1e-2), (torch.float32, 1e-4)])
@pytest.mark.parametrize("rows,cols", [(1, 128), (77, 8), (300, 64), (1000, 128), (513, 256), (4096, 512), (257, 1024), (33, 384)])
def test_rms_norm_backward(dtype, tol, rows, cols):
    if dtype == torch.float32 and cols > 512:
        pytest.skip("the fp32 kernel takes at most 512 columns")
    x, w, _b, dy = _inputs(rows, cols, dtype, rows + cols)
    xr, wr = x.float().requires_grad_(), w.float().requires_grad_()
    y = xr * torch.rsqrt(xr.pow(2).mean(dim=-1, keepdim=True) + 1e-6) * wr
    y.backward(dy.float())
    dx, dw = ops.rms_norm_backward(x.cuda(), w.cuda(), dy.cuda(), 1e-6)
    assert dx.dtype == dtype and dw.dtype == dtype and dx.shape == x.shape
    _close(dx, xr.grad, tol)
    _close(dw, wr.grad, tol)


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 1e-2), (torch.float32, 1e-4)])
@pytest.mark.parametrize("rows,cols", [(1, 128), (77, 8), (1000, 128), (4096, 512), (257, 1024), (33, 384)])
def test_layer_norm_backward(dtype, tol, rows, cols):
    if dtype == torch.float32 and cols > 512:
        pytest.skip("the fp32 kernel takes at most 512 columns")
    x, w, b, dy = _inputs(rows, cols, dtype, rows * 3 + cols)
    xr, wr, br = x.float().requires_grad_(), w.float().requires_grad_(), b.float().requires_grad_()
    torch.nn.functional.layer_norm(xr, (cols,), wr, br, 1e-5).backward(dy.float())
    dx, dw, db = ops.layer_norm_backward(x.cuda(), w.cuda(), b.cuda(), dy.cuda(), 1e-5)
    _close(dx, xr.grad, tol)
    _close(dw, wr.grad, tol)
    _close(db, br.grad, tol)


def test_norms_are_differentiable_and_repeatable():
    """`ops.rms_norm` / `ops.layer_norm` under autograd run both directions on this library's kernels; the sums of the
    weight gradients run in a fixed order, so two calls give the same bits."""
    x, w, b, dy = _inputs(2000, 512, torch.bfloat16, 5)
    xc, wc, bc = x.cuda().requires_grad_(), w.cuda().requires_grad_(), b.cuda().requires_grad_()
    ops.rms_norm(xc, wc, 1e-6).backward(dy.cuda())
    first = (xc.grad.clone(), wc.grad.clone())
    xc.grad = wc.grad = None
    ops.rms_norm(xc, wc, 1e-6).backward(dy.cuda())
    assert torch.equal(first[0], xc.grad) and torch.equal(first[1], wc.grad)
    xr, wr = x.float().requires_grad_(), w.float().requires_grad_()
    (xr * torch.rsqrt(xr.pow(2).mean(dim=-1, keepdim=True) + 1e-6) * wr).backward(dy.float())
    _close(xc.grad, xr.grad, 1e-2)
    xc.grad = None
    ops.layer_norm(xc, wc, bc, 1e-5).backward(dy.cuda())
    assert xc.grad is not None and bc.grad is not None
    # shapes the backward kernel does not take are still refused rather than silently cut off from autograd
    wide = torch.randn(4, 2048, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    with pytest.raises(RuntimeError, match="forward-only"):
        ops.rms_norm(wide, torch.ones(2048, device="cuda", dtype=torch.bfloat16))


def test_full_size_rows():
    """65 536 rows x 512 bf16 (the forward sweep's shape): dx of every row and the column sums."""
    x, w, b, dy = _inputs(65536, 512, torch.bfloat16, 1)
    dx, dw, db = ops.layer_norm_backward(x.cuda(), w.cuda(), b.cuda(), dy.cuda(), 1e-5)
    xr, wr, br = x.float().cuda().requires_grad_(), w.float().cuda().requires_grad_(), b.float().cuda().requires_grad_()
    torch.nn.functional.layer_norm(xr, (512,), wr, br, 1e-5).backward(dy.float().cuda())
    _close(dx, xr.grad.cpu(), 1e-2)
    _close(dw, wr.grad.cpu(), 1e-2)
    _close(db, br.grad.cpu(), 1e-2)
