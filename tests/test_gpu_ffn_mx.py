"""FP8 FFN with power-of-two block scales on the block-scaled tensor-core instruction (`tb200_quant_act_mx`,
`tb200_mx_gemm`) against a torch emulation of the same quantised arithmetic, and against the bf16 FFN.  The reference
has no FP8 path: parity is against the emulation (unpinned), the error against the bf16 FFN is reported as measured."""
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


def _dequant_act(q, atoms):
    rows, k = q.shape
    scales = ops.mx_atoms_to_scales(atoms, rows)                     # [rows, K / 128]
    return q.float() * scales.repeat_interleave(128, dim=1)


def _dequant_weight(q, atoms):
    n, k = q.shape
    exps = atoms[:, :, 0].to(torch.int32) - 127                      # one scale per 128 x 128 block
    scale = torch.ldexp(torch.ones_like(exps, dtype=torch.float32), exps)
    return q.float() * scale.repeat_interleave(128, dim=0).repeat_interleave(128, dim=1)


def _emulate_quant(x):
    blocks = x.float().view(x.shape[0], -1, 128)
    exps = ops.mx_scale_exponents(blocks.abs().amax(dim=2))
    scale = torch.ldexp(torch.ones_like(exps, dtype=torch.float32), exps)
    q = (blocks / scale[:, :, None]).clamp(-448, 448).reshape(x.shape).to(torch.float8_e4m3fn)
    return q, exps


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


@pytest.mark.parametrize("rows,k", [(128, 128), (300, 512), (4096, 2048)])
def test_activation_quantisation_matches_the_emulation(rows, k):
    g = torch.Generator(device="cuda").manual_seed(rows + k)
    x = (torch.randn(rows, k, generator=g, device="cuda") * torch.exp(2 * torch.randn(rows, 1, generator=g, device="cuda"))).bfloat16()
    x[1] = 0                                                         # an all-zero row: scale 1, codes 0
    q, atoms = ops.quantize_activation_mx(x)
    want_q, want_e = _emulate_quant(x)
    assert torch.equal(q.view(torch.uint8), want_q.view(torch.uint8))
    assert torch.equal(atoms, ops.mx_scale_atoms(want_e))


@pytest.mark.parametrize("rows,n,k", [(128, 256, 128), (200, 512, 512), (1000, 256, 2048), (4096, 4096, 512)])
@pytest.mark.parametrize("with_res", [False, True])
def test_linear_mode_applies_every_scale(rows, n, k, with_res):
    """Rows and weight blocks of very different magnitude: a scale factor applied to the wrong row, column block or
    K block would show at once."""
    g = torch.Generator(device="cuda").manual_seed(rows + n + k)
    x = (torch.randn(rows, k, generator=g, device="cuda") * torch.exp(2 * torch.randn(rows, k // 128, generator=g, device="cuda")
                                                                 .repeat_interleave(128, dim=1))).bfloat16()
    w = torch.randn(n, k, generator=g, device="cuda") * k ** -0.5
    w = w * torch.exp(1.5 * torch.randn(n // 128, k // 128, generator=g, device="cuda")).repeat_interleave(128, 0).repeat_interleave(128, 1)
    bias = torch.randn(n, generator=g, device="cuda")
    res = torch.randn(rows, n, generator=g, device="cuda").bfloat16() if with_res else None
    xq, xa = ops.quantize_activation_mx(x)
    wq, wa = ops.quantize_weight_mx(w)
    got = ops.mx_gemm(xq, xa, wq, wa, mode="linear", bias=bias, residual=res, check=True)
    want = _dequant_act(xq, xa) @ _dequant_weight(wq, wa).t() + bias
    if with_res:
        want = want + res.float()
    assert got.shape == (rows, n) and got.dtype == torch.bfloat16
    err = (got.float() - want).abs()
    assert bool((err <= 1e-2 * want.abs() + 1e-2 * want.abs().mean()).all()), float(err.max())
    assert torch.equal(got, ops.mx_gemm(xq, xa, wq, wa, mode="linear", bias=bias, residual=res))     # same bits on every run


@pytest.mark.parametrize("gated", [True, False])
@pytest.mark.parametrize("rows,d,hidden", [(256, 512, 2048), (1000, 256, 512), (5000, 512, 2048)])
def test_ffn_matches_the_emulation_and_reports_the_error_against_bf16(gated, rows, d, hidden):
    g = torch.Generator(device="cuda").manual_seed(rows + d)
    x = torch.randn(rows, d, generator=g, device="cuda").bfloat16()
    w_up = (torch.randn((2 if gated else 1) * hidden, d, generator=g, device="cuda") * 0.02).bfloat16()
    w_down = (torch.randn(d, hidden, generator=g, device="cuda") * 0.02).bfloat16()
    b_up = torch.randn(w_up.shape[0], generator=g, device="cuda") * 0.1
    b_down = torch.randn(d, generator=g, device="cuda") * 0.1
    weights = ops.MxFfnWeights(w_up, w_down, gated=gated, b_up=b_up, b_down=b_down)
    y = ops.ffn_mx(x, weights, check=True)
    # emulation with the same codes: GEMM 1 on the dequantised operands, activation, re-quantisation, GEMM 2
    xq, xa = ops.quantize_activation_mx(x)
    pre = _dequant_act(xq, xa) @ _dequant_weight(weights.w_up, weights.a_up).t() + weights.b_up
    if gated:
        pre = pre.view(rows, hidden // 128, 2, 128)
        h = (torch.nn.functional.silu(pre[:, :, 0]) * pre[:, :, 1]).reshape(rows, hidden)
    else:
        h = torch.nn.functional.silu(pre)
    hq, he = _emulate_quant(h)
    h_hat = hq.float() * torch.ldexp(torch.ones_like(he, dtype=torch.float32), he).repeat_interleave(128, dim=1)
    want = h_hat @ _dequant_weight(weights.w_down, weights.a_down).t() + b_down
    assert _rel(y, want) <= 1e-2            # tanh-form SiLU and code flips at rounding boundaries of the hidden activation
    # against the bf16 FFN: the error of four e4m3 roundings (reported, bounded by the measured floor)
    pre16 = x.float() @ w_up.float().t() + b_up
    if gated:
        ref = (torch.nn.functional.silu(pre16[:, :hidden]) * pre16[:, hidden:]) @ w_down.float().t() + b_down
    else:
        ref = torch.nn.functional.silu(pre16) @ w_down.float().t() + b_down
    assert _rel(y, ref) <= 7.5e-2
