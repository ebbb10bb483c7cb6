"""GPU parity of the FP8 block-scaled FFN (activation quantisation + two tcgen05 GEMMs with fused
epilogues), called through the C ABI.

Two checks per case: (1) a tight bound against a CPU emulation of the same quantised arithmetic fed
with the same weight codes, which would expose any descriptor / layout / scale-indexing mistake, and
(2) accuracy against the bf16 / fp32 torch FFN: max-abs error <= 1e-1 of the output range, and an
L2-relative error that equals the emulation's own (the format's floor, about 6e-2 for a gated FFN on
i.i.d. inputs: three mantissa bits per operand leave no room under 5e-2 in that norm).  The reference project has no FP8 path, so there is no golden vector: parity of
this operator is pinned by these two oracles only.
"""

from __future__ import annotations

import pytest
import torch

from conftest import gpu_ready
from oracle import reference_ops as R
from taac_2026_b200 import ops

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_gpu():
    if not gpu_ready():
        pytest.fail("gpu tests need an sm_100 device and a built libtb200.so")


def _activations(m, d, seed):
    """N(0,1) with 1 % Student-t(4) * 3 outliers, as bf16."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, d, generator=g)
    t4 = torch.randn(m, d, generator=g) / torch.sqrt(torch.randn(m, d, 4, generator=g).pow(2).mean(-1))
    x = torch.where(torch.rand(m, d, generator=g) < 0.01, 3.0 * t4, x)
    return x.bfloat16()


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm()).item()


def test_activation_quantisation_bit_exact():
    x = _activations(300, 512, 0)
    x[5] = 0  # an all-zero row: scale 1, zeros
    q, s = ops.quantize_activation_1x128(x.cuda())
    want_q, want_s = R.quantize_blocks_reciprocal(x.float())
    assert torch.equal(s.cpu(), want_s)
    assert torch.equal(q.cpu().float(), want_q)


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (257, 512, 384), (1000, 256, 2048), (64, 1024, 512)])
def test_linear_gemm_matches_emulation(m, n, k):
    g = torch.Generator().manual_seed(m + n + k)
    a = _activations(m, k, 1)
    w = (torch.randn(n, k, generator=g) * 0.02).bfloat16()
    bias = torch.randn(n, generator=g) * 0.1
    res = torch.randn(m, n, generator=g).bfloat16()
    qa, sa = ops.quantize_activation_1x128(a.cuda())
    qw, sw = ops.quantize_weight_128x128(w.cuda())
    got = ops.fp8_gemm(qa, sa, qw, sw, mode="linear", bias=bias.cuda(), residual=res.cuda(), check=True).cpu()
    ea, esa = R.quantize_blocks_reciprocal(a.float())
    ew, esw = qw.cpu().float(), sw.cpu()  # the device-side weight quantisation (plain tensor ops) is the input here
    ref_w, ref_sw = R.quantize_blocks(w, 128, 128)
    torch.testing.assert_close(esw, ref_sw, rtol=1e-6, atol=0)
    assert (ew != ref_w).float().mean().item() < 1e-2  # a 1-ulp scale difference may move a few roundings
    want = (R.block_scaled_matmul(ea, esa, ew, esw) + bias + res.float()).bfloat16()
    assert (got.float() - want.float()).abs().max().item() <= 2e-2 * want.float().abs().max().item() + 1e-3
    assert _rel(got, want) <= 3e-3


def _weight_codes(weights: ops.Fp8FfnWeights, hidden: int):
    """The kernel's own e4m3 weight codes, back in the original row order, for the emulation."""
    q_up, s_up = weights.w_up.cpu().float(), weights.s_up.cpu()
    if weights.gated:  # undo the per-128-block [gate | value] interleave
        k = q_up.shape[1]
        q_up = q_up.view(hidden // 128, 2, 128, k).transpose(0, 1).reshape(2 * hidden, k)
        s_up = s_up.view(hidden // 128, 2, -1).transpose(0, 1).reshape(2 * hidden // 128, -1)
    return (q_up, s_up), (weights.w_down.cpu().float(), weights.s_down.cpu())


@pytest.mark.parametrize("gated", [True, False])
@pytest.mark.parametrize("m,d,hidden", [(128, 512, 2048), (333, 256, 512), (1, 512, 2048), (4100, 512, 2048)])
def test_ffn_matches_emulation_and_bf16_reference(gated, m, d, hidden):
    g = torch.Generator().manual_seed(d + hidden + m)
    x = _activations(m, d, 2)
    w_up = (torch.randn((2 if gated else 1) * hidden, d, generator=g) * 0.02).bfloat16()
    w_down = (torch.randn(d, hidden, generator=g) * 0.02).bfloat16()
    b_up = None if gated else torch.randn(hidden, generator=g) * 0.05
    b_down = None if gated else torch.randn(d, generator=g) * 0.05
    weights = ops.Fp8FfnWeights(w_up.cuda(), w_down.cuda(), gated=gated, b_up=None if b_up is None else b_up.cuda(),
                                b_down=None if b_down is None else b_down.cuda())
    got = ops.ffn_fp8(x.cuda(), weights, check=True).cpu()
    assert got.shape == (m, d) and got.dtype == torch.bfloat16
    emu = R.fp8_ffn_emulated(x, w_up, w_down, gated=gated, b_up=b_up, b_down=b_down,
                             quantized_weights=_weight_codes(weights, hidden))
    ref = R.swiglu_ffn(x, w_up, w_down) if gated else R.silu_ffn(x, w_up, b_up, w_down, b_down)
    # (1) the kernel computes the quantised arithmetic it claims to (same weight codes on both sides)
    assert _rel(got, emu) <= 5e-3, "kernel disagrees with the emulated quantised arithmetic"
    # (2) accuracy against the unquantised FFN.  e4m3 keeps 3 mantissa bits, i.e. about 2.6 % rms rounding
    # error per operand whatever the block scale; through x, W_up (twice for a gate), the re-quantised
    # hidden and W_down that floor is about 6 % for the gated and 5 % for the plain FFN on i.i.d. data.
    # The emulation sits on the same floor, so the kernel adds nothing beyond the format itself.
    floor = _rel(emu, ref)
    assert abs(_rel(got, ref) - floor) <= 2e-3
    assert _rel(got, ref) <= 7e-2
    assert (got.float() - ref).abs().max().item() <= 1e-1 * ref.abs().max().item() + 1e-3


def test_gate_in_second_half_and_residual():
    g = torch.Generator().manual_seed(9)
    x = _activations(200, 256, 3)
    w_up = (torch.randn(1024, 256, generator=g) * 0.02).bfloat16()
    w_down = (torch.randn(256, 512, generator=g) * 0.02).bfloat16()
    res = torch.randn(200, 256, generator=g).bfloat16()
    weights = ops.Fp8FfnWeights(w_up.cuda(), w_down.cuda(), gated=True, gate_first=False)
    got = ops.ffn_fp8(x.cuda(), weights, residual=res.cuda(), check=True).cpu()
    ref = R.swiglu_ffn(x, w_up, w_down, gate_first=False) + res.float()
    assert _rel(got.float() - res.float(), ref - res.float()) <= 1e-1  # the residual itself is exact; see the floor above


def test_full_size_block_against_bf16_torch_on_device():
    """262 144 tokens, 512 -> 2 x 2048 -> 512 (the benchmark shape), compared on the device with the
    bf16 torch FFN: relative error of the whole output and of every 4 096-row slab."""
    m, d, hidden = 262144, 512, 2048
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(m, d, generator=g, device="cuda")
    t4 = torch.randn(m, d, generator=g, device="cuda") / torch.sqrt(torch.randn(m, d, 4, generator=g, device="cuda").pow(2).mean(-1))
    x = torch.where(torch.rand(m, d, generator=g, device="cuda") < 0.01, 3.0 * t4, x).bfloat16()
    w_up = (torch.randn(2 * hidden, d, generator=g, device="cuda") * 0.02).bfloat16()
    w_down = (torch.randn(d, hidden, generator=g, device="cuda") * 0.02).bfloat16()
    weights = ops.Fp8FfnWeights(w_up, w_down, gated=True)
    got = ops.ffn_fp8(x, weights, check=True).float()
    h = torch.nn.functional.linear(x, w_up)
    ref = torch.nn.functional.linear(torch.nn.functional.silu(h[:, :hidden]) * h[:, hidden:], w_down).float()
    assert ((got - ref).norm() / ref.norm()).item() <= 7e-2  # the e4m3 floor of a gated FFN, see above
    slab = ((got - ref).view(64, -1).norm(dim=1) / ref.view(64, -1).norm(dim=1)).max().item()
    assert slab <= 7e-2
    assert (got - ref).abs().max().item() <= 1e-1 * ref.abs().max().item()


@pytest.mark.parametrize("gated", [True, False])
@pytest.mark.parametrize("m,d,hidden", [(300, 256, 512), (4100, 512, 2048)])
def test_precise_mode_meets_the_5e_2_bound(gated, m, d, hidden):
    """`precise=True`: the up projection runs on the bf16 tensor cores (bias, SiLU and the gate in its epilogue), its
    bf16 hidden activation is quantised per 1 x 128 block, the down projection is e4m3.  Only the hidden activation
    and W_down are rounded to e4m3, which leaves 3.5e-2 (gated) / 3.6e-2 (plain) against the bf16 FFN: inside the
    5e-2 bound that the all-e4m3 mode misses for the gated layer."""
    g = torch.Generator().manual_seed(d + hidden + m)
    x = _activations(m, d, 2)
    w_up = (torch.randn((2 if gated else 1) * hidden, d, generator=g) * 0.02).bfloat16()
    w_down = (torch.randn(d, hidden, generator=g) * 0.02).bfloat16()
    b_up = torch.randn((2 if gated else 1) * hidden, generator=g) * 0.05
    b_down = torch.randn(d, generator=g) * 0.05
    res = torch.randn(m, d, generator=g).bfloat16()
    weights = ops.Fp8FfnWeights(w_up.cuda(), w_down.cuda(), gated=gated, b_up=b_up.cuda(), b_down=b_down.cuda(), precise=True)
    got = ops.ffn_fp8(x.cuda(), weights, residual=res.cuda(), check=True, precise=True).float().cpu()
    ref = (R.swiglu_ffn(x, w_up, w_down, b_up=b_up, b_down=b_down) if gated else R.silu_ffn(x, w_up, b_up, w_down, b_down))
    rel = _rel(got - res.float(), ref)
    assert rel <= 5e-2, rel
    coarse = ops.ffn_fp8(x.cuda(), weights, residual=res.cuda(), check=True).float().cpu()
    assert rel < _rel(coarse - res.float(), ref)          # and it is what buys the accuracy
    with pytest.raises(ValueError):
        ops.ffn_fp8(x.cuda(), ops.Fp8FfnWeights(w_up.cuda(), w_down.cuda(), gated=gated), precise=True)


def test_full_size_block_precise_mode_on_device():
    """The benchmark shape (262 144 tokens, 512 -> 2 x 2048 -> 512, SiLU-gated) in the precise mode: relative error of
    the whole output and of every 4 096-row slab against the bf16 torch FFN within 5e-2."""
    m, d, hidden = 262144, 512, 2048
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(m, d, generator=g, device="cuda")
    t4 = torch.randn(m, d, generator=g, device="cuda") / torch.sqrt(torch.randn(m, d, 4, generator=g, device="cuda").pow(2).mean(-1))
    x = torch.where(torch.rand(m, d, generator=g, device="cuda") < 0.01, 3.0 * t4, x).bfloat16()
    del t4
    w_up = (torch.randn(2 * hidden, d, generator=g, device="cuda") * 0.02).bfloat16()
    w_down = (torch.randn(d, hidden, generator=g, device="cuda") * 0.02).bfloat16()
    weights = ops.Fp8FfnWeights(w_up, w_down, gated=True, precise=True)
    got = ops.ffn_fp8(x, weights, check=True, precise=True).float()
    h = torch.nn.functional.linear(x, w_up)
    ref = torch.nn.functional.linear(torch.nn.functional.silu(h[:, :hidden]) * h[:, hidden:], w_down).float()
    del h
    assert ((got - ref).norm() / ref.norm()).item() <= 5e-2
    slab = ((got - ref).view(64, -1).norm(dim=1) / ref.view(64, -1).norm(dim=1)).max().item()
    assert slab <= 5e-2


def test_random_shapes_against_bf16_math():
    """Seeded sweep over row counts (tile tails), K, hidden widths, gating, biases and the residual: the whole FFN
    against the same layer in fp32 math on the bf16 operands, within the e4m3 noise floor (about 6e-2 relative)."""
    g = torch.Generator().manual_seed(77)
    for case in range(8):
        m = int(torch.randint(1, 700, (1,), generator=g))
        k = 128 * int(torch.randint(1, 6, (1,), generator=g))
        hidden = 256 * int(torch.randint(1, 4, (1,), generator=g))
        gated = bool(torch.randint(0, 2, (1,), generator=g))
        x = torch.randn(m, k, generator=g).bfloat16()
        w_up = (torch.randn((2 if gated else 1) * hidden, k, generator=g) * 0.05).bfloat16()
        w_down = (torch.randn(256, hidden, generator=g) * 0.05).bfloat16()
        b_up = (0.1 * torch.randn((2 if gated else 1) * hidden, generator=g)).bfloat16()
        b_down = (0.1 * torch.randn(256, generator=g)).bfloat16()
        res = torch.randn(m, 256, generator=g).bfloat16()
        weights = ops.Fp8FfnWeights(w_up.cuda(), w_down.cuda(), gated=gated, b_up=b_up.cuda(), b_down=b_down.cuda())
        got = ops.ffn_fp8(x.cuda(), weights, residual=res.cuda(), check=True).float().cpu()
        up = x.float() @ w_up.float().t() + b_up.float()
        h = torch.nn.functional.silu(up[:, :hidden]) * up[:, hidden:] if gated else torch.nn.functional.silu(up)
        want = res.float() + h @ w_down.float().t() + b_down.float()
        delta = want - res.float()
        rel = ((got - want).norm() / delta.norm().clamp_min(1e-6)).item()
        assert rel <= 9e-2, f"case {case}: m{m} k{k} hidden{hidden} gated={gated}: relative error {rel}"
