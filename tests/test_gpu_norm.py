"""GPU parity of the fused RMSNorm / LayerNorm kernels, called through the C ABI.

Oracle: the fp32 restatements in ``oracle/reference_ops.py`` (pinned to the reference) and the
committed golden outputs of the reference's torch path.  Tolerances: bf16/fp16 max-abs <= 2e-2
against the fp32-computed value (the bound the reference's benchmark applies to bf16,
src/taac2026/application/benchmarking/pcvr_tilelang_ops_benchmark.py:177-184); fp32 <= 2e-5.
"""

from __future__ import annotations

import pytest
import torch

from conftest import bf16_from_bits, gpu_ready
from oracle import reference_ops as R
from taac_2026_b200 import ops

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2, torch.float16: 5e-3}


@pytest.fixture(autouse=True)
def _need_gpu():
    if not gpu_ready():
        pytest.fail("gpu tests need an sm_100 device and a built libtb200.so")


def _inputs(rows, cols, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    n_out = max(1, rows // 100)
    x[torch.randperm(rows, generator=g)[:n_out]] *= 50.0  # 1 % outlier rows
    w = 1.0 + 0.02 * torch.randn(cols, generator=g)
    b = 0.02 * torch.randn(cols, generator=g)
    return x.to(dtype), w.to(dtype), b.to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cols", [1, 7, 8, 96, 127, 128, 256, 384, 385, 400, 512, 1024, 2048, 2560, 4096])
def test_norms_match_oracle(dtype, cols):
    rows = 333
    x, w, b = _inputs(rows, cols, dtype, seed=cols)
    xd, wd, bd = x.cuda(), w.cuda(), b.cuda()
    got = ops.rms_norm(xd, wd, 1e-6).cpu()
    want = R.rms_norm_fp32(x, w, 1e-6)
    assert (got.float() - want.float()).abs().max().item() <= TOL[dtype]
    got = ops.layer_norm(xd, wd, bd, 1e-6).cpu()
    want = R.layer_norm_fp32(x, w, b, 1e-6)
    assert (got.float() - want.float()).abs().max().item() <= TOL[dtype]


@pytest.mark.parametrize("rows", [0, 1, 2, 63, 64, 65, 1000, 4097])
def test_ragged_row_counts(rows):
    """Tile tails: row counts around the tile size, a single row and the empty matrix."""
    x, w, b = _inputs(max(rows, 1), 128, torch.bfloat16, seed=rows)
    x = x[:rows]
    got = ops.rms_norm(x.cuda(), w.cuda(), 1e-6).cpu()
    assert got.shape == x.shape
    if rows:
        assert (got.float() - R.rms_norm_fp32(x, w, 1e-6).float()).abs().max().item() <= 2e-2
    got = ops.layer_norm(x.cuda(), w.cuda(), b.cuda(), 1e-5).cpu()
    if rows:
        assert (got.float() - R.layer_norm_fp32(x, w, b, 1e-5).float()).abs().max().item() <= 2e-2


def test_leading_dims_and_kernel_reuse():
    """N-d input keeps its shape; one library serves changing row counts (no per-shape rebuild)."""
    x, w, _ = _inputs(6 * 50, 256, torch.bfloat16)
    for b in (1, 3, 6):
        xb = x[: b * 50].view(b, 50, 256)
        got = ops.rms_norm(xb.cuda(), w.cuda()).cpu()
        assert got.shape == xb.shape
        assert (got.float() - R.rms_norm_fp32(xb, w, 1e-6).float()).abs().max().item() <= 2e-2


def test_against_reference_golden(ops_golden):
    for tag, bf16 in (("f32_96", False), ("f32_128", False), ("f32_127", False), ("bf16_128", True), ("bf16_400", True)):
        load = bf16_from_bits if bf16 else (lambda a: torch.from_numpy(a.copy()))
        x, w, b = (load(ops_golden[f"norm_{tag}_{k}"]) for k in ("x", "w", "b"))
        tol = 2e-2 if bf16 else 2e-5
        got = ops.rms_norm(x.cuda(), w.cuda(), 1e-6).cpu().float()
        torch.testing.assert_close(got, load(ops_golden[f"norm_{tag}_rms"]).float(), atol=tol, rtol=tol)
        got = ops.layer_norm(x.cuda(), w.cuda(), b.cuda(), 1e-6).cpu().float()
        torch.testing.assert_close(got, load(ops_golden[f"norm_{tag}_ln"]).float(), atol=tol, rtol=tol)


@pytest.mark.parametrize("cols", [128, 256, 512, 1024])
def test_full_size_sweep_properties(cols):
    """65 536 x cols bf16 (the benchmark sweep): checked by sampled rows against the oracle and by
    size-independent properties (unit RMS before gamma; zero mean / unit variance for LayerNorm)."""
    rows = 65536
    x, w, b = _inputs(rows, cols, torch.bfloat16, seed=1)
    xd = x.cuda()
    ones = torch.ones(cols, dtype=torch.bfloat16, device="cuda")
    zeros = torch.zeros(cols, dtype=torch.bfloat16, device="cuda")
    y = ops.rms_norm(xd, ones, 1e-6).float()
    rms = y.pow(2).mean(dim=1).sqrt()
    assert (rms - 1.0).abs().max().item() < 1e-2
    z = ops.layer_norm(xd, ones, zeros, 1e-6).float()
    assert z.mean(dim=1).abs().max().item() < 1e-2
    assert (z.var(dim=1, unbiased=False) - 1.0).abs().max().item() < 2e-2
    idx = torch.randperm(rows, generator=torch.Generator().manual_seed(2))[:512]
    got = ops.rms_norm(xd, w.cuda(), 1e-6)[idx.cuda()].cpu()
    assert (got.float() - R.rms_norm_fp32(x[idx], w, 1e-6).float()).abs().max().item() <= 2e-2
    got = ops.layer_norm(xd, w.cuda(), b.cuda(), 1e-6)[idx.cuda()].cpu()
    assert (got.float() - R.layer_norm_fp32(x[idx], w, b, 1e-6).float()).abs().max().item() <= 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cols", [7, 128, 384, 512, 1024, 2560, 4096])
def test_rms_norm_with_input_bias(dtype, cols):
    """rms_norm(x, in_bias=b) == rms_norm of the fp32 sum x + b (the bias never rounds on its own)."""
    x, w, b = _inputs(257, cols, dtype, seed=cols + 1)
    got = ops.rms_norm(x.cuda(), w.cuda(), 1e-6, in_bias=b.cuda()).cpu()
    want = R.rms_norm_fp32(x.float() + b.float(), w.float(), 1e-6)
    assert (got.float() - want.float()).abs().max().item() <= TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cols", [7, 128, 384, 512, 1024, 2560, 4096])
def test_layer_norm_of_silu(dtype, cols):
    """layer_norm(x, pre_silu=True) == layer_norm(silu(x)) with the activation rounded to the dtype."""
    x, w, b = _inputs(257, cols, dtype, seed=cols + 2)
    got = ops.layer_norm(x.cuda(), w.cuda(), b.cuda(), 1e-5, pre_silu=True).cpu()
    act = torch.nn.functional.silu(x.float()).to(dtype)
    want = R.layer_norm_fp32(act, w, b, 1e-5)
    assert (got.float() - want.float()).abs().max().item() <= TOL[dtype]


def test_fused_norm_variants_edge_cases():
    """Empty matrices, a width that needs the scalar kernel, and the bias shape check."""
    w = torch.ones(48, device="cuda").bfloat16()
    b = torch.zeros(48, device="cuda").bfloat16()
    empty = torch.empty(0, 48, device="cuda", dtype=torch.bfloat16)
    assert ops.rms_norm(empty, w, 1e-6, in_bias=b).shape == (0, 48)
    assert ops.layer_norm(empty, w, b, 1e-5, pre_silu=True).shape == (0, 48)
    with pytest.raises(ValueError):
        ops.rms_norm(torch.zeros(3, 48, device="cuda").bfloat16(), w, 1e-6, in_bias=torch.zeros(47, device="cuda"))
    # 3-D input, width 5 (rows are not whole 16-byte pieces)
    x = torch.randn(2, 3, 5)
    w5, b5 = torch.rand(5) + 0.5, torch.randn(5)
    got = ops.rms_norm(x.cuda(), w5.cuda(), 1e-6, in_bias=b5.cuda()).cpu()
    want = R.rms_norm_fp32((x + b5).reshape(-1, 5), w5, 1e-6).reshape(2, 3, 5)
    assert (got - want).abs().max().item() <= 2e-5


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("cols,two", [(128, True), (512, True), (512, False), (1024, True), (1024, False)])
def test_token_tail_equals_the_separate_kernels(dtype, cols, two):
    """layer_norm(silu(x)) + gathered rows -> tokens and rms_norm(tokens) from one kernel, bit for bit the
    results of the three kernels it replaces."""
    g = torch.Generator().manual_seed(cols)
    rows = 1003
    x = (1.5 * torch.randn(rows, cols, generator=g)).to(dtype).cuda()
    w1 = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype).cuda()
    b1 = (0.1 * torch.randn(cols, generator=g)).to(dtype).cuda()
    w2 = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype).cuda()
    ta = torch.randn(65, cols, generator=g).to(dtype).cuda()
    tb = torch.randn(300, cols, generator=g).to(dtype).cuda()
    ia = torch.randint(-1, 70, (rows,), generator=g).cuda()
    ib = torch.randint(0, 300, (rows,), generator=g).cuda()
    tokens, normed = ops.token_tail(x, w1, b1, ta, ia, tb if two else None, ib if two else None, w2)
    want_tokens = ops.layer_norm(x, w1, b1, 1e-5, pre_silu=True)
    ops.add_gathered_rows(want_tokens, ta, ia, *((tb, ib) if two else ()))
    want_normed = ops.rms_norm(want_tokens, w2, 1e-6)
    assert torch.equal(tokens, want_tokens)
    assert torch.equal(normed, want_normed)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("cols", [64, 128, 512, 1024])
def test_token_tail_with_row_selection(dtype, cols):
    """With `row_dst` the first output only holds the selected rows, at their destinations, and the second
    output still holds every row; both bit for bit what the unselected call gives."""
    g = torch.Generator().manual_seed(cols + 1)
    rows = 2051
    x = (1.5 * torch.randn(rows, cols, generator=g)).to(dtype).cuda()
    w1 = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype).cuda()
    b1 = (0.1 * torch.randn(cols, generator=g)).to(dtype).cuda()
    w2 = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype).cuda()
    ta = torch.randn(65, cols, generator=g).to(dtype).cuda()
    tb = torch.randn(300, cols, generator=g).to(dtype).cuda()
    ia = torch.randint(0, 65, (rows,), generator=g).cuda()
    ib = torch.randint(0, 300, (rows,), generator=g).cuda()
    want_tokens, want_normed = ops.token_tail(x, w1, b1, ta, ia, tb, ib, w2)
    kept = torch.randperm(rows, generator=g)[:301].cuda()          # destination i <- row kept[i], any order
    row_dst = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    row_dst[kept] = torch.arange(kept.numel(), dtype=torch.int32, device="cuda")
    row_dst[(row_dst < 0).nonzero()[:5, 0]] = torch.tensor([kept.numel(), 2**31 - 1, -7, kept.numel() + 3, -2**31],
                                                           dtype=torch.int32, device="cuda")   # all skipped
    tokens, normed = ops.token_tail(x, w1, b1, ta, ia, tb, ib, w2, row_dst=row_dst, rows_out=kept.numel())
    assert tokens.shape == (kept.numel(), cols)
    assert torch.equal(tokens, want_tokens[kept])
    assert torch.equal(normed, want_normed)
    # nothing selected: no first output at all
    none = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    tokens, normed = ops.token_tail(x, w1, b1, ta, ia, tb, ib, w2, row_dst=none, rows_out=0)
    assert tokens.shape == (0, cols) and torch.equal(normed, want_normed)


def test_token_tail_rejects_rows_it_cannot_stage():
    """Rows that are not whole 16-byte pieces (or wider than 256 pieces) have no fused kernel: the call fails
    loudly instead of running something else."""
    x = torch.randn(10, 20, device="cuda").bfloat16()
    w = torch.ones(20, device="cuda").bfloat16()
    table = torch.zeros(4, 20, device="cuda").bfloat16()
    ids = torch.zeros(10, dtype=torch.int64, device="cuda")
    with pytest.raises(RuntimeError):
        ops.token_tail(x, w, w, table, ids, None, None, w)
