"""The fused sequence tokenizer (`tb200_token_project_fwd`: row gather -> tcgen05 projection -> SiLU -> LayerNorm ->
time / position rows -> first RMSNorm in one kernel) against fp32 torch math on the same bf16 operands with the
reference's rounding points (`nn.Linear -> nn.SiLU -> nn.LayerNorm`, tensor additions, RMSNorm;
src/taac2026/infrastructure/modeling/tokenizers.py:156-190), and against this library's own three-kernel path."""

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


def _case(rows, n_feat, emb, n_cols, seed, *, missing_feature=False, second_table=True):
    g = torch.Generator().manual_seed(seed)
    k = n_feat * emb
    tables = [(torch.randn(50 + 13 * f, emb, generator=g) * 0.5).bfloat16() for f in range(n_feat)]
    if missing_feature:
        tables[-1] = None
    ids = torch.stack([torch.randint(-2, 70 + 13 * f, (rows,), generator=g) for f in range(n_feat)])   # some ids outside: clamp path
    weight = (torch.randn(n_cols, k, generator=g) * k ** -0.5).bfloat16()
    bias = torch.randn(n_cols, generator=g) * 0.3
    ln_w = (1 + 0.1 * torch.randn(n_cols, generator=g)).bfloat16()
    ln_b = (0.1 * torch.randn(n_cols, generator=g)).bfloat16()
    rms_w = (1 + 0.1 * torch.randn(n_cols, generator=g)).bfloat16()
    table_a = torch.randn(64, n_cols, generator=g).bfloat16()
    ids_a = torch.randint(0, 64, (rows,), generator=g)
    table_b = torch.randn(300, n_cols, generator=g).bfloat16() if second_table else None
    ids_b = torch.randint(0, 300, (rows,), generator=g) if second_table else None
    return tables, ids, weight, bias, ln_w, ln_b, table_a, ids_a, table_b, ids_b, rms_w


def _reference(tables, ids, weight, bias, ln_w, ln_b, table_a, ids_a, table_b, ids_b, rms_w):
    cols = []
    for f, table in enumerate(tables):
        if table is None:
            cols.append(torch.zeros(ids.shape[1], weight.shape[1] // len(tables)))
        else:
            cols.append(table.float()[ids[f].clamp(0, table.shape[0] - 1)])
    x = torch.cat(cols, dim=1)
    p = x @ weight.float().t() + bias
    s = torch.nn.functional.silu(p).bfloat16().float()
    y = torch.nn.functional.layer_norm(s, (s.shape[1],), ln_w.float(), ln_b.float(), 1e-5).bfloat16()
    tokens = y + table_a[ids_a]
    if table_b is not None:
        tokens = tokens + table_b[ids_b]
    t = tokens.float()
    normed = (t * torch.rsqrt(t.pow(2).mean(dim=1, keepdim=True) + 1e-6) * rms_w.float()).bfloat16()
    return tokens, normed


def _cuda(args):
    return [None if a is None else ([None if t is None else t.cuda() for t in a] if isinstance(a, list) else a.cuda()) for a in args]


@pytest.mark.parametrize("rows,n_feat,emb,n_cols,missing,second", [
    (128, 1, 128, 512, False, True), (1, 1, 128, 512, False, True), (333, 2, 64, 512, False, False),
    (1000, 4, 32, 512, True, True), (257, 2, 32, 256, False, True), (129, 1, 64, 256, False, False),
    (40001, 1, 128, 512, False, True),
])
def test_matches_fp32_math(rows, n_feat, emb, n_cols, missing, second):
    case = _case(rows, n_feat, emb, n_cols, rows + n_feat, missing_feature=missing, second_table=second)
    want_tokens, want_normed = _reference(*case)
    dev = _cuda(case)
    tokens, normed = ops.token_project(*dev, check=True)
    assert tokens.shape == (rows, n_cols) and normed.shape == (rows, n_cols)
    # The kernel takes the LayerNorm statistics from the fp32 SiLU values (the reference rounds them to bf16 first) and
    # uses the tanh form of the SiLU, so a LayerNorm output may sit one bf16 step beside the reference's; the table rows
    # are added to values of size up to 8 (step 2^-5), whatever the size of the sum.  Hence an absolute bound of two such
    # steps on every element, and a mean error that shows the differences are rounding, not bias.
    for got, want in ((tokens, want_tokens), (normed, want_normed)):
        err = (got.float().cpu() - want.float()).abs()
        assert err.max().item() <= 7e-2
        assert err.mean().item() <= 5e-4


def test_row_selection_and_three_kernel_path():
    """`row_dst` compacts `tokens` exactly like the unfused tail does, and the fused kernel agrees with
    gather_rows -> grouped_linear -> token_tail to bf16 rounding (the projection is not rounded to bf16 here)."""
    rows, n_cols = 5000, 512
    case = _case(rows, 1, 128, n_cols, 7)
    tables, ids, weight, bias, ln_w, ln_b, table_a, ids_a, table_b, ids_b, rms_w = _cuda(case)
    full_tokens, full_normed = ops.token_project(tables, ids, weight, bias, ln_w, ln_b, table_a, ids_a, table_b, ids_b, rms_w, check=True)
    g = torch.Generator().manual_seed(1)
    keep = torch.randperm(rows, generator=g)[:700].sort().values
    row_dst = torch.full((rows,), -1, dtype=torch.int32)
    row_dst[keep] = torch.arange(700, dtype=torch.int32)
    tokens, normed = ops.token_project(tables, ids, weight, bias, ln_w, ln_b, table_a, ids_a, table_b, ids_b, rms_w,
                                       row_dst=row_dst.cuda(), rows_out=700, check=True)
    assert tokens.shape == (700, n_cols)
    assert torch.equal(tokens, full_tokens[keep.cuda()])
    assert torch.equal(normed, full_normed)
    assert torch.equal(ops.token_project(tables, ids, weight, bias, ln_w, ln_b, table_a, ids_a, table_b, ids_b, rms_w)[1], full_normed)  # same bits on every run
    gathered = ops.gather_rows(tables[0], ids[0])
    projected = ops.grouped_linear(gathered, weight, bias, check=True)
    t3, n3 = ops.token_tail(projected, ln_w, ln_b, table_a, ids_a, table_b, ids_b, rms_w)
    assert (t3.float() - full_tokens.float()).abs().max().item() <= 0.13    # two bf16 steps of values up to 16
    assert (t3.float() - full_tokens.float()).abs().mean().item() <= 2e-3
    assert (n3.float() - full_normed.float()).abs().mean().item() <= 2e-3


def test_unsupported_shapes_are_refused():
    case = _cuda(_case(64, 1, 128, 512, 3))
    tables, ids, weight = case[0], case[1], case[2]
    assert ops.token_project_supported(tables, weight)
    assert not ops.token_project_supported([t[:, :16].contiguous() for t in tables], weight[:, :16].contiguous())
    assert not ops.token_project_supported(tables, weight[:128].contiguous())
    with pytest.raises(ValueError):
        ops.token_project(tables, ids.to(torch.int32), *case[2:])
