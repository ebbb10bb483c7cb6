"""GPU parity of the embedding gather / bag-mean kernels through the C ABI: bit-exact against
the CPU oracle and the reference's golden outputs."""

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


def test_bag_mean_golden_bit_exact(ops_golden):
    table = torch.from_numpy(ops_golden["bag_table"].copy()).cuda()
    for ids_key, out_key in (("bag_ids", "bag_out"), ("bag1_ids", "bag1_out")):
        for id_dtype in (torch.int64, torch.int32):
            ids = torch.from_numpy(ops_golden[ids_key].copy()).to(id_dtype).cuda()
            got = ops.embedding_bag_mean(table, ids).cpu()
            assert torch.equal(got, torch.from_numpy(ops_golden[out_key])), (ids_key, id_dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("dim,bag", [(4, 1), (8, 3), (64, 1), (64, 4), (128, 8), (200, 2), (512, 5)])
def test_bag_mean_matches_oracle(dtype, dim, bag):
    if (dim * torch.finfo(dtype).bits // 8) % 16:
        pytest.skip("rows must be whole 16-byte chunks")
    g = torch.Generator().manual_seed(dim * 31 + bag)
    vocab = 997
    table = torch.randn(vocab + 1, dim, generator=g).to(dtype)
    table[0] = 0
    ids = torch.randint(0, vocab + 1, (301, bag), generator=g)
    ids[torch.rand(301, bag, generator=g) < 0.25] = 0  # padding
    ids[5] = 0  # an empty bag
    ids[6, 0] = vocab + 7  # outside the table: skipped
    ids[7, 0] = -3
    got = ops.embedding_bag_mean(table.cuda(), ids.cuda()).cpu()
    want = R.embedding_bag_mean(table, ids)
    assert torch.equal(got, want)


def test_fields_bag_mean_matches_feature_bank():
    """All fields of an entity in one launch == the per-field loop of the reference bank, including
    its clamp of out-of-vocabulary ids."""
    g = torch.Generator().manual_seed(5)
    specs = [(50, 0, 1), (7, 1, 3), (300, 4, 1), (20, 5, 2)]  # (vocab, offset, length)
    tables = []
    for vocab, _o, _l in specs:
        t = torch.randn(vocab + 1, 16, generator=g)
        t[0] = 0
        tables.append(t)
    ints = torch.randint(-2, 320, (257, 7), generator=g)
    ints[:, 0][::3] = 0
    want = R.feature_bank(tables, specs, ints)
    fields = ops.FieldTables([t.cuda() for t in tables], [s[1] for s in specs], [s[2] for s in specs])
    got = ops.fields_bag_mean(fields, ints.cuda()).cpu()
    assert torch.equal(got, want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sequence_gather_bit_exact(dtype):
    g = torch.Generator().manual_seed(11)
    B, F, L, dim = 9, 3, 37, 32
    vocabs = [100, 0, 1000]
    tables = [None if v == 0 else torch.randn(v + 1, dim, generator=g).to(dtype) for v in vocabs]
    ids = torch.randint(-1, 1100, (B, F, L), generator=g)
    lens = torch.randint(0, L + 1, (B,), generator=g)
    ids = torch.where((torch.arange(L)[None] < lens[:, None])[:, None, :], ids, torch.zeros_like(ids))
    want = torch.cat(
        [torch.zeros(B, L, dim, dtype=dtype) if t is None else R.gather_rows(t, ids[:, f]) for f, t in enumerate(tables)], dim=-1
    )
    got = ops.sequence_gather([None if t is None else t.cuda() for t in tables], ids.cuda()).cpu()
    assert torch.equal(got, want)
    got1 = ops.gather_rows(tables[2].cuda(), ids[:, 2].cuda()).cpu()
    assert torch.equal(got1, R.gather_rows(tables[2], ids[:, 2]))
    assert ops.gather_rows(tables[0].cuda(), torch.zeros(0, dtype=torch.int64, device="cuda")).shape == (0, dim)


def test_large_gather_checksum():
    """Full-width case (1 M-row bf16 table, 2^20 Zipf-like ids): compared with torch indexing on the
    device, which is a plain copy, so equality is exact."""
    g = torch.Generator(device="cuda").manual_seed(3)
    table = torch.randn(1_000_001, 128, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    u = torch.rand(1 << 20, generator=g, device="cuda", dtype=torch.float64)
    ids = (u.pow(8.0) * 1_000_000).long() + 1  # heavy head, long tail
    ids[::17] = 0
    got = ops.gather_rows(table, ids)
    assert torch.equal(got, table[ids])
    bag = ids.view(-1, 4)
    got = ops.embedding_bag_mean(table, bag).float()
    valid = (bag != 0).unsqueeze(-1)
    want = (table[bag].float() * valid).sum(dim=1) / valid.sum(dim=1).clamp_min(1)
    assert (got - want.to(torch.bfloat16).float()).abs().max().item() <= 2e-2  # summation order differs from torch's


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_scatter_rows_with_bias_and_residual(dtype):
    g = torch.Generator().manual_seed(21)
    rows, width, dim, groups, per = 500, 96, 32, 3, 40
    dst = torch.randn(rows, width, generator=g).to(dtype)
    src = torch.randn(groups * per, dim, generator=g).to(dtype)
    bias = torch.randn(groups, dim, generator=g).to(dtype)
    res = torch.randn(rows, dim, generator=g).to(dtype)
    ids = torch.randperm(rows, generator=g)[: groups * per]
    want = dst.clone()
    want[ids, 64:96] = src
    got = ops.scatter_rows(dst.clone().cuda(), ids.cuda(), src.cuda(), col0=64).cpu()
    assert torch.equal(got, want)  # a plain scatter is a copy
    want = dst.clone()
    want[ids, :dim] = (src.float() + bias.float().repeat_interleave(per, dim=0) + res[ids].float()).to(dtype)
    got = ops.scatter_rows(dst.clone().cuda(), ids.cuda(), src.cuda(), bias=bias.cuda(), residual=res.cuda()).cpu()
    assert torch.equal(got, want)  # one fp32 sum, one rounding
    assert ops.scatter_rows(dst.clone().cuda(), ids[:0].cuda(), src[:0].cuda()).shape == dst.shape


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("two", [False, True])
def test_add_gathered_rows_bit_exact(dtype, two):
    """In-place x += A[ia] (+= B[ib]) equals the tensor additions evaluated left to right, bit for bit."""
    g = torch.Generator().manual_seed(5)
    n, dim = 1237, 512
    x = torch.randn(n, dim, generator=g).to(dtype)
    a = torch.randn(65, dim, generator=g).to(dtype)
    b = torch.randn(1040, dim, generator=g).to(dtype)
    ia = torch.randint(-2, 70, (n,), generator=g)      # out-of-range ids clamp into the table
    ib = torch.randint(0, 1040, (n,), generator=g)
    want = x + a[ia.clamp(0, 64)]
    if two:
        want = want + b[ib]
    xd = x.cuda()
    out = ops.add_gathered_rows(xd, a.cuda(), ia.cuda(), *( (b.cuda(), ib.cuda()) if two else () ))
    assert out.data_ptr() == xd.data_ptr()
    assert torch.equal(out.cpu(), want)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_bias_silu_rows(dtype):
    """x = silu(x + bias[group]) in place against the two torch operations it replaces."""
    g = torch.Generator().manual_seed(6)
    groups, per, cols = 5, 77, 256
    x = (2.0 * torch.randn(groups, per, cols, generator=g)).to(dtype)
    bias = torch.randn(groups, 1, cols, generator=g).to(dtype)
    want = torch.nn.functional.silu((x + bias).float()).to(dtype)
    got = ops.bias_silu_rows(x.cuda(), bias.cuda()).cpu()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    diff = (got.float() - want.float()).abs()
    assert diff.max().item() <= tol
    if dtype == torch.bfloat16:   # one rounding step apart at most, identical almost everywhere
        assert (got != want).float().mean().item() < 0.02


def test_row_kernels_edge_cases():
    """Empty inputs are no-ops; shapes the kernels cannot serve are rejected on the host with ValueError."""
    dev = "cuda"
    x0 = torch.empty(0, 64, dtype=torch.bfloat16, device=dev)
    table = torch.randn(5, 64, device=dev).bfloat16()
    ids0 = torch.empty(0, dtype=torch.int64, device=dev)
    assert ops.add_gathered_rows(x0, table, ids0).shape == (0, 64)
    assert ops.bias_act_rows(torch.empty(0, 64, dtype=torch.bfloat16, device=dev).view(0, 64),
                             torch.zeros(64, device=dev), silu=True).shape == (0, 64)
    x = torch.randn(6, 64, device=dev).bfloat16()
    with pytest.raises(ValueError):
        ops.add_gathered_rows(x, table, torch.zeros(5, dtype=torch.int64, device=dev))       # one id per row
    with pytest.raises(ValueError):
        ops.add_gathered_rows(x, table.float(), torch.zeros(6, dtype=torch.int64, device=dev))  # dtype mismatch
    with pytest.raises(ValueError):
        ops.add_gathered_rows(x, table, torch.zeros(6, dtype=torch.int64, device=dev), table, None)
    with pytest.raises(ValueError):
        ops.bias_act_rows(x, torch.zeros(4, 64, device=dev), silu=False)                       # 4 groups do not divide 6 rows
    # a single group (plain bias vector) and one group per row
    want = (x.float() + 1.0).bfloat16()
    assert torch.equal(ops.bias_act_rows(x.clone(), torch.ones(64, device=dev), silu=False), want)
    per_row = torch.arange(6, device=dev, dtype=torch.float32)[:, None].expand(6, 64).contiguous()
    want = (x.float() + per_row).bfloat16()
    assert torch.equal(ops.bias_act_rows(x.clone(), per_row, silu=False), want)
    # odd widths: 24 columns = 48 bytes = three 16-byte pieces per row
    y = torch.randn(7, 24, device=dev).bfloat16()
    b = torch.randn(24, device=dev).bfloat16()
    assert torch.equal(ops.bias_act_rows(y.clone(), b, silu=False), (y.float() + b.float()).bfloat16())


@pytest.mark.parametrize("with_time", [True, False])
def test_packed_token_index_matches_the_index_arithmetic(with_time):
    """Ids (raw and hashed), positions and time-gap buckets of every packed row from one kernel, against the
    same quantities spelled out with tensor indexing."""
    g = torch.Generator().manual_seed(31)
    B, F, L, ns = 37, 3, 50, 4
    values = torch.randint(-2, 5000, (B, F, L), generator=g)
    ts = torch.randint(0, 3, (B, L), generator=g) * torch.randint(1, 10**9, (B, L), generator=g)   # a third are zero
    req = torch.randint(5 * 10**8, 2 * 10**9, (B,), generator=g)
    src = torch.stack([torch.randperm(L, generator=g) for _ in range(B)]).to(torch.int32)
    n0 = torch.randint(0, 31, (B,), generator=g)
    n0[0], n0[1] = 0, 30
    start = torch.randint(0, L - 30, (B,), generator=g)
    rows = n0 + ns
    cu = torch.zeros(B + 1, dtype=torch.long)
    cu[1:] = torch.cumsum(rows, 0)
    total = int(cu[-1])
    hash_buckets = torch.tensor([0, 97, -1])
    edges = torch.tensor(sorted(set(torch.randint(1, 10**9, (20,), generator=g).tolist())))
    ids, pos, buckets = ops.packed_token_index(values.cuda(), ts.cuda() if with_time else None, req.cuda(), src.cuda(), cu.cuda(),
                                               n0.cuda(), start.cuda(), hash_buckets.cuda(), total,
                                               edges=edges.cuda() if with_time else None)
    want_ids = torch.zeros(F, total, dtype=torch.long)
    want_pos = torch.zeros(total, dtype=torch.long)
    want_b = torch.zeros(total, dtype=torch.long)
    for b in range(B):
        for j in range(int(n0[b])):
            p = int(src[b, int(start[b]) + j])
            r = int(cu[b]) + j
            want_ids[0, r] = values[b, 0, p]
            v = int(values[b, 1, p])
            want_ids[1, r] = (v - 1) % 97 + 1 if v > 0 else 0
            want_pos[r] = j
            if ts[b, p] != 0:
                gap = max(int(req[b]) - int(ts[b, p]), 0)
                want_b[r] = min(int((edges < gap).sum()), edges.numel() - 1) + 1
    assert torch.equal(ids.cpu(), want_ids)          # the feature without a table stays zero
    assert torch.equal(pos.cpu(), want_pos)
    if with_time:
        assert torch.equal(buckets.cpu(), want_b)
    else:
        assert buckets is None


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("batch,bag,dim,vocab", [(1, 1, 8, 5), (300, 4, 64, 50), (1000, 3, 128, 1000), (77, 9, 32, 20)])
def test_bag_mean_backward_matches_autograd(dtype, batch, bag, dim, vocab):
    """The sparse table gradient of the bag mean, coalesced, against torch autograd of `F.embedding_bag(mode="mean",
    padding_idx=0)` (what the reference's sparse backward reproduces, modeling/embeddings.py:34-62)."""
    g = torch.Generator().manual_seed(batch + bag + dim)
    ids = torch.randint(0, vocab + 1, (batch, bag), generator=g)
    ids[torch.rand(batch, bag, generator=g) < 0.3] = 0          # padding, including all-padding bags
    grad_out = torch.randn(batch, dim, generator=g).to(dtype)
    table = torch.randn(vocab + 1, dim, generator=g, requires_grad=True)
    torch.nn.functional.embedding_bag(ids, table, mode="mean", padding_idx=0).backward(grad_out.float())
    got = ops.embedding_bag_mean_backward(ids.cuda(), grad_out.cuda(), vocab + 1)
    assert got.is_sparse and got.shape == (vocab + 1, dim) and got.dtype == dtype
    dense = torch.zeros(vocab + 1, dim).index_add_(0, got._indices()[0].cpu(), got._values().float().cpu())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (dense - table.grad).abs().max().item() <= tol * max(1.0, table.grad.abs().max().item())
    assert torch.equal(dense[0], torch.zeros(dim))            # the padding row receives nothing
