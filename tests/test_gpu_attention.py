"""GPU parity of the varlen masked attention forward, called through the C ABI.

Oracle: the fp32 max-subtracted softmax attention of ``oracle/reference_ops.py`` (pinned to the
reference's SDPA outputs) on the same bf16/fp16 inputs.  Tolerance: max-abs <= 2e-2 on every
computed row (the bound the task states for bf16 attention; the reference's own GPU tests use
1e-2..2e-2, tests/gpu/infrastructure/accelerators/test_tilelang_ops_cuda.py:61-183); padded
query rows must equal the value rows exactly.
"""

from __future__ import annotations

import pytest
import torch

from conftest import gpu_ready
from oracle import reference_ops as R
from taac_2026_b200 import ops

pytestmark = pytest.mark.gpu
KERNELS = [1, 2]  # 1 = mma.sync kernel (all shapes), 2 = tcgen05/TMEM kernel (head_dim 64, bf16)


def _kw(kernel, D=64, dtype=torch.bfloat16):
    if kernel == 2 and (D != 64 or dtype != torch.bfloat16):
        pytest.skip("the tcgen05 kernel serves head_dim 64 bf16")
    return {"kernel": kernel, "check": kernel == 2}



@pytest.fixture(autouse=True)
def _need_gpu():
    if not gpu_ready():
        pytest.fail("gpu tests need an sm_100 device and a built libtb200.so")


def _qkv(B, H, L, D, dtype, seed, lk=None):
    g = torch.Generator().manual_seed(seed)
    scale = D ** -0.25  # scores of order 1
    q = (torch.randn(B, H, L, D, generator=g) * scale).to(dtype)
    k = (torch.randn(B, H, lk or L, D, generator=g) * scale).to(dtype)
    v = torch.randn(B, H, lk or L, D, generator=g).to(dtype)
    return q, k, v


def _check(got, q, k, v, mask, self_rows=None, tol=2e-2):
    want = R.attention(q, k, v, mask[:, None])
    got = got.float().cpu()
    if self_rows is not None:
        sel = self_rows[:, None, :, None].expand_as(got)
        assert torch.equal(got[sel], v.float()[sel]), "padded query rows must return their value rows"
        got = torch.where(sel, torch.zeros_like(got), got)
        want = torch.where(sel, torch.zeros_like(want), want)
    assert torch.isfinite(got).all()
    err = (got - want).abs().max().item()
    assert err <= tol, err


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D", [32, 64, 128])
@pytest.mark.parametrize("L", [1, 17, 64, 65, 200, 333])
def test_key_padding_noncausal(kernel, dtype, D, L):
    B, H = 3, 2
    q, k, v = _qkv(B, H, L, D, dtype, seed=L * 7 + D)
    lens = torch.tensor([L, max(1, L // 3), max(1, L - 1)])
    got = ops.varlen_attention(q.cuda(), k.cuda(), v.cuda(), seq_len=lens.cuda(), **_kw(kernel, D, dtype))
    _check(got, q, k, v, R.structured_attention_mask(lens, L, L, False, False))


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("D", [32, 64])
@pytest.mark.parametrize("L,ns", [(1, 0), (40, 0), (64, 9), (129, 9), (300, 0), (265, 9), (128, 128)])
def test_causal_valid_with_ns_suffix(kernel, D, L, ns):
    """causal AND key-valid, padded queries self-only, with and without an always-valid suffix;
    lengths include 0 (no valid sequence token) and the full sequence."""
    B, H = 5, 2
    S = L - ns
    q, k, v = _qkv(B, H, L, D, torch.bfloat16, seed=L + ns)
    lens = torch.tensor([S, 0, min(S, 1), S // 2, max(S - 1, 0)])
    got = ops.varlen_attention(q.cuda(), k.cuda(), v.cuda(), seq_len=lens.cuda(), ns_start=S, causal=True,
                               padded_query_self=True, **_kw(kernel, D))
    mask = R.structured_attention_mask(lens, L, S, True, True)
    pos = torch.arange(L)[None]
    self_rows = (pos >= lens[:, None]) & (pos < S)
    _check(got, q, k, v, mask, self_rows)


@pytest.mark.parametrize("kernel", KERNELS)
def test_cross_lengths_and_plain_causal(kernel):
    q, k, v = _qkv(2, 4, 70, 64, torch.bfloat16, seed=3, lk=150)
    lens = torch.tensor([150, 61])
    got = ops.varlen_attention(q.cuda(), k.cuda(), v.cuda(), seq_len=lens.cuda(), **_kw(kernel))
    mask = (torch.arange(150)[None, None, :] < lens[:, None, None]).expand(2, 70, 150)
    _check(got, q, k, v, mask)
    q, k, v = _qkv(2, 4, 190, 64, torch.bfloat16, seed=4)
    got = ops.varlen_attention(q.cuda(), k.cuda(), v.cuda(), causal=True, **_kw(kernel))
    _check(got, q, k, v, R.structured_attention_mask(torch.tensor([190, 190]), 190, 190, True, False))


@pytest.mark.parametrize("kernel", KERNELS)
def test_rows_without_visible_key_are_zero(kernel):
    q, k, v = _qkv(2, 2, 50, 64, torch.bfloat16, seed=5)
    lens = torch.tensor([0, 20])
    got = ops.varlen_attention(q.cuda(), k.cuda(), v.cuda(), seq_len=lens.cuda(), **_kw(kernel)).cpu()
    assert torch.equal(got[0], torch.zeros_like(got[0]))
    _check(got[1:], q[1:], k[1:], v[1:], R.structured_attention_mask(lens[1:], 50, 50, False, False))


@pytest.mark.parametrize("kernel", KERNELS)
def test_blhd_views_of_fused_qkv_and_packed_batch(kernel):
    """(B, L, H, D) strided views of one [B, L, 3, H, D] projection, and the packed-rows form."""
    B, L, H, D = 4, 150, 4, 64
    g = torch.Generator().manual_seed(6)
    qkv = (torch.randn(B, L, 3, H, D, generator=g) * 0.5).bfloat16()
    lens = torch.tensor([150, 3, 77, 128])
    dev = qkv.cuda()
    got = ops.varlen_attention(dev[:, :, 0], dev[:, :, 1], dev[:, :, 2], seq_len=lens.cuda(), causal=True,
                               padded_query_self=True, layout="blhd", **_kw(kernel))
    assert got.shape == (B, L, H, D)
    q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    mask = R.structured_attention_mask(lens, L, L, True, True)
    self_rows = torch.arange(L)[None] >= lens[:, None]
    _check(got.permute(0, 2, 1, 3), q, k, v, mask, self_rows)
    # packed: only the valid rows of every sample, back to back
    cu = torch.zeros(B + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens, 0)
    packed = torch.cat([qkv[b, : lens[b]] for b in range(B)], dim=0).cuda()  # [rows, 3, H, D]
    got_p = ops.varlen_attention(packed[:, 0], packed[:, 1], packed[:, 2], causal=True, cu_rows=cu.cuda(),
                                 max_rows=int(lens.max()), **_kw(kernel)).cpu()
    for b in range(B):
        lo, hi = int(cu[b]), int(cu[b + 1])
        ref = got[b, : hi - lo].cpu()
        assert (got_p[lo:hi].float() - ref.float()).abs().max().item() <= (1e-6 if kernel == 1 else 4e-3)


@pytest.mark.parametrize("kernel", KERNELS)
def test_reference_signature_and_golden(kernel, ops_golden):
    if kernel == 2:
        pytest.skip("the reference's golden cases have head_dim 16 (padded to 32): mma.sync kernel only")
    """`flash_attention(q, k, v, backend="cuda", attn_mask=...)` on the reference's golden cases; fp32
    callers are served in bf16 and get fp32 back."""
    q, k, v = (torch.from_numpy(ops_golden[f"attn_{n}"].copy()) for n in "qkv")
    B, H, T, D = q.shape
    q32, k32, v32 = (torch.nn.functional.pad(t, (0, 32 - D)) for t in (q, k, v))  # head_dim 16 -> 32, zero padded
    scale_fix = (32 / D) ** 0.5  # keep softmax scale 1/sqrt(16)
    for mask_key, out_key in (("attn_mask_causal_valid", "attn_out_causal_valid"), ("attn_mask_ns", "attn_out_ns")):
        mask = torch.from_numpy(ops_golden[mask_key].copy())[:, None].expand(B, H, T, T)
        got = ops.flash_attention((q32 * scale_fix).cuda(), k32.cuda(), v32.cuda(), attn_mask=mask.cuda())
        assert got.dtype == torch.float32 and got.shape == (B, H, T, 32)
        want = torch.from_numpy(ops_golden[out_key])
        pos_self = ~mask[:, 0].any(dim=-1) | (mask[:, 0].sum(-1) == 1)
        err = (got.cpu()[..., :D] - want).abs()
        assert err.max().item() <= 2e-2
    lens = torch.from_numpy(ops_golden["attn_lens"].copy())
    key_mask = (torch.arange(T)[None] < lens[:, None])[:, None, None, :].expand(B, H, T, T)
    got = ops.flash_attention((q32 * scale_fix).cuda(), k32.cuda(), v32.cuda(), attn_mask=key_mask.cuda())
    assert (got.cpu()[..., :D] - torch.from_numpy(ops_golden["attn_out_keypad"])).abs().max().item() <= 2e-2
    got = ops.flash_attention((q32 * scale_fix).cuda(), k32.cuda(), v32.cuda(), is_causal=True)
    assert (got.cpu()[..., :D] - torch.from_numpy(ops_golden["attn_out_causal_nomask"])).abs().max().item() <= 2e-2


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("causal", [False, True])
def test_full_size_properties(kernel, causal):
    """Benchmark shape (heads 8, head_dim 64, L 1024, lengths U[32,1024]) on a batch slice: a sampled
    set of rows against the oracle, plus two size-independent properties — with v == 1 every computed
    row is exactly 1, and outputs are convex combinations (bounded by the value range)."""
    B, H, L, D = 64, 8, 1024, 64
    g = torch.Generator().manual_seed(8)
    q = (torch.randn(B, H, L, D, generator=g) / 8).bfloat16()
    k = (torch.randn(B, H, L, D, generator=g) / 8).bfloat16()
    v = (torch.randn(B, H, L, D, generator=g) / 8).bfloat16()
    lens = torch.randint(32, 1025, (B,), generator=g)
    kw = dict(seq_len=lens.cuda(), causal=causal, padded_query_self=causal, **_kw(kernel))
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    got = ops.varlen_attention(qd, kd, vd, **kw)
    ones = ops.varlen_attention(qd, kd, torch.ones_like(vd), **kw).float()
    valid_q = (torch.arange(L)[None] < lens[:, None]).cuda() if causal else torch.ones(B, L, dtype=torch.bool, device="cuda")
    sel = valid_q[:, None, :, None].expand_as(ones)
    assert (ones[sel] - 1.0).abs().max().item() <= 1e-2
    assert got.float().abs().max().item() <= v.float().abs().max().item() + 1e-3
    for b in (0, 17, 63):
        mask = R.structured_attention_mask(lens[b : b + 1], L, L, causal, causal)
        self_rows = (torch.arange(L)[None] >= lens[b : b + 1, None]) if causal else None
        _check(got[b : b + 1, :2], q[b : b + 1, :2], k[b : b + 1, :2], v[b : b + 1, :2], mask, self_rows)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("L", [1, 9, 17, 32])
def test_small_sample_kernel(dtype, L):
    """Kernel 3 (one warp per sample and head, at most 32 rows): every mask form of the other kernels."""
    B, H, D = 37, 3, 64
    q, k, v = _qkv(B, H, L, D, dtype, seed=40 + L)
    g = torch.Generator().manual_seed(L)
    lens = torch.randint(0, L + 1, (B,), generator=g)
    dq, dk, dv = q.cuda(), k.cuda(), v.cuda()
    # key padding, non-causal
    got = ops.varlen_attention(dq, dk, dv, seq_len=lens.cuda(), kernel=3)
    _check(got, q, k, v, R.structured_attention_mask(lens, L, L, False, False))
    # causal with a non-sequence suffix and padded queries returning their value rows
    ns = min(3, L)
    lens_ns = torch.minimum(lens, torch.tensor(L - ns))
    got = ops.varlen_attention(dq, dk, dv, seq_len=lens_ns.cuda(), ns_start=L - ns, causal=True, padded_query_self=True,
                               kernel=3)
    mask = R.structured_attention_mask(lens_ns, L, L - ns, True, True)
    pos = torch.arange(L)[None]
    self_rows = (pos >= lens_ns[:, None]) & (pos < L - ns)
    _check(got, q, k, v, mask, self_rows)
    # packed rows, causal: must agree with the mma.sync kernel on the same data
    lens_p = lens.clamp_min(1)
    cu = torch.zeros(B + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens_p, 0)
    rows = int(cu[-1])
    qkv = (torch.randn(rows, 3, H, D, generator=g) * 0.5).to(dtype).cuda()
    kw = dict(causal=True, cu_rows=cu.cuda(), max_rows=int(lens_p.max()))
    small = ops.varlen_attention(qkv[:, 0], qkv[:, 1], qkv[:, 2], kernel=3, **kw).float()
    ref = ops.varlen_attention(qkv[:, 0], qkv[:, 1], qkv[:, 2], kernel=1, **kw).float()
    assert (small - ref).abs().max().item() <= 1e-2
    # automatic choice takes this kernel for such samples and gives the same bits
    auto = ops.varlen_attention(qkv[:, 0], qkv[:, 1], qkv[:, 2], kernel=0, **kw).float()
    assert torch.equal(auto, small)


@pytest.mark.parametrize("causal", [True, False])
def test_packed_queries_are_the_last_rows_of_each_sample(causal):
    """cu_rows_q: q holds only the last rows of every sample; the result equals those rows of the full
    computation (the causal rule is aligned at the end of the sample)."""
    g = torch.Generator().manual_seed(77)
    B, H, D = 9, 4, 64
    lens = torch.tensor([300, 1, 64, 65, 17, 200, 128, 5, 90])
    keep = torch.tensor([40, 1, 64, 3, 0, 129, 70, 5, 1])        # 0 = no query for that sample
    cu = torch.zeros(B + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens, 0)
    cu_q = torch.zeros(B + 1, dtype=torch.int32)
    cu_q[1:] = torch.cumsum(keep, 0)
    rows = int(cu[-1])
    qkv = (torch.randn(rows, 3, H, D, generator=g) * 0.5).bfloat16().cuda()
    full = ops.varlen_attention(qkv[:, 0], qkv[:, 1], qkv[:, 2], causal=causal, cu_rows=cu.cuda(),
                                max_rows=int(lens.max()), kernel=1)
    sel = torch.cat([torch.arange(int(cu[b + 1]) - int(keep[b]), int(cu[b + 1])) for b in range(B)]).cuda()
    q_kept = qkv[:, 0].index_select(0, sel).contiguous()
    got = ops.varlen_attention(q_kept, qkv[:, 1], qkv[:, 2], causal=causal, cu_rows=cu.cuda(), max_rows=int(lens.max()),
                               cu_rows_q=cu_q.cuda(), max_rows_q=int(keep.max()))
    assert got.shape == q_kept.shape
    want = full.index_select(0, sel)
    assert (got.float() - want.float()).abs().max().item() <= 4e-3
    for kernel in (1, 4):   # the automatic choice above is the streaming kernel; both named ones agree as well
        named = ops.varlen_attention(q_kept, qkv[:, 1], qkv[:, 2], causal=causal, cu_rows=cu.cuda(), max_rows=int(lens.max()),
                                     cu_rows_q=cu_q.cuda(), max_rows_q=int(keep.max()), kernel=kernel)
        assert (named.float() - want.float()).abs().max().item() <= 4e-3
    # without separate query rows the streaming kernel computes the whole packed batch
    whole = ops.varlen_attention(qkv[:, 0], qkv[:, 1], qkv[:, 2], causal=causal, cu_rows=cu.cuda(),
                                 max_rows=int(lens.max()), kernel=4)
    assert (whole.float() - full.float()).abs().max().item() <= 4e-3
    with pytest.raises(RuntimeError):   # the tcgen05 kernel does not serve separate query rows
        ops.varlen_attention(q_kept, qkv[:, 1], qkv[:, 2], causal=causal, cu_rows=cu.cuda(), max_rows=int(lens.max()),
                             cu_rows_q=cu_q.cuda(), max_rows_q=int(keep.max()), kernel=2)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("max_keep", [4, 9, 16, 32])
def test_packed_queries_of_short_samples_take_the_small_kernel(causal, max_keep):
    """Samples of at most 32 rows with separate query rows: the one-warp kernel (explicitly and by the automatic
    choice) against the mma.sync kernel."""
    g = torch.Generator().manual_seed(max_keep)
    B, H, D = 37, 3, 64
    lens = torch.randint(1, 33, (B,), generator=g)
    lens[0], lens[1] = 32, 17
    keep = torch.minimum(torch.randint(0, max_keep + 1, (B,), generator=g), lens)
    keep[0], keep[1] = max_keep, min(9, max_keep)
    cu = torch.zeros(B + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens, 0)
    cu_q = torch.zeros(B + 1, dtype=torch.int32)
    cu_q[1:] = torch.cumsum(keep, 0)
    qkv = (torch.randn(int(cu[-1]), 3, H, D, generator=g) * 0.5).bfloat16().cuda()
    sel = torch.cat([torch.arange(int(cu[b + 1]) - int(keep[b]), int(cu[b + 1])) for b in range(B)]).cuda()
    q_kept = qkv[:, 0].index_select(0, sel).contiguous()
    kw = dict(causal=causal, cu_rows=cu.cuda(), max_rows=int(lens.max()), cu_rows_q=cu_q.cuda(), max_rows_q=int(keep.max()))
    ref = ops.varlen_attention(q_kept, qkv[:, 1], qkv[:, 2], kernel=1, **kw).float()
    small = ops.varlen_attention(q_kept, qkv[:, 1], qkv[:, 2], kernel=3, **kw).float()
    auto = ops.varlen_attention(q_kept, qkv[:, 1], qkv[:, 2], kernel=0, **kw).float()
    assert (small - ref).abs().max().item() <= 1e-2
    assert torch.equal(auto, small)
    full = ops.varlen_attention(qkv[:, 0], qkv[:, 1], qkv[:, 2], causal=causal, cu_rows=cu.cuda(), max_rows=int(lens.max()),
                                kernel=3).float()
    assert (small - full.index_select(0, sel)).abs().max().item() <= 4e-3   # the same rows of the full computation


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_streaming_kernel_on_views_of_a_fused_projection(dtype):
    """Kernel 4 with k / v as column slices of one [rows, 2 d] matrix and q from its own matrix, ragged key
    counts around the 16-row tile edges, against the fp32 oracle of the selected rows."""
    g = torch.Generator().manual_seed(5)
    H, D = 8, 64
    lens = torch.tensor([1, 15, 16, 17, 31, 32, 33, 48, 100, 257, 9, 2])
    keep = torch.tensor([1, 9, 16, 17, 9, 1, 20, 48, 9, 40, 0, 2])
    B = lens.numel()
    cu = torch.zeros(B + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens, 0)
    cu_q = torch.zeros(B + 1, dtype=torch.int32)
    cu_q[1:] = torch.cumsum(keep, 0)
    kv = (torch.randn(int(cu[-1]), 2 * H * D, generator=g) * 0.5).to(dtype).cuda()
    q = (torch.randn(int(cu_q[-1]), H * D, generator=g) * 0.5).to(dtype).cuda()
    k3, v3 = kv[:, : H * D].unflatten(-1, (H, D)), kv[:, H * D :].unflatten(-1, (H, D))
    got = ops.varlen_attention(q.unflatten(-1, (H, D)), k3, v3, causal=True, cu_rows=cu.cuda(), max_rows=int(lens.max()),
                               cu_rows_q=cu_q.cuda(), max_rows_q=int(keep.max()), kernel=4).float()
    scale = D ** -0.5
    for b in range(B):
        lk, lq = int(lens[b]), int(keep[b])
        if lq == 0:
            continue
        kb = k3[int(cu[b]) : int(cu[b + 1])].float().transpose(0, 1)      # [H, lk, D]
        vb = v3[int(cu[b]) : int(cu[b + 1])].float().transpose(0, 1)
        qb = q.unflatten(-1, (H, D))[int(cu_q[b]) : int(cu_q[b + 1])].float().transpose(0, 1)
        s = qb @ kb.transpose(1, 2) * scale
        pos = torch.arange(lq, device="cuda")[:, None] + (lk - lq)
        s = s.masked_fill(torch.arange(lk, device="cuda")[None, :] > pos, float("-inf"))
        want = (torch.softmax(s, -1) @ vb).transpose(0, 1)
        assert (got[int(cu_q[b]) : int(cu_q[b + 1])] - want).abs().max().item() <= 2e-2, b


def test_random_shapes_against_the_oracle():
    """Seeded sweep over ragged shapes and mask forms, every kernel that serves the shape, against the fp32 oracle."""
    g = torch.Generator().manual_seed(2026)
    for case in range(24):
        B = int(torch.randint(1, 6, (1,), generator=g))
        H = int(torch.randint(1, 4, (1,), generator=g))
        L = int(torch.randint(1, 300, (1,), generator=g))
        causal = bool(torch.randint(0, 2, (1,), generator=g))
        ns = int(torch.randint(0, min(L, 12) + 1, (1,), generator=g))
        lens = torch.randint(0, L - ns + 1, (B,), generator=g)
        q, k, v = _qkv(B, H, L, 64, torch.bfloat16, seed=1000 + case)
        mask = R.structured_attention_mask(lens, L, L - ns, causal, causal)
        pos = torch.arange(L)[None]
        self_rows = ((pos >= lens[:, None]) & (pos < L - ns)) if causal else None
        kernels = [1, 2] + ([3] if L <= 32 else [])
        for kernel in kernels:
            got = ops.varlen_attention(q.cuda(), k.cuda(), v.cuda(), seq_len=lens.cuda(), ns_start=L - ns, causal=causal,
                                       padded_query_self=causal, kernel=kernel, check=kernel == 2)
            try:
                _check(got, q, k, v, mask, self_rows)
            except AssertionError as exc:
                raise AssertionError(f"case {case}: B{B} H{H} L{L} ns{ns} causal={causal} kernel={kernel}: {exc}") from exc
        # packed form of the same samples (every row valid): kernels 1 and 2 against each other and the oracle
        rows_per = (lens + ns).clamp_min(1)
        cu = torch.zeros(B + 1, dtype=torch.int32)
        cu[1:] = torch.cumsum(rows_per, 0)
        qkv = (torch.randn(int(cu[-1]), 3, H, 64, generator=g) * 0.5).bfloat16().cuda()
        outs = [ops.varlen_attention(qkv[:, 0], qkv[:, 1], qkv[:, 2], causal=causal, cu_rows=cu.cuda(),
                                     max_rows=int(rows_per.max()), kernel=kern).float() for kern in (1, 2)]
        assert (outs[0] - outs[1]).abs().max().item() <= 1e-2, f"case {case}: packed kernels disagree"


@pytest.mark.parametrize("D", [32, 64, 20])
@pytest.mark.parametrize("L,ns", [(1, 0), (40, 0), (64, 9), (265, 9)])
def test_fp32_kernel_every_mask_family(D, L, ns):
    """fp32 q, k, v take the plain fp32 kernel (score-parity mode): against the fp32 oracle to 1e-5, for the
    causal-valid family with an always-valid suffix, key padding, an explicit key map, and a packed batch whose
    queries are the last rows of every sample."""
    B, H = 5, 2
    S = L - ns
    q, k, v = _qkv(B, H, L, D, torch.float32, seed=L + ns + D)
    lens = torch.tensor([S, 0, min(S, 1), S // 2, max(S - 1, 0)])
    got = ops.varlen_attention(q.cuda(), k.cuda(), v.cuda(), seq_len=lens.cuda(), ns_start=S, causal=True, padded_query_self=True)
    assert got.dtype == torch.float32
    pos = torch.arange(L)[None]
    _check(got, q, k, v, R.structured_attention_mask(lens, L, S, True, True), (pos >= lens[:, None]) & (pos < S), tol=1e-5)
    got = ops.varlen_attention(q.cuda(), k.cuda(), v.cuda(), seq_len=lens.clamp_min(1).cuda())
    _check(got, q, k, v, R.structured_attention_mask(lens.clamp_min(1), L, L, False, False), tol=1e-5)
    key_valid = torch.rand(B, L, generator=torch.Generator().manual_seed(L)) < 0.6
    key_valid[:, 0] = True
    got = ops.varlen_attention(q.cuda(), k.cuda(), v.cuda(), key_valid=key_valid.cuda())
    _check(got, q, k, v, key_valid[:, None, :].expand(B, L, L), tol=1e-5)
    # packed, queries = the last rows of every sample, causal rule aligned at the end
    lens_p = torch.tensor([L, max(1, L // 2), 1, L, max(1, L - 3)])
    keep = torch.tensor([min(L, 5), 1, 1, 0, 2]).clamp_max(lens_p)
    cu = torch.zeros(B + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens_p, 0)
    cu_q = torch.zeros(B + 1, dtype=torch.int32)
    cu_q[1:] = torch.cumsum(keep, 0)
    g = torch.Generator().manual_seed(9)
    kv = torch.randn(int(cu[-1]), 2, H, D, generator=g)
    sel = torch.cat([torch.arange(int(cu[i + 1]) - int(keep[i]), int(cu[i + 1])) for i in range(B)])
    qp = torch.randn(int(cu[-1]), H, D, generator=g) * D ** -0.25
    got = ops.varlen_attention(qp[sel].contiguous().cuda(), kv[:, 0].cuda(), kv[:, 1].cuda(), causal=True, cu_rows=cu.cuda(),
                               max_rows=L, cu_rows_q=cu_q.cuda(), max_rows_q=max(int(keep.max()), 1)).cpu()
    want = []
    for i in range(B):
        lo, hi = int(cu[i]), int(cu[i + 1])
        qi, ki, vi = (t[lo:hi].permute(1, 0, 2)[None] for t in (qp, kv[:, 0], kv[:, 1]))
        mask = torch.tril(torch.ones(hi - lo, hi - lo, dtype=torch.bool))[None, None]
        want.append(R.attention(qi, ki, vi, mask)[0].permute(1, 0, 2)[hi - lo - int(keep[i]):])
    assert (got - torch.cat(want)).abs().max().item() <= 1e-5
