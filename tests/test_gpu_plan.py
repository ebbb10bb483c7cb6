"""Row plan of the packed layout (`tb200_pyramid_plan`, `tb200_pyramid_kept_rows`) against the tensor arithmetic it
replaces, and the missing-value rows folded into the field pooling kernel against the two tensor operations of
`NonSequentialTokenizer.forward` (src/taac2026/infrastructure/modeling/tokenizers.py:66-68).  Integer results and
the pooled rows must be bit-identical."""
import pytest
import torch

from conftest import gpu_ready
from taac_2026_b200 import ops
from taac_2026_b200.onetrans import pyramid_keep_count

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_gpu():
    if not gpu_ready():
        pytest.fail("gpu tests need an sm_100 device and a built libtb200.so")


@pytest.mark.parametrize("batch,max_len,keep,layers,ns", [(1, 8, 8, 1, 0), (77, 96, 64, 3, 7), (8192, 1024, 1024, 8, 9),
                                                           (3000, 300, 200, 5, 2), (5, 16, 50, 2, 3)])
def test_plan_matches_tensor_arithmetic(batch, max_len, keep, layers, ns):
    g = torch.Generator().manual_seed(batch + layers)
    lengths = torch.randint(-2, max_len + 5, (batch,), generator=g).cuda()
    width = min(max_len, keep)
    widths = [width]
    for layer in range(layers):
        widths.append(pyramid_keep_count(widths[-1], layer, layers, ns))
    plan = ops.pyramid_plan(lengths, max_len, widths, ns)
    raw = lengths.clamp(min=0, max=max_len)
    assert torch.equal(plan["start"], (raw - width).clamp_min(0)) and torch.equal(plan["n0"], raw.clamp_max(width))
    n0 = raw.clamp_max(width)
    for l, w in enumerate(widths):
        counts = (n0 - (width - w)).clamp(min=0)
        rows = counts + ns
        cu = torch.zeros(batch + 1, dtype=torch.long, device="cuda")
        cu[1:] = torch.cumsum(rows, 0)
        assert torch.equal(plan["counts"][l], counts) and torch.equal(plan["cu"][l], cu)
        assert torch.equal(plan["cu32"][l], cu.to(torch.int32))
        assert plan["meta"][l].tolist() == [int(rows.sum()), int(rows.max())]
        if l == 0:
            assert torch.equal(plan["ns_rows0"], (cu[:-1] + counts)[:, None] + torch.arange(ns, device="cuda")[None, :])
    for l in range(layers):
        total0, total1 = int(plan["meta"][l][0]), int(plan["meta"][l + 1][0])
        src, ns_rows, row_dst = ops.pyramid_kept_rows(plan["cu"][l], plan["cu"][l + 1], plan["counts"][l], plan["counts"][l + 1],
                                                      ns, total0, total1, want_row_dst=True)
        rows1 = plan["counts"][l + 1] + ns
        owner = torch.repeat_interleave(torch.arange(batch, device="cuda"), rows1, output_size=total1)
        r = torch.arange(total1, device="cuda") - plan["cu"][l + 1][owner]
        want_src = plan["cu"][l][owner] + (plan["counts"][l] - plan["counts"][l + 1])[owner] + r
        assert torch.equal(src, want_src)
        assert torch.equal(ns_rows, (plan["cu"][l + 1][:-1] + plan["counts"][l + 1])[:, None] + torch.arange(ns, device="cuda")[None, :])
        want_dst = torch.full((total0,), -1, dtype=torch.int32, device="cuda")
        want_dst[want_src] = torch.arange(total1, dtype=torch.int32, device="cuda")
        assert torch.equal(row_dst, want_dst)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_missing_rows_inside_the_pooling_kernel(dtype):
    g = torch.Generator().manual_seed(4)
    batch, dim = 333, 64
    specs = [(50, 0, 1), (20, 1, 3), (70, 4, 2), (9, 6, 1)]              # (vocab, offset, bag length)
    tables = [torch.randn(v + 1, dim, generator=g).to(dtype).cuda() for v, _, _ in specs]
    fields = ops.FieldTables(tables, [o for _, o, _ in specs], [n for _, _, n in specs])
    ids = torch.randint(0, 60, (batch, 7), generator=g).cuda()
    missing = (torch.rand(batch, 7, generator=g) < 0.4).cuda()
    rows = (torch.randn(len(specs), dim, generator=g) * 0.02).to(dtype).cuda()
    plain = ops.fields_bag_mean(fields, ids)
    want = plain + missing[:, : len(specs)].to(dtype).unsqueeze(-1) * rows.unsqueeze(0)
    got = ops.fields_bag_mean(fields, ids, missing, rows)
    assert torch.equal(got, want)
    assert torch.equal(ops.fields_bag_mean(fields, ids, torch.zeros_like(missing), rows), plain)
