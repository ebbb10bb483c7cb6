"""Attention backward (`tb200_attn_bwd`) against torch autograd of the fp32 masked-softmax form, for every mask
family of the forward kernels, at the reference's backward tolerance (1e-2 for 16-bit tensors,
tests/gpu/infrastructure/accelerators/test_tilelang_ops_cuda.py:187-306)."""
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


def _mask(batch, lq, lk, seq_len, ns_start, causal, padded_self, key_valid=None):
    kpos, qpos = torch.arange(lk)[None, None, :], torch.arange(lq)[None, :, None]
    if key_valid is not None:
        visible = key_valid[:, None, :].bool().expand(batch, lq, lk).clone()
        padded_q = ~key_valid.bool()
    else:
        lens = torch.full((batch,), lk) if seq_len is None else seq_len
        key_ok = (kpos < lens[:, None, None]) | (kpos >= ns_start)
        visible = key_ok.expand(batch, lq, lk).clone()
        pos = torch.arange(lq)[None, :]
        padded_q = (pos >= lens[:, None]) & (pos < ns_start)
    if causal:
        visible &= kpos <= qpos
    if padded_self:
        eye = torch.eye(lq, lk, dtype=torch.bool)[None]
        visible = torch.where(padded_q[:, :, None], eye.expand(batch, -1, -1), visible)
    return visible


def _reference(q, k, v, visible, scale):
    """fp32 masked softmax attention with autograd; rows without a visible key give zeros."""
    s = torch.einsum("bhqd,bhkd->bhqk", q, k) * scale
    s = s.masked_fill(~visible[:, None], float("-inf"))
    any_visible = visible.any(dim=-1)[:, None, :, None]
    p = torch.softmax(torch.where(any_visible, s, torch.zeros_like(s)), dim=-1)
    p = torch.where(any_visible, p, torch.zeros_like(p)) * visible[:, None]
    return torch.einsum("bhqk,bhkd->bhqd", p, v)


CASES = [
    # batch, heads, lq, lk, dim, causal, with lengths, ns suffix, padded-self
    (2, 2, 17, 17, 64, False, True, 0, False),
    (3, 2, 40, 40, 32, True, True, 0, False),
    (2, 4, 33, 33, 64, False, True, 5, True),
    (2, 2, 50, 50, 128, True, True, 9, True),
    (1, 1, 8, 24, 64, False, False, 0, False),       # more keys than queries, no mask
    (2, 3, 70, 70, 64, True, False, 0, False),
]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("batch,heads,lq,lk,dim,causal,with_len,ns,padded_self", CASES)
def test_backward_matches_autograd(batch, heads, lq, lk, dim, causal, with_len, ns, padded_self, dtype, tol):
    g = torch.Generator().manual_seed(lq * 7 + dim)
    q, k, v = (torch.randn(batch, heads, n, dim, generator=g).to(dtype) for n in (lq, lk, lk))
    grad = torch.randn(batch, heads, lq, dim, generator=g).to(dtype)
    ns_start = lk - ns
    seq_len = torch.randint(0, ns_start + 1, (batch,), generator=g) if with_len else None
    if seq_len is not None:
        seq_len[0] = 0 if not causal else 1            # a sample whose prefix is (almost) empty
    visible = _mask(batch, lq, lk, seq_len, ns_start, causal, padded_self)
    scale = dim ** -0.5
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    out_ref = _reference(qr, kr, vr, visible, scale)
    out_ref.backward(grad.float())
    lens_dev = None if seq_len is None else seq_len.to(torch.int32).cuda()
    out = ops.varlen_attention(q.cuda(), k.cuda(), v.cuda(), seq_len=lens_dev, ns_start=ns_start, causal=causal,
                               padded_query_self=padded_self, layout="bhld")
    dq, dk, dv = ops.attention_backward(q.cuda(), k.cuda(), v.cuda(), out, grad.cuda(), seq_len=lens_dev, ns_start=ns_start,
                                        causal=causal, padded_query_self=padded_self)
    for got, want, name in ((dq, qr.grad, "dq"), (dk, kr.grad, "dk"), (dv, vr.grad, "dv")):
        err = (got.float().cpu() - want).abs().max().item()
        assert err <= tol * max(1.0, want.abs().max().item()), f"{name}: {err}"


def test_key_validity_map_and_autograd_route():
    g = torch.Generator().manual_seed(3)
    batch, heads, length, dim = 2, 2, 24, 64
    q, k, v = (torch.randn(batch, heads, length, dim, generator=g) for _ in range(3))
    valid = torch.rand(batch, length, generator=g) < 0.7
    valid[:, 0] = True
    visible = _mask(batch, length, length, None, length, False, False, key_valid=valid)
    qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
    grad = torch.randn(batch, heads, length, dim, generator=g)
    out_ref = _reference(qr, kr, vr, visible, dim ** -0.5)
    out_ref.backward(grad)
    dq, dk, dv = ops.attention_backward(q.cuda(), k.cuda(), v.cuda(), out_ref.detach().cuda(), grad.cuda(),
                                        key_valid=valid.cuda())
    for got, want in ((dq, qr.grad), (dk, kr.grad), (dv, vr.grad)):
        assert (got.cpu() - want).abs().max().item() <= 2e-4 * max(1.0, want.abs().max().item())
    # the dispatcher under autograd: forward on the serving kernel, backward on this one
    qc, kc, vc = (t.bfloat16().cuda().requires_grad_() for t in (q, k, v))
    mask = torch.ones(batch, 1, length, length, dtype=torch.bool).tril().cuda()
    out = ops.flash_attention(qc, kc, vc, attn_mask=None, is_causal=True)
    out.backward(grad.bfloat16().cuda())
    qr2, kr2, vr2 = (t.bfloat16().float().requires_grad_() for t in (q, k, v))
    _reference(qr2, kr2, vr2, mask[:, 0].cpu().expand(batch, -1, -1), dim ** -0.5).backward(grad.bfloat16().float())
    for got, want in ((qc.grad, qr2.grad), (kc.grad, kr2.grad), (vc.grad, vr2.grad)):
        assert got is not None and (got.float().cpu() - want).abs().max().item() <= 2e-2 * max(1.0, want.abs().max().item())
