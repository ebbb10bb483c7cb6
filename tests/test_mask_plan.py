"""CPU tests of the attention mask planner: known answers taken from the reference planner
(golden fixture) plus a round-trip property over the whole mask family."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import reference_ops as R
from taac_2026_b200 import ops


def _expand(mask: torch.Tensor, heads: int) -> torch.Tensor:
    return mask[:, None].expand(mask.shape[0], heads, mask.shape[1], mask.shape[2])


def test_known_answers_from_reference_planner(ops_golden):
    q = torch.from_numpy(ops_golden["attn_q"].copy())
    B, H, T, _ = q.shape
    lens = torch.from_numpy(ops_golden["attn_lens"].copy())
    key_mask = _expand(R.structured_attention_mask(lens, T, T, False, False), H)
    plan = ops.plan_attention_mask(q, q, key_mask, is_causal=False)
    assert np.array_equal(plan.seq_len.numpy(), ops_golden["plan_keypad_lengths"])
    assert (plan.ns_start, plan.causal, plan.padded_query_self) == (T, False, False)
    cv = _expand(torch.from_numpy(ops_golden["attn_mask_causal_valid"].copy()), H)
    plan = ops.plan_attention_mask(q, q, cv, is_causal=False)
    assert np.array_equal(plan.seq_len.numpy(), ops_golden["plan_causal_valid_lengths"])
    assert (plan.ns_start, plan.causal, plan.padded_query_self) == (T, True, True)
    positions = torch.arange(T)[None]
    assert np.array_equal((positions >= plan.seq_len[:, None]).numpy(), ops_golden["plan_causal_valid_self"])
    ns = _expand(torch.from_numpy(ops_golden["attn_mask_ns"].copy()), H)
    plan = ops.plan_attention_mask(q, q, ns, is_causal=False)  # the reference planner rejects this one
    assert np.array_equal(plan.seq_len.numpy(), ops_golden["attn_ns_seq_lens"])
    assert (plan.ns_start, plan.causal, plan.padded_query_self) == (T - 5, True, True)


def test_no_mask_plans_full_lengths():
    q = torch.zeros(3, 2, 5, 8)
    k = torch.zeros(3, 2, 9, 8)
    plan = ops.plan_attention_mask(q, k, None, is_causal=True)
    assert plan.seq_len.tolist() == [9, 9, 9] and plan.causal and not plan.padded_query_self and plan.ns_start == 9


@pytest.mark.parametrize("seed", range(40))
def test_plan_reconstructs_mask(seed):
    """Whatever lengths the planner reports, the mask they describe equals the mask it was given."""
    g = torch.Generator().manual_seed(seed)
    T = int(torch.randint(1, 14, (1,), generator=g))
    ns = int(torch.randint(0, T + 1, (1,), generator=g))
    B = int(torch.randint(1, 6, (1,), generator=g))
    lens = torch.randint(0, T - ns + 1, (B,), generator=g)
    q = torch.zeros(B, 2, T, 8)
    for causal_self in (True, False):
        mask = R.structured_attention_mask(lens, T, T - ns, causal_self, causal_self)
        plan = ops.plan_attention_mask(q, q, _expand(mask, 2), is_causal=False)
        again = R.structured_attention_mask(plan.seq_len.long(), T, plan.ns_start, plan.causal, plan.padded_query_self)
        assert torch.equal(mask, again)


def test_unsupported_masks_raise_runtime_error():
    q = torch.zeros(1, 2, 4, 8)
    with pytest.raises(RuntimeError, match="structured bool"):
        ops.plan_attention_mask(q, q, torch.zeros(1, 2, 4, 4), is_causal=False)
    with pytest.raises(RuntimeError, match="4D bool masks"):
        ops.plan_attention_mask(q, q, torch.zeros(1, 4, 4, dtype=torch.bool), is_causal=False)
    per_head = torch.zeros(1, 2, 4, 4, dtype=torch.bool)
    per_head[:, 0] = True
    with pytest.raises(RuntimeError, match="shared across heads"):
        ops.plan_attention_mask(q, q, per_head, is_causal=False)
    holes = torch.tensor([True, False, True, False]).expand(1, 2, 4, 4)
    with pytest.raises(RuntimeError, match="valid prefix"):
        ops.plan_attention_mask(q, q, holes, is_causal=False)
    window = torch.tensor([[1, 0, 0, 0], [1, 1, 0, 0], [0, 1, 1, 0], [0, 0, 1, 1]]).bool().expand(1, 2, 4, 4)
    with pytest.raises(RuntimeError, match="causal_valid_attention_mask-style"):
        ops.plan_attention_mask(q, q, window, is_causal=False)


def test_flash_attention_argument_errors(monkeypatch):
    q = torch.zeros(1, 2, 4, 8)
    with pytest.raises(ValueError, match="shape \\(batch, heads, seq_len, head_dim\\)"):
        ops.flash_attention(q[0], q[0], q[0])
    with pytest.raises(ValueError, match="matching head counts"):
        ops.flash_attention(q, q[:, :1], q[:, :1])
    with pytest.raises(ValueError, match="unsupported flash_attention backend"):
        ops.flash_attention(q, q, q, backend="tilelang")
    with pytest.raises(RuntimeError, match="dropout_p to be in"):
        ops.flash_attention(q, q, q, dropout_p=1.5)
    with pytest.raises(RuntimeError, match="only supports dropout during training"):
        ops.flash_attention(q, q, q, dropout_p=0.1)
    monkeypatch.setattr(ops, "cuda_available", lambda: True)
    with pytest.raises(RuntimeError, match="requires CUDA tensors"):
        ops.flash_attention(q, q, q)
