"""The FFN entry point that allocates nothing (``tb200_ffn_fp8_fwd_static``).

Some callers of this library cannot obtain device memory at the moment they run a layer: a serving
loop whose memory plan was fixed at start-up, or a plugin inside a host runtime that owns the
allocator.  For them the library carries a fixed scratch array and one entry point that runs the
whole FP8 FFN out of it.  This test drives that entry point through the C ABI (ctypes, raw device
pointers) and checks that, on two calls in a row with different inputs and sizes, it writes exactly
what the existing three-call path (quantise, GEMM 1, GEMM 2 with caller-provided buffers) writes —
the kernels are the same, so the comparison is bit for bit — and that a request larger than the
array is refused with a clear error instead of being launched.

The file name sorts last on purpose: a run that stops at the first failure has by then exercised
every other test.  It also passes when run alone in a fresh process (the first call does the
one-time address lookup of the scratch array).
"""

from __future__ import annotations

import ctypes

import pytest
import torch

from conftest import gpu_ready
from taac_2026_b200 import _lib, ops

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_gpu():
    if not gpu_ready():
        pytest.fail("gpu tests need an sm_100 device and a built libtb200.so")


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _call_static(x, w, out, residual=None):
    lib = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.tb200_ffn_fp8_fwd_static(
        _ptr(x), _ptr(w.w_up), _ptr(w.s_up), _ptr(w.b_up), _ptr(w.w_down), _ptr(w.s_down), _ptr(w.b_down),
        _ptr(residual), _ptr(out), x.shape[0], x.shape[1], w.hidden, w.w_down.shape[0], int(w.gated), stream,
    )


@pytest.mark.parametrize("gated", [True, False])
def test_static_scratch_ffn_matches_three_call_path(gated):
    g = torch.Generator(device="cuda").manual_seed(11 + int(gated))
    d, hidden = 512, 2048
    w_up = (torch.randn((2 if gated else 1) * hidden, d, generator=g, device="cuda") * 0.02).bfloat16()
    w_down = (torch.randn(d, hidden, generator=g, device="cuda") * 0.02).bfloat16()
    b_up = None if gated else torch.randn(hidden, generator=g, device="cuda") * 0.05
    b_down = torch.randn(d, generator=g, device="cuda") * 0.05
    weights = ops.Fp8FfnWeights(w_up, w_down, gated=gated, b_up=b_up, b_down=b_down)
    # two calls in a row: a larger request first, then a smaller one with other data, so that stale
    # bytes of the first call lie behind and beside everything the second call uses
    for rows, with_residual in ((3000, True), (777, False)):
        x = torch.randn(rows, d, generator=g, device="cuda").bfloat16()
        residual = torch.randn(rows, d, generator=g, device="cuda").bfloat16() if with_residual else None
        want = ops.ffn_fp8(x, weights, residual=residual, check=True)  # existing entry points, caller-owned buffers
        out = torch.full((rows, d), float("nan"), dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        assert _call_static(x, weights, out, residual) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before  # the torch allocator was not touched
        assert torch.isfinite(out.float()).all()
        assert torch.equal(out, want)
        # the status word lives in the same fixed array: reading it allocates nothing either
        value = ctypes.c_int32(-1)
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        assert _lib.load().tb200_ffn_fp8_static_status(stream, ctypes.byref(value)) == 0
        assert value.value == 0 and torch.cuda.memory_allocated() == before
    assert ops.ffn_fp8_static_status() == 0
    # the Python wrapper is the same call
    out2 = torch.empty_like(out)
    assert torch.equal(ops.ffn_fp8_static(x, weights, out2), want)


def test_request_beyond_the_fixed_array_is_refused():
    lib = _lib.load()
    capacity = int(lib.tb200_ffn_fp8_static_scratch_bytes())
    assert capacity == ops.ffn_fp8_static_capacity() == 64 << 20
    d, hidden = 512, 2048
    weights = ops.Fp8FfnWeights(torch.zeros(hidden, d, device="cuda").bfloat16(), torch.zeros(d, hidden, device="cuda").bfloat16(), gated=False)
    rows = capacity // (d + hidden) + 1  # needs more than the array even before the scale vectors
    x = torch.zeros(rows, d, dtype=torch.bfloat16, device="cuda")
    out = torch.ones(rows, d, dtype=torch.bfloat16, device="cuda")
    code = _call_static(x, weights, out)
    assert code == -8
    assert "fixed scratch" in _lib.strerror(code)
    torch.cuda.synchronize()
    assert torch.equal(out, torch.ones_like(out))  # nothing was launched
    with pytest.raises(ValueError, match="fixed scratch"):
        ops.ffn_fp8_static(x, weights, out)
    # the largest request that fits still runs
    fit = rows - 1
    while fit * (d + hidden) + 256 * 5 + fit * ((d + hidden) // 128) * 4 > capacity:   # four parts and the status word, 256-byte units
        fit -= 64
    assert _call_static(x[:fit], weights, out[:fit]) == 0
    torch.cuda.synchronize()
    assert torch.equal(out[:fit], torch.zeros_like(out[:fit]))  # zero weights, no bias: zeros
