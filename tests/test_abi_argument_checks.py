"""Argument validation of the C ABI, exercised without a GPU.

Every entry point checks shapes, null pointers, dtypes and alignment before it looks at the device, so the
rejections (and the empty-input successes) can be tested on any machine that can load ``libtb200.so``.  No
call here reaches a kernel launch."""

from __future__ import annotations

import ctypes

import pytest

from taac_2026_b200 import _lib

OK, ERR_NULL, ERR_DTYPE, ERR_SHAPE, ERR_ALIGN, ERR_UNSUPPORTED = 0, -1, -2, -3, -4, -5
BF16 = 2
P = ctypes.c_void_p


@pytest.fixture(scope="module")
def lib():
    if not _lib.LIB_PATH.exists():
        pytest.skip("libtb200.so is not built")
    return _lib.load()


def test_status_strings(lib):
    assert lib.tb200_strerror(OK).decode()
    for code in (ERR_NULL, ERR_DTYPE, ERR_SHAPE, ERR_ALIGN, ERR_UNSUPPORTED, -6, -7, -8):
        text = lib.tb200_strerror(code).decode()
        assert text and text != lib.tb200_strerror(OK).decode()


def test_norm_entries(lib):
    buf = (ctypes.c_uint8 * 256)()
    p = ctypes.addressof(buf)
    for fn, extra in ((lib.tb200_rmsnorm_fwd, ()), (lib.tb200_layernorm_fwd, (P(p),)), (lib.tb200_layernorm_silu_fwd, (P(p),))):
        assert fn(P(p), P(p), *extra, P(p), -1, 8, 1e-6, BF16, None) == ERR_SHAPE      # negative rows
        assert fn(P(p), P(p), *extra, P(p), 4, 0, 1e-6, BF16, None) == ERR_SHAPE       # no columns
        assert fn(P(p), P(p), *extra, P(p), 0, 8, 1e-6, BF16, None) == OK              # empty matrix: nothing to do
        assert fn(None, P(p), *extra, P(p), 4, 8, 1e-6, BF16, None) == ERR_NULL
    assert lib.tb200_rmsnorm_bias_fwd(P(p), None, P(p), P(p), 4, 8, 1e-6, BF16, None) == ERR_NULL
    assert lib.tb200_layernorm_fwd(P(p), P(p), None, P(p), 4, 8, 1e-6, BF16, None) == ERR_NULL


def test_row_kernel_entries(lib):
    buf = (ctypes.c_uint8 * 256)()
    p = ctypes.addressof(buf)
    assert lib.tb200_add_gathered_rows(P(p), 0, 8, P(p), 4, P(p), None, 0, None, BF16, None) == OK
    assert lib.tb200_add_gathered_rows(P(p), 4, 8, P(p), 0, P(p), None, 0, None, BF16, None) == ERR_SHAPE   # empty table
    assert lib.tb200_add_gathered_rows(P(p), 4, 8, None, 4, P(p), None, 0, None, BF16, None) == ERR_NULL
    assert lib.tb200_add_gathered_rows(P(p), 4, 8, P(p), 4, P(p), None, 0, None, 9, None) == ERR_DTYPE
    assert lib.tb200_add_gathered_rows(P(p), 4, 4, P(p), 4, P(p), None, 0, None, BF16, None) == ERR_ALIGN   # 8-byte rows
    assert lib.tb200_bias_act_rows(P(p), 0, 8, P(p), 1, 1, BF16, None) == OK
    assert lib.tb200_bias_act_rows(P(p), 4, 8, P(p), 0, 1, BF16, None) == ERR_SHAPE                       # group of zero rows
    assert lib.tb200_bias_act_rows(P(p), 4, 8, P(p), 1, 7, BF16, None) == ERR_UNSUPPORTED                 # unknown activation
    assert lib.tb200_bias_act_rows(P(p), 4, 8, None, 1, 0, BF16, None) == ERR_NULL


def test_attention_entry(lib):
    buf = (ctypes.c_uint8 * 256)()
    p = ctypes.addressof(buf)
    strides = (ctypes.c_int64 * 12)(*([64] * 12))

    def call(**kw):
        a = dict(q=P(p), k=P(p), v=P(p), o=P(p), B=2, H=2, Lq=4, Lk=4, D=64, strides=strides, seq_len=None, cu=None,
                 cu_q=None, kv=None, ns=4, causal=0, self_rows=0, scale=0.125, dtype=BF16, kernel=0, total=0)
        a.update(kw)
        return lib.tb200_attn_fwd(a["q"], a["k"], a["v"], a["o"], a["B"], a["H"], a["Lq"], a["Lk"], a["D"], a["strides"],
                                  a["seq_len"], a["cu"], a["cu_q"], a["kv"], a["ns"], a["causal"], a["self_rows"], a["scale"],
                                  a["dtype"], a["kernel"], a["total"], None, None)

    assert call(B=0) == OK and call(Lq=0) == OK                 # nothing to compute
    assert call(B=-1) == ERR_SHAPE and call(H=0) == ERR_SHAPE
    assert call(q=None) == ERR_NULL and call(strides=None) == ERR_NULL
    assert call(dtype=7) == ERR_DTYPE
    assert call(D=48) == ERR_UNSUPPORTED
    assert call(dtype=0, D=258) == ERR_UNSUPPORTED              # the fp32 kernel takes head dims up to 256
    assert call(self_rows=1, Lq=4, Lk=8) == ERR_SHAPE           # the self fallback needs a square problem
    assert call(ns=-1) == ERR_SHAPE
    assert call(cu_q=P(p)) == ERR_UNSUPPORTED                   # separate query rows need a packed batch
    bad = (ctypes.c_int64 * 12)(*([64] * 11 + [60]))
    assert call(strides=bad) == ERR_ALIGN                       # rows must start on 16-byte boundaries


def test_fp8_entries(lib):
    buf = (ctypes.c_uint8 * 256)()
    p = ctypes.addressof(buf)
    assert lib.tb200_quant_act_1x128(P(p), P(p), P(p), 0, 128, None) == OK
    assert lib.tb200_quant_act_1x128(P(p), P(p), P(p), 4, 100, None) == ERR_SHAPE          # K not a multiple of 128
    assert lib.tb200_quant_act_1x128(None, P(p), P(p), 4, 128, None) == ERR_NULL
    gemm = lib.tb200_fp8_gemm
    assert gemm(P(p), P(p), P(p), P(p), None, None, P(p), P(p), 0, 256, 128, 0, None, None) == OK
    assert gemm(P(p), P(p), P(p), P(p), None, None, P(p), P(p), 4, 200, 128, 0, None, None) == ERR_SHAPE   # N % 256
    assert gemm(P(p), P(p), P(p), P(p), None, None, P(p), P(p), 4, 256, 128, 5, None, None) == ERR_UNSUPPORTED
    assert gemm(P(p), P(p), P(p), P(p), None, None, P(p), None, 4, 256, 128, 1, None, None) == ERR_NULL    # scales out
    assert gemm(P(p), P(p), P(p), P(p), None, P(p), P(p), P(p), 4, 256, 128, 0, None, None) == ERR_UNSUPPORTED  # residual + swiglu
    assert lib.tb200_ffn_fp8_static_scratch_bytes() == 64 << 20


def test_grouped_gemm_entry(lib):
    buf = (ctypes.c_uint8 * 256)()
    p = ctypes.addressof(buf)
    gemm = lib.tb200_gemm_bf16_grouped
    assert gemm(P(p), P(p), None, None, P(p), 0, 8, 256, 64, 0, None, None) == OK            # no group
    assert gemm(P(p), P(p), None, None, P(p), 3, 0, 256, 64, 0, None, None) == OK            # no row
    assert gemm(P(p), P(p), None, None, P(p), 3, 8, 200, 64, 0, None, None) == ERR_SHAPE     # N % 256
    assert gemm(P(p), P(p), None, None, P(p), 3, 8, 256, 48, 0, None, None) == ERR_SHAPE     # K % 64
    assert gemm(P(p), P(p), None, None, P(p), -1, 8, 256, 64, 0, None, None) == ERR_SHAPE
    assert gemm(P(p), P(p), None, None, P(p), 3, 8, 256, 64, 3, None, None) == ERR_UNSUPPORTED   # unknown activation
    assert gemm(P(p), P(p), None, P(p), P(p), 3, 8, 256, 64, 2, None, None) == ERR_UNSUPPORTED   # the gated epilogue takes no residual
    assert gemm(None, P(p), None, None, P(p), 3, 8, 256, 64, 0, None, None) == ERR_NULL
    assert gemm(P(p), P(p), None, None, None, 3, 8, 256, 64, 0, None, None) == ERR_NULL
    assert gemm(P(p + 8), P(p), None, None, P(p), 3, 8, 256, 64, 0, None, None) == ERR_ALIGN


def test_token_tail_entries(lib):
    buf = (ctypes.c_uint8 * 256)()
    p = ctypes.addressof(buf)
    sel = lib.tb200_token_tail_select_fwd

    def call(**kw):
        a = dict(x=P(p), g=P(p), b=P(p), ta=P(p), rows_a=4, ia=P(p), tb=None, rows_b=0, ib=None, g2=P(p), dst=None, rows_out=0,
                 tokens=P(p), normed=P(p), rows=4, cols=8)
        a.update(kw)
        return sel(a["x"], a["g"], a["b"], a["ta"], a["rows_a"], a["ia"], a["tb"], a["rows_b"], a["ib"], a["g2"], a["dst"],
                   a["rows_out"], a["tokens"], a["normed"], a["rows"], a["cols"], 1e-5, 1e-6, BF16, None)

    assert call(rows=0) == OK
    assert call(rows=-1) == ERR_SHAPE and call(rows_a=0) == ERR_SHAPE
    assert call(x=None) == ERR_NULL and call(normed=None) == ERR_NULL and call(tokens=None) == ERR_NULL
    assert call(tb=P(p), rows_b=4, ib=None) == ERR_NULL                     # a second table needs its ids
    assert call(dst=P(p), rows_out=-1) == ERR_SHAPE
    assert call(rows_a=1 << 31) == ERR_UNSUPPORTED                          # ids are held as 32-bit values
    assert lib.tb200_token_tail_fwd(P(p), P(p), P(p), P(p), 4, P(p), None, 0, None, P(p), P(p), P(p), 0, 8, 1e-5, 1e-6, BF16,
                                    None) == OK


def test_static_ffn_entry_checks_everything_before_it_launches(lib):
    """A negative status from the no-allocation entry point means that none of its three kernels was enqueued:
    the checks of all three steps (shapes up to the K limit of the GEMMs, NULL and alignment of every pointer,
    the row bound) come first.  On a machine without a GPU the valid call itself ends at the device check."""
    buf = (ctypes.c_uint8 * 512)()
    p = ctypes.addressof(buf)
    p16 = (p + 15) & ~15
    ffn = lib.tb200_ffn_fp8_fwd_static
    ERR_SCRATCH = -8

    def call(**kw):
        a = dict(x=P(p16), wu=P(p16), su=P(p16), bu=None, wd=P(p16), sd=P(p16), bd=None, res=None, y=P(p16), M=64, d_in=512,
                 hidden=2048, d_out=512, gated=0)
        a.update(kw)
        return ffn(a["x"], a["wu"], a["su"], a["bu"], a["wd"], a["sd"], a["bd"], a["res"], a["y"], a["M"], a["d_in"],
                   a["hidden"], a["d_out"], a["gated"], None)

    assert call(M=0) == OK
    assert call(M=-1) == ERR_SHAPE and call(d_in=100) == ERR_SHAPE and call(hidden=128) == ERR_SHAPE and call(d_out=100) == ERR_SHAPE
    assert call(d_in=8192 + 128) == ERR_SHAPE and call(hidden=8192 + 256) == ERR_SHAPE   # the GEMMs' K limit, found up front
    assert call(x=None) == ERR_NULL and call(y=None) == ERR_NULL and call(sd=None) == ERR_NULL
    assert call(wd=P(p16 + 8)) == ERR_ALIGN and call(res=P(p16 + 4)) == ERR_ALIGN and call(y=P(p16 + 2)) == ERR_ALIGN
    assert call(M=(64 << 20) // (512 + 2048) + 1) == ERR_SCRATCH
    assert call(M=1 << 62) == ERR_SCRATCH          # no wrap-around of the size products
    assert call(M=(1 << 31) + 5) == ERR_SCRATCH
    assert lib.tb200_ffn_fp8_static_status(None, None) == ERR_NULL


def test_entries_added_for_the_host_loop_and_the_training_slice(lib):
    buf = (ctypes.c_uint8 * 4096)()
    p = ctypes.addressof(buf) + (16 - ctypes.addressof(buf) % 16) % 16      # a 16-byte aligned address inside the buffer
    strides = (ctypes.c_int64 * 12)(*([64] * 12))
    widths = (ctypes.c_int32 * 3)(8, 4, 2)
    ERR_RANGE = -9
    assert lib.tb200_strerror(ERR_RANGE).decode() != lib.tb200_strerror(OK).decode()
    # compact host format
    assert lib.tb200_host_compact_offsets(None, 0, 8, P(p)) == OK
    assert lib.tb200_host_compact_offsets(None, 4, 8, P(p)) == ERR_NULL
    assert lib.tb200_host_compact_sequence(P(p), None, None, P(p), 0, 1, 8, P(p), 8, None, 1) == OK
    assert lib.tb200_host_compact_sequence(P(p), None, None, P(p), 2, 0, 8, P(p), 8, None, 1) == ERR_SHAPE   # no feature
    assert lib.tb200_expand_sequence(P(p), None, P(p), None, P(p), P(p), None, 2, 1, 7, 8, None) == ERR_ALIGN   # odd max_len
    assert lib.tb200_expand_sequence(P(p), None, P(p), None, P(p), P(p), P(p), 2, 1, 8, 8, None) == ERR_NULL    # timestamps without gaps
    assert lib.tb200_expand_sequence(None, None, None, None, None, None, None, 0, 1, 8, 8, None) == OK
    # row plan
    assert lib.tb200_pyramid_plan(P(p), 4, 8, widths, 65, 2, P(p), P(p), P(p), P(p), P(p), P(p), P(p), None) == ERR_SHAPE
    assert lib.tb200_pyramid_plan(P(p), 4, 8, None, 2, 2, P(p), P(p), P(p), P(p), P(p), P(p), P(p), None) == ERR_NULL
    assert lib.tb200_pyramid_kept_rows(None, None, None, None, 0, 2, None, None, None, None) == OK
    assert lib.tb200_pyramid_kept_rows(P(p), P(p), P(p), P(p), 4, 2, None, P(p), None, None) == ERR_NULL
    # backward kernels
    assert lib.tb200_attn_bwd(P(p), P(p), P(p), P(p), P(p), P(p), P(p), P(p), P(p), 1, 1, 8, 8, 300, strides, None, None, 8, 0, 0,
                              0.125, BF16, None) == ERR_UNSUPPORTED                                   # head_dim above 256
    assert lib.tb200_attn_bwd(P(p), P(p), P(p), P(p), P(p), P(p), P(p), P(p), None, 1, 1, 8, 8, 64, strides, None, None, 8, 0, 0,
                              0.125, BF16, None) == ERR_NULL                                          # no workspace
    assert lib.tb200_attn_bwd(P(p), P(p), P(p), P(p), P(p), P(p), P(p), P(p), P(p), 1, 1, 8, 16, 64, strides, None, None, 16, 0, 1,
                              0.125, BF16, None) == ERR_SHAPE                                         # padded-self needs Lq == Lk
    assert lib.tb200_attn_bwd_workspace_bytes(2, 3, 5) == 2 * 3 * 5 * 8
    assert lib.tb200_bag_mean_bwd(P(p), 1, P(p), P(p), P(p), 4, 2, 12, 10, BF16, None) == ERR_ALIGN      # 24-byte rows
    assert lib.tb200_bag_mean_bwd(P(p), 1, P(p), P(p), P(p), 0, 2, 8, 10, BF16, None) == OK
    # block-scaled FFN
    assert lib.tb200_mx_scale_bytes(300, 512) == 3 * 4 * 512
    assert lib.tb200_quant_act_mx(P(p), P(p), P(p), 4, 100, None) == ERR_SHAPE
    assert lib.tb200_quant_act_mx(P(p), P(p), None, 4, 128, None) == ERR_NULL
    assert lib.tb200_mx_gemm(P(p), P(p), P(p), P(p), None, None, P(p), None, 4, 256, 128, 0, None, None) == ERR_NULL   # no scale output
    assert lib.tb200_mx_gemm(P(p), P(p), P(p), P(p), None, P(p), P(p), P(p), 4, 256, 128, 1, None, None) == ERR_UNSUPPORTED
    assert lib.tb200_mx_gemm(P(p), P(p), P(p), P(p), None, None, P(p), None, 4, 200, 128, 2, None, None) == ERR_SHAPE
    assert lib.tb200_mx_gemm(P(p), P(p), P(p), P(p), None, None, P(p), None, 0, 256, 128, 2, None, None) == OK
