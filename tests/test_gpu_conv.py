"""Convolution forward / data gradient / filter gradient against the oracle.
fp32 NCHW path: max-relative 1e-5.  bf16 NHWC tensor-core path: max-relative 2e-2 against the
oracle evaluated on the bf16-rounded operands (fp32 accumulate on both sides)."""
import ctypes as C

import numpy as np
import pytest

from arraydiff_cuda_b200 import abi
from oracle import orc
from tests import helpers as H

pytestmark = pytest.mark.gpu
TOL_F32 = 1e-5
TOL_BF16 = 2e-2


def _khw(k):
    return (k, k) if isinstance(k, int) else tuple(k)


def _out_dims(Hh, W, k, s, d, pd):
    kh, kw = _khw(k)
    return (Hh + 2 * pd - d * (kh - 1) - 1) // s + 1, (W + 2 * pd - d * (kw - 1) - 1) // s + 1


def conv_args(dtype, layout, x_shape_nchw, K, k, stride, dil, pad):
    N, Cc, Hh, W = x_shape_nchw
    kh, kw = _khw(k)
    a = abi.Conv2dArgs()
    a.dtype, a.layout = dtype, layout
    a.N, a.C, a.H, a.W, a.K, a.kh, a.kw = N, Cc, Hh, W, K, kh, kw
    a.stride_h = a.stride_w = stride
    a.dil_h = a.dil_w = dil
    a.pad_h = a.pad_w = pad
    return a


F32_CASES = [
    # N, C, H, W, K, k, stride, dil, pad
    (1, 3, 9, 10, 4, 3, 1, 1, 1),
    (2, 4, 11, 9, 5, 3, 2, 1, 1),
    (1, 2, 12, 12, 3, 3, 1, 2, 2),
    (1, 3, 37, 41, 8, 7, 2, 1, 3),
    (2, 5, 6, 7, 6, 1, 1, 1, 0),
    (1, 64, 34, 66, 64, 3, 1, 1, 0),   # one halo-padded strip of benchmark config 1 (h=32, p=1)
]


@pytest.mark.parametrize("case", F32_CASES)
def test_conv_fp32_direct(case):
    import torch
    N, Cc, Hh, W, K, k, s, d, pd = case
    x, w, b = H.uniform(1, (N, Cc, Hh, W)), H.normal(2, (K, Cc, k, k), float(np.sqrt(2.0 / (k * k * Cc)))), H.normal(3, (K,))
    y_w = orc.conv2d_fprop(x, w, b, (s, s), (d, d), (pd, pd), omp=True)
    dy = H.uniform(4, y_w.shape)
    dx_w = orc.conv2d_dgrad(dy, w, x.shape, (s, s), (d, d), (pd, pd), omp=True)
    db_w = np.zeros(K, np.float32)
    dw_w = orc.conv2d_wgrad(x, dy, w.shape, (s, s), (d, d), (pd, pd), db=db_w, omp=True)
    L = abi.lib()
    a = conv_args(abi.AD_F32, abi.AD_NCHW, x.shape, K, k, s, d, pd)
    dx_, dw_, db_ = H.dev(x), H.dev(w), H.dev(b)
    y = torch.empty(y_w.shape, device="cuda")
    a.x, a.w, a.bias, a.y = dx_.data_ptr(), dw_.data_ptr(), db_.data_ptr(), y.data_ptr()
    abi.check(L.ad_conv2d_fprop(C.byref(a), H.stream()))
    H.sync()
    assert H.max_rel(H.host(y), y_w) < TOL_F32
    ddy = H.dev(dy)
    gdx, gdw, gdb = torch.ones(x.shape, device="cuda"), torch.ones(w.shape, device="cuda"), torch.ones(K, device="cuda")
    a.y, a.dx, a.dw, a.db, a.accumulate = ddy.data_ptr(), gdx.data_ptr(), gdw.data_ptr(), gdb.data_ptr(), 1
    abi.check(L.ad_conv2d_dgrad(C.byref(a), H.stream()))
    abi.check(L.ad_conv2d_wgrad(C.byref(a), H.stream()))
    H.sync()
    assert H.max_rel(H.host(gdx) - 1, dx_w) < TOL_F32      # accumulate: += on top of the ones
    assert H.max_rel(H.host(gdw) - 1, dw_w) < 2 * TOL_F32
    assert H.max_rel(H.host(gdb) - 1, db_w) < 2 * TOL_F32


TC_CASES = [
    # N, C, H, W, K, k, stride, dil, pad           (H, W are the dims the kernel reads)
    (1, 64, 16, 16, 64, 1, 1, 1, 0),     # 1x1, single tile row block
    (2, 64, 13, 21, 256, 1, 1, 1, 0),    # 1x1 64->256, ragged tiles
    (1, 256, 9, 40, 64, 1, 1, 1, 0),     # 1x1 256->64, 4 channel slabs
    (1, 64, 18, 34, 64, 3, 1, 1, 0),     # 3x3 on a halo-padded strip (h=16, W=32, p=1)
    (2, 64, 20, 20, 128, 3, 1, 2, 0),    # dilated 3x3 (d=2) on a halo-2 strip
    (1, 128, 24, 24, 64, 3, 1, 4, 0),    # dilated 3x3 (d=4)
    (1, 64, 17, 19, 64, 3, 1, 1, 1),     # implicit zero padding through out-of-bounds fill
    (1, 64, 34, 34, 128, 3, 2, 1, 0),    # 3x3 stride 2 on a padded strip
    (1, 64, 32, 32, 256, 1, 2, 1, 0),    # 1x1 stride 2 projection
    (2, 64, 35, 33, 64, 3, 2, 1, 0),     # 3x3 stride 2, odd extents (trailing input rows / columns unused)
    (1, 192, 12, 140, 64, 1, 1, 1, 0),   # the 7x7 stem after im2col: K = 147 padded to 192
    (1, 64, 8, 8, 19, 1, 1, 1, 0),       # 19-class head (ragged output channels)
    (2, 128, 10, 12, 19, 1, 1, 1, 0),    # 19-class head, 2 channel slabs
    (8, 64, 7, 7, 128, 3, 1, 1, 1),      # 7x7 maps: a tile spans 16 images (here 8 real ones)
    (5, 128, 14, 14, 64, 1, 1, 1, 0),    # 14x14 maps: 4 images per tile, ragged last block of images
    (3, 64, 9, 9, 19, 3, 1, 1, 1),       # small maps through the scattered-store epilogue (ragged channels)
    (1, 256, 14, 30, 128, 3, 1, 2, 0),   # 256 input channels: the filter gradient's 256-wide channel tile
    (2, 512, 12, 20, 64, 1, 1, 1, 0),    # 512 input channels, 1x1: two 256-wide channel tiles
]


# Shapes served by the row-streaming kernels (64 input channels, at most 64 output channels, stride 1, rows of at
# least 96 output pixels): the kernels behind every wide 64-channel layer.  The last three entries name the kernel
# family (abi.CONV_TC_*) that forward, data gradient and filter gradient must report for the shape.
ROW, GEN = abi.CONV_TC_ROW, abi.CONV_TC_GENERAL
ROW_CASES = [
    # N, C, H, W, K, k, stride, dil, pad, (fprop, dgrad, wgrad kernel family)
    (2, 64, 22, 140, 64, 3, 1, 3, 0, (ROW, ROW, ROW)),      # 3x3 dilation 3 on a halo-3 strip, one ragged tile pair
    (1, 64, 12, 200, 64, 3, 1, 1, 1, (ROW, ROW, ROW)),      # 3x3 with implicit zero padding (out-of-bounds fill)
    (1, 64, 14, 300, 64, 3, 1, 2, 0, (ROW, ROW, ROW)),      # 3x3 dilation 2, three tiles per row
    (1, 64, 11, 98, 64, 3, 1, 1, 0, (ROW, ROW, ROW)),       # the narrowest row the kernels take (96 output pixels)
    (1, 64, 7, 263, 64, 3, 1, 1, 0, (ROW, ROW, ROW)),       # 261 output pixels: a 5-pixel trailing tile
    (3, 64, 8, 100, 8, 3, 1, 1, 0, (ROW, ROW, ROW)),        # 8 output channels, 3 images
    (1, 64, 9, 130, 32, 1, 1, 1, 0, (ROW, ROW, ROW)),       # 1x1, 32 output channels
    (3, 64, 5, 257, 64, 1, 1, 1, 0, (ROW, ROW, ROW)),       # 1x1, ragged width
    (1, 64, 10, 131, 24, 2, 1, 1, 0, (ROW, ROW, ROW)),      # 2x2: the filter-extent-at-run-time instantiation
    (1, 64, 12, 140, 64, (3, 1), 1, 2, 0, (ROW, ROW, ROW)), # 3x1 column filter, dilation 2
    (1, 64, 9, 150, 48, (1, 3), 1, 1, 0, (ROW, ROW, ROW)),  # 1x3 row filter
    (1, 64, 6, 160, 19, 1, 1, 1, 0, (ROW, ROW, GEN)),       # 19-class head on a wide map: ragged output channels
    (1, 64, 22, 518, 64, 3, 1, 3, 0, (ROW, ROW, ROW)),      # one image of the benchmark strip: 16 x 512 out, dil 3
    (2, 64, 19, 1030, 64, 3, 1, 1, 0, (ROW, ROW, ROW)),     # stage-1 3x3 of a 1024-wide strip
]


def _kinds(case):
    return case[9] if len(case) > 9 else (None, None, None)


def _tc_setup(case, seed=10):
    N, Cc, Hh, W, K, k, s, d, pd = case[:9]
    kh, kw = _khw(k)
    x = orc.round_bf16(H.uniform(seed, (N, Cc, Hh, W)))
    w = orc.round_bf16(H.normal(seed + 1, (K, Cc, kh, kw), float(np.sqrt(2.0 / (kh * kw * Cc)))))
    return x, w


def _check_kind(L, want):
    if want is not None:
        assert L.ad_conv2d_last_kernel() == want, (L.ad_conv2d_last_kernel(), want)


@pytest.mark.parametrize("case", TC_CASES + ROW_CASES)
def test_conv_tc_fprop(case):
    import torch
    N, Cc, Hh, W, K, k, s, d, pd = case[:9]
    x, w = _tc_setup(case)
    b = H.normal(12, (K,))
    y_w = orc.conv2d_fprop(x, w, b, (s, s), (d, d), (pd, pd), omp=True)
    L = abi.lib()
    a = conv_args(abi.AD_BF16, abi.AD_NHWC, x.shape, K, k, s, d, pd)
    dx_ = H.dev_bf16(orc.nchw_to_nhwc(x))
    dw_ = H.dev_bf16(np.ascontiguousarray(np.transpose(w, (0, 2, 3, 1))))  # KRSC
    db_ = H.dev(b)
    P, Q = y_w.shape[2:]
    y = torch.full((N, P, Q, K), 7.0, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    a.x, a.w, a.bias, a.y = dx_.data_ptr(), dw_.data_ptr(), db_.data_ptr(), y.data_ptr()
    a.scratch, a.scratch_bytes = status.data_ptr(), 16
    abi.check(L.ad_conv2d_fprop(C.byref(a), H.stream()))
    _check_kind(L, _kinds(case)[0])
    H.sync()
    assert status[0].item() == 0
    got = orc.nhwc_to_nchw(H.host(y))
    err = H.max_rel(got, y_w)
    assert err < TOL_BF16, err
    a.relu = 1
    abi.check(L.ad_conv2d_fprop(C.byref(a), H.stream()))
    H.sync()
    assert H.max_rel(orc.nhwc_to_nchw(H.host(y)), np.maximum(y_w, 0)) < TOL_BF16
    assert status[0].item() == 0
    # no bias: the epilogue's other uniform branch
    a.relu, a.bias = 0, None
    abi.check(L.ad_conv2d_fprop(C.byref(a), H.stream()))
    H.sync()
    assert H.max_rel(orc.nhwc_to_nchw(H.host(y)), y_w - b.reshape(1, -1, 1, 1)) < TOL_BF16


@pytest.mark.parametrize("case", TC_CASES + ROW_CASES)
def test_conv_tc_dgrad(case):
    import torch
    N, Cc, Hh, W, K, k, s, d, pd = case[:9]
    x, w = _tc_setup(case)
    P, Q = _out_dims(Hh, W, k, s, d, pd)
    dy = orc.round_bf16(H.uniform(13, (N, K, P, Q)))
    dx_w = orc.conv2d_dgrad(dy, w, x.shape, (s, s), (d, d), (pd, pd), omp=True)
    L = abi.lib()
    a = conv_args(abi.AD_BF16, abi.AD_NHWC, x.shape, K, k, s, d, pd)
    dw_ = H.dev_bf16(np.ascontiguousarray(np.transpose(w, (0, 2, 3, 1))))
    ddy = H.dev_bf16(orc.nchw_to_nhwc(dy))
    dx = torch.full((N, Hh, W, Cc), 3.0, dtype=torch.bfloat16, device="cuda")
    nscr = L.ad_conv2d_scratch_bytes(C.byref(a), 1)
    scratch = torch.zeros(nscr, dtype=torch.uint8, device="cuda")
    a.w, a.y, a.dx, a.scratch, a.scratch_bytes = dw_.data_ptr(), ddy.data_ptr(), dx.data_ptr(), scratch.data_ptr(), nscr
    abi.check(L.ad_conv2d_dgrad(C.byref(a), H.stream()))
    _check_kind(L, _kinds(case)[1])
    H.sync()
    assert scratch[:4].view(torch.int32).item() == 0
    err = H.max_rel(orc.nhwc_to_nchw(H.host(dx)), dx_w)
    assert err < TOL_BF16, err
    a.accumulate = 1
    abi.check(L.ad_conv2d_dgrad(C.byref(a), H.stream()))
    H.sync()
    assert H.max_rel(orc.nhwc_to_nchw(H.host(dx)), 2 * dx_w) < 2 * TOL_BF16


@pytest.mark.parametrize("case", TC_CASES + ROW_CASES)
def test_conv_tc_wgrad(case):
    import torch
    N, Cc, Hh, W, K, k, s, d, pd = case[:9]
    kh, kw = _khw(k)
    x, w = _tc_setup(case)
    P, Q = _out_dims(Hh, W, k, s, d, pd)
    dy = orc.round_bf16(H.uniform(14, (N, K, P, Q)))
    db_w = np.zeros(K, np.float32)
    dw_w = orc.conv2d_wgrad(x, dy, w.shape, (s, s), (d, d), (pd, pd), db=db_w, omp=True)
    L = abi.lib()
    a = conv_args(abi.AD_BF16, abi.AD_NHWC, x.shape, K, k, s, d, pd)
    dx_ = H.dev_bf16(orc.nchw_to_nhwc(x))
    ddy = H.dev_bf16(orc.nchw_to_nhwc(dy))
    dw = torch.full((K, kh, kw, Cc), 5.0, device="cuda")
    db = torch.full((K,), 5.0, device="cuda")
    nscr = L.ad_conv2d_scratch_bytes(C.byref(a), 2)
    scratch = torch.zeros(nscr, dtype=torch.uint8, device="cuda")
    a.x, a.y, a.dw, a.db, a.scratch, a.scratch_bytes = dx_.data_ptr(), ddy.data_ptr(), dw.data_ptr(), db.data_ptr(), scratch.data_ptr(), nscr
    abi.check(L.ad_conv2d_wgrad(C.byref(a), H.stream()))
    _check_kind(L, _kinds(case)[2])
    H.sync()
    assert scratch[:4].view(torch.int32).item() == 0
    got = np.transpose(H.host(dw), (0, 3, 1, 2))  # KRSC -> KCRS
    err = H.max_rel(got, dw_w)
    assert err < 1e-3, err       # operands are exact in bf16 and the sum is fp32: far inside 2e-2
    assert H.max_rel(H.host(db), db_w) < 1e-4
    first = H.host(dw).copy()
    abi.check(L.ad_conv2d_wgrad(C.byref(a), H.stream()))
    H.sync()
    assert np.array_equal(H.host(dw), first)  # fixed-order split reduction: bit-reproducible
    # the same gradient written in the reference's KCRS order, added onto what the buffer holds
    dw2 = torch.full((K, Cc, kh, kw), 1.0, device="cuda")
    a.dw, a.db, a.dw_kcrs, a.accumulate = dw2.data_ptr(), None, 1, 1
    abi.check(L.ad_conv2d_wgrad(C.byref(a), H.stream()))
    H.sync()
    assert np.array_equal(H.host(dw2) - 1.0, (np.transpose(first, (0, 3, 1, 2)) + 1.0) - 1.0)
    assert scratch[:4].view(torch.int32).item() == 0


def test_conv_rejects_bad_arguments():
    L = abi.lib()
    a = conv_args(abi.AD_BF16, abi.AD_NCHW, (1, 64, 8, 8), 64, 3, 1, 1, 0)
    assert L.ad_conv2d_fprop(C.byref(a), H.stream()) == abi.AD_ERR_UNSUPPORTED   # no bf16 NCHW kernel
    a = conv_args(abi.AD_BF16, abi.AD_NHWC, (1, 48, 8, 8), 64, 3, 1, 1, 0)
    x = H.dev_bf16(np.zeros((1, 8, 8, 48), np.float32))
    a.x = a.w = a.y = x.data_ptr()
    assert L.ad_conv2d_fprop(C.byref(a), H.stream()) == abi.AD_ERR_UNSUPPORTED   # C not a multiple of 64
    a = conv_args(abi.AD_F32, abi.AD_NCHW, (1, 4, 2, 2), 4, 3, 1, 1, 0)
    assert L.ad_conv2d_fprop(C.byref(a), H.stream()) == abi.AD_ERR_BAD_ARG       # kernel larger than input
    assert L.ad_conv2d_fprop(None, H.stream()) == abi.AD_ERR_BAD_ARG


@pytest.mark.parametrize("case", [(2, 64, 22, 140, 64, 3, 1, 3, 0), (1, 128, 20, 24, 128, 3, 1, 1, 0), (1, 64, 34, 34, 128, 3, 2, 1, 0),
                                  (1, 64, 14, 300, 32, 3, 1, 2, 0)])
def test_conv_tc_fprop_row_ranges_compose(case):
    """Interior rows first, boundary rows later (what the halo overlap does) == one full call, bit for bit,
    and rows outside a range are not touched."""
    import torch
    N, Cc, Hh, W, K, k, s, d, pd = case
    x, w = _tc_setup(case)
    y_w = orc.conv2d_fprop(x, w, None, (s, s), (d, d), (pd, pd), omp=True)
    L = abi.lib()
    a = conv_args(abi.AD_BF16, abi.AD_NHWC, x.shape, K, k, s, d, pd)
    dx_ = H.dev_bf16(orc.nchw_to_nhwc(x))
    dw_ = H.dev_bf16(np.ascontiguousarray(np.transpose(w, (0, 2, 3, 1))))
    P, Q = _out_dims(Hh, W, k, s, d, pd)
    full = torch.zeros((N, P, Q, K), dtype=torch.bfloat16, device="cuda")
    parts = torch.full((N, P, Q, K), 9.0, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    a.x, a.w, a.scratch, a.scratch_bytes = dx_.data_ptr(), dw_.data_ptr(), status.data_ptr(), 16
    a.y = full.data_ptr()
    abi.check(L.ad_conv2d_fprop(C.byref(a), H.stream()))
    a.y = parts.data_ptr()
    b = 3
    a.out_row_begin, a.out_row_count = b, P - 2 * b
    abi.check(L.ad_conv2d_fprop(C.byref(a), H.stream()))
    H.sync()
    assert torch.all(parts[:, :b] == 9.0) and torch.all(parts[:, P - b:] == 9.0)
    a.out_row_begin, a.out_row_count = 0, b
    abi.check(L.ad_conv2d_fprop(C.byref(a), H.stream()))
    a.out_row_begin, a.out_row_count = P - b, b
    abi.check(L.ad_conv2d_fprop(C.byref(a), H.stream()))
    H.sync()
    assert torch.equal(parts, full) and status[0].item() == 0
    assert H.max_rel(orc.nhwc_to_nchw(H.host(parts)), y_w) < TOL_BF16
    a.out_row_begin, a.out_row_count = P - 1, 2
    assert L.ad_conv2d_fprop(C.byref(a), H.stream()) == abi.AD_ERR_BAD_ARG


@pytest.mark.parametrize("case", [(2, 64, 22, 140, 64, 3, 1, 3, 0), (1, 128, 20, 40, 128, 3, 1, 1, 0), (1, 64, 34, 34, 128, 3, 2, 1, 0),
                                  (1, 64, 14, 300, 32, 3, 1, 2, 0)])
def test_conv_tc_dgrad_column_range(case):
    """The data gradient restricted to the interior columns of a halo-padded buffer == those columns of the
    full gradient, bit for bit, and the pad columns are not touched."""
    import torch
    N, Cc, Hh, W, K, k, s, d, pd = case
    x, w = _tc_setup(case)
    P, Q = _out_dims(Hh, W, k, s, d, pd)
    dy = orc.round_bf16(H.uniform(14, (N, K, P, Q)))
    dx_w = orc.conv2d_dgrad(dy, w, x.shape, (s, s), (d, d), (pd, pd), omp=True)
    L = abi.lib()
    a = conv_args(abi.AD_BF16, abi.AD_NHWC, x.shape, K, k, s, d, pd)
    dw_ = H.dev_bf16(np.ascontiguousarray(np.transpose(w, (0, 2, 3, 1))))
    ddy = H.dev_bf16(orc.nchw_to_nhwc(dy))
    full = torch.zeros((N, Hh, W, Cc), dtype=torch.bfloat16, device="cuda")
    part = torch.full((N, Hh, W, Cc), 5.0, dtype=torch.bfloat16, device="cuda")
    nscr = L.ad_conv2d_scratch_bytes(C.byref(a), 1)
    scratch = torch.zeros(nscr, dtype=torch.uint8, device="cuda")
    a.w, a.y, a.scratch, a.scratch_bytes = dw_.data_ptr(), ddy.data_ptr(), scratch.data_ptr(), nscr
    a.dx = full.data_ptr()
    abi.check(L.ad_conv2d_dgrad(C.byref(a), H.stream()))
    p = d * (k - 1) // 2
    a.dx = part.data_ptr()
    a.dx_col_begin, a.dx_col_count = p, W - 2 * p
    abi.check(L.ad_conv2d_dgrad(C.byref(a), H.stream()))
    H.sync()
    assert scratch[:4].view(torch.int32).item() == 0
    assert torch.equal(part[:, :, p:W - p], full[:, :, p:W - p])
    assert H.max_rel(orc.nhwc_to_nchw(H.host(part))[:, :, :, p:W - p], dx_w[:, :, :, p:W - p]) < TOL_BF16
    assert torch.all(part[:, :, :p] == 5.0) and torch.all(part[:, :, W - p:] == 5.0)
    a.dx_col_begin, a.dx_col_count = W - 1, 2
    assert L.ad_conv2d_dgrad(C.byref(a), H.stream()) == abi.AD_ERR_BAD_ARG
    a32 = conv_args(abi.AD_F32, abi.AD_NCHW, (1, 4, 8, 8), 4, 3, 1, 1, 0)
    a32.dx_col_begin, a32.dx_col_count = 1, 6
    z = torch.zeros(1024, device="cuda")
    a32.y = a32.w = a32.dx = z.data_ptr()
    assert L.ad_conv2d_dgrad(C.byref(a32), H.stream()) == abi.AD_ERR_UNSUPPORTED


@pytest.mark.parametrize("case", ROW_CASES[:6] + ROW_CASES[8:10])
def test_conv_tc_row_kernels_agree_with_general_kernels(case, monkeypatch):
    """The same call served by the row-streaming kernels and, with ARRAYDIFF_B200_NO_ROW_KERNEL set, by the general
    tile kernels: two independent implementations of one contraction must agree to rounding (both accumulate in
    fp32; outputs are bf16 for fprop / dgrad, fp32 for the filter gradient) and report different kernel families."""
    import os
    import torch
    N, Cc, Hh, W, K, k, s, d, pd = case[:9]
    kh, kw = _khw(k)
    x, w = _tc_setup(case)
    P, Q = _out_dims(Hh, W, k, s, d, pd)
    dy = orc.round_bf16(H.uniform(21, (N, K, P, Q)))
    L = abi.lib()
    a = conv_args(abi.AD_BF16, abi.AD_NHWC, x.shape, K, k, s, d, pd)
    dx_ = H.dev_bf16(orc.nchw_to_nhwc(x))
    dw_ = H.dev_bf16(np.ascontiguousarray(np.transpose(w, (0, 2, 3, 1))))
    ddy = H.dev_bf16(orc.nchw_to_nhwc(dy))
    nscr = max(L.ad_conv2d_scratch_bytes(C.byref(a), 1), L.ad_conv2d_scratch_bytes(C.byref(a), 2))
    scratch = torch.zeros(nscr, dtype=torch.uint8, device="cuda")
    a.scratch, a.scratch_bytes = scratch.data_ptr(), nscr
    res, kinds = {}, {}
    for mode in ("row", "general"):
        if mode == "general":
            monkeypatch.setenv("ARRAYDIFF_B200_NO_ROW_KERNEL", "1")
        else:
            monkeypatch.delenv("ARRAYDIFF_B200_NO_ROW_KERNEL", raising=False)
        y = torch.zeros((N, P, Q, K), dtype=torch.bfloat16, device="cuda")
        gx = torch.zeros((N, Hh, W, Cc), dtype=torch.bfloat16, device="cuda")
        gw = torch.zeros((K, kh, kw, Cc), device="cuda")
        a.x, a.w, a.y = dx_.data_ptr(), dw_.data_ptr(), y.data_ptr()
        abi.check(L.ad_conv2d_fprop(C.byref(a), H.stream()))
        kf = L.ad_conv2d_last_kernel()
        a.y, a.dx, a.dw = ddy.data_ptr(), gx.data_ptr(), gw.data_ptr()
        abi.check(L.ad_conv2d_dgrad(C.byref(a), H.stream()))
        kd = L.ad_conv2d_last_kernel()
        abi.check(L.ad_conv2d_wgrad(C.byref(a), H.stream()))
        kw_ = L.ad_conv2d_last_kernel()
        H.sync()
        assert scratch[:4].view(torch.int32).item() == 0
        res[mode], kinds[mode] = (H.host(y), H.host(gx), H.host(gw)), (kf, kd, kw_)
    monkeypatch.delenv("ARRAYDIFF_B200_NO_ROW_KERNEL", raising=False)
    assert kinds["row"] == tuple(_kinds(case)) and kinds["general"] == (GEN, GEN, GEN), kinds
    for got, ref, tol in zip(res["row"], res["general"], (TOL_BF16, TOL_BF16, 1e-4)):
        assert H.max_rel(got, ref) < tol


@pytest.mark.parametrize("case", [(2, 64, 22, 140, 64, 3, 1, 3, 0), (1, 64, 18, 262, 64, 3, 1, 1, 0), (3, 64, 12, 104, 32, 3, 1, 2, 0),
                                  (1, 64, 9, 132, 8, 3, 1, 3, 1)])
@pytest.mark.parametrize("kcrs,accumulate", [(0, 0), (1, 1)])
def test_conv_tc_filter_gradient_forms_agree(case, kcrs, accumulate, monkeypatch):
    """The 3x3 filter gradient of a 64-channel layer has two tensor-core forms: filter rows stacked on the MMA's N axis
    (default) and, with ARRAYDIFF_B200_WGRAD_PAIRS=1, tap pairs stacked on M.  Both accumulate in fp32 over the same
    pixels in different orders: they agree to rounding, with each other and with the oracle, for dense and KCRS
    outputs, overwrite and accumulate, ragged widths, fewer than 64 output channels and implicit zero padding."""
    import torch
    N, Cc, Hh, W, K, k, s, d, pd = case
    x, w = _tc_setup(case)
    P, Q = _out_dims(Hh, W, k, s, d, pd)
    dy = orc.round_bf16(H.uniform(33, (N, K, P, Q)))
    dw_w = orc.conv2d_wgrad(x, dy, w.shape, (s, s), (d, d), (pd, pd), omp=True)      # KCRS
    L = abi.lib()
    a = conv_args(abi.AD_BF16, abi.AD_NHWC, x.shape, K, k, s, d, pd)
    dx_ = H.dev_bf16(orc.nchw_to_nhwc(x))
    ddy = H.dev_bf16(orc.nchw_to_nhwc(dy))
    nscr = L.ad_conv2d_scratch_bytes(C.byref(a), 2)
    scratch = torch.zeros(nscr, dtype=torch.uint8, device="cuda")
    a.x, a.y, a.scratch, a.scratch_bytes = dx_.data_ptr(), ddy.data_ptr(), scratch.data_ptr(), nscr
    a.dw_kcrs, a.accumulate = kcrs, accumulate
    shape = (K, Cc, 3, 3) if kcrs else (K, 3, 3, Cc)
    got = {}
    for form in ("rows", "pairs"):
        if form == "pairs":
            monkeypatch.setenv("ARRAYDIFF_B200_WGRAD_PAIRS", "1")
        else:
            monkeypatch.delenv("ARRAYDIFF_B200_WGRAD_PAIRS", raising=False)
        gw = torch.full(shape, 0.5 if accumulate else 7.0, device="cuda")
        a.dw = gw.data_ptr()
        abi.check(L.ad_conv2d_wgrad(C.byref(a), H.stream()))
        _check_kind(L, ROW)
        H.sync()
        assert scratch[:4].view(torch.int32)[0].item() == 0
        g = H.host(gw) - (0.5 if accumulate else 0.0)
        got[form] = g if kcrs else np.transpose(g, (0, 3, 1, 2))
    monkeypatch.delenv("ARRAYDIFF_B200_WGRAD_PAIRS", raising=False)
    assert H.max_rel(got["rows"], dw_w) < 1e-4 and H.max_rel(got["pairs"], dw_w) < 1e-4
    assert H.max_rel(got["rows"], got["pairs"]) < 1e-5
