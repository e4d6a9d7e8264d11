"""Packed array arithmetic, SGD, softmax / NLL, batch norm, pooling, ReLU / add / convert
kernels against the oracle."""
import ctypes as C

import numpy as np
import pytest

from arraydiff_cuda_b200 import abi
from oracle import orc
from tests import helpers as H

pytestmark = pytest.mark.gpu
f32 = C.c_float


@pytest.mark.parametrize("n", [1, 5, 1031, 1 << 20])
@pytest.mark.parametrize("misalign", [0, 1])
def test_array_ops_bit_exact(n, misalign):
    L = abi.lib()
    x, y = H.normal(1, (n + 1,), 3.0), H.normal(2, (n + 1,), 3.0)
    a, b = 0.37, -1.21
    calls = {
        "add": lambda dx, dy: L.ad_array_add(n, dx, dy, H.stream()),
        "add_scaled": lambda dx, dy: L.ad_array_add_scaled(n, f32(a), f32(b), dx, dy, H.stream()),
        "add_online": lambda dx, dy: L.ad_array_add_online(n, f32(a), dx, dy, H.stream()),
        "scale": lambda dx, dy: L.ad_array_scale(n, f32(a), dx, dy, H.stream()),
        "scale_add": lambda dx, dy: L.ad_array_scale_add(n, f32(a), dx, dy, H.stream()),
    }
    for name, call in calls.items():
        dx, dy = H.dev(x), H.dev(y)
        off = 4 * misalign
        abi.check(call(C.c_void_p(dx.data_ptr() + off), C.c_void_p(dy.data_ptr() + off)))
        H.sync()
        want = y[misalign:misalign + n].copy()
        orc.array_op(name, np.ascontiguousarray(x[misalign:misalign + n]), want, a, b)
        got = H.host(dy)
        assert np.array_equal(got[misalign:misalign + n], want), name
        assert got[misalign + n:].tolist() == y[misalign + n:].tolist()
    d = H.dev(y)
    abi.check(L.ad_array_set_constant(n, f32(2.5), H.ptr(d), H.stream()))
    H.sync()
    assert np.all(H.host(d)[:n] == 2.5)


@pytest.mark.parametrize("nesterov", [0, 1])
@pytest.mark.parametrize("l2", [0.0, 1e-4])
def test_sgd_step_bit_exact_with_bf16_shadow(nesterov, l2):
    import torch
    n = 100003
    th, g, m = H.normal(3, (n,)), H.normal(4, (n,)), H.normal(5, (n,))
    dth, dg, dm = H.dev(th), H.dev(g), H.dev(m)
    shadow = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    abi.check(abi.lib().ad_sgd_step(n, H.ptr(dth), H.ptr(dg), H.ptr(dm), f32(l2), f32(0.9), f32(0.1), f32(0.05), nesterov,
                                    H.ptr(shadow), H.stream()))
    H.sync()
    orc.sgd_step(th, g, m, l2, 0.9, 0.1, 0.05, nesterov)
    assert np.array_equal(H.host(dth), th) and np.array_equal(H.host(dg), g) and np.array_equal(H.host(dm), m)
    assert np.array_equal(H.bits_bf16(shadow), orc.f32_to_bf16(th))


def test_nll_loss_kernels():
    import torch
    B, Cc = 1000, 1000
    y = H.uniform(6, (B, Cc), 1e-3, 1.0)
    label = H.rng(7).integers(0, Cc, (B,)).astype(np.uint32)
    label[:2] = [0, Cc - 1]
    dloss, dx0 = H.uniform(8, (B,)), H.uniform(9, (B, Cc))
    dy_, dl, ddl, ddx = H.dev(y), torch.from_numpy(label.view(np.int32)).cuda(), H.dev(dloss), H.dev(dx0)
    loss = torch.empty(B, device="cuda")
    L = abi.lib()
    abi.check(L.ad_softmax_nll_loss_fwd(Cc, B, H.ptr(dy_), H.ptr(dl), H.ptr(loss), H.stream()))
    abi.check(L.ad_softmax_nll_loss_bwd(Cc, B, H.ptr(dy_), H.ptr(dl), H.ptr(ddl), H.ptr(ddx), H.stream()))
    H.sync()
    np.testing.assert_allclose(H.host(loss), orc.softmax_nll_loss_fwd(y, label), rtol=1e-6)
    want = dx0.copy()
    orc.softmax_nll_loss_bwd(y, label, dloss, want)
    assert np.array_equal(H.host(ddx), want)  # label indexing and rounding both exact


@pytest.mark.parametrize("Cc", [2, 19, 1000])
@pytest.mark.parametrize("layout", [abi.AD_NCHW, abi.AD_NHWC])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_softmax_ce_pixel(Cc, layout, dtype):
    import torch
    N, HW = 2, 77
    logits = H.normal(10, (N, Cc, HW), 2.0)
    if dtype == "bf16":
        logits = orc.round_bf16(logits)
    label = H.rng(11).integers(0, Cc, (N, HW)).astype(np.uint32)
    label[0, :2] = [0, Cc - 1]
    dloss = H.uniform(12, (N, HW))
    loss_w, _, picked_w = orc.softmax_ce_pixel_fwd(logits, label)
    dlog_w = orc.softmax_ce_pixel_bwd(logits, label, dloss)
    arr = logits if layout == abi.AD_NCHW else np.ascontiguousarray(np.transpose(logits, (0, 2, 1)))
    d = H.dev(arr) if dtype == "f32" else H.dev_bf16(arr)
    dl = torch.from_numpy(label.view(np.int32)).cuda()
    loss = torch.empty((N, HW), device="cuda")
    picked = torch.empty((N, HW), dtype=torch.int64, device="cuda")
    dlog = torch.zeros_like(d)
    L = abi.lib()
    dt = abi.AD_F32 if dtype == "f32" else abi.AD_BF16
    abi.check(L.ad_softmax_ce_pixel_fwd(dt, layout, N, Cc, HW, H.ptr(d), H.ptr(dl), H.ptr(loss), H.ptr(picked), H.stream()))
    ddl = H.dev(dloss)
    abi.check(L.ad_softmax_ce_pixel_bwd(dt, layout, N, Cc, HW, H.ptr(d), H.ptr(dl), H.ptr(ddl), H.ptr(dlog), 0, H.stream()))
    H.sync()
    # label index: bit-exact
    pk = picked.cpu().numpy().astype(np.uint64)
    if layout == abi.AD_NCHW:
        assert np.array_equal(pk, picked_w)
    else:
        n_idx, t_idx = np.meshgrid(np.arange(N), np.arange(HW), indexing="ij")
        assert np.array_equal(pk, ((n_idx * HW + t_idx) * Cc + label).astype(np.uint64))
    assert H.max_rel(H.host(loss), loss_w) < 1e-5
    got = H.host(dlog)
    if layout == abi.AD_NHWC:
        got = np.transpose(got, (0, 2, 1))
    assert H.max_rel(got, dlog_w) < (1e-5 if dtype == "f32" else 2e-2)


def _views(arr_nchw, layout, dtype, pad=0):
    """Device tensor (optionally inside a zero halo-padded buffer) + Tensor4 view of the interior."""
    import torch
    N, Cc, Hh, W = arr_nchw.shape
    buf = np.zeros((N, Cc, Hh + 2 * pad, W + 2 * pad), np.float32)
    buf[:, :, pad:pad + Hh, pad:pad + W] = arr_nchw
    if layout == abi.AD_NHWC:
        buf = orc.nchw_to_nhwc(buf)
    t = H.dev(buf) if dtype == "f32" else H.dev_bf16(buf)
    mk = H.view_nchw if layout == abi.AD_NCHW else H.view_nhwc
    return t, mk(t, (pad, Hh, W) if pad else None)


def _back(t, layout, pad, Hh, W):
    a = H.host(t)
    if layout == abi.AD_NHWC:
        a = orc.nhwc_to_nchw(a)
    return a[:, :, pad:pad + Hh, pad:pad + W]


@pytest.mark.parametrize("layout", [abi.AD_NCHW, abi.AD_NHWC])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("relu", [0, 1])
@pytest.mark.parametrize("Cc", [37, 64])        # 64: the 8-channels-per-thread NHWC bf16 kernels
def test_batch_norm_fwd_bwd(layout, dtype, relu, Cc):
    import torch
    N, Hh, W = 2, 19, 23
    x = H.normal(20, (N, Cc, Hh, W)) * H.uniform(21, (1, Cc, 1, 1), 0.5, 2.0) + H.uniform(22, (1, Cc, 1, 1))
    dy = H.uniform(23, (N, Cc, Hh, W))
    if dtype == "bf16":
        x, dy = orc.round_bf16(x), orc.round_bf16(dy)
    gamma, beta = H.uniform(24, (Cc,), 0.5, 1.5), H.uniform(25, (Cc,), -0.5, 0.5)
    y_w, mean_w, invstd_w, var_w = orc.bn_fwd_train(x, gamma, beta, relu=relu)
    dx_w, dg_w, db_w = orc.bn_bwd(x, dy, gamma, beta, mean_w, invstd_w, relu=relu)
    L = abi.lib()
    tx, vx = _views(x, layout, dtype)
    ty, vy = _views(np.zeros_like(x), layout, dtype, pad=1)   # output lands inside a halo-padded buffer
    tdy, vdy = _views(dy, layout, dtype)
    tdx, vdx = _views(np.zeros_like(x), layout, dtype)
    dgm, dbt = H.dev(gamma), H.dev(beta)
    mean, invstd, var = (torch.empty(Cc, device="cuda") for _ in range(3))
    dgam, dbet = torch.zeros(Cc, device="cuda"), torch.zeros(Cc, device="cuda")
    nscr = L.ad_bn_scratch_bytes(Cc)
    scratch = torch.empty(nscr, dtype=torch.uint8, device="cuda")
    abi.check(L.ad_bn_fwd_train(C.byref(vx), C.byref(vy), H.ptr(dgm), H.ptr(dbt), H.ptr(mean), H.ptr(invstd), H.ptr(var),
                                f32(1e-5), relu, H.ptr(scratch), nscr, H.stream()))
    abi.check(L.ad_bn_bwd(C.byref(vx), C.byref(vdy), C.byref(vdx), H.ptr(dgm), H.ptr(dbt), H.ptr(mean), H.ptr(invstd),
                          H.ptr(dgam), H.ptr(dbet), relu, 0, H.ptr(scratch), nscr, H.stream()))
    H.sync()
    tol = 1e-5 if dtype == "f32" else 2e-2
    assert H.max_rel(H.host(mean), mean_w) < 1e-5 and H.max_rel(H.host(invstd), invstd_w) < 1e-5
    assert H.max_rel(H.host(var), var_w) < 1e-5
    assert H.max_rel(_back(ty, layout, 1, Hh, W), y_w) < tol
    ypad = H.host(ty) if layout == abi.AD_NCHW else orc.nhwc_to_nchw(H.host(ty))
    assert np.all(ypad[:, :, 0, :] == 0) and np.all(ypad[:, :, :, 0] == 0)  # halo cells untouched
    # backward is checked with the device's own saved statistics (what the op consumes)
    assert H.max_rel(_back(tdx, layout, 0, Hh, W), dx_w) < (5e-5 if dtype == "f32" else 2e-2)
    assert H.max_rel(H.host(dgam), dg_w) < 5e-5 and H.max_rel(H.host(dbet), db_w) < 5e-5
    assert L.ad_bn_fwd_train(C.byref(vx), C.byref(vy), H.ptr(dgm), H.ptr(dbt), H.ptr(mean), H.ptr(invstd), H.ptr(var),
                             f32(1e-5), relu, H.ptr(scratch), 8, H.stream()) == abi.AD_ERR_SCRATCH


@pytest.mark.parametrize("layout", [abi.AD_NCHW, abi.AD_NHWC])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("relu", [0, 1])
def test_batch_norm_fixed_statistics(layout, dtype, relu):
    """Inference form (cudnnBatchNormalizationForwardInference at the reference's call site): fixed mean / variance."""
    import torch
    N, Cc, Hh, W = 2, 64, 9, 11
    x = H.normal(30, (N, Cc, Hh, W)) * 1.7 + 0.3
    if dtype == "bf16":
        x = orc.round_bf16(x)
    gamma, beta = H.uniform(31, (Cc,), 0.5, 1.5), H.uniform(32, (Cc,), -0.5, 0.5)
    mean, var = H.uniform(33, (Cc,), -0.4, 0.4), H.uniform(34, (Cc,), 0.2, 3.0)
    sh = (1, Cc, 1, 1)
    y_w = gamma.reshape(sh).astype(np.float64) * (x.astype(np.float64) - mean.reshape(sh)) / np.sqrt(var.reshape(sh).astype(np.float64) + 1e-5) + beta.reshape(sh)
    if relu:
        y_w = np.maximum(y_w, 0)
    L = abi.lib()
    tx, vx = _views(x, layout, dtype)
    ty, vy = _views(np.zeros_like(x), layout, dtype, pad=1)
    d = [H.dev(a) for a in (gamma, beta, mean, var)]
    invstd = torch.empty(Cc, device="cuda")
    abi.check(L.ad_bn_fwd_inference(C.byref(vx), C.byref(vy), *[H.ptr(t) for t in d], H.ptr(invstd), f32(1e-5), relu, H.stream()))
    H.sync()
    assert H.max_rel(_back(ty, layout, 1, Hh, W), y_w) < (1e-5 if dtype == "f32" else 2e-2)
    assert H.max_rel(H.host(invstd), 1.0 / np.sqrt(var.astype(np.float64) + 1e-5)) < 1e-6


def test_batch_norm_two_phase_matches_single_call_across_strips():
    """Statistics over R strips via partial sums + host-side sum == statistics over the whole tensor."""
    import torch
    N, Cc, Hh, W, R = 1, 8, 16, 12, 4
    x = H.normal(26, (N, Cc, Hh, W))
    gamma, beta = np.ones(Cc, np.float32), np.zeros(Cc, np.float32)
    y_w, mean_w, invstd_w, _ = orc.bn_fwd_train(x, gamma, beta, relu=True)
    L = abi.lib()
    nscr = L.ad_bn_scratch_bytes(Cc)
    scratch = torch.empty(nscr, dtype=torch.uint8, device="cuda")
    h = Hh // R
    sums = torch.zeros((R, 2 * Cc), device="cuda")
    strips = []
    for r in range(R):
        t, v = _views(np.ascontiguousarray(x[:, :, r * h:(r + 1) * h]), abi.AD_NCHW, "f32")
        strips.append((t, v))
        abi.check(L.ad_bn_partial_stats(C.byref(v), C.c_void_p(sums.data_ptr() + r * 8 * Cc), H.ptr(scratch), nscr, H.stream()))
    total = sums.sum(dim=0).contiguous()   # stands in for the 2C-float allreduce
    mean, invstd = torch.empty(Cc, device="cuda"), torch.empty(Cc, device="cuda")
    dgm, dbt = H.dev(gamma), H.dev(beta)
    for r in range(R):
        t, v = strips[r]
        out = torch.empty_like(t)
        vo = H.view_nchw(out)
        abi.check(L.ad_bn_finalize_apply(C.byref(v), C.byref(vo), H.ptr(total), C.c_double(N * Hh * W), H.ptr(dgm),
                                         H.ptr(dbt), H.ptr(mean), H.ptr(invstd), None, f32(1e-5), 1, H.stream()))
        H.sync()
        assert H.max_rel(H.host(out), y_w[:, :, r * h:(r + 1) * h]) < 1e-5
    assert H.max_rel(H.host(mean), mean_w) < 1e-5


@pytest.mark.parametrize("layout", [abi.AD_NCHW, abi.AD_NHWC])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("Cc", [5, 16])
def test_maxpool_3x3_s2_on_padded_input(layout, dtype, Cc):
    """The reference's pool sees the explicit zero pad cells (pad value 0, not -inf)."""
    N, Hh, W, p = 2, 12, 14, 1
    x = H.normal(30, (N, Cc, Hh, W)) - 0.5      # mostly negative at some borders: pad zeros win there
    if dtype == "bf16":
        x = orc.round_bf16(x)
    xp = np.zeros((N, Cc, Hh + 2, W + 2), np.float32)
    xp[:, :, 1:-1, 1:-1] = x
    y_w = orc.maxpool2d_fwd(xp, (3, 3), (2, 2))
    dy = H.uniform(31, y_w.shape)
    if dtype == "bf16":
        dy = orc.round_bf16(dy)
    dx_w = orc.maxpool2d_bwd(xp, dy, (3, 3), (2, 2))
    tx, vx = _views(xp, layout, dtype)
    ty, vy = _views(np.zeros_like(y_w), layout, dtype)
    tdy, vdy = _views(dy, layout, dtype)
    tdx, vdx = _views(np.zeros_like(xp), layout, dtype)
    L = abi.lib()
    abi.check(L.ad_maxpool2d_fwd(C.byref(vx), C.byref(vy), 3, 3, 2, 2, H.stream()))
    abi.check(L.ad_maxpool2d_bwd(C.byref(vx), C.byref(vdy), C.byref(vdx), 3, 3, 2, 2, 0, H.stream()))
    H.sync()
    assert np.array_equal(_back(ty, layout, 0, *y_w.shape[2:]), y_w)
    got = _back(tdx, layout, 0, Hh + 2, W + 2)
    if dtype == "f32":
        np.testing.assert_allclose(got, dx_w, rtol=0, atol=1e-6)
    else:
        assert H.max_rel(got, dx_w) < 2e-2


@pytest.mark.parametrize("layout", [abi.AD_NCHW, abi.AD_NHWC])
@pytest.mark.parametrize("Cc", [6, 16])
def test_relu_add_convert(layout, Cc):
    N, Hh, W = 2, 5, 7
    a, b = H.normal(40, (N, Cc, Hh, W)), H.normal(41, (N, Cc, Hh, W))
    L = abi.lib()
    ta, va = _views(a, layout, "f32")
    tb, vb = _views(b, layout, "f32")
    ty, vy = _views(np.zeros_like(a), layout, "f32", pad=2)
    abi.check(L.ad_relu_fwd(C.byref(va), C.byref(vy), H.stream()))
    H.sync()
    assert np.array_equal(_back(ty, layout, 2, Hh, W), np.maximum(a, 0))
    abi.check(L.ad_add(C.byref(va), C.byref(vb), C.byref(vy), H.stream()))
    H.sync()
    assert np.array_equal(_back(ty, layout, 2, Hh, W), a + b)
    tdx, vdx = _views(np.ones_like(a), layout, "f32")
    abi.check(L.ad_relu_bwd(C.byref(va), C.byref(vb), C.byref(vdx), 1, H.stream()))
    H.sync()
    want = np.ones_like(a)
    orc.relu_bwd(a, b, want)
    assert np.array_equal(_back(tdx, layout, 0, Hh, W), want)
    # NCHW fp32 -> NHWC bf16 (graph edge conversion) and back
    tn, vn = _views(a, abi.AD_NCHW, "f32")
    th, vh = _views(np.zeros_like(a), abi.AD_NHWC, "bf16")
    abi.check(L.ad_convert(C.byref(vn), C.byref(vh), 0, H.stream()))
    H.sync()
    assert np.array_equal(H.bits_bf16(th), orc.f32_to_bf16(orc.nchw_to_nhwc(a)))
    tback, vback = _views(np.zeros_like(a), abi.AD_NCHW, "f32")
    abi.check(L.ad_convert(C.byref(vh), C.byref(vback), 0, H.stream()))
    H.sync()
    assert np.array_equal(H.host(tback), orc.round_bf16(a))


def test_nhwc_bf16_vector_paths_match_scalar_semantics():
    """relu / add / relu-bwd / accumulate-convert on aligned NHWC bf16 views (8 channels per thread), with the
    output inside a halo-padded buffer."""
    N, Cc, Hh, W = 2, 64, 9, 11
    a, b = orc.round_bf16(H.normal(50, (N, Cc, Hh, W))), orc.round_bf16(H.normal(51, (N, Cc, Hh, W)))
    L = abi.lib()
    ta, va = _views(a, abi.AD_NHWC, "bf16")
    tb, vb = _views(b, abi.AD_NHWC, "bf16")
    ty, vy = _views(np.zeros_like(a), abi.AD_NHWC, "bf16", pad=1)
    abi.check(L.ad_add(C.byref(va), C.byref(vb), C.byref(vy), H.stream()))
    H.sync()
    assert np.array_equal(_back(ty, abi.AD_NHWC, 1, Hh, W), orc.round_bf16(a + b))
    abi.check(L.ad_relu_fwd(C.byref(va), C.byref(vy), H.stream()))
    H.sync()
    assert np.array_equal(_back(ty, abi.AD_NHWC, 1, Hh, W), np.maximum(a, 0))
    tdx, vdx = _views(b, abi.AD_NHWC, "bf16")
    abi.check(L.ad_relu_bwd(C.byref(va), C.byref(vb), C.byref(vdx), 1, H.stream()))
    H.sync()
    assert np.array_equal(_back(tdx, abi.AD_NHWC, 0, Hh, W), orc.round_bf16(b + np.where(a > 0, b, 0)))
    abi.check(L.ad_convert(C.byref(va), C.byref(vdx), 1, H.stream()))
    H.sync()
    assert np.array_equal(_back(tdx, abi.AD_NHWC, 0, Hh, W), orc.round_bf16(orc.round_bf16(b + np.where(a > 0, b, 0)) + a))


@pytest.mark.parametrize("layout", [abi.AD_NCHW, abi.AD_NHWC])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("R,scale", [(1, 8), (2, 8), (4, 2), (2, 3)])
def test_upsample_bilinear_strips_equal_unpartitioned(layout, dtype, R, scale):
    """Each strip (with one halo row on its inner edges) upsamples to exactly its rows of the oracle's
    unpartitioned result; the strip gradients, overlap-added over the halo rows, give the oracle's gradient."""
    N, Cc, Hh, W = 2, 5, 8, 6
    x = H.normal(50, (N, Cc, Hh, W))
    dy = H.uniform(51, (N, Cc, Hh * scale, W * scale))
    if dtype == "bf16":
        x, dy = orc.round_bf16(x), orc.round_bf16(dy)
    y_w = orc.upsample_bilinear_fwd(x, scale)
    dx_w = orc.upsample_bilinear_bwd(dy, scale)
    L = abi.lib()
    h = Hh // R
    dx_sum = np.zeros((N, Cc, Hh + 2, W), np.float64)     # row i holds global row i - 1
    for r in range(R):
        xs = np.zeros((N, Cc, h + 2, W), np.float32)
        lo, hi = max(0, r * h - 1), min(Hh, (r + 1) * h + 1)
        xs[:, :, lo - (r * h - 1):hi - (r * h - 1)] = x[:, :, lo:hi]
        tx, vx = _views(xs, layout, dtype)
        ty, vy = _views(np.zeros((N, Cc, h * scale, W * scale), np.float32), layout, dtype)
        tdy, vdy = _views(dy[:, :, r * h * scale:(r + 1) * h * scale], layout, dtype)
        tdx, vdx = _views(np.full((N, Cc, h + 2, W), 7.0, np.float32), layout, dtype)
        abi.check(L.ad_upsample_bilinear_fwd(C.byref(vx), C.byref(vy), scale, r * h - 1, Hh, r * h * scale, H.stream()))
        abi.check(L.ad_upsample_bilinear_bwd(C.byref(vdy), C.byref(vdx), scale, r * h - 1, Hh, r * h * scale, 0, H.stream()))
        H.sync()
        got = _back(ty, layout, 0, h * scale, W * scale)
        want = y_w[:, :, r * h * scale:(r + 1) * h * scale]
        assert H.max_rel(got, want) < (1e-6 if dtype == "f32" else 8e-3)
        g = _back(tdx, layout, 0, h + 2, W).astype(np.float64)
        if r == 0:
            assert np.all(g[:, :, 0] == 0)                # the row above the tensor receives nothing
        if r == R - 1:
            assert np.all(g[:, :, -1] == 0)
        dx_sum[:, :, r * h:r * h + h + 2] += g
    assert H.max_rel(dx_sum[:, :, 1:-1], dx_w) < (1e-5 if dtype == "f32" else 8e-3)
    # a view that lacks a needed source row is refused before any launch
    tx, vx = _views(np.zeros((N, Cc, Hh - 1, W), np.float32), layout, dtype)
    ty, vy = _views(np.zeros((N, Cc, Hh * scale, W * scale), np.float32), layout, dtype)
    assert L.ad_upsample_bilinear_fwd(C.byref(vx), C.byref(vy), scale, 0, Hh, 0, H.stream()) == abi.AD_ERR_BAD_ARG


@pytest.mark.parametrize("layout", [abi.AD_NCHW, abi.AD_NHWC])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("k,s", [((8, 8), (8, 8)), ((2, 3), (2, 1))])
def test_average_pool(layout, dtype, k, s):
    """Global (window = input) and windowed mean pooling against the numpy restatement."""
    N, Cc, Hh, W = 2, 12, 8, 8
    x = H.normal(60, (N, Cc, Hh, W))
    if dtype == "bf16":
        x = orc.round_bf16(x)
    y_w = orc.avgpool2d_fwd(x, k, s)
    dy = H.uniform(61, y_w.shape)
    if dtype == "bf16":
        dy = orc.round_bf16(dy)
    dx_w = orc.avgpool2d_bwd(dy, x.shape, k, s)
    tx, vx = _views(x, layout, dtype)
    ty, vy = _views(np.zeros_like(y_w), layout, dtype)
    tdy, vdy = _views(dy, layout, dtype)
    tdx, vdx = _views(np.ones_like(x), layout, dtype)
    L = abi.lib()
    abi.check(L.ad_avgpool2d_fwd(C.byref(vx), C.byref(vy), k[0], k[1], s[0], s[1], H.stream()))
    abi.check(L.ad_avgpool2d_bwd(C.byref(vdy), C.byref(vdx), k[0], k[1], s[0], s[1], 1, H.stream()))
    H.sync()
    tol = 1e-6 if dtype == "f32" else 8e-3
    assert H.max_rel(_back(ty, layout, 0, *y_w.shape[2:]), y_w) < tol
    assert H.max_rel(_back(tdx, layout, 0, Hh, W), dx_w + 1.0) < tol
    assert L.ad_avgpool2d_fwd(C.byref(vx), C.byref(vdx), k[0], k[1], s[0], s[1], H.stream()) == abi.AD_ERR_BAD_ARG


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("B,I,O", [(4, 512, 1000), (3, 70, 19)])
def test_linear_layer(dtype, B, I, O):
    """y = x w^T + b and its three gradients against the numpy restatement."""
    x, w, b = H.normal(70, (B, I)), H.normal(71, (O, I), 0.05), H.normal(72, (O,))
    dy = H.uniform(73, (B, O))
    if dtype == "bf16":
        x, dy = orc.round_bf16(x), orc.round_bf16(dy)
    y_w = orc.linear_fwd(x, w, b)
    dx_w, dw_w, db_w = orc.linear_bwd(x, w, dy)
    mk = H.dev if dtype == "f32" else H.dev_bf16
    tx, tdy = mk(x), mk(dy)
    ty, tdx = mk(np.zeros_like(y_w)), mk(np.full_like(x, 2.0))
    tw, tb = H.dev(w), H.dev(b)
    tdw, tdb = H.dev(np.zeros_like(w)), H.dev(np.zeros_like(b))
    L = abi.lib()
    dt = abi.AD_F32 if dtype == "f32" else abi.AD_BF16
    abi.check(L.ad_linear_fwd(dt, B, I, O, H.ptr(tx), H.ptr(tw), H.ptr(tb), H.ptr(ty), H.stream()))
    abi.check(L.ad_linear_bwd(dt, B, I, O, H.ptr(tx), H.ptr(tw), H.ptr(tdy), H.ptr(tdx), H.ptr(tdw), H.ptr(tdb), 1, 0, H.stream()))
    H.sync()
    tol = 2e-6 if dtype == "f32" else 8e-3
    assert H.max_rel(H.host(ty), y_w) < tol
    assert H.max_rel(H.host(tdx), dx_w + 2.0) < tol
    assert H.max_rel(H.host(tdw), dw_w) < 2e-6 and H.max_rel(H.host(tdb), db_w) < 2e-6


def test_sgd_step_guard_skips_the_update_after_a_timed_out_wait():
    import torch
    L = abi.lib()
    n = 1000
    theta0, g0 = H.normal(70, (n,)), H.normal(71, (n,))
    for flag, changed in ((0, True), (abi.AD_ERR_TIMEOUT, False)):
        theta, g, m = H.dev(theta0), H.dev(g0), torch.zeros(n, device="cuda")
        status = torch.tensor([flag], dtype=torch.int32, device="cuda")
        abi.check(L.ad_sgd_step_guarded(n, H.ptr(theta), H.ptr(g), H.ptr(m), f32(1e-4), f32(0.9), f32(0.1), f32(0.1), 1, None,
                                        H.ptr(status), H.stream()))
        H.sync()
        assert (not np.array_equal(H.host(theta), theta0)) == changed
        if changed:
            ref = H.dev(theta0)
            g2, m2 = H.dev(g0), torch.zeros(n, device="cuda")
            abi.check(L.ad_sgd_step(n, H.ptr(ref), H.ptr(g2), H.ptr(m2), f32(1e-4), f32(0.9), f32(0.1), f32(0.1), 1, None, H.stream()))
            H.sync()
            assert torch.equal(ref, theta)
        else:
            assert np.array_equal(H.host(m), np.zeros(n, np.float32))
