"""CPU tests of the oracle itself: internal consistency, the partition identities that the
spatially parallel path rests on, and agreement with an independent implementation
(torch's CPU operators, float64) for the cuDNN-defined ops."""
import numpy as np
import pytest

from oracle import orc
from tests import helpers as H


@pytest.mark.parametrize("R", [2, 4, 8])
@pytest.mark.parametrize("p", [1, 2, 3])
@pytest.mark.parametrize("layout", [orc.NCHW, orc.NHWC])
def test_exchange_equals_window_of_padded_full_tensor(R, p, layout):
    N, Cc, W = 2, 3, 5
    h = 2 * p + 1
    full = H.uniform(1, (N, Cc, h * R, W))
    strips = H.split_strips(full, R, p)
    want = H.expected_strips_after_exchange(full, R, p)
    if layout == orc.NHWC:
        strips = [orc.nchw_to_nhwc(s) for s in strips]
    orc.halo_exchange(strips, layout, p, W, h, Cc, N)
    for r in range(R):
        got = orc.nhwc_to_nchw(strips[r]) if layout == orc.NHWC else strips[r]
        assert np.array_equal(got, want[r])


def test_exchange_leaves_w_pad_and_outer_halos_untouched():
    R, p, N, Cc, W, h = 2, 2, 1, 2, 4, 4
    strips = [np.full((N, Cc, h + 2 * p, W + 2 * p), 7.0 + r, np.float32) for r in range(R)]
    orc.halo_exchange(strips, orc.NCHW, p, W, h, Cc, N)
    assert np.all(strips[0][:, :, :p, :] == 7.0)            # rank 0 top halo
    assert np.all(strips[1][:, :, p + h:, :] == 8.0)        # last rank bottom halo
    assert np.all(strips[0][:, :, :, :p] == 7.0) and np.all(strips[0][:, :, :, p + W:] == 7.0)
    assert np.all(strips[0][:, :, p + h:, p:p + W] == 8.0)  # bottom halo now rank 1's rows
    assert np.all(strips[1][:, :, :p, p:p + W] == 7.0)


@pytest.mark.parametrize("R", [2, 4, 8])
@pytest.mark.parametrize("p", [1, 3])
def test_reduce_is_overlap_add(R, p):
    """Summing padded gradient strips into the full gradient == reduce then take interiors."""
    N, Cc, W = 1, 2, 6
    h = 2 * p + 2
    g = [H.uniform(10 + r, (N, Cc, h + 2 * p, W + 2 * p)) for r in range(R)]
    full = np.zeros((N, Cc, h * R + 2 * p, W + 2 * p), np.float64)
    for r in range(R):
        full[:, :, r * h:r * h + h + 2 * p, :] += g[r]
    work = [x.copy() for x in g]
    orc.halo_reduce(work, orc.NCHW, p, W, h, Cc, N)
    for r in range(R):
        got = work[r][:, :, p:p + h, p:p + W]
        want = full[:, :, p + r * h:p + (r + 1) * h, p:p + W]
        np.testing.assert_allclose(got, want, rtol=0, atol=1e-6)
        # halo rows and W-pad columns are not modified
        assert np.array_equal(work[r][:, :, :p], g[r][:, :, :p])
        assert np.array_equal(work[r][:, :, :, :p], g[r][:, :, :, :p])


def test_reduce_bf16_rounds_to_nearest_even():
    p, W, h, Cc, N = 1, 3, 2, 1, 1
    a = orc.f32_to_bf16(H.uniform(3, (N, Cc, h + 2, W + 2)))
    b = orc.f32_to_bf16(H.uniform(4, (N, Cc, h + 2, W + 2)))
    wa, wb = a.copy(), b.copy()
    orc.halo_reduce([wa, wb], orc.NCHW, p, W, h, Cc, N)
    want = orc.f32_to_bf16(orc.bf16_to_f32(a[:, :, h, 1:1 + W]) + orc.bf16_to_f32(b[:, :, 0, 1:1 + W]))
    assert np.array_equal(wa[:, :, h, 1:1 + W], want)


def test_bf16_conversion_matches_torch():
    import torch
    x = H.normal(5, (4096,), 3.0)
    x[:4] = [0.0, -0.0, 1.0000001, 65504.0]
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(orc.f32_to_bf16(x), want)


def test_slice_pad_roundtrip():
    x = H.uniform(6, (2, 3, 4, 5))
    y = orc.halo_pad_fwd(x, 2)
    assert y.shape == (2, 3, 8, 9) and np.array_equal(y[:, :, 2:6, 2:7], x) and y.sum() == pytest.approx(x.sum(), rel=1e-5)
    dx = np.ones_like(x)
    orc.halo_pad_bwd(y, dx, 2)
    assert np.array_equal(dx, x + 1)


CONV_CASES = [
    # N, C, H, W, K, k, stride, dil, pad
    (1, 3, 9, 10, 4, 3, 1, 1, 1),
    (2, 4, 11, 9, 5, 3, 2, 1, 1),
    (1, 2, 12, 12, 3, 3, 1, 2, 2),
    (1, 3, 15, 14, 4, 7, 2, 1, 3),
    (2, 5, 6, 7, 6, 1, 1, 1, 0),
]


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv_oracle_matches_torch_float64(case):
    import torch
    import torch.nn.functional as F
    N, Cc, Hh, W, K, k, s, d, pd = case
    x, w, b = H.uniform(7, (N, Cc, Hh, W)), H.normal(8, (K, Cc, k, k), 0.2), H.normal(9, (K,))
    xt = torch.from_numpy(x).double().requires_grad_()
    wt = torch.from_numpy(w).double().requires_grad_()
    bt = torch.from_numpy(b).double().requires_grad_()
    yt = F.conv2d(xt, wt, bt, stride=s, padding=pd, dilation=d)
    dy = H.uniform(10, tuple(yt.shape))
    yt.backward(torch.from_numpy(dy).double())
    y = orc.conv2d_fprop(x, w, b, (s, s), (d, d), (pd, pd))
    np.testing.assert_allclose(y, yt.detach().numpy(), rtol=1e-5, atol=1e-6)
    dx = orc.conv2d_dgrad(dy, w, x.shape, (s, s), (d, d), (pd, pd))
    np.testing.assert_allclose(dx, xt.grad.numpy(), rtol=1e-5, atol=1e-6)
    db = np.zeros(K, np.float32)
    dw = orc.conv2d_wgrad(x, dy, w.shape, (s, s), (d, d), (pd, pd), db=db)
    np.testing.assert_allclose(dw, wt.grad.numpy(), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(db, bt.grad.numpy(), rtol=1e-5, atol=1e-5)


def test_pool_bn_softmax_oracle_match_torch_float64():
    import torch
    import torch.nn.functional as F
    x = H.normal(11, (2, 3, 9, 11))
    xt = torch.from_numpy(x).double().requires_grad_()
    yt = F.max_pool2d(xt, 3, 2)
    dy = H.uniform(12, tuple(yt.shape))
    yt.backward(torch.from_numpy(dy).double())
    np.testing.assert_array_equal(orc.maxpool2d_fwd(x, (3, 3), (2, 2)), yt.detach().float().numpy())
    np.testing.assert_allclose(orc.maxpool2d_bwd(x, dy, (3, 3), (2, 2)), xt.grad.numpy(), atol=1e-6)

    gamma, beta = H.uniform(13, (3,), 0.5, 1.5), H.uniform(14, (3,))
    xt = torch.from_numpy(x).double().requires_grad_()
    gt = torch.from_numpy(gamma).double().requires_grad_()
    bt = torch.from_numpy(beta).double().requires_grad_()
    yt = F.relu(F.batch_norm(xt, None, None, gt, bt, training=True, eps=1e-5))
    dy = H.uniform(15, x.shape)
    yt.backward(torch.from_numpy(dy).double())
    y, mean, invstd, var = orc.bn_fwd_train(x, gamma, beta, relu=True)
    np.testing.assert_allclose(y, yt.detach().numpy(), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(var, x.astype(np.float64).var(axis=(0, 2, 3)), rtol=1e-5)
    dx, dg, db = orc.bn_bwd(x, dy, gamma, beta, mean, invstd, relu=True)
    np.testing.assert_allclose(dx, xt.grad.numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(dg, gt.grad.numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(db, bt.grad.numpy(), rtol=1e-4, atol=1e-5)

    logits = H.normal(16, (2, 19, 35), 2.0)
    label = H.rng(17).integers(0, 19, (2, 35)).astype(np.uint32)
    label[0, 0], label[0, 1] = 0, 18
    lt = torch.from_numpy(logits).double().requires_grad_()
    loss_t = F.cross_entropy(lt, torch.from_numpy(label.astype(np.int64)), reduction="none")
    dloss = H.uniform(18, (2, 35))
    loss_t.backward(torch.from_numpy(dloss).double())
    loss, prob, picked = orc.softmax_ce_pixel_fwd(logits, label)
    np.testing.assert_allclose(loss, loss_t.detach().numpy(), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(orc.softmax_ce_pixel_bwd(logits, label, dloss), lt.grad.numpy(), rtol=1e-5, atol=1e-6)
    n, t = 1, 7
    assert picked[n, t] == (n * 19 + label[n, t]) * 35 + t
    np.testing.assert_allclose(prob.sum(axis=1), 1.0, rtol=1e-5)

    up = F.interpolate(torch.from_numpy(x).double(), scale_factor=8, mode="bilinear", align_corners=False)
    np.testing.assert_allclose(orc.upsample_bilinear_fwd(x, 8), up.numpy(), rtol=1e-5, atol=1e-6)
    xt = torch.from_numpy(x).double().requires_grad_()
    up = F.interpolate(xt, scale_factor=8, mode="bilinear", align_corners=False)
    dyu = H.uniform(19, tuple(up.shape))
    up.backward(torch.from_numpy(dyu).double())
    np.testing.assert_allclose(orc.upsample_bilinear_bwd(dyu, 8), xt.grad.numpy(), rtol=1e-4, atol=1e-5)


def test_nll_kernels_reference_form():
    B, Cc = 6, 5
    y = H.uniform(20, (B, Cc), 0.05, 1.0)
    label = np.array([0, 4, 2, 1, 3, 4], np.uint32)
    loss = orc.softmax_nll_loss_fwd(y, label)
    np.testing.assert_allclose(loss, -np.log(y[np.arange(B), label].astype(np.float64)), rtol=1e-6)
    dloss = H.uniform(21, (B,))
    dx = np.zeros((B, Cc), np.float32)
    orc.softmax_nll_loss_bwd(y, label, dloss, dx)
    onehot = np.eye(Cc, dtype=np.float32)[label]
    np.testing.assert_allclose(dx, dloss[:, None] * (y - onehot), rtol=1e-6, atol=1e-7)


def test_sgd_step_nesterov_and_plain():
    n = 257
    for nesterov in (0, 1):
        th, g, m = H.normal(22, (n,)), H.normal(23, (n,)), H.normal(24, (n,))
        th0, g0, m0 = th.copy(), g.copy(), m.copy()
        orc.sgd_step(th, g, m, 1e-4, 0.9, 0.1, 0.05, nesterov)
        g1 = g0 + 1e-4 * th0
        m1 = g1 + 0.9 * m0
        want = th0 - 0.1 * g1 - 0.05 * 0.9 * m1 if nesterov else th0 - 0.1 * m1
        np.testing.assert_allclose(th, want, rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(m, m1, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("R", [2, 4])
def test_config1_partitioned_conv_equals_unpartitioned(R):
    """benchmark config 1: 3x3 conv, stride 1, pad 1, fp32, N=1, C=K=64, 64x64, split into H-strips
    with 1-row halos exchanged in host memory; fwd + dgrad + wgrad vs the unsplit conv."""
    N, Cc, K, Hh, W, p = 1, 64, 64, 64, 64, 1
    x = H.uniform(100, (N, Cc, Hh, W))
    w = H.normal(101, (K, Cc, 3, 3), float(np.sqrt(2.0 / (9 * 64))))
    b = np.zeros(K, np.float32)
    dy = H.uniform(102, (N, K, Hh, W))
    h = Hh // R
    y_full = orc.conv2d_fprop(x, w, b, pad=(1, 1), omp=True)
    dx_full = orc.conv2d_dgrad(dy, w, x.shape, pad=(1, 1), omp=True)
    dw_full = orc.conv2d_wgrad(x, dy, w.shape, pad=(1, 1), omp=True)

    strips = [orc.halo_pad_fwd(np.ascontiguousarray(x[:, :, r * h:(r + 1) * h]), p) for r in range(R)]
    orc.halo_exchange(strips, orc.NCHW, p, W, h, Cc, N)
    gpad, dw_sum = [], np.zeros_like(w)
    for r in range(R):
        y_r = orc.conv2d_fprop(strips[r], w, b, omp=True)          # halo-padded input, pad 0
        assert np.allclose(y_r, y_full[:, :, r * h:(r + 1) * h], rtol=0, atol=1e-5 * np.abs(y_full).max())
        dy_r = np.ascontiguousarray(dy[:, :, r * h:(r + 1) * h])
        gpad.append(orc.conv2d_dgrad(dy_r, w, strips[r].shape, omp=True))
        dw_sum += orc.conv2d_wgrad(strips[r], dy_r, w.shape, omp=True)  # "allreduce" of weight grads
    orc.halo_reduce(gpad, orc.NCHW, p, W, h, Cc, N)
    for r in range(R):
        dx_r = np.zeros((N, Cc, h, W), np.float32)
        orc.halo_pad_bwd(gpad[r], dx_r, p)
        assert H.max_rel(dx_r, dx_full[:, :, r * h:(r + 1) * h]) < 1e-5
    assert H.max_rel(dw_sum, dw_full) < 1e-5
