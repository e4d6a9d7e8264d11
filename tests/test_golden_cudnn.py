"""The CPU oracle's convolution, pooling, batch normalisation and softmax against golden vectors recorded from the
cuDNN legacy-API calls the reference makes for those operators (tests/golden/reference_cudnn.npz, produced by
tests/golden/make_golden_cudnn.py on a B200 with the descriptors of the reference's call sites).  This is what pins
the dense-operator half of the oracle to the reference: max-relative 1e-5, the fp32 tolerance of the parity bar."""
import os

import numpy as np
import pytest

from oracle import orc
from tests import helpers as H

PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_cudnn.npz")
pytestmark = pytest.mark.skipif(not os.path.exists(PATH), reason="cuDNN golden fixture not generated yet")
TOL = 1e-5


@pytest.fixture(scope="module")
def fx():
    return dict(np.load(PATH))


def check_conv(fx, i, tol=TOL):
    N, Cc, Hh, W, K, kh, kw, s, d, pd, halo = (int(v) for v in fx[f"conv{i}_meta"])
    p = 0 if halo else pd       # a halo-padded input is convolved with descriptor pad 0 (src/op.cc:1354-1362)
    x, w, b, dy = fx[f"conv{i}_x"], fx[f"conv{i}_w"], fx[f"conv{i}_b"], fx[f"conv{i}_dy"]
    y = orc.conv2d_fprop(x, w, b, (s, s), (d, d), (p, p), omp=True)
    assert H.max_rel(y, fx[f"conv{i}_y"]) < tol
    dx = orc.conv2d_dgrad(dy, w, x.shape, (s, s), (d, d), (p, p), omp=True)
    assert H.max_rel(dx, fx[f"conv{i}_dx"]) < tol
    db = np.zeros(K, np.float32)
    dw = orc.conv2d_wgrad(x, dy, w.shape, (s, s), (d, d), (p, p), db=db, omp=True)
    assert H.max_rel(dw, fx[f"conv{i}_dw"]) < tol
    assert H.max_rel(db, fx[f"conv{i}_db"]) < tol


def check_pool(fx, i, tol=TOL):
    N, Cc, Hh, W, kh, kw, s, avg = (int(v) for v in fx[f"pool{i}_meta"])
    x, dy = fx[f"pool{i}_x"], fx[f"pool{i}_dy"]
    if avg:
        y, dx = orc.avgpool2d_fwd(x, (kh, kw), (s, s)), orc.avgpool2d_bwd(dy, x.shape, (kh, kw), (s, s))
    else:
        y, dx = orc.maxpool2d_fwd(x, (kh, kw), (s, s)), orc.maxpool2d_bwd(x, dy, (kh, kw), (s, s))
    if avg:
        assert H.max_rel(y, fx[f"pool{i}_y"]) < tol
    else:
        assert np.array_equal(y, fx[f"pool{i}_y"])          # a maximum is a selection: exact
    assert H.max_rel(dx, fx[f"pool{i}_dx"]) < tol


def check_bn(fx, i, tol=TOL):
    x, g, b, dy = fx[f"bn{i}_x"], fx[f"bn{i}_gamma"], fx[f"bn{i}_beta"], fx[f"bn{i}_dy"]
    n = x.shape[0] * x.shape[2] * x.shape[3]
    y, mean, invstd, var = orc.bn_fwd_train(x, g, b, 1e-5)
    assert H.max_rel(y, fx[f"bn{i}_y"]) < tol
    assert H.max_rel(mean, fx[f"bn{i}_save_mean"]) < tol
    assert H.max_rel(invstd, fx[f"bn{i}_save_invstd"]) < tol
    # factor 1.0: the "running" outputs are the batch mean and the unbiased batch variance (src/op.cc:3963)
    assert H.max_rel(mean, fx[f"bn{i}_run_mean"]) < tol
    assert H.max_rel(var * (n / (n - 1.0)), fx[f"bn{i}_run_var"]) < tol
    dx, dg, db = orc.bn_bwd(x, dy, g, b, mean, invstd)
    assert H.max_rel(dx, fx[f"bn{i}_dx"]) < 2 * tol
    assert H.max_rel(dg, fx[f"bn{i}_dgamma"]) < tol
    assert H.max_rel(db, fx[f"bn{i}_dbeta"]) < tol


def check_softmax(fx, i, tol=TOL):
    x, y_ref = fx[f"softmax{i}_x"], fx[f"softmax{i}_y"]
    N, Cc, Hh, W = x.shape
    mode = int(fx[f"softmax{i}_mode"][0])
    # MODE_INSTANCE on [B][C][1][1] and MODE_CHANNEL on [N][C][H][W] are both a softmax over C per (n, pixel)
    assert mode == 1 or (Hh == 1 and W == 1)
    rng = np.random.default_rng(7 + i)
    label = rng.integers(0, Cc, (N, Hh * W)).astype(np.uint32)
    label[0, 0], label[-1, -1] = 0, Cc - 1
    loss, prob, picked = orc.softmax_ce_pixel_fwd(x.reshape(N, Cc, Hh * W), label)
    assert H.max_rel(prob.reshape(x.shape), y_ref) < tol
    # the reference's loss on top of those probabilities: -log y[label] (src/kernels/softmax.cu:36-54)
    want = -np.log(np.take_along_axis(y_ref.reshape(N, Cc, Hh * W).astype(np.float64), label[:, None, :].astype(np.int64), axis=1))[:, 0]
    assert np.max(np.abs(loss - want)) < 1e-5 * max(1.0, float(np.max(np.abs(want))))


def test_conv_matches_reference_cudnn_calls(fx):
    for i in range(int(fx["counts"][0])):
        check_conv(fx, i)


def test_pool_matches_reference_cudnn_calls(fx):
    for i in range(int(fx["counts"][1])):
        check_pool(fx, i)


def test_batch_norm_matches_reference_cudnn_calls(fx):
    for i in range(int(fx["counts"][2])):
        check_bn(fx, i)


def test_softmax_matches_reference_cudnn_calls(fx):
    for i in range(int(fx["counts"][3])):
        check_softmax(fx, i)
