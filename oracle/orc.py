"""numpy front end to the CPU oracle (oracle/oracle.c).  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module.
Arrays are C-contiguous numpy arrays; float32 unless stated, bf16 as uint16 bit patterns.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
NCHW, NHWC = 0, 1
F32, BF16 = 0, 1

_libs = {}


def build():
    subprocess.check_call(["make", "-s", "-C", HERE, "all"])


def _load(omp=False):
    key = "omp" if omp else "st"
    if key not in _libs:
        path = os.path.join(HERE, "liboracle_omp.so" if omp else "liboracle.so")
        if not os.path.exists(path):
            build()
        _libs[key] = C.CDLL(path)
        _libs[key].orc_num_threads.restype = C.c_int
    return _libs[key]


def num_threads(omp=False):
    return _load(omp).orc_num_threads()


def set_num_threads(n=None):
    """Give the OpenMP build `n` threads (default: every core this process may run on), overriding an inherited
    OMP_NUM_THREADS.  Returns the thread count now in force."""
    if n is None:
        n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    _load(True).orc_set_num_threads(C.c_int(int(n)))
    return num_threads(True)


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a


def f32_to_bf16(x):
    x = _f32(x)
    y = np.empty(x.shape, np.uint16)
    _load().orc_cast_f32_to_bf16(C.c_size_t(x.size), _p(x), _p(y))
    return y


def bf16_to_f32(x):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    y = np.empty(x.shape, np.float32)
    _load().orc_cast_bf16_to_f32(C.c_size_t(x.size), _p(x), _p(y))
    return y


def round_bf16(x):
    return bf16_to_f32(f32_to_bf16(x))


def _ptr_array(bufs):
    arr = (C.c_void_p * len(bufs))()
    for i, b in enumerate(bufs):
        assert b.flags["C_CONTIGUOUS"]
        arr[i] = b.ctypes.data
    return arr


def halo_exchange(bufs, layout, p, W, h, Cc, N):
    """In place on the list of padded strips (float32 or uint16 arrays)."""
    es = bufs[0].dtype.itemsize
    _load().orc_halo_exchange(len(bufs), _ptr_array(bufs), es, layout, p, W, h, Cc, N)


def halo_reduce(bufs, layout, p, W, h, Cc, N):
    dt = F32 if bufs[0].dtype == np.float32 else BF16
    _load().orc_halo_reduce(len(bufs), _ptr_array(bufs), dt, layout, p, W, h, Cc, N)


def halo2d_exchange(bufs, layout, gw, gh, p, w, h, Cc, N):
    """In place on the padded buffers of a gh x gw rank grid (rank = gy * gw + gx); float32 or uint16 (bf16 bits)."""
    _load().orc_halo2d_exchange(gw, gh, _ptr_array(bufs), bufs[0].dtype.itemsize, layout, p, w, h, Cc, N)


def halo2d_reduce(bufs, layout, gw, gh, p, w, h, Cc, N):
    dt = F32 if bufs[0].dtype == np.float32 else BF16
    _load().orc_halo2d_reduce(gw, gh, _ptr_array(bufs), dt, layout, p, w, h, Cc, N)


def slice2d(add, count_w, count_h, src, src_w_off, src_h_off, dst, dst_w_off, dst_h_off):
    """src, dst: [N][C][H][W] float32; dst updated in place."""
    N, Cc, sh, sw = src.shape
    _, _, dh, dw = dst.shape
    u = C.c_uint32
    _load().orc_slice2d_hw_nchw_packed(int(add), u(count_w), u(count_h), u(sw), u(sh), u(dw), u(dh), u(Cc), u(N),
                                       _p(src), u(src_w_off), u(src_h_off), _p(dst), u(dst_w_off), u(dst_h_off))


def halo_pad_fwd(x, p):
    N, Cc, h, W = x.shape
    y = np.empty((N, Cc, h + 2 * p, W + 2 * p), np.float32)
    _load().orc_halo_pad_fwd(p, W, h, Cc, N, _p(_f32(x)), _p(y))
    return y


def halo_pad_bwd(dy_padded, dx, p):
    N, Cc, h, W = dx.shape
    _load().orc_halo_pad_bwd(p, W, h, Cc, N, _p(dy_padded), _p(dx))


def _conv_dims(x_shape, w_shape, stride, dil, pad):
    N, Cc, H, W = x_shape
    K, _, kh, kw = w_shape
    P = (H + 2 * pad[0] - dil[0] * (kh - 1) - 1) // stride[0] + 1
    Q = (W + 2 * pad[1] - dil[1] * (kw - 1) - 1) // stride[1] + 1
    return N, Cc, H, W, K, kh, kw, P, Q


def conv2d_fprop(x, w, bias=None, stride=(1, 1), dil=(1, 1), pad=(0, 0), omp=False):
    x, w = _f32(x), _f32(w)
    N, Cc, H, W, K, kh, kw, P, Q = _conv_dims(x.shape, w.shape, stride, dil, pad)
    y = np.empty((N, K, P, Q), np.float32)
    b = _f32(bias) if bias is not None else None
    _load(omp).orc_conv2d_fprop(_p(x), _p(w), _p(b), _p(y), N, Cc, H, W, K, kh, kw, stride[0], stride[1], dil[0], dil[1],
                                pad[0], pad[1])
    return y


def conv2d_dgrad(dy, w, x_shape, stride=(1, 1), dil=(1, 1), pad=(0, 0), dx=None, omp=False):
    dy, w = _f32(dy), _f32(w)
    N, Cc, H, W, K, kh, kw, P, Q = _conv_dims(x_shape, w.shape, stride, dil, pad)
    if dx is None:
        dx = np.zeros(x_shape, np.float32)
    _load(omp).orc_conv2d_dgrad(_p(dy), _p(w), _p(dx), N, Cc, H, W, K, kh, kw, stride[0], stride[1], dil[0], dil[1],
                                pad[0], pad[1])
    return dx


def conv2d_wgrad(x, dy, w_shape, stride=(1, 1), dil=(1, 1), pad=(0, 0), dw=None, db=None, omp=False):
    x, dy = _f32(x), _f32(dy)
    N, Cc, H, W, K, kh, kw, P, Q = _conv_dims(x.shape, w_shape, stride, dil, pad)
    if dw is None:
        dw = np.zeros(w_shape, np.float32)
    _load(omp).orc_conv2d_wgrad(_p(x), _p(dy), _p(dw), _p(db), N, Cc, H, W, K, kh, kw, stride[0], stride[1], dil[0],
                                dil[1], pad[0], pad[1])
    return dw


def maxpool2d_fwd(x, k, s, omp=False):
    x = _f32(x)
    N, Cc, H, W = x.shape
    P, Q = (H - k[0]) // s[0] + 1, (W - k[1]) // s[1] + 1
    y = np.empty((N, Cc, P, Q), np.float32)
    _load(omp).orc_maxpool2d_fwd(_p(x), _p(y), None, N, Cc, H, W, k[0], k[1], s[0], s[1])
    return y


def maxpool2d_bwd(x, dy, k, s, dx=None, omp=False):
    x, dy = _f32(x), _f32(dy)
    N, Cc, H, W = x.shape
    if dx is None:
        dx = np.zeros_like(x)
    _load(omp).orc_maxpool2d_bwd(_p(x), _p(dy), _p(dx), N, Cc, H, W, k[0], k[1], s[0], s[1])
    return dx


def bn_fwd_train(x, gamma, beta, eps=1e-5, relu=False, omp=False):
    x = _f32(x)
    N, Cc, H, W = x.shape
    y = np.empty_like(x)
    mean, invstd, var = (np.empty(Cc, np.float32) for _ in range(3))
    _load(omp).orc_bn_fwd_train(_p(x), _p(_f32(gamma)), _p(_f32(beta)), _p(y), _p(mean), _p(invstd), _p(var), N, Cc,
                                H * W, C.c_float(eps), int(relu))
    return y, mean, invstd, var


def bn_bwd(x, dy, gamma, beta, mean, invstd, relu=False, dx=None, omp=False):
    x, dy = _f32(x), _f32(dy)
    N, Cc, H, W = x.shape
    if dx is None:
        dx = np.zeros_like(x)
    dgamma, dbeta = np.zeros(Cc, np.float32), np.zeros(Cc, np.float32)
    _load(omp).orc_bn_bwd(_p(x), _p(dy), _p(_f32(gamma)), _p(_f32(beta)), _p(_f32(mean)), _p(_f32(invstd)), _p(dx),
                          _p(dgamma), _p(dbeta), N, Cc, H * W, int(relu))
    return dx, dgamma, dbeta


def relu_fwd(x):
    x = _f32(x)
    y = np.empty_like(x)
    _load().orc_relu_fwd(C.c_size_t(x.size), _p(x), _p(y))
    return y


def relu_bwd(x, dy, dx):
    _load().orc_relu_bwd(C.c_size_t(x.size), _p(_f32(x)), _p(_f32(dy)), _p(dx))
    return dx


def array_op(name, x, y, a=0.0, b=0.0):
    """In place on y.  name: add | add_scaled | add_online | scale | scale_add."""
    n = C.c_size_t(y.size)
    L = _load()
    fa, fb = C.c_float(a), C.c_float(b)
    if name == "add":
        L.orc_array_add(n, _p(x), _p(y))
    elif name == "add_scaled":
        L.orc_array_add_scaled(n, fa, fb, _p(x), _p(y))
    elif name == "add_online":
        L.orc_array_add_online(n, fa, _p(x), _p(y))
    elif name == "scale":
        L.orc_array_scale(n, fa, _p(x), _p(y))
    elif name == "scale_add":
        L.orc_array_scale_add(n, fa, _p(x), _p(y))
    else:
        raise ValueError(name)
    return y


def softmax_nll_loss_fwd(y, label):
    B, Cc = y.shape
    loss = np.empty(B, np.float32)
    _load().orc_softmax_nll_loss_fwd(C.c_uint32(Cc), C.c_uint32(B), _p(_f32(y)), _p(label), _p(loss))
    return loss


def softmax_nll_loss_bwd(y, label, dloss, dx):
    B, Cc = y.shape
    _load().orc_softmax_nll_loss_bwd(C.c_uint32(Cc), C.c_uint32(B), _p(_f32(y)), _p(label), _p(_f32(dloss)), _p(dx))
    return dx


def softmax_ce_pixel_fwd(logits, label, omp=False):
    """logits [N][C][HW] float32, label [N][HW] uint32 -> (loss [N][HW], prob, picked uint64)."""
    logits = _f32(logits)
    N, Cc, HW = logits.shape
    loss = np.empty((N, HW), np.float32)
    prob = np.empty_like(logits)
    picked = np.empty((N, HW), np.uint64)
    _load(omp).orc_softmax_ce_pixel_fwd(_p(logits), _p(label), _p(prob), _p(loss), _p(picked), N, Cc, HW)
    return loss, prob, picked


def softmax_ce_pixel_bwd(logits, label, dloss, dlogits=None, omp=False):
    logits = _f32(logits)
    N, Cc, HW = logits.shape
    if dlogits is None:
        dlogits = np.zeros_like(logits)
    _load(omp).orc_softmax_ce_pixel_bwd(_p(logits), _p(label), _p(_f32(dloss)), _p(dlogits), N, Cc, HW)
    return dlogits


def upsample_bilinear_fwd(x, scale):
    x = _f32(x)
    N, Cc, H, W = x.shape
    y = np.empty((N, Cc, H * scale, W * scale), np.float32)
    _load().orc_upsample_bilinear_fwd(_p(x), _p(y), N * Cc, H, W, scale)
    return y


def upsample_bilinear_bwd(dy, scale, dx=None):
    dy = _f32(dy)
    N, Cc, OH, OW = dy.shape
    if dx is None:
        dx = np.zeros((N, Cc, OH // scale, OW // scale), np.float32)
    _load().orc_upsample_bilinear_bwd(_p(dy), _p(dx), N * Cc, OH // scale, OW // scale, scale)
    return dx


def avgpool2d_fwd(x, k, s):
    """Mean over kh x kw windows, no implicit pad (cudnnPoolingForward, AVERAGE; reference src/op.cc:3496-3513)."""
    x = np.asarray(x, np.float64)
    N, Cc, H, W = x.shape
    P, Q = (H - k[0]) // s[0] + 1, (W - k[1]) // s[1] + 1
    y = np.zeros((N, Cc, P, Q), np.float64)
    for a in range(k[0]):
        for b in range(k[1]):
            y += x[:, :, a:a + (P - 1) * s[0] + 1:s[0], b:b + (Q - 1) * s[1] + 1:s[1]]
    return (y / (k[0] * k[1])).astype(np.float32)


def avgpool2d_bwd(dy, x_shape, k, s):
    dy = np.asarray(dy, np.float64)
    N, Cc, P, Q = dy.shape
    dx = np.zeros(x_shape, np.float64)
    for a in range(k[0]):
        for b in range(k[1]):
            dx[:, :, a:a + (P - 1) * s[0] + 1:s[0], b:b + (Q - 1) * s[1] + 1:s[1]] += dy
    return (dx / (k[0] * k[1])).astype(np.float32)


def linear_fwd(x, w, bias=None):
    """y = x w^T + bias, w [out][in] (cublasSgemm + bias add, reference src/op.cc:1199-1247)."""
    y = np.asarray(x, np.float64) @ np.asarray(w, np.float64).T
    if bias is not None:
        y = y + np.asarray(bias, np.float64)
    return y.astype(np.float32)


def linear_bwd(x, w, dy):
    """(dx, dw, db) of linear_fwd (reference src/op.cc:1249-1340)."""
    x, w, dy = np.asarray(x, np.float64), np.asarray(w, np.float64), np.asarray(dy, np.float64)
    return (dy @ w).astype(np.float32), (dy.T @ x).astype(np.float32), dy.sum(axis=0).astype(np.float32)


def sgd_step(theta, g, m, l2, mu, alpha, alpha_next, nesterov):
    f = C.c_float
    _load().orc_sgd_step(C.c_size_t(theta.size), _p(theta), _p(g), _p(m), f(l2), f(mu), f(alpha), f(alpha_next),
                         int(nesterov))


def nchw_to_nhwc(x):
    return np.ascontiguousarray(np.transpose(x, (0, 2, 3, 1)))


def nhwc_to_nchw(x):
    return np.ascontiguousarray(np.transpose(x, (0, 3, 1, 2)))
