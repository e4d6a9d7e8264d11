"""Generates tests/golden/reference_cudnn.npz: outputs of the cuDNN legacy-API calls the REFERENCE makes for
convolution, pooling, batch normalisation and softmax (same descriptors as its call sites in src/op.cc,
issued by oracle/ref_cudnn_shim.cu -> oracle/_ref/libref_cudnn.so, built by `make -C oracle refcudnn`),
recorded on a GPU for small seeded fp32 tensors.

    python tests/golden/make_golden_cudnn.py [output_dir]

Every fixture stores inputs and outputs, so the CPU tests can check the oracle against what the reference's
library calls compute without a GPU, cuDNN or the reference.
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from tests import helpers as H  # noqa: E402

LIB = os.path.join(ROOT, "oracle", "_ref", "libref_cudnn.so")

# N, C, H, W, K, kh, kw, stride, dil, pad, halo_padded  (H, W: the dims the call reads)
CONV_CASES = [
    (1, 64, 34, 66, 64, 3, 3, 1, 1, 1, 1),    # benchmark config 1: one halo-padded strip (h = 32, p = 1)
    (2, 3, 37, 41, 8, 7, 7, 2, 1, 3, 0),      # 7x7 stride-2 stem with implicit zero padding
    (2, 5, 22, 27, 6, 3, 3, 1, 3, 3, 1),      # dilation 3 on a halo-3 strip (the microbenchmark's geometry)
    (1, 8, 20, 20, 4, 3, 3, 1, 2, 2, 1),      # dilation 2
    (1, 6, 24, 24, 5, 3, 3, 1, 4, 4, 0),      # dilation 4, implicit padding
    (2, 4, 11, 9, 5, 3, 3, 2, 1, 1, 0),       # 3x3 stride 2, odd extents
    (3, 16, 6, 7, 12, 1, 1, 1, 1, 0, 0),      # 1x1
    (1, 16, 9, 9, 8, 1, 1, 2, 1, 0, 0),       # 1x1 stride-2 projection
]
POOL_CASES = [(2, 3, 12, 14, 3, 3, 2, 0), (1, 4, 9, 9, 3, 3, 2, 0), (2, 5, 7, 7, 7, 7, 1, 1), (1, 3, 8, 8, 2, 2, 2, 1)]
BN_CASES = [(2, 3, 5, 7), (1, 8, 16, 16), (4, 2, 3, 3)]
SOFTMAX_CASES = [(9, 7, 1, 1, 0), (4, 1000, 1, 1, 0), (2, 19, 6, 5, 1), (1, 2, 4, 4, 1)]


def shim():
    lib = C.CDLL(LIB)
    return lib


def P(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def conv(lib, case, x, w, b, dy_seed):
    N, Cc, Hh, W, K, kh, kw, s, d, pd, halo = case
    p = 0 if halo else pd
    Pp = (Hh + 2 * p - d * (kh - 1) - 1) // s + 1
    Q = (W + 2 * p - d * (kw - 1) - 1) // s + 1
    dy = H.uniform(dy_seed, (N, K, Pp, Q))
    y, dx, dw, db = np.empty_like(dy), np.empty_like(x), np.empty_like(w), np.empty(K, np.float32)
    po, qo = C.c_int(), C.c_int()
    st = lib.refcudnn_conv(N, Cc, Hh, W, K, kh, kw, s, d, pd, halo, P(x), P(w), P(b), P(dy), P(y), P(dx), P(dw), P(db),
                           C.byref(po), C.byref(qo))
    assert st == 0, st
    assert (po.value, qo.value) == (Pp, Q)
    return dy, y, dx, dw, db


def main(out_dir):
    lib = shim()
    fx = {"cudnn_version": np.array([lib.refcudnn_version()], np.int64)}
    for i, case in enumerate(CONV_CASES):
        N, Cc, Hh, W, K, kh, kw, s, d, pd, halo = case
        x = H.uniform(100 + i, (N, Cc, Hh, W))
        w = H.normal(200 + i, (K, Cc, kh, kw), float(np.sqrt(2.0 / (kh * kw * Cc))))
        b = H.normal(300 + i, (K,))
        dy, y, dx, dw, db = conv(lib, case, x, w, b, 400 + i)
        fx.update({f"conv{i}_meta": np.array(case, np.int64), f"conv{i}_x": x, f"conv{i}_w": w, f"conv{i}_b": b, f"conv{i}_dy": dy,
                   f"conv{i}_y": y, f"conv{i}_dx": dx, f"conv{i}_dw": dw, f"conv{i}_db": db})
    for i, (N, Cc, Hh, W, kh, kw, s, avg) in enumerate(POOL_CASES):
        x = H.uniform(500 + i, (N, Cc, Hh, W))
        Pp, Q = (Hh - kh) // s + 1, (W - kw) // s + 1
        dy = H.uniform(600 + i, (N, Cc, Pp, Q))
        y, dx = np.empty_like(dy), np.empty_like(x)
        assert lib.refcudnn_pool(N, Cc, Hh, W, kh, kw, s, avg, P(x), P(dy), P(y), P(dx)) == 0
        fx.update({f"pool{i}_meta": np.array([N, Cc, Hh, W, kh, kw, s, avg], np.int64), f"pool{i}_x": x, f"pool{i}_dy": dy,
                   f"pool{i}_y": y, f"pool{i}_dx": dx})
    for i, (N, Cc, Hh, W) in enumerate(BN_CASES):
        x = H.normal(700 + i, (N, Cc, Hh, W), 1.5) + 0.25
        g, b = H.uniform(800 + i, (Cc,), 0.5, 1.5), H.uniform(900 + i, (Cc,), -0.5, 0.5)
        dy = H.uniform(1000 + i, x.shape)
        y, dx = np.empty_like(x), np.empty_like(x)
        sm, si, rm, rv, dg, dbt = (np.empty(Cc, np.float32) for _ in range(6))
        assert lib.refcudnn_bn(N, Cc, Hh, W, P(x), P(g), P(b), P(dy), P(y), P(sm), P(si), P(rm), P(rv), P(dx), P(dg), P(dbt)) == 0
        fx.update({f"bn{i}_x": x, f"bn{i}_gamma": g, f"bn{i}_beta": b, f"bn{i}_dy": dy, f"bn{i}_y": y, f"bn{i}_save_mean": sm,
                   f"bn{i}_save_invstd": si, f"bn{i}_run_mean": rm, f"bn{i}_run_var": rv, f"bn{i}_dx": dx, f"bn{i}_dgamma": dg,
                   f"bn{i}_dbeta": dbt})
    for i, (N, Cc, Hh, W, mode) in enumerate(SOFTMAX_CASES):
        x = H.normal(1100 + i, (N, Cc, Hh, W), 3.0)
        y = np.empty_like(x)
        assert lib.refcudnn_softmax(N, Cc, Hh, W, mode, P(x), P(y)) == 0
        fx.update({f"softmax{i}_mode": np.array([mode], np.int64), f"softmax{i}_x": x, f"softmax{i}_y": y})
    fx["counts"] = np.array([len(CONV_CASES), len(POOL_CASES), len(BN_CASES), len(SOFTMAX_CASES)], np.int64)
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, "reference_cudnn.npz")
    np.savez_compressed(path, **fx)
    print("wrote", path, len(fx), "arrays, cuDNN", int(fx["cudnn_version"][0]))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__)))
