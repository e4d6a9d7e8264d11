"""The allocation-free batch-norm entry point against the ordinary one.

Some users of the library cannot allocate device memory for the statistics scratch -- their
code runs inside a framework whose own pool owns the device, or inside a loop where cudaMalloc's
implicit synchronisation is not acceptable.  ad_bn_fwd_train_noalloc serves them from a fixed
array inside the library (at most 2048 channels).  This file is collected last on purpose, so a
run that stops at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from arraydiff_cuda_b200 import abi
from tests import helpers as H

pytestmark = pytest.mark.gpu
f32 = C.c_float


def _run_pair(seed, N, Cc, Hh, W, relu):
    """Same inputs through both entry points; returns (outputs of existing, outputs of no-alloc)."""
    import torch
    L = abi.lib()
    x = H.normal(seed, (N, Hh, W, Cc)) * 1.5 + 0.25
    gamma, beta = H.uniform(seed + 1, (Cc,), 0.5, 1.5), H.uniform(seed + 2, (Cc,), -0.5, 0.5)
    dx, dg, db = H.dev_bf16(x), H.dev(gamma), H.dev(beta)
    vx = H.view_nhwc(dx)
    outs = []
    for noalloc in (False, True):
        y = torch.zeros_like(dx)
        vy = H.view_nhwc(y)
        mean, invstd, var = (torch.zeros(Cc, device="cuda") for _ in range(3))
        if noalloc:
            st = L.ad_bn_fwd_train_noalloc(C.byref(vx), C.byref(vy), H.ptr(dg), H.ptr(db), H.ptr(mean), H.ptr(invstd),
                                           H.ptr(var), f32(1e-5), relu, H.stream())
        else:
            n = L.ad_bn_scratch_bytes(Cc)
            scratch = torch.empty(n, dtype=torch.uint8, device="cuda")
            st = L.ad_bn_fwd_train(C.byref(vx), C.byref(vy), H.ptr(dg), H.ptr(db), H.ptr(mean), H.ptr(invstd),
                                   H.ptr(var), f32(1e-5), relu, H.ptr(scratch), n, H.stream())
        abi.check(st)
        H.sync()
        outs.append([H.host(t) for t in (y, mean, invstd, var)])
    return outs


def test_noalloc_batch_norm_matches_existing_entry_point_twice_in_a_row():
    # two calls in a row with different shapes and data: the second must not see the first's leftovers
    for seed, shape, relu in ((100, (2, 96, 33, 29), 1), (200, (1, 320, 17, 41), 0)):
        N, Cc, Hh, W = shape
        ref, got = _run_pair(seed, N, Cc, Hh, W, relu)
        for a, b in zip(ref, got):
            assert H.max_rel(b, a) < 1e-5


@pytest.mark.parametrize("shape", [(2, 64, 31, 20), (1, 256, 9, 33), (1, 2048, 6, 7)])
def test_noalloc_batch_norm_vector_kernels_and_channel_limit(shape):
    # 64 and 256 channels take the 16-byte vector kernels; 2048 channels use the built-in array to its last byte
    N, Cc, Hh, W = shape
    for seed, relu in ((300, 0), (400, 1)):
        ref, got = _run_pair(seed + Cc, N, Cc, Hh, W, relu)
        for a, b in zip(ref, got):
            assert H.max_rel(b, a) < 1e-5


def test_noalloc_batch_norm_refuses_more_channels_than_its_array_holds():
    import torch
    L = abi.lib()
    Cc = 2049
    x = torch.zeros((1, 2, 2, Cc), dtype=torch.bfloat16, device="cuda")
    y = torch.zeros_like(x)
    v = torch.zeros(Cc, device="cuda")
    before = L.ad_launch_count()
    st = L.ad_bn_fwd_train_noalloc(C.byref(H.view_nhwc(x)), C.byref(H.view_nhwc(y)), H.ptr(v), H.ptr(v), H.ptr(v), H.ptr(v),
                                   H.ptr(v), f32(1e-5), 0, H.stream())
    assert st == abi.AD_ERR_LIMIT
    assert b"limit" in L.ad_status_string(st)
    assert L.ad_launch_count() == before
