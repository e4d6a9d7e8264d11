"""Halo exchange and accumulate-back on 2-D rank grids (W-split, 2 x 2, 2 x 4 ...) against the CPU oracle, bit for bit;
all ranks share one GPU and move in one call (the reference's single-process model)."""
import ctypes as C

import numpy as np
import pytest

from arraydiff_cuda_b200 import abi
from oracle import orc
from tests import helpers as H
from tests.test_halo2d_oracle import split2d, windows2d

pytestmark = pytest.mark.gpu
GRIDS = [(2, 1), (1, 2), (2, 2), (4, 2), (2, 4), (8, 1), (3, 2)]      # (grid_w, grid_h)


def args2d(bufs, dtype, layout, gw, gh, p, w, h, Cc, N, push=1, first=0, count=None):
    a = abi.Halo2dArgs()
    a.dtype, a.layout = dtype, layout
    a.halo_pad, a.base_width, a.base_height, a.num_channels, a.batch_size = p, w, h, Cc, N
    a.grid_w, a.grid_h, a.rank_first, a.rank_count, a.push = gw, gh, first, len(bufs) if count is None else count, push
    for i, b in enumerate(bufs):
        a.bufs[i] = b.data_ptr()
    return a


def to_dev(arrs, layout, bf16):
    out = []
    for x in arrs:
        if layout == abi.AD_NHWC:
            x = np.ascontiguousarray(x.transpose(0, 2, 3, 1))
        out.append(H.dev_bf16(x) if bf16 else H.dev(x))
    return out


def to_host(t, layout):
    x = H.host(t)
    return x.transpose(0, 3, 1, 2) if layout == abi.AD_NHWC else x


@pytest.mark.parametrize("grid", GRIDS)
@pytest.mark.parametrize("layout", [abi.AD_NCHW, abi.AD_NHWC])
@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("push", [1, 0])
def test_exchange_2d_bit_exact(grid, layout, bf16, push):
    gw, gh = grid
    p, N, Cc, h, w = 3, 2, 5, 7, 9
    full = H.uniform(11, (N, Cc, gh * h, gw * w))
    if bf16:
        full = orc.round_bf16(full)
    want = windows2d(full, gw, gh, p)
    bufs = to_dev(split2d(full, gw, gh, p), layout, bf16)
    a = args2d(bufs, abi.AD_BF16 if bf16 else abi.AD_F32, layout, gw, gh, p, w, h, Cc, N, push=push)
    abi.check(abi.lib().ad_halo2d_exchange(C.byref(a), H.stream()))
    H.sync()
    for r, b in enumerate(bufs):
        assert np.array_equal(to_host(b, layout), want[r]), r


@pytest.mark.parametrize("grid", GRIDS)
@pytest.mark.parametrize("layout", [abi.AD_NCHW, abi.AD_NHWC])
@pytest.mark.parametrize("bf16", [False, True])
def test_reduce_2d_bit_exact(grid, layout, bf16):
    gw, gh = grid
    p, N, Cc, h, w = 2, 1, 4, 6, 5
    grads = [H.uniform(30 + r, (N, Cc, h + 2 * p, w + 2 * p)) for r in range(gw * gh)]
    if bf16:
        grads = [orc.round_bf16(g) for g in grads]
    if bf16:
        ref = [orc.f32_to_bf16(g) for g in grads]
        orc.halo2d_reduce(ref, orc.NCHW, gw, gh, p, w, h, Cc, N)
        want = [orc.bf16_to_f32(g) for g in ref]
    else:
        want = [g.copy() for g in grads]
        orc.halo2d_reduce(want, orc.NCHW, gw, gh, p, w, h, Cc, N)
    bufs = to_dev(grads, layout, bf16)
    a = args2d(bufs, abi.AD_BF16 if bf16 else abi.AD_F32, layout, gw, gh, p, w, h, Cc, N)
    abi.check(abi.lib().ad_halo2d_reduce(C.byref(a), H.stream()))
    H.sync()
    for r, b in enumerate(bufs):
        assert np.array_equal(to_host(b, layout), want[r]), r


@pytest.mark.parametrize("grid", [(2, 2), (2, 4)])
def test_exchange_2d_full_size_windows(grid):
    """N=8, C=256, 224 x 224 (the halo microbenchmark's tensor) on a 2-D grid, bf16 NHWC: every buffer equals its window of
    the zero-padded whole tensor, checked on the device."""
    import torch
    gw, gh = grid
    p, N, Cc, Hh, W = 3, 8, 256, 224, 224
    h, w = Hh // gh, W // gw
    g = torch.Generator(device="cuda").manual_seed(5)
    full = (torch.rand((N, Hh, W, Cc), device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)
    padded = torch.zeros((N, Hh + 2 * p, W + 2 * p, Cc), dtype=torch.bfloat16, device="cuda")
    padded[:, p:p + Hh, p:p + W] = full
    bufs = []
    for gy in range(gh):
        for gx in range(gw):
            b = torch.zeros((N, h + 2 * p, w + 2 * p, Cc), dtype=torch.bfloat16, device="cuda")
            b[:, p:p + h, p:p + w] = full[:, gy * h:(gy + 1) * h, gx * w:(gx + 1) * w]
            bufs.append(b)
    a = args2d(bufs, abi.AD_BF16, abi.AD_NHWC, gw, gh, p, w, h, Cc, N)
    abi.check(abi.lib().ad_halo2d_exchange(C.byref(a), H.stream()))
    H.sync()
    for gy in range(gh):
        for gx in range(gw):
            assert torch.equal(bufs[gy * gw + gx], padded[:, gy * h:gy * h + h + 2 * p, gx * w:gx * w + w + 2 * p])


def test_halo2d_rejects_bad_arguments():
    import torch
    L = abi.lib()
    b = [torch.zeros(4096, device="cuda") for _ in range(4)]
    a = args2d(b, abi.AD_F32, abi.AD_NCHW, 2, 2, 3, 4, 8, 1, 1)       # w = 4 < 2p
    assert L.ad_halo2d_exchange(C.byref(a), H.stream()) == abi.AD_ERR_BAD_ARG
    a = args2d(b, abi.AD_F32, abi.AD_NCHW, 3, 3, 1, 4, 4, 1, 1)       # 9 ranks
    assert L.ad_halo2d_exchange(C.byref(a), H.stream()) == abi.AD_ERR_BAD_ARG
    a = args2d(b[:3], abi.AD_F32, abi.AD_NCHW, 2, 2, 1, 4, 4, 1, 1, count=3)   # a missing buffer
    assert L.ad_halo2d_reduce(C.byref(a), H.stream()) == abi.AD_ERR_BAD_ARG
    assert L.ad_halo2d_exchange(None, H.stream()) == abi.AD_ERR_BAD_ARG


@pytest.mark.parametrize("grid", [(2, 1), (2, 2), (2, 4)])
@pytest.mark.parametrize("reduce", [0, 1])
def test_spatial2dcomm_group_calls_on_a_2d_grid(grid, reduce):
    """The host-side communicator (Spatial2DComm::InitAll(comms, R_w, R_h), group_start / halo_* / group_end) on grids
    with a W split, ranks sharing the GPU: same bits as the oracle."""
    from arraydiff_cuda_b200 import hostlib
    gw, gh = grid
    p, N, Cc, h, w = 2, 2, 8, 6, 8
    ctx = hostlib.Context([0] * (gw * gh), hostlib.BF16_NHWC, arena_mb=64)
    if reduce:
        host = [orc.round_bf16(H.uniform(60 + r, (N, Cc, h + 2 * p, w + 2 * p))) for r in range(gw * gh)]
        ref = [orc.f32_to_bf16(g) for g in host]
        orc.halo2d_reduce(ref, orc.NCHW, gw, gh, p, w, h, Cc, N)
        want = [orc.bf16_to_f32(g) for g in ref]
    else:
        full = orc.round_bf16(H.uniform(61, (N, Cc, gh * h, gw * w)))
        host, want = split2d(full, gw, gh, p), windows2d(full, gw, gh, p)
    bufs = to_dev(host, abi.AD_NHWC, True)
    H.sync()
    ctx.halo2d(gw, gh, reduce, [b.data_ptr() for b in bufs], True, True, p, w, h, Cc, N)
    for r, b in enumerate(bufs):
        assert np.array_equal(to_host(b, abi.AD_NHWC), want[r]), r
    ctx.close()
