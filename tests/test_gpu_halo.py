"""Halo exchange / accumulate-back / slice / pad kernels against the oracle: bit-exact."""
import ctypes as C

import numpy as np
import pytest

from arraydiff_cuda_b200 import abi
from oracle import orc
from tests import helpers as H

pytestmark = pytest.mark.gpu
GUARD = 64  # sentinel elements either side of every buffer


def guarded(arr):
    """Device copy of arr with sentinel guard bands; returns (whole tensor, view)."""
    import torch
    flat = np.ascontiguousarray(arr).reshape(-1)
    sent = np.full(GUARD, 12345.0 if arr.dtype == np.float32 else 0x4E4E, arr.dtype)
    whole = torch.from_numpy(np.concatenate([sent, flat, sent]).view(np.int32 if arr.dtype == np.float32 else np.int16)).cuda()
    return whole, GUARD * arr.dtype.itemsize


def unguard(whole, arr):
    raw = whole.cpu().numpy().view(arr.dtype)
    sent = 12345.0 if arr.dtype == np.float32 else 0x4E4E
    assert np.all(raw[:GUARD] == sent) and np.all(raw[-GUARD:] == sent), "guard band overwritten"
    return raw[GUARD:-GUARD].reshape(arr.shape)


GEOMS = [
    # p, W, h, C, N
    (1, 5, 2, 3, 2), (2, 8, 4, 2, 1), (3, 17, 6, 1, 2), (1, 1, 2, 2, 1), (3, 224, 7, 4, 2), (1, 600, 3, 2, 1),
]


@pytest.mark.parametrize("R", [2, 4, 8])
@pytest.mark.parametrize("geom", GEOMS)
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("layout", [abi.AD_NCHW, abi.AD_NHWC])
@pytest.mark.parametrize("push", [1, 0])
def test_halo_exchange_bit_exact(R, geom, dtype, layout, push):
    p, W, h, Cc, N = geom
    full = H.uniform(11, (N, Cc, h * R, W))
    strips = H.split_strips(full, R, p)
    if layout == abi.AD_NHWC:
        strips = [orc.nchw_to_nhwc(s) for s in strips]
    if dtype == "bf16":
        strips = [orc.f32_to_bf16(s) for s in strips]
    want = [s.copy() for s in strips]
    orc.halo_exchange(want, layout, p, W, h, Cc, N)
    g = [guarded(s) for s in strips]
    bufs = [w.data_ptr() + off for w, off in g]
    a = H.halo_args(bufs, abi.AD_F32 if dtype == "f32" else abi.AD_BF16, layout, p, W, h, Cc, N, push=push)
    abi.check(abi.lib().ad_halo_exchange(C.byref(a), H.stream()))
    H.sync()
    for r in range(R):
        assert np.array_equal(unguard(g[r][0], strips[r]), want[r]), r


@pytest.mark.parametrize("R", [2, 4, 8])
@pytest.mark.parametrize("geom", GEOMS)
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("layout", [abi.AD_NCHW, abi.AD_NHWC])
def test_halo_reduce_bit_exact(R, geom, dtype, layout):
    p, W, h, Cc, N = geom
    if h < 2 * p:
        pytest.skip("h < 2p")
    shape = (N, Cc, h + 2 * p, W + 2 * p) if layout == abi.AD_NCHW else (N, h + 2 * p, W + 2 * p, Cc)
    strips = [H.uniform(20 + r, shape) for r in range(R)]
    if dtype == "bf16":
        strips = [orc.f32_to_bf16(s) for s in strips]
    want = [s.copy() for s in strips]
    orc.halo_reduce(want, layout, p, W, h, Cc, N)
    g = [guarded(s) for s in strips]
    bufs = [w.data_ptr() + off for w, off in g]
    a = H.halo_args(bufs, abi.AD_F32 if dtype == "f32" else abi.AD_BF16, layout, p, W, h, Cc, N)
    abi.check(abi.lib().ad_halo_reduce(C.byref(a), H.stream()))
    H.sync()
    for r in range(R):
        assert np.array_equal(unguard(g[r][0], strips[r]), want[r]), r


def test_halo_per_rank_launches_equal_one_launch():
    """One launch per rank (the multi-GPU calling pattern) gives the same bytes as one launch for all."""
    R, (p, W, h, Cc, N) = 4, (2, 31, 5, 3, 2)
    full = H.uniform(30, (N, Cc, h * R, W))
    strips = H.split_strips(full, R, p)
    want = [s.copy() for s in strips]
    orc.halo_exchange(want, orc.NCHW, p, W, h, Cc, N)
    d = [H.dev(s) for s in strips]
    for r in range(R):
        a = H.halo_args(d, abi.AD_F32, abi.AD_NCHW, p, W, h, Cc, N, rank_first=r, rank_count=1)
        abi.check(abi.lib().ad_halo_exchange(C.byref(a), H.stream()))
    H.sync()
    for r in range(R):
        assert np.array_equal(H.host(d[r]), want[r])


def test_halo_signal_and_bounded_wait():
    """The exchange publishes its epoch; a wait on a flag nobody sets gives up with a status, no hang."""
    import torch
    R, (p, W, h, Cc, N) = 2, (1, 16, 4, 2, 1)
    d = [H.dev(s) for s in H.split_strips(H.uniform(31, (N, Cc, h * R, W)), R, p)]
    flags = torch.zeros(R, dtype=torch.int64, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    a = H.halo_args(d, abi.AD_F32, abi.AD_NCHW, p, W, h, Cc, N)
    for r in range(R):
        a.signal_flags[r] = flags.data_ptr() + 8 * r
    a.epoch = 5
    a.block_counter = counter.data_ptr()
    L = abi.lib()
    abi.check(L.ad_halo_exchange(C.byref(a), H.stream()))
    abi.check(L.ad_flag_wait(C.c_void_p(flags.data_ptr()), 5, 100_000_000, C.c_void_p(status.data_ptr()), H.stream()))
    H.sync()
    assert flags.tolist() == [5, 5] and counter.item() == 0 and status[0].item() == 0
    # a flag that nothing sets: the wait must end by itself and report
    abi.check(L.ad_flag_wait(C.c_void_p(flags.data_ptr() + 8), 99, 20_000_000, C.c_void_p(status.data_ptr() + 4), H.stream()))
    H.sync()
    assert status[1].item() == abi.AD_ERR_TIMEOUT
    abi.check(L.ad_flag_signal(C.c_void_p(flags.data_ptr() + 8), 99, H.stream()))
    H.sync()
    assert flags[1].item() == 99


def test_relative_flag_values_and_peer_sum():
    """Flag values relative to a device-resident base (what lets a recorded step replay): signal / wait / advance,
    the exchange's published value, and the fixed-order sum over buffers that the gradient exchange is built from."""
    import torch
    L = abi.lib()
    base = torch.full((1,), 10, dtype=torch.int64, device="cuda")
    flags = torch.zeros(2, dtype=torch.int64, device="cuda")
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    vp = lambda t, off=0: C.c_void_p(t.data_ptr() + off)
    for _ in range(3):       # the same three calls "replayed": the base moves, the offsets stay
        abi.check(L.ad_flag_signal_rel(vp(flags), vp(base), 2, H.stream()))
        abi.check(L.ad_flag_wait_rel(vp(flags), vp(base), 2, 100_000_000, vp(status), H.stream()))
        abi.check(L.ad_flag_advance(vp(base), 2, H.stream()))
    H.sync()
    assert flags[0].item() == 16 and base.item() == 16 and status[0].item() == 0
    abi.check(L.ad_flag_wait_rel(vp(flags, 8), vp(base), 1, 20_000_000, vp(status, 4), H.stream()))   # nobody sets it
    H.sync()
    assert status[1].item() == abi.AD_ERR_TIMEOUT
    R, (p, W, h, Cc, N) = 2, (1, 16, 4, 2, 1)
    d = [H.dev(s) for s in H.split_strips(H.uniform(32, (N, Cc, h * R, W)), R, p)]
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    a = H.halo_args(d, abi.AD_F32, abi.AD_NCHW, p, W, h, Cc, N)
    for r in range(R):
        a.signal_flags[r] = flags.data_ptr() + 8 * r
    a.epoch, a.epoch_base, a.block_counter = 3, base.data_ptr(), counter.data_ptr()
    abi.check(L.ad_halo_exchange(C.byref(a), H.stream()))
    H.sync()
    assert flags.tolist() == [19, 19]
    # sum over 3 buffers of a ragged range, in buffer order; elements outside the range are not touched
    n = 1003
    bufs = [H.dev(H.uniform(40 + q, (n,))) for q in range(3)]
    out = torch.full((n,), 7.0, device="cuda")
    ptrs = (C.c_void_p * 3)(*[b.data_ptr() for b in bufs])
    abi.check(L.ad_peer_sum(3, ptrs, vp(out), 5, 998, H.stream()))
    H.sync()
    want = (H.host(bufs[0]) + H.host(bufs[1])) + H.host(bufs[2])
    got = H.host(out)
    assert np.array_equal(got[5:998], want[5:998]) and np.all(got[:5] == 7.0) and np.all(got[998:] == 7.0)
    assert L.ad_peer_sum(9, ptrs, vp(out), 0, n, H.stream()) == abi.AD_ERR_BAD_ARG
    assert L.ad_peer_sum(3, ptrs, vp(out, 4), 0, n, H.stream()) == abi.AD_ERR_ALIGN


def test_halo_bad_arguments_rejected_before_launch():
    d = [H.dev(np.zeros((1, 1, 4, 6), np.float32)) for _ in range(2)]
    L = abi.lib()
    before = L.ad_launch_count()
    a = H.halo_args(d, abi.AD_F32, abi.AD_NCHW, 2, 2, 2, 1, 1)          # h < 2p
    assert L.ad_halo_exchange(C.byref(a), H.stream()) == abi.AD_ERR_BAD_ARG
    a = H.halo_args(d, 7, abi.AD_NCHW, 1, 4, 2, 1, 1)                    # unknown dtype
    assert L.ad_halo_exchange(C.byref(a), H.stream()) == abi.AD_ERR_UNSUPPORTED
    a = H.halo_args(d, abi.AD_F32, abi.AD_NCHW, 1, 4, 2, 1, 1)
    a.num_ranks = 9
    assert L.ad_halo_reduce(C.byref(a), H.stream()) == abi.AD_ERR_BAD_ARG
    a = H.halo_args(d, abi.AD_F32, abi.AD_NCHW, 1, 4, 2, 1, 1)
    a.bufs[1] = None
    assert L.ad_halo_exchange(C.byref(a), H.stream()) == abi.AD_ERR_BAD_ARG
    assert L.ad_halo_exchange(None, H.stream()) == abi.AD_ERR_BAD_ARG
    assert L.ad_launch_count() == before


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("add", [0, 1])
@pytest.mark.parametrize("case", [
    # count_w, count_h, src (H, W), dst (H, W), src off (w, h), dst off (w, h), C, N
    (4, 3, (7, 9), (5, 11), (2, 1), (5, 2), 3, 2),
    (224, 28, (112, 224), (28, 224), (0, 56), (0, 0), 4, 2),   # scatter a strip out of a full image
    (33, 5, (5, 33), (11, 39), (0, 0), (3, 3), 2, 1),           # halo pad: interior into a padded buffer
    (1, 1, (1, 1), (1, 1), (0, 0), (0, 0), 1, 1),
    (1100, 2, (2, 1100), (4, 1102), (0, 0), (1, 1), 1, 1),
])
def test_slice_copy_add_bit_exact(dtype, add, case):
    cw, ch, (sh, sw), (dh, dw), (swo, sho), (dwo, dho), Cc, N = case
    src, dst = H.uniform(40, (N, Cc, sh, sw)), H.uniform(41, (N, Cc, dh, dw))
    want = dst.copy()
    if dtype == "bf16":
        src, dst = orc.round_bf16(src), orc.round_bf16(dst)
        want = dst.copy()
        orc.slice2d(add, cw, ch, src, swo, sho, want, dwo, dho)
        want = orc.f32_to_bf16(want)  # one rounding of an exact fp32 sum == fp32 add + RNE
        src_b, dst_b = orc.f32_to_bf16(src), orc.f32_to_bf16(dst)
        gs, gd = guarded(src_b), guarded(dst_b)
    else:
        orc.slice2d(add, cw, ch, src, swo, sho, want, dwo, dho)
        gs, gd = guarded(src), guarded(dst)
    L = abi.lib()
    fn = L.ad_slice2d_add_hw_nchw_packed if add else L.ad_slice2d_copy_hw_nchw_packed
    abi.check(fn(abi.AD_F32 if dtype == "f32" else abi.AD_BF16, cw, ch, sw, sh, dw, dh, Cc, N,
                 C.c_void_p(gs[0].data_ptr() + gs[1]), swo, sho, C.c_void_p(gd[0].data_ptr() + gd[1]), dwo, dho, H.stream()))
    H.sync()
    got = unguard(gd[0], dst_b if dtype == "bf16" else dst)
    assert np.array_equal(got, want)
    unguard(gs[0], src_b if dtype == "bf16" else src)


def test_slice_rejects_windows_outside_the_tensors():
    d = H.dev(np.zeros((1, 1, 4, 4), np.float32))
    L = abi.lib()
    st = L.ad_slice2d_copy_hw_nchw_packed(abi.AD_F32, 3, 3, 4, 4, 4, 4, 1, 1, H.ptr(d), 2, 0, H.ptr(d), 0, 0, H.stream())
    assert st == abi.AD_ERR_BAD_ARG


def test_config2_full_size_exchange_and_reduce():
    """benchmark config 2 at full size: N=8, C=256, 224x224, R in {2,4,8}, p in {1,3}, fp32 and bf16.
    Checked through a size-independent property: after the exchange each strip equals the window of
    the zero-padded full tensor (compared on the device), and reduce is the overlap-add."""
    import torch
    N, Cc, Hh, W = 8, 256, 224, 224
    gen = torch.Generator(device="cuda").manual_seed(50)
    full = torch.rand((N, Cc, Hh, W), device="cuda", generator=gen) * 2 - 1
    L = abi.lib()
    for dt, tdt in ((abi.AD_F32, torch.float32), (abi.AD_BF16, torch.bfloat16)):
        f = full.to(tdt)
        for R in (2, 4, 8):
            for p in (1, 3):
                h = Hh // R
                padded = torch.zeros((N, Cc, Hh + 2 * p, W + 2 * p), device="cuda", dtype=tdt)
                padded[:, :, p:p + Hh, p:p + W] = f
                strips = []
                for r in range(R):
                    s = torch.zeros((N, Cc, h + 2 * p, W + 2 * p), device="cuda", dtype=tdt)
                    s[:, :, p:p + h, p:p + W] = f[:, :, r * h:(r + 1) * h]
                    strips.append(s)
                a = H.halo_args(strips, dt, abi.AD_NCHW, p, W, h, Cc, N)
                abi.check(L.ad_halo_exchange(C.byref(a), H.stream()))
                for r in range(R):
                    assert torch.equal(strips[r], padded[:, :, r * h:r * h + h + 2 * p]), (dt, R, p, r)
                # reduce: strips now hold overlapping windows; overlap-add of interiors
                before = [s.clone() for s in strips]
                abi.check(L.ad_halo_reduce(C.byref(a), H.stream()))
                for r in range(R):
                    want = before[r].clone().float()
                    if r + 1 < R:
                        want[:, :, h:h + p, p:p + W] += before[r + 1][:, :, 0:p, p:p + W].float()
                    if r > 0:
                        want[:, :, p:2 * p, p:p + W] += before[r - 1][:, :, p + h:, p:p + W].float()
                    assert torch.equal(strips[r], want.to(tdt)), (dt, R, p, r)
