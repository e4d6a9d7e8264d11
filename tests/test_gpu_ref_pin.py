"""Pins the CPU oracle against the reference's own CUDA kernels, run live on the GPU
(oracle/_ref/libref_kernels.so, built from the reference sources by `make -C oracle ref`)."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import orc
from tests import helpers as H

REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libref_kernels.so")
pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not os.path.exists(REF), reason="reference kernels not built")]


@pytest.fixture(scope="module")
def ref():
    return C.CDLL(REF)


@pytest.mark.parametrize("R", [2, 4])
@pytest.mark.parametrize("geom", [(1, 224, 8, 5, 2), (3, 33, 7, 3, 1)])
def test_reference_halo_kernels_match_oracle(ref, R, geom):
    import torch
    p, W, h, Cc, N = geom
    u = C.c_uint32
    full = H.uniform(1, (N, Cc, h * R, W))
    for reduce in (0, 1):
        strips = H.split_strips(full, R, p) if not reduce else [H.uniform(2 + r, (N, Cc, h + 2 * p, W + 2 * p)) for r in range(R)]
        d = [torch.from_numpy(s.copy()).cuda() for s in strips]
        ptrs = [C.c_void_p(t.data_ptr()) for t in d]
        for r in range(R):
            fn = ref.ref_halo_1x2 if R == 2 else ref.ref_halo_1x4
            assert fn(reduce, u(r), u(p), u(W), u(h), u(Cc), u(N), *ptrs, None) == 0
        torch.cuda.synchronize()
        want = [s.copy() for s in strips]
        (orc.halo_reduce if reduce else orc.halo_exchange)(want, orc.NCHW, p, W, h, Cc, N)
        for r in range(R):
            assert np.array_equal(d[r].cpu().numpy(), want[r]), (reduce, r)


@pytest.mark.parametrize("R,p", [(2, 1), (4, 3)])
def test_speed_against_reference_halo_kernels(ref, R, p):
    """Same GPU, same tensors (benchmark config 2, fp32): this library's exchange against the reference's
    own kernel, one launch per rank as the reference does.  Prints both.  The small case (3.5 MiB) sits on
    the launch floor of both; on the larger one ours must be at least 2x faster."""
    import torch
    from arraydiff_cuda_b200 import abi
    N, Cc, Hh, W = 8, 256, 224, 224
    h = Hh // R
    u = C.c_uint32
    bufs = [torch.randn((N, Cc, h + 2 * p, W + 2 * p), device="cuda") for _ in range(R)]
    ptrs = [C.c_void_p(t.data_ptr()) for t in bufs]
    fn = ref.ref_halo_1x2 if R == 2 else ref.ref_halo_1x4

    def run_ref():
        for r in range(R):
            fn(0, u(r), u(p), u(W), u(h), u(Cc), u(N), *ptrs, None)

    a = H.halo_args(bufs, abi.AD_F32, abi.AD_NCHW, p, W, h, Cc, N)
    L = abi.lib()

    def run_ours():
        abi.check(L.ad_halo_exchange(C.byref(a), H.stream()))

    def timed(f):
        for _ in range(5):
            f()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(50):
            f()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 50 * 1e3

    t_ref, t_ours = timed(run_ref), timed(run_ours)
    payload = 2 * (R - 1) * N * Cc * p * W * 4
    print(f"\nhalo exchange R={R} p={p} fp32: reference {t_ref:.1f} us ({payload / t_ref / 1e3:.0f} GB/s), "
          f"this library {t_ours:.1f} us ({payload / t_ours / 1e3:.0f} GB/s)")
    assert t_ours < t_ref
    if payload > (16 << 20):
        assert t_ours * 2 < t_ref
