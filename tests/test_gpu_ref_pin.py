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
