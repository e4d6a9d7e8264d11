"""Pins the CPU oracle's dense operators against the reference's cuDNN call sequences run LIVE on the GPU
(oracle/_ref/libref_cudnn.so, built by `make -C oracle refcudnn`): regenerates the golden vectors in a scratch
folder and runs the same checks as tests/test_golden_cudnn.py on them, then compares with the committed fixture."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIM = os.path.join(ROOT, "oracle", "_ref", "libref_cudnn.so")
pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not os.path.exists(SHIM), reason="cuDNN shim not built")]


def test_oracle_matches_live_cudnn_and_committed_fixture(tmp_path):
    from tests import test_golden_cudnn as G
    subprocess.check_call([sys.executable, os.path.join(ROOT, "tests", "golden", "make_golden_cudnn.py"), str(tmp_path)])
    live = dict(np.load(tmp_path / "reference_cudnn.npz"))
    nc, npool, nbn, nsm = (int(v) for v in live["counts"])
    for i in range(nc):
        G.check_conv(live, i)
    for i in range(npool):
        G.check_pool(live, i)
    for i in range(nbn):
        G.check_bn(live, i)
    for i in range(nsm):
        G.check_softmax(live, i)
    if os.path.exists(G.PATH):
        # the committed vectors are what this box's cuDNN computes too (algorithm choice may differ: tolerance, not bits)
        old = dict(np.load(G.PATH))
        for k, v in live.items():
            if v.dtype == np.float32 and k in old:
                assert np.max(np.abs(v.astype(np.float64) - old[k])) <= 2e-5 * max(1.0, float(np.max(np.abs(old[k])))), k
