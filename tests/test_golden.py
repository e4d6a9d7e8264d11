"""The CPU oracle against golden vectors recorded from the reference's own CUDA kernels
(tests/golden/reference_kernels.npz, produced by tests/golden/make_golden.py on a B200)."""
import os

import numpy as np
import pytest

from oracle import orc

PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_kernels.npz")
pytestmark = pytest.mark.skipif(not os.path.exists(PATH), reason="golden fixture not generated yet")


@pytest.fixture(scope="module")
def fx():
    return dict(np.load(PATH))


def test_halo_exchange_and_reduce_bit_exact(fx):
    for case in range(int(fx["halo_cases"][0])):
        R, p, W, h, Cc, N = (int(v) for v in fx[f"halo{case}_meta"])
        strips = [fx[f"halo{case}_in{r}"].copy() for r in range(R)]
        orc.halo_exchange(strips, orc.NCHW, p, W, h, Cc, N)
        for r in range(R):
            assert np.array_equal(strips[r], fx[f"halo{case}_exch{r}"]), (case, r)
        g = [fx[f"halo{case}_gin{r}"].copy() for r in range(R)]
        orc.halo_reduce(g, orc.NCHW, p, W, h, Cc, N)
        for r in range(R):
            assert np.array_equal(g[r], fx[f"halo{case}_red{r}"]), (case, r)


def test_slice_bit_exact(fx):
    for add in (0, 1):
        dst = fx["slice_dst_in"].copy()
        orc.slice2d(add, 4, 3, fx["slice_src"], 2, 1, dst, 5, 2)
        assert np.array_equal(dst, fx[f"slice_out{add}"])


def test_nll_label_indexing_and_values(fx):
    y, label = fx["nll_y"], fx["nll_label"]
    loss = orc.softmax_nll_loss_fwd(y, label)
    # index exactness: the loss must be that of the labelled entry and of no other
    np.testing.assert_allclose(loss, fx["nll_loss"], rtol=2e-7, atol=0)
    dx = fx["nll_dx_in"].copy()
    orc.softmax_nll_loss_bwd(y, label, fx["nll_dloss"], dx)
    assert np.array_equal(dx, fx["nll_dx_out"])


@pytest.mark.parametrize("name", ["add", "add_scaled", "add_online", "scale", "scale_add"])
def test_array_ops_bit_exact(fx, name):
    y = fx["arr_y"].copy()
    orc.array_op(name, fx["arr_x"], y, float(fx["arr_a"]), float(fx["arr_b"]))
    assert np.array_equal(y, fx[f"arr_{name}"])
