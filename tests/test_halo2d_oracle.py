"""The 2-D rank-grid halo oracle on the CPU: after the exchange every rank's padded buffer is its window of the
zero-padded whole tensor; the accumulate-back is the transpose of that (overlap-add); a 1 x R grid agrees with the
1-D oracle that is pinned to the reference's kernels."""
import numpy as np
import pytest

from oracle import orc
from tests import helpers as H

GRIDS = [(1, 2), (2, 1), (2, 2), (4, 2), (2, 4), (8, 1), (1, 8), (3, 2)]     # (grid_w, grid_h)


def split2d(full, gw, gh, p):
    N, Cc, Hh, W = full.shape
    h, w = Hh // gh, W // gw
    out = []
    for gy in range(gh):
        for gx in range(gw):
            s = np.zeros((N, Cc, h + 2 * p, w + 2 * p), full.dtype)
            s[:, :, p:p + h, p:p + w] = full[:, :, gy * h:(gy + 1) * h, gx * w:(gx + 1) * w]
            out.append(s)
    return out


def windows2d(full, gw, gh, p):
    N, Cc, Hh, W = full.shape
    h, w = Hh // gh, W // gw
    padded = np.zeros((N, Cc, Hh + 2 * p, W + 2 * p), full.dtype)
    padded[:, :, p:p + Hh, p:p + W] = full
    return [np.ascontiguousarray(padded[:, :, gy * h:gy * h + h + 2 * p, gx * w:gx * w + w + 2 * p]) for gy in range(gh) for gx in range(gw)]


def overlap_add2d(grads, gw, gh, p):
    """Expected accumulate-back: sum all padded gradient buffers into the padded whole tensor, then every rank's interior
    edge cells hold the whole-tensor sum (float64 here; the device adds in a fixed order in float32)."""
    N, Cc, Hp, Wp = grads[0].shape
    h, w = Hp - 2 * p, Wp - 2 * p
    total = np.zeros((N, Cc, gh * h + 2 * p, gw * w + 2 * p), np.float64)
    for gy in range(gh):
        for gx in range(gw):
            total[:, :, gy * h:gy * h + Hp, gx * w:gx * w + Wp] += grads[gy * gw + gx]
    return [total[:, :, p + gy * h:p + (gy + 1) * h, p + gx * w:p + (gx + 1) * w] for gy in range(gh) for gx in range(gw)]


@pytest.mark.parametrize("grid", GRIDS)
@pytest.mark.parametrize("layout", [orc.NCHW, orc.NHWC])
@pytest.mark.parametrize("p", [1, 3])
def test_exchange_gives_every_rank_its_window(grid, layout, p):
    gw, gh = grid
    N, Cc, h, w = 2, 3, 6, 7
    full = H.uniform(40 + p, (N, Cc, gh * h, gw * w))
    bufs = split2d(full, gw, gh, p)
    want = windows2d(full, gw, gh, p)
    if layout == orc.NHWC:
        bufs = [np.ascontiguousarray(b.transpose(0, 2, 3, 1)) for b in bufs]
    orc.halo2d_exchange(bufs, layout, gw, gh, p, w, h, Cc, N)
    for r, b in enumerate(bufs):
        got = b.transpose(0, 3, 1, 2) if layout == orc.NHWC else b
        assert np.array_equal(got, want[r]), r


@pytest.mark.parametrize("grid", GRIDS)
@pytest.mark.parametrize("p", [1, 2])
def test_reduce_is_overlap_add(grid, p):
    gw, gh = grid
    N, Cc, h, w = 1, 2, 5, 6
    grads = [H.uniform(70 + r, (N, Cc, h + 2 * p, w + 2 * p)) for r in range(gw * gh)]
    want = overlap_add2d(grads, gw, gh, p)
    bufs = [g.copy() for g in grads]
    orc.halo2d_reduce(bufs, orc.NCHW, gw, gh, p, w, h, Cc, N)
    for r, b in enumerate(bufs):
        np.testing.assert_allclose(b[:, :, p:p + h, p:p + w], want[r], rtol=1e-6, atol=1e-6)
        # halo cells are sources only
        m = np.ones_like(b, bool)
        m[:, :, p:p + h, p:p + w] = False
        assert np.array_equal(b[m], grads[r][m])


@pytest.mark.parametrize("R", [2, 4, 8])
def test_one_dimensional_grid_equals_the_strip_oracle(R):
    p, W, h, Cc, N = 2, 9, 5, 3, 2
    full = H.uniform(90, (N, Cc, h * R, W))
    a = H.split_strips(full, R, p)
    b = [x.copy() for x in a]
    orc.halo_exchange(a, orc.NCHW, p, W, h, Cc, N)
    orc.halo2d_exchange(b, orc.NCHW, 1, R, p, W, h, Cc, N)
    for x, y in zip(a, b):
        assert np.array_equal(x, y)
    ga = [H.uniform(91 + r, x.shape) for r, x in enumerate(a)]
    gb = [x.copy() for x in ga]
    orc.halo_reduce(ga, orc.NCHW, p, W, h, Cc, N)
    orc.halo2d_reduce(gb, orc.NCHW, 1, R, p, W, h, Cc, N)
    for x, y in zip(ga, gb):
        assert np.array_equal(x, y)
