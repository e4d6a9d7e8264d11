"""The multi-rank host logic on CPU: two (and four) gloo ranks run the halo plan with numpy strips,
moving rows with send/recv and signalling through a store, and must reproduce the oracle.  Also the
failure path: a neighbour that never signals makes the bounded wait give up with an error, no hang."""
import os
import socket
import time

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from arraydiff_cuda_b200.dist import HaloPlan
from oracle import orc
from tests import helpers as H


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _wait_flag(store, key, epoch, timeout_s):
    """Host twin of ad_flag_wait: poll until flag >= epoch or give up after timeout_s."""
    t0 = time.time()
    while time.time() - t0 < timeout_s:
        if int(store.add(key, 0)) >= epoch:
            return True
        time.sleep(0.005)
    return False


def _worker(rank, world, port, p, W, h, Cc, N, drop_signal_from, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    store = dist.distributed_c10d._get_default_store()
    plan = HaloPlan(rank, world)
    full = H.uniform(77, (N, Cc, h * world, W))
    strip = H.split_strips(full, world, p)[rank]
    want = H.expected_strips_after_exchange(full, world, p)[rank]
    epoch = 1
    # forward push: send my edge rows, the peer stores them and I raise its flag
    reqs = []
    for peer, src_row, _ in plan.push_rows(p, h):
        reqs.append(dist.isend(torch.from_numpy(np.ascontiguousarray(strip[:, :, src_row:src_row + p, p:p + W])), peer))
    for peer, _, _ in plan.push_rows(p, h):       # symmetric: what the peer pushes to me
        peer_plan = HaloPlan(peer, world)
        for tgt, _, dst_row in peer_plan.push_rows(p, h):
            if tgt == rank:
                buf = torch.empty((N, Cc, p, W))
                dist.recv(buf, peer)
                strip[:, :, dst_row:dst_row + p, p:p + W] = buf.numpy()
    for r in reqs:
        r.wait()
    for peer, slot in plan.exchange_signals():
        if drop_signal_from is not None and rank == drop_signal_from:
            continue                                # injected fault: this rank never signals
        store.add(f"flag/{peer}/{slot}", epoch)
    ok = all(_wait_flag(store, f"flag/{rank}/{slot}", epoch, 1.0) for slot in plan.exchange_waits())
    exch_ok = bool(np.array_equal(strip, want))
    # backward: pull the neighbours' halo rows of a gradient strip and add
    g = H.uniform(90 + rank, strip.shape)
    allg = [H.uniform(90 + r, strip.shape) for r in range(world)]
    wantg = [x.copy() for x in allg]
    orc.halo_reduce(wantg, orc.NCHW, p, W, h, Cc, N)
    reqs = []
    for peer, halo_row, _ in plan.pull_rows(p, h):
        # the peer needs MY halo rows facing it: those are its (peer, halo_row) seen from its side
        peer_plan = HaloPlan(peer, world)
        for tgt, my_halo_row, _ in peer_plan.pull_rows(p, h):
            if tgt == rank:
                reqs.append(dist.isend(torch.from_numpy(np.ascontiguousarray(g[:, :, my_halo_row:my_halo_row + p, p:p + W])), peer))
    for peer, _, dst_row in plan.pull_rows(p, h):
        buf = torch.empty((N, Cc, p, W))
        dist.recv(buf, peer)
        g[:, :, dst_row:dst_row + p, p:p + W] += buf.numpy()
    for r in reqs:
        r.wait()
    result[rank] = (exch_ok, ok, bool(np.array_equal(g, wantg[rank])))
    dist.barrier()
    dist.destroy_process_group()


def _run(world, drop=None, geom=(2, 9, 5, 3, 2)):
    p, W, h, Cc, N = geom
    mgr = mp.Manager()
    result = mgr.dict()
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, world, port, p, W, h, Cc, N, drop, result)) for r in range(world)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(120)
        assert pr.exitcode == 0
    return dict(result)


@pytest.mark.parametrize("world", [2, 4])
def test_halo_plan_over_gloo_matches_oracle(world):
    res = _run(world)
    assert len(res) == world
    for r in range(world):
        exch_ok, flags_ok, red_ok = res[r]
        assert exch_ok and flags_ok and red_ok, (r, res[r])


def test_missing_signal_is_detected_not_waited_for_forever():
    res = _run(2, drop=0)
    # rank 0 never signalled: rank 1's bounded wait gives up; rank 0 itself was signalled by rank 1
    assert res[1][1] is False and res[0][1] is True
    assert res[0][0] and res[1][0]      # the data itself did arrive


def test_halo_plan_tables():
    assert HaloPlan(0, 1).exchange_signals() == [] and HaloPlan(0, 1).exchange_waits() == []
    pl = HaloPlan(1, 4)
    assert pl.exchange_signals() == [(2, 0), (0, 1)] and pl.exchange_waits() == [0, 1]
    assert pl.reduce_signals() == [(2, 2), (0, 3)] and pl.reduce_waits() == [2, 3]
    assert pl.push_rows(3, 10) == [(2, 10, 0), (0, 3, 13)]
    assert pl.pull_rows(3, 10) == [(2, 0, 10), (0, 13, 3)]
    assert HaloPlan(3, 4).exchange_waits() == [0] and HaloPlan(0, 4).exchange_waits() == [1]
    with pytest.raises(ValueError):
        HaloPlan(0, 9)
