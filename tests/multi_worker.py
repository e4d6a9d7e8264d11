"""One rank of the multi-GPU tests (launched by tests/test_gpu_multi.py through torch.distributed.run).
Checks, with one process per GPU and peers mapped through CUDA IPC:
  1. halo push with release flags + bounded waits, and the pull-accumulate, bit-exact vs the oracle;
  2. the C++ host layer in distributed mode: partitioned 3x3 conv forward / backward / SGD step with
     the filter-gradient allreduce over NCCL, vs the unpartitioned oracle."""
import ctypes as C
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from arraydiff_cuda_b200 import abi, hostlib  # noqa: E402
from arraydiff_cuda_b200.dist import HaloPlan, SymmetricArena, _Raw  # noqa: E402
from oracle import orc  # noqa: E402
from tests import helpers as H  # noqa: E402


def halo_part(rank, world):
    L = abi.load()
    p, W, h, Cc, N = 3, 50, 8, 5, 2
    full = H.uniform(500, (N, Cc, h * world, W))
    strips = H.split_strips(full, world, p)
    want = H.expected_strips_after_exchange(full, world, p)[rank]
    arena = SymmetricArena(8 << 20, rank, world)
    buf, off = arena.alloc(strips[rank].shape, torch.float32)
    gbuf, goff = arena.alloc(strips[rank].shape, torch.float32)
    flags, foff = arena.alloc((8,), torch.int64)
    buf.copy_(torch.from_numpy(strips[rank]))
    allg = [H.uniform(600 + r, strips[r].shape) for r in range(world)]
    gbuf.copy_(torch.from_numpy(allg[rank]))
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    dist.barrier()
    plan = HaloPlan(rank, world)
    s = H.stream()
    a = H.halo_args(arena.peers(off), abi.AD_F32, abi.AD_NCHW, p, W, h, Cc, N, rank_first=rank, rank_count=1, push=1)
    fp = arena.peers(foff)
    for peer, slot in plan.exchange_signals():
        a.signal_flags[peer] = fp[peer] + 8 * slot
    a.epoch, a.block_counter = 1, counter.data_ptr()
    abi.check(L.ad_halo_exchange(C.byref(a), s))
    for slot in plan.exchange_waits():
        abi.check(L.ad_flag_wait(C.c_void_p(flags.data_ptr() + 8 * slot), 1, 2_000_000_000, H.ptr(status), s))
    torch.cuda.synchronize()
    assert status.item() == 0, "flag wait timed out"
    assert np.array_equal(buf.cpu().numpy(), want), "halo exchange mismatch"
    # backward: signal, wait, pull-accumulate
    for peer, slot in plan.reduce_signals():
        abi.check(L.ad_flag_signal(C.c_void_p(fp[peer] + 8 * slot), 1, s))
    for slot in plan.reduce_waits():
        abi.check(L.ad_flag_wait(C.c_void_p(flags.data_ptr() + 8 * slot), 1, 2_000_000_000, H.ptr(status), s))
    g = H.halo_args(arena.peers(goff), abi.AD_F32, abi.AD_NCHW, p, W, h, Cc, N, rank_first=rank, rank_count=1)
    abi.check(L.ad_halo_reduce(C.byref(g), s))
    torch.cuda.synchronize()
    wantg = [x.copy() for x in allg]
    orc.halo_reduce(wantg, orc.NCHW, p, W, h, Cc, N)
    assert status.item() == 0
    assert np.array_equal(gbuf.cpu().numpy(), wantg[rank]), "halo reduce mismatch"
    dist.barrier()
    arena.close()


_keep = []


def make_dist_ctx(rank, world, local, mode, arena_mb):
    """One rank of a distributed host-layer context: arena handles exchanged through torch.distributed."""
    Lh = hostlib.load()
    ctxh = Lh.adh_context_create_distributed(rank, world, local, mode, arena_mb)
    hb = C.create_string_buffer(64)
    assert Lh.adh_context_arena_handle(ctxh, hb) == 0
    mine = torch.from_numpy(np.frombuffer(hb.raw, dtype=np.uint8).copy()).cuda()
    allh = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(allh, mine)
    for r in range(world):
        if r != rank:
            assert Lh.adh_context_set_peer_handle(ctxh, r, bytes(allh[r].cpu().numpy().tobytes())) == 0

    class Ctx:  # minimal stand-in for hostlib.Context around the distributed handle
        pass
    ctx = Ctx()
    ctx.L, ctx.h, ctx.num_ranks = Lh, ctxh, world
    return ctx


def host_part(rank, world, local):
    Lh = hostlib.load()
    ctx0 = make_dist_ctx(rank, world, local, hostlib.F32_NCHW, 1536)
    ctxh = ctx0.h
    # filter-gradient allreduce over NCCL on the host layer's own stream
    HOOK = C.CFUNCTYPE(None, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p)

    def allreduce(buf, count, stream, user):
        t = torch.as_tensor(_Raw(buf, count * 4), device="cuda").view(torch.float32)
        with torch.cuda.stream(torch.cuda.ExternalStream(stream)):
            dist.all_reduce(t)

    hook = HOOK(allreduce)
    _keep.append(hook)
    Lh.adh_context_set_allreduce_hook(ctxh, C.cast(hook, C.c_void_p), None)

    ctx = ctx0
    N, Cc, K, Hh, W = 1, 64, 64, 64, 64
    net = hostlib.Net(ctx, "conv3x3", Hh, W, Cc, N, K, seed=3)
    x = H.uniform(100, (N, Cc, Hh, W))
    w = H.normal(101, (K, Cc, 3, 3), float(np.sqrt(2.0 / (9 * 64))))
    dy = H.uniform(102, (N, K, Hh, W))
    net.set_params(w.reshape(-1))
    net.configure_sgd(0.1, 0.9, l2=0.0, nesterov=False)
    h = Hh // world
    dist.barrier()
    net.forward(x)
    y = net.output(rank)
    y_w = orc.conv2d_fprop(x, w, None, pad=(1, 1), omp=True)
    assert H.max_rel(y, y_w[:, :, rank * h:(rank + 1) * h]) < 1e-5, "partitioned forward mismatch"
    net.set_output_grad(rank, dy[:, :, rank * h:(rank + 1) * h])
    dist.barrier()
    net.backward()
    dx = net.input_grad(rank)
    dx_w = orc.conv2d_dgrad(dy, w, x.shape, pad=(1, 1), omp=True)
    assert H.max_rel(dx[:, :, rank * h:(rank + 1) * h], dx_w[:, :, rank * h:(rank + 1) * h]) < 1e-5, "dgrad mismatch"
    dist.barrier()
    net.sgd_step()
    net.sync()
    assert net.status() == 0
    dw_w = orc.conv2d_wgrad(x, dy, w.shape, pad=(1, 1), omp=True)
    theta, g, m = w.reshape(-1).copy(), dw_w.reshape(-1).copy(), np.zeros(w.size, np.float32)
    orc.sgd_step(theta, g, m, 0.0, 0.9, 0.1, 0.1, 0)
    assert H.max_rel(net.params(rank), theta) < 1e-5, "update after allreduce mismatch"
    dist.barrier()
    classifier_part(ctx, rank, world)
    graph_part(ctx, rank, world, local, hostlib.F32_NCHW)
    # the tensor-core path, with the convolutions forced to run their interior rows before the halo waits (by default
    # only layers large enough to hide the two extra launches do that), then with the default choice
    os.environ["ARRAYDIFF_B200_HALO_OVERLAP"] = "2"
    graph_part(make_dist_ctx(rank, world, local, hostlib.BF16_NHWC, 1536), rank, world, local, hostlib.BF16_NHWC)
    os.environ.pop("ARRAYDIFF_B200_HALO_OVERLAP")
    graph_part(make_dist_ctx(rank, world, local, hostlib.BF16_NHWC, 1536), rank, world, local, hostlib.BF16_NHWC)


def graph_part(ctx, rank, world, local, mode):
    """Without an allreduce hook the filter gradients are summed by the built-in peer exchange and the whole
    training step replays from a CUDA graph in every process.  In fp32 the parameters after the same steps equal,
    bit for bit, those of the same net run as `world` strips inside one process (eagerly, on rank 0's GPU).  With
    bf16 activations a gradient that two consumers accumulate into is rounded after each of them, and the two
    set-ups walk the consumers in different orders, so there the check is in two parts: replay from the graph
    equals the eager steps of a second net between the same processes bit for bit, and the first step's filter
    gradients agree with the in-process run to bf16 accuracy."""
    ctx.L.adh_context_set_allreduce_hook(ctx.h, None, None)
    bf16 = mode == hostlib.BF16_NHWC
    N, Cc, Hh, W = 1, 3, 64 * world, 64
    x = H.uniform(700, (N, Cc, Hh, W), 0.0, 1.0)
    dy = H.normal(701, (N, 256, Hh // 4, W // 4))
    h = dy.shape[2] // world

    def train(net, ranks, graph, init=None):
        net.configure_sgd(1e-3, 0.9, l2=1e-4, nesterov=True)
        if init is not None:      # the draw order of the shared generator differs between the two set-ups
            net.set_params(init)
        net.forward(x)
        for r in ranks:
            net.set_output_grad(r, dy[:, :, r * h:(r + 1) * h])
        net.backward()
        net.sync()
        first = net.param_grads(ranks[0]).copy()
        net.sgd_step()
        net.step_resident(True)
        for _ in range(3):
            net.step_graph(True) if graph else net.step_resident(True)
        net.step_resident(True)
        net.sync()
        assert net.status() == 0
        return net.params(ranks[0]), first

    net = hostlib.Net(ctx, "stem_stage1", Hh, W, Cc, N, seed=29)
    start = net.params(rank).copy()
    mine, first = train(net, [rank], True)
    assert net.graph_launches() > 100, "the step was not captured"
    got = torch.from_numpy(mine).cuda()
    ref = got.clone()
    dist.broadcast(ref, 0)
    assert torch.equal(got, ref), "replicas diverged"
    if bf16:
        eager, _ = train(hostlib.Net(ctx, "stem_stage1", Hh, W, Cc, N, seed=29), [rank], False, init=start)
        assert np.array_equal(mine, eager), float(np.abs(mine - eager).max())
    if rank == 0:
        local_ctx = hostlib.Context([local] * world, mode, arena_mb=512)
        want, first_w = train(hostlib.Net(local_ctx, "stem_stage1", Hh, W, Cc, N, seed=29), list(range(world)), False, init=start)
        if bf16:
            assert H.max_rel(first, first_w) < 2e-2, H.max_rel(first, first_w)
        else:
            assert np.array_equal(mine, want), float(np.abs(mine - want).max())
    dist.barrier()


def classifier_part(ctx, rank, world):
    """The spatially parallel classifier between processes: strips all-gathered with peer loads ordered by flag
    words, the head replicated per rank, the feature gradient reduce-scattered the same way."""
    from tests.oracle_nets import ParallelResNet18
    N, Cc, Hh, W, classes = 2, 3, 64 * world, 64, 10
    net = hostlib.Net(ctx, "parallel_resnet18", Hh, W, Cc, N, filters=classes, seed=23)
    man = net.manifest()
    flat = net.params(rank)
    rng = np.random.default_rng(9)
    for name, (off, size) in man.items():      # wide-margin BN affine: every ReLU passes everything
        if name.endswith(".scale"):
            flat[off:off + size] = rng.uniform(0.05, 0.15, size)
        if name.endswith(".shift"):
            flat[off:off + size] = rng.uniform(1.0, 1.4, size)
        if name.endswith(".bias"):
            flat[off:off + size] = rng.uniform(-0.5, 0.5, size)
    net.set_params(flat)
    shapes = {"conv1.kernel": (64, 3, 7, 7), "fc1.kernel": (classes, 512, 1, 1)}
    cin = 64
    for b, proj in ParallelResNet18.BLOCKS:
        f = {"2": 64, "3": 128, "4": 256, "5": 512, "6": 512}[b[3]]
        shapes[b + ".conv1.kernel"], shapes[b + ".conv2.kernel"] = (f, cin, 3, 3), (f, f, 3, 3)
        if proj:
            shapes[b + ".proj.kernel"] = (f, cin, 1, 1)
        cin = f
    P = {k: flat[o:o + n].reshape(shapes[k]) if k in shapes else flat[o:o + n] for k, (o, n) in man.items()}
    x = H.uniform(600, (N, Cc, Hh, W), 0.0, 1.0)
    labels = np.array([1, classes - 1], np.uint32)
    net.set_labels(rank, labels.reshape(N, 1, 1))
    ref = ParallelResNet18(P, world)
    logits_w, loss_w = ref.forward(x, labels)
    dist.barrier()      # the CPU oracle above takes seconds and not the same on every rank; the device waits are bounded at 2 s
    net.forward(x)
    assert H.max_rel(net.output(rank).reshape(N, classes), logits_w) < 5e-5, "gathered logits mismatch"
    s, px = net.loss()
    assert abs(s / px - loss_w) < 1e-5 * max(1.0, abs(loss_w))
    G = ref.backward()
    dist.barrier()
    net.backward()
    net.sync()
    assert net.status() == 0
    g = torch.from_numpy(net.param_grads(rank)).cuda()
    dist.all_reduce(g)
    g = g.cpu().numpy()
    for name, (off, size) in man.items():
        a, b = g[off:off + size], G[name].reshape(-1)
        # fp32 sums in a different order through 18 layers with batch statistics over 2 images: a few 1e-3 of the
        # largest entry (2.2e-3 seen at 4 strips)
        assert float(np.abs(a - b).max()) <= 5e-3 * float(np.abs(b).max()) + 1e-6, (name, H.max_rel(a, b))
    dist.barrier()


def hybrid_part(rank, world, local):
    """Data-parallel replicas of 2-strip spatial groups (world 4 = 2 x 2): the built-in gradient exchange spans
    all processes; after a few SGD steps on different data per group the parameters equal those of the same run
    with the gradients summed by NCCL (up to the summation order)."""
    Sg = 2
    D, srank, group = world // Sg, rank % Sg, rank // Sg
    N, Cc, Hh, W, classes = 2, 3, 128, 64, 10
    x = H.uniform(900 + group, (N, Cc, Hh, W), 0.0, 1.0)
    labels = np.array([group, classes - 1 - group], np.uint32).reshape(N, 1, 1)
    results = []
    for use_nccl in (False, True):
        Lh = hostlib.load()
        ctxh = Lh.adh_context_create_distributed(srank, Sg, local, hostlib.F32_NCHW, 1024)
        hb = C.create_string_buffer(64)
        assert Lh.adh_context_arena_handle(ctxh, hb) == 0
        mine = torch.from_numpy(np.frombuffer(hb.raw, dtype=np.uint8).copy()).cuda()
        allh = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allh, mine)
        handle = lambda r: bytes(allh[r].cpu().numpy().tobytes())
        for q in range(Sg):
            if q != srank:
                assert Lh.adh_context_set_peer_handle(ctxh, q, handle(group * Sg + q)) == 0
        if use_nccl:
            HOOK = C.CFUNCTYPE(None, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p)

            def allreduce(buf, count, stream, user):
                t = torch.as_tensor(_Raw(buf, count * 4), device="cuda").view(torch.float32)
                with torch.cuda.stream(torch.cuda.ExternalStream(stream)):
                    dist.all_reduce(t)

            hook = HOOK(allreduce)
            _keep.append(hook)
            Lh.adh_context_set_allreduce_hook(ctxh, C.cast(hook, C.c_void_p), None)
        else:
            assert Lh.adh_context_set_world(ctxh, rank, world) == 0
            for wr in range(world):
                if wr == rank:
                    continue
                if wr // Sg == group:
                    assert Lh.adh_context_set_world_peer_from_group(ctxh, wr, wr % Sg) == 0
                else:
                    assert Lh.adh_context_set_world_peer_handle(ctxh, wr, handle(wr)) == 0

        class Ctx:
            pass
        ctx = Ctx()
        ctx.L, ctx.h, ctx.num_ranks = Lh, ctxh, Sg
        net = hostlib.Net(ctx, "parallel_resnet18", Hh, W, Cc, N, filters=classes, seed=37)
        net.configure_sgd(1e-2, 0.9, l2=1e-4, nesterov=True)
        net.set_loss_weight(1.0 / (N * D * Sg))
        start = torch.from_numpy(net.params(srank)).cuda()
        dist.broadcast(start, 0)                      # every replica starts from rank 0's draw
        net.set_params(start.cpu().numpy())
        net.set_labels(srank, labels)
        net.forward(x)
        net.backward()
        net.sgd_step()
        for _ in range(3):
            net.step_graph(True)                      # replays a graph without the hook, runs eagerly with it
        net.sync()
        assert net.status() == 0
        if not use_nccl:
            assert net.graph_launches() > 100, "the step was not captured"
        p = torch.from_numpy(net.params(srank)).cuda()
        ref = p.clone()
        dist.broadcast(ref, 0)
        assert torch.equal(p, ref), "replicas diverged"
        results.append(p.cpu().numpy())
        dist.barrier()
    assert H.max_rel(results[0], results[1]) < 1e-4, H.max_rel(results[0], results[1])


def dp_part(rank, world, local):
    """Pure data parallelism, one unpartitioned replica per process (the reference's multi-process optimizer,
    include/arraydiff/optimize_mpi.hh): worker 0's parameters are broadcast over the built-in exchange (bit for bit),
    every worker trains on its own data, gradients are summed over all workers; replicas stay identical and match the
    same run with the gradients summed by NCCL."""
    N, Cc, Hh, W = 1, 3, 64, 64
    x = H.uniform(1000 + rank, (N, Cc, Hh, W), 0.0, 1.0)
    results, firsts = [], []
    for use_nccl in (False, True):
        Lh = hostlib.load()
        ctxh = Lh.adh_context_create_distributed(0, 1, local, hostlib.F32_NCHW, 512)
        hb = C.create_string_buffer(64)
        assert Lh.adh_context_arena_handle(ctxh, hb) == 0
        mine = torch.from_numpy(np.frombuffer(hb.raw, dtype=np.uint8).copy()).cuda()
        allh = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allh, mine)
        assert Lh.adh_context_set_world(ctxh, rank, world) == 0
        for wr in range(world):
            if wr != rank:
                assert Lh.adh_context_set_world_peer_handle(ctxh, wr, bytes(allh[wr].cpu().numpy().tobytes())) == 0

        class Ctx:
            pass
        ctx = Ctx()
        ctx.L, ctx.h, ctx.num_ranks = Lh, ctxh, 1
        net = hostlib.Net(ctx, "stem_stage1", Hh, W, Cc, N, seed=50 + rank)      # every worker draws its own start
        net.configure_sgd(1e-3, 0.9, l2=1e-4, nesterov=True)
        own = torch.from_numpy(net.params(0)).cuda()
        root = own.clone()
        dist.broadcast(root, 0)
        assert rank == 0 or not torch.equal(own, root)
        net.broadcast_params()                        # built-in exchange: the others add zeros to worker 0's values
        assert torch.equal(torch.from_numpy(net.params(0)).cuda(), root), "broadcast is not bit-exact"
        if use_nccl:
            HOOK = C.CFUNCTYPE(None, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p)

            def allreduce(buf, count, stream, user):
                t = torch.as_tensor(_Raw(buf, count * 4), device="cuda").view(torch.float32)
                with torch.cuda.stream(torch.cuda.ExternalStream(stream)):
                    dist.all_reduce(t)

            hook = HOOK(allreduce)
            _keep.append(hook)
            Lh.adh_context_set_allreduce_hook(ctxh, C.cast(hook, C.c_void_p), None)
        dy = H.normal(1100 + rank, net.strip_shape)
        for it in range(3):
            net.forward(x)
            net.set_output_grad(0, dy)
            net.backward()
            net.sgd_step()
            if it == 0:
                net.sync()
                firsts.append(net.params(0).copy())
        net.sync()
        assert net.status() == 0
        p = torch.from_numpy(net.params(0)).cuda()
        ref = p.clone()
        dist.broadcast(ref, 0)
        assert torch.equal(p, ref), "replicas diverged"
        assert not torch.equal(p, root), "nothing was learnt"
        results.append(p.cpu().numpy())
        dist.barrier()
    # the two exchanges add the workers' gradients in different orders: one step differs by fp32 rounding; through
    # batch statistics over one image the following steps amplify that (7e-4 seen after three steps of 4 workers)
    assert H.max_rel(firsts[0], firsts[1]) < 1e-5, H.max_rel(firsts[0], firsts[1])
    assert H.max_rel(results[0], results[1]) < 1e-2, H.max_rel(results[0], results[1])


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if os.environ.get("AD_MULTI_PART") == "dp":
        dp_part(rank, world, local)
        if rank == 0:
            print("DP_OK", world)
        dist.destroy_process_group()
        return
    if os.environ.get("AD_MULTI_PART") == "hybrid":
        hybrid_part(rank, world, local)
        if rank == 0:
            print("HYBRID_OK", world)
        dist.destroy_process_group()
        return
    halo_part(rank, world)
    host_part(rank, world, local)
    if rank == 0:
        print("MULTI_OK", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
