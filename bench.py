"""Benchmark of the spatially parallel convolution path.

    python bench.py --gpus 1 --steps 20 --warmup 5                  # this library
    python bench.py --impl reference --gpus 1 --steps 3 --warmup 1  # the CPU path on the host cores
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W      # one rank per GPU

Workload (`config.workload` = "microbench_spatial_conv"): the shape the reference fixes for its
own measurement of this path -- 3x3 convolution, dilation 3, halo 3, batch 32, 64 -> 64 channels,
512 x 512 pixels, the H axis cut into one strip per GPU (tools/microbench_spatial_conv.cc:25-41,
:101-107).  One step = halo exchange + forward conv + data gradient + filter gradient +
halo-gradient accumulate-back + filter-gradient allreduce.  The total work is fixed as GPUs are
added ("strong" scaling).  bf16 operands, fp32 accumulate; synthetic seeded inputs.

metric  = spatial conv fwd+bwd TFLOP/s, FLOPs = 3 x 2*N*K*C*9*P*Q counted on the unpartitioned
          output (halo recompute and padding are not credited).
value   = with inputs resident in HBM;  e2e = same step fed from pinned host buffers through the
          C ABI, with the host->device copies of x and dy and the device->host read of dw timed.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BATCH, CH, SIZE, KS, DIL, PAD = 32, 64, 512, 3, 3, 3
METRIC, UNIT = "spatial_conv_fwd_bwd_tflops", "TFLOP/s"


def flops_per_pass(n=None, rows=SIZE, cols=SIZE):
    return 2.0 * (BATCH if n is None else n) * CH * CH * KS * KS * rows * cols


# DRAM traffic per launch (dram__bytes_read + dram__bytes_write) of the three conv kernels, from the ncu
# capture summarised in profiles/conv_tc_microbench_spatial_conv.md: measured at batch 4 on one GPU; traffic
# grows in proportion to the pixels a launch processes, so it is scaled by batch / 4 / strips.
NCU_TRAFFIC_BATCH4 = {"fprop": 233.7e6, "dgrad": 232.9e6, "wgrad": 276.1e6}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "tf_burst": d["bf16_tflops"], "tf_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tf_burst": 1590.0, "tf_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------- CPU arm
def cpu_conv_sample(target_seconds, threads_omp=True):
    """Times the oracle's conv fwd + dgrad + wgrad on a strip sample of the workload (one image,
    `rows` output rows, full width, dilation 3, halo-padded input) sized for ~target_seconds."""
    from oracle import orc
    from tests import helpers as H

    def run(rows):
        x = H.uniform(1, (1, CH, rows + 2 * PAD, SIZE + 2 * PAD))
        w = H.normal(2, (CH, CH, KS, KS), float(np.sqrt(2.0 / (KS * KS * CH))))
        dy = H.uniform(3, (1, CH, rows, SIZE))
        t0 = time.perf_counter()
        y = orc.conv2d_fprop(x, w, None, dil=(DIL, DIL), omp=threads_omp)
        orc.conv2d_dgrad(dy, w, x.shape, dil=(DIL, DIL), omp=threads_omp)
        orc.conv2d_wgrad(x, dy, w.shape, dil=(DIL, DIL), omp=threads_omp)
        dt = time.perf_counter() - t0
        assert y.shape == (1, CH, rows, SIZE)
        return dt, 3 * flops_per_pass(1, rows, SIZE)

    dt, fl = run(2)                       # calibration
    rows = int(max(2, min(SIZE, 2 * target_seconds / max(dt, 1e-6))))
    dt, fl = run(rows)
    return fl / dt / 1e12, dt, rows, orc.num_threads(threads_omp)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    budget = 120.0 / max(1, args.steps + args.warmup)
    vals, rows, cores, secs = [], 0, 1, 0.0
    for i in range(args.warmup + args.steps):
        v, dt, rows, cores = cpu_conv_sample(min(20.0, budget))
        if i >= args.warmup:
            vals.append(v); secs += dt
    value = float(np.mean(vals))
    sample = f"oracle conv fwd+dgrad+wgrad on a {rows}-row x {SIZE}-col strip of one image per step (of 32 x 512 rows)"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * secs / max(1, args.steps), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "microbench_spatial_conv", "batch": BATCH, "channels": CH, "image": [SIZE, SIZE],
                   "kernel": KS, "dilation": DIL, "halo": PAD, "bounded_sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ----------------------------------------------------------------------------- GPU arm
class Step:
    """Buffers and the per-step call sequence of one rank (one H-strip)."""

    def __init__(self, rank, world):
        import torch
        from arraydiff_cuda_b200 import abi, dist as addist
        self.torch, self.abi = torch, abi
        self.L = abi.load()
        self.rank, self.world = rank, world
        self.h = SIZE // world
        h, Wp, Hp = self.h, SIZE + 2 * PAD, SIZE // world + 2 * PAD
        bf = torch.bfloat16
        xbytes = BATCH * Hp * Wp * CH * 2
        self.arena = addist.SymmetricArena(2 * xbytes + (1 << 20), rank, world)
        self.x, self.x_off = self.arena.alloc((BATCH, Hp, Wp, CH), bf)       # halo-padded input strip
        self.gx, self.gx_off = self.arena.alloc((BATCH, Hp, Wp, CH), bf)     # halo-padded input gradient
        self.flags, self.flags_off = self.arena.alloc((8,), torch.int64)      # 0 from_prev 1 from_next 2 gprev 3 gnext
        self.counter = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.status = torch.zeros(4, dtype=torch.int32, device="cuda")
        g = torch.Generator(device="cuda").manual_seed(1234 + rank)
        self.x.zero_()
        self.x[:, PAD:PAD + h, PAD:PAD + SIZE] = (torch.rand((BATCH, h, SIZE, CH), device="cuda", generator=g) * 2 - 1).to(bf)
        gw = torch.Generator(device="cuda").manual_seed(99)
        self.w = (torch.randn((CH, KS, KS, CH), device="cuda", generator=gw) * float(np.sqrt(2.0 / (KS * KS * CH)))).to(bf)
        self.y = torch.empty((BATCH, h, SIZE, CH), dtype=bf, device="cuda")
        self.dy = (torch.rand((BATCH, h, SIZE, CH), device="cuda", generator=g) * 2 - 1).to(bf)
        self.dw = torch.zeros((CH, KS, KS, CH), device="cuda")
        a = abi.Conv2dArgs()
        a.dtype, a.layout = abi.AD_BF16, abi.AD_NHWC
        a.N, a.C, a.H, a.W, a.K, a.kh, a.kw = BATCH, CH, Hp, Wp, CH, KS, KS
        a.stride_h = a.stride_w = 1
        a.dil_h = a.dil_w = DIL
        nscr = max(self.L.ad_conv2d_scratch_bytes(C.byref(a), 1), self.L.ad_conv2d_scratch_bytes(C.byref(a), 2), 16)
        self.scratch = torch.zeros(nscr, dtype=torch.uint8, device="cuda")
        a.x, a.w, a.scratch, a.scratch_bytes = self.x.data_ptr(), self.w.data_ptr(), self.scratch.data_ptr(), nscr
        self.conv = a
        self.epoch = 0
        self.halo = True       # False: the same step without halo transfers (measures what they cost exposed)
        self.marks = None      # a list: run() brackets every conv call with CUDA events and appends (name, e0, e1)
        ha = abi.HaloArgs()
        ha.dtype, ha.layout = abi.AD_BF16, abi.AD_NHWC
        ha.halo_pad, ha.base_width, ha.base_height, ha.num_channels, ha.batch_size = PAD, SIZE, h, CH, BATCH
        ha.num_ranks, ha.rank_first, ha.rank_count, ha.push = world, rank, 1, 1
        self.hx, self.hg = ha, abi.HaloArgs.from_buffer_copy(ha)
        xp, gp, fp = self.arena.peers(self.x_off), self.arena.peers(self.gx_off), self.arena.peers(self.flags_off)
        for r in range(world):
            self.hx.bufs[r], self.hg.bufs[r] = xp[r], gp[r]
        self.side = torch.cuda.Stream()
        self.plan = addist.HaloPlan(rank, world)
        for peer, slot in self.plan.exchange_signals():
            self.hx.signal_flags[peer] = fp[peer] + 8 * slot
        self.hx.block_counter = self.counter.data_ptr()
        self.fp = fp
        # pinned host copies for the end-to-end variant
        self.hx_host = torch.empty(self.x.shape, dtype=bf).pin_memory()
        self.hx_host.copy_(self.x.cpu())
        self.dy_host = torch.empty(self.dy.shape, dtype=bf).pin_memory()
        self.dy_host.copy_(self.dy.cpu())
        self.dw_host = torch.empty(self.dw.shape, dtype=torch.float32).pin_memory()

    def _s(self):
        return C.c_void_p(self.torch.cuda.current_stream().cuda_stream)

    def _wait(self, slot, epoch):
        self.abi.check(self.L.ad_flag_wait(C.c_void_p(self.flags.data_ptr() + 8 * slot), epoch, 2_000_000_000,
                                           C.c_void_p(self.status.data_ptr()), self._s()), "flag wait")

    def _signal(self, rank, slot, epoch):
        self.abi.check(self.L.ad_flag_signal(C.c_void_p(self.fp[rank] + 8 * slot), epoch, self._s()), "flag signal")

    def _timed(self, name, fn):
        if self.marks is None:
            return fn()
        e0, e1 = self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        self.marks.append((name, e0, e1))

    def run(self, e2e=False):
        L, abi, a, s = self.L, self.abi, self.conv, self._s()
        r, R = self.rank, self.world
        self.epoch += 1
        ep = self.epoch
        if e2e:
            self.x.copy_(self.hx_host, non_blocking=True)
            self.dy.copy_(self.dy_host, non_blocking=True)
        # forward: push my edge rows into the neighbours' halo rows on a side stream and wait there for
        # theirs, while the main stream already convolves the interior rows; the PAD boundary rows at
        # either end follow once the halo has landed
        a.y, a.accumulate = self.y.data_ptr(), 0
        if R > 1 and self.halo:
            main = self.torch.cuda.current_stream()
            self.side.wait_stream(main)
            with self.torch.cuda.stream(self.side):
                s2 = self._s()
                self.hx.epoch = ep
                abi.check(L.ad_halo_exchange(C.byref(self.hx), s2), "halo exchange")
                for slot in self.plan.exchange_waits():
                    self._wait(slot, ep)
                landed = self.side.record_event()
            a.out_row_begin, a.out_row_count = PAD, self.h - 2 * PAD
            self._timed("fprop", lambda: abi.check(L.ad_conv2d_fprop(C.byref(a), s), "fprop interior"))
            main.wait_event(landed)
            for q0 in (0, self.h - PAD):
                a.out_row_begin, a.out_row_count = q0, PAD
                self._timed("fprop", lambda: abi.check(L.ad_conv2d_fprop(C.byref(a), s), "fprop boundary"))
            a.out_row_begin, a.out_row_count = 0, 0
        else:
            self._timed("fprop", lambda: abi.check(L.ad_conv2d_fprop(C.byref(a), s), "fprop"))
        # backward: data gradient over the whole padded strip, filter gradient, halo-gradient accumulate-back
        a.y, a.dx, a.dw = self.dy.data_ptr(), self.gx.data_ptr(), self.dw.data_ptr()
        a.dx_col_begin, a.dx_col_count = PAD, SIZE     # the W-pad columns of the gradient buffer are never read
        self._timed("dgrad", lambda: abi.check(L.ad_conv2d_dgrad(C.byref(a), s), "dgrad"))
        if R > 1 and self.halo:
            # the halo-gradient accumulate-back (signal, wait for the neighbours, pull + add) runs on the
            # side stream underneath the filter gradient
            main = self.torch.cuda.current_stream()
            self.side.wait_stream(main)
            with self.torch.cuda.stream(self.side):
                s2 = self._s()
                for peer, slot in self.plan.reduce_signals():
                    self._signal(peer, slot, ep)
                for slot in self.plan.reduce_waits():
                    self._wait(slot, ep)
                abi.check(L.ad_halo_reduce(C.byref(self.hg), s2), "halo reduce")
        self._timed("wgrad", lambda: abi.check(L.ad_conv2d_wgrad(C.byref(a), s), "wgrad"))
        if R > 1:
            import torch.distributed as dist
            dist.all_reduce(self.dw)       # filter-gradient allreduce over NCCL / NVLink
            self.torch.cuda.current_stream().wait_stream(self.side)
        if e2e:
            self.dw_host.copy_(self.dw, non_blocking=True)

    def check_status(self):
        st = self.status.cpu().tolist() + self.scratch[:4].view(self.torch.int32).cpu().tolist()
        if any(v != 0 for v in st):
            raise RuntimeError(f"device-side bounded wait reported {st}")


def timed_loop(torch, dist, step, steps, e2e, world):
    """Barrier + synchronize on both sides, device time by CUDA events, max over ranks."""
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step.run(e2e=e2e)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    return ms


def step_distribution(torch, dist, step, n, world):
    """n individually timed steps (CUDA events around each, no host synchronisation in between); per step
    the max over ranks; returns (median, p10, p90) in ms."""
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(n + 1)]
    ev[0].record()
    for i in range(n):
        step.run()
        ev[i + 1].record()
    torch.cuda.synchronize()
    t = torch.tensor([ev[i].elapsed_time(ev[i + 1]) for i in range(n)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    v = np.sort(t.cpu().numpy())
    return float(np.median(v)), float(v[int(0.1 * (n - 1))]), float(v[int(round(0.9 * (n - 1)))])


def kernel_times_in_step(torch, dist, step, steps, world):
    """Average device time per step of each conv pass, from CUDA events around its launches inside `steps` full
    steps run back to back (the conditions of the timed region: warm clocks, halo traffic alongside)."""
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    step.marks = []
    for _ in range(steps):
        step.run()
    torch.cuda.synchronize()
    marks, step.marks = step.marks, None
    tot = {}
    for name, e0, e1 in marks:
        tot[name] = tot.get(name, 0.0) + e0.elapsed_time(e1)
    return {k: v / steps * 1e-3 for k, v in tot.items()}


def kernel_times(torch, step, iters=10):
    """Per-kernel device time (CUDA events on the launching stream), each launch after an L2 flush."""
    L, abi, a = step.L, step.abi, step.conv
    s = step._s()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def t(fn):
        fn(); torch.cuda.synchronize()
        out = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record(); torch.cuda.synchronize()
            out.append(e0.elapsed_time(e1))
        return float(np.mean(out)) * 1e-3

    def fprop():
        a.y = step.y.data_ptr(); abi.check(L.ad_conv2d_fprop(C.byref(a), s))

    def dgrad():
        a.y, a.dx = step.dy.data_ptr(), step.gx.data_ptr()
        a.dx_col_begin, a.dx_col_count = PAD, SIZE
        abi.check(L.ad_conv2d_dgrad(C.byref(a), s))

    def wgrad():
        a.y, a.dw = step.dy.data_ptr(), step.dw.data_ptr(); abi.check(L.ad_conv2d_wgrad(C.byref(a), s))

    return {"fprop": t(fprop), "dgrad": t(dgrad), "wgrad": t(wgrad)}


# ----------------------------------------------------------------------------- halo microbenchmark
def run_halo_workload(args):
    """`--workload halo`: benchmark config 2 -- NCHW tensors N=8, C=256, 224x224 cut into H-strips, halo
    1 and 3, fp32 and bf16; forward exchange and backward accumulate.  On one GPU the R strips share the
    device and move in ONE launch (HBM-bound: payload read + written); on N GPUs each rank pushes to /
    pulls from its neighbours over NVLink, with NCCL send/recv of packed faces timed beside it."""
    import torch
    import torch.distributed as dist
    from arraydiff_cuda_b200 import abi, dist as addist
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    L = abi.load()
    N, Cc, Hh, W = 8, 256, 224, 224
    cases = []
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def timed(fn, iters):
        for _ in range(max(3, args.warmup)):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms * 1e-3

    launches0 = L.ad_launch_count()
    for R in ([world] if world > 1 else [2, 4, 8]):
        h = Hh // R
        for dt, tdt, es in ((abi.AD_F32, torch.float32, 4), (abi.AD_BF16, torch.bfloat16, 2)):
            for p in (1, 3):
                shape = (N, Cc, h + 2 * p, W + 2 * p)
                payload = 2 * (R - 1) * N * Cc * p * W * es
                a = abi.HaloArgs()
                a.dtype, a.layout = dt, abi.AD_NCHW
                a.halo_pad, a.base_width, a.base_height, a.num_channels, a.batch_size = p, W, h, Cc, N
                a.num_ranks = R
                rec = {"strips": R, "halo": p, "dtype": "f32" if es == 4 else "bf16", "payload_bytes": payload}
                if world == 1:
                    bufs = [torch.randn(shape, device="cuda").to(tdt) for _ in range(R)]
                    a.rank_first, a.rank_count, a.push = 0, R, 1
                    for r in range(R):
                        a.bufs[r] = bufs[r].data_ptr()
                    te = timed(lambda: abi.check(L.ad_halo_exchange(C.byref(a), s)), args.steps)
                    tr = timed(lambda: abi.check(L.ad_halo_reduce(C.byref(a), s)), args.steps)
                else:
                    arena = addist.SymmetricArena(int(np.prod(shape)) * es + (1 << 20), rank, world)
                    buf, off = arena.alloc(shape, tdt)
                    flags, foff = arena.alloc((8,), torch.int64)
                    buf.copy_(torch.randn(shape, device="cuda").to(tdt))
                    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
                    status = torch.zeros(1, dtype=torch.int32, device="cuda")
                    plan = addist.HaloPlan(rank, world)
                    a.rank_first, a.rank_count, a.push = rank, 1, 1
                    peers, fp = arena.peers(off), arena.peers(foff)
                    for r in range(R):
                        a.bufs[r] = peers[r]
                    for peer, slot in plan.exchange_signals():
                        a.signal_flags[peer] = fp[peer] + 8 * slot
                    a.block_counter = counter.data_ptr()
                    ep = [0]

                    def exch():
                        ep[0] += 1
                        a.epoch = ep[0]
                        abi.check(L.ad_halo_exchange(C.byref(a), s))
                        for slot in plan.exchange_waits():
                            abi.check(L.ad_flag_wait(C.c_void_p(flags.data_ptr() + 8 * slot), ep[0], 2_000_000_000,
                                                     C.c_void_p(status.data_ptr()), s))

                    def red():
                        ep[0] += 1
                        for peer, slot in plan.reduce_signals():
                            abi.check(L.ad_flag_signal(C.c_void_p(fp[peer] + 8 * slot), ep[0], s))
                        for slot in plan.reduce_waits():
                            abi.check(L.ad_flag_wait(C.c_void_p(flags.data_ptr() + 8 * slot), ep[0], 2_000_000_000,
                                                     C.c_void_p(status.data_ptr()), s))
                        abi.check(L.ad_halo_reduce(C.byref(a), s))

                    def nccl():
                        ops, recvs = [], []
                        for peer, src, dst in plan.push_rows(p, h):
                            send = buf[:, :, src:src + p, p:p + W].contiguous()
                            recv = torch.empty_like(send)
                            mine = [d for (q, _, d) in addist.HaloPlan(peer, world).push_rows(p, h) if q == rank][0]
                            ops += [dist.P2POp(dist.isend, send, peer), dist.P2POp(dist.irecv, recv, peer)]
                            recvs.append((recv, mine))
                        for w_ in dist.batch_isend_irecv(ops):
                            w_.wait()
                        for recv, dst in recvs:
                            buf[:, :, dst:dst + p, p:p + W] = recv

                    te, tr, tn = timed(exch, args.steps), timed(red, args.steps), timed(nccl, args.steps)
                    if int(status.item()) != 0:
                        raise RuntimeError("bounded flag wait timed out")
                    rec["nccl_sendrecv_us"] = tn * 1e6
                    rec["nccl_sendrecv_gbs"] = payload / tn / 1e9
                    dist.barrier()
                    arena.close()
                rec.update(exchange_us=te * 1e6, exchange_gbs=payload / te / 1e9, reduce_us=tr * 1e6, reduce_gbs=payload / tr / 1e9)
                cases.append(rec)
    if rank == 0:
        peaks = measured_peaks()
        top = max(cases, key=lambda c: c["payload_bytes"])
        # one GPU: every payload byte is read and written locally; N GPUs: bytes into the busiest GPU over NVLink
        if world == 1:
            achieved, peak, bound = 2 * top["payload_bytes"] / (top["exchange_us"] * 1e-6) / 1e9, peaks["hbm_gbs"], "hbm"
        else:
            per_gpu = top["payload_bytes"] / (world - 1)      # two faces land in an interior rank
            achieved, peak, bound = per_gpu / (top["exchange_us"] * 1e-6) / 1e9, 770.0, "nvlink"
        print(json.dumps({
            "metric": "halo_exchange_gbs", "value": top["exchange_gbs"], "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": top["exchange_us"] / 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "halo_microbench", "tensor": [N, Cc, Hh, W], "layout": "NCHW",
                       "l2": "same buffers every iteration (payload smaller than L2; launch-latency dominated below ~10 MiB)"},
            "gpu_launches": int(L.ad_launch_count() - launches0),
            "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None},
            "cases": cases,
        }))
    if world > 1:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------- config 3 through the C++ op graph
def segnet_flops(N, Hh, W, classes=19, blocks=(3, 4, 6, 3), base=64):
    """fwd + dgrad + wgrad FLOPs of the dilated ResNet-50 segmentation net (2*N*K*C*kh*kw*P*Q per pass on the
    unpartitioned output, stem data gradient excluded)."""
    total = 2.0 * N * base * 3 * 49 * (Hh // 2) * (W // 2) * 2          # stem: fprop + wgrad
    px, cin = N * (Hh // 4) * (W // 4), base
    for st in range(4):
        mid, out = base << st, (base << st) * 4
        for i in range(blocks[st]):
            px_out = px // 4 if (st == 1 and i == 0) else px
            f = 2.0 * px * mid * cin                                     # conv1 1x1
            f += 2.0 * px_out * mid * mid * 9                            # conv2 3x3 (carries the stride)
            f += 2.0 * px_out * out * mid                                # conv3 1x1
            if i == 0:
                f += 2.0 * px_out * out * cin                            # projection
            total += 3.0 * f
            px, cin = px_out, out
    total += 3.0 * 2.0 * px * classes * cin
    return total


def resnet50_flops(N, Hh, W, classes=1000):
    """fwd + dgrad + wgrad FLOPs of the ResNet-50 classifier (stem data gradient excluded)."""
    total = 2.0 * N * 64 * 3 * 49 * (Hh // 2) * (W // 2) * 2
    px, cin = N * (Hh // 4) * (W // 4), 64
    for st, nb in enumerate((3, 4, 6, 3)):
        mid, out = 64 << st, (64 << st) * 4
        for i in range(nb):
            px_out = px // 4 if (st > 0 and i == 0) else px
            f = 2.0 * px * mid * cin + 2.0 * px_out * mid * mid * 9 + 2.0 * px_out * out * mid
            if i == 0:
                f += 2.0 * px_out * out * cin
            total += 3.0 * f
            px, cin = px_out, out
    return total + 3.0 * 2.0 * N * classes * cin


def run_net_workload(args, kind):
    """`--workload stem_stage1`: benchmark config 3 -- ResNet-50 stem + stage 1 on one 3x1024x1024 image,
    H-partitioned over the GPUs (or over `--strips` ranks sharing one GPU), bf16 operands, forward +
    backward against an upstream gradient N(0,1), filter-gradient allreduce and SGD update, all through
    the C++ host layer (zoo builder -> op graph -> C ABI kernels).  93.6 GFLOP per step (stem dgrad excluded).
    `--workload segnet`: benchmark config 4 -- dilated ResNet-50 at output stride 8 on 2x3x1024x2048 with a
    19-class head, x8 bilinear upsample and per-pixel softmax NLL against uniform random labels.
    `--workload resnet50_hybrid`: benchmark config 5 -- ResNet-50 classifier on 224 x 224, global batch 256, the
    GPUs in data-parallel groups of 2 H-strips each (8 GPUs: 4 data x 2 spatial; halos and the all-gather by peer
    loads inside a group, filter gradients summed over all GPUs with NCCL).  On one GPU: one group (batch 64) as
    2 strips sharing the device."""
    import torch
    import torch.distributed as dist
    from arraydiff_cuda_b200 import abi, hostlib
    from arraydiff_cuda_b200.dist import _Raw
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    seg, hyb = kind == "segnet", kind == "resnet50_hybrid"
    S = 224 if hyb and args.image == 1024 else args.image
    Hh, Ww, NB = (S, 2 * S, 2) if seg else (S, S, 1)
    Sg = 2 if hyb else world                 # ranks per spatial group
    if hyb and world > 1 and world % Sg:
        raise SystemExit("resnet50_hybrid needs an even number of GPUs")
    D = max(1, world // Sg) if hyb else 1    # data-parallel groups
    srank, group = (rank % Sg, rank // Sg) if hyb else (rank, 0)
    if hyb:
        NB = 256 // (D if world > 1 else 4)
    L = abi.load()
    Lh = hostlib.load()
    keep = []
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        h = Lh.adh_context_create_distributed(srank, Sg, local, hostlib.BF16_NHWC,
                                              24576 if hyb else (40960 // world + 2048) if seg else 4096)
        hb = C.create_string_buffer(64)
        assert Lh.adh_context_arena_handle(h, hb) == 0
        mine = torch.from_numpy(np.frombuffer(hb.raw, dtype=np.uint8).copy()).cuda()
        allh = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allh, mine)
        for q in range(Sg):                   # the peers of my spatial group
            wr = group * Sg + q
            if q != srank:
                assert Lh.adh_context_set_peer_handle(h, q, bytes(allh[wr].cpu().numpy().tobytes())) == 0
        HOOK = C.CFUNCTYPE(None, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p)

        def allreduce(buf, count, stream, user):
            t = torch.as_tensor(_Raw(buf, count * 4), device="cuda").view(torch.float32)
            with torch.cuda.stream(torch.cuda.ExternalStream(stream)):
                dist.all_reduce(t)

        if hyb and D > 1 and not args.nccl_allreduce:
            # several data groups: the built-in gradient exchange spans all processes (same net, same arena offsets)
            assert Lh.adh_context_set_world(h, rank, world) == 0
            for wr in range(world):
                if wr == rank:
                    continue
                if wr // Sg == group:
                    assert Lh.adh_context_set_world_peer_from_group(h, wr, wr % Sg) == 0
                else:
                    assert Lh.adh_context_set_world_peer_handle(h, wr, bytes(allh[wr].cpu().numpy().tobytes())) == 0
        if args.nccl_allreduce:
            # filter gradients over NCCL (torch.distributed) instead of the built-in peer exchange; such a
            # step is launched eagerly
            hook = HOOK(allreduce)
            keep.append(hook)
            Lh.adh_context_set_allreduce_hook(h, C.cast(hook, C.c_void_p), None)

        class Ctx:
            pass
        ctx = Ctx()
        ctx.L, ctx.h, ctx.num_ranks = Lh, h, Sg
        ranks, strips = [srank], Sg
    else:
        strips = max(2 if hyb else 1, args.strips)
        ctx = hostlib.Context([local] * strips, hostlib.BF16_NHWC,
                              arena_mb=24576 if hyb else max(512, int((40960 if seg else 4096) * (S / 1024.0) ** 2) // strips + 256))
        ranks = list(range(strips))
    net = hostlib.Net(ctx, "segnet50" if seg else "parallel_resnet50" if hyb else "stem_stage1", Hh, Ww, 3, NB,
                      filters=1000 if hyb else 64, seed=1)
    net.configure_sgd(0.01, 0.9, l2=1e-4, nesterov=True)
    if hyb:
        net.set_loss_weight(1.0 / (NB * D * strips))     # mean over the global batch, shared out over a group's replicas of the head
    rng = np.random.default_rng(7 + group)
    x = rng.uniform(0, 1, (NB, 3, Hh, Ww)).astype(np.float32)
    if seg:
        labels = rng.integers(0, 19, (NB, Hh, Ww)).astype(np.uint32)
        hs = Hh // strips
        dy = []
    elif hyb:
        labels = rng.integers(0, 1000, (NB, 1, 1)).astype(np.uint32)
        dy = []
    else:
        dy = [rng.standard_normal(net.strip_shape).astype(np.float32) for _ in range(strips)]

    # the end-to-end step moves its tensors between PINNED host buffers and the device
    def pinned(a):
        return torch.from_numpy(a).pin_memory().numpy()
    x = pinned(x)
    dy = [pinned(d) for d in dy]
    if seg or hyb:
        labels = pinned(labels)
    out_host = pinned(np.empty(net.strip_shape, np.float32))

    def e2e_step():
        net.forward(x)                       # host image -> every local rank (H2D inside)
        for r in ranks:
            if seg:
                net.set_labels(r, labels[:, r * hs:(r + 1) * hs])   # host labels -> device
            elif hyb:
                net.set_labels(r, labels)
            else:
                net.set_output_grad(r, dy[r])    # host upstream gradient -> device
        net.backward()
        net.sgd_step()
        return net.loss() if (seg or hyb) else net.output(ranks[0], out=out_host)          # D2H read of a result

    # steady-state step: the resident step replayed from a CUDA graph (flag values between processes are
    # relative to a device-resident base, the gradient allreduce is the built-in peer exchange)
    use_graph = not args.no_graph and not (world > 1 and args.nccl_allreduce)
    step = (lambda: net.step_graph(True)) if use_graph else (lambda: net.step_resident(True))
    e2e_step()
    net.step_resident(True)
    for _ in range(max(3, args.warmup)):
        step()
    net.sync()
    assert net.status() == 0, "a bounded device wait timed out"
    streams = [torch.cuda.ExternalStream(Lh.adh_context_stream(ctx.h, r)) for r in ranks]
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = L.ad_launch_count()
    e0 = torch.cuda.Event(enable_timing=True)
    e0.record(streams[0])
    for _ in range(args.steps):
        step()
    ends = []
    for st in streams:
        e = torch.cuda.Event(enable_timing=True)
        e.record(st)
        ends.append(e)
    torch.cuda.synchronize()
    ms = max(e0.elapsed_time(e) for e in ends)
    launches = net.graph_launches() * args.steps if use_graph else L.ad_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    assert net.status() == 0
    k_e2e = max(3, args.steps // 4)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(k_e2e):
        e2e_step()
    net.sync()
    t_e2e = (time.perf_counter() - t0) / k_e2e
    if world > 1:
        t = torch.tensor([t_e2e], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_e2e = float(t.item())
    scale = (S / 1024.0) ** 2
    flops = segnet_flops(NB, Hh, Ww) if seg else resnet50_flops(NB * D, Hh, Ww) if hyb else 93.6e9 * scale
    if rank == 0:
        step_s = ms / args.steps * 1e-3
        print(json.dumps({
            "metric": METRIC, "value": flops / step_s / 1e12, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "images_per_s": NB * D / step_s,
            "config": {"workload": "resnet50_dilated_segnet" if seg else f"resnet50_hybrid_{D}x{strips}" if hyb else "resnet50_stem_stage1",
                       "image": [NB * D, 3, Hh, Ww], "strips": strips, "data_groups": D, "layout": "NHWC",
                       "bn_statistics": "per strip (as the reference)", "update": "allreduce (%s) + Nesterov SGD" % ("nccl" if world > 1 and args.nccl_allreduce else "peer loads" if strips > 1 or D > 1 else "single rank"), "launch": "cuda graph" if use_graph else "eager",
                       "l2": "activations of one step total more than 1 GB, larger than L2", "parallelism": f"data{D}-spatial-h{strips}" if hyb else f"spatial-h{strips}"},
            "e2e": {"value": flops / t_e2e / 1e12, "unit": UNIT, "h2d_bytes_per_step": int(x.nbytes // (Sg if world > 1 else 1) + (labels.nbytes if hyb else labels.nbytes // world if seg else sum(d.nbytes for d in dy))),
                    "d2h_bytes_per_step": int(NB * 4 if hyb else np.prod(net.strip_shape[2:]) * NB * 4 if seg else np.prod(net.strip_shape) * 4), "steps": k_e2e, "timing": "host clock between synchronisations"},
            "gpu_launches": int(launches), "clocks": clocks,
        }))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    global BATCH
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--workload", default="conv", choices=["conv", "halo", "stem_stage1", "segnet", "resnet50_hybrid"],
                    help="conv: the headline spatial conv step; halo: the halo-exchange microbenchmark (config 2); "
                         "stem_stage1: ResNet-50 stem + stage 1 through the C++ op graph (config 3); "
                         "segnet: dilated ResNet-50 segmentation net, 2x3x1024x2048 (config 4; --image = height); "
                         "resnet50_hybrid: ResNet-50 classifier, 224 x 224, batch 256, data-parallel groups of 2 strips (config 5)")
    ap.add_argument("--strips", type=int, default=1, help="stem_stage1 on one GPU: ranks sharing the device")
    ap.add_argument("--image", type=int, default=1024, help="stem_stage1: image height = width")
    ap.add_argument("--nccl-allreduce", action="store_true",
                    help="stem_stage1 / segnet on several GPUs: sum the filter gradients with NCCL instead of the built-in peer exchange")
    ap.add_argument("--no-graph", action="store_true", help="stem_stage1: launch every kernel eagerly instead of replaying a CUDA graph")
    ap.add_argument("--batch", type=int, default=BATCH,
                    help="images per step; the default is the workload's, smaller values are for profiler captures")
    args = ap.parse_args()
    BATCH = args.batch
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.workload == "halo":
        run_halo_workload(args)
        return
    if args.workload in ("stem_stage1", "segnet", "resnet50_hybrid"):
        run_net_workload(args, args.workload)
        return

    import torch
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    if SIZE % world:
        raise SystemExit("image height must divide by the number of GPUs")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from arraydiff_cuda_b200 import abi
    L = abi.load()   # raises if the CUDA library is missing: no fallback
    step = Step(rank, world)
    for _ in range(args.warmup):
        step.run()
    torch.cuda.synchronize()
    step.check_status()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = L.ad_launch_count()
    ms = timed_loop(torch, dist, step, args.steps, False, world)
    launches = L.ad_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    step.check_status()
    for _ in range(2):
        step.run(e2e=True)
    e2e_steps = max(3, args.steps // 4)
    ms_e2e = timed_loop(torch, dist, step, e2e_steps, True, world)
    step.check_status()

    med, p10, p90 = step_distribution(torch, dist, step, max(100, args.steps), world)
    ms_nohalo = None
    if world > 1:
        step.halo = False
        for _ in range(3):
            step.run()
        ms_nohalo = timed_loop(torch, dist, step, args.steps, False, world)
        step.halo = True
    kt_step = kernel_times_in_step(torch, dist, step, args.steps, world)
    step.check_status()

    total_flops = 3 * flops_per_pass()
    value = total_flops / (ms / args.steps * 1e-3) / 1e12
    e2e_value = total_flops / (ms_e2e / e2e_steps * 1e-3) / 1e12
    if rank == 0:
        peaks = measured_peaks()
        kt = kernel_times(torch, step)
        top = max(kt_step, key=kt_step.get)
        per_launch_flops = flops_per_pass(BATCH, step.h, SIZE)
        achieved = per_launch_flops / kt_step[top] / 1e12
        cpu = None
        if world == 1:
            v, dt, rows, cores = cpu_conv_sample(args.cpu_seconds)
            cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                   "sample": f"oracle conv fwd+dgrad+wgrad on a {rows}-row x {SIZE}-col strip of one image ({dt:.1f} s)"}
        hbytes = step.hx_host.numel() * 2 + step.dy_host.numel() * 2
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "microbench_spatial_conv", "batch": BATCH, "channels": CH, "image": [SIZE, SIZE],
                       "kernel": KS, "dilation": DIL, "halo": PAD, "strips": world, "layout": "NHWC",
                       "l2": "inputs larger than L2 (%.2f GB activations per pass)" % (BATCH * SIZE * SIZE * CH * 2 / 1e9), "parallelism": f"spatial-h{world}"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": hbytes,
                    "d2h_bytes_per_step": step.dw_host.numel() * 4, "steps": e2e_steps},
            "gpu_launches": int(launches),
            "step_ms": {"median": med, "p10": p10, "p90": p90, "samples": max(100, args.steps)},
            "halo_exposed_ms": None if ms_nohalo is None else ms / args.steps - ms_nohalo / args.steps,
            "roofline": {"bound": "tensor", "kernel": f"conv_tc_{top}", "achieved": achieved, "peak": peaks["tf_sustained"],
                         "unit": "TFLOP/s", "frac": achieved / peaks["tf_sustained"],
                         "traffic": NCU_TRAFFIC_BATCH4[top] * BATCH / 4 / world,
                         "peak_source": peaks["source"] + " (sustained: the kernel is timed with CUDA events inside full steps run back to back)",
                         "kernels_us": {k: v * 1e6 for k, v in kt_step.items()},
                         "kernels_alone_us": {k: v * 1e6 for k, v in kt.items()},
                         "frac_alone_of_burst": per_launch_flops / kt[top] / 1e12 / peaks["tf_burst"]},
            "clocks": clocks,
        }
        if cpu:
            line["cpu_baseline"] = cpu
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
