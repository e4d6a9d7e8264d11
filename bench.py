"""Benchmark of the spatially parallel convolution path.

    python bench.py --gpus 1 --steps 20 --warmup 5                  # this library
    python bench.py --impl reference --gpus 1 --steps 3 --warmup 1  # the CPU path on the host cores
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W      # one rank per GPU

Headline workload (`config.workload` = "resnet50_dilated_segnet"): the semantic-segmentation net on
2 x 3 x 1024 x 2048 images -- ResNet-50 backbone at output stride 8 (dilated 3x3 in stages 3-4), 1x1 to
19 classes, bilinear x8, per-pixel softmax cross-entropy -- H-partitioned over the GPUs; one step =
forward + backward + filter-gradient allreduce + SGD through the C++ op-graph layer.  The total work
is fixed as GPUs are added ("strong" scaling).  bf16 operands, fp32 accumulate; synthetic seeded inputs.

metric  = spatial conv fwd+bwd TFLOP/s: the convolution FLOPs of one step by the layer table in
          segnet_flops() (2*N*K*C*kh*kw*P*Q per pass on the unpartitioned output) over the step time.
value   = resident step (inputs in HBM), median of individually timed steps run back to back for >= 2 s;
e2e     = the same step fed from pinned host NCHW fp32 images and labels through the host layer's public
          calls (host->device copy, layout / dtype conversion, device->host read of the loss inside).
also    = one result per other workload of the benchmark configuration list, measured in the same run:
          conv (the reference's own spatial-conv microbenchmark shape, with its roofline and an oracle check of
          the partitioned results), halo (exchange / accumulate GB/s), stem_stage1 and resnet50_hybrid (images/s).
`--workload NAME` runs one of them alone and prints its line.
"""
import argparse
import ctypes as C
import datetime
import json
import math
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
MIN_SECONDS = 2.0          # every arm's timed region lasts at least this long
MAX_TIMED_STEPS = 20000


def flops_per_pass(n=None, rows=SIZE, cols=SIZE):
    return 2.0 * (BATCH if n is None else n) * CH * CH * KS * KS * rows * cols


# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the three conv kernels of the
# microbenchmark shape, from an `ncu --set full --clock-control none` capture of one launch each at batch 4 on
# one GPU; traffic grows in proportion to the pixels a launch processes, so it is scaled by batch / 4 / strips.
NCU_TRAFFIC_BATCH4 = {"fprop": 226.1e6, "dgrad": 223.3e6, "wgrad": 275.6e6}


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


class Env:
    """Rank / world of this process and the one process group every workload shares."""

    def __init__(self, gpus):
        import torch
        self.rank, self.world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != gpus:
            raise SystemExit(f"--gpus {gpus} but WORLD_SIZE={self.world}: launch with torch.distributed.run --nproc-per-node {gpus}")
        torch.cuda.set_device(self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local),
                                    timeout=datetime.timedelta(seconds=300))
            self.dist = dist

    def barrier(self):
        if self.dist:
            self.dist.barrier()

    def max_over_ranks(self, values):
        """element-wise maximum of a list of floats over all ranks"""
        import torch
        t = torch.tensor(list(values), device="cuda", dtype=torch.float64)
        if self.dist:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.cpu().numpy()

    def close(self):
        if self.dist:
            self.dist.barrier()
            self.dist.destroy_process_group()


def timed_steps(env, run_step, marks, steps, min_seconds=None):
    """Barrier + synchronize, then n = max(steps, ceil(min_seconds / step)) steps back to back with CUDA events
    after every step on the launching stream(s); synchronize + barrier.  `marks()` records one event per stream
    the step ends on and returns them.  Returns (per-step ms as the max over ranks, n, region seconds)."""
    import torch
    if min_seconds is None:
        min_seconds = MIN_SECONDS
    env.barrier()
    torch.cuda.synchronize()
    t0 = marks()
    for _ in range(3):
        run_step()
    t1 = marks()
    torch.cuda.synchronize()
    est = float(env.max_over_ranks([max(a.elapsed_time(b) for a in t0 for b in t1) / 3.0])[0])
    n = int(min(MAX_TIMED_STEPS, max(steps, math.ceil(min_seconds * 1e3 / max(est, 1e-3)))))
    env.barrier()
    torch.cuda.synchronize()
    ev = [marks()]
    for _ in range(n):
        run_step()
        ev.append(marks())
    torch.cuda.synchronize()
    origin = ev[0][0]
    ends = [max(origin.elapsed_time(e) for e in evs) for evs in ev]
    per = [ends[i + 1] - ends[i] for i in range(n)]
    per = env.max_over_ranks(per)
    env.barrier()
    return per, n, float(np.sum(per)) * 1e-3


def step_stats(per):
    v = np.sort(np.asarray(per))
    n = len(v)
    return {"median": float(np.median(v)), "p10": float(v[int(0.1 * (n - 1))]), "p90": float(v[int(round(0.9 * (n - 1)))]),
            "mean": float(np.mean(v)), "samples": n}


# ----------------------------------------------------------------------------- CPU arm
def cpu_conv_sample(target_seconds, ch_in=CH, ch_out=CH, width=SIZE, dil=DIL, max_rows=SIZE):
    """Times the oracle's conv fwd + dgrad + wgrad (3x3, given dilation, halo-padded input) on a strip sample of a
    layer (one image, `rows` output rows, full width) sized for ~target_seconds, on every core this process may
    use -- the OpenMP team is set explicitly, an inherited OMP_NUM_THREADS=1 does not apply."""
    from oracle import orc
    from tests import helpers as H
    threads = orc.set_num_threads()

    def run(rows):
        x = H.uniform(1, (1, ch_in, rows + 2 * dil, width + 2 * dil))
        w = H.normal(2, (ch_out, ch_in, KS, KS), float(np.sqrt(2.0 / (KS * KS * ch_in))))
        dy = H.uniform(3, (1, ch_out, rows, width))
        t0 = time.perf_counter()
        y = orc.conv2d_fprop(x, w, None, dil=(dil, dil), omp=True)
        orc.conv2d_dgrad(dy, w, x.shape, dil=(dil, dil), omp=True)
        orc.conv2d_wgrad(x, dy, w.shape, dil=(dil, dil), omp=True)
        dt = time.perf_counter() - t0
        assert y.shape == (1, ch_out, rows, width)
        return dt, 3 * 2.0 * ch_in * ch_out * KS * KS * rows * width

    dt, fl = run(2)                       # calibration
    rows = int(max(2, min(max_rows, 2 * target_seconds / max(dt, 1e-6))))
    dt, fl = run(rows)
    return fl / dt / 1e12, dt, rows, threads


def cpu_small_configs():
    """The two configurations small enough to run whole on the host cores: config 1 (3x3 conv, 64 -> 64, 64 x 64, two
    H-strips with 1-row halos exchanged in host memory: fwd + dgrad + wgrad, 0.906 GFLOP) and config 2 (halo exchange +
    accumulate-back, N=8, C=256, 224 x 224, 8 strips, halo 3, fp32), through the oracle."""
    from oracle import orc
    from tests import helpers as H
    orc.set_num_threads()
    x, w = H.uniform(1, (1, 64, 64, 64)), H.normal(2, (64, 64, 3, 3), float(np.sqrt(2.0 / 576)))
    dy = H.uniform(3, (1, 64, 64, 64))
    t0 = time.perf_counter()
    strips = H.split_strips(x, 2, 1)
    orc.halo_exchange(strips, orc.NCHW, 1, 64, 32, 64, 1)
    for r in range(2):
        orc.conv2d_fprop(strips[r], w, None, omp=True)
        orc.conv2d_dgrad(dy[:, :, r * 32:(r + 1) * 32], w, strips[r].shape, omp=True)
        orc.conv2d_wgrad(strips[r], dy[:, :, r * 32:(r + 1) * 32], w.shape, omp=True)
    t1 = time.perf_counter() - t0
    R, p, N, Cc, Hh, W = 8, 3, 8, 256, 224, 224
    bufs = [np.zeros((N, Cc, Hh // R + 2 * p, W + 2 * p), np.float32) for _ in range(R)]
    t0 = time.perf_counter()
    orc.halo_exchange(bufs, orc.NCHW, p, W, Hh // R, Cc, N)
    t2 = time.perf_counter() - t0
    t0 = time.perf_counter()
    orc.halo_reduce(bufs, orc.NCHW, p, W, Hh // R, Cc, N)
    t3 = time.perf_counter() - t0
    payload = 2 * (R - 1) * N * Cc * p * W * 4
    return {"config1_conv3x3_2strips": {"seconds": t1, "tflops": 0.906e9 / t1 / 1e12},
            "config2_halo_r8_p3_f32": {"exchange_gbs": payload / t2 / 1e9, "reduce_gbs": payload / t3 / 1e9, "payload_bytes": payload}}


# the layer the CPU arm samples for the segmentation net: a stage-3 3x3 (256 -> 256, dilation 2) on its
# 128 x 256 map -- the most frequent conv of the net (6 blocks)
SEG_CPU_LAYER = dict(ch_in=256, ch_out=256, width=256, dil=2, max_rows=128)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    conv = args.workload == "conv"
    budget = 120.0 / max(1, args.steps + args.warmup)
    vals, rows, cores, secs = [], 0, 1, 0.0
    for i in range(args.warmup + args.steps):
        v, dt, rows, cores = cpu_conv_sample(min(20.0, budget)) if conv else cpu_conv_sample(min(20.0, budget), **SEG_CPU_LAYER)
        if i >= args.warmup:
            vals.append(v); secs += dt
    value = float(np.mean(vals))
    if conv:
        sample = f"oracle conv fwd+dgrad+wgrad on a {rows}-row x {SIZE}-col strip of one image per step (of 32 x 512 rows)"
        config = {"workload": "microbench_spatial_conv", "batch": BATCH, "channels": CH, "image": [SIZE, SIZE],
                  "kernel": KS, "dilation": DIL, "halo": PAD, "bounded_sample": sample}
    else:
        sample = (f"oracle conv fwd+dgrad+wgrad of one stage-3 layer of the net (3x3, 256->256, dilation 2) on a {rows}-row x 256-col "
                  "strip of one image per step; the net's other operators are not timed on the CPU")
        config = {"workload": "resnet50_dilated_segnet", "image": [2, 3, 1024, 2048], "bounded_sample": sample}
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * secs / max(1, args.steps), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ----------------------------------------------------------------------------- conv microbenchmark step
class Step:
    """Buffers and the per-step call sequence of one rank (one H-strip) of the spatial conv microbenchmark."""

    def __init__(self, env, batch=None):
        import torch
        from arraydiff_cuda_b200 import abi, dist as addist
        self.torch, self.abi, self.env = torch, abi, env
        self.L = abi.load()
        rank, world = env.rank, env.world
        self.rank, self.world = rank, world
        self.batch = B = BATCH if batch is None else batch
        self.h = SIZE // world
        h, Wp, Hp = self.h, SIZE + 2 * PAD, SIZE // world + 2 * PAD
        bf = torch.bfloat16
        xbytes = B * Hp * Wp * CH * 2
        self.arena = addist.SymmetricArena(2 * xbytes + (1 << 20), rank, world)
        self.x, self.x_off = self.arena.alloc((B, Hp, Wp, CH), bf)       # halo-padded input strip
        self.gx, self.gx_off = self.arena.alloc((B, Hp, Wp, CH), bf)     # halo-padded input gradient
        self.flags, self.flags_off = self.arena.alloc((8,), torch.int64)      # 0 from_prev 1 from_next 2 gprev 3 gnext
        self.counter = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.status = torch.zeros(4, dtype=torch.int32, device="cuda")
        # flag values are *ebase + 1 in every step and the base advances by one at the end of the step (on the device), so
        # that a step recorded into a CUDA graph replays with fresh values; all ranks advance in lockstep
        self.ebase = torch.zeros(1, dtype=torch.int64, device="cuda")
        g = torch.Generator(device="cuda").manual_seed(1234 + rank)
        self.x.zero_()
        self.x[:, PAD:PAD + h, PAD:PAD + SIZE] = (torch.rand((B, h, SIZE, CH), device="cuda", generator=g) * 2 - 1).to(bf)
        gw = torch.Generator(device="cuda").manual_seed(99)
        self.w = (torch.randn((CH, KS, KS, CH), device="cuda", generator=gw) * float(np.sqrt(2.0 / (KS * KS * CH)))).to(bf)
        self.y = torch.empty((B, h, SIZE, CH), dtype=bf, device="cuda")
        self.dy = (torch.rand((B, h, SIZE, CH), device="cuda", generator=g) * 2 - 1).to(bf)
        # two filter-gradient buffers: the allreduce of one step's gradient runs on its own stream underneath the
        # next step, so consecutive steps must not share the buffer
        self.dws = [torch.zeros((CH, KS, KS, CH), device="cuda") for _ in range(2)]
        self.dw = self.dws[0]
        self.ar_stream = torch.cuda.Stream()
        self.ar_done = [None, None]
        a = abi.Conv2dArgs()
        a.dtype, a.layout = abi.AD_BF16, abi.AD_NHWC
        a.N, a.C, a.H, a.W, a.K, a.kh, a.kw = B, CH, Hp, Wp, CH, KS, KS
        a.stride_h = a.stride_w = 1
        a.dil_h = a.dil_w = DIL
        nscr = max(self.L.ad_conv2d_scratch_bytes(C.byref(a), 1), self.L.ad_conv2d_scratch_bytes(C.byref(a), 2), 16)
        self.scratch = torch.zeros(nscr, dtype=torch.uint8, device="cuda")
        a.x, a.w, a.scratch, a.scratch_bytes = self.x.data_ptr(), self.w.data_ptr(), self.scratch.data_ptr(), nscr
        self.conv = a
        self.epoch = 0
        self.halo = True       # False: the same step without halo transfers (measures what they cost exposed)
        self.use_graph = True  # the resident step replays CUDA graphs (False: every call launched from the host)
        self.marks = None      # a list: run() brackets every conv call with CUDA events and appends (name, e0, e1)
        ha = abi.HaloArgs()
        ha.dtype, ha.layout = abi.AD_BF16, abi.AD_NHWC
        ha.halo_pad, ha.base_width, ha.base_height, ha.num_channels, ha.batch_size = PAD, SIZE, h, CH, B
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
        self.hx.epoch, self.hx.epoch_base = 1, self.ebase.data_ptr()
        self.fp = fp
        self.host = None
        self.graphs = {}       # (halo, dw buffer) -> (captured step, kernel launches in it)
        self.replayed_launches = 0

    def make_host_buffers(self):
        """Pinned host tensors in the reference's boundary format (NCHW fp32, unpadded strip) and the device staging
        buffers the end-to-end step converts from."""
        torch, B, h = self.torch, self.batch, self.h
        from tests import helpers as H
        self.H = H
        self.x32 = torch.empty((B, CH, h, SIZE), device="cuda")
        self.dy32 = torch.empty((B, CH, h, SIZE), device="cuda")
        self.x32.copy_(self.x[:, PAD:PAD + h, PAD:PAD + SIZE].permute(0, 3, 1, 2))
        self.dy32.copy_(self.dy.permute(0, 3, 1, 2))
        self.x_host = torch.empty(self.x32.shape, dtype=torch.float32).pin_memory()
        self.dy_host = torch.empty(self.dy32.shape, dtype=torch.float32).pin_memory()
        self.x_host.copy_(self.x32)
        self.dy_host.copy_(self.dy32)
        self.dw_host = torch.empty(self.dw.shape, dtype=torch.float32).pin_memory()
        self.cv = [(H.view_nchw(self.x32), H.view_nhwc(self.x, interior=(PAD, h, SIZE))),
                   (H.view_nchw(self.dy32), H.view_nhwc(self.dy))]
        self.host = True

    def _s(self):
        return C.c_void_p(self.torch.cuda.current_stream().cuda_stream)

    def _wait(self, slot):
        self.abi.check(self.L.ad_flag_wait_rel(C.c_void_p(self.flags.data_ptr() + 8 * slot), C.c_void_p(self.ebase.data_ptr()), 1,
                                               2_000_000_000, C.c_void_p(self.status.data_ptr()), self._s()), "flag wait")

    def _signal(self, rank, slot):
        self.abi.check(self.L.ad_flag_signal_rel(C.c_void_p(self.fp[rank] + 8 * slot), C.c_void_p(self.ebase.data_ptr()), 1,
                                                 self._s()), "flag signal")

    def _timed(self, name, fn):
        if self.marks is None:
            return fn()
        e0, e1 = self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        self.marks.append((name, e0, e1))

    def run(self, e2e=False):
        """One step.  The resident step (no host buffers, no per-call events) replays a CUDA graph of everything but the
        filter-gradient allreduce: one graph per gradient buffer and halo mode, recorded on first use."""
        torch = self.torch
        self.epoch += 1
        k = self.epoch & 1
        main = torch.cuda.current_stream()
        if e2e:
            # host NCHW fp32 -> device staging -> bf16 NHWC (into the interior of the halo-padded strip)
            self.x32.copy_(self.x_host, non_blocking=True)
            self.dy32.copy_(self.dy_host, non_blocking=True)
            for src, dst in self.cv:
                self.abi.check(self.L.ad_convert(C.byref(src), C.byref(dst), 0, self._s()), "convert")
        if self.world > 1 and self.ar_done[k] is not None:
            # this step's gradient buffer: free again once the allreduce that last used it (two steps ago) is done
            main.wait_event(self.ar_done[k])
        self.dw = self.dws[k]
        if self.use_graph and not e2e and self.marks is None and self.epoch > 4:   # the first steps run eagerly
            key = (self.halo, k)
            if key not in self.graphs:
                l0 = self.L.ad_launch_count()
                g = torch.cuda.CUDAGraph()
                # thread-local: the process group's watchdog thread may query events while this thread records
                with torch.cuda.graph(g, capture_error_mode="thread_local"):
                    self._body(k)
                self.graphs[key] = (g, int(self.L.ad_launch_count() - l0))
            g, n = self.graphs[key]
            g.replay()
            self.replayed_launches += n
        else:
            self._body(k)
        if self.world > 1:
            # filter-gradient allreduce over NCCL / NVLink on its own stream: it overlaps the next step's exchange and
            # forward pass (an optimizer would consume it after that step's backward pass)
            self.ar_stream.wait_stream(main)
            with torch.cuda.stream(self.ar_stream):
                self.env.dist.all_reduce(self.dws[k])
                self.ar_done[k] = self.ar_stream.record_event()
            if e2e:
                main.wait_stream(self.ar_stream)
        if e2e:
            self.dw_host.copy_(self.dws[k], non_blocking=True)

    def _body(self, k):
        """Halo exchange, forward, data gradient, halo-gradient accumulate-back and filter gradient into buffer k, on the
        current stream and the side stream forked from it (joined again at the end)."""
        L, abi, a, s = self.L, self.abi, self.conv, self._s()
        r, R = self.rank, self.world
        # forward: push my edge rows into the neighbours' halo rows on a side stream and wait there for
        # theirs, while the main stream already convolves the interior rows; the PAD boundary rows at
        # either end follow once the halo has landed
        a.y, a.accumulate = self.y.data_ptr(), 0
        if R > 1 and self.halo:
            main = self.torch.cuda.current_stream()
            self.side.wait_stream(main)
            with self.torch.cuda.stream(self.side):
                s2 = self._s()
                abi.check(L.ad_halo_exchange(C.byref(self.hx), s2), "halo exchange")
                for slot in self.plan.exchange_waits():
                    self._wait(slot)
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
        self.dw = self.dws[k]
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
                    self._signal(peer, slot)
                for slot in self.plan.reduce_waits():
                    self._wait(slot)
                abi.check(L.ad_halo_reduce(C.byref(self.hg), s2), "halo reduce")
        self._timed("wgrad", lambda: abi.check(L.ad_conv2d_wgrad(C.byref(a), s), "wgrad"))
        if R > 1 and self.halo:
            self.torch.cuda.current_stream().wait_stream(self.side)
            # all of this step's flag values are used up: the next step's are one higher
            abi.check(L.ad_flag_advance(C.c_void_p(self.ebase.data_ptr()), 1, s), "flag advance")

    def check_status(self):
        st = self.status.cpu().tolist() + self.scratch[:4].view(self.torch.int32).cpu().tolist()
        if any(v != 0 for v in st):
            raise RuntimeError(f"device-side bounded wait reported {st}")

    def close(self):
        self.arena.close(barrier=self.env.barrier)


def verify_conv_step(env, step):
    """After one resident step: results of the partitioned step against the CPU oracle evaluated on windows of the
    UNPARTITIONED seeded tensors (edge rows of every rank are gathered first).  Ranks 0 and R-1 check, for the first
    and last image: the PAD output rows at each strip edge (they read the neighbour's halo rows), PAD interior
    rows, and the PAD first / last interior rows of the input gradient after the halo accumulate-back.  Every rank
    checks 32 sampled entries of the all-reduced filter gradient against float64 dot products of the resident tensors
    summed over ranks.  Tolerance: max-relative 2e-2 (bf16 outputs), 1e-3 for the fp32 filter gradient."""
    import torch
    from oracle import orc
    torch_, dist, r, R, p, h, B = torch, env.dist, step.rank, step.world, PAD, step.h, step.batch
    step.run()
    torch.cuda.synchronize()     # includes the gradient allreduce on its own stream
    env.barrier()
    step.check_status()
    imgs = sorted({0, B - 1})
    e = 3 * p

    def gather(t):
        t = t.contiguous()
        if R == 1:
            return [t]
        out = [torch.empty_like(t) for _ in range(R)]
        dist.all_gather(out, t)
        return out

    xi = step.x[imgs][:, p:p + h, p:p + SIZE]
    x_top, x_bot = gather(xi[:, :e]), gather(xi[:, h - e:])
    dyi = step.dy[imgs]
    dy_top, dy_bot = gather(dyi[:, :e]), gather(dyi[:, h - e:])

    def nchw(t):     # [n][rows][W][C] bf16 device -> float32 NCHW host
        return np.ascontiguousarray(t.float().cpu().numpy().transpose(0, 3, 1, 2))

    w = np.ascontiguousarray(step.w.float().cpu().numpy().transpose(0, 3, 1, 2))      # KRSC -> KCRS
    zeros = np.zeros((len(imgs), CH, e, SIZE), np.float32)
    errs = {}

    def rel(a, b):
        return float(np.max(np.abs(a.astype(np.float64) - b)) / max(float(np.max(np.abs(b))), 1e-30))

    def padw(a):
        return np.pad(a, ((0, 0), (0, 0), (0, 0), (p, p)))

    if r in (0, R - 1):
        orc.set_num_threads()
        y = step.y[imgs]
        gx = step.gx[imgs][:, :, p:p + SIZE]
        for side in ("top", "bottom"):
            if side == "top":
                xa = nchw(x_bot[r - 1]) if r > 0 else zeros
                xw = np.concatenate([xa, nchw(x_top[r])], axis=2)
                da = nchw(dy_bot[r - 1]) if r > 0 else zeros
                dw_ = np.concatenate([da, nchw(dy_top[r])], axis=2)
                yo, go = slice(2 * p, 3 * p), slice(4 * p, 5 * p)
                y_got, g_got = nchw(y[:, :p]), nchw(gx[:, p:2 * p])
            else:
                xb = nchw(x_top[r + 1]) if r + 1 < R else zeros
                xw = np.concatenate([nchw(x_bot[r]), xb], axis=2)
                db = nchw(dy_top[r + 1]) if r + 1 < R else zeros
                dw_ = np.concatenate([nchw(dy_bot[r]), db], axis=2)
                yo, go = slice(p, 2 * p), slice(3 * p, 4 * p)
                y_got, g_got = nchw(y[:, h - p:]), nchw(gx[:, h:h + p])
            y_w = orc.conv2d_fprop(padw(xw), w, None, dil=(DIL, DIL), omp=True)
            errs[f"y_{side}_rows"] = rel(y_got, y_w[:, :, yo])
            g_w = orc.conv2d_dgrad(dw_, w, (len(imgs), CH, 2 * e + 2 * p, SIZE + 2 * p), dil=(DIL, DIL), omp=True)
            errs[f"dx_{side}_rows"] = rel(g_got, g_w[:, :, go, p:p + SIZE])
        m = h // 2
        xw = nchw(step.x[imgs][:, m:m + 3 * p])
        y_w = orc.conv2d_fprop(xw, w, None, dil=(DIL, DIL), omp=True)
        errs["y_interior_rows"] = rel(nchw(step.y[imgs][:, m:m + p]), y_w)
    # sampled filter-gradient entries: dw[k,r,s,c] = sum over images and pixels of x[.., q + r*dil, t + s*dil, c] * dy[.., q, t, k]
    rng = np.random.default_rng(5)
    ks = [(int(rng.integers(CH)), int(rng.integers(KS)), int(rng.integers(KS)), int(rng.integers(CH))) for _ in range(32)]
    part = torch.stack([(step.x[:, rr * DIL:rr * DIL + h, ss * DIL:ss * DIL + SIZE, c].double() * step.dy[:, :, :, k].double()).sum()
                        for (k, rr, ss, c) in ks])
    if R > 1:
        dist.all_reduce(part)
    got = torch.stack([step.dw[k, rr, ss, c] for (k, rr, ss, c) in ks]).double()
    errs["dw_sampled"] = float((got - part).abs().max() / part.abs().max().clamp_min(1e-30))
    tol = {k: (1e-3 if k == "dw_sampled" else 2e-2) for k in errs}
    ok = all(v < tol[k] for k, v in errs.items())
    flags = env.max_over_ranks([0.0 if ok else 1.0, max(errs.values())])
    # the edge checks of the last rank, for the record on rank 0
    worst = {k: float(v) for k, v in errs.items()}
    return {"ok": bool(flags[0] == 0.0), "max_rel": float(flags[1]), "rank0": worst,
            "checked_by_ranks": sorted({0, R - 1}), "oracle": "CPU restatement on windows of the unpartitioned tensors"}


def kernel_times_in_step(env, step, steps):
    """Average device time per step of each conv pass, from CUDA events around its launches inside `steps` full
    steps run back to back (the conditions of the timed region: warm clocks, halo traffic alongside)."""
    import torch
    env.barrier()
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


def run_conv_workload(env, args, with_cpu=True):
    """`--workload conv`: the shape the reference fixes for its own measurement of this path -- 3x3 convolution,
    dilation 3, halo 3, batch 32, 64 -> 64 channels, 512 x 512 pixels, the H axis cut into one strip per GPU
    (tools/microbench_spatial_conv.cc:25-41, :101-107).  One step = halo exchange + forward conv + data gradient +
    filter gradient + halo-gradient accumulate-back + filter-gradient allreduce, driven through the C ABI."""
    import torch
    from arraydiff_cuda_b200 import abi
    world, rank = env.world, env.rank
    if SIZE % world:
        raise SystemExit("image height must divide by the number of GPUs")
    L = abi.load()   # raises if the CUDA library is missing: no fallback
    step = Step(env)
    step.use_graph = not args.no_graph
    for _ in range(max(8, args.warmup)):     # the first 4 run eagerly, the next two record the graphs
        step.run()
    torch.cuda.synchronize()
    step.check_status()

    def marks():
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return [e]

    sampler = ClockSampler(env.local)
    if rank == 0:
        sampler.start()
    launches0, replayed0 = L.ad_launch_count(), step.replayed_launches
    per, n, secs = timed_steps(env, step.run, marks, args.steps)
    launches = L.ad_launch_count() - launches0 + step.replayed_launches - replayed0
    clocks = sampler.stop() if rank == 0 else None
    step.check_status()
    st = step_stats(per)

    # what the halo transfers cost exposed: the same step with and without them, both launched call by call (the two
    # recorded graphs differ in more than the transfers: one forward launch instead of three)
    halo_exposed = None
    if world > 1:
        recorded, step.use_graph = step.use_graph, False
        per_h, _, _ = timed_steps(env, step.run, marks, args.steps, min_seconds=0.5)
        step.halo = False
        per_nh, _, _ = timed_steps(env, step.run, marks, args.steps, min_seconds=0.5)
        step.halo, step.use_graph = True, recorded
        halo_exposed = float(np.median(per_h)) - float(np.median(per_nh))
    # as long as a second, like the timed region: a short burst runs at higher clocks than the power cap sustains
    kt_step = kernel_times_in_step(env, step, int(min(MAX_TIMED_STEPS, max(20, args.steps, math.ceil(min(1.0, MIN_SECONDS) * 1e3 / st["median"])))))
    step.check_status()
    verify = verify_conv_step(env, step)

    step.make_host_buffers()
    for _ in range(2):
        step.run(e2e=True)
    per_e2e, n_e2e, _ = timed_steps(env, lambda: step.run(e2e=True), marks, 3, min_seconds=0.5)
    step.check_status()

    total_flops = 3 * flops_per_pass()
    med = st["median"]
    line = None
    if rank == 0:
        peaks = measured_peaks()
        kt = kernel_times(torch, step)
        top = max(kt_step, key=kt_step.get)
        per_launch_flops = flops_per_pass(BATCH, step.h, SIZE)
        achieved = per_launch_flops / kt_step[top] / 1e12
        hbytes = step.x_host.numel() * 4 + step.dy_host.numel() * 4
        line = {
            "metric": METRIC, "value": total_flops / (med * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": med, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "timing": f"median of {n} individually timed steps run back to back over {secs:.2f} s (CUDA events, max over ranks per step)",
            "config": {"workload": "microbench_spatial_conv", "batch": BATCH, "channels": CH, "image": [SIZE, SIZE],
                       "kernel": KS, "dilation": DIL, "halo": PAD, "strips": world, "layout": "NHWC",
                       "filter_gradient_allreduce": "none (one strip)" if world == 1 else "NCCL on its own stream, double-buffered: overlaps the next step's exchange and forward pass",
                       "l2": "inputs larger than L2 (%.2f GB activations per pass)" % (BATCH * SIZE * SIZE * CH * 2 / 1e9), "parallelism": f"spatial-h{world}",
                       "launch": "cuda graph per step (the NCCL allreduce is launched beside it)" if step.use_graph else "eager"},
            "e2e": {"value": total_flops / (float(np.median(per_e2e)) * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": hbytes,
                    "d2h_bytes_per_step": step.dw_host.numel() * 4, "steps": n_e2e,
                    "boundary": "pinned host NCHW fp32 strips (the reference's boundary format); the conversion to bf16 NHWC is inside the timed step"},
            "gpu_launches": int(launches), "timed_steps": n, "timed_region_s": secs,
            "step_ms": st,
            "halo_exposed_ms": halo_exposed,
            "roofline": {"bound": "tensor", "kernel": {"fprop": "conv_tc_stream_fwd_kernel<3,3> (fprop)", "dgrad": "conv_tc_stream_fwd_kernel<3,3> (dgrad)",
                                                        "wgrad": "conv_tc_rows_wgrad_kernel<3,3>"}[top], "achieved": achieved, "peak": peaks["tf_sustained"],
                         "unit": "TFLOP/s", "frac": achieved / peaks["tf_sustained"],
                         "traffic": NCU_TRAFFIC_BATCH4[top] * BATCH / 4 / world,
                         "peak_source": peaks["source"] + " (sustained: the kernel is timed with CUDA events inside full steps run back to back)",
                         "kernels_us": {k: v * 1e6 for k, v in kt_step.items()},
                         "kernels_alone_us": {k: v * 1e6 for k, v in kt.items()},
                         "frac_alone_of_burst": per_launch_flops / kt[top] / 1e12 / peaks["tf_burst"]},
            "verify": verify,
            "clocks": clocks,
        }
        if world == 1 and with_cpu:
            v, dt, rows, cores = cpu_conv_sample(args.cpu_seconds)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": f"oracle conv fwd+dgrad+wgrad on a {rows}-row x {SIZE}-col strip of one image ({dt:.1f} s)"}
    step.close()
    return line


# ----------------------------------------------------------------------------- halo microbenchmark
def run_halo_workload(env, args):
    """`--workload halo`: benchmark config 2 -- NCHW tensors N=8, C=256, 224x224 cut into H-strips, halo
    1 and 3, fp32 and bf16; forward exchange and backward accumulate.  On one GPU the R strips share the
    device and move in ONE launch (HBM-bound: payload read + written); on N GPUs each rank pushes to /
    pulls from its neighbours over NVLink, with NCCL send/recv of packed faces timed beside it."""
    import torch
    from arraydiff_cuda_b200 import abi, dist as addist
    rank, world, dist = env.rank, env.world, env.dist
    L = abi.load()
    N, Cc, Hh, W = 8, 256, 224, 224
    iters = max(args.steps, 50)
    cases = []
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def timed(fn, iters):
        for _ in range(max(3, args.warmup)):
            fn()
        env.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return float(env.max_over_ranks([e0.elapsed_time(e1) / iters])[0]) * 1e-3

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
                    te = timed(lambda: abi.check(L.ad_halo_exchange(C.byref(a), s)), iters)
                    tr = timed(lambda: abi.check(L.ad_halo_reduce(C.byref(a), s)), iters)
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

                    te, tr, tn = timed(exch, iters), timed(red, iters), timed(nccl, min(iters, 50))
                    if int(status.item()) != 0:
                        raise RuntimeError("bounded flag wait timed out")
                    rec["nccl_sendrecv_us"] = tn * 1e6
                    rec["nccl_sendrecv_gbs"] = payload / tn / 1e9
                    arena.close(barrier=env.barrier)
                rec.update(exchange_us=te * 1e6, exchange_gbs=payload / te / 1e9, reduce_us=tr * 1e6, reduce_gbs=payload / tr / 1e9)
                cases.append(rec)
    line = None
    if rank == 0:
        peaks = measured_peaks()
        top = max(cases, key=lambda c: c["payload_bytes"])
        # one GPU: every payload byte is read and written locally; N GPUs: bytes into the busiest GPU over NVLink
        if world == 1:
            achieved, peak, bound = 2 * top["payload_bytes"] / (top["exchange_us"] * 1e-6) / 1e9, peaks["hbm_gbs"], "hbm"
        else:
            per_gpu = top["payload_bytes"] / (world - 1)      # two faces land in an interior rank
            achieved, peak, bound = per_gpu / (top["exchange_us"] * 1e-6) / 1e9, 770.0, "nvlink"
        line = {
            "metric": "halo_exchange_gbs", "value": top["exchange_gbs"], "unit": "GB/s", "n_gpus": world, "steps": iters,
            "warmup": max(3, args.warmup), "ms_per_step": top["exchange_us"] / 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "halo_microbench", "tensor": [N, Cc, Hh, W], "layout": "NCHW",
                       "l2": "same buffers every iteration (payload smaller than L2; launch-latency dominated below ~10 MiB)"},
            "gpu_launches": int(L.ad_launch_count() - launches0),
            "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                         "peak_source": "measured copy bandwidth" if world == 1 else "peer copy rate measured on this pool, per direction"},
            "cases": cases,
        }
    return line


# ----------------------------------------------------------------------------- nets through the C++ op graph
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


def conv_profile_of_step(abi, eager_step, sync, step_ms):
    """One eagerly launched step with every convolution call bracketed by CUDA events on its stream (the library's
    per-call timing): returns the roofline record of the shape that takes the most time and a short table."""
    L = abi.load()
    eager_step(); sync()
    # up to a second of steps back to back, like the timed region: one step alone runs at higher clocks than the power
    # cap sustains
    reps = int(max(1, min(40, math.ceil(min(1.0, MIN_SECONDS) * 1e3 / step_ms)))) if step_ms else 1
    # the filter gradients stay on the main stream while the calls are timed: underneath other kernels (where the
    # timed step runs them) a call's elapsed time is not the kernel's
    prev = os.environ.get("ARRAYDIFF_B200_WGRAD_OVERLAP")
    os.environ["ARRAYDIFF_B200_WGRAD_OVERLAP"] = "0"
    L.ad_conv2d_profile(1)
    for _ in range(reps):
        eager_step()
    sync()
    recs = abi.conv_profile_read()
    L.ad_conv2d_profile(0)
    if prev is None:
        os.environ.pop("ARRAYDIFF_B200_WGRAD_OVERLAP", None)
    else:
        os.environ["ARRAYDIFF_B200_WGRAD_OVERLAP"] = prev
    groups = {}
    for e in recs:
        if e.ms < 0 or e.status != 0:
            continue
        key = (e.pass_, e.kernel, e.N, e.C, e.H, e.W, e.K, e.kh, e.kw, e.stride, e.dil, e.pad, e.out_rows)
        g = groups.setdefault(key, [0.0, 0])
        g[0] += e.ms / reps; g[1] += 1
    for g in groups.values():
        g[1] = max(1, g[1] // reps)
    if not groups:
        return None
    names = {0: "fprop", 1: "dgrad", 2: "wgrad"}
    fam = {1: "conv_direct_f32", 2: "conv_tc (general tiles)", 3: "conv_tc_row (row streaming)"}

    def flops(key):
        ps, kern, N, Cc, Hh, W, K, kh, kw, st, dil, pad, rows = key
        P = (Hh + 2 * pad - dil * (kh - 1) - 1) // st + 1
        Q = (W + 2 * pad - dil * (kw - 1) - 1) // st + 1
        if rows:
            P = rows
        return 2.0 * N * K * Cc * kh * kw * P * Q

    total = sum(g[0] for g in groups.values())
    ranked = sorted(groups.items(), key=lambda kv: -kv[1][0])
    peaks = measured_peaks()
    table = []
    for key, (ms, cnt) in ranked[:4]:
        table.append({"pass": names[key[0]], "kernel": fam.get(key[1], "?"), "shape": {"N": key[2], "C": key[3], "H": key[4], "W": key[5], "K": key[6],
                      "k": [key[7], key[8]], "stride": key[9], "dil": key[10]}, "launches": cnt, "us_per_launch": ms / cnt * 1e3,
                      "tflops": flops(key) / (ms / cnt * 1e-3) / 1e12, "share_of_conv_time": ms / total})
    key, (ms, cnt) = ranked[0]
    achieved = flops(key) / (ms / cnt * 1e-3) / 1e12
    return {"bound": "tensor", "kernel": f"{fam.get(key[1], '?')} {names[key[0]]} {key[3]}->{key[6]} {key[7]}x{key[8]} dil {key[10]} on {key[2]}x{key[4]}x{key[5]}",
            "achieved": achieved, "peak": peaks["tf_sustained"], "unit": "TFLOP/s", "frac": achieved / peaks["tf_sustained"], "traffic": None,
            "peak_source": peaks["source"] + f" (sustained); kernel timed by CUDA events around its launches inside {reps} eagerly launched steps run back to back",
            "profiled_steps": reps,
            "conv_ms_per_step": total, "conv_share_of_step": total / step_ms if step_ms else None, "top": table}


def run_net_workload(env, args, kind):
    """`segnet`: benchmark config 4 -- dilated ResNet-50 at output stride 8 on 2x3x1024x2048 with a 19-class head, x8
    bilinear upsample and per-pixel softmax NLL against uniform random labels.
    `stem_stage1`: benchmark config 3 -- ResNet-50 stem + stage 1 on one 3x1024x1024 image, forward + backward against an
    upstream gradient N(0,1).  93.6 GFLOP per step (stem dgrad excluded).
    `resnet50_hybrid`: benchmark config 5 -- ResNet-50 classifier on 224 x 224, global batch 256, the GPUs in
    data-parallel groups of 2 H-strips each (8 GPUs: 4 data x 2 spatial).  On one GPU: one group (batch 64) as 2 strips
    sharing the device.
    All H-partitioned over the GPUs (or over `--strips` ranks sharing one GPU), bf16 operands, filter-gradient allreduce and
    SGD update, through the C++ host layer (zoo builder -> op graph -> C ABI kernels)."""
    import torch
    from arraydiff_cuda_b200 import abi, hostlib
    from arraydiff_cuda_b200.dist import _Raw
    rank, world, local, dist = env.rank, env.world, env.local, env.dist
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
    # the stem workload has no loss: its objective <dy, y> with a fixed random dy is unbounded, so any positive rate
    # walks the weights off to infinity over thousands of timed steps; rate 0 runs the same update kernel on the same
    # bytes and keeps the parameters where they are
    net.configure_sgd(0.01 if (seg or hyb) else 0.0, 0.9, l2=1e-4, nesterov=True)
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

    use_graph = not args.no_graph and not (world > 1 and args.nccl_allreduce)

    def e2e_step():
        # host image -> every local rank (H2D and the conversion to bf16 NHWC inside), host labels / upstream gradient ->
        # device, then the step itself: replayed from the CUDA graph like the resident step (or launched call by call)
        net.load_input(x) if use_graph else net.forward(x)
        for r in ranks:
            if seg:
                net.set_labels(r, labels[:, r * hs:(r + 1) * hs])
            elif hyb:
                net.set_labels(r, labels)
            else:
                net.set_output_grad(r, dy[r])
        if use_graph:
            net.step_graph(True)
        else:
            net.backward()
            net.sgd_step()
        return net.loss() if (seg or hyb) else net.output(ranks[0], out=out_host)          # D2H read of a result

    # steady-state step: the resident step replayed from a CUDA graph (flag values between processes are
    # relative to a device-resident base, the gradient allreduce is the built-in peer exchange)
    step = (lambda: net.step_graph(True)) if use_graph else (lambda: net.step_resident(True))
    net.forward(x)                           # first step call by call: every lazily allocated buffer exists afterwards
    for r in ranks:
        if seg:
            net.set_labels(r, labels[:, r * hs:(r + 1) * hs])
        elif hyb:
            net.set_labels(r, labels)
        else:
            net.set_output_grad(r, dy[r])
    net.backward()
    net.sgd_step()
    net.step_resident(True)
    for _ in range(max(3, args.warmup)):
        step()
    net.sync()
    assert net.status() == 0, "a bounded device wait timed out"
    streams = [torch.cuda.ExternalStream(Lh.adh_context_stream(ctx.h, r)) for r in ranks]

    def marks():
        out = []
        for st in streams:
            e = torch.cuda.Event(enable_timing=True)
            e.record(st)
            out.append(e)
        return out

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = L.ad_launch_count()
    per, n, secs = timed_steps(env, step, marks, args.steps)
    launches = net.graph_launches() * n if use_graph else L.ad_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    assert net.status() == 0
    st = step_stats(per)
    med = st["median"]

    # end to end: host clock between synchronisations around k full steps
    k_e2e = max(3, min(args.steps, int(1.0 / max(med * 3e-3, 1e-3))))
    env.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(k_e2e):
        res = e2e_step()
    net.sync()
    t_e2e = float(env.max_over_ranks([(time.perf_counter() - t0) / k_e2e])[0])

    # which convolution dominates, and how close to the tensor peak it runs
    roof = conv_profile_of_step(abi, lambda: net.step_resident(True), net.sync, med)

    # consistency record: no bounded wait ran out, the loss is finite, every replica holds the same parameters
    loss = None
    if seg or hyb:
        lsum, lcnt = res
        loss = lsum / max(1, lcnt)
    sums = [float(np.sum(net.params(r).astype(np.float64))) for r in ranks]
    lo = -env.max_over_ranks([-min(sums)])[0]
    hi = env.max_over_ranks([max(sums)])[0]
    verify = {"ok": bool(net.status() == 0 and lo == hi and (loss is None or math.isfinite(loss))),
              "status_word": int(net.status()), "loss_per_pixel": loss, "param_sum_identical_on_all_ranks": bool(lo == hi),
              "param_sum": float(hi)}

    scale = (S / 1024.0) ** 2
    flops = segnet_flops(NB, Hh, Ww) if seg else resnet50_flops(NB * D, Hh, Ww) if hyb else 93.6e9 * scale
    line = None
    if rank == 0:
        step_s = med * 1e-3
        line = {
            "metric": METRIC, "value": flops / step_s / 1e12, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": med, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "images_per_s": NB * D / step_s,
            "timing": f"median of {n} individually timed steps run back to back over {secs:.2f} s (CUDA events, max over ranks per step)",
            "config": {"workload": "resnet50_dilated_segnet" if seg else f"resnet50_hybrid_{D}x{strips}" if hyb else "resnet50_stem_stage1",
                       "image": [NB * D, 3, Hh, Ww], "strips": strips, "data_groups": D, "layout": "NHWC",
                       "bn_statistics": "per strip (as the reference)", "update": "allreduce (%s) + Nesterov SGD" % ("nccl" if world > 1 and args.nccl_allreduce else "peer loads" if strips > 1 or D > 1 else "single rank"), "launch": "cuda graph" if use_graph else "eager",
                       "flops_per_step": flops,
                       "l2": "activations of one step total more than 1 GB, larger than L2", "parallelism": f"data{D}-spatial-h{strips}" if hyb else f"spatial-h{strips}"},
            "e2e": {"value": flops / t_e2e / 1e12, "unit": UNIT, "images_per_s": NB * D / t_e2e,
                    "h2d_bytes_per_step": int(x.nbytes // (Sg if world > 1 else 1) + (labels.nbytes if hyb else labels.nbytes // world if seg else sum(d.nbytes for d in dy))),
                    "d2h_bytes_per_step": int(8 * len(ranks) if (hyb or seg) else np.prod(net.strip_shape) * 4), "steps": k_e2e,
                    "timing": "host clock between synchronisations",
                    "boundary": "pinned host NCHW fp32 images and uint32 labels through the host layer's public calls; copies and the conversion to bf16 NHWC are inside"},
            "gpu_launches": int(launches), "timed_steps": n, "timed_region_s": secs, "step_ms": st,
            "roofline": roof, "verify": verify, "clocks": clocks,
        }
    env.barrier()
    _KEEP_ALIVE.append((net, ctx, keep))     # arenas stay mapped in the peers until the process ends
    return line


_KEEP_ALIVE = []


def compact(line):
    """What an `also` entry keeps of a workload's line."""
    if line is None:
        return None
    keep = ("metric", "value", "unit", "ms_per_step", "images_per_s", "timing", "timed_region_s", "gpu_launches", "step_ms",
            "halo_exposed_ms", "roofline", "verify", "e2e", "cpu_baseline", "cases", "error")
    out = {k: line[k] for k in keep if k in line}
    out["workload"] = line.get("config", {}).get("workload")
    return out


def main():
    global BATCH, MIN_SECONDS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--workload", default="all", choices=["all", "segnet", "conv", "halo", "stem_stage1", "resnet50_hybrid"],
                    help="all: segnet as the headline with the others under `also`; segnet: dilated ResNet-50 segmentation net, "
                         "2x3x1024x2048 (config 4; --image = height); conv: the spatial conv microbenchmark step; halo: the "
                         "halo-exchange microbenchmark (config 2); stem_stage1: ResNet-50 stem + stage 1 (config 3); "
                         "resnet50_hybrid: ResNet-50 classifier, 224 x 224, batch 256, data-parallel groups of 2 strips (config 5)")
    ap.add_argument("--strips", type=int, default=1, help="net workloads on one GPU: ranks sharing the device")
    ap.add_argument("--image", type=int, default=1024, help="net workloads: image height")
    ap.add_argument("--nccl-allreduce", action="store_true",
                    help="net workloads on several GPUs: sum the filter gradients with NCCL instead of the built-in peer exchange")
    ap.add_argument("--no-graph", action="store_true", help="net workloads: launch every kernel eagerly instead of replaying a CUDA graph")
    ap.add_argument("--batch", type=int, default=BATCH,
                    help="conv: images per step; the default is the workload's, smaller values are for profiler captures")
    ap.add_argument("--min-seconds", type=float, default=MIN_SECONDS, help="least length of every timed region")
    args = ap.parse_args()
    BATCH = args.batch
    MIN_SECONDS = args.min_seconds
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
        return

    env = Env(args.gpus)
    runners = {
        "segnet": lambda: run_net_workload(env, args, "segnet"),
        "conv": lambda: run_conv_workload(env, args),
        "halo": lambda: run_halo_workload(env, args),
        "stem_stage1": lambda: run_net_workload(env, args, "stem_stage1"),
        "resnet50_hybrid": lambda: run_net_workload(env, args, "resnet50_hybrid"),
    }
    if args.workload != "all":
        line = runners[args.workload]()
        if env.rank == 0:
            print(json.dumps(line))
        env.close()
        return

    line = runners["segnet"]()
    also = {}
    for name in ("conv", "halo", "stem_stage1", "resnet50_hybrid"):
        if name == "resnet50_hybrid" and env.world > 1 and env.world % 2:
            continue
        try:
            also[name] = compact(runners[name]())
        except Exception as e:      # keep the headline; say what failed
            also[name] = {"error": f"{type(e).__name__}: {e}"}
    if env.rank == 0:
        if env.world == 1:
            v, dt, rows, cores = cpu_conv_sample(args.cpu_seconds, **SEG_CPU_LAYER)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": f"oracle conv fwd+dgrad+wgrad of one stage-3 layer of the net (3x3, 256->256, dilation 2) on a {rows}-row x 256-col strip of one image ({dt:.1f} s)",
                                    "small_configs": cpu_small_configs()}
        conv_v = (also.get("conv") or {}).get("verify") or {}
        line["verify"] = {"ok": bool(line["verify"]["ok"] and conv_v.get("ok", False)), "net": line["verify"], "conv_step": conv_v}
        line["also"] = also
        print(json.dumps(line))
    env.close()


if __name__ == "__main__":
    main()
