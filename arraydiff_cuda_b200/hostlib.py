"""ctypes view of the C entry points of the C++ host layer (host/src/capi.cc): contexts, nets,
forward / backward / update with host tensors.  Plumbing for tests and the benchmark."""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libarraydiff_host.so")
F32_NCHW, BF16_NHWC = 0, 1
_lib = None


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing -- build it with `python -m arraydiff_cuda_b200.host.build`")
        from . import abi
        abi.load()  # the kernel library must be resident first
        L = C.CDLL(LIB_PATH)
        vp = C.c_void_p
        L.adh_context_create.restype = vp
        L.adh_context_create.argtypes = [C.POINTER(C.c_int), C.c_int, C.c_int, C.c_size_t]
        L.adh_context_create_distributed.restype = vp
        L.adh_context_create_distributed.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_size_t]
        L.adh_context_destroy.argtypes = [vp]
        L.adh_context_arena_handle.argtypes = [vp, C.c_char_p]
        L.adh_context_set_peer_handle.argtypes = [vp, C.c_int, C.c_char_p]
        L.adh_context_set_allreduce_hook.argtypes = [vp, vp, vp]
        L.adh_context_set_world.argtypes = [vp, C.c_int, C.c_int]
        L.adh_context_set_world_peer_handle.argtypes = [vp, C.c_int, C.c_char_p]
        L.adh_context_set_world_peer_from_group.argtypes = [vp, C.c_int, C.c_int]
        L.adh_context_halo2d.argtypes = [vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int] + [C.c_uint32] * 5 + [C.POINTER(vp)]
        L.adh_context_stream.restype = vp
        L.adh_context_stream.argtypes = [vp, C.c_int]
        L.adh_net_create.restype = vp
        L.adh_net_create.argtypes = [vp, C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint64]
        L.adh_net_destroy.argtypes = [vp]
        L.adh_net_configure_sgd.argtypes = [vp, C.c_double, C.c_double, C.c_double, C.c_int]
        L.adh_net_param_manifest.restype = C.c_size_t
        L.adh_net_param_manifest.argtypes = [vp, C.c_char_p, C.c_size_t]
        L.adh_net_param_count.restype = C.c_size_t
        L.adh_net_param_count.argtypes = [vp]
        for name in ("adh_net_get_params", "adh_net_get_output", "adh_net_set_output_grad", "adh_net_get_param_grads",
                     "adh_net_get_input_grad"):
            getattr(L, name).argtypes = [vp, C.c_int, vp]
        L.adh_net_set_params.argtypes = [vp, vp]
        L.adh_net_output_dims.argtypes = [vp, C.POINTER(C.c_int)]
        L.adh_net_forward.argtypes = [vp, vp]
        L.adh_net_load_input.argtypes = [vp, vp]
        L.adh_net_step_resident.argtypes = [vp, C.c_int]
        L.adh_net_set_labels.argtypes = [vp, C.c_int, vp]
        L.adh_net_set_loss_weight.argtypes = [vp, C.c_float]
        L.adh_net_loss.argtypes = [vp, C.POINTER(C.c_double), C.POINTER(C.c_uint64)]
        L.adh_net_get_output_grad.argtypes = [vp, C.c_int, vp]
        L.adh_net_step_graph.argtypes = [vp, C.c_int]
        L.adh_net_graph_launches.restype = C.c_uint64
        L.adh_net_graph_launches.argtypes = [vp]
        for name in ("adh_net_backward", "adh_net_sgd_step", "adh_net_sync", "adh_net_status"):
            getattr(L, name).argtypes = [vp]
        L.adh_net_save_checkpoint.argtypes = [vp, C.c_char_p]
        L.adh_net_load_checkpoint.argtypes = [vp, C.c_char_p]
        L.adh_net_broadcast_params.argtypes = [vp]
        L.adh_net_iteration.restype = C.c_size_t
        L.adh_net_iteration.argtypes = [vp]
        L.adh_net_arena_used.restype = C.c_size_t
        L.adh_net_arena_used.argtypes = [vp, C.c_int]
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


class Context:
    def __init__(self, devices, mode=F32_NCHW, arena_mb=1024):
        self.L = load()
        arr = (C.c_int * len(devices))(*devices)
        self.h = self.L.adh_context_create(arr, len(devices), mode, arena_mb)
        self.num_ranks = len(devices)

    def halo2d(self, grid_w, grid_h, reduce, bufs, nhwc, bf16, p, w, h, ch, n):
        """Spatial2DComm group call on a grid_h x grid_w grid over this context's ranks; bufs: device pointers."""
        arr = (C.c_void_p * len(bufs))(*bufs)
        assert self.L.adh_context_halo2d(self.h, grid_w, grid_h, int(reduce), int(nhwc), int(bf16), p, w, h, ch, n, arr) == 0

    def close(self):
        if self.h:
            self.L.adh_context_destroy(self.h)
            self.h = None


class Net:
    """kind: 'conv3x3', 'stem_stage1', 'parallel_resnet18', 'parallel_resnet50', 'segnet50' or 'segnet_small' (one block per stage; `filters` = stem width)."""

    def __init__(self, ctx, kind, H, W, Cin, batch=1, filters=64, seed=1):
        self.L, self.ctx = ctx.L, ctx
        self.h = self.L.adh_net_create(ctx.h, kind.encode(), H, W, Cin, batch, filters, seed)
        if not self.h:
            raise ValueError(kind)
        self.in_shape = (batch, Cin, H, W)
        d = (C.c_int * 4)()
        self.L.adh_net_output_dims(self.h, d)
        self.strip_shape = tuple(d)
        self.nparam = self.L.adh_net_param_count(self.h)

    def manifest(self):
        n = self.L.adh_net_param_manifest(self.h, None, 0)
        buf = C.create_string_buffer(n + 1)
        self.L.adh_net_param_manifest(self.h, buf, n + 1)
        out = {}
        for line in buf.value.decode().splitlines():
            name, off, size = line.split()
            out[name] = (int(off), int(size))
        return out

    def params(self, rank=0):
        a = np.empty(self.nparam, np.float32)
        self.L.adh_net_get_params(self.h, rank, _p(a))
        return a

    def set_params(self, flat):
        flat = np.ascontiguousarray(flat, np.float32)
        self.L.adh_net_set_params(self.h, _p(flat))

    def forward(self, x):
        x = np.ascontiguousarray(x, np.float32)
        assert x.shape == self.in_shape
        self.L.adh_net_forward(self.h, _p(x))

    def load_input(self, x):
        """Host image -> the local ranks' input buffers, without evaluating anything: the next step_resident() /
        step_graph() runs on it."""
        x = np.ascontiguousarray(x, np.float32)
        assert x.shape == self.in_shape
        assert self.L.adh_net_load_input(self.h, _p(x)) == 0

    def output(self, rank, out=None):
        """`out`: a float32 array of strip_shape to fill (e.g. in pinned memory) instead of a fresh one"""
        a = np.empty(self.strip_shape, np.float32) if out is None else out
        assert a.shape == self.strip_shape and a.dtype == np.float32 and a.flags.c_contiguous
        assert self.L.adh_net_get_output(self.h, rank, _p(a)) == 0
        return a

    def full_output(self):
        return np.concatenate([self.output(r) for r in range(self.ctx.num_ranks)], axis=2)

    def set_output_grad(self, rank, dy):
        dy = np.ascontiguousarray(dy, np.float32)
        assert dy.shape == self.strip_shape
        assert self.L.adh_net_set_output_grad(self.h, rank, _p(dy)) == 0

    def backward(self):
        self.L.adh_net_backward(self.h)

    def set_labels(self, rank, labels):
        """uint32 [N][h][W] labels of `rank`'s strip (nets that end in the per-pixel loss)"""
        labels = np.ascontiguousarray(labels, np.uint32)
        assert labels.shape == (self.strip_shape[0],) + self.strip_shape[2:]
        assert self.L.adh_net_set_labels(self.h, rank, _p(labels)) == 0

    def set_loss_weight(self, w):
        assert self.L.adh_net_set_loss_weight(self.h, w) == 0

    def loss(self):
        """(sum of the per-pixel losses over the local strips, pixels behind it) of the last forward"""
        s, n = C.c_double(), C.c_uint64()
        assert self.L.adh_net_loss(self.h, C.byref(s), C.byref(n)) == 0
        return s.value, n.value

    def output_grad(self, rank):
        a = np.empty(self.strip_shape, np.float32)
        assert self.L.adh_net_get_output_grad(self.h, rank, _p(a)) == 0
        return a

    def param_grads(self, rank):
        a = np.empty(self.nparam, np.float32)
        self.L.adh_net_get_param_grads(self.h, rank, _p(a))
        return a

    def input_grad(self, rank):
        a = np.empty(self.in_shape, np.float32)
        assert self.L.adh_net_get_input_grad(self.h, rank, _p(a)) == 0
        return a

    def configure_sgd(self, step_size, momentum, l2=0.0, nesterov=False):
        self.L.adh_net_configure_sgd(self.h, step_size, momentum, l2, int(nesterov))

    def step_resident(self, with_update=True):
        """forward + backward (+ allreduce and SGD) on the image and output gradients already on the device"""
        self.L.adh_net_step_resident(self.h, int(with_update))

    def step_graph(self, with_update=True):
        """the resident step replayed from a CUDA graph (recorded on the first call)"""
        assert self.L.adh_net_step_graph(self.h, int(with_update)) == 0

    def graph_launches(self):
        """kernels one graph replay launches"""
        return int(self.L.adh_net_graph_launches(self.h))

    def save_checkpoint(self, path):
        """parameters, momentum, running statistics and the iteration counter -> one file (format: optimize.hh)"""
        assert self.L.adh_net_save_checkpoint(self.h, str(path).encode()) == 0

    def load_checkpoint(self, path):
        return self.L.adh_net_load_checkpoint(self.h, str(path).encode()) == 0

    def iteration(self):
        return int(self.L.adh_net_iteration(self.h))

    def broadcast_params(self):
        """one process per GPU: worker 0's parameters become everyone's"""
        assert self.L.adh_net_broadcast_params(self.h) == 0

    def sgd_step(self):
        self.L.adh_net_sgd_step(self.h)

    def sync(self):
        self.L.adh_net_sync(self.h)

    def status(self):
        return self.L.adh_net_status(self.h)

    def close(self):
        if self.h:
            self.L.adh_net_destroy(self.h)
            self.h = None


def read_checkpoint(path):
    """Parses a checkpoint file written by Net.save_checkpoint (layout documented in host/include/arraydiff/optimize.hh):
    returns dict(version, param_dim, stat_dim, iteration, manifest={name: (offset, size)}, params, momentum, stats)."""
    import struct
    with open(path, "rb") as f:
        raw = f.read()
    assert raw[:8] == b"ADB2CKPT", "not a checkpoint file"
    version, pd, sd, it, n = struct.unpack_from("<IQQQI", raw, 8)
    pos = 8 + 4 + 8 * 3 + 4
    man = {}
    for _ in range(n):
        (ln,) = struct.unpack_from("<I", raw, pos)
        pos += 4
        name = raw[pos:pos + ln].decode()
        pos += ln
        off, size = struct.unpack_from("<QQ", raw, pos)
        pos += 16
        man[name] = (off, size)
    theta = np.frombuffer(raw, np.float32, pd, pos)
    mom = np.frombuffer(raw, np.float32, pd, pos + 4 * pd)
    stats = np.frombuffer(raw, np.float32, sd, pos + 8 * pd)
    assert pos + 8 * pd + 4 * sd == len(raw), "trailing or missing bytes"
    return dict(version=version, param_dim=pd, stat_dim=sd, iteration=it, manifest=man, params=theta, momentum=mom, stats=stats)
