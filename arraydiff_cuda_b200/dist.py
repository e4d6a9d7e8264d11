"""One-process-per-GPU plumbing: a symmetric device arena per rank, mapped into every peer
through CUDA IPC, with torch.distributed used only to pass the handles around.

The reference is a single process that owns all GPUs and simply dereferences peer pointers
(src/spatial.cc:13-50).  Launched one rank per GPU, each rank instead allocates ONE arena,
publishes its IPC handle, and sub-allocates every halo buffer and flag word at the same offset
on every rank; a peer's copy of a buffer is then `peer_base[r] + offset`.
"""
import ctypes as C

import numpy as np

from . import abi


class _Raw:
    """Exposes a raw device pointer to torch through __cuda_array_interface__."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class SymmetricArena:
    def __init__(self, nbytes, rank=0, world=1, group=None):
        import torch
        self.rank, self.world, self.nbytes = rank, world, int(nbytes)
        L = abi.lib()
        p = C.c_void_p()
        abi.check(L.ad_device_malloc(self.nbytes, C.byref(p)), "arena allocation")
        self.base = p.value
        self.bytes = torch.as_tensor(_Raw(self.base, self.nbytes), device=f"cuda:{torch.cuda.current_device()}")
        self.bytes.zero_()
        self.offset = 0
        self.peer_base = [None] * world
        self.peer_base[rank] = self.base
        self._opened = []
        if world > 1:
            import torch.distributed as dist
            h = C.create_string_buffer(64)
            abi.check(L.ad_ipc_get_handle(C.c_void_p(self.base), h), "ipc handle")
            mine = torch.from_numpy(np.frombuffer(h.raw, dtype=np.uint8).copy()).cuda()
            allh = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(allh, mine, group=group)
            for r in range(world):
                if r == rank:
                    continue
                q = C.c_void_p()
                abi.check(L.ad_ipc_open_handle(bytes(allh[r].cpu().numpy().tobytes()), C.byref(q)), f"open arena of rank {r}")
                self.peer_base[r] = q.value
                self._opened.append(q.value)
            dist.barrier(group=group)

    def alloc(self, shape, dtype, align=1024):
        """Same call sequence on every rank => same offsets on every rank."""
        import torch
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        self.offset = (self.offset + align - 1) // align * align
        if self.offset + n > self.nbytes:
            raise MemoryError("symmetric arena exhausted")
        t = self.bytes[self.offset:self.offset + n].view(dtype).view(*shape)
        off = self.offset
        self.offset += n
        return t, off

    def peers(self, offset):
        """Pointer to the same allocation on every rank (usable from this rank's kernels)."""
        return [b + offset for b in self.peer_base]

    def close(self):
        L = abi.lib()
        for q in self._opened:
            L.ad_ipc_close_handle(C.c_void_p(q))
        self._opened = []
        self.bytes = None
        L.ad_device_free(C.c_void_p(self.base))
