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

    def close(self, barrier=None):
        """Unmap the peers' arenas, then free this rank's.  `barrier` (a callable every rank runs) keeps a
        rank from freeing memory a peer still has mapped or is still writing: it is called before the unmapping
        and again before the free."""
        L = abi.lib()
        if barrier:
            barrier()
        for q in self._opened:
            L.ad_ipc_close_handle(C.c_void_p(q))
        self._opened = []
        self.bytes = None
        if barrier:
            barrier()
        L.ad_device_free(C.c_void_p(self.base))


class HaloPlan:
    """Who talks to whom for one rank of a 1 x R strip grid, and over which flag words.

    Every rank owns four 64-bit flag words at the same arena offset:
        0 from_prev   set by rank-1 when its rows have landed in my top halo
        1 from_next   set by rank+1 when its rows have landed in my bottom halo
        2 grad_prev   set by rank-1 when its halo-gradient rows are final (I may pull them)
        3 grad_next   set by rank+1 likewise
    Epochs only grow; nothing is ever reset.  This is the host logic that replaces the epoch
    rendez-vous of Spatial2DComm::group_end (reference src/spatial.cc:58-70)."""
    FROM_PREV, FROM_NEXT, GRAD_PREV, GRAD_NEXT = 0, 1, 2, 3

    def __init__(self, rank, world):
        if not (1 <= world <= 8) or not (0 <= rank < world):
            raise ValueError("rank/world out of range (1 x R grid, R <= 8)")
        self.rank, self.world = rank, world
        self.prev = rank - 1 if rank > 0 else None
        self.next = rank + 1 if rank + 1 < world else None

    def exchange_signals(self):
        """(peer rank, flag slot on that peer) pairs this rank sets after pushing its edge rows."""
        out = []
        if self.next is not None:
            out.append((self.next, self.FROM_PREV))
        if self.prev is not None:
            out.append((self.prev, self.FROM_NEXT))
        return out

    def exchange_waits(self):
        """Own flag slots this rank waits on before reading its halo rows."""
        return ([self.FROM_PREV] if self.prev is not None else []) + ([self.FROM_NEXT] if self.next is not None else [])

    def reduce_signals(self):
        out = []
        if self.next is not None:
            out.append((self.next, self.GRAD_PREV))
        if self.prev is not None:
            out.append((self.prev, self.GRAD_NEXT))
        return out

    def reduce_waits(self):
        return ([self.GRAD_PREV] if self.prev is not None else []) + ([self.GRAD_NEXT] if self.next is not None else [])

    def push_rows(self, p, h):
        """(peer, my first source row, peer's first destination row) for the forward push; rows are
        indices into the padded strip (height h + 2p)."""
        out = []
        if self.next is not None:
            out.append((self.next, h, 0))
        if self.prev is not None:
            out.append((self.prev, p, p + h))
        return out

    def pull_rows(self, p, h):
        """(peer, peer's first halo row, my first interior row) for the backward accumulate."""
        out = []
        if self.next is not None:
            out.append((self.next, 0, h))
        if self.prev is not None:
            out.append((self.prev, p + h, p))
        return out
