"""Host side of the mirrored-destination path (see ruyb200_mul_async_mirrored): buffers that every rank of a
torch.distributed job can store into, and the flag exchange that ends a step.

One process per GPU.  `PeerBuffer(nbytes)` allocates the same-sized buffer on every rank, exchanges the IPC
handles through the process group (an object all-gather on the host), and maps every peer's buffer into this
process.  Only stores go to a peer's memory (the kernel's epilogue and the flag writes); nothing loads from it."""
import ctypes as C

import torch
import torch.distributed as dist

from ._lib import lib
from .api import _check, make_desc


class _RawCuda:
    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class PeerBuffer:
    def __init__(self, nbytes, device):
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.nbytes = nbytes
        p = C.c_void_p()
        _check(lib().ruyb200_peer_alloc(nbytes, C.byref(p)), "ruyb200_peer_alloc")
        self.local_ptr = p.value
        handle = C.create_string_buffer(64)
        _check(lib().ruyb200_peer_export(self.local_ptr, handle), "ruyb200_peer_export")
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw)
        self.ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self.local_ptr)
            else:
                q = C.c_void_p()
                _check(lib().ruyb200_peer_open(h, C.byref(q)), "ruyb200_peer_open")
                self.ptrs.append(q.value)
        self.tensor = torch.as_tensor(_RawCuda(self.local_ptr, nbytes), device=device)   # uint8 view of the local buffer

    def close(self):
        torch.cuda.synchronize()
        dist.barrier()
        for r, p in enumerate(self.ptrs):
            if r != self.rank and p:
                lib().ruyb200_peer_close(p)
        dist.barrier()
        if self.local_ptr:
            lib().ruyb200_peer_free(self.local_ptr)
            self.local_ptr = None


class MulticastBuffer:
    """The same-sized buffer on every rank plus an NVLink multicast mapping bound to all of them: one store to
    `multicast_ptr + offset` lands at `offset` in every rank's buffer.  Allocation, handle exchange and binding are
    torch's symmetric memory (plumbing); raises RuntimeError where the platform offers no multicast mapping, and the
    caller falls back to PeerBuffer."""

    def __init__(self, nbytes, device):
        import torch.distributed._symmetric_memory as symm_mem
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.nbytes = nbytes
        self.tensor = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, dist.group.WORLD.group_name)
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        if not self.multicast_ptr:
            raise RuntimeError("no multicast mapping on this platform")
        self.local_ptr = self.tensor.data_ptr()
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]

    def close(self):
        # the mapping must stay bound until every rank is done with it
        torch.cuda.synchronize()
        dist.barrier()
        self.handle = None
        self.tensor = None
        dist.barrier()


class StepFlags:
    """flags[r] on every rank is raised by rank r at the end of its step; a rank's step is over when all are up."""

    def __init__(self, device):
        self.buf = PeerBuffer(256, device)
        w, r = self.buf.world, self.buf.rank
        targets = torch.tensor([p + 4 * r for p in self.buf.ptrs], dtype=torch.int64, device=device)
        self.targets = targets          # device array of addresses: flags[r] in every rank's buffer (own included)
        self.world = w

    def signal_and_wait(self, ctx, value):
        _check(lib().ruyb200_peer_exchange(ctx._h, C.c_void_p(self.targets.data_ptr()), C.c_void_p(self.buf.local_ptr), self.world,
                                           value), "ruyb200_peer_exchange")

    def close(self):
        self.buf.close()


def mul_async_mirrored(lhs, rhs, mul_params, context, dst, mirror_ptrs, flags=None, value=0):
    """The mul whose epilogue also stores into `mirror_ptrs`; with `flags` (a StepFlags) the launch ends with the
    step's flag exchange (raise this rank's flag on every rank to `value`, wait for everybody's)."""
    d = make_desc(lhs, rhs, mul_params, dst)
    arr = (C.c_void_p * max(1, len(mirror_ptrs)))(*mirror_ptrs)
    if flags is None:
        _check(lib().ruyb200_mul_async_mirrored(context._h, C.byref(d), arr, len(mirror_ptrs)), "ruyb200_mul_async_mirrored")
    else:
        _check(lib().ruyb200_mul_async_mirrored_exchange(context._h, C.byref(d), arr, len(mirror_ptrs),
                                                         C.c_void_p(flags.targets.data_ptr()), C.c_void_p(flags.buf.local_ptr),
                                                         flags.world, value), "ruyb200_mul_async_mirrored_exchange")


def mul_async_multicast(lhs, rhs, mul_params, context, dst, multicast_ptr, flags, value):
    """The mul whose epilogue stores every piece of the destination once, to `multicast_ptr` (the address of dst in a
    MulticastBuffer's mapping), and whose launch ends with the step's flag exchange."""
    d = make_desc(lhs, rhs, mul_params, dst)
    _check(lib().ruyb200_mul_async_multicast_exchange(context._h, C.byref(d), C.c_void_p(multicast_ptr),
                                                      C.c_void_p(flags.targets.data_ptr()), C.c_void_p(flags.buf.local_ptr),
                                                      flags.world, value), "ruyb200_mul_async_multicast_exchange")
