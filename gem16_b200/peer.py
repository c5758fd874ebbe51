"""Buffers that every rank of a process group can address: the peer-memory plumbing under the
expert-parallel pull kernels.  torch's symmetric memory does the mapping where the driver allows
it; otherwise the buffer is shared through CUDA IPC handles.  Either way the result is a local
uint8 tensor plus, for every rank, the device address of that rank's buffer as seen from here.
Peers are only ever read with this library's own kernels (plain global loads)."""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist


class PeerBuffer:
    def __init__(self, nbytes: int, dev, group=None, how: str = "auto"):
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.nbytes = nbytes
        self._keep = []
        errors = []
        self.how = None
        if self.world == 1:
            self.local = torch.zeros((nbytes,), dtype=torch.uint8, device=dev)
            self.ptrs = [self.local.data_ptr()]
            self.how = "single"
        for method in (("symm", "ipc") if how == "auto" else (how,)):
            if self.how is not None:
                break
            try:
                getattr(self, "_" + method)(nbytes, dev, group)
                self.how = method
            except Exception as exc:   # fall through to the next method on every rank alike
                errors.append(f"{method}: {type(exc).__name__}: {exc}")
            # every rank must have taken the same path
            ok = torch.tensor([1 if self.how == method else 0], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if int(ok.item()) == 0:
                self.how = None
        if self.how is None:
            raise RuntimeError("no peer-memory path works here: " + "; ".join(errors))
        self.table = (C.c_uint64 * self.world)(*self.ptrs)   # host array for the C ABI

    def _symm(self, nbytes, dev, group):
        import torch.distributed._symmetric_memory as symm
        self.local = symm.empty(nbytes, dtype=torch.uint8, device=dev)
        self.local.zero_()
        hdl = symm.rendezvous(self.local, group if group is not None else dist.group.WORLD)
        self.ptrs = [int(p) for p in hdl.buffer_ptrs]
        self._keep.append(hdl)

    def _ipc(self, nbytes, dev, group):
        self.local = torch.zeros((nbytes,), dtype=torch.uint8, device=dev)
        handle = self.local.untyped_storage()._share_cuda_()
        handles = [None] * self.world
        dist.all_gather_object(handles, handle, group=group)
        self.ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self.local.data_ptr())
                continue
            storage = torch.UntypedStorage._new_shared_cuda(dev.index, *h[1:])
            t = torch.empty(0, dtype=torch.uint8, device=dev).set_(storage)
            self._keep.append(t)
            self.ptrs.append(t.data_ptr())


class LocalBuffer:
    """Stand-in for PeerBuffer when several ranks are emulated on one GPU: a plain device buffer whose
    table of "peer" addresses the caller fills in."""

    def __init__(self, nbytes: int, dev):
        self.local = torch.zeros((nbytes,), dtype=torch.uint8, device=dev)
        self.how = "emulated"
        self.table = None

    def set_table(self, ptrs):
        self.ptrs = list(ptrs)
        self.table = (C.c_uint64 * len(ptrs))(*ptrs)
