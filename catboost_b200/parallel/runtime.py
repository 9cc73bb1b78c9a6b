"""Device runtime: one process per GPU, ``torch.distributed`` for the plumbing, and a peer-mapped exchange
arena for the in-kernel collectives.

This replaces the reference's device manager (one master thread feeding a worker thread per GPU through
task queues, catboost/cuda/cuda_lib/cuda_manager.h:107, gpu_single_worker.h:33), its stripe/mirror buffers and
its host-orchestrated reduce (cuda_buffer_helpers/reduce_scatter.h).  Here every rank is an ordinary process
that owns its shard as torch tensors; the only shared object is the *arena*: a buffer of identical layout on
every rank that all peers map (``torch.distributed._symmetric_memory``; CUDA IPC handles as the fallback).
Kernels write into peers' arenas directly over NVLink:

    [mailbox payload 2 x R x mbox_bytes][mailbox tags 2 x R x u64][slot tags R x u64][slots R x slot_floats x f32]

NCCL is used for bootstrap (exchange of handles, barriers) and for the baseline reduce path only.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import List, Optional

import torch

from ..ops import native


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


@dataclass
class ArenaLayout:
    nranks: int
    mbox_bytes: int
    slot_floats: int

    @property
    def off_mbox(self):
        return 0

    @property
    def off_mbox_flag(self):
        return _align(2 * self.nranks * self.mbox_bytes)

    @property
    def off_slot_flag(self):
        return self.off_mbox_flag + _align(2 * self.nranks * 8)

    @property
    def off_slots(self):
        return self.off_slot_flag + _align(self.nranks * 8)

    @property
    def total_bytes(self):
        return self.off_slots + _align(self.nranks * self.slot_floats * 4)


class DistContext:
    """Rank / world bookkeeping.  ``DistContext.current()`` reflects torch.distributed when it is initialised
    (torchrun or the launcher of this package), else a single-rank context."""

    def __init__(self, rank: int = 0, world: int = 1, device: Optional[torch.device] = None, group=None):
        self.rank, self.world, self.device, self.group = rank, world, device, group

    @staticmethod
    def current(device=None) -> "DistContext":
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            return DistContext(dist.get_rank(), dist.get_world_size(), device, dist.group.WORLD)
        return DistContext(0, 1, device, None)

    @property
    def is_distributed(self):
        return self.world > 1

    @property
    def single_host(self) -> bool:
        """True when every rank runs on the same machine (peer-mapped memory is only possible then).  Ranks on several
        machines (torchrun --nnodes > 1) train with the NCCL reduction path instead of the peer arena."""
        if not self.is_distributed:
            return True
        cached = getattr(self, "_single_host", None)
        if cached is None:
            import socket
            names = self.all_gather_object(socket.gethostname() + ":" + os.environ.get("GROUP_RANK", "0"))
            cached = self._single_host = len(set(names)) == 1
        return cached

    def barrier(self):
        if self.is_distributed:
            import torch.distributed as dist
            if self.device is not None and self.device.type == "cuda":
                dist.barrier(device_ids=[self.device.index])
            else:
                dist.barrier()

    def all_reduce_sum_(self, t: torch.Tensor):
        if self.is_distributed:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t

    def all_gather_object(self, obj):
        if not self.is_distributed:
            return [obj]
        import torch.distributed as dist
        out = [None] * self.world
        dist.all_gather_object(out, obj, group=self.group)
        return out

    def gather_rows(self, arr, dst: int = 0):
        """The rows of every rank's 2-D numpy array, concatenated in rank order, on rank ``dst`` (None elsewhere).
        Goes through tensor collectives (padded to the longest piece), not through pickled objects."""
        import numpy as np
        if not self.is_distributed:
            return arr
        import torch.distributed as dist
        counts = self.all_gather_object(int(arr.shape[0]))
        m = max(max(counts), 1)
        on_gpu = dist.get_backend(self.group) == "nccl"
        dev = self.device if (on_gpu and self.device is not None) else torch.device("cpu")
        t = torch.zeros((m,) + tuple(arr.shape[1:]), dtype=torch.from_numpy(arr[:0]).dtype)
        t[: arr.shape[0]] = torch.from_numpy(np.ascontiguousarray(arr))
        t = t.to(dev)
        if self.rank == dst:
            outs = [torch.empty_like(t) for _ in range(self.world)]
            dist.gather(t, outs, dst=dst, group=self.group)
            return np.concatenate([outs[r][: counts[r]].cpu().numpy() for r in range(self.world)], 0)
        dist.gather(t, None, dst=dst, group=self.group)
        return None

    def broadcast_object(self, obj, src=0):
        if not self.is_distributed:
            return obj
        import torch.distributed as dist
        box = [obj]
        dist.broadcast_object_list(box, src=src, group=self.group)
        return box[0]


class PeerArena:
    """The exchange arena of this rank plus the addresses of every peer's arena in this process."""

    def __init__(self, ctx: DistContext, layout: ArenaLayout, timeout_s: float = 5.0):
        self.ctx, self.layout = ctx, layout
        dev = ctx.device
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)
        self.epoch = torch.zeros(2, dtype=torch.int64, device=dev)
        self._keep = []
        self.kind = "local"
        nbytes = layout.total_bytes
        if ctx.world == 1:
            self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
            self.peer_ptrs = [self.buf.data_ptr()]
        else:
            self.buf, self.peer_ptrs = self._map_peers(nbytes)
        self.handle = self._create_comm(timeout_s)
        ctx.barrier()

    # -- peer mapping -----------------------------------------------------------------------------------
    def _map_peers(self, nbytes):
        ctx = self.ctx
        err = None
        if os.environ.get("CB200_ARENA", "symm") == "symm":
            try:
                import torch.distributed._symmetric_memory as symm
                buf = symm.empty(nbytes, dtype=torch.uint8, device=ctx.device)
                hdl = symm.rendezvous(buf, group=ctx.group)
                buf.zero_()
                ptrs = [int(p) for p in hdl.buffer_ptrs]
                self._keep.append(hdl)
                self.kind = "symmetric_memory"
                torch.cuda.synchronize(ctx.device)
                return buf, ptrs
            except Exception as e:  # pragma: no cover - depends on the box
                err = e
        # CUDA IPC fallback: share the storage handle, open the peers' storages
        buf = torch.zeros(nbytes, dtype=torch.uint8, device=ctx.device)
        torch.cuda.synchronize(ctx.device)
        try:
            shared = buf.untyped_storage()._share_cuda_()
            handles = ctx.all_gather_object(shared)
            ptrs = []
            for r, h in enumerate(handles):
                if r == ctx.rank:
                    ptrs.append(buf.data_ptr())
                    continue
                (dev_idx, handle, size_bytes, offset_bytes, ref_h, ref_off, ev_h, ev_sync) = h
                st = torch.UntypedStorage._new_shared_cuda(ctx.device.index, handle, size_bytes, offset_bytes, ref_h,
                                                           ref_off, ev_h, ev_sync)
                self._keep.append(st)
                ptrs.append(st.data_ptr())
            self.kind = "cuda_ipc"
            return buf, ptrs
        except Exception as e2:  # pragma: no cover
            raise RuntimeError(f"cannot map peer memory: symmetric memory failed with {err!r}; CUDA IPC failed with {e2!r}")

    def _create_comm(self, timeout_s):
        L, R = self.layout, self.ctx.world
        arr = ctypes.c_void_p * R
        mbox = arr(*[p + L.off_mbox for p in self.peer_ptrs])
        mflag = arr(*[p + L.off_mbox_flag for p in self.peer_ptrs])
        slot = arr(*[p + L.off_slots for p in self.peer_ptrs])
        sflag = arr(*[p + L.off_slot_flag for p in self.peer_ptrs])
        h = native.cuda_lib().cb_comm_create(self.ctx.rank, R, int(timeout_s * 1e9),
                                             ctypes.c_void_p(self.status.data_ptr()),
                                             ctypes.c_void_p(self.epoch.data_ptr()), mbox, mflag, L.mbox_bytes, slot,
                                             sflag, L.slot_floats)
        if not h:
            raise RuntimeError("cb_comm_create failed")
        return h

    def local_slot_ptr(self, src_rank: int) -> int:
        return self.peer_ptrs[self.ctx.rank] + self.layout.off_slots + src_rank * self.layout.slot_floats * 4

    def local_slots_tensor(self) -> torch.Tensor:
        L = self.layout
        return self.buf[L.off_slots: L.off_slots + self.ctx.world * L.slot_floats * 4].view(torch.float32)

    def check_status(self):
        """Raise if a device-side wait timed out (the kernels never hang or trap; they flag and carry on)."""
        st = self.status.cpu().tolist()
        if st[0] != 0:
            what = {1: "peer histogram push", 2: "mailbox message", 3: "bad argument"}.get(st[0], "unknown")
            raise RuntimeError(f"rank {self.ctx.rank}: device-side wait for {what} from rank {st[1]} timed out; "
                               f"a peer has failed or fallen behind")

    def close(self):
        if self.handle:
            native.cuda_lib().cb_comm_destroy(ctypes.c_void_p(self.handle))
            self.handle = 0

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


def split_columns(feat_off, nranks: int):
    """Contiguous feature ranges per rank, balanced by histogram columns.
    Returns (feature boundaries [R+1], column boundaries [R+1])."""
    F = len(feat_off) - 1
    total = int(feat_off[-1])
    fb = [0]
    for r in range(1, nranks):
        target = total * r / nranks
        f = fb[-1]
        while f < F and feat_off[f + 1] <= target:
            f += 1
        # pick the nearer boundary
        if f < F and abs(feat_off[f + 1] - target) < abs(feat_off[f] - target):
            f += 1
        fb.append(max(f, fb[-1]))
    fb.append(F)
    cb = [int(feat_off[f]) for f in fb]
    return fb, cb
