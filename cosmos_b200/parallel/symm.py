"""Symmetric memory for the fused compute+collective kernels.

A `SymmGroup` owns, per process group, buffers that every rank allocates with the same size and
maps into its peers' address spaces (allocation and handle exchange by
`torch.distributed._symmetric_memory`, i.e. cuMem + POSIX-fd export over NVLink; the kernels
that read and write the peers' mappings are this package's own). It also owns the signal pads
of the group barrier: int32 words [slot][64], written with st.release.sys and polled with
ld.acquire.sys under a bounded wait (csrc/comm.cu). Epochs only grow, so pads are never reset.

On CPU (gloo tests) the same interface is backed by ordinary tensors plus `dist.barrier`, so
the host-side bookkeeping (offsets, routing tables, epochs) is exercised without a GPU.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

N_SLOTS = 64
PAD_WORDS = N_SLOTS * 64


class SymmBuffer:
    def __init__(self, local: torch.Tensor, peer_ptrs: List[int], multicast_ptr: int = 0):
        self.local = local                # uint8 view of this rank's allocation
        self.peer_ptrs = peer_ptrs        # device addresses of every rank's allocation (own included)
        self.multicast_ptr = multicast_ptr

    def view(self, offset_bytes: int, shape, dtype) -> torch.Tensor:
        n = int(torch.tensor(shape).prod().item()) * torch.empty((), dtype=dtype).element_size()
        return self.local[offset_bytes:offset_bytes + n].view(dtype).view(*shape)

    def peer_addr(self, rank: int, offset_bytes: int = 0) -> int:
        return self.peer_ptrs[rank] + offset_bytes


class SymmGroup:
    def __init__(self, group, ranks: List[int], device: torch.device):
        self.group = group
        self.ranks = ranks
        self.world = len(ranks)
        self.rank = ranks.index(dist.get_rank()) if dist.is_initialized() else 0
        self.device = device
        self.on_gpu = device.type == "cuda"
        self._epochs: Dict[int, int] = {}
        self._bufs: Dict[str, SymmBuffer] = {}
        self._meets: Dict[str, int] = {}
        self.pads = self.alloc("__pads__", PAD_WORDS * 4, zero=True)
        self.pads_dev = torch.tensor(self.pads.peer_ptrs, dtype=torch.int64, device=device)
        # Epochs of the signal slots that kernels advance themselves (CUDA-graph-safe collectives): one int32 per
        # slot, owned by the group like the pads they are compared with, so every user of a slot (a second
        # TPContext or decoder on the same ranks, an engine that is rebuilt) continues one epoch stream.
        self.counters = torch.zeros(N_SLOTS, dtype=torch.int32, device=device)
        self.barrier_host()

    # ------------------------------------------------------------------ allocation
    def alloc(self, name: str, nbytes: int, zero: bool = False) -> SymmBuffer:
        if name in self._bufs:
            if self._bufs[name].local.numel() >= nbytes:
                return self._bufs[name]
            raise ValueError(f"symmetric buffer '{name}' already exists with a smaller size")
        nbytes = (nbytes + 255) // 256 * 256
        self._meet(name)
        if self.on_gpu and self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem

            t = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
            if zero:
                t.zero_()
            hdl = symm_mem.rendezvous(t, self.group)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
            mc = int(hdl.multicast_ptr) if getattr(hdl, "multicast_ptr", 0) else 0
            buf = SymmBuffer(t, ptrs, mc)
            buf._handle = hdl  # keeps the mappings alive
        else:
            t = torch.zeros(nbytes, dtype=torch.uint8, device=self.device) if zero else \
                torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            buf = SymmBuffer(t, [t.data_ptr()] * max(self.world, 1))
        self._bufs[name] = buf
        return buf

    def _meet(self, name: str) -> None:
        """Host-side guard in front of the handle exchange: every rank of the group announces that it reached
        the allocation of `name` and waits, with a limit (COSMOS_SYMM_TIMEOUT_S, default 300 s), for the others.
        A rank that never gets here is named in a PeerFailure on the survivors instead of leaving them blocked
        inside the exchange."""
        if self.world <= 1 or not dist.is_initialized():
            return
        import os

        from torch.distributed.distributed_c10d import _get_default_store

        from .health import bounded_rendezvous
        tag = "symm/" + "-".join(str(r) for r in self.ranks) + f"/{self.device.type}/{name}/{self._meets.get(name, 0)}"
        self._meets[name] = self._meets.get(name, 0) + 1
        bounded_rendezvous(_get_default_store(), tag, self.rank, self.world,
                           float(os.environ.get("COSMOS_SYMM_TIMEOUT_S", "300")))

    # ------------------------------------------------------------------ synchronisation
    def next_epoch(self, slot: int, count: int = 1) -> int:
        e = self._epochs.get(slot, 0) + 1
        self._epochs[slot] = e + count - 1
        return e

    def barrier(self, slot: int = 0) -> None:
        """Device-side barrier on the current stream (no host synchronisation)."""
        if self.world == 1:
            return
        if self.on_gpu:
            torch.ops.cosmos_b200.comm_barrier(self.pads_dev, self.rank, self.world, slot, self.next_epoch(slot))
        else:
            dist.barrier(self.group)

    def barrier_counted(self, slot: int) -> None:
        """Device-side barrier whose epoch lives in `self.counters[slot]` (advanced by the kernel): the launch
        arguments never change, so the call may be captured in a CUDA graph. A slot is used either this way or
        through `barrier` (host-side epochs), never both."""
        if self.world == 1:
            return
        if self.on_gpu:
            torch.ops.cosmos_b200.comm_barrier_counted(self.pads_dev, self.rank, self.world, slot, self.counters)
        else:
            dist.barrier(self.group)

    def use_multicast(self, buf: "SymmBuffer") -> int:
        """NVLink multicast address of `buf` for the multimem kernels, or 0 (no mapping, or COSMOS_NVLS=0:
        plain peer loads; runs whose ranks may leave mid-job keep it off, a rank that dies while bound to a
        multicast object can fault its peers)."""
        import os
        if os.environ.get("COSMOS_NVLS", "1") == "0":
            return 0
        return int(buf.multicast_ptr or 0)

    def barrier_host(self) -> None:
        if self.world > 1 and dist.is_initialized():
            if self.on_gpu:
                torch.cuda.synchronize()
            dist.barrier(self.group)


_GROUPS: Dict[Tuple, SymmGroup] = {}


def symm_group(group, ranks: List[int], device) -> SymmGroup:
    key = (tuple(ranks), str(device))
    if key not in _GROUPS:
        _GROUPS[key] = SymmGroup(group, ranks, torch.device(device))
    return _GROUPS[key]
