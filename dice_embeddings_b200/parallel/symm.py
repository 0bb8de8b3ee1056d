"""Symmetric-memory runtime: one peer-mapped heap per rank, carved into named regions.

Every rank allocates the same heap through ``torch.distributed._symmetric_memory`` (CUDA VMM + handle exchange over
the process group's store); after the rendezvous each rank holds the base address of every peer's heap, so a
region's address on rank ``r`` is ``buffer_ptrs[r] + offset``.  The kernels of this framework receive *tables* of
such addresses and talk to peer memory with plain loads, stores and ``red`` over NVLink.  Signal slots for the
device-side barrier live in the same heap.

The reference has nothing comparable: its only cross-device traffic is DDP's all-reduce and ``.to('cuda:0')``
copies (``dicee/trainer/torch_trainer_ddp.py:88``, ``dicee/models/ensemble.py:92-98``).

When the fabric supports it the heap is also bound to an NVLink multicast object (NVSwitch): ``mc_base`` is then the
multicast address of the heap, and a region's multicast address is ``mc_base + offset``.  A ``multimem.st`` to that
address stores into every rank's copy of the region and a ``multimem.ld_reduce`` returns the sum over all ranks,
formed inside the switch.  ``DICE_B200_MULTICAST=0`` (or ``multicast=False``) keeps the heap unicast-only; a rank must
never exit while its peers still issue ``multimem`` operations, so every user of the heap ends with a barrier and the
kernels stop touching peer memory once their status word holds an error.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

_ALIGN = 1024


def _nbytes(shape: Sequence[int], dtype: torch.dtype) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n * torch.empty((), dtype=dtype).element_size()


class SymmetricHeap:
    """Declare regions with :meth:`plan`, call :meth:`commit` once (collective), then use :meth:`local`,
    :meth:`peer` and :meth:`table`."""

    def __init__(self, group=None, device=None, multicast: Optional[bool] = None):
        self.group = group if group is not None else dist.group.WORLD
        self.multicast = (os.environ.get("DICE_B200_MULTICAST", "1") != "0") if multicast is None else bool(multicast)
        self.mc_base = 0
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self._plan: Dict[str, Tuple[Tuple[int, ...], torch.dtype, int]] = {}
        self._size = 0
        self._heap = None
        self._hdl = None
        self._views: Dict[Tuple[str, int], torch.Tensor] = {}

    def plan(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> None:
        assert self._heap is None, "heap already committed"
        assert name not in self._plan
        off = (self._size + _ALIGN - 1) // _ALIGN * _ALIGN
        self._plan[name] = (tuple(int(s) for s in shape), dtype, off)
        self._size = off + _nbytes(shape, dtype)

    def commit(self) -> "SymmetricHeap":
        import torch.distributed._symmetric_memory as symm_mem
        if not self.multicast:   # read by the allocator when the first block of the process is created
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        total = (self._size + _ALIGN - 1) // _ALIGN * _ALIGN
        self._heap = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        self._heap.zero_()
        self._hdl = symm_mem.rendezvous(self._heap, self.group)
        self.base_ptrs: List[int] = [int(p) for p in self._hdl.buffer_ptrs]
        mc = int(getattr(self._hdl, "multicast_ptr", 0) or 0) if (self.multicast and self.world > 1) else 0
        # every rank must take the same path: use the multicast mapping only when all of them have one
        flag = torch.tensor([1 if mc else 0], dtype=torch.int32, device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        self.mc_base = mc if int(flag.item()) == 1 else 0
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        return self

    # ------------------------------------------------------------------ access
    def _view(self, name: str, rank: int) -> torch.Tensor:
        key = (name, rank)
        if key not in self._views:
            shape, dtype, off = self._plan[name]
            esz = torch.empty((), dtype=dtype).element_size()
            if rank == self.rank:
                n = _nbytes(shape, dtype)
                t = self._heap[off:off + n].view(dtype).view(shape)
            else:
                t = self._hdl.get_buffer(rank, shape, dtype, off // esz)
            self._views[key] = t
        return self._views[key]

    def local(self, name: str) -> torch.Tensor:
        return self._view(name, self.rank)

    def peer(self, name: str, rank: int) -> torch.Tensor:
        """Tensor view of ``name`` on ``rank`` (peer memory; only pass it to kernels of this framework or copy
        from/to it — never hand it to a library GEMM)."""
        return self._view(name, rank)

    def address(self, name: str, rank: int) -> int:
        return self.base_ptrs[rank] + self._plan[name][2]

    def mc_address(self, name: str) -> int:
        """Multicast address of region ``name`` (0 when the heap has no multicast mapping)."""
        return self.mc_base + self._plan[name][2] if self.mc_base else 0

    def table(self, name: str) -> torch.Tensor:
        """Device int64 tensor with the address of region ``name`` on every rank (index = rank)."""
        return torch.tensor([self.address(name, r) for r in range(self.world)], dtype=torch.int64, device=self.device)

    def host_barrier(self) -> None:
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
