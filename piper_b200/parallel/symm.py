"""Symmetric memory: buffers that every rank of a process group maps into its own address space.

``SymmetricBuffer.create(nbytes, ranks, group)`` allocates ``nbytes`` of zeroed device memory on each rank of
the group (collective call), exchanges the CUDA IPC handles through ``torch.distributed`` and maps the peers'
buffers.  ``peer_ptrs`` is a device ``int64`` tensor with one address per group rank (the local buffer for the
calling rank), ready to be handed to a kernel that reads or writes peer memory with ordinary loads and stores
over NVLink.  Typed views of the local buffer are taken with ``view(dtype, numel, offset_bytes)``.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import native


class SymmetricBuffer:
    def __init__(self, local: torch.Tensor, ptrs: list[int], my_index: int, imported: list[int]) -> None:
        self.local = local                      # uint8 tensor owning the local allocation
        self.ptrs = ptrs                        # device address of every group rank's buffer in this process
        self.my_index = my_index
        self._imported = imported
        self.peer_ptrs = torch.tensor(ptrs, dtype=torch.int64, device=local.device)

    @classmethod
    def create(cls, nbytes: int, ranks: list[int], group) -> "SymmetricBuffer":
        lib = native.lib()
        nbytes = (int(nbytes) + 255) // 256 * 256
        local = lib.symm_alloc(nbytes)
        handle = lib.symm_export(local)
        if len(ranks) == 1:
            return cls(local, [local.data_ptr()], 0, [])       # single rank: nothing to exchange
        me = dist.get_rank()
        my_index = list(ranks).index(me)
        gathered: list = [None] * len(ranks)
        dist.all_gather_object(gathered, handle.tolist(), group=group)
        ptrs, imported = [], []
        for i, h in enumerate(gathered):
            if i == my_index:
                ptrs.append(local.data_ptr())
            else:
                p = int(lib.symm_import(torch.tensor(h, dtype=torch.uint8)))
                ptrs.append(p)
                imported.append(p)
        return cls(local, ptrs, my_index, imported)

    def view(self, dtype: torch.dtype, numel: int, offset_bytes: int = 0) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        return self.local[offset_bytes:offset_bytes + numel * esz].view(dtype)

    def offset_ptrs(self, offset_bytes: int) -> torch.Tensor:
        return self.peer_ptrs + int(offset_bytes)

    def close(self) -> None:
        """Unmaps the peers' buffers (the local allocation is freed with the object)."""
        imported, self._imported = self._imported, []
        if imported:
            lib = native.lib()
            for p in imported:
                lib.symm_release(p)

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass
