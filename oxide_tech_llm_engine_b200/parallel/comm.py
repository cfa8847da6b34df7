"""Symmetric peer memory for the fused compute+collective kernels.

Every rank allocates one workspace with raw `cudaMalloc`, exports it with CUDA IPC and maps the
workspaces of all peers, so a kernel can address `ptr[rank] + offset` of any GPU directly over
NVLink. Handles travel through `torch.distributed` (object all-gather); NCCL itself is only the
bootstrap and the baseline data path. With one rank the workspace is an ordinary tensor.

The reference has no counterpart: its NcclCommunicator never calls NCCL
(oxide-backend-cuda/src/nccl.rs:18-69) and is not linked (build.rs:91-94).
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .._build import cuda_ext

_DT = {"bf16": (torch.bfloat16, 2), "f32": (torch.float32, 4), "i32": (torch.int32, 4), "u8": (torch.uint8, 1)}


class SymmetricWorkspace:
    """Named regions inside one symmetric allocation per rank."""

    def __init__(self, specs: dict[str, tuple[tuple[int, ...], str]], *, rank: int = 0, world: int = 1,
                 group=None, device: Optional[torch.device] = None):
        self.rank, self.world, self.group = rank, world, group
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.offsets: dict[str, int] = {}
        self.specs = specs
        off = 0
        for name, (shape, dt) in specs.items():
            self.offsets[name] = off
            n = int(np.prod(shape)) * _DT[dt][1]
            off += (n + 255) // 256 * 256
        self.nbytes = max(off, 256)
        self._peer_bases: list[int] = []
        self._owned = False
        ext = cuda_ext()
        if world == 1:
            self._buf = torch.zeros(self.nbytes, dtype=torch.uint8, device=self.device)
            self.base = self._buf.data_ptr()
            self._peer_bases = [self.base]
        else:
            import torch.distributed as dist

            with torch.cuda.device(self.device):
                self.base = ext.ipc_alloc(self.nbytes)
                self._owned = True
                handle = ext.ipc_get_handle(self.base)
                handles: list = [None] * world
                dist.all_gather_object(handles, handle, group=group)
                for r in range(world):
                    self._peer_bases.append(self.base if r == rank else ext.ipc_open_handle(handles[r]))
                dist.barrier(group=group)
        self._tensors: dict[str, torch.Tensor] = {}

    def local(self, name: str) -> torch.Tensor:
        if name not in self._tensors:
            shape, dt = self.specs[name]
            self._tensors[name] = cuda_ext().tensor_from_ptr(self.base + self.offsets[name], list(shape), dt,
                                                             self.device.index or 0)
        return self._tensors[name]

    def ptr(self, name: str, rank: int, byte_offset: int = 0) -> int:
        return self._peer_bases[rank] + self.offsets[name] + byte_offset

    def ptrs(self, name: str, byte_offset: int = 0) -> list[int]:
        return [self.ptr(name, r, byte_offset) for r in range(self.world)]

    def zero_(self) -> None:
        """Clears the local workspace (after an error the flag state is undefined)."""
        t = cuda_ext().tensor_from_ptr(self.base, [self.nbytes], "u8", self.device.index or 0)
        t.zero_()

    def close(self) -> None:
        if self._owned:
            ext = cuda_ext()
            torch.cuda.synchronize(self.device)
            for r, b in enumerate(self._peer_bases):
                if r != self.rank:
                    ext.ipc_close_handle(b)
            ext.ipc_free(self.base)
            self._owned = False
