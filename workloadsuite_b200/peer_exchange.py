"""All-gather of per-rank fp32 blocks through NVLink peer memory (``ssd_b200_xchg_*`` of ``include/ssd_b200.h``).

One process per GPU on one node.  The ranks' receive buffers are plain ``cudaMalloc`` memory opened by the other
ranks through CUDA IPC handles, which travel once through ``torch.distributed.all_gather_object``; afterwards an
exchange is one kernel launch per rank (peer stores and system-scope flags, every wait bounded) and can be
captured into a CUDA graph.  The reference has no multi-GPU path; the blocks exchanged here are the operands of
``fold_states`` (``model_ref.py:152-157`` applied across shards).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from . import _lib


class _DevicePointer:
    """Minimal ``__cuda_array_interface__`` holder so that torch can view memory this library allocated."""

    def __init__(self, ptr: int, numel: int):
        self.__cuda_array_interface__ = {"shape": (numel,), "typestr": "<f4", "data": (ptr, False), "version": 3,
                                         "strides": None}


class PeerExchange:
    """``all_gather(send)`` writes this rank's ``numel`` floats into slot ``rank`` of every rank's ``recv``
    (float32 ``[world, slot]`` on this rank's device, ``slot >= numel`` rounded up to 4 floats) and returns once all
    ranks' blocks have arrived here.  Collective: every rank constructs it and calls it the same number of times."""

    def __init__(self, numel: int, group: Optional[dist.ProcessGroup] = None, device=None, wait_limit_ms: int = 0):
        if not torch.cuda.is_available():
            raise RuntimeError("PeerExchange needs CUDA devices (there is no CPU path)")
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.numel = int(numel)
        self.slot = (self.numel + 3) // 4 * 4
        self.wait_limit_ms = int(wait_limit_ms)
        self._lib = _lib.load()
        self._ctx = C.c_void_p()
        handle = (C.c_ubyte * _lib.XCHG_HANDLE_BYTES)()
        with torch.cuda.device(self.device):
            rc = self._lib.ssd_b200_xchg_create(self.slot * 4, self.world, C.byref(self._ctx), handle)
        ok = torch.tensor([1 if rc == _lib.SSD_OK else 0], device=self.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok.item()) == 0:
            self.close(collective=False)
            raise RuntimeError(f"ssd_b200_xchg_create failed on some rank (here: {_lib.strerror(rc) if rc else 'ok'})")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        blob = b"".join(handles)
        with torch.cuda.device(self.device):
            rc = self._lib.ssd_b200_xchg_connect(self._ctx, blob, self.rank)
        ok = torch.tensor([1 if rc == _lib.SSD_OK else 0], device=self.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)     # (also: every buffer is zeroed before anyone writes)
        if int(ok.item()) == 0:
            dist.barrier(group=group)
            self.close(collective=False)
            raise RuntimeError("the ranks could not open each other's device buffers (CUDA IPC): "
                               f"{_lib.strerror(rc) if rc else 'failed on another rank'}")
        ptr = self._lib.ssd_b200_xchg_buffer(self._ctx)
        self.recv = torch.as_tensor(_DevicePointer(ptr, self.world * self.slot), device=self.device).view(
            self.world, self.slot)

    def all_gather(self, send: torch.Tensor, status: Optional[torch.Tensor] = None) -> torch.Tensor:
        if send.device != self.device or send.dtype != torch.float32 or not send.is_contiguous():
            raise ValueError("send must be a contiguous float32 tensor on this rank's device")
        if send.numel() != self.slot and send.numel() != self.numel:
            raise ValueError(f"send has {send.numel()} elements, the exchange was built for {self.numel}")
        nbytes = send.numel() * 4
        if nbytes % 16 or send.data_ptr() % 16:
            raise ValueError("send must be 16-byte aligned and a multiple of 16 bytes long (pad to 4 floats)")
        with torch.cuda.device(self.device):
            rc = self._lib.ssd_b200_xchg_all_gather(self._ctx, send.data_ptr(), nbytes,
                                                    None if status is None else status.data_ptr(),
                                                    self.wait_limit_ms, torch.cuda.current_stream().cuda_stream)
        if rc != _lib.SSD_OK:
            raise RuntimeError(f"ssd_b200_xchg_all_gather: {_lib.strerror(rc)}")
        return self.recv

    def close(self, collective: bool = True):
        """Unmaps the peers' buffers and frees this rank's.  Collective by default: no rank frees its buffer while
        another may still be writing to it.  (A process that simply exits leaves the clean-up to the driver.)"""
        if getattr(self, "_ctx", None) is not None and self._ctx.value:
            with torch.cuda.device(self.device):
                torch.cuda.synchronize(self.device)
                if collective and self.world > 1 and getattr(self, "recv", None) is not None:
                    dist.barrier(group=self.group)
                self._lib.ssd_b200_xchg_destroy(self._ctx)
            self._ctx = C.c_void_p()
            self.recv = None
