"""Device memory for kernels written in the kernel language (zse-compiler/zse_compiler/runtime/memory.py:12-527: raw
``cuMemAlloc`` / copies / pinned host memory / streams through the driver API).

Here storage comes from torch's caching allocator, so it can be shared freely with the rest of the engine, copies
are stream-ordered torch copies, and pinned buffers are torch pinned tensors.  Without a GPU the same calls work on
CPU tensors, which is what the emulator consumes."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import numpy as np
import torch

from . import dtypes
from .dtypes import DType, Tensor


class GPUMemory:
    def __init__(self, device: Optional[object] = None):
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        self._live: Dict[int, int] = {}            # data_ptr -> bytes, for the accounting below
        self._allocated = 0
        self._peak = 0

    def ensure_context(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.init()
            torch.cuda.set_device(self.device)

    # ---- allocation -------------------------------------------------------------------------------------------
    def _track(self, t: Tensor) -> Tensor:
        self._live[t.data_ptr] = t.nbytes
        self._allocated += t.nbytes
        self._peak = max(self._peak, self._allocated)
        return t

    def allocate(self, shape: Tuple[int, ...], dtype: DType = dtypes.float32) -> Tensor:
        return self._track(dtypes.empty(shape, dtype, self.device))

    def zeros(self, shape: Tuple[int, ...], dtype: DType = dtypes.float32) -> Tensor:
        return self._track(dtypes.zeros(shape, dtype, self.device))

    def free(self, t: Tensor) -> None:
        n = self._live.pop(t.data_ptr, 0)
        self._allocated -= n
        t.data = None

    def allocate_pinned(self, nbytes: int) -> torch.Tensor:
        """Page-locked host bytes (plain host memory when there is no GPU)."""
        return torch.empty(int(nbytes), dtype=torch.uint8, pin_memory=self.device.type == "cuda")

    # ---- copies -----------------------------------------------------------------------------------------------
    @staticmethod
    def _host_tensor(data, like: torch.Tensor) -> torch.Tensor:
        if isinstance(data, torch.Tensor):
            return data
        if isinstance(data, (bytes, bytearray, memoryview)):
            return torch.frombuffer(bytearray(data), dtype=torch.uint8)
        return torch.from_numpy(np.ascontiguousarray(data))

    def copy_host_to_device(self, data, dst: Tensor, non_blocking: bool = False) -> None:
        src = self._host_tensor(data, dst.data)
        flat = dst.data.view(-1)
        if src.dtype != flat.dtype:
            src = src.contiguous().view(-1).view(torch.uint8)
            flat = flat.view(torch.uint8)
        flat[: src.numel()].copy_(src.reshape(-1), non_blocking=non_blocking)

    def copy_device_to_host(self, src: Tensor, nbytes: Optional[int] = None) -> bytes:
        raw = src.data.contiguous().view(-1).view(torch.uint8)
        n = raw.numel() if nbytes is None else int(nbytes)
        return raw[:n].cpu().numpy().tobytes()

    def copy_device_to_device(self, src: Tensor, dst: Tensor, non_blocking: bool = True) -> None:
        d, s = dst.data.view(-1).view(torch.uint8), src.data.view(-1).view(torch.uint8)
        d[: s.numel()].copy_(s, non_blocking=non_blocking)

    copy_host_to_device_async = copy_host_to_device
    copy_device_to_device_async = copy_device_to_device

    def to_numpy(self, t: Tensor) -> np.ndarray:
        x = t.data.detach().cpu()
        return x.float().numpy() if x.dtype == torch.bfloat16 else x.numpy()

    def memset(self, t: Tensor, value: int = 0) -> None:
        t.data.view(-1).view(torch.uint8).fill_(int(value) & 0xFF)

    # ---- streams and facts ------------------------------------------------------------------------------------
    def create_stream(self):
        return torch.cuda.Stream(self.device) if self.device.type == "cuda" else None

    def synchronize(self, stream=None) -> None:
        if self.device.type != "cuda":
            return
        if stream is not None:
            stream.synchronize()
        else:
            torch.cuda.synchronize(self.device)

    def get_free_memory(self) -> int:
        return int(torch.cuda.mem_get_info(self.device)[0]) if self.device.type == "cuda" else 0

    def get_total_memory(self) -> int:
        return int(torch.cuda.mem_get_info(self.device)[1]) if self.device.type == "cuda" else 0

    # ---- raw addresses (zse-compiler/zse_compiler/runtime/memory.py:176-354) --------------------------------------
    # The reference hands out bare device and pinned-host addresses; here each address is backed by a torch byte tensor
    # that this object keeps alive until the matching free.
    def _raw_tables(self):
        if not hasattr(self, "_raw"):
            self._raw: Dict[int, torch.Tensor] = {}
            self._pinned: Dict[int, torch.Tensor] = {}
        return self._raw, self._pinned

    def malloc_raw(self, nbytes: int) -> int:
        if nbytes <= 0:
            return 0
        raw, _ = self._raw_tables()
        t = torch.empty(int(nbytes), dtype=torch.uint8, device=self.device)
        raw[int(t.data_ptr())] = t
        self._allocated += int(nbytes)
        self._peak = max(self._peak, self._allocated)
        return int(t.data_ptr())

    def free_raw(self, ptr: int) -> None:
        raw, _ = self._raw_tables()
        t = raw.pop(int(ptr), None)
        if t is not None:
            self._allocated -= t.numel()

    def _raw_view(self, ptr: int, nbytes: int) -> torch.Tensor:
        """The bytes ``[ptr, ptr + nbytes)`` of one of this object's raw allocations."""
        raw, _ = self._raw_tables()
        for base, t in raw.items():
            if base <= ptr and ptr + nbytes <= base + t.numel():
                return t[ptr - base: ptr - base + nbytes]
        raise ValueError(f"{nbytes} bytes at {ptr:#x} are not inside an allocation of malloc_raw")

    @staticmethod
    def _host_view(ptr: int, nbytes: int) -> torch.Tensor:
        import ctypes
        return torch.frombuffer((ctypes.c_ubyte * int(nbytes)).from_address(int(ptr)), dtype=torch.uint8)

    def copy_host_to_device_raw(self, host_data: bytes, dst_ptr: int, nbytes: int) -> None:
        if nbytes > 0:
            src = torch.frombuffer(bytearray(host_data[:nbytes]), dtype=torch.uint8)
            self._raw_view(int(dst_ptr), int(nbytes)).copy_(src)

    def copy_host_to_device_raw_ptr(self, src_ptr: int, dst_ptr: int, nbytes: int) -> None:
        if nbytes > 0:
            self._raw_view(int(dst_ptr), int(nbytes)).copy_(self._host_view(src_ptr, nbytes))

    def copy_host_to_device_async_raw_ptr(self, src_ptr: int, dst_ptr: int, nbytes: int, stream=None) -> None:
        """Returns at once when the source is pinned; the caller synchronises ``stream`` before reusing the buffer."""
        if nbytes <= 0:
            return
        dst, src = self._raw_view(int(dst_ptr), int(nbytes)), self._host_view(src_ptr, nbytes)
        if self.device.type == "cuda" and stream is not None and hasattr(stream, "synchronize"):
            with torch.cuda.stream(stream):
                dst.copy_(src, non_blocking=True)
        else:
            dst.copy_(src, non_blocking=True)

    def pinned_alloc(self, nbytes: int) -> int:
        if nbytes <= 0:
            return 0
        _, pinned = self._raw_tables()
        t = self.allocate_pinned(nbytes)
        pinned[int(t.data_ptr())] = t
        return int(t.data_ptr())

    def pinned_free(self, ptr: int) -> None:
        self._raw_tables()[1].pop(int(ptr), None)

    def destroy_stream(self, stream) -> None:
        """Streams are torch objects here and go away with their last reference; waits for the stream's work first."""
        self.synchronize_stream(stream)

    def synchronize_stream(self, stream=None) -> None:
        self.synchronize(stream if hasattr(stream, "synchronize") else None)

    @property
    def allocated_bytes(self) -> int:
        return self._allocated

    @property
    def peak_bytes(self) -> int:
        return self._peak
