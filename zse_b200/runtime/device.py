"""Device discovery (zse-compiler/zse_compiler/runtime/device.py:14-292): name, compute capability, memory, SM count,
shared memory, warp size of every visible GPU, through torch."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch


@dataclass
class DeviceInfo:
    index: int
    name: str
    compute_capability: tuple
    total_memory: int
    free_memory: int
    sm_count: int
    shared_mem_per_block_optin: int
    warp_size: int = 32

    @property
    def is_blackwell(self) -> bool:
        return self.compute_capability[0] == 10

    # the reference's field names (zse-compiler/zse_compiler/runtime/device.py:14-40)
    backend = "cuda"

    @property
    def vram_total_bytes(self) -> int:
        return self.total_memory

    @property
    def vram_free_bytes(self) -> int:
        return self.free_memory

    @property
    def vram_total_gb(self) -> float:
        return self.total_memory / (1024 ** 3)

    @property
    def vram_free_gb(self) -> float:
        return self.free_memory / (1024 ** 3)

    @property
    def num_sms(self) -> int:
        return self.sm_count


def detect_backend() -> str:
    return "cuda" if torch.cuda.is_available() else "cpu"


def get_devices() -> List[DeviceInfo]:
    out = []
    if not torch.cuda.is_available():
        return out
    for i in range(torch.cuda.device_count()):
        p = torch.cuda.get_device_properties(i)
        free, total = torch.cuda.mem_get_info(i)
        out.append(DeviceInfo(i, p.name, (p.major, p.minor), total, free, p.multi_processor_count,
                              getattr(p, "shared_memory_per_block_optin", 0), getattr(p, "warp_size", 32)))
    return out


def describe_devices() -> List[str]:
    devs = get_devices()
    lines = [f"  backend: {detect_backend()}"]
    if not devs:
        lines.append("  no CUDA device visible (the engine runs on the CPU reference path)")
    for d in devs:
        lines.append(f"  device {d.index}: {d.name}, sm_{d.compute_capability[0]}{d.compute_capability[1]}, "
                     f"{d.sm_count} SMs, {d.total_memory / 2**30:.1f} GiB ({d.free_memory / 2**30:.1f} free), "
                     f"{d.shared_mem_per_block_optin // 1024} KB smem/CTA"
                     + ("" if d.is_blackwell else "  [not sm_100: the native kernels will not load]"))
    return lines
