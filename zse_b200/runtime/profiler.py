"""Event-timed kernel profiler and launch-configuration tuner.

``KernelProfiler`` (zse-compiler/zse_compiler/runtime/profiler.py:41-128): warm-up, then N launches timed with CUDA
events on the launching stream with a synchronise on both sides; between timed launches a buffer larger than L2 is
written so every launch starts cold; reports ms/launch, GB/s and TFLOP/s and, when measured peaks are known, the
fraction of them.  ``AutoTuner`` (zse-compiler/zse_compiler/runtime/autotune.py:72-170) sweeps candidate
configurations of a launch and keeps the fastest.
"""
from __future__ import annotations

import json
import os
import statistics
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional

import torch


def measured_peaks() -> Dict[str, float]:
    """HBM copy bandwidth (GB/s) and bf16 tensor throughput (TFLOP/s) measured on this pool, if a record exists next
    to the package; otherwise conservative earlier measurements."""
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "tflops": float(d["bf16_tflops"]),
                    "tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
        except (OSError, ValueError, KeyError):
            pass
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


@dataclass
class ProfileResult:
    name: str
    ms: float
    ms_min: float
    launches: int
    bytes: int = 0
    flops: int = 0
    extra: Dict[str, float] = field(default_factory=dict)

    @property
    def gbs(self) -> float:
        return self.bytes / (self.ms * 1e6) if self.ms > 0 and self.bytes else 0.0

    @property
    def tflops(self) -> float:
        return self.flops / (self.ms * 1e9) if self.ms > 0 and self.flops else 0.0

    def row(self, peaks: Optional[Dict[str, float]] = None) -> dict:
        d = {"name": self.name, "us": round(self.ms * 1000, 2), "us_min": round(self.ms_min * 1000, 2),
             "GB/s": round(self.gbs, 1), "TFLOP/s": round(self.tflops, 2)}
        if peaks:
            d["frac_hbm"] = round(self.gbs / peaks["hbm_gbs"], 3) if self.bytes else None
            d["frac_tensor"] = round(self.tflops / peaks["tflops"], 3) if self.flops else None
        d.update(self.extra)
        return d


class KernelProfiler:
    def __init__(self, device="cuda", warmup: int = 3, iters: int = 20, flush_l2: bool = True):
        self.device = torch.device(device)
        self.warmup, self.iters, self.flush_l2 = max(3, warmup), iters, flush_l2
        self._flush = None
        if flush_l2 and self.device.type == "cuda":
            self._flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.device)    # > 126 MB of L2

    def _cold(self) -> None:
        if self._flush is not None:
            self._flush.zero_()

    def time(self, name: str, fn: Callable[[], None], nbytes: int = 0, flops: int = 0, **extra) -> ProfileResult:
        for _ in range(self.warmup):
            self._cold()
            fn()
        torch.cuda.synchronize(self.device)
        samples = []
        for _ in range(self.iters):
            self._cold()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize(self.device)
            samples.append(a.elapsed_time(b))
        return ProfileResult(name, statistics.median(samples), min(samples), self.iters, nbytes, flops, dict(extra))


class AutoTuner:
    """``tune(name, make_fn, candidates)``: ``make_fn(candidate)`` returns the launch closure; the fastest candidate
    wins.  Results are remembered per name."""

    def __init__(self, profiler: Optional[KernelProfiler] = None):
        self.profiler = profiler or KernelProfiler(iters=10)
        self.best: Dict[str, dict] = {}

    def tune(self, name: str, make_fn: Callable[[object], Callable[[], None]], candidates: Iterable) -> dict:
        results = []
        for cand in candidates:
            try:
                r = self.profiler.time(f"{name}[{cand}]", make_fn(cand))
            except Exception as exc:      # a candidate the kernel rejects is simply not eligible
                results.append({"candidate": cand, "error": str(exc)})
                continue
            results.append({"candidate": cand, "ms": r.ms})
        ok = [r for r in results if "ms" in r]
        if not ok:
            raise RuntimeError(f"no candidate of {name} could be launched")
        win = min(ok, key=lambda r: r["ms"])
        self.best[name] = {"best": win["candidate"], "ms": win["ms"], "all": results}
        return self.best[name]
