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


@dataclass
class KernelProfile:
    """Time of one compiled kernel under one launch configuration, the record of the reference's profiler
    (zse-compiler/zse_compiler/runtime/profiler.py:14-38)."""
    kernel_name: str
    backend: str
    elapsed_ms: float            # per launch
    grid: tuple
    block: tuple
    num_runs: int = 1
    total_flops: Optional[int] = None

    @property
    def throughput_gflops(self) -> Optional[float]:
        """GFLOP/s, once the caller has set ``total_flops`` (None before)."""
        if self.total_flops is None or self.elapsed_ms <= 0:
            return None
        return self.total_flops / (self.elapsed_ms * 1e6)

    def bandwidth_gb_s(self, total_bytes: int) -> float:
        return 0.0 if self.elapsed_ms <= 0 else (total_bytes / 1e9) / (self.elapsed_ms / 1e3)

    def __repr__(self) -> str:
        return f"KernelProfile('{self.kernel_name}', {self.elapsed_ms:.3f}ms, grid={self.grid}, block={self.block})"


BLOCK_SIZES_1D = [32, 64, 128, 256, 512, 1024]
BLOCK_SIZES_2D = [(8, 8), (16, 8), (8, 16), (16, 16), (32, 8), (8, 32), (32, 16), (16, 32), (32, 32)]


@dataclass
class TuneResult:
    """Outcome of a sweep over launch configurations (zse-compiler/zse_compiler/runtime/autotune.py:24-60)."""
    kernel_name: str
    best_config: object          # dsl.LaunchConfig
    best_time_ms: float
    all_results: List[KernelProfile]

    def summary(self) -> str:
        lines = [f"Auto-tune results for '{self.kernel_name}':", f"{'Config':<20} {'Time (ms)':<12} {'Speedup':<10}",
                 "-" * 42]
        worst = max((r.elapsed_ms for r in self.all_results), default=1.0)
        for r in sorted(self.all_results, key=lambda x: x.elapsed_ms):
            block = f"{r.block[0]}" + (f"x{r.block[1]}" if len(r.block) > 1 and r.block[1] > 1 else "")
            speed = worst / r.elapsed_ms if r.elapsed_ms > 0 else 0.0
            mark = "  <- best" if r.elapsed_ms == self.best_time_ms else ""
            lines.append(f"  block={block:<12} {r.elapsed_ms:<12.3f} {speed:<10.2f}x{mark}")
        return "\n".join(lines)


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

    def profile(self, kernel, config, args: tuple, warmup_runs: int = 3, profile_runs: int = 10,
                launcher=None) -> KernelProfile:
        """The reference's call (zse-compiler/zse_compiler/runtime/profiler.py:47-128): a COMPILED kernel of the
        kernel language, a ``LaunchConfig`` and the argument values.  ``args`` may be a ``PrepackedArgs`` or plain
        values (tensors, ints, floats).  Timed with CUDA events around each launch on a GPU; where there is none (or
        with a stand-in ``launcher`` in tests) with the wall clock, as the reference does for its other back ends."""
        import time as _time
        from ..dsl.launcher import KernelLauncher, PrepackedArgs
        launcher = launcher or KernelLauncher()
        packed = args if isinstance(args, PrepackedArgs) else PrepackedArgs.from_args(*args)
        run = lambda: launcher.launch_prepacked(kernel, config, packed)
        for _ in range(max(0, warmup_runs)):
            run()
        on_gpu = self.device.type == "cuda" and torch.cuda.is_available()
        samples = []
        for _ in range(max(1, profile_runs)):
            if on_gpu:
                self._cold()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                run()
                b.record()
                torch.cuda.synchronize(self.device)
                samples.append(a.elapsed_time(b))
            else:
                t0 = _time.perf_counter()
                run()
                samples.append((_time.perf_counter() - t0) * 1000.0)
        return KernelProfile(getattr(kernel, "name", "kernel"), "cuda" if on_gpu else "host",
                             statistics.median(samples), tuple(config.grid), tuple(config.block), len(samples))


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

    # ---- the reference's sweeps over a compiled kernel (zse-compiler/zse_compiler/runtime/autotune.py:80-170) ---------
    def _sweep(self, kernel, args, configs, what: str, launcher=None) -> TuneResult:
        from ..dsl.errors import KernelError
        results = []
        for cfg in configs:
            try:
                results.append(self.profiler.profile(kernel, cfg, args, warmup_runs=self.profiler.warmup,
                                                     profile_runs=self.profiler.iters, launcher=launcher))
            except (ValueError, RuntimeError, KernelError):
                continue                      # a configuration the kernel or the device refuses is not eligible
        if not results:
            raise RuntimeError(f"No valid configurations found for {what}")
        best = min(results, key=lambda r: r.elapsed_ms)
        from ..dsl.launcher import LaunchConfig
        return TuneResult(getattr(kernel, "name", "kernel"), LaunchConfig(best.grid, best.block), best.elapsed_ms,
                          results)

    def tune_1d(self, kernel, args: tuple, total_threads: int, block_sizes: Optional[List[int]] = None,
                launcher=None) -> TuneResult:
        """Block sizes that divide ``total_threads``; the grid follows."""
        from ..dsl.errors import KernelError
        from ..dsl.launcher import LaunchConfig
        configs = []
        for bs in (block_sizes or BLOCK_SIZES_1D):
            if bs <= total_threads and total_threads % bs == 0:
                try:
                    configs.append(LaunchConfig((total_threads // bs,), (bs,)))
                except KernelError:
                    pass
        return self._sweep(kernel, args, configs, f"{total_threads} threads", launcher)

    def tune_2d(self, kernel, args: tuple, grid_shape, block_sizes=None, launcher=None) -> TuneResult:
        """Two-dimensional blocks over ``grid_shape = (rows, cols)`` elements (x covers the columns)."""
        from ..dsl.errors import KernelError
        from ..dsl.launcher import LaunchConfig
        rows, cols = grid_shape
        configs = []
        for bx, by in (block_sizes or BLOCK_SIZES_2D):
            try:
                configs.append(LaunchConfig(((cols + bx - 1) // bx, (rows + by - 1) // by), (bx, by)))
            except KernelError:
                pass
        return self._sweep(kernel, args, configs, f"a {rows} x {cols} grid", launcher)
