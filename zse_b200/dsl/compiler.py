"""CUDA text -> cubin for sm_100a -> loaded module (the reference's runtime compiler goes through NVRTC to PTX and
``cuModuleLoadData``, zse-compiler/zse_compiler/runtime/compiler.py:35-367).

Here nvcc builds a cubin for the one target (``-gencode arch=compute_100a,code=sm_100a``), so compiling needs no GPU
and the result can be made ahead of time; cubins are kept in memory and on disk under a key made of the source text,
the flags and the compiler version.  Loading and launching go through the CUDA driver API (``cuda.bindings.driver``)
on the context torch already holds."""
from __future__ import annotations

import hashlib
import os
import subprocess
import tempfile
import threading
from dataclasses import dataclass, field
from typing import Dict, Optional

from ..ops.build import nvcc_path
from .errors import KernelCompileError, KernelLaunchError
from ..utils import env

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo"]


def cache_dir() -> str:
    d = os.path.expanduser(env.text("ZSE_KERNEL_CACHE"))
    os.makedirs(d, exist_ok=True)
    return d


@dataclass
class CompiledKernel:
    name: str
    source: str
    cubin: bytes
    key: str
    from_cache: bool = False
    _module: Optional[object] = field(default=None, repr=False)
    _function: Optional[object] = field(default=None, repr=False)

    def function(self):
        """The driver handle of the kernel, loaded into the current context on first use."""
        if self._function is None:
            drv = _driver()
            import torch
            torch.cuda.init()
            torch.empty(1, device=f"cuda:{torch.cuda.current_device()}")     # torch's primary context is now current
            err, mod = drv.cuModuleLoadData(self.cubin)
            _check(err, f"loading the module of '{self.name}'")
            err, fn = drv.cuModuleGetFunction(mod, self.name.encode())
            _check(err, f"finding '{self.name}' in its module")
            self._module, self._function = mod, fn
        return self._function

    def unload(self) -> None:
        if self._module is not None:
            _driver().cuModuleUnload(self._module)
            self._module = self._function = None


def _driver():
    try:
        from cuda.bindings import driver
    except ImportError:                                      # older layout of the same package
        from cuda import cuda as driver
    return driver


def _check(err, what: str) -> None:
    if int(err) != 0:
        drv = _driver()
        try:
            _, name = drv.cuGetErrorName(err)
            name = name.decode() if isinstance(name, bytes) else str(name)
        except Exception:
            name = str(err)
        raise KernelLaunchError(f"{what} failed: {name}")


class RuntimeCompiler:
    def __init__(self, extra_flags=None, use_disk_cache: bool = True):
        self.flags = BASE_FLAGS + list(extra_flags or [])
        self.use_disk_cache = use_disk_cache
        self._mem: Dict[str, CompiledKernel] = {}
        self._lock = threading.Lock()
        self.stats = {"compiled": 0, "memory_hits": 0, "disk_hits": 0}

    def _version(self) -> str:
        v = getattr(RuntimeCompiler, "_nvcc_version", None)
        if v is None:
            out = subprocess.run([nvcc_path(), "--version"], capture_output=True, text=True).stdout
            v = RuntimeCompiler._nvcc_version = out.strip().splitlines()[-1] if out.strip() else "nvcc"
        return v

    def key(self, source: str, name: str) -> str:
        h = hashlib.sha256()
        for part in (source, name, " ".join(ARCH_FLAGS + self.flags), self._version()):
            h.update(part.encode())
            h.update(b"\0")
        return h.hexdigest()

    def compile(self, source: str, name: str, backend: str = "cuda") -> CompiledKernel:
        if backend != "cuda":
            raise ValueError(f"this package compiles for CUDA sm_100a only (asked for {backend!r})")
        key = self.key(source, name)
        with self._lock:
            hit = self._mem.get(key)
            if hit is not None:
                self.stats["memory_hits"] += 1
                return hit
        path = os.path.join(cache_dir(), key[:32] + ".cubin") if self.use_disk_cache else None
        if path and os.path.exists(path):
            with open(path, "rb") as f:
                ck = CompiledKernel(name, source, f.read(), key, True)
            self.stats["disk_hits"] += 1
        else:
            ck = CompiledKernel(name, source, self._nvcc(source, name), key)
            self.stats["compiled"] += 1
            if path:
                tmp = f"{path}.{os.getpid()}.tmp"
                with open(tmp, "wb") as f:
                    f.write(ck.cubin)
                os.replace(tmp, path)
        with self._lock:
            self._mem[key] = ck
        return ck

    def _nvcc(self, source: str, name: str) -> bytes:
        with tempfile.TemporaryDirectory(prefix="zse_kernel_") as d:
            src, out = os.path.join(d, name + ".cu"), os.path.join(d, name + ".cubin")
            with open(src, "w") as f:
                f.write(source)
            res = subprocess.run([nvcc_path()] + ARCH_FLAGS + self.flags + ["-cubin", "-o", out, src],
                                 capture_output=True, text=True)
            if res.returncode != 0:
                raise KernelCompileError(f"nvcc rejected kernel '{name}'", (res.stdout + res.stderr).strip(), source)
            with open(out, "rb") as f:
                return f.read()

    def resource_usage(self, source: str, name: str) -> Dict[str, int]:
        """What ptxas reports for the kernel (``-Xptxas -v``): registers per thread, spill bytes, static shared
        memory, stack frame.  A separate nvcc run; nothing is cached."""
        import re
        with tempfile.TemporaryDirectory(prefix="zse_kernel_") as d:
            src, out = os.path.join(d, name + ".cu"), os.path.join(d, name + ".cubin")
            with open(src, "w") as f:
                f.write(source)
            res = subprocess.run([nvcc_path()] + ARCH_FLAGS + self.flags + ["-Xptxas", "-v", "-cubin", "-o", out, src],
                                 capture_output=True, text=True)
            if res.returncode != 0:
                raise KernelCompileError(f"nvcc rejected kernel '{name}'", (res.stdout + res.stderr).strip(), source)
        log = res.stdout + res.stderr
        grab = lambda pat: int(m.group(1)) if (m := re.search(pat, log)) else 0
        return {"registers": grab(r"Used (\d+) registers"), "spill_stores": grab(r"(\d+) bytes spill stores"),
                "spill_loads": grab(r"(\d+) bytes spill loads"), "stack_frame": grab(r"(\d+) bytes stack frame"),
                "shared_bytes": grab(r"(\d+) bytes smem"), "barriers": grab(r"used (\d+) barriers")}

    def clear_cache(self) -> None:
        with self._lock:
            self._mem.clear()


_default: Optional[RuntimeCompiler] = None


def default_compiler() -> RuntimeCompiler:
    global _default
    if _default is None:
        _default = RuntimeCompiler()
    return _default
