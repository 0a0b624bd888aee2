"""Ahead-of-time build of the native library (``zse_b200/_C/libzse_b200.so``).

Every ``csrc/*.cu`` and ``csrc/host/*.cpp`` is compiled for ``sm_100a`` only
(``-gencode arch=compute_100a,code=sm_100a -lineinfo``) into an object cached under ``build/`` by the hash of its
source, the headers and the flags, then linked into one shared library that lives inside the package so that it
travels with the source tree.  nvcc cross-compiles without a GPU.  This is the counterpart of the reference's
start-up NVRTC/gcc compilation with its on-disk caches (zse-engine/zse_engine/orchestrator/kernels.py:2846-3010,
format/fast_quant.py:243-288) moved to build time.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from typing import List

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
CSRC = os.path.join(ROOT, "csrc")
OUT_DIR = os.path.join(ROOT, "zse_b200", "_C")
LIB_PATH = os.path.join(OUT_DIR, "libzse_b200.so")
OBJ_DIR = os.path.join(ROOT, "build", "obj")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-Xcudafe", "--diag_suppress=177"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put /usr/local/cuda/bin on PATH)")


def sources() -> List[str]:
    out = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith(".cu")]
    host = os.path.join(CSRC, "host")
    if os.path.isdir(host):
        out += [os.path.join(host, f) for f in sorted(os.listdir(host)) if f.endswith(".cpp")]
    return out


def _headers_digest() -> bytes:
    h = hashlib.sha256()
    for base, _, files in sorted(os.walk(CSRC)):
        for f in sorted(files):
            if f.endswith((".h", ".cuh", ".hpp")):
                with open(os.path.join(base, f), "rb") as fh:
                    h.update(fh.read())
    return h.digest()


def _object_for(src: str, hdr: bytes, extra: tuple = ()) -> str:
    h = hashlib.sha256(hdr)
    with open(src, "rb") as f:
        h.update(f.read())
    h.update(" ".join(NVCC_FLAGS + list(extra)).encode())
    return os.path.join(OBJ_DIR, f"{os.path.basename(src)}.{h.hexdigest()[:16]}.o")


def _compile(nvcc: str, src: str, obj: str, verbose: bool, extra: tuple = ()) -> None:
    if os.path.exists(obj):
        return
    cmd = [nvcc] + NVCC_FLAGS + list(extra) + ["-I", CSRC, "-c", src, "-o", obj + ".tmp"]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
    os.replace(obj + ".tmp", obj)


def _prune() -> None:
    """Drops cached objects that no linked library refers to any more (every edit of a source leaves one behind)."""
    keep = set()
    for f in os.listdir(OUT_DIR) if os.path.isdir(OUT_DIR) else []:
        if f.endswith(".stamp"):
            with open(os.path.join(OUT_DIR, f)) as fh:
                keep |= set(fh.read().split())
    for f in os.listdir(OBJ_DIR) if os.path.isdir(OBJ_DIR) else []:
        if f.endswith(".o") and f not in keep:
            try:
                os.unlink(os.path.join(OBJ_DIR, f))
            except OSError:
                pass


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile what changed and (re)link.  Returns the library path."""
    nvcc = nvcc_path()
    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(OUT_DIR, exist_ok=True)
    hdr = _headers_digest()
    srcs = sources()
    objs = [_object_for(s, hdr) for s in srcs]
    if force:
        for o in objs:
            if os.path.exists(o):
                os.unlink(o)
    stamp = os.path.join(OUT_DIR, "libzse_b200.stamp")
    want = "\n".join(os.path.basename(o) for o in objs)
    if not force and os.path.exists(LIB_PATH) and os.path.exists(stamp) and open(stamp).read() == want:
        return LIB_PATH
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        list(pool.map(lambda so: _compile(nvcc, so[0], so[1], verbose), zip(srcs, objs)))
    cmd = [nvcc] + ARCH_FLAGS + ["-shared", "-o", LIB_PATH + ".tmp"] + objs
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    os.replace(LIB_PATH + ".tmp", LIB_PATH)
    with open(stamp, "w") as f:
        f.write(want)
    _prune()
    return LIB_PATH


# Instrumented variants of the library: the same sources with extra defines, linked beside the ordinary library as
# libzse_b200.<name>.so.  ZSE_NATIVE_LIB=<path> makes a process load one (zse_b200/runtime/kernel_counters.py does).
VARIANTS = {
    # per-role cycle counters (clock64) in the INT4 GEMM kernels, written to a buffer set by zse_gemm_w4*_set_timing
    "timing": ("-DZSE_DEC_TIMING", "-DZSE_W4_TIMING", "-DZSE_ATTN_TIMING"),
}


def variant_path(name: str) -> str:
    return os.path.join(OUT_DIR, f"libzse_b200.{name}.so")


def build_variant(name: str, verbose: bool = False) -> str:
    extra = VARIANTS[name]
    nvcc = nvcc_path()
    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(OUT_DIR, exist_ok=True)
    hdr = _headers_digest()
    srcs = sources()
    objs = [_object_for(s, hdr, extra) for s in srcs]
    out = variant_path(name)
    stamp = out + ".stamp"
    want = "\n".join(os.path.basename(o) for o in objs)
    if os.path.exists(out) and os.path.exists(stamp) and open(stamp).read() == want:
        return out
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        list(pool.map(lambda so: _compile(nvcc, so[0], so[1], verbose, extra), zip(srcs, objs)))
    res = subprocess.run([nvcc] + ARCH_FLAGS + ["-shared", "-o", out + ".tmp"] + objs, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    os.replace(out + ".tmp", out)
    with open(stamp, "w") as f:
        f.write(want)
    _prune()
    return out


def is_built() -> bool:
    return os.path.exists(LIB_PATH)


if __name__ == "__main__":
    if "--variant" in sys.argv:
        print(build_variant(sys.argv[sys.argv.index("--variant") + 1], verbose="-v" in sys.argv))
    else:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
