"""Cold-start weight streaming: the WEIGHT_DATA section of a ``.zse`` file goes to the device in one pass through a
ring of pinned buffers - reader threads fill them with ``preadv`` (the GIL is released, so several run at once), the
main thread queues one asynchronous copy per chunk on a private stream.  Tensors are then device views into that
mirror, and the re-tiling kernels read their input from device memory instead of from a host copy.

Same idea as zse-engine/zse_engine/orchestrator/weight_loader.py:22-409 (one allocation mirroring the section, 4 x 64 MB
pinned ring, ``ZSE_LOAD_CHUNK_MB`` / ``ZSE_LOAD_RING``), built on torch streams and events."""
from __future__ import annotations

import os
import queue
import threading
import time
from typing import Dict, Optional

import numpy as np
import torch
from ..utils import env

_DTYPES = {"uint8": torch.uint8, "int8": torch.int8, "float16": torch.float16}


class DeviceMirror:
    def __init__(self, loader, device, chunk_mb: Optional[int] = None, ring: Optional[int] = None, readers: int = 4):
        self.offset, self.size = loader.weight_data_section()
        self.device = torch.device(device)
        chunk = int(chunk_mb or env.integer("ZSE_LOAD_CHUNK_MB")) << 20
        ring = max(2, int(ring or env.integer("ZSE_LOAD_RING")))
        readers = max(1, min(readers, ring - 1))
        t0 = time.monotonic()
        self.base = torch.empty(self.size, dtype=torch.uint8, device=self.device)
        fd = loader.file_descriptor
        chunks = [(pos, min(chunk, self.size - pos)) for pos in range(0, self.size, chunk)]
        pinned = [torch.empty(chunk, dtype=torch.uint8, pin_memory=True) for _ in range(ring)]
        views = [p.numpy() for p in pinned]
        free_slots: "queue.Queue[int]" = queue.Queue()
        for i in range(ring):
            free_slots.put(i)
        ready: Dict[int, int] = {}
        cond = threading.Condition()
        counter = [0]
        errors = []

        def reader() -> None:
            try:
                while True:
                    # a staging buffer first, the chunk index second: every claimed chunk then owns a buffer, and the
                    # chunk the consumer waits for is always claimed by a reader that can fill it (claiming the index
                    # first lets readers of later chunks hold every buffer while the next chunk's reader has none)
                    slot = free_slots.get()
                    with cond:
                        k = counter[0]
                        if k >= len(chunks):
                            free_slots.put(slot)
                            return
                        counter[0] += 1
                    pos, n = chunks[k]
                    got = 0
                    mv = memoryview(views[slot])[:n]
                    while got < n:
                        r = os.preadv(fd, [mv[got:]], self.offset + pos + got)
                        if r <= 0:
                            raise IOError(f"short read at offset {self.offset + pos + got}")
                        got += r
                    with cond:
                        ready[k] = slot
                        cond.notify_all()
            except BaseException as exc:      # surfaced on the main thread
                with cond:
                    errors.append(exc)
                    cond.notify_all()

        threads = [threading.Thread(target=reader, daemon=True) for _ in range(readers)]
        for t in threads:
            t.start()
        stream = torch.cuda.Stream(device=self.device)
        inflight = []
        with torch.cuda.stream(stream):
            for k, (pos, n) in enumerate(chunks):
                with cond:
                    waited = 0.0
                    while k not in ready and not errors:
                        cond.wait(0.5)
                        waited += 0.5
                        if waited > 300.0:
                            raise TimeoutError(f"weight chunk {k} of {len(chunks)} did not arrive within 300 s")
                    if errors:
                        raise errors[0]
                    slot = ready.pop(k)
                self.base[pos:pos + n].copy_(pinned[slot][:n], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(stream)
                inflight.append((ev, slot))
                while len(inflight) > ring - readers:
                    e, s = inflight.pop(0)
                    e.synchronize()
                    free_slots.put(s)
        stream.synchronize()
        for t in threads:
            t.join()
        self.seconds = time.monotonic() - t0

    def view(self, rel_offset: int, nbytes: int, dtype: str = "uint8") -> torch.Tensor:
        """Device view of ``nbytes`` at ``rel_offset`` inside WEIGHT_DATA (no copy; keeps the mirror alive)."""
        t = self.base[rel_offset:rel_offset + nbytes]
        return t if dtype == "uint8" else t.view(_DTYPES[dtype])

    def release(self) -> None:
        self.base = None


def open_mirror(loader, device, stats: Optional[dict] = None) -> Optional["DeviceMirror"]:
    """The streamed copy of the weight section, or None when it is switched off (``ZSE_STREAM_WEIGHTS=0``), the device
    is not a GPU, or the streamed pass failed - the caller then copies tensor by tensor, as the reference falls back
    from its streamed path (zse-engine/zse_engine/orchestrator/weight_loader.py:188-199).  With ``ZSE_DEBUG_LOAD=1`` the
    failure is printed with its traceback; ``stats`` receives the throughput or the reason."""
    dev = torch.device(device)
    if dev.type != "cuda" or not env.flag("ZSE_STREAM_WEIGHTS"):
        return None
    try:
        mirror = DeviceMirror(loader, dev)
    except (OSError, RuntimeError, TimeoutError, MemoryError) as exc:
        if stats is not None:
            stats["stream_error"] = " ".join(str(exc).split())[:200] or type(exc).__name__
        if env.flag("ZSE_DEBUG_LOAD"):
            import sys
            import traceback
            traceback.print_exc()
            print(f"[zse] streamed weight load failed ({type(exc).__name__}: {exc}); copying tensor by tensor",
                  file=sys.stderr)
        return None
    if stats is not None:
        stats["stream_s"] = round(mirror.seconds, 3)
        stats["stream_gbs"] = round(mirror.size / max(mirror.seconds, 1e-9) / 1e9, 2)
    return mirror


class HostMirror:
    """The same interface over the file mapping, for a CPU device: tensors are views of the mapped pages."""

    def __init__(self, loader):
        self.offset, self.size = loader.weight_data_section()
        self.device = torch.device("cpu")
        t0 = time.monotonic()
        buf = np.frombuffer(loader._span(0, self.size), dtype=np.uint8) if self.size else np.zeros(0, np.uint8)
        self.base = torch.from_numpy(buf.copy())
        self.seconds = time.monotonic() - t0

    view = DeviceMirror.view
    release = DeviceMirror.release


# ---- name-based store over the mirror (zse-engine/zse_engine/orchestrator/weight_loader.py:50-409) --------------------
class GPUWeight:
    """One stored tensor on the device: ``data`` / ``scales`` / ``zeros`` are views into the mirror, in the layout of the
    file (row-major or tiled nibbles, fp16 scales and zero points per group).  The ``*_ptr`` / ``*_nbytes`` fields are
    the ones the reference's record carries."""

    def __init__(self, name, shape, dtype, data, scales=None, zeros=None, group_size=128, quant_method=0,
                 layout="rowmajor"):
        self.name, self.shape, self.dtype = name, tuple(shape), dtype
        self.data, self.scales, self.zeros = data, scales, zeros
        self.group_size, self.quant_method, self.layout = group_size, quant_method, layout
        n = 1
        for d in self.shape:
            n *= int(d)
        self.num_elements = n

    @staticmethod
    def _ptr(t) -> int:
        return int(t.data_ptr()) if t is not None and t.numel() else 0

    @staticmethod
    def _nbytes(t) -> int:
        return int(t.numel() * t.element_size()) if t is not None else 0

    data_ptr = property(lambda self: self._ptr(self.data))
    scales_ptr = property(lambda self: self._ptr(self.scales))
    zeros_ptr = property(lambda self: self._ptr(self.zeros))
    data_nbytes = property(lambda self: self._nbytes(self.data))
    scales_nbytes = property(lambda self: self._nbytes(self.scales))
    zeros_nbytes = property(lambda self: self._nbytes(self.zeros))

    @property
    def total_gpu_bytes(self) -> int:
        return self.data_nbytes + self.scales_nbytes + self.zeros_nbytes

    def to_float(self) -> torch.Tensor:
        """The tensor dequantised to fp32 on the host (a check and debugging aid, not a hot path)."""
        from ..format import quantize as q
        if self.dtype == "float16":
            return self.data.detach().float().cpu().reshape(self.shape)
        data = self.data.detach().cpu().contiguous().numpy()
        scales = self.scales.detach().cpu().contiguous().numpy()
        if self.dtype == "int8":
            return torch.from_numpy(np.asarray(q.dequantize_tensor_int8(data, scales, self.shape, self.group_size),
                                               np.float32).reshape(self.shape))
        zeros = self.zeros.detach().cpu().contiguous().numpy()
        if self.layout != "rowmajor":
            data = q.untile_int4_64x8(data.reshape(-1), self.shape[0], self.shape[1])
        K = self.shape[-1]
        if data.ndim == 2 and K % self.group_size == 0:      # a sliced shard: groups run along each row
            flat = q.dequantize_int4_arrays(data, scales, zeros, self.num_elements, self.group_size)
        else:
            flat = q.dequantize_int4_arrays(data.reshape(-1), scales.reshape(-1), zeros.reshape(-1),
                                            self.num_elements, self.group_size)
        return torch.from_numpy(np.asarray(flat, np.float32).reshape(self.shape))


class WeightStore:
    """Every tensor of a model by stored name (``layers.0.self_attn.q_proj.weight``; a leading ``model.`` is ignored)."""

    def __init__(self):
        self._weights: Dict[str, GPUWeight] = {}
        self._total_bytes = 0
        self._mirror = None

    @staticmethod
    def _key(name: str) -> str:
        return name[6:] if name.startswith("model.") else name

    def add(self, weight: GPUWeight) -> None:
        self._weights[self._key(weight.name)] = weight
        self._total_bytes += weight.total_gpu_bytes

    def get(self, name: str) -> GPUWeight:
        return self._weights[self._key(name)]

    def find(self, name: str) -> Optional[GPUWeight]:
        return self._weights.get(self._key(name))

    def has(self, name: str) -> bool:
        return self._key(name) in self._weights

    __contains__ = has

    def __iter__(self):
        return iter(self._weights.values())

    def __len__(self) -> int:
        return len(self._weights)

    @property
    def total_bytes(self) -> int:
        return self._total_bytes

    @property
    def num_weights(self) -> int:
        return len(self._weights)

    def summary(self) -> str:
        lines = [f"WeightStore: {self.num_weights} tensors, {self._total_bytes / 1024**2:.1f}MB on device"]
        by_dtype: Dict[str, list] = {}
        for w in self._weights.values():
            c = by_dtype.setdefault(w.dtype, [0, 0])
            c[0] += 1
            c[1] += w.total_gpu_bytes
        for dtype, (count, nbytes) in sorted(by_dtype.items()):
            lines.append(f"  {dtype}: {count} tensors, {nbytes / 1024**2:.1f}MB")
        return "\n".join(lines)

    def destroy(self, gpu_mem=None) -> None:
        """Drops every view and the single allocation behind them (``gpu_mem`` is accepted for the reference's
        signature; the caching allocator owns the memory here)."""
        self._weights.clear()
        self._total_bytes = 0
        if self._mirror is not None:
            self._mirror.release()
            self._mirror = None


class WeightLoader:
    """``WeightLoader(loader, device).load_all(progress_fn)`` -> ``WeightStore``: the weight section is mirrored to the
    device in one streamed pass and every index entry becomes views into it.  ``progress_fn(name, i, n)`` is called
    once per tensor, as the reference does."""

    def __init__(self, loader, device="cuda", chunk_mb: Optional[int] = None, ring: Optional[int] = None):
        self.loader = loader
        self.device = torch.device(device) if not hasattr(device, "type") else device
        self.chunk_mb, self.ring = chunk_mb, ring
        self.seconds = 0.0

    def load_all(self, progress_fn=None) -> WeightStore:
        if self.device.type == "cuda":
            mirror = DeviceMirror(self.loader, self.device, self.chunk_mb, self.ring)
        else:
            mirror = HostMirror(self.loader)
        self.seconds = mirror.seconds
        store = WeightStore()
        store._mirror = mirror
        entries = list(self.loader.weight_index)
        for i, e in enumerate(entries):
            if e.dtype == "float16":
                data = mirror.view(e.data_offset, e.data_nbytes, "float16").reshape(tuple(e.shape))
            elif e.dtype == "int8":
                data = mirror.view(e.data_offset, e.data_nbytes, "int8").reshape(tuple(e.shape))
            else:
                data = mirror.view(e.data_offset, e.data_nbytes)
            scales = mirror.view(e.scale_offset, e.scale_nbytes, "float16") if e.scale_nbytes else None
            zeros = mirror.view(e.zeros_offset, e.zeros_nbytes, "float16") if e.zeros_nbytes else None
            store.add(GPUWeight(e.name, e.shape, e.dtype, data, scales, zeros, e.group_size, e.quant_method,
                                self.loader.int4_layout_of(e)))
            if progress_fn is not None:
                progress_fn(e.name, i + 1, len(entries))
        return store
