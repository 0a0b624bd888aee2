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

_DTYPES = {"uint8": torch.uint8, "int8": torch.int8, "float16": torch.float16}


class DeviceMirror:
    def __init__(self, loader, device, chunk_mb: Optional[int] = None, ring: Optional[int] = None, readers: int = 4):
        self.offset, self.size = loader.weight_data_section()
        self.device = torch.device(device)
        chunk = int(chunk_mb or os.environ.get("ZSE_LOAD_CHUNK_MB", 64)) << 20
        ring = max(2, int(ring or os.environ.get("ZSE_LOAD_RING", 6)))
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
                    with cond:
                        k = counter[0]
                        if k >= len(chunks):
                            return
                        counter[0] += 1
                    slot = free_slots.get()
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
                    while k not in ready and not errors:
                        cond.wait(0.5)
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
