"""Record-once / replay-many wrapper for a launch sequence, under the reference's class name and call order
(zse-engine/zse_engine/orchestrator/cuda_graph.py:24-136, hip_graph.py:35-228: begin_capture -> launches ->
end_capture -> replay, inputs living in fixed device buffers).  It stands on ``torch.cuda.CUDAGraph``, so captured
allocations come from a private pool and the graph can hold library kernels as well as this package's own.  The decode
buckets of ``runtime/runner.py`` use the same mechanism directly; this class is for callers that drive kernels
themselves (``ops.native`` entry points, ``NativeStep.forward``)."""
from __future__ import annotations

from typing import Optional

import torch


class CUDAGraphRunner:
    def __init__(self, device=None):
        self._device = device
        self._graph: Optional["torch.cuda.CUDAGraph"] = None
        self._ctx = None
        self._stream: Optional["torch.cuda.Stream"] = None
        self._captured = False

    def create_stream(self) -> "torch.cuda.Stream":
        return torch.cuda.Stream(device=self._device)

    def begin_capture(self, stream: Optional["torch.cuda.Stream"] = None) -> None:
        """Starts recording: every launch on the current stream until ``end_capture`` goes into the graph."""
        if not torch.cuda.is_available():
            raise RuntimeError("CUDA graphs need a GPU")
        if self._ctx is not None:
            raise RuntimeError("a capture is already open")
        self.destroy()
        self._stream = stream if stream is not None else self.create_stream()
        self._stream.wait_stream(torch.cuda.current_stream(self._device))
        self._graph = torch.cuda.CUDAGraph()
        self._ctx = torch.cuda.graph(self._graph, stream=self._stream)
        self._ctx.__enter__()

    def end_capture(self) -> None:
        if self._ctx is None:
            raise RuntimeError("no capture is open")
        ctx, self._ctx = self._ctx, None
        ctx.__exit__(None, None, None)
        self._captured = True

    def abort_capture(self, exc: BaseException) -> None:
        """Closes a capture that failed half-way, so that the stream leaves capture mode."""
        if self._ctx is not None:
            ctx, self._ctx = self._ctx, None
            try:
                ctx.__exit__(type(exc), exc, exc.__traceback__)
            finally:
                self._graph, self._captured = None, False

    def replay(self, stream: Optional["torch.cuda.Stream"] = None) -> None:
        if not self._captured or self._graph is None:
            raise RuntimeError("No graph captured yet")
        if stream is None:
            self._graph.replay()
        else:
            with torch.cuda.stream(stream):
                self._graph.replay()

    @property
    def is_captured(self) -> bool:
        return self._captured

    def sync(self, stream: Optional["torch.cuda.Stream"] = None) -> None:
        s = stream or self._stream
        if s is not None:
            s.synchronize()
        elif torch.cuda.is_available():
            torch.cuda.synchronize(self._device)

    def destroy(self) -> None:
        self._graph = None
        self._captured = False
