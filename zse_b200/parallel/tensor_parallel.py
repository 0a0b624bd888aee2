"""The reference's tensor-parallel primitives under their own names: ``TPConfig``, ``TensorParallelGroup``,
``tp_launch`` and the weight split maps (zse-engine/zse_engine/orchestrator/tensor_parallel.py:35-350).

The reference wraps libnccl through ctypes and hands a 128-byte unique id to every rank.  Here a group is a
``torch.distributed`` process group (NCCL on GPUs, gloo on CPU ranks): ``unique_id`` is the rendezvous string that
``tp_launch`` passes around (``"127.0.0.1:<port>"``).  The engine itself does not go through this class on its hot path
(see ``parallel/comm.py``); it exists so that code written against the reference's primitives keeps working.
Differences: shard ranges follow ``parallel/shard_plan.py`` (uneven, group-aligned shards are allowed where the
reference requires divisibility), and ``lm_head`` shards are gathered properly.
"""
from __future__ import annotations

import ctypes
import multiprocessing
import os
import socket
from dataclasses import dataclass
from typing import Any, Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

from .comm import NcclComm
from .shard_plan import split_units

COLUMN_PARALLEL = "column"    # split along the output dimension
ROW_PARALLEL = "row"          # split along the input dimension
REPLICATED = "replicated"

WEIGHT_SPLIT_MAP = {
    "self_attn.q_proj.weight": COLUMN_PARALLEL, "self_attn.k_proj.weight": COLUMN_PARALLEL,
    "self_attn.v_proj.weight": COLUMN_PARALLEL, "self_attn.q_proj.bias": COLUMN_PARALLEL,
    "self_attn.k_proj.bias": COLUMN_PARALLEL, "self_attn.v_proj.bias": COLUMN_PARALLEL,
    "self_attn.o_proj.weight": ROW_PARALLEL, "mlp.gate_proj.weight": COLUMN_PARALLEL,
    "mlp.up_proj.weight": COLUMN_PARALLEL, "mlp.down_proj.weight": ROW_PARALLEL,
    "input_layernorm.weight": REPLICATED, "post_attention_layernorm.weight": REPLICATED,
}
NON_LAYER_SPLIT_MAP = {"embed_tokens.weight": REPLICATED, "model.norm.weight": REPLICATED, "norm.weight": REPLICATED,
                       "lm_head.weight": COLUMN_PARALLEL}


@dataclass
class TPConfig:
    tp_size: int = 1
    backend: str = "cuda"

    def is_enabled(self) -> bool:
        return self.tp_size > 1

    def validate(self, num_heads: int, num_kv_heads: int, intermediate_size: int) -> None:
        if self.tp_size <= 1:
            return
        if num_heads % self.tp_size:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by tp_size ({self.tp_size})")
        if num_kv_heads % self.tp_size:
            raise ValueError(f"num_kv_heads ({num_kv_heads}) must be divisible by tp_size ({self.tp_size})")
        if intermediate_size < self.tp_size:
            raise ValueError(f"intermediate_size ({intermediate_size}) is smaller than tp_size ({self.tp_size})")


class TensorParallelGroup:
    """One instance per rank; every rank calls the collectives in the same order."""

    def __init__(self, tp_size: int, rank: int, backend: str = "cuda", unique_id=None, stream: int = 0):
        self.tp_size, self.rank, self.backend = tp_size, rank, backend
        self._comm: Optional[NcclComm] = None
        self._owns_group = False
        if tp_size <= 1:
            return
        if not dist.is_initialized():
            if unique_id is None:
                raise ValueError("unique_id (the rendezvous address 'host:port') is required for tp_size > 1")
            addr = unique_id.decode() if isinstance(unique_id, (bytes, bytearray)) else str(unique_id)
            host, _, port = addr.rpartition(":")
            os.environ.setdefault("MASTER_ADDR", host or "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", port)
            on_gpu = backend != "cpu" and torch.cuda.is_available()
            if on_gpu:
                torch.cuda.set_device(rank % torch.cuda.device_count())
            dist.init_process_group("nccl" if on_gpu else "gloo", rank=rank, world_size=tp_size)
            self._owns_group = True
        device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else \
            torch.device("cpu")
        self._comm = NcclComm(rank, tp_size, device)

    # ---- collectives ------------------------------------------------------------------------------------
    def all_reduce_inplace(self, tensor: torch.Tensor, op: str = "sum") -> None:
        if self._comm is None:
            return
        ops = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN,
               "prod": dist.ReduceOp.PRODUCT}
        dist.all_reduce(tensor, op=ops[op])

    def all_gather(self, tensor: torch.Tensor) -> torch.Tensor:
        return tensor if self._comm is None else self._comm.all_gather(tensor)

    def broadcast(self, tensor: torch.Tensor, root: int = 0) -> torch.Tensor:
        return tensor if self._comm is None else self._comm.broadcast(tensor, src=root)

    def reduce_scatter(self, tensor: torch.Tensor) -> torch.Tensor:
        return tensor if self._comm is None else self._comm.reduce_scatter(tensor)

    def barrier(self) -> None:
        if self._comm is not None:
            self._comm.barrier()

    def sync_stream(self) -> None:
        if self._comm is not None and self._comm.device.type == "cuda":
            torch.cuda.current_stream().synchronize()

    # ---- sharding ---------------------------------------------------------------------------------------
    def get_split_strategy(self, weight_name: str) -> str:
        for table in (NON_LAYER_SPLIT_MAP, WEIGHT_SPLIT_MAP):
            for suffix, strategy in table.items():
                if weight_name == suffix or weight_name.endswith("." + suffix) or weight_name.endswith(suffix):
                    return strategy
        return REPLICATED

    def compute_shard_range(self, full_size: int, strategy: str, unit: int = 1) -> Tuple[int, int]:
        """``[start, end)`` of this rank's shard of a dimension of ``full_size``; ``unit`` keeps shard borders on
        multiples of it (heads, quantisation groups), shards may then differ by one unit."""
        if self.tp_size <= 1 or strategy == REPLICATED:
            return 0, full_size
        if unit > 1 and full_size % unit == 0:
            a, b = split_units(full_size // unit, self.tp_size)[self.rank]
            return a * unit, b * unit
        return split_units(full_size, self.tp_size)[self.rank]

    def shard_size(self, full_size: int, strategy: str, unit: int = 1) -> int:
        a, b = self.compute_shard_range(full_size, strategy, unit)
        return b - a

    def destroy(self) -> None:
        self._comm = None
        if self._owns_group and dist.is_initialized():
            dist.destroy_process_group()
            self._owns_group = False

    def __repr__(self) -> str:
        return f"TensorParallelGroup(tp={self.tp_size}, rank={self.rank}, backend={self.backend})"


def is_nccl_available(backend: str = "cuda") -> bool:
    return bool(dist.is_available() and dist.is_nccl_available() and torch.cuda.is_available())


class NcclCommunicator:
    """The communicator of the reference's NCCL wrapper (zse-compiler/zse_compiler/runtime/nccl.py:174-410) for
    callers that use it directly.  Buffers are tensors here (the reference passes raw device addresses and element
    counts); collectives run on the current stream of the process group's backend."""

    def __init__(self, nranks: int, rank: int, unique_id=None, backend: str = "cuda", stream: int = 0):
        self._group = TensorParallelGroup(nranks, rank, backend, unique_id, stream)

    @property
    def rank(self) -> int:
        return self._group.rank

    @property
    def nranks(self) -> int:
        return self._group.tp_size

    def all_reduce(self, sendbuf: torch.Tensor, recvbuf: Optional[torch.Tensor] = None, count: Optional[int] = None,
                   dtype=None, op: str = "sum", stream=None) -> torch.Tensor:
        out = sendbuf if recvbuf is None or recvbuf is sendbuf else recvbuf.copy_(sendbuf)
        self._group.all_reduce_inplace(out, op)
        return out

    def all_reduce_inplace(self, buf: torch.Tensor, count: Optional[int] = None, dtype=None, op: str = "sum",
                           stream=None) -> None:
        self._group.all_reduce_inplace(buf, op)

    def all_gather(self, sendbuf: torch.Tensor, recvbuf: Optional[torch.Tensor] = None, sendcount=None, dtype=None,
                   stream=None) -> torch.Tensor:
        got = self._group.all_gather(sendbuf)
        return got if recvbuf is None else recvbuf.view(-1).copy_(got.view(-1)).view_as(recvbuf)

    def broadcast(self, buf: torch.Tensor, count=None, dtype=None, root: int = 0, stream=None) -> torch.Tensor:
        return self._group.broadcast(buf, root)

    def reduce_scatter(self, sendbuf: torch.Tensor, recvbuf: Optional[torch.Tensor] = None, recvcount=None, dtype=None,
                       op: str = "sum", stream=None) -> torch.Tensor:
        got = self._group.reduce_scatter(sendbuf)
        return got if recvbuf is None else recvbuf.view(-1).copy_(got.view(-1)).view_as(recvbuf)

    def barrier(self) -> None:
        self._group.barrier()

    def stream_synchronize(self) -> None:
        self._group.sync_stream()

    def destroy(self) -> None:
        self._group.destroy()

    def __repr__(self) -> str:
        return f"NcclCommunicator(rank={self.rank}, nranks={self.nranks})"


NCCL_UNIQUE_ID_BYTES = 128


class NcclUniqueId(ctypes.Structure):
    """The reference's 128-byte id record (zse-compiler/zse_compiler/runtime/nccl.py:69-71).  Here the id that ranks
    share is the rendezvous address; ``from_address`` / ``address`` move it in and out of the record, for code that
    passes ids around in this form."""
    _fields_ = [("internal", ctypes.c_char * NCCL_UNIQUE_ID_BYTES)]

    @classmethod
    def from_address_string(cls, address) -> "NcclUniqueId":
        raw = address if isinstance(address, (bytes, bytearray)) else str(address).encode()
        if len(raw) >= NCCL_UNIQUE_ID_BYTES:
            raise ValueError("the rendezvous address does not fit a 128-byte id")
        uid = cls()
        uid.internal = bytes(raw)
        return uid

    @property
    def address(self) -> bytes:
        return bytes(self.internal).split(b"\x00", 1)[0]


def get_unique_id(backend: str = "cuda") -> bytes:
    """A rendezvous address on this host with a free port, in the place of the reference's NCCL unique id."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return f"127.0.0.1:{s.getsockname()[1]}".encode()


def comm_init_all(ndev: int, backend: str = "cuda"):
    """The reference builds every rank's communicator inside one process here
    (zse-compiler/zse_compiler/runtime/nccl.py:134-165, ``ncclCommInitAll``) and drives the GPUs from threads.  This
    package runs one process per GPU, so there is nothing of that shape to return: the call says so and names the
    entry points that start the ranks."""
    raise RuntimeError(f"comm_init_all({ndev}): ranks are separate processes here, one per GPU; start them with "
                       "tp_launch(tp_size, rank_fn) or TPEngine, which hand every rank its communicator")


def _tp_worker(rank, tp_size, uid, backend, rank_fn, result_q, error_q):
    try:
        result_q.put((rank, rank_fn(rank, tp_size, uid, backend)))
    except Exception as exc:                     # reported to the parent, which raises
        error_q.put((rank, f"{type(exc).__name__}: {exc}"))


def tp_launch(tp_size: int, rank_fn: Callable[[int, int, bytes, str], Any], backend: str = "cuda",
              timeout_s: float = 600.0) -> List[Any]:
    """Runs ``rank_fn(rank, tp_size, unique_id, backend)`` in ``tp_size`` processes and returns their results in rank
    order.  ``rank_fn`` must be importable (a module-level function): the ranks are spawned, not forked."""
    if tp_size <= 1:
        raise ValueError("tp_launch requires tp_size >= 2")
    uid = get_unique_id(backend)
    ctx = multiprocessing.get_context("spawn")
    result_q, error_q = ctx.Queue(), ctx.Queue()
    procs = [ctx.Process(target=_tp_worker, args=(r, tp_size, uid, backend, rank_fn, result_q, error_q))
             for r in range(tp_size)]
    for p in procs:
        p.start()
    results: List[Any] = [None] * tp_size
    got = 0
    errors: List[str] = []
    import queue as _queue
    import time as _time
    deadline = _time.monotonic() + timeout_s
    while got + len(errors) < tp_size and _time.monotonic() < deadline:
        try:
            rank, res = result_q.get(timeout=0.2)
            results[rank] = res
            got += 1
        except _queue.Empty:
            pass
        while not error_q.empty():
            rank, msg = error_q.get_nowait()
            errors.append(f"Rank {rank}: {msg}")
        if all(not p.is_alive() for p in procs) and result_q.empty() and error_q.empty():
            break
    for p in procs:
        p.join(timeout=10)
        if p.is_alive():
            p.kill()
    if errors or got < tp_size:
        raise RuntimeError("Tensor parallel launch failed:\n" + "\n".join(errors or ["a rank ended without a result"]))
    return results
