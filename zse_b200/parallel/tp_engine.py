"""Tensor-parallel serving: one worker process per GPU, fronted by an object with the streamer's interface.

The reference's ``TPEngine`` (zse-engine/zse_engine/orchestrator/tp_engine.py:46-482) decodes one sequence at a time
and has none of the methods its HTTP server calls.  Here every rank runs the full continuous-batching engine
(``ZStreamerEngine``) on its shard, SPMD: rank 0 receives commands (new requests, cancellations, stop) from the
parent through a queue and broadcasts them over a gloo group before every step, so all ranks schedule the same
batch and stay in lock-step; token ids are identical on all ranks by construction (``comm.select_tokens``), rank 0
reports them back.  The parent keeps the tokenizer, turns events into ``on_token`` / ``on_finish`` callbacks and
watches the workers:

* every worker bumps a heartbeat counter between steps; a worker that exits, raises or stops beating marks the
  group unhealthy, in-flight requests finish with ``error`` and new ones are refused, while the HTTP front end keeps
  answering;
* ``restart()`` tears the group down and brings it up again from the model file (cold start is cheap).

With ``device="cpu"`` the workers use gloo and the torch reference ops, which is how the control plane and the
failure handling are tested without GPUs.
"""
from __future__ import annotations

import os
import queue
import threading
import time
import traceback
from dataclasses import dataclass
from typing import Callable, Dict, Iterator, List, Optional

import torch
import torch.multiprocessing as mp

from ..config import EngineConfig
from ..sched.request import FinishReason, RequestOutput

CMD_ADD, CMD_CANCEL, CMD_STOP, CMD_FAIL = "add", "cancel", "stop", "fail"


def _free_port() -> int:
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, model_path: str, cfg: EngineConfig, port: int, cmd_q, evt_q, beats, ready) -> None:
    """Body of one rank.  ``cmd_q`` is only read by rank 0."""
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    try:
        on_gpu = torch.cuda.is_available() and cfg.device != "cpu"
        if on_gpu:
            torch.cuda.set_device(rank)
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
        ctrl = dist.new_group(backend="gloo")          # control plane (objects), separate from the data group
        from ..engine import ZStreamerEngine
        from .comm import make_comm
        from ..format.loader import ZSELoader
        cfg = EngineConfig(**{**cfg.__dict__, "tp_size": world, "device_index": rank, "quiet": True})
        with ZSELoader(model_path) as l:
            hidden = l.config.hidden_size
        dev = torch.device(f"cuda:{rank}" if on_gpu else "cpu")
        # the plain collective paths also run on gloo; the fused kernels need GPUs
        backend = cfg.comm_backend if on_gpu or cfg.comm_backend.startswith("nccl") else "nccl"
        comm = make_comm(backend, rank, world, dev, hidden_size=hidden,
                         max_tokens=max(cfg.max_batch_tokens, cfg.prefill_chunk_size))
        eng = ZStreamerEngine(model_path, config=cfg, comm=comm, tp_rank=rank)
        if rank == 0:
            info = dict(eng.init_times)
            if on_gpu:
                props = torch.cuda.get_device_properties(dev)
                info["device_name"], info["device_vram_gb"] = props.name, props.total_memory / 2 ** 30
            else:
                info["device_name"], info["device_vram_gb"] = "cpu", 0.0
            ready.put(("ready", info))
        fail_at = None
        # time-based decisions (time-outs, deadline order) use rank 0's clock of this iteration on every rank
        from ..sched import request as _request
        tick = [time.monotonic()]
        _request.set_decision_clock(lambda: tick[0])
        while True:
            beats[rank] += 1
            if rank == 0:
                cmds = []
                try:
                    cmds.append(cmd_q.get(timeout=0.0005 if eng.has_work() else 0.02))
                    while True:
                        cmds.append(cmd_q.get_nowait())
                except queue.Empty:
                    pass
                box = [cmds, time.monotonic()]
            else:
                box = [None, 0.0]
            dist.broadcast_object_list(box, src=0, group=ctrl)
            tick[0] = box[1]
            stop = False
            for c in box[0]:
                if c[0] == CMD_ADD:
                    _, rid, ids, kw = c
                    cbs = {}
                    if rank == 0:
                        cbs = {"on_token": (lambda t, r=rid: evt_q.put(("tok", r, t))),
                               "on_finish": (lambda o, r=rid: evt_q.put(("end", r, o)))}
                    try:
                        if eng.add_request_tokens(ids, request_id=rid, **kw, **cbs) is None and rank == 0:
                            evt_q.put(("rejected", rid, "request queue is full"))
                    except Exception as exc:
                        if rank == 0:
                            evt_q.put(("rejected", rid, str(exc)))
                elif c[0] == CMD_CANCEL:
                    eng.cancel_request(c[1])
                elif c[0] == CMD_FAIL and c[1] == rank:     # test hook: this rank leaves between steps
                    fail_at = c[2]
                elif c[0] == CMD_STOP:
                    stop = True
            if stop:
                break
            if fail_at == "raise":
                raise RuntimeError("injected worker failure")
            if fail_at == "exit":
                os._exit(17)
            if eng.has_work():
                eng.step()
        dist.barrier(group=ctrl)
        dist.destroy_process_group()
    except Exception:
        try:
            evt_q.put(("worker_error", rank, traceback.format_exc()))
            ready.put(("error", traceback.format_exc()))
        except Exception:
            pass
        os._exit(1)


@dataclass
class TPStats:
    healthy: bool
    tp_size: int
    total_requests: int
    total_tokens_generated: int
    active_requests: int
    uptime_s: float
    restarts: int
    last_error: Optional[str]


@dataclass
class TPEngineStats:
    """What start-up cost, under the reference's field names (zse-engine/zse_engine/orchestrator/tp_engine.py:54-62).
    ``kernel_compile_time_s`` is the time to bring up buffers, graphs and the communication layer: the kernels are
    built ahead of time."""
    tp_size: int
    backend: str
    device_names: List[str]
    total_vram_gb: float
    weight_load_time_s: float
    kernel_compile_time_s: float
    total_init_time_s: float


class TPEngine:
    """Parent-side handle with the part of ``ZStreamerEngine``'s interface the HTTP layer uses."""

    HEARTBEAT_TIMEOUT_S = 30.0

    def __init__(self, model_path: str, tp_size: int = 2, config=None, start_timeout_s: float = 600.0,
                 quiet: Optional[bool] = None):
        """``config``: an ``EngineConfig``; the reference's third argument is ``quiet`` (zse-engine/zse_engine/
        orchestrator/tp_engine.py:46-63), so a bool given there is taken as that."""
        from ..format.loader import ZSELoader
        if isinstance(config, bool):
            quiet, config = config, None
        self.model_path, self.tp_size = model_path, tp_size
        self.engine_config = config or EngineConfig(tp_size=tp_size)
        self.engine_config.tp_size = tp_size
        if quiet is not None:
            self.engine_config.quiet = bool(quiet)
        with ZSELoader(model_path) as l:
            self._config = l.config
            self._tokenizer = l.tokenizer
        self._max_seq_len = min(self.engine_config.max_seq_len or self._config.max_seq_len, self._config.max_seq_len, 32768)
        self._lock = threading.Lock()
        self._pending: Dict[str, dict] = {}
        self._completed: Dict[str, RequestOutput] = {}
        self._counter = 0
        self._running = False
        self._healthy = False
        self._last_error: Optional[str] = None
        self._restarts = -1
        self._total_requests = self._total_tokens = 0
        self._start_time = time.monotonic()
        self._start_timeout = start_timeout_s
        self._procs: List[mp.Process] = []
        self.init_times: dict = {}
        self._start_workers()

    # ---- worker management --------------------------------------------------------------------------------
    def _start_workers(self) -> None:
        ctx = mp.get_context("spawn")
        self._cmd_q, self._evt_q, ready = ctx.Queue(), ctx.Queue(), ctx.Queue()
        self._beats = ctx.Array("q", self.tp_size, lock=False)
        port = _free_port()
        self._procs = [ctx.Process(target=_worker, daemon=True,
                                   args=(r, self.tp_size, self.model_path, self.engine_config, port, self._cmd_q,
                                         self._evt_q, self._beats, ready)) for r in range(self.tp_size)]
        for p in self._procs:
            p.start()
        try:
            kind, info = ready.get(timeout=self._start_timeout)
        except queue.Empty:
            self._kill()
            raise RuntimeError(f"tensor-parallel workers did not come up within {self._start_timeout:.0f} s")
        if kind != "ready":
            self._kill()
            raise RuntimeError(f"tensor-parallel worker failed to start:\n{info}")
        self.init_times = info
        self._healthy = True
        self._restarts += 1
        self._beat_seen = (list(self._beats), time.monotonic())

    def _kill(self) -> None:
        for p in self._procs:
            if p.is_alive():
                p.terminate()
        for p in self._procs:
            p.join(timeout=5)
        self._procs = []
        self._healthy = False

    def restart(self) -> None:
        """Tear the group down and bring it up again from the model file; in-flight requests are failed first."""
        self._fail_all("tensor-parallel group restarted")
        self._kill()
        self._start_workers()

    def _check_health(self) -> None:
        if not self._healthy:
            return
        dead = [i for i, p in enumerate(self._procs) if not p.is_alive()]
        now = time.monotonic()
        beats = list(self._beats)
        if beats != self._beat_seen[0]:
            self._beat_seen = (beats, now)
        stalled = now - self._beat_seen[1] > self.HEARTBEAT_TIMEOUT_S
        if dead or stalled:
            why = f"worker rank(s) {dead} exited" if dead else f"no heartbeat for {self.HEARTBEAT_TIMEOUT_S:.0f} s"
            self._mark_unhealthy(why)

    def _mark_unhealthy(self, why: str) -> None:
        self._healthy = False
        self._last_error = why
        self._fail_all(why)
        # ranks that survive sit in a collective that can never complete: take them down too
        self._kill()

    def _fail_all(self, why: str) -> None:
        with self._lock:
            pending, self._pending = self._pending, {}
        for rid, rec in pending.items():
            out = RequestOutput(rid, rec["prompt"], rec["tokens"], FinishReason.ERROR, 0.0,
                                (time.monotonic() - rec["t0"]) * 1000.0, 0.0, 0.0, why)
            self._deliver_finish(rid, rec, out)

    # ---- the streamer interface ---------------------------------------------------------------------------
    @property
    def tokenizer(self):
        return self._tokenizer

    @property
    def config(self):
        """The model's configuration, as ``TPEngine.config`` of the reference."""
        return self._config

    @property
    def model_config(self):
        return self._config

    @property
    def lora_manager(self):
        return None        # adapters under tensor parallelism are loaded per worker; not exposed over HTTP yet

    @property
    def healthy(self) -> bool:
        return self._healthy

    def default_stop_tokens(self) -> List[int]:
        from ..engine import CHAT_STOP_MARKERS
        stops, tok = [], self._tokenizer
        if tok is None:
            return stops
        eos = tok.special_tokens.eos_id
        if eos is not None and not (self._config.vocab_size > 50000 and eos < 100):
            stops.append(eos)
        for m in CHAT_STOP_MARKERS:
            tid = tok.token_to_id(m)
            if tid is not None and tid not in stops:
                stops.append(tid)
        return stops

    def add_request(self, prompt: str, **kw) -> Optional[str]:
        if self._tokenizer is None:
            raise RuntimeError("this model file has no tokenizer; use add_request_tokens")
        return self.add_request_tokens(self._tokenizer.encode(prompt), **kw)

    def add_request_tokens(self, token_ids: List[int], request_id: Optional[str] = None,
                           on_token: Optional[Callable] = None, on_finish: Optional[Callable] = None,
                           stop_tokens: Optional[List[int]] = None, **kw) -> Optional[str]:
        if not self._healthy:
            return None
        if len(token_ids) == 0:
            raise ValueError("empty prompt")
        if len(token_ids) >= self._max_seq_len:
            raise ValueError(f"prompt length {len(token_ids)} exceeds max_seq_len {self._max_seq_len}")
        if kw.get("lora_id") is not None:
            raise ValueError("LoRA adapters are not available with --tp > 1 yet")
        kw.pop("lora_id", None)
        with self._lock:
            if len(self._pending) >= self.engine_config.max_queue_size + self.engine_config.max_batch_seqs:
                return None
            self._counter += 1
            rid = request_id or f"req-{self._counter}"
            self._pending[rid] = {"on_token": on_token, "on_finish": on_finish, "prompt": list(token_ids),
                                  "tokens": [], "t0": time.monotonic()}
            self._total_requests += 1
        kw["stop_tokens"] = self.default_stop_tokens() if stop_tokens is None else list(stop_tokens)
        self._cmd_q.put((CMD_ADD, rid, list(token_ids), kw))
        return rid

    def cancel_request(self, request_id: str) -> None:
        if self._healthy:
            self._cmd_q.put((CMD_CANCEL, request_id))

    def inject_failure(self, rank: int, how: str = "exit") -> None:
        """Test hook: the given rank leaves between two steps (``"exit"``) or raises (``"raise"``)."""
        self._cmd_q.put((CMD_FAIL, rank, how))

    def _deliver_finish(self, rid: str, rec: dict, out: RequestOutput) -> None:
        with self._lock:
            self._completed[rid] = out
            if len(self._completed) > 10000:
                self._completed.pop(next(iter(self._completed)))
        if rec.get("on_finish") is not None:
            try:
                rec["on_finish"](out)
            except Exception:
                pass

    def poll(self, timeout: float = 0.01) -> int:
        """Drains worker events (tokens, finished requests, errors); returns how many were handled."""
        n = 0
        try:
            evt = self._evt_q.get(timeout=timeout)
        except queue.Empty:
            self._check_health()
            return 0
        while True:
            n += 1
            kind = evt[0]
            if kind == "tok":
                rec = self._pending.get(evt[1])
                if rec is not None:
                    rec["tokens"].append(evt[2])
                    self._total_tokens += 1
                    if rec["on_token"] is not None:
                        try:
                            rec["on_token"](evt[2])
                        except Exception:
                            pass
            elif kind == "end":
                with self._lock:
                    rec = self._pending.pop(evt[1], None)
                if rec is not None:
                    self._deliver_finish(evt[1], rec, evt[2])
            elif kind == "rejected":
                with self._lock:
                    rec = self._pending.pop(evt[1], None)
                if rec is not None:
                    out = RequestOutput(evt[1], rec["prompt"], [], FinishReason.ERROR, 0.0, 0.0, 0.0, 0.0, evt[2])
                    self._deliver_finish(evt[1], rec, out)
            elif kind == "worker_error":
                self._mark_unhealthy(f"rank {evt[1]} failed: {evt[2].strip().splitlines()[-1]}")
            try:
                evt = self._evt_q.get_nowait()
            except queue.Empty:
                break
        self._check_health()
        return n

    def run(self) -> None:
        """Event pump (call from a dedicated thread); returns after ``stop()``."""
        self._running = True
        while self._running:
            self.poll(0.02)

    def run_until_done(self, timeout_s: float = 600.0) -> None:
        t0 = time.monotonic()
        while self._pending and time.monotonic() - t0 < timeout_s:
            self.poll(0.02)

    def has_work(self) -> bool:
        return bool(self._pending)

    # ---- one request at a time (zse-engine/zse_engine/orchestrator/tp_engine.py:329-443) ------------------------
    def stream_generate_tokens(self, prompt: str, max_tokens: int = 128, temperature: float = 1.0, top_k: int = 50,
                               top_p: float = 0.9, stop_tokens: Optional[List[int]] = None,
                               timeout_s: float = 600.0, **kw) -> Iterator[int]:
        """Yields the generated token ids of one request while polling the ranks on the calling thread."""
        fresh: List[int] = []
        done: List[RequestOutput] = []
        rid = self.add_request(prompt, max_tokens=max_tokens, temperature=temperature, top_k=top_k, top_p=top_p,
                               stop_tokens=stop_tokens, on_token=fresh.append, on_finish=done.append, **kw)
        if rid is None:
            raise RuntimeError("the tensor-parallel engine is not accepting requests: " + str(self._last_error))
        deadline = time.monotonic() + timeout_s
        try:
            while not done and time.monotonic() < deadline:
                self.poll(0.01)
                while fresh:
                    yield fresh.pop(0)
            while fresh:
                yield fresh.pop(0)
        finally:
            if not done:
                self.cancel_request(rid)
        self.get_result(rid)
        if not done:
            raise TimeoutError(f"no answer from the ranks within {timeout_s}s")
        if done[0].finish_reason == FinishReason.ERROR:
            raise RuntimeError(f"generation failed: {done[0].error}")

    def generate(self, prompt: str, max_tokens: int = 128, temperature: float = 1.0, top_k: int = 50,
                 top_p: float = 0.9, stop_tokens: Optional[List[int]] = None, **kw) -> str:
        stops = set(self.default_stop_tokens() if stop_tokens is None else stop_tokens)
        ids = [t for t in self.stream_generate_tokens(prompt, max_tokens, temperature, top_k, top_p, stop_tokens, **kw)
               if t not in stops]
        return self._tokenizer.decode(ids)

    def stream_generate(self, prompt: str, max_tokens: int = 128, temperature: float = 1.0, top_k: int = 50,
                        **kw) -> Iterator[str]:
        stops = set(self.default_stop_tokens() if kw.get("stop_tokens") is None else kw["stop_tokens"])
        ids: List[int] = []
        sent = ""
        for t in self.stream_generate_tokens(prompt, max_tokens, temperature, top_k, **kw):
            if t in stops:
                continue
            ids.append(t)
            text = self._tokenizer.decode(ids)
            if not text.endswith("\ufffd") and len(text) > len(sent):
                yield text[len(sent):]
                sent = text
        text = self._tokenizer.decode(ids)
        if len(text) > len(sent):
            yield text[len(sent):]

    def summary(self) -> str:
        st = self.stats()
        rate = st.total_tokens_generated / st.uptime_s if st.uptime_s > 0 else 0.0
        return (f"TPEngine: {self.tp_size}-way tensor parallel ({'healthy' if st.healthy else 'unhealthy'})\n"
                f"  model: {self.model_path}\n  init: {self.init_times.get('total', 0.0):.2f}s\n"
                f"  tokens generated: {st.total_tokens_generated} ({rate:.1f} tok/s over the uptime)")

    def get_result(self, request_id: str) -> Optional[RequestOutput]:
        with self._lock:
            return self._completed.pop(request_id, None)

    def init_stats(self) -> TPEngineStats:
        t = self.init_times
        name = str(t.get("device_name", "cpu"))
        return TPEngineStats(self.tp_size, "cpu" if name == "cpu" else "cuda",
                             [f"{name} #{r}" for r in range(self.tp_size)],
                             float(t.get("device_vram_gb", 0.0)) * self.tp_size, float(t.get("weights", 0.0)),
                             float(t.get("runtime", 0.0)), float(t.get("total", 0.0)))

    def stats(self) -> TPStats:
        return TPStats(self._healthy, self.tp_size, self._total_requests, self._total_tokens, len(self._pending),
                       time.monotonic() - self._start_time, max(self._restarts, 0), self._last_error)

    def stop(self) -> None:
        self._running = False
        if self._healthy and self._procs:
            try:
                self._cmd_q.put((CMD_STOP,))
                for p in self._procs:
                    p.join(timeout=10)
            except Exception:
                pass
        self._kill()

    destroy = stop
