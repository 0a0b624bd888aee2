"""Tensor-parallel collectives of the decoder.

Two back ends behind one interface:

``FusedComm`` (product path) - the reduction after every row-parallel projection happens inside
  ``tp_reduce_add_rmsnorm`` (csrc/comm.cu): split-K planes -> fp16 row in symmetric memory -> per-row flags pushed to
  the peers -> rows pulled over NVLink (or reduced in the NVSwitch with ``multimem.ld_reduce``) -> residual add ->
  RMSNorm, all in one kernel and without a NCCL call; greedy token selection over the vocabulary-sharded lm_head uses
  the same flag protocol (``tp_argmax``).  Symmetric buffers come from ``torch.distributed._symmetric_memory``.
``NcclComm`` (baseline) - ``dist.all_reduce`` between the unfused kernels, like the reference's ``ncclAllReduce``
  after o_proj and down_proj (zse-engine/zse_engine/orchestrator/model_runner.py:2622-2635,2694-2705).

Both are SPMD: every rank runs the same engine on the same requests, so no control plane is needed in the hot loop.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist
from ..utils import env


class NcclComm:
    name = "nccl"
    graph_safe = True          # NCCL collectives can be captured in CUDA graphs
    fused_norm = False

    def __init__(self, rank: int, world: int, device, group=None, sequence_parallel: Optional[bool] = None):
        self.rank, self.world, self.device, self.group = rank, world, device, group
        self._gather = None
        # sequence parallelism for passes of at least ``sp_min_rows`` tokens: the residual stream is split by rows,
        # a reduce-scatter follows each row-parallel projection and an all-gather precedes each column-parallel one
        if sequence_parallel is None:
            sequence_parallel = env.flag("ZSE_TP_SP")
        self.sequence_parallel = bool(sequence_parallel)
        self.sp_min_rows = env.integer("ZSE_TP_SP_MIN_ROWS")
        self.sp_passes = 0
        self._sp_bufs: dict = {}

    def use_sequence_parallel(self, M: int) -> bool:
        return self.sequence_parallel and M >= max(self.sp_min_rows, self.world)

    def _sp_buf(self, name: str, rows: int, H: int, dtype) -> torch.Tensor:
        t = self._sp_bufs.get(name)
        if t is None or t.shape[0] < rows or t.shape[1] != H or t.dtype != dtype:
            t = self._sp_bufs[name] = torch.zeros(rows, H, dtype=dtype, device=self.device)
        return t[:rows]

    def reduce_scatter_add_rmsnorm(self, ops, residual, partials, planes: int, weight, out, M: int, eps: float) -> None:
        """Sequence-parallel form of "sum over ranks, add to the residual, normalise": every rank receives the sum of
        its own ``ceil(M / world)`` rows only (reduce-scatter), adds them to its rows of the residual stream and
        normalises those, and the normalised rows are gathered so that the column-parallel projection that follows
        sees all ``M``.  Same bytes on the wire as the all-reduce, 1/world of the residual and norm work per rank,
        and rows of the residual a rank does not own are never touched again after the embedding."""
        H, w = partials.shape[-1], self.world
        m = (M + w - 1) // w
        pl = partials.view(-1)[: planes * M * H].view(planes, M, H)
        full = self._sp_buf("send", m * w, H, pl.dtype)
        if planes > 1:
            torch.sum(pl, dim=0, out=full[:M])
        else:
            full[:M].copy_(pl[0])
        if m * w > M:
            full[M:].zero_()
        mine = self._sp_buf("mine", m, H, pl.dtype)
        try:
            dist.reduce_scatter_tensor(mine, full, group=self.group)
        except (RuntimeError, NotImplementedError):     # back ends without the primitive (gloo)
            dist.all_reduce(full, group=self.group)
            mine.copy_(full[self.rank * m: (self.rank + 1) * m])
        r0 = self.rank * m
        n = max(0, min(M, r0 + m) - r0)
        normed = self._sp_buf("normed", m, H, out.dtype)
        if n < m:
            normed[n:].zero_()
        if n > 0:
            ops.add_rmsnorm(residual[r0:r0 + n], mine, 1, None, weight, normed, n, eps)
        gathered = self._sp_buf("gathered", m * w, H, out.dtype)
        try:
            dist.all_gather_into_tensor(gathered, normed, group=self.group)
        except (RuntimeError, NotImplementedError):
            parts = [torch.empty_like(normed) for _ in range(w)]
            dist.all_gather(parts, normed, group=self.group)
            torch.cat(parts, dim=0, out=gathered)
        out[:M].copy_(gathered[:M])
        self.sp_passes += 1

    def all_reduce_partials(self, partials: torch.Tensor, planes: int, M: int) -> int:
        """Sums this rank's planes into plane 0 and all-reduces it; returns the number of planes left (1)."""
        H = partials.shape[-1]
        pl = partials.view(-1)[: planes * M * H].view(planes, M, H)      # planes are packed: [plane][M rows][H]
        p0 = pl[0]
        if planes > 1:
            p0.add_(pl[1:].sum(dim=0))
        dist.all_reduce(p0, group=self.group)
        return 1

    def select_tokens(self, runner, n_rows: int, greedy: bool, step: int) -> None:
        b, ops, plan = runner.buf, runner.model.ops, runner.model.plan
        V = plan.vocab_size
        stride = (runner.model.config.vocab_size + self.world - 1) // self.world
        if greedy:
            vals, idx = b.logits[:n_rows, :V].float().max(dim=-1)
            both = torch.stack([vals, (idx + plan.vocab[0]).float()], dim=-1).contiguous()
            parts = [torch.empty_like(both) for _ in range(self.world)]
            dist.all_gather(parts, both, group=self.group)
            gathered = torch.stack(parts, dim=0)
            best = gathered[:, :, 0].argmax(dim=0)       # first rank wins ties -> lowest token id
            b.out_tokens[:n_rows] = gathered[best, torch.arange(n_rows, device=self.device), 1].to(torch.int32)
        else:
            full = self.gather_logits(runner, n_rows)
            ops.sample(full, b.out_tokens, n_rows, b.temperature, b.top_k, b.top_p, b.seeds, step)

    def gather_logits(self, runner, n_rows: int) -> torch.Tensor:
        """Full-vocabulary fp16 logits [n_rows, vocab] on every rank (shards may be uneven by one row)."""
        b, plan = runner.buf, runner.model.plan
        vocab = runner.model.config.vocab_size
        width = (vocab + self.world - 1) // self.world
        local = torch.full((n_rows, width), float("-inf"), dtype=torch.float16, device=self.device)
        local[:, : plan.vocab_size] = b.logits[:n_rows, : plan.vocab_size]
        out = [torch.empty_like(local) for _ in range(self.world)]
        dist.all_gather(out, local, group=self.group)
        from .shard_plan import split_units
        parts = [out[r][:, : hi - lo] for r, (lo, hi) in enumerate(split_units(vocab, self.world))]
        return torch.cat(parts, dim=1).contiguous()

    def barrier(self) -> None:
        dist.barrier(group=self.group)

    # ---- general collectives (the facade of the reference's TensorParallelGroup,
    # zse-engine/zse_engine/orchestrator/tensor_parallel.py:158-203): sum all-reduce in place, all-gather along
    # dim 0, broadcast from a rank, sum reduce-scatter along dim 0.  The decoder's hot loop uses the fused kernels;
    # these serve model families without a fused path and user code.
    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(t, group=self.group)
        return t

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        parts = [torch.empty_like(t) for _ in range(self.world)]
        dist.all_gather(parts, t.contiguous(), group=self.group)
        return torch.cat(parts, dim=0)

    def broadcast(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        dist.broadcast(t, src=src, group=self.group)
        return t

    def reduce_scatter(self, t: torch.Tensor) -> torch.Tensor:
        """Rank r gets rows [r*n, (r+1)*n) of the sum over ranks; dim 0 must divide by the world size."""
        if t.shape[0] % self.world:
            raise ValueError(f"reduce_scatter: {t.shape[0]} rows do not divide by {self.world} ranks")
        n = t.shape[0] // self.world
        out = torch.empty((n,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        try:
            dist.reduce_scatter_tensor(out, t.contiguous(), group=self.group)
        except (RuntimeError, NotImplementedError):     # back ends without the primitive (gloo): reduce, then slice
            full = t.clone()
            dist.all_reduce(full, group=self.group)
            out.copy_(full[self.rank * n: (self.rank + 1) * n])
        return out

    def close(self) -> None:
        pass


class FusedComm(NcclComm):
    name = "fused"
    graph_safe = True
    fused_norm = True

    def __init__(self, rank: int, world: int, device, hidden_size: int, max_tokens: int, group=None,
                 use_multimem: Optional[bool] = None):
        super().__init__(rank, world, device, group)
        import torch.distributed._symmetric_memory as symm
        from ..ops import native
        self._n = native
        self.m_cap = max_tokens
        self.H = hidden_size
        grp = group or dist.group.WORLD
        # one symmetric allocation, carved into: row data, row flags, exchange words, exchange flags
        data_bytes = 2 * max_tokens * hidden_size * 2
        flag_bytes = 2 * world * max_tokens * 4
        xchg_bytes = 2 * world * max_tokens * 8
        align = lambda n: (n + 255) // 256 * 256
        offs = [0, align(data_bytes)]
        offs.append(offs[-1] + align(flag_bytes))
        offs.append(offs[-1] + align(xchg_bytes))
        total = offs[-1] + align(flag_bytes)
        self._buf = symm.empty(total, dtype=torch.uint8, device=device)
        self._buf.zero_()
        self._hdl = symm.rendezvous(self._buf, grp)
        torch.cuda.synchronize(device)
        dist.barrier(group=grp)
        ptrs = [int(p) for p in self._hdl.buffer_ptrs]
        want_mm = use_multimem if use_multimem is not None else env.flag("ZSE_TP_MULTIMEM")
        mc = 0
        if want_mm:
            try:
                mc = int(self._hdl.multicast_ptr or 0)     # 0 when the fabric has no NVLS multicast
            except Exception:
                mc = 0
        self.use_multimem = bool(mc) and want_mm
        self._ctx = native.tp_ctx_create(world, rank, max_tokens, hidden_size, [p + offs[0] for p in ptrs],
                                         [p + offs[1] for p in ptrs], (mc + offs[0]) if mc else 0,
                                         [p + offs[2] for p in ptrs], [p + offs[3] for p in ptrs])
        self._calls = 0
        # Push exchange (ZSE_TP_PUSH=1): the row-parallel GEMM itself sends its fp16 rows to every rank's inbox
        # (multimem.st through NVSwitch, or peer stores) and the consumer adds local rows only.
        self.push = env.flag("ZSE_TP_PUSH")
        self.push_rows = min(256, max_tokens)
        self._push_ready = False
        # Decode-sized passes: the row-parallel projection, the all-reduce, the residual add and the next RMSNorm are ONE
        # kernel (csrc/gemm_w4_dec.cu, kDecAllReduceNorm); it uses the same inboxes and counters as the push exchange.
        # measured per decode step of the 14B shape, one kernel vs two: 6.66 vs 6.20 ms on two GPUs, 5.45 vs 5.07 on
        # four, 5.14 vs 4.85 on eight (the kernel's tail - a grid-wide hand-over through L2 - costs more than the second
        # launch), so the two-kernel form is the default
        self.fused_k1 = env.flag("ZSE_TP_FUSED_K1")
        self.k1_calls = 0
        if self.push or self.fused_k1:
            self._init_push(symm, grp, world, rank, device, hidden_size, want_mm)
        # passes with at least this many rows (prefill) use the two-shot kernel: reduce-scatter by rows + all-gather,
        # 2(tp-1)/tp rows over NVLink per rank and row instead of tp-1
        self.two_shot_min_rows = env.integer("ZSE_TP_TWO_SHOT_ROWS")
        # Large passes (prefill) go through ncclAllReduce of the fp16 row sums by default: measured on B200 x2/x4, the
        # per-row kernels above lose to NCCL once a pass has hundreds of rows (they are built for latency, one CTA per
        # row), while for decode-sized passes they win by 1.2-1.4x.  ZSE_TP_NCCL_ROWS moves the switch-over point.
        self.nccl_min_rows = env.integer("ZSE_TP_NCCL_ROWS")
        self._f16: Optional[torch.Tensor] = None
        # Passes of many rows (prefill): the row-parallel GEMM scatters its tiles to the owners of 64-row blocks, the
        # owner reduces + normalises and stores the rows to every rank, and the next GEMM waits for its tiles' rows in
        # its prologue (csrc/gemm_w4.cu kEpiScatterF16 / gather_wait_tile, csrc/comm.cu tp_sp_sum_norm_gather_kernel).
        self.sp_min_rows = env.integer("ZSE_TP_FUSED_SP_ROWS")
        self.sp_xnorm: Optional[torch.Tensor] = None
        self.sp_calls = 0
        self._sp_slot = 0
        if self.sp_min_rows > 0 and hidden_size % 128 == 0 and hidden_size <= 8192:
            self._init_sp(symm, grp, world, rank, device, hidden_size, max_tokens, want_mm)

    def _init_push(self, symm, grp, world, rank, device, H, want_mm) -> None:
        align = lambda n: (n + 255) // 256 * 256
        inbox_bytes = 2 * world * self.push_rows * H * 2
        offs = [0, align(inbox_bytes)]
        total = offs[1] + align(2 * world * 4)
        self._pbuf = symm.empty(total, dtype=torch.uint8, device=device)
        self._pbuf.zero_()
        self._phdl = symm.rendezvous(self._pbuf, grp)
        torch.cuda.synchronize(device)
        dist.barrier(group=grp)
        ptrs = [int(p) for p in self._phdl.buffer_ptrs]
        mc = 0
        if want_mm:
            try:
                mc = int(self._phdl.multicast_ptr or 0)
            except Exception:
                mc = 0
        self.push_multimem = bool(mc)
        self._pstate = torch.zeros(4, dtype=torch.int32, device=device)
        state_ptrs = [self._pstate.data_ptr() if r == rank else 0 for r in range(world)]
        self._n.tp_ctx_set_push(self._ctx, self.push_rows, [p + offs[0] for p in ptrs], (mc + offs[0]) if mc else 0,
                                [p + offs[1] for p in ptrs], (mc + offs[1]) if mc else 0, state_ptrs)
        self._push_ready = True

    def _init_sp(self, symm, grp, world, rank, device, H, max_tokens, want_mm) -> None:
        align = lambda n: (n + 255) // 256 * 256
        nblk = (max_tokens + 63) // 64
        own_cap = (nblk + world - 1) // world * 64
        sizes = [2 * world * own_cap * H * 2, 2 * world * nblk * 4, nblk * 64 * H * 2, nblk * 4]
        offs = [0]
        for n in sizes:
            offs.append(offs[-1] + align(n))
        self._sbuf = symm.empty(offs[-1], dtype=torch.uint8, device=device)
        self._sbuf.zero_()
        self._shdl = symm.rendezvous(self._sbuf, grp)
        torch.cuda.synchronize(device)
        dist.barrier(group=grp)
        ptrs = [int(p) for p in self._shdl.buffer_ptrs]
        mc = 0
        if want_mm:
            try:
                mc = int(self._shdl.multicast_ptr or 0)
            except Exception:
                mc = 0
        self.sp_multimem = bool(mc)
        self._sstate = torch.zeros(4 + nblk, dtype=torch.int32, device=device)
        state_ptrs = [self._sstate.data_ptr() if r == rank else 0 for r in range(world)]
        self._n.tp_ctx_set_sp(self._ctx, own_cap, nblk, [p + offs[0] for p in ptrs], [p + offs[1] for p in ptrs],
                              [p + offs[2] for p in ptrs], (mc + offs[2]) if mc else 0, [p + offs[3] for p in ptrs],
                              state_ptrs)
        # the gathered activations are the decoder's normalised-activation buffer itself
        self.sp_xnorm = self._sbuf[offs[2]: offs[2] + nblk * 64 * H * 2].view(torch.float16).view(nblk * 64, H)

    def can_sp(self, w, M: int) -> bool:
        """Whether ``linear_scatter_norm`` takes this row-parallel projection."""
        return bool(self.sp_xnorm is not None and M >= max(65, self.sp_min_rows) and M <= self.sp_xnorm.shape[0]
                    and w.kind == "w4t" and w.N == self.H and w.bias is None)

    def linear_scatter_norm(self, ops, w, x, M: int, residual, weight, eps: float) -> None:
        """Own rows of ``residual`` += reduce-scatter(x W^T); ``sp_xnorm`` on every rank = RMSNorm of those rows.  Two
        launches, no NCCL: the GEMM's epilogue is the scatter, the reduce kernel's stores are the gather."""
        self._n.tp_gemm_w4_scatter(self._ctx, w.data, x, x.shape[0], M, w.N, w.K, self._sp_slot, ops.status.ptr)
        self._n.tp_sp_sum_norm_gather(self._ctx, residual, weight, M, float(eps), self._sp_slot, self.sp_multimem,
                                      ops.status.ptr)
        self._sp_slot ^= 1
        self.sp_calls += 1

    def sp_wait(self, ops, M: int) -> None:
        """Orders readers that are not gather-aware GEMMs after the arrival of all rows of the pass."""
        self._n.tp_sp_wait(self._ctx, M, ops.status.ptr)

    def can_fuse_k1(self, ops, w, M: int) -> bool:
        """Whether ``linear_allreduce_norm`` takes this projection (tiled INT4 / INT8 weights, at most 64 rows)."""
        return bool(self.fused_k1 and self._push_ready and w.kind in ("w4t", "w8t") and M <= min(64, self.push_rows)
                    and w.N == self.H and w.bias is None and self._n.gemm_w4_dec_supported(M, w.N, w.K, 4)
                    and self._n.gemm_w4_dec_plan(w.N, w.K, 4, ops.sm_count)[1] > 0)

    def linear_allreduce_norm(self, ops, w, x, M: int, residual, weight, out, eps: float) -> None:
        """residual += all-reduce(x W^T); out = RMSNorm(residual) * weight - one kernel, no NCCL, no separate reduce."""
        self._n.tp_gemm_dec_allreduce_norm(self._ctx, w.data, w.kind == "w8t", x, x.shape[0], M, w.N, w.K,
                                           self._calls & 1, self.push_multimem, residual, weight, out, float(eps),
                                           ops.dec_ws, ops.status.ptr)
        self._calls += 1
        self.k1_calls += 1

    def can_push(self, w, M: int) -> bool:
        # the older exchange in the epilogue of the tiled GEMM (ZSE_TP_PUSH=1) is validated on two and four ranks; on
        # eight it produced wrong tokens (cause not found), and the decode kernel's own exchange replaces it there
        return (self._push_ready and self.world <= 4 and w.kind == "w4t" and M <= self.push_rows and w.N == self.H
                and w.bias is None)

    def linear_push(self, ops, w, x, M: int) -> int:
        """Row-parallel INT4 GEMM with the exchange in its epilogue; returns the CTA count for sum_add_rmsnorm."""
        return self._n.tp_gemm_w4_push(self._ctx, w.data, x, x.shape[0], M, w.N, w.K, self._calls & 1,
                                       self.push_multimem, ops.status.ptr)

    def sum_add_rmsnorm(self, ops, residual, weight, out, M: int, eps: float, ctas: int) -> None:
        self._n.tp_sum_add_rmsnorm(self._ctx, residual, weight, out, M, float(eps), self._calls & 1, ctas,
                                   ops.status.ptr)
        self._calls += 1

    def begin_pass(self) -> None:
        """Every pass makes an even number of reductions (two per layer), so restarting the slot sequence at 0 keeps
        consecutive calls on alternating slots across passes and across CUDA-graph replays."""
        self._calls = 0
        self._sp_slot = 0

    # The decoder calls this instead of (all_reduce_partials + add_rmsnorm).
    def reduce_add_rmsnorm(self, ops, residual, partials, planes, weight, out, M, eps) -> None:
        if M >= self.nccl_min_rows and M < self.two_shot_min_rows:
            H = partials.shape[-1]
            if self._f16 is None or self._f16.shape[0] < M:
                self._f16 = torch.empty(max(M, self.m_cap), H, dtype=torch.float16, device=self.device)
            pl = partials.view(-1)[: planes * M * H].view(planes, M, H)
            tmp = self._f16[:M]
            tmp.copy_(pl[0] if planes == 1 else pl.sum(dim=0))
            dist.all_reduce(tmp, group=self.group)
            ops.add_rmsnorm(residual, partials, 0, tmp, weight, out, M, eps)
            return
        fn = self._n.tp_reduce_scatter_add_rmsnorm if (M >= self.two_shot_min_rows and out is not None) \
            else self._n.tp_reduce_add_rmsnorm
        fn(self._ctx, residual, partials, planes, weight, out, M, float(eps), self._calls & 1, self.use_multimem,
           ops.status.ptr)
        self._calls += 1

    def select_tokens(self, runner, n_rows: int, greedy: bool, step: int) -> None:
        if not greedy:
            return super().select_tokens(runner, n_rows, greedy, step)
        b, plan = runner.buf, runner.model.plan
        from .shard_plan import split_units
        bounds = split_units(runner.model.config.vocab_size, self.world)
        # shards are contiguous and (nearly) even: rank r starts at bounds[r][0]; the kernel wants a stride, so it is
        # only exact when the split is even - otherwise fall back to the gather path
        sizes = {hi - lo for lo, hi in bounds}
        if len(sizes) != 1:
            return super().select_tokens(runner, n_rows, greedy, step)
        self._n.tp_argmax(self._ctx, b.logits, b.logits.stride(0), b.out_tokens, n_rows, plan.vocab_size,
                          bounds[1][0] - bounds[0][0] if self.world > 1 else plan.vocab_size, 0,
                          runner.model.ops.status.ptr)

    def gather_logits(self, runner, n_rows: int) -> torch.Tensor:
        """Full-vocabulary logits rows on every rank without a library call: every rank stores its shard into every
        rank's symmetric buffer and waits for the others (csrc/comm.cu, tp_gather_rows_kernel).  Needs equally wide
        shards (a multiple of 8 columns); anything else takes the NCCL path of the base class."""
        b, plan = runner.buf, runner.model.plan
        vocab, W = runner.model.config.vocab_size, plan.vocab_size
        if W * self.world != vocab or W % 8 or b.logits.stride(0) % 8 or not env.flag("ZSE_TP_FUSED_GATHER"):
            return super().gather_logits(runner, n_rows)
        if getattr(self, "_gbuf", None) is None:
            if torch.cuda.is_current_stream_capturing():     # set-up is a collective: never inside a capture
                return super().gather_logits(runner, n_rows)
            self._init_gather(b.logits.shape[0], W)
        if n_rows > self._g_rows:
            return super().gather_logits(runner, n_rows)
        slot = self._g_calls & 1
        self._n.tp_gather_rows(self._ctx, b.logits, b.logits.stride(0), n_rows, slot, runner.model.ops.status.ptr)
        self._g_calls += 1
        return self._g_view[slot][:n_rows]

    def _init_gather(self, rows_cap: int, width: int) -> None:
        import torch.distributed._symmetric_memory as symm
        grp = self.group or dist.group.WORLD
        align = lambda n: (n + 255) // 256 * 256
        data = 2 * rows_cap * self.world * width * 2
        total = align(data) + align(2 * self.world * rows_cap * 4)
        self._gbuf = symm.empty(total, dtype=torch.uint8, device=self.device)
        self._gbuf.zero_()
        self._ghdl = symm.rendezvous(self._gbuf, grp)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=grp)
        ptrs = [int(p) for p in self._ghdl.buffer_ptrs]
        self._n.tp_ctx_set_gather(self._ctx, rows_cap, width, ptrs, [p + align(data) for p in ptrs])
        self._g_rows, self._g_calls = rows_cap, 0
        self._g_view = self._gbuf[:data].view(torch.float16).view(2, rows_cap, self.world * width)

    def close(self) -> None:
        if self._ctx:
            self._n.tp_ctx_destroy(self._ctx)
            self._ctx = None


def make_comm(backend: str, rank: int, world: int, device, hidden_size: int = 0, max_tokens: int = 0, group=None):
    if world <= 1:
        return None
    if backend in ("nccl", "nccl-sp"):       # "nccl-sp": sequence-parallel prefill on the NCCL path
        return NcclComm(rank, world, device, group, sequence_parallel=True if backend == "nccl-sp" else None)
    if backend == "fused":
        return FusedComm(rank, world, device, hidden_size, max_tokens, group)
    raise ValueError(f"unknown tensor-parallel comm backend '{backend}' (fused | nccl | nccl-sp)")
