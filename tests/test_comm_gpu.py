"""Fused tensor-parallel reduction kernels.

On one GPU the protocol (per-row flags, two slots, pull over peer pointers, flag take-down) is exercised by the
emulated entry points: one cooperative launch plays every rank on buffers of the same device.  With two or more
GPUs the real kernels run in child processes over symmetric memory, against NCCL and against an fp32 restatement.
"""
import os
import subprocess
import sys

import pytest
import torch

from zse_b200.ops import reference as ref

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def ops():
    from zse_b200.ops.backend import CudaOps
    return CudaOps("cuda")


def _emulated_ctx(tp, m_cap, H):
    from zse_b200.ops import native
    dev = "cuda"
    data = [torch.zeros(2 * m_cap * H, dtype=torch.float16, device=dev) for _ in range(tp)]
    flags = [torch.zeros(2 * tp * m_cap, dtype=torch.int32, device=dev) for _ in range(tp)]
    xchg = [torch.zeros(2 * tp * m_cap, dtype=torch.int64, device=dev) for _ in range(tp)]
    xflags = [torch.zeros(2 * tp * m_cap, dtype=torch.int32, device=dev) for _ in range(tp)]
    ctx = native.tp_ctx_create(tp, 0, m_cap, H, [t.data_ptr() for t in data], [t.data_ptr() for t in flags], 0,
                               [t.data_ptr() for t in xchg], [t.data_ptr() for t in xflags])
    return ctx, (data, flags, xchg, xflags)


@pytest.mark.gpu
@pytest.mark.parametrize("tp,M,H,planes", [(2, 5, 512, 1), (4, 16, 1024, 3), (8, 7, 5120, 2)])
def test_reduce_add_rmsnorm_emulated_ranks(tp, M, H, planes):
    from zse_b200.ops import native
    ctx, keep = _emulated_ctx(tp, 32, H)
    status = native.Status("cuda")
    w = (1 + 0.1 * torch.randn(H, device="cuda")).half()
    res0 = torch.randn(M, H, device="cuda")
    residuals = [res0.clone() for _ in range(tp)]
    partials = [torch.randn(planes, M, H, device="cuda") for _ in range(tp)]
    outs = [torch.zeros(M, H, dtype=torch.float16, device="cuda") for _ in range(tp)]
    for call in range(4):            # several calls: slots alternate, flags are taken down and raised again
        native.tp_reduce_add_rmsnorm_emulated(ctx, residuals, partials, planes, w, outs, M, 1e-6, call & 1, status.ptr)
        torch.cuda.synchronize()
        status.check()
        total = sum(p.sum(0).half().float() for p in partials)     # each rank's row is rounded to fp16 on the wire
        want_res = res0 + (call + 1) * total
        for r in range(tp):
            assert torch.allclose(residuals[r], want_res, atol=2e-3, rtol=1e-4), (call, r)
            assert torch.equal(residuals[r], residuals[0])          # every rank holds bit-identical residuals
            got, want = outs[r].float(), ref.rmsnorm(want_res, w, 1e-6).float()
            assert (got - want).abs().max() < 1e-2
        assert all(int(f.abs().sum()) == 0 for f in keep[1])        # all flags are down again
    native.tp_ctx_destroy(ctx)


@pytest.mark.gpu
@pytest.mark.parametrize("tp,M,H,planes", [(2, 9, 512, 1), (4, 30, 1024, 3), (8, 17, 2048, 2)])
def test_reduce_scatter_add_rmsnorm_emulated_ranks(tp, M, H, planes):
    """Two-shot form: row r is reduced by rank r % tp only (its residual row is the only current one), the normalised
    rows are complete and identical on every rank."""
    from zse_b200.ops import native
    ctx, keep = _emulated_ctx(tp, 32, H)
    status = native.Status("cuda")
    w = (1 + 0.1 * torch.randn(H, device="cuda")).half()
    res0 = torch.randn(M, H, device="cuda")
    residuals = [res0.clone() for _ in range(tp)]
    partials = [torch.randn(planes, M, H, device="cuda") for _ in range(tp)]
    outs = [torch.zeros(M, H, dtype=torch.float16, device="cuda") for _ in range(tp)]
    rows = torch.arange(M, device="cuda")
    for call in range(4):
        native.tp_reduce_scatter_add_rmsnorm_emulated(ctx, residuals, partials, planes, w, outs, M, 1e-6, call & 1,
                                                      status.ptr)
        torch.cuda.synchronize()
        status.check()
        total = sum(p.sum(0).half().float() for p in partials)
        want_res = res0 + (call + 1) * total
        want_out = ref.rmsnorm(want_res, w, 1e-6).float()
        for r in range(tp):
            own = rows % tp == r
            assert torch.allclose(residuals[r][own], want_res[own], atol=2e-3, rtol=1e-4), (call, r)
            assert torch.equal(residuals[r][~own], res0[~own])      # rows of other owners are not touched
            assert torch.equal(outs[r], outs[0])
            assert (outs[r].float() - want_out).abs().max() < 1e-2
        assert all(int(f.abs().sum()) == 0 for f in keep[1])        # all flags are down again
    # mixing with the one-shot form afterwards works on the same context (flags are all down)
    residuals = [res0.clone() for _ in range(tp)]
    native.tp_reduce_add_rmsnorm_emulated(ctx, residuals, partials, planes, w, outs, M, 1e-6, 0, status.ptr)
    torch.cuda.synchronize()
    status.check()
    assert torch.allclose(residuals[tp - 1], res0 + sum(p.sum(0).half().float() for p in partials), atol=2e-3, rtol=1e-4)
    native.tp_ctx_destroy(ctx)


@pytest.mark.gpu
@pytest.mark.parametrize("tp,M,H,Kr", [(2, 5, 1024, 1024), (4, 64, 1024, 512), (8, 33, 5120, 640), (4, 64, 5120, 3456)])
def test_gemm_push_exchange_emulated_ranks(ops, tp, M, H, Kr):
    """The exchange inside the GEMM: every emulated rank runs its row-parallel INT4 GEMM, whose epilogue writes the fp16
    partial rows into every rank's inbox and counts its CTAs in; the consumer then only adds local rows.  Producers
    never wait, so running them one after the other on one GPU is a faithful test of the data path and counters."""
    from zse_b200.ops import native
    from test_kernels_gpu import _w4_parts_gpu
    m_cap = 64
    ctx, keep = _emulated_ctx(tp, m_cap, H)
    inbox = [torch.zeros(2 * tp * m_cap * H, dtype=torch.float16, device="cuda") for _ in range(tp)]
    arrive = [torch.zeros(2 * tp, dtype=torch.int32, device="cuda") for _ in range(tp)]
    state = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(tp)]
    native.tp_ctx_set_push(ctx, m_cap, [t.data_ptr() for t in inbox], 0, [t.data_ptr() for t in arrive], 0,
                           [t.data_ptr() for t in state])
    status = native.Status("cuda")
    wn = (1 + 0.1 * torch.randn(H, device="cuda")).half()
    res0 = torch.randn(M, H, device="cuda")
    residuals = [res0.clone() for _ in range(tp)]
    outs = [torch.zeros(M, H, dtype=torch.float16, device="cuda") for _ in range(tp)]
    shards, xs, partial = [], [], []
    for r in range(tp):
        part, wd = _w4_parts_gpu(H, Kr, 40 + r)
        shards.append(ops.make_linear([part], Kr, 128))
        xs.append((torch.randn(M, Kr, device="cuda") * 0.5).half())
        partial.append((xs[r].float() @ wd.T).half().float())     # what arrives: fp16 rows
    want = res0.clone()
    for call in range(3):
        slot = call & 1
        ctas = [native.tp_gemm_w4_push(ctx, shards[r].data, xs[r], M, M, H, Kr, slot, False, status.ptr,
                                       rank_override=r) for r in range(tp)]
        assert len(set(ctas)) == 1 and ctas[0] > 0
        native.tp_sum_add_rmsnorm_emulated(ctx, residuals, wn, outs, M, 1e-6, slot, ctas[0], status.ptr)
        torch.cuda.synchronize()
        status.check()
        want = want + sum(partial)
        for r in range(tp):
            assert _rel_close(residuals[r], want), (call, r)
            assert torch.equal(residuals[r], residuals[0])
            assert (outs[r].float() - ref.rmsnorm(want, wn, 1e-6).float()).abs().max() < 3e-2
    # a consumer whose producers did not run gives up with a status instead of hanging
    native.tp_sum_add_rmsnorm_emulated(ctx, residuals, wn, outs, M, 1e-6, 1, ctas[0], status.ptr)
    torch.cuda.synchronize()
    code, _, where, _ = status.read()
    assert (code, where) == (3, 34)
    native.tp_ctx_destroy(ctx)


@pytest.mark.gpu
@pytest.mark.parametrize("tp,M,H", [(2, 130, 1024), (4, 300, 1024), (8, 1000, 2560)])
def test_scatter_reduce_gather_emulated_ranks(ops, tp, M, H):
    """The prefill exchange on one GPU: every emulated rank runs its row-parallel INT4 GEMM, whose epilogue stores each
    64-row block of fp16 partial sums into the inbox of the block's owner and counts (tile, chunk) units in - shards of
    different width, hence different K splits, must add up to the same total.  The reduce kernel (all ranks in one
    launch, nothing waits for a kernel that is not running) adds the rows, applies residual + RMSNorm on the owner and
    stores the rows into every rank's gathered buffer; a GEMM reading that buffer passes its prologue wait."""
    from zse_b200.ops import native
    from test_kernels_gpu import _w4_parts_gpu
    m_cap = 1024
    nblk = m_cap // 64
    own_cap = (nblk + tp - 1) // tp * 64
    ctx, keep = _emulated_ctx(tp, 64, H)
    z = lambda n, dt: [torch.zeros(n, dtype=dt, device="cuda") for _ in range(tp)]
    inbox, arrive = z(2 * tp * own_cap * H, torch.float16), z(2 * tp * nblk, torch.int32)
    xg, gflag, state = z(nblk * 64 * H, torch.float16), z(nblk, torch.int32), z(4 + nblk, torch.int32)
    ptr = lambda ts: [t.data_ptr() for t in ts]
    native.tp_ctx_set_sp(ctx, own_cap, nblk, ptr(inbox), ptr(arrive), ptr(xg), 0, ptr(gflag), ptr(state))
    status = native.Status("cuda")
    wn = (1 + 0.1 * torch.randn(H, device="cuda")).half()
    res0 = torch.randn(M, H, device="cuda")
    residuals = [res0.clone() for _ in range(tp)]
    shards, xs, partial = [], [], []
    for r in range(tp):
        Kr = 512 + 384 * (r % 3)                      # uneven shards: the ranks plan different K splits
        part, wd = _w4_parts_gpu(H, Kr, 70 + r)
        shards.append(ops.make_linear([part], Kr, 128))
        xs.append((torch.randn(M, Kr, device="cuda") * 0.5).half())
        partial.append((xs[r].float() @ wd.T).half().float())
    nb = (M + 63) // 64
    owner_of_row = (torch.arange(M, device="cuda") // 64) % tp
    want = res0.clone()
    part2, wd2 = _w4_parts_gpu(256, H, 5)
    w2 = ops.make_linear([part2], H, 128)
    for call in range(3):
        slot = call & 1
        for r in range(tp):
            native.tp_gemm_w4_scatter(ctx, shards[r].data, xs[r], M, M, H, shards[r].K, slot, status.ptr,
                                      rank_override=r)
        native.tp_sp_sum_norm_gather_emulated(ctx, residuals, wn, M, 1e-6, slot, status.ptr)
        torch.cuda.synchronize()
        status.check()
        want = want + sum(partial)
        normed = ref.rmsnorm(want, wn, 1e-6).float()
        for r in range(tp):
            mine = owner_of_row == r
            assert _rel_close(residuals[r][mine], want[mine]), (call, r)
            got = xg[r].view(nblk * 64, H)[:M].float()
            assert (got - normed).abs().max() < 3e-2, (call, r)
            assert torch.equal(xg[r], xg[0])                       # every rank holds the same gathered rows
            assert torch.all(gflag[r][:nb] == call + 1) and int(state[r][0]) == call + 1
            assert int(arrive[r].abs().sum()) == 0                 # counters taken down for the call after next
        # rows a rank does not own keep their old residual (the stream is sharded by rows during such a pass)
        other = owner_of_row != 0
        assert torch.equal(residuals[0][other], res0[other])
        # the consumer GEMM on the gathered buffer (prologue wait satisfied) equals the plain GEMM on the same rows
        a = torch.zeros(M, 256, dtype=torch.float16, device="cuda")
        bb = torch.zeros_like(a)
        xv = xg[1 % tp].view(nblk * 64, H)
        native.tp_gemm_w4_gathered(ctx, w2.data, xv, xv.shape[0], None, a, M, 256, H, 256, 0, 0, status.ptr,
                                   rank_override=1 % tp)
        native.gemm_w4(w2.data, xv, xv.shape[0], None, bb, M, 256, H, 256, 0, 0, status.ptr)
        torch.cuda.synchronize()
        status.check()
        assert torch.equal(a, bb)
    # rows that never arrive: the GEMM's prologue gives up with a status instead of hanging, and loads nothing
    state[0][0] += 1                                               # rank 0 expects an epoch nobody has published
    native.tp_gemm_w4_gathered(ctx, w2.data, xg[0].view(nblk * 64, H), nblk * 64, None, a, M, 256, H, 256, 0, 0,
                               status.ptr, rank_override=0)
    torch.cuda.synchronize()
    code, _, where, _ = status.read()
    assert (code, where) == (3, 36)
    native.tp_ctx_destroy(ctx)


def _k1_ctx(tp, m_cap, H):
    from zse_b200.ops import native
    ctx, keep = _emulated_ctx(tp, m_cap, H)
    inbox = [torch.zeros(2 * tp * m_cap * H, dtype=torch.float16, device="cuda") for _ in range(tp)]
    arrive = [torch.zeros(2 * tp, dtype=torch.int32, device="cuda") for _ in range(tp)]
    state = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(tp)]
    native.tp_ctx_set_push(ctx, m_cap, [t.data_ptr() for t in inbox], 0, [t.data_ptr() for t in arrive], 0,
                           [t.data_ptr() for t in state])
    return ctx, (keep, inbox, arrive, state)


@pytest.mark.gpu
@pytest.mark.parametrize("M,H,K,int8", [(1, 1024, 512, False), (7, 1024, 1792, False), (64, 5120, 640, False),
                                        (33, 2560, 1024, True), (64, 5120, 1792, False), (4, 1024, 128, False),
                                        (8, 1024, 256, False)])
def test_projection_residual_norm_in_one_kernel_single_rank(ops, M, H, K, int8):
    """kDecAllReduceNorm with one rank: projection, residual add and RMSNorm are one launch (no peers to wait for)."""
    from zse_b200.ops import native
    from test_kernels_gpu import _w4_parts_gpu
    from test_gemm_dec_gpu import _parts8
    ctx, keep = _k1_ctx(1, 64, H)
    status = native.Status("cuda")
    ws = native.gemm_w4_dec_workspace("cuda", ops.sm_count)
    part, wd = _parts8(H, K, 3) if int8 else _w4_parts_gpu(H, K, 3)
    w = ops.make_linear([part], K, 128)
    assert w.kind == ("w8t" if int8 else "w4t")
    x = (torch.randn(M, K, device="cuda") * 0.5).half()
    wn = (1 + 0.1 * torch.randn(H, device="cuda")).half()
    res0 = torch.randn(M + 2, H, device="cuda")
    residual = res0.clone()
    out = torch.full((M + 2, H), 3.0, dtype=torch.float16, device="cuda")
    want = res0[:M].clone()
    for call in range(3):
        native.tp_gemm_dec_allreduce_norm(ctx, w.data, int8, x, M, M, H, K, call & 1, False, residual, wn, out, 1e-6,
                                          ws, status.ptr)
        torch.cuda.synchronize()
        status.check()
        want = want + (x.float() @ wd.T).half().float()
        assert _rel_close(residual[:M], want), call
        assert (out[:M].float() - ref.rmsnorm(want, wn, 1e-6).float()).abs().max() < 3e-2
    assert torch.equal(residual[M:], res0[M:]) and torch.all(out[M:] == 3.0)      # rows past M untouched
    native.tp_ctx_destroy(ctx)


@pytest.mark.gpu
@pytest.mark.parametrize("tp,M,H,K", [(2, 5, 1024, 512), (4, 64, 1024, 1024), (8, 40, 5120, 640), (8, 4, 1024, 128)])
def test_one_kernel_all_reduce_with_peers_that_have_delivered(ops, tp, M, H, K):
    """The multi-rank data path on one GPU without any kernel waiting for another: this rank's launch finds the other
    ranks' rows already in its inbox and their counters already at the target (written here by the host), sends its
    own rows to every inbox, and must add all tp sources in rank order."""
    from zse_b200.ops import native
    from test_kernels_gpu import _w4_parts_gpu
    m_cap = 64
    ctx, (keep, inbox, arrive, state) = _k1_ctx(tp, m_cap, H)
    status = native.Status("cuda")
    ws = native.gemm_w4_dec_workspace("cuda", ops.sm_count)
    me = 1 % tp
    part, wd = _w4_parts_gpu(H, K, 11)
    w = ops.make_linear([part], K, 128)
    x = (torch.randn(M, K, device="cuda") * 0.5).half()
    wn = (1 + 0.1 * torch.randn(H, device="cuda")).half()
    res0 = torch.randn(M, H, device="cuda")
    residual = res0.clone()
    out = torch.zeros(M, H, dtype=torch.float16, device="cuda")
    nt = 16 if M <= 16 else 32 if M <= 32 else 64
    units = (H // 128) * (nt // 8)
    want = res0.clone()
    for call in range(4):
        slot = call & 1
        peers = {r: (torch.randn(M, H, device="cuda") * 0.3).half() for r in range(tp) if r != me}
        box = inbox[me].view(2, tp, m_cap, H)
        for r, rows in peers.items():
            box[slot, r, :M] = rows
            arrive[me].view(2, tp)[slot, r] += units                       # "rank r has delivered"
        native.tp_gemm_dec_allreduce_norm(ctx, w.data, False, x, M, M, H, K, slot, False, residual, wn, out, 1e-6, ws,
                                          status.ptr, rank_override=me)
        torch.cuda.synchronize()
        status.check()
        mine = (x.float() @ wd.T).half().float()
        want = want + mine + sum(p.float() for p in peers.values())
        assert _rel_close(residual, want), call
        assert (out.float() - ref.rmsnorm(want, wn, 1e-6).float()).abs().max() < 3e-2
        # this rank's rows went to every rank's inbox and its units were counted in everywhere
        for r in range(tp):
            got = inbox[r].view(2, tp, m_cap, H)[slot, me, :M].float()
            assert _rel_close(got, mine, tol=2e-3)
            # the rank's own counter is fed by each of its twenty worker warps, the peers' once per CTA
            assert int(arrive[r].view(2, tp)[slot, me]) == units * (call // 2 + 1) * (20 if r == me else 1)
    native.tp_ctx_destroy(ctx)


def _rel_close(a, b, tol=4e-3):
    return float((a - b).abs().max()) <= tol * max(1.0, float(b.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("tp,M,W", [(2, 5, 512), (4, 64, 1000), (8, 33, 19008)])
def test_logits_all_gather_emulated_ranks(tp, M, W):
    """Every emulated rank stores its vocabulary shard of the logits rows into every rank's buffer and waits for the
    others (one cooperative launch plays all ranks): all ranks end with the concatenation, call after call."""
    from zse_b200.ops import native
    ctx, keep = _emulated_ctx(tp, 64, 1024)
    rows_cap = 64
    bufs = [torch.zeros(2 * rows_cap * tp * W, dtype=torch.float16, device="cuda") for _ in range(tp)]
    flags = [torch.zeros(2 * tp * rows_cap, dtype=torch.int32, device="cuda") for _ in range(tp)]
    native.tp_ctx_set_gather(ctx, rows_cap, W, [t.data_ptr() for t in bufs], [t.data_ptr() for t in flags])
    status = native.Status("cuda")
    for call in range(3):
        slot = call & 1
        ld = W + 8 * (call + 1)                                  # rows of the local logits may be padded
        shards = [torch.randn(M, ld, device="cuda").half() for _ in range(tp)]
        native.tp_gather_rows_emulated(ctx, shards, ld, M, slot, status.ptr)
        torch.cuda.synchronize()
        status.check()
        want = torch.cat([t[:, :W] for t in shards], dim=1)
        for r in range(tp):
            got = bufs[r].view(2, rows_cap, tp * W)[slot, :M]
            assert torch.equal(got, want), (call, r)
        assert all(int(f.abs().sum()) == 0 for f in flags)       # every flag was taken down again
    native.tp_ctx_destroy(ctx)


@pytest.mark.gpu
def test_tp_argmax_emulated_ranks():
    from zse_b200.ops import native
    tp, M, V_local = 4, 6, 1000
    ctx, keep = _emulated_ctx(tp, 32, 512)
    status = native.Status("cuda")
    full = (torch.randn(M, tp * V_local, device="cuda") * 3).half()
    full[1, 10] = full[1, 3010] = 60.0            # a tie across ranks: the lower token id wins
    shards = [full[:, r * V_local:(r + 1) * V_local].contiguous() for r in range(tp)]
    outs = [torch.zeros(M, dtype=torch.int32, device="cuda") for _ in range(tp)]
    for _ in range(2):
        native.tp_argmax_emulated(ctx, shards, V_local, outs, M, V_local, V_local, 0, status.ptr)
        torch.cuda.synchronize()
        status.check()
        want = full.float().argmax(-1).int()
        assert int(want[1]) == 10
        for r in range(tp):
            assert torch.equal(outs[r], want)
    native.tp_ctx_destroy(ctx)


@pytest.mark.gpu
def test_peer_wait_times_out_with_status_instead_of_hanging():
    """A flag that nothing raises: the bounded wait gives up, the kernel returns, the context stays usable and the
    host sees a 'peer wait timed out' status.  (One real rank whose peer table points at a rank that never runs.)"""
    from zse_b200.ops import native
    tp, H, M = 2, 512, 1
    ctx, keep = _emulated_ctx(tp, 8, H)
    status = native.Status("cuda")
    res = torch.zeros(M, H, device="cuda")
    part = torch.ones(1, M, H, device="cuda")
    out = torch.zeros(M, H, dtype=torch.float16, device="cuda")
    w = torch.ones(H, dtype=torch.float16, device="cuda")
    # the real (non-emulated) entry point runs rank 0 only; rank 1 never raises its flag
    native.tp_reduce_add_rmsnorm(ctx, res, part, 1, w, out, M, 1e-6, 0, False, status.ptr)
    torch.cuda.synchronize()
    code, _, where, detail = status.read()
    assert (code, where, detail) == (3, 31, 1)
    with pytest.raises(native.DeviceStatusError):
        status.check()
    assert float(res.abs().sum()) == 0.0          # the row was left alone
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0     # device still answers
    native.tp_ctx_destroy(ctx)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_fused_comm_matches_nccl_on_real_gpus():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "1"))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", "29633",
                        os.path.join(ROOT, "tests", "dist_fused_comm_worker.py")], capture_output=True, text=True,
                       timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-12000:]
    assert "FUSED_COMM_OK" in r.stdout


@pytest.mark.gpu
@pytest.mark.multigpu
def test_tp_engine_on_real_gpus_matches_single_gpu():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", "29641",
                        os.path.join(ROOT, "tests", "dist_tp_engine_worker.py")], capture_output=True, text=True,
                       timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-12000:]
    assert "TP_ENGINE_OK" in r.stdout
