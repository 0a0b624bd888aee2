"""Child process of tests/test_comm_gpu.py: one rank per GPU (launched by torch.distributed.run)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
    from zse_b200.ops.backend import CudaOps
    from zse_b200.ops import reference as ref
    from zse_b200.parallel.comm import FusedComm
    ops = CudaOps(dev)
    H, M_cap = 2048, 1024
    for use_mm in (False, True):
        comm = FusedComm(rank, world, dev, H, M_cap, use_multimem=use_mm)
        comm.two_shot_min_rows, comm.nccl_min_rows = 128, 1 << 30          # exercise both kernels here
        if use_mm and not comm.use_multimem:
            if rank == 0:
                print("no multicast support here: multimem variant skipped")
            comm.close()
            continue
        torch.manual_seed(1234)
        w = (1 + 0.1 * torch.randn(H, device=dev)).half()
        for M, planes in ((1, 1), (64, 3), (200, 2), (700, 1)):
            torch.manual_seed(77 + M)                    # the residual stream is replicated: same on every rank
            res0 = torch.randn(M, H, device=dev)
            residual = res0.clone()
            torch.manual_seed(100 + rank)
            partials = torch.randn(planes, M, H, device=dev)
            out = torch.zeros(M, H, dtype=torch.float16, device=dev)
            comm.begin_pass()
            for call in range(4):
                comm.reduce_add_rmsnorm(ops, residual, partials, planes, w, out, M, 1e-6)
            torch.cuda.synchronize()
            ops.check()
            mine = partials.sum(0).half().float()
            dist.all_reduce(mine)
            want = res0 + 4 * mine
            two_shot = M >= comm.two_shot_min_rows
            if two_shot:
                # reduce-scatter form: only the rows this rank owns (row % world == rank) carry the residual
                own = torch.arange(M, device=dev) % world == rank
                assert torch.equal(residual[~own], res0[~own])
                err = (residual - want).abs() * own[:, None]
            else:
                err = (residual - want).abs()
            if use_mm:
                # the switch returns the cross-rank sum as fp16: up to a few fp16 ulps of the sum per call
                bound = 4 * world * 2.0 ** -10 * mine.abs() + 4e-3
                assert bool((err <= bound).all()), (use_mm, M, float(err.max()), float((err - bound).max()))
            else:
                assert bool((err <= 5e-3 + 1e-4 * want.abs()).all()), (use_mm, M, float(err.max()))
            assert (out.float() - ref.rmsnorm(want, w, 1e-6).float()).abs().max() < (6e-2 if use_mm else 2e-2)
            # every rank must hold the same residual (bitwise for the pull variant)
            gathered = [torch.empty_like(residual) for _ in range(world)]
            dist.all_gather(gathered, residual)
            if not use_mm and not two_shot:
                assert all(torch.equal(g, gathered[0]) for g in gathered)
            # the normalised rows are complete and identical on every rank in both forms
            outs = [torch.empty_like(out) for _ in range(world)]
            dist.all_gather(outs, out)
            assert all(torch.equal(o, outs[0]) for o in outs)
        comm.close()
    dist.barrier()
    if rank == 0:
        print("FUSED_COMM_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
