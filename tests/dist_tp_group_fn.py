"""Rank function of tests/test_convert_tp_lora.py::test_tensor_parallel_group_facade (must be importable by the
spawned ranks)."""
import torch


def rank_fn(rank, tp_size, unique_id, backend):
    from zse_b200.parallel.tensor_parallel import COLUMN_PARALLEL, ROW_PARALLEL, TensorParallelGroup
    g = TensorParallelGroup(tp_size, rank, backend, unique_id)
    t = torch.full((4,), float(rank + 1))
    g.all_reduce_inplace(t)
    gathered = g.all_gather(torch.tensor([float(rank)]))
    b = g.broadcast(torch.tensor([float(rank * 10)]), root=1)
    g.barrier()
    out = {"sum": t.tolist(), "gathered": gathered.tolist(), "bcast": b.tolist(),
           "q": g.compute_shard_range(8 * 64, COLUMN_PARALLEL, unit=64),
           "down": g.compute_shard_range(13824, ROW_PARALLEL, unit=128),
           "strategy": [g.get_split_strategy("layers.3.self_attn.o_proj.weight"),
                        g.get_split_strategy("layers.0.mlp.up_proj.weight"), g.get_split_strategy("norm.weight")]}
    from zse_b200.parallel.tensor_parallel import NcclCommunicator
    c = NcclCommunicator(tp_size, rank, unique_id, backend)          # joins the process group that already exists
    recv = torch.zeros(3)
    c.all_reduce(torch.full((3,), float(rank + 1)), recv)
    rs = c.reduce_scatter(torch.arange(4.0) + rank)
    out["comm"] = {"rank": c.rank, "nranks": c.nranks, "sum": recv.tolist(), "rs": rs.tolist()}
    c.barrier()
    g.destroy()
    if rank == 1 and tp_size == 99:
        raise RuntimeError("unreachable")
    return out
