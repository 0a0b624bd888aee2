"""One gloo rank of tests/test_convert_tp_lora.py::test_collectives_facade: exercises NcclComm's general collectives
(the names say NCCL; on the CPU the same calls run over gloo) and exits 0 when every result is right."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from zse_b200.parallel.comm import NcclComm  # noqa: E402


def main():
    rank, world, port = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    c = NcclComm(rank, world, torch.device("cpu"))
    t = torch.full((4, 3), float(rank + 1))
    assert torch.equal(c.all_reduce(t.clone()), torch.full((4, 3), float(sum(range(1, world + 1)))))
    g = c.all_gather(torch.full((2, 3), float(rank)))
    assert g.shape == (2 * world, 3) and all(float(g[2 * r, 0]) == r for r in range(world))
    b = c.broadcast(torch.full((5,), float(rank)), src=world - 1)
    assert torch.equal(b, torch.full((5,), float(world - 1)))
    x = torch.arange(2 * world * 3, dtype=torch.float32).view(2 * world, 3) * (rank + 1)
    rs = c.reduce_scatter(x)
    want = torch.arange(2 * world * 3, dtype=torch.float32).view(2 * world, 3)[2 * rank: 2 * rank + 2] * sum(
        range(1, world + 1))
    assert torch.equal(rs, want), (rs, want)
    try:
        c.reduce_scatter(torch.zeros(2 * world + 1, 3))
        raise SystemExit("uneven reduce_scatter was accepted")
    except ValueError:
        pass
    c.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
