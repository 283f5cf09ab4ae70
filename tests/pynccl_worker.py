"""Child process of the PyNccl test: one rank, one GPU; results are checked in place."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from sonar_b200.distributed.pynccl import PyNcclCommunicator  # noqa: E402
from sonar_b200.distributed.stateless import StatelessProcessGroup  # noqa: E402


def main() -> None:
    rank, world, port = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    torch.cuda.set_device(rank)
    g = StatelessProcessGroup.create("127.0.0.1", port, rank, world, timeout_s=60)
    comm = PyNcclCommunicator(g, rank)
    dev = torch.device("cuda", rank)
    x = torch.full((1024,), float(rank + 1), device=dev)
    comm.all_reduce(x)
    assert torch.allclose(x, torch.full_like(x, world * (world + 1) / 2))
    mine = torch.full((4, 8), float(rank), device=dev, dtype=torch.bfloat16)
    out = torch.empty((4 * world, 8), device=dev, dtype=torch.bfloat16)
    comm.all_gather(out, mine)
    for r in range(world):
        assert (out[4 * r:4 * r + 4] == r).all()
    rs = torch.empty((4, 8), device=dev, dtype=torch.bfloat16)
    comm.reduce_scatter(rs, out.clone())
    assert (rs == rank * world).all()
    sizes = [r + 1 for r in range(world)]
    part = torch.full((sizes[rank], 8), float(rank + 1), device=dev)
    gv = torch.empty((sum(sizes), 8), device=dev)
    comm.all_gatherv(gv, part, sizes)
    off = 0
    for r, n in enumerate(sizes):
        assert (gv[off:off + n] == r + 1).all()
        off += n
    if rank == 0:
        comm.send(torch.arange(16, device=dev, dtype=torch.float32), 1)
    elif rank == 1:
        buf = torch.empty(16, device=dev)
        comm.recv(buf, 0)
        assert torch.equal(buf, torch.arange(16, device=dev, dtype=torch.float32))
    torch.cuda.synchronize()
    g.barrier(timeout_s=60)
    comm.destroy()
    print("ok", rank, flush=True)


if __name__ == "__main__":
    main()
