"""Stateless process group over a TCPStore (threads stand in for ranks) and the NCCL symbol table."""
import socket
import threading

from sonar_b200.distributed.stateless import StatelessProcessGroup


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_stateless_group_collectives():
    port, world = _free_port(), 3
    results: dict[int, dict] = {}

    def run(rank):
        g = StatelessProcessGroup.create("127.0.0.1", port, rank, world, timeout_s=30)
        res = {}
        res["bcast"] = g.broadcast_obj({"x": 42} if rank == 1 else None, 1)
        res["gather"] = g.all_gather_obj(rank * 10)
        if rank == 0:
            g.send_obj("hello", 2)
        if rank == 2:
            res["p2p"] = g.recv_obj(0)
        g.barrier(timeout_s=30)
        res["gather2"] = g.all_gather_obj(f"r{rank}")
        results[rank] = res

    ts = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    [t.start() for t in ts]
    [t.join(60) for t in ts]
    assert len(results) == world
    for r in range(world):
        assert results[r]["bcast"] == {"x": 42}
        assert results[r]["gather"] == [0, 10, 20]
        assert results[r]["gather2"] == ["r0", "r1", "r2"]
    assert results[2]["p2p"] == "hello"


def test_nccl_library_binds():
    from sonar_b200.distributed.pynccl import NCCLLibrary
    lib = NCCLLibrary()
    assert lib.version().split(".")[0] == "2"
