"""Expert load balancing: policy invariants, balance improvement, weight shuffle (1 rank and 2 gloo ranks)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sonar_b200.distributed.eplb import EplbConfig, EplbState, rebalance_experts, shuffle_expert_weights


def _check_mapping(phy2log, log2phy, logcnt, e, p):
    layers = phy2log.shape[0]
    assert phy2log.shape == (layers, p) and logcnt.shape == (layers, e)
    assert (logcnt >= 1).all() and (logcnt.sum(-1) == p).all()
    for li in range(layers):
        for x in range(e):
            slots = [s for s in log2phy[li, x].tolist() if s >= 0]
            assert len(slots) == int(logcnt[li, x]) and all(int(phy2log[li, s]) == x for s in slots)


@pytest.mark.parametrize("nodes,groups", [(1, 1), (2, 8)])
def test_policy_invariants_and_balance(nodes, groups):
    torch.manual_seed(0)
    e, p, gpus = 64, 80, 8
    load = (torch.distributions.Zipf(1.2).sample((3, e)) if hasattr(torch.distributions, "Zipf")
            else torch.rand(3, e).pow(-1.2)).float()
    phy2log, log2phy, logcnt = rebalance_experts(load, p, groups, nodes, gpus)
    _check_mapping(phy2log, log2phy, logcnt, e, p)
    # per-GPU load under the new mapping vs the trivial one (experts in order, spares replicate the first)
    def gpu_max(mapping, cnt):
        share = (load / cnt).gather(1, mapping)
        return share.view(3, gpus, -1).sum(-1).max(-1).values
    trivial = (torch.arange(p) % e).repeat(3, 1)
    tcnt = torch.zeros(3, e, dtype=torch.int64).scatter_add_(1, trivial, torch.ones_like(trivial))
    assert (gpu_max(phy2log, logcnt) <= gpu_max(trivial, tcnt) + 1e-3).all()
    # the hottest expert is replicated
    assert (logcnt.gather(1, load.argmax(-1, keepdim=True)) > 1).all()
    if nodes > 1:   # groups stay on one node
        gsz, per_node = e // groups, p // nodes
        for li in range(3):
            for n in range(nodes):
                on_node = set((phy2log[li, n * per_node:(n + 1) * per_node] // gsz).tolist())
                assert len(on_node) == groups // nodes


def test_state_window_and_single_rank_shuffle():
    st = EplbState(num_layers=2, num_logical=8, cfg=EplbConfig(num_redundant_experts=4, window_size=4, step_interval=3),
                   world_size=2)
    w13 = [torch.stack([torch.full((3, 2), float(int(x))) for x in st.phy2log[li]]) for li in range(2)]
    rearranged = False
    for step in range(3):
        for li in range(2):
            ids = torch.tensor([0, 0, 0, 0, 1, 5, 5, 7])           # expert 0 is hot
            st.record(li, st.log2phy[li, ids, 0])
        rearranged = st.step()
    assert rearranged
    before = st.balancedness()
    st.rearrange([[w] for w in w13])
    assert int(st.logcnt[0, 0]) > 1
    for li in range(2):                                              # every slot now holds the weights of its expert
        assert torch.equal(w13[li][:, 0, 0], st.phy2log[li].float())
    load_phys = (st.logical_load().float() / st.logcnt).gather(1, st.phy2log)
    assert st.balancedness(load_phys) >= before - 1e-6


def _worker(rank, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=2)
    old = torch.tensor([[0, 1, 2, 3, 0, 1]])           # 6 slots, 3 per rank
    new = torch.tensor([[3, 2, 3, 0, 1, 0]])
    local_old = old[0, rank * 3:(rank + 1) * 3]
    w = torch.stack([torch.full((4,), float(int(x))) for x in local_old])
    got = shuffle_expert_weights(old, new, [[w]])
    out.put((rank, w[:, 0].tolist(), got))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_weight_shuffle():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_worker, args=(r, port, q)) for r in range(2)]
    [p.start() for p in ps]
    res = dict((r, (vals, got)) for r, vals, got in (q.get(timeout=120) for _ in range(2)))
    [p.join(60) for p in ps]
    assert res[0][0] == [3.0, 2.0, 3.0] and res[1][0] == [0.0, 1.0, 0.0]
    assert res[0][1] == 2 and res[1][1] == 0      # rank 0 received expert 3 twice; rank 1 had everything locally
