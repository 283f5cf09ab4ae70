"""Expert-parallel load balancing: replicate hot experts, pack replicas evenly over GPUs, move weights.

Vocabulary: a model layer has ``E`` *logical* experts (what the router picks) and ``P ≥ E``
*physical* slots spread evenly over the expert-parallel ranks (``P / world`` per rank).  A mapping
``phy2log [layers, P]`` says which logical expert each slot holds; hot experts occupy several slots
and their tokens are spread over the replicas.

* ``rebalance_experts`` — the policy: from a load matrix ``[layers, E]`` to ``(phy2log, log2phy,
  logcnt)``.  Hierarchical when expert groups divide evenly over nodes (groups are first packed onto
  nodes so group-limited routing stays node-local, then replicated and packed onto GPUs inside each
  node), global otherwise.
* ``EplbState`` — sliding window of per-slot token counts, periodic rearrangement.
* ``shuffle_expert_weights`` — executes a mapping change: local copies where the rank already holds
  the expert, point-to-point transfers (``torch.distributed`` batch isend/irecv) otherwise.

Parity: ``aphrodite/distributed/eplb/policy/default.py`` (replicate + balanced packing),
``eplb_state.py`` (window, step interval), ``rebalance_execute.py`` (weight shuffle).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


# --------------------------------------------------------------------------- policy
def _pack_even(loads: list[float], bins: int) -> list[list[int]]:
    """Split ``len(loads)`` items into ``bins`` bins of equal item count, sums as even as one greedy
    pass makes them: heaviest item first, always into the lightest bin that still has room."""
    n = len(loads)
    assert n % bins == 0, (n, bins)
    room = n // bins
    out: list[list[int]] = [[] for _ in range(bins)]
    sums = [0.0] * bins
    for item in sorted(range(n), key=lambda i: (-loads[i], i)):
        b = min((k for k in range(bins) if len(out[k]) < room), key=lambda k: (sums[k], k))
        out[b].append(item)
        sums[b] += loads[item]
    return out


def _replicate(loads: list[float], slots: int) -> list[int]:
    """Replica count per expert: every expert gets one slot, each spare slot goes to the expert whose
    load per replica is currently highest."""
    counts = [1] * len(loads)
    for _ in range(slots - len(loads)):
        hot = max(range(len(loads)), key=lambda i: (loads[i] / counts[i], -i))
        counts[hot] += 1
    return counts


def _place_layer(loads: list[float], slots: int, gpus: int, nodes: int, groups: int) -> list[int]:
    """One layer: the logical expert held by each of ``slots`` physical slots, GPU-major order."""
    e = len(loads)
    per_node_slots = slots // nodes
    gpus_per_node = gpus // nodes
    if nodes > 1:
        gsz = e // groups
        gload = [sum(loads[g * gsz:(g + 1) * gsz]) for g in range(groups)]
        node_groups = _pack_even(gload, nodes)                     # expert groups stay together on a node
        node_experts = [[x for g in sorted(gs) for x in range(g * gsz, (g + 1) * gsz)] for gs in node_groups]
    else:
        node_experts = [list(range(e))]
    placement: list[int] = []
    for experts in node_experts:
        counts = _replicate([loads[x] for x in experts], per_node_slots)
        replicas = [x for x, c in zip(experts, counts) for _ in range(c)]
        share = [loads[x] / c for x, c in zip(experts, counts) for _ in range(c)]
        for gpu_items in _pack_even(share, gpus_per_node):
            placement.extend(replicas[i] for i in sorted(gpu_items, key=lambda i: (replicas[i], i)))
    return placement


def rebalance_experts(weight: torch.Tensor, num_replicas: int, num_groups: int = 1, num_nodes: int = 1,
                      num_gpus: int = 1) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``weight [L, E]`` token counts → ``(phy2log [L, P], log2phy [L, E, max_replicas] (−1 padded),
    logcnt [L, E])`` with ``P = num_replicas`` physical slots, ``P / num_gpus`` per GPU."""
    layers, e = weight.shape
    assert num_replicas >= e and num_replicas % num_gpus == 0 and num_gpus % num_nodes == 0
    hierarchical = num_nodes > 1 and num_groups % num_nodes == 0 and e % num_groups == 0 \
        and num_replicas % num_nodes == 0
    nodes, groups = (num_nodes, num_groups) if hierarchical else (1, 1)
    w = weight.double().cpu().tolist()
    phy2log = torch.tensor([_place_layer(w[li], num_replicas, num_gpus, nodes, groups) for li in range(layers)],
                           dtype=torch.int64)
    logcnt = torch.zeros((layers, e), dtype=torch.int64)
    logcnt.scatter_add_(1, phy2log, torch.ones_like(phy2log))
    max_rep = int(logcnt.max())
    log2phy = torch.full((layers, e, max_rep), -1, dtype=torch.int64)
    for li in range(layers):
        seen = [0] * e
        for slot, x in enumerate(phy2log[li].tolist()):
            log2phy[li, x, seen[x]] = slot
            seen[x] += 1
    return phy2log, log2phy, logcnt


# --------------------------------------------------------------------------- weight movement
def shuffle_expert_weights(old_phy2log: torch.Tensor, new_phy2log: torch.Tensor,
                           layer_weights: list[list[torch.Tensor]], group=None) -> int:
    """Make every rank's local slots hold the experts ``new_phy2log`` assigns them.

    ``old/new_phy2log [L, P]``; ``layer_weights[l]`` = this rank's stacked expert tensors of layer ``l``
    (each ``[P_local, …]``).  Returns the number of expert tensors received from other ranks."""
    world = dist.get_world_size(group) if (group is not None or dist.is_initialized()) else 1
    rank = dist.get_rank(group) if world > 1 else 0
    layers, p = old_phy2log.shape
    local = p // world
    received = 0
    for li in range(layers):
        old, new = old_phy2log[li].tolist(), new_phy2log[li].tolist()
        if old == new:
            continue
        weights = layer_weights[li]
        snapshot = [w.clone() for w in weights]
        holders: dict[int, list[int]] = {}
        for slot, e in enumerate(old):
            holders.setdefault(e, []).append(slot)
        ops_: list = []
        recv_bufs: list[tuple[int, int, torch.Tensor]] = []
        for slot in range(p):
            e = new[slot]
            dst_rank = slot // local
            src_slots = holders[e]
            on_dst = [s for s in src_slots if s // local == dst_rank]
            if on_dst:
                if dst_rank == rank:
                    for wi, w in enumerate(weights):
                        w[slot % local].copy_(snapshot[wi][on_dst[0] % local])
                continue
            # deterministic sender: spread over the holders by destination slot
            src = src_slots[slot % len(src_slots)]
            src_rank = src // local
            if src_rank == rank:
                for wi in range(len(weights)):
                    ops_.append(dist.P2POp(dist.isend, snapshot[wi][src % local].contiguous(),
                                           dist.get_global_rank(group, dst_rank) if group is not None else dst_rank,
                                           group))
            if dst_rank == rank:
                for wi, w in enumerate(weights):
                    buf = torch.empty_like(w[slot % local])
                    recv_bufs.append((wi, slot % local, buf))
                    ops_.append(dist.P2POp(dist.irecv, buf,
                                           dist.get_global_rank(group, src_rank) if group is not None else src_rank,
                                           group))
                received += 1
        if ops_:
            for req in dist.batch_isend_irecv(ops_):
                req.wait()
        for wi, ls, buf in recv_bufs:
            weights[wi][ls].copy_(buf)
    return received


# --------------------------------------------------------------------------- state
@dataclass
class EplbConfig:
    num_redundant_experts: int = 0
    window_size: int = 1000          # steps of load history
    step_interval: int = 3000        # rearrange every this many steps
    num_groups: int = 1
    num_nodes: int = 1


class EplbState:
    """Load statistics and the current mapping of every MoE layer of one model."""

    def __init__(self, num_layers: int, num_logical: int, cfg: EplbConfig, world_size: int, device="cpu") -> None:
        self.cfg = cfg
        self.world = world_size
        self.num_logical = num_logical
        self.num_phys = num_logical + cfg.num_redundant_experts
        if self.num_phys % world_size:
            raise ValueError(f"{self.num_phys} physical experts do not divide over {world_size} ranks")
        self.window = torch.zeros((cfg.window_size, num_layers, self.num_phys), dtype=torch.int64, device=device)
        self.pass_load = torch.zeros((num_layers, self.num_phys), dtype=torch.int64, device=device)
        self.cursor = 0
        self.steps = 0
        # initial mapping: logical experts in order, spare slots replicate the first experts
        init = torch.arange(self.num_phys) % num_logical
        self.phy2log = init.repeat(num_layers, 1)
        self.log2phy, self.logcnt = self._derive(self.phy2log)
        self.rearrangements = 0

    def _derive(self, phy2log: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        layers, p = phy2log.shape
        logcnt = torch.zeros((layers, self.num_logical), dtype=torch.int64)
        logcnt.scatter_add_(1, phy2log, torch.ones_like(phy2log))
        log2phy = torch.full((layers, self.num_logical, int(logcnt.max())), -1, dtype=torch.int64)
        for li in range(layers):
            seen = [0] * self.num_logical
            for slot, x in enumerate(phy2log[li].tolist()):
                log2phy[li, x, seen[x]] = slot
                seen[x] += 1
        return log2phy, logcnt

    def record(self, layer: int, phys_ids: torch.Tensor) -> None:
        """Count the tokens routed to each physical slot of ``layer`` in this forward pass."""
        flat = phys_ids.reshape(-1).to(self.pass_load.device, torch.int64)
        self.pass_load[layer].scatter_add_(0, flat, torch.ones_like(flat))

    def step(self, group=None) -> bool:
        """End of an engine step.  Returns True when it is time to rearrange."""
        self.window[self.cursor] = self.pass_load
        self.pass_load.zero_()
        self.cursor = (self.cursor + 1) % self.cfg.window_size
        self.steps += 1
        return self.steps % self.cfg.step_interval == 0

    def logical_load(self, group=None) -> torch.Tensor:
        """Window-summed load per logical expert ``[layers, E]`` (summed over ranks when in a group)."""
        phys = self.window.sum(0)
        if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(phys, group=group)
        out = torch.zeros((phys.shape[0], self.num_logical), dtype=torch.int64, device=phys.device)
        out.scatter_add_(1, self.phy2log.to(phys.device), phys)
        return out

    def rearrange(self, layer_weights: list[list[torch.Tensor]], group=None) -> int:
        load = self.logical_load(group).cpu()
        new_phy2log, log2phy, logcnt = rebalance_experts(load, self.num_phys, self.cfg.num_groups,
                                                         self.cfg.num_nodes, self.world)
        moved = shuffle_expert_weights(self.phy2log, new_phy2log, layer_weights, group)
        self.phy2log, self.log2phy, self.logcnt = new_phy2log, log2phy, logcnt
        self.rearrangements += 1
        return moved

    def balancedness(self, load: torch.Tensor | None = None) -> float:
        """mean / max of per-rank load under the current mapping (1.0 = perfectly even)."""
        phys = (self.window.sum(0) if load is None else load).float()
        per_rank = phys.view(phys.shape[0], self.world, -1).sum(-1)
        return float((per_rank.mean(-1) / per_rank.max(-1).values.clamp_min(1)).mean())
