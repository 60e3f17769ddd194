"""Expert placement balancing under expert parallelism.

Every expert-parallel rank holds ``E / ep`` experts of each MoE layer and the grouped GEMMs of a step finish when the most
loaded rank finishes.  The balancer accumulates how many (token, k) slots the router sent to every expert, searches for a few
pairwise exchanges of experts between ranks that lower the heaviest rank's load, and carries them out: the two experts' weights and
their optimiser state (fp32 master values and both moments, wherever the ZeRO sharding put them) change ranks, and the two rows
of the replicated router matrix trade places, so that the network computes the same function as before with a different
physical layout.  A slot therefore has no identity beyond "row of the router": checkpoints written afterwards are consistent
by construction (their expert keys are slot numbers, and the router rows were permuted with them).

The search is a beam search over sequences of exchanges scored by (load of the heaviest rank, sum of squared rank loads); it
stops when the heaviest rank is within ``tolerance`` of the mean or when no candidate improves.  Each layer gets its own plan.

The reference vendors the same capability (ColossalAI ``colossalai/moe/load_balance.py:112-260`` beam search over swaps judged
by the deviation from the mean, ``:278-430`` exchange of parameters and low-level-ZeRO optimiser shards); its first-party
trainer never reaches it because its model is never converted to expert parallelism.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

Swap = Tuple[int, int]  # two slots (global expert positions: rank * E_local + local index) that trade places


def rank_loads(load: Sequence[float], e_local: int) -> List[float]:
    return [float(sum(load[r * e_local:(r + 1) * e_local])) for r in range(len(load) // e_local)]


def _score(v: Sequence[float], e_local: int) -> Tuple[float, float]:
    rl = rank_loads(v, e_local)
    return max(rl), sum(x * x for x in rl)


def plan_swaps(load: Sequence[float], e_local: int, beam_width: int = 8, tolerance: float = 0.1,
               max_swaps: Optional[int] = None) -> List[Swap]:
    """``load[s]`` = demand of the expert in slot ``s`` (rank ``s // e_local``).  Returns the exchanges, in order."""
    E = len(load)
    ranks = E // e_local
    total = float(sum(load))
    if ranks < 2 or e_local < 2 or total <= 0:
        return []  # one expert per rank: every placement has the same rank loads
    mean = total / ranks
    max_swaps = max_swaps if max_swaps is not None else E
    start = tuple(float(x) for x in load)
    best_v, best_swaps, best_s = start, [], _score(start, e_local)
    frontier: List[Tuple[Tuple[float, ...], List[Swap]]] = [(start, [])]
    for _ in range(max_swaps):
        if best_s[0] <= mean * (1.0 + tolerance):
            break
        cand: Dict[Tuple[float, ...], List[Swap]] = {}
        for v, swaps in frontier:
            rl = rank_loads(v, e_local)
            heavy = max(range(ranks), key=rl.__getitem__)
            for a in range(heavy * e_local, (heavy + 1) * e_local):
                for b in range(E):
                    if b // e_local == heavy or v[b] >= v[a]:
                        continue  # only exchanges that take load off the heaviest rank
                    w = list(v)
                    w[a], w[b] = w[b], w[a]
                    cand.setdefault(tuple(w), swaps + [(a, b)])
        if not cand:
            break
        ranked = sorted(cand.items(), key=lambda kv: _score(kv[0], e_local))[:beam_width]
        frontier = ranked
        s0 = _score(ranked[0][0], e_local)
        if s0 < best_s:
            best_v, best_swaps, best_s = ranked[0][0], ranked[0][1], s0
        else:
            break
    return best_swaps


def imbalance(load: Sequence[float], e_local: int) -> float:
    """Heaviest rank's load over the mean rank load (1.0 = perfectly even)."""
    rl = rank_loads(load, e_local)
    m = sum(rl) / max(len(rl), 1)
    return max(rl) / m if m > 0 else 1.0


class ExpertLoadBalancer:
    """``balance()`` is collective over all ranks of the mesh.  ``engine`` is the ZeRO optimiser that owns the parameters
    (``parallel/zero.py: ShardedEngine``); without one only the weights move."""

    def __init__(self, model, mesh, engine=None, beam_width: int = 8, tolerance: float = 0.1, max_swaps: Optional[int] = None):
        self.model, self.mesh, self.engine = model, mesh, engine
        self.beam_width, self.tolerance, self.max_swaps = beam_width, tolerance, max_swaps
        self.layers = list(model.get_moe_layers())
        self.names = {id(p): n for n, p in model.named_parameters()}
        self.history: List[Dict[str, Any]] = []

    # -- measurement ------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def demand(self) -> List[torch.Tensor]:
        """Per layer, the slots routed to every expert since the statistics were last reset, summed over all ranks."""
        if not self.layers:
            return []
        d = torch.stack([l.expert_demand.to(torch.float64) for l in self.layers])
        if dist.is_initialized() and self.mesh.world > 1:
            # ranks of one tensor / pipeline group see different layers or the same tokens; plain data-parallel and
            # expert-parallel ranks see different tokens: their counts add up
            dev = d.device
            if dist.get_backend() == "nccl" and not d.is_cuda:
                d = d.cuda()
            dist.all_reduce(d, group=self.mesh.group("dp"))
            d = d.to(dev)
        return list(d)

    def plan(self, demand: Optional[List[torch.Tensor]] = None) -> List[List[Swap]]:
        demand = demand if demand is not None else self.demand()
        ep = self.mesh.ep_size
        return [plan_swaps(d.tolist(), l.num_experts // ep, self.beam_width, self.tolerance, self.max_swaps)
                for l, d in zip(self.layers, demand)]

    # -- execution ----------------------------------------------------------------------------------------------------
    def _exchange(self, mine: torch.Tensor, peer_ep: int) -> torch.Tensor:
        """Trades a tensor with the rank at expert-parallel coordinate ``peer_ep`` (same position on every other axis)."""
        got = torch.empty_like(mine)
        c = self.mesh.coord
        peer = self.mesh.rank_of(c.pp, c.dp, peer_ep, c.tp, c.sp)
        ops = [dist.P2POp(dist.isend, mine.contiguous(), peer), dist.P2POp(dist.irecv, got, peer)]
        if self.mesh.rank > peer:
            ops.reverse()
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        return got

    @torch.no_grad()
    def _swap_experts(self, layer, a: int, b: int) -> None:
        ep, me = self.mesh.ep_size, self.mesh.coord.ep
        el = layer.num_experts // ep
        ra, rb = a // el, b // el
        eng = self.engine
        # expert weights and their optimiser state: the two owners trade rows (every expert-data-parallel replica with its twin)
        for p in (layer.experts_w1, layer.experts_w2):
            name = self.names[id(p)]
            if ra == rb:
                if me == ra:
                    la, lb = a % el, b % el
                    if eng is not None:
                        st = eng.read_rows(name, [la, lb])
                        eng.write_rows(name, [lb, la], st)
                    else:
                        tmp = p.data[la].clone()
                        p.data[la].copy_(p.data[lb])
                        p.data[lb].copy_(tmp)
                continue
            if me not in (ra, rb):
                continue
            local, peer = (a % el, rb) if me == ra else (b % el, ra)
            if eng is not None:
                st = eng.read_rows(name, [local])
                eng.write_rows(name, [local], self._exchange(st, peer))
            else:
                p.data[local].copy_(self._exchange(p.data[local].clone(), peer))
        # router rows (replicated on every rank; state possibly sharded over the data-parallel group)
        g = layer.gate.weight
        gname = self.names[id(g)]
        if eng is not None:
            st = eng.read_rows(gname, [a, b])
            eng.write_rows(gname, [b, a], st)
        else:
            tmp = g.data[a].clone()
            g.data[a].copy_(g.data[b])
            g.data[b].copy_(tmp)
        d = layer.expert_demand
        d[a], d[b] = d[b].clone(), d[a].clone()

    @torch.no_grad()
    def apply(self, plans: List[List[Swap]]) -> int:
        n = 0
        for layer, swaps in zip(self.layers, plans):
            for a, b in swaps:
                self._swap_experts(layer, a, b)
                n += 1
        return n

    def balance(self, reset_statistics: bool = True) -> Dict[str, Any]:
        """Measure, plan, exchange.  Returns what was done: per layer the heaviest-rank-over-mean ratio before and after."""
        demand = self.demand()
        plans = self.plan(demand)
        ep = self.mesh.ep_size
        report: Dict[str, Any] = {"swaps": 0, "layers": []}
        for layer, d, swaps in zip(self.layers, demand, plans):
            el = layer.num_experts // ep
            v = d.tolist()
            before = imbalance(v, el)
            for a, b in swaps:
                v[a], v[b] = v[b], v[a]
            report["layers"].append({"layer": layer.layer_idx, "before": before, "after": imbalance(v, el), "swaps": list(swaps)})
        report["swaps"] = self.apply(plans)
        if reset_statistics:
            for layer in self.layers:
                layer.get_routing_stats(reset=True)
        self.history.append(report)
        return report
