"""Layerwise-disaggregated training: U-shaped edge / cloud pipeline with unequal stage widths.

The reference's LDT patches (mindspeed_mm/patchs/layerwise_disaggregated_training/: ``u_shaped_split_learning_patch.py:41``,
``schedules_patch.py:127,732``, ``p2p_communication_patch.py:31,433-600``, ``parallel_state_patch.py:84``) let an *edge*
device keep the first layers and the last layers + loss (raw inputs and labels never leave it) while the *cloud*
runs the middle of the network, possibly with a different tensor-parallel width than the edge ("virtual" TP / DP).

Here the same thing is one schedule over a list of *virtual stages*:

* ``stages[i] = StageSpec(ranks=[...])`` names the global ranks that run stage ``i`` together.  A U-shape is
  ``[edge], [cloud...], [edge]``: the edge rank owns the first and the last stage.
* Between consecutive stages of different width a ``link`` fans activations out (every rank of the wider stage
  receives the tensor from its parent in the narrower one: the replicated input of a TP group) and fans gradients
  in (the narrower side receives from the first rank of each fan; TP stages hold identical input gradients after
  their own all-reduce, replicated DP stages are summed).
* The per-rank order of forwards and backwards comes from a unit-time simulation of 1F1B over the virtual stages
  (backward first, at most ``n_stages - i`` forwards of stage ``i`` in flight), so every rank executes a fixed
  list of operations; activations and gradients travel on separate process groups and are matched by order.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


@dataclass
class StageSpec:
    ranks: List[int]
    reduce: str = "first"            # how input gradients of a wider stage collapse: "first" (TP) or "sum" (replicas)


def u_shaped(edge_rank: int, cloud: Sequence[Sequence[int]]) -> List[StageSpec]:
    """``[edge] -> cloud stage 0 -> ... -> [edge]``; every cloud stage is a list of ranks (its TP group)."""
    return [StageSpec([edge_rank])] + [StageSpec(list(c)) for c in cloud] + [StageSpec([edge_rank])]


def simulate_1f1b(n_stages: int, n_micro: int, owner_of: Sequence[Sequence[int]]) -> Dict[int, List[Tuple[str, int, int]]]:
    """Unit-time simulation.  Returns for every rank its ordered list of ("F" | "B", stage, micro_batch)."""
    ranks = sorted({r for rs in owner_of for r in rs})
    done_f: Dict[Tuple[int, int], int] = {}
    done_b: Dict[Tuple[int, int], int] = {}
    plan: Dict[int, List[Tuple[str, int, int]]] = {r: [] for r in ranks}
    next_f = [0] * n_stages
    next_b = [0] * n_stages
    t = 0
    total = 2 * n_stages * n_micro
    executed = 0
    while executed < total:
        t += 1
        busy = set()
        chosen: List[Tuple[str, int, int]] = []
        # backward first, deepest stage first (it frees memory soonest)
        for s in range(n_stages - 1, -1, -1):
            mb = next_b[s]
            if mb >= n_micro or any(r in busy for r in owner_of[s]):
                continue
            ready = done_f.get((s, mb), 1 << 30) < t and (s == n_stages - 1 or done_b.get((s + 1, mb), 1 << 30) < t)
            if ready:
                chosen.append(("B", s, mb))
                busy.update(owner_of[s])
        for s in range(n_stages):
            mb = next_f[s]
            if mb >= n_micro or any(r in busy for r in owner_of[s]):
                continue
            in_flight = next_f[s] - next_b[s]
            ready = (s == 0 or done_f.get((s - 1, mb), 1 << 30) < t) and in_flight < n_stages - s
            if ready:
                chosen.append(("F", s, mb))
                busy.update(owner_of[s])
        if not chosen and t > 4 * total + 16:
            raise RuntimeError("pipeline simulation made no progress")
        for kind, s, mb in chosen:
            if kind == "F":
                done_f[(s, mb)] = t
                next_f[s] += 1
            else:
                done_b[(s, mb)] = t
                next_b[s] += 1
            for r in owner_of[s]:
                plan[r].append((kind, s, mb))
            executed += 1
    return plan


class DisaggregatedPipeline:
    """Runs ``stage_fn(stage, x, micro_batch)`` for the stages this rank belongs to, in simulated 1F1B order.

    ``stage_fn`` returns the activation for the next stage, or the scalar loss on the last stage.  ``shape_fn(stage,
    micro_batch)`` gives the shape of the activation *entering* ``stage``.
    """

    def __init__(self, stages: Sequence[StageSpec], stage_fn: Callable, shape_fn: Callable, dtype, device,
                 fwd_group=None, bwd_group=None, after_backward: Optional[Callable[[int], None]] = None):
        self.stages = list(stages)
        self.stage_fn, self.shape_fn, self.dtype, self.device = stage_fn, shape_fn, dtype, torch.device(device)
        self.rank = dist.get_rank()
        self.fwd_group, self.bwd_group = fwd_group, bwd_group
        self.after_backward = after_backward
        self.mine = [i for i, s in enumerate(self.stages) if self.rank in s.ranks]
        self._pending: List = []

    # ---------------------------------------------------------------------------------- links
    @staticmethod
    def _fan(narrow: List[int], wide: List[int]) -> Dict[int, List[int]]:
        """parent in the narrow stage -> its children in the wide stage (contiguous blocks)."""
        if len(wide) % len(narrow):
            raise ValueError(f"stage widths {len(narrow)} and {len(wide)} do not divide")
        k = len(wide) // len(narrow)
        return {p: wide[i * k:(i + 1) * k] for i, p in enumerate(narrow)}

    def _peers(self, src_stage: int, dst_stage: int) -> Tuple[List[int], List[int]]:
        """(ranks this rank sends to, ranks it receives from) for data flowing src_stage -> dst_stage."""
        a, b = self.stages[src_stage].ranks, self.stages[dst_stage].ranks
        send_to: List[int] = []
        recv_from: List[int] = []
        if len(b) >= len(a):
            fan = self._fan(a, b)
            if self.rank in a:
                send_to = fan[self.rank]
            if self.rank in b:
                recv_from = [p for p, ch in fan.items() if self.rank in ch]
        else:
            fan = self._fan(b, a)                   # many -> few: the reducing direction
            if self.rank in a:
                parent = [p for p, ch in fan.items() if self.rank in ch][0]
                first = fan[parent][0]
                if self.stages[src_stage].reduce == "sum" or self.rank == first:
                    send_to = [parent]
            if self.rank in b:
                ch = fan[self.rank]
                recv_from = ch if self.stages[src_stage].reduce == "sum" else ch[:1]
        return send_to, recv_from

    def _send(self, t, dsts, group):
        t = t.contiguous()
        for d in dsts:
            if d == self.rank:
                self._local.append(t)
            else:
                self._pending.append((dist.isend(t, dst=d, group=group), t))

    def _recv(self, srcs, shape, group):
        total = None
        for s in srcs:
            if s == self.rank:
                t = self._local.pop(0)
            else:
                t = torch.empty(shape, dtype=self.dtype, device=self.device)
                dist.recv(t, src=s, group=group)
            total = t if total is None else total + t
        return total

    # ---------------------------------------------------------------------------------- run
    def run(self, micro_batches: Sequence[dict]) -> List[torch.Tensor]:
        n = len(self.stages)
        plan = simulate_1f1b(n, len(micro_batches), [s.ranks for s in self.stages])[self.rank]
        store: Dict[Tuple[int, int], Tuple[Optional[torch.Tensor], torch.Tensor]] = {}
        losses: List[torch.Tensor] = []
        self._local: List[torch.Tensor] = []
        for kind, s, i in plan:
            mb = micro_batches[i]
            if kind == "F":
                x = None
                if s > 0:
                    _, srcs = self._peers(s - 1, s)
                    x = self._recv(srcs, self.shape_fn(s, mb), self.fwd_group).requires_grad_()
                out = self.stage_fn(s, x, mb)
                if s < n - 1:
                    dsts, _ = self._peers(s, s + 1)
                    self._send(out.detach(), dsts, self.fwd_group)
                else:
                    losses.append(out.detach())
                store[(s, i)] = (x, out)
            else:
                x, out = store.pop((s, i))
                if s == n - 1:
                    out.backward()
                else:
                    # gradients flow (s + 1) -> s: the roles of the two stages are swapped
                    _, srcs = self._peers_back(s)
                    g = self._recv(srcs, tuple(out.shape), self.bwd_group)
                    torch.autograd.backward(out, g)
                if s > 0:
                    dsts, _ = self._peers_back(s - 1)
                    self._send(x.grad, dsts, self.bwd_group)
                if self.after_backward is not None:
                    self.after_backward(s)
        for w, _ in self._pending:
            w.wait()
        self._pending = []
        return losses

    def _peers_back(self, s: int) -> Tuple[List[int], List[int]]:
        """Peers for the gradient of the activation between stage ``s`` and ``s + 1`` (flows s + 1 -> s)."""
        a, b = self.stages[s + 1].ranks, self.stages[s].ranks           # a = gradient producers, b = consumers
        send_to: List[int] = []
        recv_from: List[int] = []
        if len(a) >= len(b):
            fan = self._fan(b, a)
            mode = self.stages[s + 1].reduce
            if self.rank in a:
                parent = [p for p, ch in fan.items() if self.rank in ch][0]
                if mode == "sum" or self.rank == fan[parent][0]:
                    send_to = [parent]
            if self.rank in b:
                ch = fan[self.rank]
                recv_from = ch if mode == "sum" else ch[:1]
        else:
            fan = self._fan(a, b)                   # narrow producer -> wide consumers: replicate the gradient
            if self.rank in a:
                send_to = fan[self.rank]
            if self.rank in b:
                recv_from = [p for p, ch in fan.items() if self.rank in ch]
        return send_to, recv_from
