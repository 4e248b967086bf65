"""Expert parallelism: token dispatch / combine around locally held experts.

Each rank of the EP group owns ``E / ep`` consecutive experts.  ``ep_forward`` does
  1. histogram of local routing, all-gathered over the group (``[ep, E]`` counts)
  2. permute local (token, slot) pairs to expert order; all-to-all-v dispatch with
        input_splits[r]  = tokens I route to rank r's experts,
        output_splits[r] = tokens rank r routes to my experts
  3. received tokens arrive source-rank-major; a second permute makes them expert-major
  4. grouped GEMM -> SwiGLU -> grouped GEMM on the local experts
  5. inverse permute, all-to-all-v combine, prob-weighted un-permute (sum over the k slots)
which is the algebra of the reference's ``alltoall`` dispatcher
(mindspeed_mm/fsdp/distributed/expert_parallel/ep_dispatcher.py:175-319; splits at :192-212, second permute
:284-286).  The ``allgather`` dispatcher gathers all tokens, computes local experts on the tokens routed to
them and reduce-scatters the outputs (comm.py:45-231).  A rank that receives no tokens still runs the
experts on an empty slab so that every parameter gets a (zero) gradient (ep_dispatcher.py:142-152).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops


class _AllToAllV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, in_splits, out_splits, group):
        ctx.in_splits, ctx.out_splits, ctx.group = in_splits, out_splits, group
        out = x.new_empty(sum(out_splits), *x.shape[1:])
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty(sum(ctx.in_splits), *g.shape[1:])
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.in_splits, input_split_sizes=ctx.out_splits,
                               group=ctx.group)
        return out, None, None, None


def all_to_all_v(x, in_splits: List[int], out_splits: List[int], group):
    return _AllToAllV.apply(x, list(in_splits), list(out_splits), group)


def dispatch_plan(topk_ids: torch.Tensor, num_experts: int, group) -> Tuple[torch.Tensor, List[int], List[int], torch.Tensor]:
    """Returns (hist_all [ep, E] on CPU, input_splits, output_splits, tokens_per_local_expert_by_source [ep, E_local])."""
    ep = dist.get_world_size(group)
    rank = dist.get_rank(group)
    e_local = num_experts // ep
    hist = torch.bincount(topk_ids.reshape(-1), minlength=num_experts)
    allh = torch.empty(ep * num_experts, dtype=hist.dtype, device=hist.device)
    dist.all_gather_into_tensor(allh, hist, group=group)
    allh_c = allh.view(ep, num_experts).cpu()
    input_splits = allh_c[rank].view(ep, e_local).sum(1).tolist()
    mine = allh_c[:, rank * e_local:(rank + 1) * e_local]            # [src rank, local expert]
    output_splits = mine.sum(1).tolist()
    return allh_c, input_splits, output_splits, mine


def experts_mlp(x, gate_up, down, counts):
    """x rows grouped by expert (counts per expert); gate_up [E,H,2F], down [E,F,H]."""
    if x.is_cuda and x.shape[0] and ops.get_tier() == "native" and ops._nat().moe_supported(x, gate_up, down):
        # the tcgen05 grouped kernels work on the 128-aligned expert layout: hand them the rows as a top-1 routing whose
        # expert ids are already sorted (the permutation into the aligned layout is then a copy with gaps)
        c = torch.as_tensor([int(v) for v in counts], dtype=torch.long, device=x.device)
        ids = torch.repeat_interleave(torch.arange(c.numel(), device=x.device), c, output_size=x.shape[0])
        return ops.moe_experts(x, ids[:, None], torch.ones(x.shape[0], 1, dtype=x.dtype, device=x.device), gate_up, down)
    h = ops.grouped_gemm(x, gate_up, counts)
    return ops.grouped_gemm(ops.swiglu(h), down, counts)


def ep_forward_alltoall(tokens, topk_ids, probs, gate_up, down, num_experts: int, group) -> torch.Tensor:
    """tokens [T,H]; topk_ids/probs [T,k]; gate_up/down hold this rank's E/ep experts."""
    T, k = topk_ids.shape
    ep = dist.get_world_size(group)
    e_local = num_experts // ep
    _, in_splits, out_splits, by_src = dispatch_plan(topk_ids, num_experts, group)
    permuted, order = ops.moe_permute(tokens, topk_ids)              # expert-major == destination-rank-major
    recv = all_to_all_v(permuted, in_splits, out_splits, group)       # source-rank-major, expert-minor
    # second permute: (src, expert) blocks -> expert-major
    blk = by_src.reshape(-1)                                          # lengths of the (src, e) blocks in arrival order
    starts = torch.cumsum(blk, 0) - blk
    idx = []
    for e in range(e_local):
        for s in range(ep):
            b = s * e_local + e
            idx.append(torch.arange(int(starts[b]), int(starts[b] + blk[b])))
    gather_idx = (torch.cat(idx) if idx else torch.zeros(0, dtype=torch.long)).to(recv.device)
    x = recv.index_select(0, gather_idx)
    counts = by_src.sum(0).tolist()
    y = experts_mlp(x, gate_up, down, counts)
    back = torch.empty_like(y).index_copy(0, gather_idx, y) if y.shape[0] else y
    combined = all_to_all_v(back, out_splits, in_splits, group)
    return ops.moe_unpermute(combined, order, probs)


def ep_forward_allgather(tokens, topk_ids, probs, gate_up, down, num_experts: int, group) -> torch.Tensor:
    """All-gather tokens and routing, run the local experts on what is routed to them, reduce-scatter back."""
    ep, rank = dist.get_world_size(group), dist.get_rank(group)
    e_local = num_experts // ep
    all_tok = _AllGather0.apply(tokens, group)
    ids = [torch.empty_like(topk_ids) for _ in range(ep)]
    dist.all_gather(ids, topk_ids.contiguous(), group=group)
    all_ids = torch.cat(ids)
    all_probs = _AllGather0.apply(probs, group)
    lo = rank * e_local
    local = (all_ids >= lo) & (all_ids < lo + e_local)
    ids_l = torch.where(local, all_ids - lo, torch.full_like(all_ids, e_local))      # e_local = "not mine" bucket
    permuted, order = ops.moe_permute(all_tok, ids_l)
    counts = torch.bincount(ids_l.reshape(-1), minlength=e_local + 1).tolist()
    n_mine = sum(counts[:e_local])
    y = experts_mlp(permuted[:n_mine], gate_up, down, counts[:e_local])
    y = torch.cat([y, y.new_zeros(permuted.shape[0] - n_mine, y.shape[1])])
    out_full = ops.moe_unpermute(y, order, all_probs * local.to(all_probs.dtype))
    return _ReduceScatter0.apply(out_full, group)


class _AllGather0(torch.autograd.Function):
    """All-gather along dim 0; backward SUMS the ranks' gradients for my slice (reduce-scatter), because
    every rank used my tokens for different experts."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        outs = [torch.empty_like(x) for _ in range(dist.get_world_size(group))]
        dist.all_gather(outs, x.contiguous(), group=group)
        return torch.cat(outs)

    @staticmethod
    def backward(ctx, g):
        return _ReduceScatter0.apply(g, ctx.group), None


class _ReduceScatter0(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w = dist.get_world_size(group)
        out = x.new_empty(x.shape[0] // w, *x.shape[1:])
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group) if x.is_cuda else _rs_cpu(out, x, group)
        return out

    @staticmethod
    def backward(ctx, g):
        w = dist.get_world_size(ctx.group)
        outs = [torch.empty_like(g) for _ in range(w)]
        dist.all_gather(outs, g.contiguous(), group=ctx.group)
        return torch.cat(outs), None


def _rs_cpu(out, x, group):
    w, r = dist.get_world_size(group), dist.get_rank(group)
    y = x.clone()
    dist.all_reduce(y, group=group)
    out.copy_(y.chunk(w)[r])


def load_balancing_loss(router_logits: torch.Tensor, topk_ids: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Switch-style auxiliary loss: E * sum_e (fraction of routed slots to e) * (mean router prob of e)."""
    p = torch.softmax(router_logits.float(), dim=-1)
    k = topk_ids.shape[1]
    frac = torch.zeros(num_experts, device=p.device).index_add_(0, topk_ids.reshape(-1), torch.ones(topk_ids.numel(), device=p.device))
    frac = frac / topk_ids.numel() * k
    return num_experts * (frac / k * p.mean(0)).sum() * k


# ----------------------------------------------------------------------------------------------------------------
# Peer-memory dispatcher ("mc2" in the reference's naming: fused communication + expert GEMM input layout,
# fsdp/ops/moe_ops/gemm_mc2.py, ep_dispatcher.py:319-397).  A token row travels once: straight from the sender's
# activation tensor into its row of the destination rank's 128-aligned expert slab over NVLink, and the expert
# outputs are pulled back the same way.  All-to-all, permute and the alignment padding are one pass.
class P2PDispatcher:
    """Symmetric-memory slabs + row maps for one EP group.  ``capacity_factor`` bounds the rows a rank can receive
    (relative to a perfectly balanced routing); above it the caller falls back to the all-to-all dispatcher."""

    _instances: dict = {}

    @classmethod
    def get(cls, group, hidden: int, device, pairs: int, e_local: int, capacity_factor: float = 2.0):
        key = (id(group), hidden, str(device))
        inst = cls._instances.get(key)
        need = int(pairs * capacity_factor) + 128 * e_local
        if inst is None or inst.cap_rows < need:
            inst = cls._instances[key] = cls(group, hidden, device, need)
        return inst

    def __init__(self, group, hidden: int, device, cap_rows: int):
        from ..comm.symm import SymmArena
        self.group, self.H = group, hidden
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.cap_rows = (cap_rows + 127) // 128 * 128
        nbytes = self.cap_rows * hidden * 2
        self.arena = SymmArena(2 * nbytes + 8192, group, torch.device(device))
        self.off_in, self.off_out = self.arena.carve(nbytes), self.arena.carve(nbytes)
        self.buf_in = self.arena.view(self.off_in, self.cap_rows * hidden, torch.bfloat16).view(self.cap_rows, hidden)
        self.buf_out = self.arena.view(self.off_out, self.cap_rows * hidden, torch.bfloat16).view(self.cap_rows, hidden)
        self.ptrs_in, self.ptrs_out = self.arena.peer_ptrs(self.off_in), self.arena.peer_ptrs(self.off_out)

    # -- kernels -------------------------------------------------------------------------------------------------
    def push(self, src, src_row, dst_rank, dst_row, R: int, pad_rows):
        """Rows of ``src`` -> peers' incoming slabs; returns this rank's slab [R, H] (pad rows zero)."""
        from ..ops import native
        self.arena.barrier()
        native._check(native.lib().mm_p2p_scatter_rows(src.data_ptr(), src_row.data_ptr(), dst_rank.data_ptr(),
                                                       dst_row.data_ptr(), self.ptrs_in, src_row.numel(), self.H,
                                                       self.world, native._st()), "p2p_scatter_rows")
        self.arena.barrier()
        x = self.buf_in[:R].clone()
        if pad_rows.numel():
            x.index_fill_(0, pad_rows, 0)
        return x

    def pull(self, y, dst_rank, dst_row):
        """Publishes ``y`` [R, H] as this rank's outgoing slab and fetches the rows (dst_rank, dst_row) from peers."""
        from ..ops import native
        n = dst_rank.numel()
        out = torch.empty(n, self.H, dtype=torch.bfloat16, device=y.device)
        self.buf_out[: y.shape[0]].copy_(y)
        self.arena.barrier()
        native._check(native.lib().mm_p2p_gather_rows(out.data_ptr(), dst_rank.data_ptr(), dst_row.data_ptr(), self.ptrs_out,
                                                      n, self.H, self.world, native._st()), "p2p_gather_rows")
        self.arena.barrier()
        return out


class _P2PPush(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, disp, plan):
        ctx.disp, ctx.plan = disp, plan
        return disp.push(tokens.contiguous(), plan["pair_token"], plan["dst_rank"], plan["dst_row"], plan["R"], plan["pad_rows"])

    @staticmethod
    def backward(ctx, g):
        plan = ctx.plan
        pairs = ctx.disp.pull(g.contiguous(), plan["dst_rank"], plan["dst_row"])          # [T*k, H]
        return pairs.view(plan["T"], plan["k"], -1).sum(1), None, None


class _P2PPull(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, disp, plan):
        ctx.disp, ctx.plan = disp, plan
        return disp.pull(y.contiguous(), plan["dst_rank"], plan["dst_row"])

    @staticmethod
    def backward(ctx, g):
        plan = ctx.plan
        return ctx.disp.push(g.contiguous(), plan["pair_index"], plan["dst_rank"], plan["dst_row"], plan["R"],
                             plan["pad_rows"]), None, None


def p2p_plan(topk_ids: torch.Tensor, num_experts: int, group):
    """Row maps of the peer-memory dispatch.  Returns (plan dict, max rows any rank receives)."""
    ep, rank = dist.get_world_size(group), dist.get_rank(group)
    e_local = num_experts // ep
    T, k = topk_ids.shape
    dev = topk_ids.device
    flat = topk_ids.reshape(-1)
    hist = torch.bincount(flat, minlength=num_experts)
    allh = torch.empty(ep * num_experts, dtype=hist.dtype, device=dev)
    dist.all_gather_into_tensor(allh, hist, group=group)
    allh = allh.view(ep, num_experts)
    tot = allh.sum(0)                                              # rows per global expert
    padded = (tot + 127) // 128 * 128
    per_rank = padded.view(ep, e_local)
    off = torch.zeros(ep, e_local + 1, dtype=torch.int64, device=dev)
    off[:, 1:] = per_rank.cumsum(1)                                # slab offsets on every destination rank
    before_me = allh[:rank].sum(0)                                 # rows of earlier source ranks inside each expert's slab
    start_me = off[:, :-1].reshape(-1) + before_me                 # [E]: first row of MY block in expert e's slab
    order = torch.sort(flat, stable=True).indices
    ustart = torch.zeros(num_experts + 1, dtype=torch.int64, device=dev)
    ustart[1:] = hist.cumsum(0)
    sorted_e = flat[order]
    within = torch.empty_like(flat)
    within[order] = torch.arange(flat.numel(), device=dev) - ustart[sorted_e]
    my_off = off[rank]
    my_tot = tot.view(ep, e_local)[rank]
    # pad rows of my slabs: [off[e] + tot[e], off[e + 1])
    R_all = off[:, -1]
    R_max, R = int(R_all.max()), int(R_all[rank])                  # one host sync per layer, like the all-to-all splits
    ar = torch.arange(R, device=dev)
    e_of_row = torch.bucketize(ar, my_off[1:], right=True).clamp(max=e_local - 1)
    pad_rows = ar[ar >= (my_off[:-1] + my_tot)[e_of_row]]
    plan = dict(T=T, k=k, R=R, off=my_off.to(torch.int32), pad_rows=pad_rows,
                dst_rank=(flat // e_local).to(torch.int32), dst_row=(start_me[flat] + within).to(torch.int32),
                pair_token=(torch.arange(flat.numel(), device=dev) // k).to(torch.int32),
                pair_index=torch.arange(flat.numel(), device=dev, dtype=torch.int32))
    return plan, R_max


def ep_forward_p2p(tokens, topk_ids, probs, gate_up, down, num_experts: int, group, capacity_factor: float = 2.0):
    """Peer-memory dispatcher (GPU, bf16).  Falls back to the all-to-all dispatcher when a rank would receive more
    rows than the slabs hold; every rank sees the same histogram, so all ranks take the same branch."""
    from ..ops import native
    T, k = topk_ids.shape
    ep = dist.get_world_size(group)
    e_local = num_experts // ep
    disp = P2PDispatcher.get(group, tokens.shape[1], tokens.device, T * k, e_local, capacity_factor)
    plan, R_max = p2p_plan(topk_ids, num_experts, group)
    if R_max > disp.cap_rows:
        return ep_forward_alltoall(tokens, topk_ids, probs, gate_up, down, num_experts, group)
    x = _P2PPush.apply(tokens, disp, plan)
    h = native._AlignedGroupedGemm.apply(x, gate_up, plan["off"])
    y = native._AlignedGroupedGemm.apply(ops.swiglu(h), down, plan["off"])
    pairs = _P2PPull.apply(y, disp, plan)
    return native._AlignedUnpermute.apply(pairs, plan["pair_index"], probs)
