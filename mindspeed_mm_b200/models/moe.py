"""Top-k routed mixture-of-experts FFN shared by the Qwen3-VL-MoE and Qwen3.5 decoders.

Reference behaviour (mindspeed_mm/fsdp/models/qwen3vl/modeling_qwen3_vl_moe.py:104-180): router =
``softmax(fp32) -> top-k -> renormalise -> cast``; experts stored fused as ``gate_up_proj [E, H, 2F]`` and
``down_proj [E, F, H]``.  Under expert parallelism the experts module only holds its rank's ``E / ep`` experts and its
forward is the dispatcher in ``parallel/ep.py``; the auxiliary load-balancing loss is kept when
``router_aux_loss_coef > 0``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..parallel import ep as epmod
from ..parallel.state import get_parallel_state
from .qwen2_5_vl import Linear, TextConfig


@dataclass
class MoETextConfig(TextConfig):
    num_experts: int = 128
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 768
    norm_topk_prob: bool = True
    router_aux_loss_coef: float = 0.0
    qk_norm: bool = True
    ep_dispatcher: str = "alltoall"


class FusedExperts(nn.Module):
    """Holds ``num_local`` experts; ``forward`` routes through the EP dispatcher when the group is > 1."""

    def __init__(self, c: MoETextConfig, num_local: Optional[int] = None):
        super().__init__()
        self.c = c
        n = num_local if num_local is not None else c.num_experts
        self.gate_up_proj = nn.Parameter(torch.empty(n, c.hidden_size, 2 * c.moe_intermediate_size))
        self.down_proj = nn.Parameter(torch.empty(n, c.moe_intermediate_size, c.hidden_size))
        # > 0 (``features.enable_ep_balance``): duplicate up to that many hot experts per rank for each call
        self.ep_balance_max_dup = 0
        self.last_balance_plan = None

    def forward(self, tokens, topk_ids, probs):
        ps = get_parallel_state()
        if ps.enabled("ep"):
            kind = self.c.ep_dispatcher
            if kind in ("p2p", "mc2") and not (tokens.is_cuda and tokens.dtype == torch.bfloat16 and ops.get_tier() == "native"):
                kind = "alltoall"                      # the peer-memory dispatcher is GPU / bf16 only
            fn = {"allgather": epmod.ep_forward_allgather, "p2p": epmod.ep_forward_p2p,
                  "mc2": epmod.ep_forward_p2p}.get(kind, epmod.ep_forward_alltoall)
            if self.ep_balance_max_dup > 0 and kind in ("alltoall", "allgather"):
                from ..parallel.ep_balance import balanced_forward
                out, self.last_balance_plan = balanced_forward(fn, tokens, topk_ids, probs, self.gate_up_proj, self.down_proj,
                                                               self.c.num_experts, ps.get_ep_group(), self.ep_balance_max_dup)
                return out
            return fn(tokens, topk_ids, probs, self.gate_up_proj, self.down_proj, self.c.num_experts, ps.get_ep_group())
        return ops.moe_experts(tokens, topk_ids, probs, self.gate_up_proj, self.down_proj)


class _AttachAux(torch.autograd.Function):
    """Identity on ``y`` whose backward also feeds ``scale`` into the auxiliary loss, so that the router receives the
    load-balancing gradient wherever the block's backward runs (inside a recomputed unit too) without the term being
    part of the scalar the training loop differentiates.  The scale is that of the main loss: ``coef / moe_layers``
    (the model-level term is ``coef * mean over layers``); gradient accumulation and data-parallel averaging are applied
    by the engine to both alike."""

    @staticmethod
    def forward(ctx, y, aux, scale):
        ctx.scale = scale
        ctx.aux_meta = (aux.dtype, aux.device)
        return y

    @staticmethod
    def backward(ctx, gy):
        dt, dev = ctx.aux_meta
        return gy, torch.full((), ctx.scale, dtype=dt, device=dev), None


class SparseMoeBlock(nn.Module):
    def __init__(self, c: MoETextConfig, num_local: Optional[int] = None):
        super().__init__()
        self.c = c
        self.gate = Linear(c.hidden_size, c.num_experts, bias=False)
        self.experts = FusedExperts(c, num_local)
        self.aux_loss = None       # detached value of the last call (for logging)
        self.aux_scale = None      # gradient scale of the auxiliary term; models set coef / number of MoE layers

    def forward(self, x):
        logits = F.linear(x, self.gate.weight)                     # tiny GEMM; keep in torch
        p = torch.softmax(logits.float(), dim=-1)
        w, ids = torch.topk(p, self.c.num_experts_per_tok, dim=-1)
        if self.c.norm_topk_prob:
            w = w / w.sum(-1, keepdim=True)
        w = w.to(x.dtype)
        run = getattr(self.experts, "_fsdp_run", None)
        out = run(self.experts, x, ids, w) if run is not None else self.experts(x, ids, w)
        self.aux_loss = None
        if self.c.router_aux_loss_coef > 0:
            aux = epmod.load_balancing_loss(logits, ids, self.c.num_experts)
            self.aux_loss = aux.detach()
            if torch.is_grad_enabled() and aux.requires_grad:
                scale = self.aux_scale if self.aux_scale is not None else self.c.router_aux_loss_coef
                out = _AttachAux.apply(out, aux, float(scale))
        return out
