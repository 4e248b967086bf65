"""Optimizers beyond the fused sharded AdamW: Muon and a host-swapped AdamW.

* ``newton_schulz`` / ``Muon`` - momentum orthogonalised by a quintic Newton-Schulz iteration with the
  coefficients (3.4445, -4.7750, 2.0315); update scale ``lr * sqrt(max(rows, cols)) * matched_adamw_rms`` so a Muon
  step has the RMS of an AdamW step; embeddings, heads and 1-D parameters fall back to AdamW
  (mindspeed_mm/optimizer/muon.py:11-57, mindspeed_mm/fsdp/optimizer/optimizer.py:158-197).
* ``AdamWSwap`` - AdamW whose moments live in pinned host memory and visit the GPU one parameter at a time,
  bounded by a byte budget (mindspeed_mm/fsdp/optimizer/swap_optimizer.py:8-257).
Both are ``torch.optim.Optimizer`` subclasses for modules trained outside the sharding engine (LoRA adapters,
reward heads, AE training).  Inside the sharding engine ``training.optimizer: muon`` runs the same update on the flat
shards (``parallel/fsdp.py: FSDPEngine._muon``, which calls ``newton_schulz`` here) and ``adamw_swap`` keeps the
engine's optimizer state on the host (``offload_optimizer``).
"""
from __future__ import annotations

from typing import Iterable, Optional

import torch


def newton_schulz(g: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    """Approximate the orthogonal polar factor of a 2-D matrix."""
    a, b, c = 3.4445, -4.7750, 2.0315
    x = g.bfloat16() if g.is_cuda else g.float()         # bf16 tensor-core GEMMs on the GPU, as Muon is usually run
    transposed = x.shape[0] > x.shape[1]
    if transposed:
        x = x.t()
    x = x / (x.norm() + eps)
    for _ in range(steps):
        s = x @ x.t()
        x = a * x + (b * s + c * s @ s) @ x
    return (x.t() if transposed else x).to(g.dtype)


class Muon(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, momentum=0.95, nesterov=True, ns_steps=5, weight_decay=0.0,
                 matched_adamw_rms=0.2, adamw_betas=(0.9, 0.999), adamw_eps=1e-8):
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps,
                                      weight_decay=weight_decay, matched_adamw_rms=matched_adamw_rms,
                                      adamw_betas=adamw_betas, adamw_eps=adamw_eps, use_muon=True))

    @torch.no_grad()
    def step(self):
        for grp in self.param_groups:
            for p in grp["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                g = p.grad
                if grp["use_muon"] and p.dim() == 2:
                    buf = st.setdefault("momentum", torch.zeros_like(g))
                    buf.mul_(grp["momentum"]).add_(g)
                    upd = g.add(buf, alpha=grp["momentum"]) if grp["nesterov"] else buf
                    o = newton_schulz(upd, grp["ns_steps"])
                    scale = grp["matched_adamw_rms"] * max(p.shape[0], p.shape[1]) ** 0.5
                    p.mul_(1 - grp["lr"] * grp["weight_decay"]).add_(o, alpha=-grp["lr"] * scale)
                else:
                    b1, b2 = grp["adamw_betas"]
                    st["step"] = st.get("step", 0) + 1
                    m = st.setdefault("exp_avg", torch.zeros_like(g))
                    v = st.setdefault("exp_avg_sq", torch.zeros_like(g))
                    m.mul_(b1).add_(g, alpha=1 - b1)
                    v.mul_(b2).addcmul_(g, g, value=1 - b2)
                    den = (v / (1 - b2 ** st["step"])).sqrt_().add_(grp["adamw_eps"])
                    p.mul_(1 - grp["lr"] * grp["weight_decay"]).addcdiv_(m / (1 - b1 ** st["step"]), den, value=-grp["lr"])


def muon_param_groups(named_params: Iterable, adamw_name_keys=("embed", "lm_head", "norm", "bias")):
    """2-D hidden matrices -> Muon; embeddings / heads / norms / biases -> AdamW."""
    mu, ad = [], []
    for n, p in named_params:
        (ad if (p.dim() != 2 or any(k in n for k in adamw_name_keys)) else mu).append(p)
    return [dict(params=mu, use_muon=True), dict(params=ad, use_muon=False)]


class AdamWSwap(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, device_budget_bytes: int = 1 << 30):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.budget = device_budget_bytes
        self.peak_device_state_bytes = 0

    def _host(self, like):
        t = torch.zeros(like.shape, dtype=torch.float32)
        return t.pin_memory() if torch.cuda.is_available() else t

    @torch.no_grad()
    def step(self):
        for grp in self.param_groups:
            b1, b2 = grp["betas"]
            for p in grp["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st.update(step=0, exp_avg=self._host(p), exp_avg_sq=self._host(p))
                st["step"] += 1
                nbytes = 2 * p.numel() * 4
                if nbytes > self.budget:
                    raise RuntimeError(f"parameter state of {nbytes} bytes exceeds the swap budget {self.budget}")
                m = st["exp_avg"].to(p.device, non_blocking=True)
                v = st["exp_avg_sq"].to(p.device, non_blocking=True)
                self.peak_device_state_bytes = max(self.peak_device_state_bytes, nbytes)
                g = p.grad.float()
                m.mul_(b1).add_(g, alpha=1 - b1)
                v.mul_(b2).addcmul_(g, g, value=1 - b2)
                den = (v / (1 - b2 ** st["step"])).sqrt_().add_(grp["eps"])
                p.mul_(1 - grp["lr"] * grp["weight_decay"])
                p.add_((-(grp["lr"]) * (m / (1 - b1 ** st["step"])) / den).to(p.dtype))
                st["exp_avg"].copy_(m, non_blocking=True)
                st["exp_avg_sq"].copy_(v, non_blocking=True)
