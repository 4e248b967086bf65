"""Preference optimisation and RL post-training losses.

* ``dpo_loss``            - Direct Preference Optimisation on sequence log-probabilities (policy vs frozen reference),
                            with the sigmoid / hinge / IPO variants and label smoothing
                            (mindspeed_mm/tasks/rl/dpo/dpo_trainer.py; posttrain_sora_dpo.py for the diffusion variant).
* ``diffusion_dpo_loss``  - Diffusion-DPO: preferences on denoising errors instead of log-probabilities.
* ``grpo_advantages`` / ``grpo_loss`` - group-relative advantages (reward normalised inside each prompt group) and the
                            clipped policy-gradient objective with an optional KL penalty, as used by DanceGRPO for
                            Wan / FLUX (mindspeed_mm/tasks/rl/soragrpo/{sora_grpo_trainer,flux_grpo_trainer}.py).
* ``sde_step_logprob``    - log-probability of one stochastic flow-matching sampler step (the "action" in DanceGRPO).
* ``bradley_terry_loss``  - reward-model loss (models/reward_model.py:17).
All are pure functions of tensors so they run on any backend and are unit-tested on CPU.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def sequence_logprobs(token_logprobs: torch.Tensor, labels: torch.Tensor, cu_seqlens: torch.Tensor, ignore_index=-100):
    """Sum of token log-probs per packed sample.  token_logprobs, labels: [T]."""
    seg = torch.bucketize(torch.arange(labels.numel(), device=labels.device), cu_seqlens[1:].long(), right=True)
    valid = (labels != ignore_index).to(token_logprobs.dtype)
    n = cu_seqlens.numel() - 1
    return torch.zeros(n, dtype=token_logprobs.dtype, device=labels.device).index_add_(0, seg, token_logprobs * valid)


def dpo_loss(policy_chosen, policy_rejected, ref_chosen, ref_rejected, beta: float = 0.1, label_smoothing: float = 0.0,
             loss_type: str = "sigmoid") -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    logits = (policy_chosen - policy_rejected) - (ref_chosen - ref_rejected)
    if loss_type == "sigmoid":
        loss = -F.logsigmoid(beta * logits) * (1 - label_smoothing) - F.logsigmoid(-beta * logits) * label_smoothing
    elif loss_type == "hinge":
        loss = torch.relu(1 - beta * logits)
    elif loss_type == "ipo":
        loss = (logits - 1 / (2 * beta)) ** 2
    else:
        raise ValueError(f"unknown dpo loss_type {loss_type}")
    return loss.mean(), beta * (policy_chosen - ref_chosen).detach(), beta * (policy_rejected - ref_rejected).detach()


def diffusion_dpo_loss(err_policy_w, err_policy_l, err_ref_w, err_ref_l, beta: float = 5000.0):
    """err_*: per-sample denoising MSE of the preferred (w) / rejected (l) sample under policy / reference."""
    inside = -0.5 * beta * ((err_policy_w - err_ref_w) - (err_policy_l - err_ref_l))
    return -F.logsigmoid(inside).mean()


def grpo_advantages(rewards: torch.Tensor, group_size: int, eps: float = 1e-6) -> torch.Tensor:
    """rewards [n_prompts * group_size] -> advantages normalised inside each group of samples of one prompt."""
    r = rewards.view(-1, group_size)
    return ((r - r.mean(1, keepdim=True)) / (r.std(1, keepdim=True) + eps)).reshape(-1)


def grpo_loss(logp_new, logp_old, advantages, clip_range: float = 1e-4, adv_clip_max: float = 5.0,
              kl: Optional[torch.Tensor] = None, kl_coef: float = 0.0):
    adv = advantages.clamp(-adv_clip_max, adv_clip_max)
    ratio = torch.exp(logp_new - logp_old)
    unclipped = -adv * ratio
    clipped = -adv * ratio.clamp(1 - clip_range, 1 + clip_range)
    loss = torch.maximum(unclipped, clipped).mean()
    if kl is not None and kl_coef > 0:
        loss = loss + kl_coef * kl.mean()
    return loss


def sde_step_logprob(prev_sample, sample, model_output, sigma, sigma_next, eta: float = 0.3):
    """Gaussian log-density of ``prev_sample`` under the stochastic flow-matching step from ``sample``.
    mean = x + v * dt + drift correction, std = eta * sqrt(-dt)."""
    dt = sigma_next - sigma
    std = eta * math.sqrt(max(-float(dt), 1e-12))
    pred_x0 = sample - sigma * model_output
    score = -(sample - pred_x0 * (1 - sigma)) / (sigma ** 2 + 1e-12)
    mean = sample + model_output * dt - 0.5 * (std ** 2) * score
    lp = -((prev_sample.detach() - mean) ** 2) / (2 * std ** 2) - math.log(std) - 0.5 * math.log(2 * math.pi)
    return lp.flatten(1).mean(1)


def bradley_terry_loss(reward_chosen, reward_rejected):
    return -F.logsigmoid(reward_chosen - reward_rejected).mean()
