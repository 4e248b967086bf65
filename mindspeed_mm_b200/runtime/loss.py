"""Loss normalisation modes of the native trainer.

``raw`` leaves the model's own loss untouched; ``default`` is the token mean of the micro-batch;
``per_token_loss`` divides the token-sum by the *global* number of valid tokens in the optimizer
step (all-reduced over data-parallel ranks) so that every token weighs the same whatever the
packing; ``per_sample_loss`` averages each packed sample first and then the samples.
Reference: mindspeed_mm/fsdp/loss/loss_func.py:51-142.  The model returns ``(loss_sum, n_valid)``
(optionally per-token losses for the per-sample mode) and this module turns it into the scalar that
is back-propagated; the engine's reduce-scatter then divides by the data-parallel size.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

LOSS_TYPES = ("raw", "default", "per_token_loss", "per_sample_loss")


def build_loss(loss_type: str = "default", dp_group=None, dp_world: int = 1, alpha: Optional[float] = None):
    if loss_type not in LOSS_TYPES:
        raise ValueError(f"loss_type must be one of {LOSS_TYPES}, got {loss_type!r}")

    def loss_fn(loss_sum: torch.Tensor, n_valid: torch.Tensor, per_sample: Optional[torch.Tensor] = None):
        if loss_type == "raw":
            return loss_sum
        if loss_type == "default":
            return loss_sum / n_valid.clamp(min=1).to(loss_sum.dtype)
        if loss_type == "per_token_loss":
            if alpha is not None:
                return loss_sum / alpha
            total = n_valid.detach().clone().float()
            if dp_world > 1:
                dist.all_reduce(total, group=dp_group)
            # the engine averages gradients over dp ranks, so undo that with * dp_world
            return loss_sum * dp_world / total.clamp(min=1)
        if per_sample is None:
            raise ValueError("per_sample_loss needs the per-sample means from the model")
        return per_sample.mean()

    return loss_fn


def per_sample_means(token_losses: torch.Tensor, labels: torch.Tensor, cu_seqlens: torch.Tensor,
                     ignore_index: int = -100) -> torch.Tensor:
    """Mean loss of every packed sample (samples without valid tokens contribute 0)."""
    n = cu_seqlens.numel() - 1
    seg = torch.bucketize(torch.arange(labels.numel(), device=labels.device), cu_seqlens[1:].long(), right=True)
    valid = (labels != ignore_index).to(token_losses.dtype)
    s = torch.zeros(n, dtype=token_losses.dtype, device=labels.device).index_add_(0, seg, token_losses * valid)
    c = torch.zeros(n, dtype=token_losses.dtype, device=labels.device).index_add_(0, seg, valid)
    return s / c.clamp(min=1)
