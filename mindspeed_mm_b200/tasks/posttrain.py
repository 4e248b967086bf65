"""Post-training loops built on the loss functions of :mod:`.preference`.

* ``DiffusionDPOTrainer``  -- Diffusion-DPO for the DiTs: the preferred / rejected latents of a pair are noised with
  the SAME noise and timestep, the policy and a frozen reference predict the velocity, and the per-sample error
  differences enter ``diffusion_dpo_loss`` (mindspeed_mm/tasks/rl/dpo/sora_dpo_trainer.py, posttrain_sora_dpo.py:41).
* ``FlowGRPOTrainer``      -- DanceGRPO for flow-matching generators (SoRA / FLUX): for every prompt a group of samples
  is drawn with stochastic (SDE) Euler steps whose Gaussian log-densities are recorded, a reward callable scores the
  final latents, advantages are normalised inside each group and a clipped policy-gradient step is taken on a
  subset of the recorded timesteps (mindspeed_mm/tasks/rl/soragrpo/{sora_grpo_trainer.py, flux_grpo_trainer.py}).
* ``VLMDPOTrainer``        -- DPO for packed VLM batches: sequence log-probabilities of chosen / rejected responses
  under the policy and a frozen reference (mindspeed_mm/tasks/rl/dpo/qwen2vl_dpo_trainer.py).

The trainers only need ``model(...)`` callables and an ``engine`` with ``set_lr / end_micro_step / finish_step``
(:class:`~mindspeed_mm_b200.parallel.fsdp.FSDPEngine`) or, without an engine, a plain ``torch.optim`` optimizer.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from .preference import (diffusion_dpo_loss, dpo_loss, grpo_advantages, grpo_loss, sde_step_logprob, sequence_logprobs)


class _Stepper:
    """Uniform optimizer-step interface over the sharding engine or a torch optimizer."""

    def __init__(self, engine=None, optimizer: Optional[torch.optim.Optimizer] = None, lr: float = 1e-5):
        if engine is None and optimizer is None:
            raise ValueError("give an engine or an optimizer")
        self.engine, self.optimizer, self.lr = engine, optimizer, lr

    @property
    def run(self):
        return self.engine.run if self.engine is not None else None

    def step(self, loss: torch.Tensor):
        if self.engine is not None:
            self.engine.set_lr(self.lr)
            loss.backward()
            self.engine.end_micro_step()
            return self.engine.finish_step()
        self.optimizer.zero_grad(set_to_none=True)
        loss.backward()
        self.optimizer.step()
        return None


# ------------------------------------------------------------------------------------------ diffusion DPO
class DiffusionDPOTrainer:
    def __init__(self, policy: Callable, reference: Callable, scheduler, beta: float = 5000.0, engine=None, optimizer=None,
                 lr: float = 1e-5, seed: int = 0):
        """``policy(x_t, t, cond) -> velocity`` (trainable), ``reference`` the same signature (frozen)."""
        self.policy, self.reference, self.scheduler, self.beta = policy, reference, scheduler, beta
        self.stepper = _Stepper(engine, optimizer, lr)
        self.gen = torch.Generator().manual_seed(seed)

    def _errors(self, model, x_t, t, cond, target):
        pred = model(x_t, t, cond)
        return (pred.float() - target.float()).pow(2).flatten(1).mean(1)

    def loss(self, latents_w, latents_l, cond) -> torch.Tensor:
        noise = torch.randn(latents_w.shape, generator=self.gen, dtype=torch.float32).to(latents_w.device, latents_w.dtype)
        x_w, _, t = self.scheduler.q_sample(latents_w, noise=noise, generator=self.gen)
        x_l, _, _ = self.scheduler.q_sample(latents_l, noise=noise, t=t)
        tt = t.expand(latents_w.shape[0])
        tgt_w, tgt_l = noise - latents_w, noise - latents_l
        with torch.no_grad():
            ref_w = self._errors(self.reference, x_w, tt, cond, tgt_w)
            ref_l = self._errors(self.reference, x_l, tt, cond, tgt_l)
        pol_w = self._errors(self.policy, x_w, tt, cond, tgt_w)
        pol_l = self._errors(self.policy, x_l, tt, cond, tgt_l)
        return diffusion_dpo_loss(pol_w, pol_l, ref_w, ref_l, self.beta)

    def train_step(self, batch: Dict[str, torch.Tensor]) -> Dict[str, float]:
        loss = self.loss(batch["latents_win"], batch["latents_lose"], batch["prompt"])
        self.stepper.step(loss)
        return {"loss": float(loss.detach())}


# ------------------------------------------------------------------------------------------ flow GRPO
class FlowGRPOTrainer:
    def __init__(self, policy: Callable, scheduler, reward_fn: Callable[[torch.Tensor, object], torch.Tensor], group_size: int = 4,
                 num_steps: int = 8, eta: float = 0.3, clip_range: float = 1e-4, adv_clip_max: float = 5.0,
                 train_timestep_fraction: float = 0.5, engine=None, optimizer=None, lr: float = 1e-5, seed: int = 0):
        """``policy(x, t, cond) -> velocity``; ``reward_fn(final_latents, cond) -> [n]`` scores every sample."""
        self.policy, self.scheduler, self.reward_fn = policy, scheduler, reward_fn
        self.G, self.num_steps, self.eta = group_size, num_steps, eta
        self.clip_range, self.adv_clip_max, self.frac = clip_range, adv_clip_max, train_timestep_fraction
        self.stepper = _Stepper(engine, optimizer, lr)
        self.gen = torch.Generator().manual_seed(seed)

    def _sigmas(self) -> torch.Tensor:
        s = torch.linspace(1.0, 0.0, self.num_steps + 1)
        shift = getattr(self.scheduler, "shift", 1.0)
        return shift * s / (1 + (shift - 1) * s)

    @torch.no_grad()
    def rollout(self, cond, shape, device, dtype):
        """Samples ``G`` trajectories for the prompt.  Returns the visited states, the per-step log-probs and sigmas."""
        sig = self._sigmas()
        x = torch.randn((self.G,) + tuple(shape), generator=self.gen, dtype=torch.float32).to(device, dtype)
        states, nexts, logps = [], [], []
        for i in range(self.num_steps):
            s, s_next = float(sig[i]), float(sig[i + 1])
            t = torch.full((self.G,), s * 1000.0, device=device)
            v = self.policy(x, t, cond)
            dt = s_next - s
            std = self.eta * math.sqrt(max(-dt, 1e-12))
            pred_x0 = x - s * v
            score = -(x - pred_x0 * (1 - s)) / (s ** 2 + 1e-12)
            mean = x + v * dt - 0.5 * (std ** 2) * score
            noise = torch.randn(x.shape, generator=self.gen, dtype=torch.float32).to(device, dtype)
            nxt = mean + (std * noise if i < self.num_steps - 1 else 0.0)
            states.append(x)
            nexts.append(nxt)
            logps.append(sde_step_logprob(nxt, x, v, s, s_next, self.eta))
            x = nxt
        return states, nexts, torch.stack(logps, 1), sig, x

    def train_step(self, cond, shape, device="cpu", dtype=torch.float32) -> Dict[str, float]:
        states, nexts, logp_old, sig, final = self.rollout(cond, shape, device, dtype)
        rewards = self.reward_fn(final, cond).float()
        adv = grpo_advantages(rewards, self.G)
        n_train = max(1, int(round(self.frac * (self.num_steps - 1))))
        picks = torch.randperm(self.num_steps - 1, generator=self.gen)[:n_train].tolist()
        total = 0.0
        loss_acc = None
        for i in picks:
            s, s_next = float(sig[i]), float(sig[i + 1])
            t = torch.full((self.G,), s * 1000.0, device=device)
            v = self.policy(states[i], t, cond)
            logp_new = sde_step_logprob(nexts[i], states[i], v, s, s_next, self.eta)
            l = grpo_loss(logp_new, logp_old[:, i], adv, self.clip_range, self.adv_clip_max) / n_train
            loss_acc = l if loss_acc is None else loss_acc + l
            total += float(l.detach())
        self.stepper.step(loss_acc)
        return {"loss": total, "reward_mean": float(rewards.mean()), "reward_std": float(rewards.std())}


# ------------------------------------------------------------------------------------------ VLM DPO
class VLMDPOTrainer:
    def __init__(self, policy_logits: Callable[[dict], torch.Tensor], reference_logits: Callable[[dict], torch.Tensor],
                 beta: float = 0.1, label_smoothing: float = 0.0, loss_type: str = "sigmoid", engine=None, optimizer=None,
                 lr: float = 1e-6):
        """``*_logits(batch) -> [T, V]`` for a packed batch whose samples alternate chosen, rejected, chosen, ..."""
        self.policy, self.reference = policy_logits, reference_logits
        self.beta, self.ls, self.loss_type = beta, label_smoothing, loss_type
        self.stepper = _Stepper(engine, optimizer, lr)

    @staticmethod
    def _seq_logps(logits, batch):
        labels = batch["labels"]
        lp = torch.log_softmax(logits.float(), -1).gather(1, labels.clamp(min=0)[:, None]).squeeze(1)
        return sequence_logprobs(lp, labels, batch["cu_seqlens"])

    def loss(self, batch: dict):
        with torch.no_grad():
            ref = self._seq_logps(self.reference(batch), batch)
        pol = self._seq_logps(self.policy(batch), batch)
        loss, rc, rr = dpo_loss(pol[0::2], pol[1::2], ref[0::2], ref[1::2], self.beta, self.ls, self.loss_type)
        return loss, (rc > rr).float().mean()

    def train_step(self, batch: dict) -> Dict[str, float]:
        loss, acc = self.loss(batch)
        self.stepper.step(loss)
        return {"loss": float(loss.detach()), "reward_accuracy": float(acc)}
