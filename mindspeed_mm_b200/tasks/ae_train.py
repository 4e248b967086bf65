"""Autoencoder training: reconstruction + KL + (optional) perceptual + adversarial losses and the alternating
generator / discriminator step (mindspeed_mm/models/ae/training/training.py, mindspeed_mm/models/ae/losses/*).

* ``NLayerDiscriminator3D`` -- PatchGAN over (T, H, W): strided 3-D convolutions with LeakyReLU, hinge loss.
* ``VAELoss``               -- L1 (or L2) reconstruction, KL of the diagonal Gaussian posterior, an optional
                               perceptual callable (``models/ae/lpips.py: LPIPS`` with the published weight
                               files, or any ``f(x, y) -> per-sample distance``), and the generator's adversarial term with the adaptive weight
                               ``|grad_rec| / |grad_gan|`` taken at the decoder's last layer.
* ``AETrainer``             -- alternates a generator step and a discriminator step once ``disc_start`` is reached.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


class NLayerDiscriminator3D(nn.Module):
    def __init__(self, in_channels: int = 3, base: int = 64, n_layers: int = 3):
        super().__init__()
        layers = [nn.Conv3d(in_channels, base, 3, stride=(1, 2, 2), padding=1), nn.LeakyReLU(0.2, True)]
        ch = base
        for i in range(1, n_layers):
            nxt = min(base * 2 ** i, base * 8)
            layers += [nn.Conv3d(ch, nxt, 3, stride=(2 if i > 1 else 1, 2, 2), padding=1), nn.GroupNorm(8, nxt),
                       nn.LeakyReLU(0.2, True)]
            ch = nxt
        layers += [nn.Conv3d(ch, 1, 3, padding=1)]
        self.net = nn.Sequential(*layers)

    def forward(self, x):
        return self.net(x)


def hinge_d_loss(logits_real, logits_fake):
    return 0.5 * (F.relu(1.0 - logits_real).mean() + F.relu(1.0 + logits_fake).mean())


def kl_diag_gaussian(mean, logvar):
    return 0.5 * (mean.pow(2) + logvar.exp() - 1.0 - logvar).flatten(1).sum(1)


class VAELoss(nn.Module):
    def __init__(self, kl_weight: float = 1e-6, perceptual: Optional[Callable] = None, perceptual_weight: float = 1.0,
                 disc_weight: float = 0.5, disc_start: int = 0, rec: str = "l1"):
        super().__init__()
        self.kl_weight, self.perceptual, self.pw = kl_weight, perceptual, perceptual_weight
        self.disc_weight, self.disc_start, self.rec = disc_weight, disc_start, rec

    def adaptive_weight(self, nll, g_loss, last_layer):
        gn = torch.autograd.grad(nll, last_layer, retain_graph=True)[0]
        gg = torch.autograd.grad(g_loss, last_layer, retain_graph=True)[0]
        return (gn.norm() / (gg.norm() + 1e-4)).clamp(0.0, 1e4).detach() * self.disc_weight

    def generator(self, x, recon, mean, logvar, step: int, disc: Optional[nn.Module] = None, last_layer=None):
        rec = (x - recon).abs() if self.rec == "l1" else (x - recon).pow(2)
        nll = rec.flatten(1).mean(1)
        if self.perceptual is not None:
            nll = nll + self.pw * self.perceptual(x, recon)
        nll = nll.mean()
        kl = kl_diag_gaussian(mean, logvar).mean()
        loss = nll + self.kl_weight * kl
        logs = {"rec": float(nll.detach()), "kl": float(kl.detach())}
        if disc is not None and step >= self.disc_start:
            g_loss = -disc(recon).mean()
            w = self.adaptive_weight(nll, g_loss, last_layer) if last_layer is not None else self.disc_weight
            loss = loss + w * g_loss
            logs.update(g_loss=float(g_loss.detach()), d_weight=float(w))
        return loss, logs

    def discriminator(self, x, recon, disc: nn.Module):
        return hinge_d_loss(disc(x.detach()), disc(recon.detach()))


class AETrainer:
    def __init__(self, vae, loss: VAELoss, disc: Optional[nn.Module] = None, lr: float = 1e-4, disc_lr: float = 1e-4,
                 ema_decay: float = 0.0):
        """``ema_decay`` > 0 keeps a moving average of the autoencoder weights (the reference's ``--ema --ema_decay``),
        updated after every generator step; ``self.ema.apply_shadow() / restore()`` brackets an evaluation."""
        from ..runtime.ema import ModuleEMA
        self.vae, self.loss, self.disc = vae, loss, disc
        self.ema = ModuleEMA(vae, ema_decay) if ema_decay > 0 else None
        self.opt = torch.optim.AdamW(vae.parameters(), lr=lr, betas=(0.9, 0.95))
        self.opt_d = torch.optim.AdamW(disc.parameters(), lr=disc_lr, betas=(0.9, 0.95)) if disc is not None else None
        self.step = 0

    def _forward(self, video):
        moments = self.vae.quant_conv(self.vae.encoder(video))
        mean, logvar = moments.chunk(2, dim=1)
        logvar = logvar.clamp(-30.0, 20.0)
        z = mean + torch.exp(0.5 * logvar) * torch.randn_like(mean)
        recon = self.vae.decoder(self.vae.post_quant_conv(z))
        return recon, mean, logvar

    def train_step(self, video: torch.Tensor) -> Dict[str, float]:
        recon, mean, logvar = self._forward(video)
        last = self.vae.decoder.conv_out.weight
        g, logs = self.loss.generator(video, recon, mean, logvar, self.step, self.disc, last)
        self.opt.zero_grad(set_to_none=True)
        g.backward()
        self.opt.step()
        if self.ema is not None:
            self.ema.update()
        if self.disc is not None and self.step >= self.loss.disc_start:
            d = self.loss.discriminator(video, recon, self.disc)
            self.opt_d.zero_grad(set_to_none=True)
            d.backward()
            self.opt_d.step()
            logs["d_loss"] = float(d.detach())
        self.step += 1
        logs["loss"] = float(g.detach())
        return logs
