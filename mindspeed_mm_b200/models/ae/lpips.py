"""Learned perceptual image patch similarity (LPIPS, VGG-16 variant) as the perceptual term of autoencoder training.

Reference: mindspeed_mm/models/ae/losses/lpips.py:8-99 (VGG-16 feature taps after relu1_2 / 2_2 / 3_3 / 4_3 / 5_3,
unit-normalised over channels, squared difference weighted by one learned non-negative 1 x 1 convolution per tap, averaged
over space and summed over taps).  Pretrained weights are not bundled.  ``load_pretrained`` reads the two public files:
the LPIPS linear heads (``lin{i}.model.1.weight``) and a torchvision VGG-16 state dict (``features.{n}.weight``), or one
file that already holds this module's own keys (``net.slice{k}.{n}.*`` + ``lin{i}.model.1.weight``, the layout the
reference saves).  Parameters are frozen: the module only scores.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

# torchvision VGG-16 ``features`` indices of the convolutions in each tap's slice (ReLU after each, max-pool between)
_SLICES = ((0, 2), (5, 7), (10, 12, 14), (17, 19, 21), (24, 26, 28))
_CHANNELS = (64, 128, 256, 512, 512)


class _VGG16Taps(nn.Module):
    def __init__(self):
        super().__init__()
        cin = 3
        for k, (idxs, cout) in enumerate(zip(_SLICES, _CHANNELS), 1):
            layers: Dict[str, nn.Module] = {}
            if k > 1:
                layers[str(idxs[0] - 1)] = nn.MaxPool2d(2, 2)
            for i in idxs:
                layers[str(i)] = nn.Conv2d(cin, cout, 3, padding=1)
                layers[str(i + 1)] = nn.ReLU(inplace=False)
                cin = cout
            seq = nn.Sequential()
            for name, m in layers.items():
                seq.add_module(name, m)
            setattr(self, f"slice{k}", seq)

    def forward(self, x):
        outs = []
        for k in range(1, 6):
            x = getattr(self, f"slice{k}")(x)
            outs.append(x)
        return outs


class _Lin(nn.Module):
    def __init__(self, cin: int, dropout: bool):
        super().__init__()
        self.model = nn.Sequential(nn.Dropout() if dropout else nn.Identity(), nn.Conv2d(cin, 1, 1, bias=False))


class LPIPS(nn.Module):
    """``forward(x, y) -> [B]`` distance of images in [-1, 1] (``[B, 3, H, W]``, or video ``[B, 3, T, H, W]``: frames
    are scored one by one and averaged)."""

    def __init__(self, pretrained: Optional[str] = None, vgg_pretrained: Optional[str] = None, use_dropout: bool = True):
        super().__init__()
        self.register_buffer("shift", torch.tensor([-.030, -.088, -.188]).view(1, 3, 1, 1))
        self.register_buffer("scale", torch.tensor([.458, .448, .450]).view(1, 3, 1, 1))
        self.net = _VGG16Taps()
        for i, c in enumerate(_CHANNELS):
            setattr(self, f"lin{i}", _Lin(c, use_dropout))
        if pretrained or vgg_pretrained:
            self.load_pretrained(pretrained, vgg_pretrained)
        self.eval()
        for p in self.parameters():
            p.requires_grad_(False)

    def load_pretrained(self, lpips_path: Optional[str], vgg_path: Optional[str] = None) -> None:
        sd: Dict[str, torch.Tensor] = {}
        if vgg_path:
            vgg = torch.load(vgg_path, map_location="cpu", weights_only=True)
            where = {i: k for k, idxs in enumerate(_SLICES, 1) for i in idxs}
            for name, t in vgg.items():
                parts = name.split(".")
                if parts[0] == "features" and int(parts[1]) in where:
                    sd[f"net.slice{where[int(parts[1])]}.{parts[1]}.{parts[2]}"] = t
        if lpips_path:
            sd.update(torch.load(lpips_path, map_location="cpu", weights_only=True))
        missing, unexpected = self.load_state_dict(sd, strict=False)
        bad = [k for k in unexpected if not k.startswith(("scaling_layer.",))]
        if bad:
            raise KeyError(f"unexpected keys in the perceptual checkpoint: {bad[:6]}")
        lin_missing = [k for k in missing if k.startswith("lin")]
        if lpips_path and lin_missing:
            raise KeyError(f"the perceptual checkpoint lacks {lin_missing}")

    def train(self, mode: bool = True):          # scoring only: dropout stays off whatever the caller's mode
        return super().train(False)

    def forward(self, x, y):
        if x.dim() == 5:
            B, C, T, H, W = x.shape
            fold = lambda t: t.permute(0, 2, 1, 3, 4).reshape(B * T, C, H, W)
            return self.forward(fold(x), fold(y)).view(B, T).mean(1)
        fx = self.net((x - self.shift) / self.scale)
        fy = self.net((y - self.shift) / self.scale)
        total = 0.0
        for i, (a, b) in enumerate(zip(fx, fy)):
            a = a / (a.pow(2).sum(1, keepdim=True).sqrt() + 1e-10)
            b = b / (b.pow(2).sum(1, keepdim=True).sqrt() + 1e-10)
            total = total + getattr(self, f"lin{i}").model((a - b) ** 2).mean((1, 2, 3))
        return total
