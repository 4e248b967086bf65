"""Neural audio codec used by the speech LMs: causal convolutional encoder / decoder around a residual vector quantiser.

Covers what the reference's speech tokenizers provide to training and inference
(mindspeed_mm/fsdp/models/qwen3tts/core/tokenizer_12hz/modeling_qwen3_tts_tokenizer_v2.py: strided causal conv encoder,
transformer bottleneck, split residual VQ with one "semantic" codebook followed by acoustic ones, transposed-conv
decoder; tokenizer_25hz/vq/core_vq.py: Euclidean codebooks with EMA updates and dead-code revival):

* ``ResidualVQ``     -- n_q codebooks applied to the running residual; straight-through gradients, commitment loss, optional
  EMA codebook updates (k-means style) with revival of unused codes, ``encode`` / ``decode`` between latents and indices.
* ``SplitResidualVQ``-- first ``n_semantic`` codebooks quantise the signal itself, the remaining ones its residual stream
  separately (the layout of the 12.5 Hz tokenizer).
* ``AudioCodec``     -- waveform [B, 1, samples] -> codes [B, n_q, frames] -> waveform; total stride = prod(ratios).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


class CausalConv1d(nn.Module):
    def __init__(self, cin, cout, k, stride=1, dilation=1):
        super().__init__()
        self.pad = (k - 1) * dilation - (stride - 1)
        self.conv = nn.Conv1d(cin, cout, k, stride=stride, dilation=dilation)

    def forward(self, x):
        return self.conv(F.pad(x, (max(self.pad, 0), 0)))


class CausalConvTranspose1d(nn.Module):
    def __init__(self, cin, cout, k, stride):
        super().__init__()
        self.trim = k - stride
        self.conv = nn.ConvTranspose1d(cin, cout, k, stride=stride)

    def forward(self, x):
        y = self.conv(x)
        return y[..., : y.shape[-1] - self.trim] if self.trim > 0 else y


class ResUnit(nn.Module):
    def __init__(self, c, dilation):
        super().__init__()
        self.c1, self.c2 = CausalConv1d(c, c // 2, 3, dilation=dilation), CausalConv1d(c // 2, c, 1)

    def forward(self, x):
        return x + self.c2(F.elu(self.c1(F.elu(x))))


class VectorQuantize(nn.Module):
    def __init__(self, dim: int, codebook_size: int, codebook_dim: Optional[int] = None, ema_decay: Optional[float] = 0.99,
                 revive_threshold: float = 1.0):
        super().__init__()
        cd = codebook_dim or dim
        self.proj_in = nn.Linear(dim, cd) if cd != dim else nn.Identity()
        self.proj_out = nn.Linear(cd, dim) if cd != dim else nn.Identity()
        self.ema_decay, self.revive_threshold = ema_decay, revive_threshold
        emb = torch.randn(codebook_size, cd) / math.sqrt(cd)
        if ema_decay is None:
            self.codebook = nn.Parameter(emb)
        else:
            self.register_buffer("codebook", emb)
            self.register_buffer("cluster_size", torch.ones(codebook_size))
            self.register_buffer("embed_sum", emb.clone())

    def lookup(self, z):
        """z [N, cd] -> nearest code indices [N]."""
        e = self.codebook.float()
        d = z.float().pow(2).sum(1, keepdim=True) - 2 * z.float() @ e.t() + e.pow(2).sum(1)
        return d.argmin(1)

    @torch.no_grad()
    def _ema_update(self, z, idx):
        K = self.codebook.shape[0]
        onehot = F.one_hot(idx, K).to(z.dtype)
        self.cluster_size.mul_(self.ema_decay).add_(onehot.sum(0), alpha=1 - self.ema_decay)
        self.embed_sum.mul_(self.ema_decay).add_(onehot.t() @ z, alpha=1 - self.ema_decay)
        n = self.cluster_size.sum()
        smoothed = (self.cluster_size + 1e-5) / (n + K * 1e-5) * n
        self.codebook.copy_(self.embed_sum / smoothed[:, None])
        dead = self.cluster_size < self.revive_threshold
        if bool(dead.any()) and z.shape[0] > 0:                 # re-seed unused codes from the current batch
            pick = torch.randint(0, z.shape[0], (int(dead.sum()),), device=z.device)
            self.codebook[dead] = z[pick].to(self.codebook.dtype)
            self.embed_sum[dead] = z[pick].to(self.embed_sum.dtype)
            self.cluster_size[dead] = self.revive_threshold

    def forward(self, x):
        """x [B, D, T] -> (quantised [B, D, T] with straight-through gradient, indices [B, T], commitment loss)."""
        B, D, T = x.shape
        z = self.proj_in(x.transpose(1, 2)).reshape(B * T, -1)
        idx = self.lookup(z)
        q = F.embedding(idx, self.codebook).to(z.dtype)
        if self.training and self.ema_decay is not None:
            self._ema_update(z.detach().float(), idx)
        commit = F.mse_loss(z, q.detach())
        if self.ema_decay is None:
            commit = commit + F.mse_loss(q, z.detach())
        q = z + (q - z).detach()
        return self.proj_out(q).reshape(B, T, D).transpose(1, 2), idx.view(B, T), commit

    def decode(self, idx):
        return self.proj_out(F.embedding(idx, self.codebook)).transpose(1, 2)


class ResidualVQ(nn.Module):
    def __init__(self, n_q: int, dim: int, codebook_size: int, codebook_dim: Optional[int] = None, ema_decay: Optional[float] = 0.99):
        super().__init__()
        self.layers = nn.ModuleList(VectorQuantize(dim, codebook_size, codebook_dim, ema_decay) for _ in range(n_q))

    def forward(self, x, n_q: Optional[int] = None):
        res, out, codes, loss = x, torch.zeros_like(x), [], x.new_zeros(())
        for layer in self.layers[: n_q or len(self.layers)]:
            q, idx, commit = layer(res)
            res = res - q.detach()
            out = out + q
            codes.append(idx)
            loss = loss + commit
        return out, torch.stack(codes, 1), loss / len(codes)

    @torch.no_grad()
    def encode(self, x, n_q: Optional[int] = None):
        was = self.training
        self.eval()
        codes = self.forward(x, n_q)[1]
        self.train(was)
        return codes

    def decode(self, codes):
        return sum(layer.decode(codes[:, i]) for i, layer in enumerate(self.layers[: codes.shape[1]]))


class SplitResidualVQ(nn.Module):
    def __init__(self, n_q: int, dim: int, codebook_size: int, n_semantic: int = 1, codebook_dim: Optional[int] = None,
                 ema_decay: Optional[float] = 0.99):
        super().__init__()
        self.n_semantic = n_semantic
        self.semantic = ResidualVQ(n_semantic, dim, codebook_size, codebook_dim, ema_decay)
        self.acoustic = ResidualVQ(n_q - n_semantic, dim, codebook_size, codebook_dim, ema_decay)

    def forward(self, x):
        qs, cs, ls = self.semantic(x)
        qa, ca, la = self.acoustic(x)
        return qs + qa, torch.cat([cs, ca], 1), (ls + la) / 2

    @torch.no_grad()
    def encode(self, x):
        return torch.cat([self.semantic.encode(x), self.acoustic.encode(x)], 1)

    def decode(self, codes):
        return self.semantic.decode(codes[:, : self.n_semantic]) + self.acoustic.decode(codes[:, self.n_semantic:])


@dataclass
class AudioCodecConfig:
    channels: int = 64
    dim: int = 512
    ratios: Sequence[int] = (8, 6, 5, 4)         # encoder strides; x2 from the frame-rate conv below -> 1920 samples / frame
    frame_stride: int = 2
    n_q: int = 16
    n_semantic: int = 1
    codebook_size: int = 2048
    codebook_dim: int = 256
    transformer_layers: int = 0
    transformer_heads: int = 8
    sample_rate: int = 24000

    @staticmethod
    def tiny(**kw):
        d = dict(channels=8, dim=32, ratios=(4, 2), frame_stride=2, n_q=4, codebook_size=32, codebook_dim=16, transformer_layers=1,
                 transformer_heads=2)
        d.update(kw)
        return AudioCodecConfig(**d)

    @property
    def hop(self) -> int:
        return int(math.prod(self.ratios)) * self.frame_stride


class _CausalTransformer(nn.Module):
    def __init__(self, dim, heads, layers):
        super().__init__()
        self.layers = nn.ModuleList(nn.TransformerEncoderLayer(dim, heads, 4 * dim, dropout=0.0, batch_first=True, norm_first=True)
                                    for _ in range(layers))

    def forward(self, x):                       # [B, D, T]
        h = x.transpose(1, 2)
        mask = torch.triu(torch.ones(h.shape[1], h.shape[1], dtype=torch.bool, device=h.device), 1)
        for l in self.layers:
            h = l(h, src_mask=mask)
        return h.transpose(1, 2)


class AudioCodec(nn.Module):
    def __init__(self, config: Optional[AudioCodecConfig] = None):
        super().__init__()
        self.config = c = config or AudioCodecConfig.tiny()
        enc: List[nn.Module] = [CausalConv1d(1, c.channels, 7)]
        ch = c.channels
        for r in c.ratios:
            enc += [ResUnit(ch, 1), ResUnit(ch, 3), nn.ELU(), CausalConv1d(ch, 2 * ch, 2 * r, stride=r)]
            ch *= 2
        enc += [nn.ELU(), CausalConv1d(ch, c.dim, 3)]
        self.encoder = nn.Sequential(*enc)
        self.enc_transformer = _CausalTransformer(c.dim, c.transformer_heads, c.transformer_layers) if c.transformer_layers else None
        self.downsample = CausalConv1d(c.dim, c.dim, 2 * c.frame_stride, stride=c.frame_stride)
        self.quantizer = SplitResidualVQ(c.n_q, c.dim, c.codebook_size, c.n_semantic, c.codebook_dim)
        self.upsample = CausalConvTranspose1d(c.dim, c.dim, 2 * c.frame_stride, c.frame_stride)
        self.dec_transformer = _CausalTransformer(c.dim, c.transformer_heads, c.transformer_layers) if c.transformer_layers else None
        dec: List[nn.Module] = [CausalConv1d(c.dim, ch, 7)]
        for r in reversed(list(c.ratios)):
            dec += [nn.ELU(), CausalConvTranspose1d(ch, ch // 2, 2 * r, r), ResUnit(ch // 2, 1), ResUnit(ch // 2, 3)]
            ch //= 2
        dec += [nn.ELU(), CausalConv1d(ch, 1, 7)]
        self.decoder = nn.Sequential(*dec)

    def _latent(self, wav):
        pad = (-wav.shape[-1]) % self.config.hop
        h = self.encoder(F.pad(wav, (0, pad)))
        if self.enc_transformer is not None:
            h = self.enc_transformer(h)
        return self.downsample(h)

    def _synth(self, q):
        h = self.upsample(q)
        if self.dec_transformer is not None:
            h = self.dec_transformer(h)
        return self.decoder(h)

    @torch.no_grad()
    def encode(self, wav):
        """wav [B, 1, samples] -> codes [B, n_q, ceil(samples / hop)]."""
        return self.quantizer.encode(self._latent(wav))

    @torch.no_grad()
    def decode(self, codes):
        return self._synth(self.quantizer.decode(codes))

    def forward(self, wav):
        """Training pass: (reconstruction cropped to the input length, codes, commitment loss)."""
        q, codes, commit = self.quantizer(self._latent(wav))
        return self._synth(q)[..., : wav.shape[-1]], codes, commit


def multi_scale_mel_loss(pred, target, sample_rate: int = 24000, ffts: Sequence[int] = (256, 512, 1024), n_mels: int = 40):
    """L1 on log-mel magnitudes at several STFT sizes: the reconstruction term codec training uses next to the
    adversarial ones."""
    loss = pred.new_zeros(())
    for n_fft in ffts:
        win = torch.hann_window(n_fft, device=pred.device)
        fb = _mel_filterbank(n_fft // 2 + 1, n_mels, sample_rate, pred.device)
        mags = []
        for x in (pred, target):
            spec = torch.stft(x.squeeze(1).float(), n_fft, hop_length=n_fft // 4, window=win, return_complex=True).abs()
            mags.append(torch.log((fb @ spec).clamp(min=1e-5)))
        loss = loss + F.l1_loss(mags[0], mags[1])
    return loss / len(ffts)


def _mel_filterbank(n_freq, n_mels, sr, device):
    hz2mel = lambda f: 2595.0 * math.log10(1.0 + f / 700.0)           # noqa: E731
    mel2hz = lambda m: 700.0 * (10 ** (m / 2595.0) - 1.0)             # noqa: E731
    pts = torch.tensor([mel2hz(m) for m in torch.linspace(hz2mel(0.0), hz2mel(sr / 2), n_mels + 2).tolist()], device=device)
    freqs = torch.linspace(0, sr / 2, n_freq, device=device)
    lo, ce, hi = pts[:-2, None], pts[1:-1, None], pts[2:, None]
    return torch.minimum((freqs - lo) / (ce - lo), (hi - freqs) / (hi - ce)).clamp(min=0)
