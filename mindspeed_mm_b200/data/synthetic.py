"""Synthetic datasets of the benchmark shapes (no network, no files).

The reference ships a mock-data generator for VLMs
(mindspeed_mm/fsdp/tools/data_tool/generate_mock_data_for_vlmodel.py) that writes images and a
JSON to disk; here the samples are produced in memory, already in the form the collators emit:
token ids with image placeholders, CLIP-normalised patches flattened the way the HF image
processor does it, labels with the image tokens masked, and the (t, h, w) grid per image.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
from torch.utils.data import Dataset

from ..models.registry import data_register

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def patchify_image(img: torch.Tensor, patch: int = 14, temporal: int = 2, merge: int = 2) -> torch.Tensor:
    """[3, H, W] in [0,1] -> [H/p * W/p, 3*temporal*p*p] patches in 2x2-merge order (HF Qwen2-VL layout)."""
    C, H, W = img.shape
    mean = torch.tensor(CLIP_MEAN).view(3, 1, 1)
    std = torch.tensor(CLIP_STD).view(3, 1, 1)
    x = ((img - mean) / std).unsqueeze(0).repeat(temporal, 1, 1, 1)          # [tp, C, H, W]
    gh, gw = H // patch, W // patch
    x = x.view(1, temporal, C, gh // merge, merge, patch, gw // merge, merge, patch)
    x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)                                  # gt, gh/m, gw/m, m, m, C, tp, p, p
    return x.reshape(gh * gw, C * temporal * patch * patch)


@dataclass
class SyntheticVLMSpec:
    seq_len: int = 1024             # tokens per sample (text + image placeholders)
    images_per_sample: int = 2
    image_size: int = 224
    vocab_size: int = 32000
    image_token_id: int = 31999
    vision_start_token_id: int = 31997
    patch: int = 14
    temporal_patch: int = 2
    merge: int = 2
    num_samples: int = 1 << 30
    seed: int = 0
    pixel_dtype: torch.dtype = torch.float32


@data_register.register("synthetic_vlm")
class SyntheticVLMDataset(Dataset):
    """Deterministic random VLM samples: item i depends only on (seed, i)."""

    def __init__(self, spec: SyntheticVLMSpec):
        self.spec = spec
        g = spec.image_size // spec.patch
        self.grid = (1, g, g)
        self.vis_tokens = g * g // (spec.merge ** 2)
        need = spec.images_per_sample * (self.vis_tokens + 1)
        if need >= spec.seq_len:
            raise ValueError(f"seq_len {spec.seq_len} cannot hold {spec.images_per_sample} images ({need} tokens)")

    def __len__(self):
        return self.spec.num_samples

    def __getitem__(self, i: int) -> Dict[str, torch.Tensor]:
        s = self.spec
        g = torch.Generator().manual_seed(s.seed * 1_000_003 + i)
        n_text = s.seq_len - s.images_per_sample * (self.vis_tokens + 1)
        # reserve the special ids at the top of the vocabulary for the placeholders
        text = torch.randint(0, min(s.vocab_size, s.vision_start_token_id) - 1, (n_text,), generator=g)
        cuts = sorted(torch.randint(0, n_text + 1, (s.images_per_sample,), generator=g).tolist())
        pieces, prev = [], 0
        img_block = torch.cat([torch.tensor([s.vision_start_token_id]),
                               torch.full((self.vis_tokens,), s.image_token_id)])
        for c in cuts:
            pieces += [text[prev:c], img_block]
            prev = c
        pieces.append(text[prev:])
        ids = torch.cat(pieces)
        labels = ids.clone()
        labels[(ids == s.image_token_id) | (ids == s.vision_start_token_id)] = -100
        imgs = torch.rand(s.images_per_sample, 3, s.image_size, s.image_size, generator=g)
        if s.images_per_sample:
            pix = torch.cat([patchify_image(im, s.patch, s.temporal_patch, s.merge) for im in imgs]).to(s.pixel_dtype)
        else:
            pix = torch.zeros(0, 3 * s.temporal_patch * s.patch * s.patch, dtype=s.pixel_dtype)
        grid = torch.tensor([self.grid] * s.images_per_sample, dtype=torch.long).view(-1, 3)
        return dict(input_ids=ids, labels=labels, pixel_values=pix, image_grid_thw=grid)


@dataclass
class SyntheticVideoLatentSpec:
    """Pre-extracted features for DiT training (the reference's ``load_video_features`` mode,
    mindspeed_mm/data/datasets/feature_dataset.py:29)."""
    channels: int = 16
    frames: int = 21
    height: int = 90
    width: int = 160
    text_len: int = 512
    text_dim: int = 4096
    num_samples: int = 1 << 30
    seed: int = 0
    dtype: torch.dtype = torch.float32
    pooled_dim: int = 0          # > 0: also emit ``added_cond`` = pooled prompt embedding + six size / crop numbers (SDXL)


@data_register.register("synthetic_video_latents")
class SyntheticVideoLatentDataset(Dataset):
    def __init__(self, spec: SyntheticVideoLatentSpec):
        self.spec = spec

    def __len__(self):
        return self.spec.num_samples

    def __getitem__(self, i):
        s = self.spec
        g = torch.Generator().manual_seed(s.seed * 1_000_003 + i)
        out = dict(
            latents=torch.randn(s.channels, s.frames, s.height, s.width, generator=g).to(s.dtype),
            prompt=torch.randn(s.text_len, s.text_dim, generator=g).to(s.dtype),
            prompt_mask=torch.ones(s.text_len, dtype=torch.bool))
        if s.pooled_dim:
            px = (8.0 * s.height, 8.0 * s.width)
            out["added_cond"] = torch.cat([torch.randn(s.pooled_dim, generator=g),
                                           torch.tensor([*px, 0.0, 0.0, *px])]).to(s.dtype)
        return out


# ------------------------------------------------------------------------------------------------- speech
@dataclass
class SyntheticSpeechSpec:
    """Utterances for the speech-token LMs: a text id list, a codec frame matrix and a reference mel clip."""
    num_samples: int = 64
    text_len: int = 12
    frames: int = 20
    n_codebooks: int = 4
    text_vocab: int = 100
    audio_vocab: int = 32
    n_mels: int = 20
    ref_frames: int = 30
    seed: int = 0


@data_register.register("synthetic_speech")
class SyntheticSpeechDataset(Dataset):
    def __init__(self, spec: SyntheticSpeechSpec):
        self.spec = spec

    def __len__(self):
        return self.spec.num_samples

    def __getitem__(self, i):
        s = self.spec
        g = torch.Generator().manual_seed(s.seed * 1_000_003 + i)
        n_text = int(torch.randint(max(2, s.text_len // 2), s.text_len + 1, (1,), generator=g))
        n_frames = int(torch.randint(max(2, s.frames // 2), s.frames + 1, (1,), generator=g))
        return dict(text=torch.randint(1, s.text_vocab, (n_text,), generator=g),
                    codes=torch.randint(0, s.audio_vocab, (n_frames, s.n_codebooks), generator=g),
                    ref_mel=torch.randn(s.ref_frames, s.n_mels, generator=g))


# ------------------------------------------------------------------------------------------------- speech recognition
def audio_token_count(frames: int, n_window: int) -> int:
    """Embeddings the windowed audio tower (``models/encoders.py: WindowedAudioEncoder``) returns for a clip of ``frames``
    mel frames: windows of ``2 * n_window`` frames, a stride-2 convolution per window, then pairs averaged."""
    win = 2 * n_window
    total = sum((min(win, frames - s) + 1) // 2 for s in range(0, frames, win))
    return 1 if total == 1 else total // 2


@dataclass
class SyntheticASRSpec:
    """Speech-recognition samples for the audio-conditioned decoders (FunASR, Qwen3-ASR, the omni models): a mel clip,
    its placeholder tokens, then the transcript, which is the only supervised span."""
    num_samples: int = 64
    frames: int = 120                 # longest clip (mel frames); clips are drawn from [frames / 2, frames]
    text_len: int = 24
    n_mels: int = 16
    n_window: int = 20
    vocab_size: int = 1000
    audio_token_id: int = 999
    seed: int = 0


@data_register.register("synthetic_asr")
class SyntheticASRDataset(Dataset):
    def __init__(self, spec: SyntheticASRSpec):
        self.spec = spec

    def __len__(self):
        return self.spec.num_samples

    def __getitem__(self, i):
        s = self.spec
        g = torch.Generator().manual_seed(s.seed * 1_000_003 + i)
        frames = int(torch.randint(max(8, s.frames // 2), s.frames + 1, (1,), generator=g))
        n_text = int(torch.randint(max(2, s.text_len // 2), s.text_len + 1, (1,), generator=g))
        n_audio = audio_token_count(frames, s.n_window)
        text = torch.randint(0, min(s.vocab_size, s.audio_token_id) - 1, (n_text,), generator=g)
        ids = torch.cat([torch.full((n_audio,), s.audio_token_id), text])
        labels = ids.clone()
        labels[:n_audio] = -100
        return dict(input_ids=ids, labels=labels, audio_features=torch.randn(s.n_mels, frames, generator=g))


class ASRPackCollator:
    """Packs speech-recognition samples: next-token labels inside each sample, 1-D positions, ``cu_seqlens``, the list of
    mel clips in sample order."""

    def __init__(self, ignore_index: int = -100):
        self.ignore_index = ignore_index

    def __call__(self, samples):
        ids, labels, pos, lens, mels = [], [], [], [], []
        for s in samples:
            i, l = s["input_ids"], s["labels"]
            ids.append(i)
            labels.append(torch.cat([l[1:], l.new_full((1,), self.ignore_index)]))
            pos.append(torch.arange(len(i)))
            lens.append(len(i))
            mels.append(s["audio_features"])
        input_ids = torch.cat(ids)
        cu = torch.tensor([0] + lens).cumsum(0).to(torch.int32)
        return dict(input_ids=input_ids, labels=torch.cat(labels), position_ids=torch.cat(pos), cu_seqlens=cu,
                    max_seqlen=max(lens), audio_features=mels, n_tokens=int(input_ids.numel()))


# ------------------------------------------------------------------------------------------------- audio + video latents
@dataclass
class SyntheticAVLatentSpec:
    """Pre-encoded joint audio-video samples in the layout of the LTX-2 trainer: patchified video latents with (t, h, w)
    positions, audio latents with time positions, text features, flow-matching targets at one sigma per sample."""
    num_samples: int = 32
    grid: Sequence[int] = (3, 4, 4)
    video_channels: int = 8
    audio_tokens: int = 6
    audio_channels: int = 6
    text_len: int = 7
    text_dim: int = 24
    first_frame_clean: bool = True
    seed: int = 0


@data_register.register("synthetic_av_latents")
class SyntheticAVLatentDataset(Dataset):
    def __init__(self, spec: SyntheticAVLatentSpec):
        self.spec = spec

    def __len__(self):
        return self.spec.num_samples

    def __getitem__(self, i):
        s = self.spec
        g = torch.Generator().manual_seed(s.seed * 1_000_003 + i)
        t, h, w = s.grid
        n = t * h * w
        idx = torch.arange(n)
        pos = torch.stack([idx // (h * w), (idx // w) % h, idx % w]).float()
        clean, noise = torch.randn(n, s.video_channels, generator=g), torch.randn(n, s.video_channels, generator=g)
        sigma = float(torch.rand(1, generator=g))
        sig = torch.full((n,), sigma)
        mask = torch.ones(n, dtype=torch.bool)
        if s.first_frame_clean:
            sig[: h * w] = 0.0
            mask[: h * w] = False
        a_clean, a_noise = torch.randn(s.audio_tokens, s.audio_channels, generator=g), torch.randn(s.audio_tokens, s.audio_channels, generator=g)
        return dict(video_latent=(1 - sig[:, None]) * clean + sig[:, None] * noise, video_timesteps=sig * 1000.0, video_positions=pos,
                    video_target_velocity=noise - clean, loss_mask=mask,
                    audio_latent=(1 - sigma) * a_clean + sigma * a_noise, audio_timesteps=torch.full((s.audio_tokens,), sigma * 1000.0),
                    audio_positions=torch.arange(s.audio_tokens).float()[None] * (t / max(s.audio_tokens, 1)),
                    audio_target_velocity=a_noise - a_clean,
                    context=torch.randn(s.text_len, s.text_dim, generator=g), context_mask=torch.ones(s.text_len, dtype=torch.bool))
