"""Speech-token language models (TTS): multi-codebook delay LM, CosyVoice3 LM, Qwen3-TTS talker + code predictor.

All three put extra embedding tables and output heads around a decoder stack; the stack is a
:class:`~mindspeed_mm_b200.models.composable.ComposableLM` fed with ``inputs_embeds`` so that they train through the
same packed-sequence kernels, ZeRO-3 units and checkpoint paths as the VLMs.

* ``MultiCodebookLM``  -- MOSS-TTS "delay" model (mindspeed_mm/fsdp/models/moss_tts_delay/modeling_moss_tts.py:159): token
  = (text id, n_vq audio codes); embeddings are summed, one head per channel, channel-weighted loss; audio codebooks
  are shifted against each other by the delay pattern (processing_moss_tts.py).
* ``CosyVoice3LM``     -- mindspeed_mm/fsdp/models/cosyvoice3/llm.py:64: [sos, instruct, text, task_id, speech...] sequences
  (or the interleaved "bistream" form with ``mix_ratio`` text : speech tokens), label-smoothed loss, repetition-aware
  sampling.
* ``Qwen3TTSTalker``   -- mindspeed_mm/fsdp/models/qwen3tts/core/models/modeling_qwen3_tts.py:1585,1845: the talker predicts
  codebook 0 of every frame from summed text + codec embeddings (with a speaker-embedding slot); a small "code
  predictor" decoder, run once per frame on [talker hidden, code 0, ..., code G-2], predicts codebooks 1..G-1; loss =
  talker CE + 0.3 * predictor CE.  ``SpeakerEncoder`` is the ECAPA-TDNN of :340.
"""
from __future__ import annotations

import math
import random
from dataclasses import dataclass, field, replace
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .composable import ComposableConfig, ComposableLM, DecoderConfig
from .qwen2_5_vl import Embedding
from .registry import model_register

IGNORE = -100


def _text_lm(text: DecoderConfig) -> ComposableLM:
    return ComposableLM(ComposableConfig(replace(text, rope="rope1d"), None))


def _ce_mean(h, weight, labels):
    """Mean token cross entropy of ``h @ weight.T`` without materialising the logits."""
    total, n = ops.linear_cross_entropy(h, weight, labels)
    return total / n.clamp(min=1).to(total.dtype)


def _positions(cu: torch.Tensor, total: int, device) -> torch.Tensor:
    """position ids [total] restarting at every sequence start of ``cu``."""
    starts = torch.zeros(total, dtype=torch.long, device=device)
    lens = (cu[1:] - cu[:-1]).long()
    starts = torch.repeat_interleave(cu[:-1].long(), lens)
    return torch.arange(total, device=device) - starts


class _Wrapped(nn.Module):
    """Common plumbing: ``self.backbone`` + extra tables / heads, exposed to the sharding engine as units."""

    backbone: ComposableLM

    def _extra_units(self) -> List[Tuple[str, nn.Module]]:
        return []

    def fsdp_units(self):
        return self._extra_units() + [(f"backbone.{n}", m) for n, m in self.backbone.fsdp_units()]

    def hidden(self, embeds, batch: dict, run=None):
        b = {k: v for k, v in batch.items() if k not in ("labels", "input_ids")}
        b.update(inputs_embeds=embeds, return_hidden=True)
        if "position_ids" not in b:
            b["position_ids"] = _positions(b["cu_seqlens"], embeds.shape[0], embeds.device)
        return self.backbone(b, run)

    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: float = 0.02):
        self.backbone.init_weights(seed)
        g = torch.Generator().manual_seed(seed + 1)
        for n, p in self.named_parameters():
            if not n.startswith("backbone.") and p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g) * std)


# ------------------------------------------------------------------------------------------------- delay pattern
def apply_delay_pattern(codes: torch.Tensor, pad: int) -> torch.Tensor:
    """``codes`` [T, n_vq] -> [T + n_vq - 1, n_vq]: codebook k is shifted k steps later, holes filled with ``pad``."""
    T, n = codes.shape
    out = codes.new_full((T + n - 1, n), pad)
    for k in range(n):
        out[k:k + T, k] = codes[:, k]
    return out


def revert_delay_pattern(delayed: torch.Tensor) -> torch.Tensor:
    L, n = delayed.shape
    T = L - n + 1
    return torch.stack([delayed[k:k + T, k] for k in range(n)], 1)


@dataclass
class MultiCodebookConfig:
    text: DecoderConfig = field(default_factory=DecoderConfig)
    n_vq: int = 8
    audio_vocab_size: int = 1024
    channel_loss_weight: Optional[Sequence[float]] = None

    @staticmethod
    def tiny(**kw):
        from .composable import _tiny_text
        return MultiCodebookConfig(text=_tiny_text(rope="rope1d"), n_vq=3, audio_vocab_size=32, **kw)


@model_register.register("moss_tts_delay")
class MultiCodebookLM(_Wrapped):
    """``batch``: ``input_ids`` [T, 1 + n_vq], ``labels`` [T, 1 + n_vq] (already shifted, -100 ignored), ``cu_seqlens``,
    ``max_seqlen``.  Returns the weighted loss, or the list of per-channel logits when there are no labels."""
    config_class = MultiCodebookConfig

    def __init__(self, config: Optional[MultiCodebookConfig] = None):
        super().__init__()
        self.config = c = config or MultiCodebookConfig.tiny()
        self.backbone = _text_lm(c.text)
        H = c.text.hidden_size
        self.emb_ext = nn.ModuleList(Embedding(c.audio_vocab_size + 1, H) for _ in range(c.n_vq))
        self.audio_heads = nn.ParameterList(nn.Parameter(torch.empty(c.audio_vocab_size + 1, H)) for _ in range(c.n_vq))

    def _extra_units(self):
        return [("emb_ext", self.emb_ext), ("audio_heads", self.audio_heads)]

    def embed(self, ids, run=None):
        run = run or (lambda m, *a, **k: m(*a, **k))
        x = run(self.backbone.embed_tokens, ids[:, 0])
        for k, emb in enumerate(self.emb_ext):
            x = x + emb(ids[:, k + 1])
        return x

    def forward(self, batch: dict, run=None):
        c = self.config
        ids = batch["input_ids"]
        if ids.dim() != 2 or ids.shape[1] != c.n_vq + 1:
            raise ValueError("input_ids must be [tokens, 1 + n_vq]")
        h = self.hidden(self.embed(ids, run), batch, run)
        h = self.backbone.lm_head.norm(h)
        # the last index of every audio table is an input-only padding code: it is never predicted
        weights = [self.backbone.lm_head.weight] + [w[:-1] for w in self.audio_heads]
        labels = batch.get("labels")
        if labels is None:
            return [ops.linear(h, w) for w in weights]
        cw = list(c.channel_loss_weight or [1.0] * len(weights))
        total, parts = h.new_zeros((), dtype=torch.float32), []
        for k, w in enumerate(weights):
            lab = labels[:, k]
            if bool((lab != IGNORE).any()):
                lk = _ce_mean(h, w, lab)
                parts.append(lk.detach())
                total = total + cw[k] * lk
            else:
                parts.append(h.new_zeros((), dtype=torch.float32))
        self.last_channel_losses = torch.stack(parts)
        return total / sum(cw)

    def collate(self, samples: Sequence[dict], audio_slot: int = 0) -> dict:
        """Utterances (``text`` ids, ``codes`` [frames, >= n_vq]) -> one packed batch: text rows carry the text id and padding
        codes, audio rows carry ``audio_slot`` in the text channel and the delayed codes; labels are the inputs shifted
        by one row inside each utterance (padding codes are not predicted)."""
        c = self.config
        pad = c.audio_vocab_size
        rows, labels, cu = [], [], [0]
        for smp in samples:
            text, codes = smp["text"].long(), smp["codes"][:, : c.n_vq].long()
            delayed = apply_delay_pattern(codes, pad)
            t_rows = torch.cat([text[:, None], torch.full((text.numel(), c.n_vq), pad)], 1)
            a_rows = torch.cat([torch.full((delayed.shape[0], 1), audio_slot), delayed], 1)
            seq = torch.cat([t_rows, a_rows])
            lab = torch.cat([seq[1:], torch.full((1, c.n_vq + 1), IGNORE)])
            lab[:, 1:][lab[:, 1:] == pad] = IGNORE
            lab[: text.numel() - 1, 1:] = IGNORE
            lab[text.numel() - 1:, 0] = IGNORE               # inside the audio span only the code channels are trained
            rows.append(seq)
            labels.append(lab)
            cu.append(cu[-1] + seq.shape[0])
        lens = [b - a for a, b in zip(cu[:-1], cu[1:])]
        return dict(input_ids=torch.cat(rows), labels=torch.cat(labels), cu_seqlens=torch.tensor(cu, dtype=torch.int32),
                    max_seqlen=max(lens))

    @torch.no_grad()
    def generate_codes(self, prompt_ids: torch.Tensor, steps: int, pad_code: Optional[int] = None, temperature: float = 0.0,
                       generator=None) -> torch.Tensor:
        """Greedy / sampled continuation of the audio channels in delay layout; returns un-delayed codes [steps, n_vq].
        The text channel of generated positions holds ``prompt_ids[-1, 0]`` (the audio-slot token)."""
        c = self.config
        pad = c.audio_vocab_size if pad_code is None else pad_code
        seq = prompt_ids.clone()
        slot = int(prompt_ids[-1, 0])
        total = steps + c.n_vq - 1
        for s in range(total):
            T = seq.shape[0]
            b = dict(input_ids=seq, cu_seqlens=torch.tensor([0, T], dtype=torch.int32, device=seq.device), max_seqlen=T)
            logits = self.forward(b)
            nxt = [slot]
            for k in range(c.n_vq):
                if s < k or s - k >= steps:
                    nxt.append(pad)
                    continue
                lg = logits[k + 1][-1].float()
                if temperature > 0:
                    nxt.append(int(torch.multinomial(F.softmax(lg / temperature, -1).cpu(), 1, generator=generator)))
                else:
                    nxt.append(int(lg.argmax()))
            seq = torch.cat([seq, torch.tensor([nxt], device=seq.device, dtype=seq.dtype)], 0)
        return revert_delay_pattern(seq[prompt_ids.shape[0]:, 1:])


# ------------------------------------------------------------------------------------------------- CosyVoice3
def label_smoothing_loss(logits: torch.Tensor, target: torch.Tensor, smoothing: float = 0.0, normalize_length: bool = False,
                         batch_size: int = 1) -> torch.Tensor:
    """KL to the smoothed one-hot distribution, summed over non-ignored tokens and divided by the token count
    (``normalize_length``) or by the batch size (cosyvoice3/llm.py:415)."""
    keep = target != IGNORE
    logp = F.log_softmax(logits.float()[keep], -1)
    tgt = target[keep]
    V = logits.shape[-1]
    true = torch.full_like(logp, smoothing / max(V - 1, 1))
    true.scatter_(1, tgt[:, None], 1.0 - smoothing)
    kl = (true * (torch.log(true.clamp(min=1e-20)) - logp)).sum()
    return kl / (int(keep.sum()) if normalize_length else batch_size)


def ras_sampling(scores: torch.Tensor, decoded: Sequence[int], top_p: float = 0.8, top_k: int = 25, win_size: int = 10,
                 tau_r: float = 0.1, generator=None) -> int:
    """Repetition-aware sampling: nucleus (top-p within top-k) draw; if the drawn token already fills more than
    ``tau_r`` of the last ``win_size`` tokens, redraw from the full distribution."""
    prob = F.softmax(scores.float(), -1).cpu()
    sp, si = prob.sort(descending=True)
    cum = torch.cumsum(sp, 0)
    n = int(min(top_k, max(1, int((cum < top_p).sum()) + 1)))
    pick = int(si[:n][torch.multinomial(sp[:n], 1, generator=generator)])
    recent = list(decoded[-win_size:])
    if recent and recent.count(pick) >= win_size * tau_r:
        pick = int(torch.multinomial(prob, 1, generator=generator))
    return pick


@dataclass
class CosyVoice3Config:
    text: DecoderConfig = field(default_factory=DecoderConfig)
    speech_token_size: int = 6561
    lsm_weight: float = 0.0
    length_normalized_loss: bool = True
    mix_ratio: Tuple[int, int] = (5, 15)
    bistream_prob: float = 0.5

    @staticmethod
    def tiny(**kw):
        from .composable import _tiny_text
        d = dict(text=_tiny_text(rope="rope1d"), speech_token_size=40, mix_ratio=(2, 6))
        d.update(kw)
        return CosyVoice3Config(**d)


@model_register.register("cosyvoice3")
class CosyVoice3LM(_Wrapped):
    """Special speech ids: ``sos = S``, ``eos = S + 1``, ``task_id = S + 2``, ``fill = S + 3`` (S = speech_token_size); the speech
    table and the output head have S + 200 rows, every id >= S stops generation."""
    config_class = CosyVoice3Config

    def __init__(self, config: Optional[CosyVoice3Config] = None):
        super().__init__()
        self.config = c = config or CosyVoice3Config.tiny()
        self.backbone = _text_lm(c.text)
        S, H = c.speech_token_size, c.text.hidden_size
        self.sos, self.eos, self.task_id, self.fill = S, S + 1, S + 2, S + 3
        self.speech_embedding = Embedding(S + 200, H)
        self.llm_decoder = Embedding(S + 200, H)       # output table (rows = speech ids incl. the special ones)
        self.rng = random.Random(0)

    def _extra_units(self):
        return [("speech_embedding", self.speech_embedding), ("llm_decoder", self.llm_decoder)]

    # ------------------------------------------------------------------ sequence building
    def build_sample(self, text: Sequence[int], speech: Sequence[int], instruct: Sequence[int] = (), bistream: bool = False):
        """Returns ``(kinds, ids, targets)``: ``kinds[i]`` is "t" (text table) or "s" (speech table) for input ``ids[i]``;
        ``targets[i]`` is what position i must predict (-100 = nothing)."""
        r_t, r_s = self.config.mix_ratio
        text, speech, instruct = list(text), list(speech), list(instruct)
        kinds, ids, tgt = ["s"], [self.sos], [IGNORE]
        kinds += ["t"] * len(instruct)
        ids += instruct
        tgt += [IGNORE] * len(instruct)
        if bistream and len(speech) / max(len(text), 1) > r_s / r_t:
            n_blocks = math.ceil((len(text) + 1) / r_t)
            for j in range(n_blocks):
                tt, ss = text[j * r_t:(j + 1) * r_t], speech[j * r_s:(j + 1) * r_s]
                if len(tt) == r_t:
                    # a full text block: its last token starts predicting the speech block, which ends with "fill"
                    kinds += ["t"] * r_t + ["s"] * len(ss)
                    ids += tt + ss
                    tgt += [IGNORE] * (r_t - 1) + ss + [self.fill]
                else:
                    rest = speech[j * r_s:]
                    kinds += ["t"] * len(tt) + ["s"] + ["s"] * len(rest)
                    ids += tt + [self.task_id] + rest
                    tgt += [IGNORE] * len(tt) + rest + [self.eos]
                    break
        else:
            kinds += ["t"] * len(text) + ["s"] + ["s"] * len(speech)
            ids += text + [self.task_id] + speech
            tgt += [IGNORE] * len(text) + speech + [self.eos]
        assert len(kinds) == len(ids) == len(tgt)
        return kinds, ids, tgt

    def pack(self, samples: Sequence[dict], device="cpu") -> dict:
        """``samples``: dicts with ``text``, ``speech`` and optional ``instruct`` id lists -> one packed batch."""
        kinds, ids, tgt, cu = [], [], [], [0]
        for s in samples:
            bi = self.training and self.rng.random() < self.config.bistream_prob
            k, i, t = self.build_sample(s["text"], s["speech"], s.get("instruct", ()), bi)
            kinds += k
            ids += i
            tgt += t
            cu.append(len(ids))
        lens = [b - a for a, b in zip(cu[:-1], cu[1:])]
        return dict(input_ids=torch.tensor(ids, device=device), is_speech=torch.tensor([k == "s" for k in kinds], device=device),
                    labels=torch.tensor(tgt, device=device), cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=device),
                    max_seqlen=max(lens), n_samples=len(samples))

    def collate(self, samples: Sequence[dict]) -> dict:
        """Dataset rows (``text`` ids, ``codes`` whose first codebook is the speech token stream, optional ``instruct``)."""
        S = self.config.speech_token_size
        return self.pack([dict(text=s["text"].tolist(), speech=(s["codes"][:, 0] % S).tolist(),
                               instruct=s["instruct"].tolist() if "instruct" in s else ()) for s in samples])

    # ------------------------------------------------------------------ model
    def embed(self, ids, is_speech, run=None):
        run = run or (lambda m, *a, **k: m(*a, **k))
        text_vocab = self.backbone.embed_tokens.weight.shape[0]
        te = run(self.backbone.embed_tokens, torch.where(is_speech, torch.zeros_like(ids), ids).clamp(max=text_vocab - 1))
        se = run(self.speech_embedding, torch.where(is_speech, ids, torch.zeros_like(ids)))
        return torch.where(is_speech[:, None], se, te)

    def forward(self, batch: dict, run=None):
        c = self.config
        h = self.hidden(self.embed(batch["input_ids"], batch["is_speech"], run), batch, run)
        h = self.backbone.lm_head.norm(h)
        labels = batch.get("labels")
        if labels is None:
            return ops.linear(h, self.llm_decoder.weight)
        if c.lsm_weight == 0.0 and c.length_normalized_loss:
            loss = _ce_mean(h, self.llm_decoder.weight, labels)
        else:
            loss = label_smoothing_loss(ops.linear(h, self.llm_decoder.weight), labels, c.lsm_weight, c.length_normalized_loss,
                                        batch.get("n_samples", 1))
        with torch.no_grad():
            keep = labels != IGNORE
            pred = ops.linear(h[keep], self.llm_decoder.weight).argmax(-1)
            self.last_accuracy = (pred == labels[keep]).float().mean() if bool(keep.any()) else h.new_zeros(())
        return loss

    @torch.no_grad()
    def generate(self, text: Sequence[int], prompt_speech: Sequence[int] = (), instruct: Sequence[int] = (), max_len: int = 64,
                 min_len: int = 0, generator=None, **sampling) -> List[int]:
        kinds = ["s"] + ["t"] * (len(instruct) + len(text)) + ["s"] + ["s"] * len(prompt_speech)
        ids = [self.sos] + list(instruct) + list(text) + [self.task_id] + list(prompt_speech)
        dev = self.llm_decoder.weight.device
        out: List[int] = []
        for step in range(max_len):
            T = len(ids)
            b = dict(input_ids=torch.tensor(ids, device=dev), is_speech=torch.tensor([k == "s" for k in kinds], device=dev),
                     cu_seqlens=torch.tensor([0, T], dtype=torch.int32, device=dev), max_seqlen=T)
            scores = self.forward(b)[-1].float()
            if step < min_len:
                scores[self.config.speech_token_size:] = -float("inf")
            tok = ras_sampling(scores, out, generator=generator, **sampling)
            if tok >= self.config.speech_token_size:
                break
            out.append(tok)
            ids.append(tok)
            kinds.append("s")
        return out


# ------------------------------------------------------------------------------------------------- Qwen3-TTS
class _TDNN(nn.Module):
    def __init__(self, cin, cout, k, dilation=1):
        super().__init__()
        self.conv = nn.Conv1d(cin, cout, k, dilation=dilation, padding=dilation * (k - 1) // 2, padding_mode="reflect")

    def forward(self, x):
        return F.relu(self.conv(x))


class _SERes2Net(nn.Module):
    """TDNN -> Res2Net (hierarchical dilated convs over channel groups) -> TDNN -> squeeze-excitation, residual."""

    def __init__(self, c, scale=8, k=3, dilation=1, se=128):
        super().__init__()
        self.scale = scale
        w = c // scale
        self.tdnn1, self.tdnn2 = _TDNN(c, c, 1), _TDNN(c, c, 1)
        self.res2 = nn.ModuleList(_TDNN(w, w, k, dilation) for _ in range(scale - 1))
        self.se1, self.se2 = nn.Conv1d(c, se, 1), nn.Conv1d(se, c, 1)

    def forward(self, x):
        h = self.tdnn1(x)
        parts, prev, outs = h.chunk(self.scale, 1), None, []
        for i, p in enumerate(parts):
            if i == 0:
                prev = p
            else:
                prev = self.res2[i - 1](p if i == 1 else p + prev)
            outs.append(prev)
        h = self.tdnn2(torch.cat(outs, 1))
        g = torch.sigmoid(self.se2(F.relu(self.se1(h.mean(2, keepdim=True)))))
        return x + h * g


class SpeakerEncoder(nn.Module):
    """ECAPA-TDNN: mel [B, T, n_mels] -> speaker embedding [B, dim] (attentive statistics pooling over time)."""

    def __init__(self, n_mels: int = 128, channels: int = 512, dim: int = 1024, attn: int = 128, scale: int = 8):
        super().__init__()
        self.inp = _TDNN(n_mels, channels, 5)
        self.blocks = nn.ModuleList(_SERes2Net(channels, scale, 3, d, attn) for d in (2, 3, 4))
        self.mfa = _TDNN(3 * channels, 3 * channels, 1)
        self.att1, self.att2 = nn.Conv1d(9 * channels, attn, 1), nn.Conv1d(attn, 3 * channels, 1)
        self.fc = nn.Conv1d(6 * channels, dim, 1)

    def forward(self, mel):
        x = self.inp(mel.transpose(1, 2))
        feats = []
        for b in self.blocks:
            x = b(x)
            feats.append(x)
        h = self.mfa(torch.cat(feats, 1))
        mu, sd = h.mean(2, keepdim=True), h.std(2, keepdim=True).clamp(min=1e-5)
        a = self.att2(torch.tanh(self.att1(torch.cat([h, mu.expand_as(h), sd.expand_as(h)], 1))))
        w = F.softmax(a, 2)
        mean = (w * h).sum(2)
        std = ((w * (h - mean[:, :, None]) ** 2).sum(2)).clamp(min=1e-5).sqrt()
        return self.fc(torch.cat([mean, std], 1)[:, :, None])[:, :, 0]


@dataclass
class Qwen3TTSConfig:
    talker: DecoderConfig = field(default_factory=DecoderConfig)          # vocab_size = codec vocabulary
    predictor: DecoderConfig = field(default_factory=DecoderConfig)       # the small per-frame decoder
    text_vocab_size: int = 151936
    text_hidden_size: int = 2048
    num_code_groups: int = 16
    speaker_dim: int = 1024
    n_mels: int = 128
    speaker_channels: int = 512
    sub_talker_weight: float = 0.3

    @staticmethod
    def tiny(**kw):
        from .composable import _tiny_text
        d = dict(talker=_tiny_text(rope="rope1d", vocab_size=64), predictor=_tiny_text(rope="rope1d", vocab_size=64, hidden_size=64,
                 intermediate_size=128, num_attention_heads=2, num_key_value_heads=1, head_dim=32, num_layers=1),
                 text_vocab_size=100, text_hidden_size=48, num_code_groups=4, speaker_dim=128, n_mels=20, speaker_channels=32)
        d.update(kw)
        return Qwen3TTSConfig(**d)


class CodePredictor(_Wrapped):
    """Per-frame decoder over the codebook axis: inputs [talker hidden, emb(code 0), ..., emb(code G-2)] (all in the
    talker's width, projected down), position i + 1 predicts code i + 1 with its own head."""

    def __init__(self, c: Qwen3TTSConfig):
        super().__init__()
        G, Ht, Hp, V = c.num_code_groups, c.talker.hidden_size, c.predictor.hidden_size, c.predictor.vocab_size
        self.G = G
        self.backbone = _text_lm(c.predictor)
        self.codec_embedding = nn.ModuleList(Embedding(V, Ht) for _ in range(G - 1))     # tables of codes 1 .. G-1
        self.small_to_mtp_projection = nn.Linear(Ht, Hp) if Ht != Hp else nn.Identity()
        self.heads = nn.ParameterList(nn.Parameter(torch.empty(V, Hp)) for _ in range(G - 1))

    def _extra_units(self):
        return [("codec_embedding", self.codec_embedding), ("small_to_mtp_projection", self.small_to_mtp_projection),
                ("heads", self.heads)]

    def frame_hidden(self, frame_inputs: torch.Tensor, run=None) -> torch.Tensor:
        """``frame_inputs`` [N, L <= G, Ht] -> normed hidden [N, L, Hp]; every frame is its own causal sequence."""
        N, L, _ = frame_inputs.shape
        x = self.small_to_mtp_projection(frame_inputs).reshape(N * L, -1)
        cu = torch.arange(0, (N + 1) * L, L, dtype=torch.int32, device=x.device)
        h = self.hidden(x, dict(cu_seqlens=cu, max_seqlen=L), run)
        return self.backbone.lm_head.norm(h).reshape(N, L, -1)

    def loss(self, talker_hidden, codec_ids, code0_embed, run=None):
        """``talker_hidden`` [N, Ht], ``codec_ids`` [N, G], ``code0_embed`` [N, Ht] (from the talker's own codec table)."""
        G = self.G
        seq = [talker_hidden[:, None], code0_embed[:, None]] + \
              [self.codec_embedding[i - 1](codec_ids[:, i])[:, None] for i in range(1, G - 1)]
        h = self.frame_hidden(torch.cat(seq, 1), run)                                     # [N, G, Hp]
        total = h.new_zeros((), dtype=torch.float32)
        for i in range(1, G):
            total = total + _ce_mean(h[:, i], self.heads[i - 1], codec_ids[:, i])
        return total / (G - 1)

    @torch.no_grad()
    def generate(self, talker_hidden, code0, code0_embed, temperature: float = 0.0, generator=None):
        """Greedy / sampled codes 1 .. G-1 for N frames given their talker hidden state and code 0."""
        seq = torch.cat([talker_hidden[:, None], code0_embed[:, None]], 1)
        codes = [code0]
        for i in range(1, self.G):
            h = self.frame_hidden(seq)[:, -1]
            lg = ops.linear(h, self.heads[i - 1]).float()
            nxt = lg.argmax(-1) if temperature <= 0 else torch.multinomial(F.softmax(lg / temperature, -1).cpu(), 1,
                                                                            generator=generator)[:, 0].to(lg.device)
            codes.append(nxt)
            if i < self.G - 1:
                seq = torch.cat([seq, self.codec_embedding[i - 1](nxt)[:, None]], 1)
        return torch.stack(codes, 1)


@model_register.register("qwen3tts")
class Qwen3TTSTalker(_Wrapped):
    """Packed batch (one row per position):

    ``text_ids`` [T], ``text_mask`` [T] (1 where the text embedding takes part), ``codec_in`` [T] (codec-vocabulary id fed at
    this position: control ids in the prefix, code 0 of the previous frame inside the audio span), ``codec_in_mask`` [T],
    ``codec_ids`` [T, G] + ``codec_mask`` [T] (positions that carry a full frame whose codes 1.. are added to the input),
    ``labels`` [T] (code 0 to predict, -100 elsewhere), ``speaker_pos`` [n_seq] (row that receives the speaker embedding),
    ``ref_mels`` [n_seq, frames, n_mels] or ``speaker_embedding`` [n_seq, H], ``cu_seqlens``, ``max_seqlen``.
    """
    config_class = Qwen3TTSConfig

    def __init__(self, config: Optional[Qwen3TTSConfig] = None):
        super().__init__()
        self.config = c = config or Qwen3TTSConfig.tiny()
        H = c.talker.hidden_size
        self.backbone = _text_lm(c.talker)                      # embed_tokens = codec embedding, lm_head = codec head
        self.text_embedding = Embedding(c.text_vocab_size, c.text_hidden_size)
        self.text_projection = nn.Sequential(nn.Linear(c.text_hidden_size, c.text_hidden_size), nn.SiLU(),
                                             nn.Linear(c.text_hidden_size, H))
        self.code_predictor = CodePredictor(c)
        self.speaker_encoder = SpeakerEncoder(c.n_mels, c.speaker_channels, c.speaker_dim)
        self.speaker_proj = nn.Linear(c.speaker_dim, H) if c.speaker_dim != H else nn.Identity()

    def _extra_units(self):
        return [("text_embedding", self.text_embedding), ("text_projection", self.text_projection),
                ("speaker_encoder", self.speaker_encoder), ("speaker_proj", self.speaker_proj)] + \
               [(f"code_predictor.{n}", m) for n, m in self.code_predictor.fsdp_units()]

    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: float = 0.02):
        super().init_weights(seed, std)
        self.code_predictor.init_weights(seed + 7, std)

    def embed(self, batch, run=None):
        run = run or (lambda m, *a, **k: m(*a, **k))
        dt = self.backbone.embed_tokens.weight.dtype
        x = self.text_projection(run(self.text_embedding, batch["text_ids"])) * batch["text_mask"][:, None].to(dt)
        x = x + run(self.backbone.embed_tokens, batch["codec_in"]) * batch["codec_in_mask"][:, None].to(dt)
        spk = batch.get("speaker_embedding")
        if spk is None and batch.get("ref_mels") is not None:
            spk = self.speaker_encoder(batch["ref_mels"].to(dt)).detach()
        if spk is not None:
            x = x.index_copy(0, batch["speaker_pos"], x[batch["speaker_pos"]] * 0 + self.speaker_proj(spk.to(dt)))
        cm = batch["codec_mask"]
        if bool(cm.any()):
            add = x.new_zeros(int(cm.sum()), x.shape[1])
            frames = batch["codec_ids"][cm]
            for i in range(1, self.config.num_code_groups):
                add = add + self.code_predictor.codec_embedding[i - 1](frames[:, i])
            x = x.index_add(0, cm.nonzero(as_tuple=True)[0], add)
        return x

    def forward(self, batch: dict, run=None):
        c = self.config
        h = self.hidden(self.embed(batch, run), batch, run)
        labels = batch.get("labels")
        hn = self.backbone.lm_head.norm(h)
        if labels is None:
            return ops.linear(hn, self.backbone.lm_head.weight)
        loss = _ce_mean(hn, self.backbone.lm_head.weight, labels)
        # the position that predicts code 0 of a frame also conditions that frame's remaining codebooks
        has_frame = labels != IGNORE
        if batch.get("eos_rows") is not None:
            has_frame = has_frame.index_fill(0, batch["eos_rows"].to(labels.device), False)    # eos has no frame behind it
        pred_pos = has_frame.nonzero(as_tuple=True)[0]
        frames = batch.get("label_codec_ids")
        if frames is not None and pred_pos.numel():
            code0_embed = self.backbone.embed_tokens(frames[:, 0])
            sub = self.code_predictor.loss(hn[pred_pos], frames, code0_embed, run)
            self.last_sub_talker_loss = sub.detach()
            loss = loss + c.sub_talker_weight * sub
        return loss

    def collate(self, samples: Sequence[dict]) -> dict:
        """Dataset rows (``text``, ``codes`` [frames, G], ``ref_mel``).  The last three ids of the codec vocabulary serve as
        bos / eos / pad."""
        c = self.config
        V = c.talker.vocab_size
        built = [self.build_sample(s["text"].tolist(), s["codes"][:, : c.num_code_groups].long() % (V - 3), V - 3, V - 2, V - 1)
                 for s in samples]
        return self.pack(built, ref_mels=torch.stack([s["ref_mel"] for s in samples]))

    @staticmethod
    def build_sample(text_ids: Sequence[int], codes: torch.Tensor, bos: int, eos: int, pad: int, speaker_slot: bool = True) -> dict:
        """One utterance -> rows.  Layout: [speaker slot] [text tokens, each with codec pad] [bos] [frame 0] ... [frame F-1];
        row r predicts code 0 of the frame that row r + 1 feeds, the last frame row predicts ``eos``."""
        Fr, G = codes.shape
        n_text = len(text_ids)
        pre = (1 if speaker_slot else 0) + n_text + 1
        T = pre + Fr
        text = torch.zeros(T, dtype=torch.long)
        tmask = torch.zeros(T, dtype=torch.bool)
        cin = torch.full((T,), pad, dtype=torch.long)
        cmask = torch.ones(T, dtype=torch.bool)
        off = 1 if speaker_slot else 0
        text[off:off + n_text] = torch.tensor(list(text_ids), dtype=torch.long)
        tmask[off:off + n_text] = True
        cin[pre - 1] = bos
        cin[pre:] = codes[:, 0]
        frame_mask = torch.zeros(T, dtype=torch.bool)
        frame_mask[pre:] = True
        cids = torch.zeros(T, G, dtype=torch.long)
        cids[pre:] = codes
        labels = torch.full((T,), IGNORE, dtype=torch.long)
        labels[pre - 1:T - 1] = codes[:, 0]
        labels[T - 1] = eos
        # the eos row has no frame to hand to the code predictor
        return dict(text_ids=text, text_mask=tmask, codec_in=cin, codec_in_mask=cmask, codec_ids=cids, codec_mask=frame_mask,
                    labels=labels, label_codec_ids=codes.clone(), length=T, eos_rows=torch.tensor([T - 1]))

    @staticmethod
    def pack(samples: Sequence[dict], speaker_embedding=None, ref_mels=None) -> dict:
        keys = ("text_ids", "text_mask", "codec_in", "codec_in_mask", "codec_ids", "codec_mask", "labels")
        out = {k: torch.cat([s[k] for s in samples]) for k in keys}
        lens = [s["length"] for s in samples]
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        out["cu_seqlens"] = torch.tensor(cu, dtype=torch.int32)
        out["max_seqlen"] = max(lens)
        out["speaker_pos"] = torch.tensor(cu[:-1])
        # rows whose label is a real code 0 (not eos) line up, in order, with the frames of label_codec_ids
        out["label_codec_ids"] = torch.cat([s["label_codec_ids"] for s in samples])
        eos_rows = torch.cat([s["eos_rows"] + c for s, c in zip(samples, cu[:-1])])
        out["eos_rows"] = eos_rows
        if speaker_embedding is not None:
            out["speaker_embedding"] = speaker_embedding
        if ref_mels is not None:
            out["ref_mels"] = ref_mels
        return out
