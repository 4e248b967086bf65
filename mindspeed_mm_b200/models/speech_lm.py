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


class SummedEmbeddings(nn.Module):
    """``n`` embedding tables looked up by the columns of an id matrix: ``forward(ids [T, n])`` returns the sum [T, D],
    ``forward(ids, stack=True)`` the separate rows [T, n, D]."""

    def __init__(self, n: int, vocab: int, dim: int):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(n, vocab, dim))

    def forward(self, ids, stack: bool = False):
        n, V, D = self.weight.shape
        flat = self.weight.view(n * V, D)
        e = F.embedding(ids + torch.arange(ids.shape[1], device=ids.device) * V, flat)      # [T, k, D], k <= n
        return e if stack else e.sum(1)


class NormedHeads(nn.Module):
    """The decoder's final norm followed by one or several output tables.  Owns the backbone's ``lm_head`` module (so
    that norm and tables are gathered together as one sharding unit) plus ``extra`` tables of its own.

    ``forward(h, labels [T, n_tables] or None, drop_last)``: returns the per-table mean cross entropies [n_tables] (tables
    whose label column is all -100 give 0) or, without labels, the list of logits.  ``drop_last[i]`` removes the last
    row of table i from the prediction (an input-only padding id)."""

    def __init__(self, lm_head: nn.Module, extra: Sequence[Tuple[int, int]] = (), use_lm_table: bool = True):
        super().__init__()
        self.lm_head = lm_head
        self.use_lm_table = use_lm_table
        if not use_lm_table:
            self.lm_head.weight = None
        self.extra = nn.ParameterList(nn.Parameter(torch.empty(v, d)) for v, d in extra)

    def tables(self, drop_last: Sequence[bool] = ()):
        ws = ([self.lm_head.weight] if self.use_lm_table else []) + list(self.extra)
        return [w[:-1] if i < len(drop_last) and drop_last[i] else w for i, w in enumerate(ws)]

    def forward(self, h, labels=None, drop_last: Sequence[bool] = (), return_normed: bool = False):
        hn = self.lm_head.norm(h)
        ws = self.tables(drop_last)
        if labels is None:
            out = [ops.linear(hn, w) for w in ws]
            return (out, hn) if return_normed else out
        if labels.dim() == 1:
            labels = labels[:, None]
        losses = []
        for k, w in enumerate(ws):
            lab = labels[:, k]
            losses.append(_ce_mean(hn, w, lab) if bool((lab != IGNORE).any()) else hn.new_zeros((), dtype=torch.float32))
        out = torch.stack(losses)
        return (out, hn) if return_normed else out


class _Wrapped(nn.Module):
    """Common plumbing: ``self.backbone`` + extra tables / heads, exposed to the sharding engine as units."""

    backbone: ComposableLM

    def _extra_units(self) -> List[Tuple[str, nn.Module]]:
        return []

    def fsdp_units(self):
        # the backbone's lm_head belongs to this model's ``heads`` unit
        return self._extra_units() + [(f"backbone.{n}", m) for n, m in self.backbone.fsdp_units() if n != "lm_head"]

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
        self.emb_ext = SummedEmbeddings(c.n_vq, c.audio_vocab_size + 1, H)
        self.heads = NormedHeads(self.backbone.lm_head, [(c.audio_vocab_size + 1, H)] * c.n_vq)

    def _extra_units(self):
        return [("emb_ext", self.emb_ext), ("heads", self.heads)]

    def embed(self, ids, run=None):
        run = run or (lambda m, *a, **k: m(*a, **k))
        return run(self.backbone.embed_tokens, ids[:, 0]) + run(self.emb_ext, ids[:, 1:])

    def forward(self, batch: dict, run=None):
        c = self.config
        ids = batch["input_ids"]
        if ids.dim() != 2 or ids.shape[1] != c.n_vq + 1:
            raise ValueError("input_ids must be [tokens, 1 + n_vq]")
        run = run or (lambda m, *a, **k: m(*a, **k))
        h = self.hidden(self.embed(ids, run), batch, run)
        # the last index of every audio table is an input-only padding code: it is never predicted
        drop = [False] + [True] * c.n_vq
        labels = batch.get("labels")
        if labels is None:
            return run(self.heads, h, None, drop)
        parts = run(self.heads, h, labels, drop)
        cw = torch.tensor(list(c.channel_loss_weight or [1.0] * (c.n_vq + 1)), dtype=parts.dtype, device=parts.device)
        self.last_channel_losses = parts.detach()
        return (parts * cw).sum() / cw.sum()

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
        # output table over the speech ids (incl. the special ones) behind the decoder's final norm; the text-vocabulary
        # table of the backbone is dropped
        self.heads = NormedHeads(self.backbone.lm_head, [(S + 200, H)], use_lm_table=False)
        self.rng = random.Random(0)

    def _extra_units(self):
        return [("speech_embedding", self.speech_embedding), ("heads", self.heads)]

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
        text_vocab = self.config.text.vocab_size
        te = run(self.backbone.embed_tokens, torch.where(is_speech, torch.zeros_like(ids), ids).clamp(max=text_vocab - 1))
        se = run(self.speech_embedding, torch.where(is_speech, ids, torch.zeros_like(ids)))
        return torch.where(is_speech[:, None], se, te)

    def forward(self, batch: dict, run=None):
        c = self.config
        run = run or (lambda m, *a, **k: m(*a, **k))
        h = self.hidden(self.embed(batch["input_ids"], batch["is_speech"], run), batch, run)
        labels = batch.get("labels")
        if labels is None:
            return run(self.heads, h)[0]
        if c.lsm_weight == 0.0 and c.length_normalized_loss:
            return run(self.heads, h, labels)[0]
        return label_smoothing_loss(run(self.heads, h)[0], labels, c.lsm_weight, c.length_normalized_loss, batch.get("n_samples", 1))

    @torch.no_grad()
    def accuracy(self, batch: dict) -> torch.Tensor:
        """Share of label positions whose arg-max prediction is right (the reference logs it next to the loss)."""
        logits = self.forward({k: v for k, v in batch.items() if k != "labels"})
        keep = batch["labels"] != IGNORE
        return (logits[keep].argmax(-1) == batch["labels"][keep]).float().mean()

    @torch.no_grad()
    def generate(self, text: Sequence[int], prompt_speech: Sequence[int] = (), instruct: Sequence[int] = (), max_len: int = 64,
                 min_len: int = 0, generator=None, **sampling) -> List[int]:
        kinds = ["s"] + ["t"] * (len(instruct) + len(text)) + ["s"] + ["s"] * len(prompt_speech)
        ids = [self.sos] + list(instruct) + list(text) + [self.task_id] + list(prompt_speech)
        dev = self.speech_embedding.weight.device
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


class _FrameHeads(nn.Module):
    """Heads of the code predictor: final norm, then head i - 1 reads position i of every frame sequence."""

    def __init__(self, lm_head: nn.Module, n_heads: int, vocab: int, dim: int):
        super().__init__()
        self.lm_head = lm_head
        self.lm_head.weight = None
        self.weight = nn.Parameter(torch.empty(n_heads, vocab, dim))

    def forward(self, h, codec_ids=None, position: Optional[int] = None):
        """``h`` [N, L, D].  With ``codec_ids`` [N, G]: mean CE over heads 1 .. G-1.  With ``position`` i: logits of head i - 1
        at the last position."""
        hn = self.lm_head.norm(h)
        if codec_ids is None:
            return ops.linear(hn[:, -1], self.weight[position - 1])
        G = codec_ids.shape[1]
        total = hn.new_zeros((), dtype=torch.float32)
        for i in range(1, G):
            total = total + _ce_mean(hn[:, i], self.weight[i - 1], codec_ids[:, i])
        return total / (G - 1)


class CodePredictor(_Wrapped):
    """Per-frame decoder over the codebook axis: inputs [talker hidden, emb(code 0), ..., emb(code G-2)] (all in the
    talker's width, projected down), position i + 1 predicts code i + 1 with its own head."""

    def __init__(self, c: Qwen3TTSConfig):
        super().__init__()
        G, Ht, Hp, V = c.num_code_groups, c.talker.hidden_size, c.predictor.hidden_size, c.predictor.vocab_size
        self.G = G
        self.backbone = _text_lm(c.predictor)
        self.backbone.embed_tokens = None                                  # inputs are always embeddings
        self.codec_embedding = SummedEmbeddings(G - 1, V, Ht)              # tables of codes 1 .. G-1
        self.small_to_mtp_projection = nn.Linear(Ht, Hp)
        self.heads = _FrameHeads(self.backbone.lm_head, G - 1, V, Hp)

    def _extra_units(self):
        return [("codec_embedding", self.codec_embedding), ("small_to_mtp_projection", self.small_to_mtp_projection),
                ("heads", self.heads)]

    def fsdp_units(self):
        return [(n, m) for n, m in super().fsdp_units() if m is not None]

    def frame_hidden(self, frame_inputs: torch.Tensor, run=None) -> torch.Tensor:
        """``frame_inputs`` [N, L <= G, Ht] -> hidden [N, L, Hp]; every frame is its own causal sequence."""
        run = run or (lambda m, *a, **k: m(*a, **k))
        N, L, _ = frame_inputs.shape
        x = run(self.small_to_mtp_projection, frame_inputs).reshape(N * L, -1)
        cu = torch.arange(0, (N + 1) * L, L, dtype=torch.int32, device=x.device)
        return self.hidden(x, dict(cu_seqlens=cu, max_seqlen=L), run).reshape(N, L, -1)

    def loss(self, talker_hidden, codec_ids, code0_embed, run=None):
        """``talker_hidden`` [N, Ht], ``codec_ids`` [N, G], ``code0_embed`` [N, Ht] (from the talker's own codec table)."""
        run = run or (lambda m, *a, **k: m(*a, **k))
        seq = [talker_hidden[:, None], code0_embed[:, None]]
        if self.G > 2:
            seq.append(run(self.codec_embedding, codec_ids[:, 1:self.G - 1], True))
        h = self.frame_hidden(torch.cat(seq, 1), run)                                     # [N, G, Hp]
        return run(self.heads, h, codec_ids)

    @torch.no_grad()
    def generate(self, talker_hidden, code0, code0_embed, temperature: float = 0.0, generator=None):
        """Greedy / sampled codes 1 .. G-1 for N frames given their talker hidden state and code 0."""
        seq = torch.cat([talker_hidden[:, None], code0_embed[:, None]], 1)
        codes = [code0]
        for i in range(1, self.G):
            lg = self.heads(self.frame_hidden(seq), None, i).float()
            nxt = lg.argmax(-1) if temperature <= 0 else torch.multinomial(F.softmax(lg / temperature, -1).cpu(), 1,
                                                                            generator=generator)[:, 0].to(lg.device)
            codes.append(nxt)
            if i < self.G - 1:
                V = self.codec_embedding.weight.shape[1]
                emb = F.embedding(nxt + (i - 1) * V, self.codec_embedding.weight.view(-1, self.codec_embedding.weight.shape[2]))
                seq = torch.cat([seq, emb[:, None]], 1)
        return torch.stack(codes, 1)


class _TextFrontEnd(nn.Module):
    """Text id -> talker width: embedding in the text model's width followed by a two-layer projection."""

    def __init__(self, vocab, text_hidden, hidden):
        super().__init__()
        self.embedding = Embedding(vocab, text_hidden)
        self.fc1, self.fc2 = nn.Linear(text_hidden, text_hidden), nn.Linear(text_hidden, hidden)

    def forward(self, ids):
        return self.fc2(F.silu(self.fc1(self.embedding(ids))))


class _SpeakerFrontEnd(nn.Module):
    def __init__(self, c: "Qwen3TTSConfig", hidden):
        super().__init__()
        self.encoder = SpeakerEncoder(c.n_mels, c.speaker_channels, c.speaker_dim)
        self.proj = nn.Linear(c.speaker_dim, hidden)

    def forward(self, mels=None, embedding=None):
        if embedding is None:
            embedding = self.encoder(mels).detach()            # the reference trains with a frozen speaker embedding
        return self.proj(embedding)


@model_register.register("qwen3tts")
class Qwen3TTSTalker(_Wrapped):
    """Packed batch (one row per position):

    ``text_ids`` [T], ``text_mask`` [T] (1 where the text embedding takes part), ``codec_in`` [T] (codec-vocabulary id fed at
    this position: control ids in the prefix, code 0 of the previous frame inside the audio span), ``codec_in_mask`` [T],
    ``codec_ids`` [T, G] + ``codec_mask`` [T] (positions that carry a full frame whose codes 1.. are added to the input),
    ``labels`` [T] (code 0 to predict, -100 elsewhere), ``speaker_pos`` [n_seq] (row that receives the speaker embedding),
    ``ref_mels`` [n_seq, frames, n_mels] or ``speaker_embedding`` [n_seq, speaker_dim], ``cu_seqlens``, ``max_seqlen``.
    """
    config_class = Qwen3TTSConfig

    def __init__(self, config: Optional[Qwen3TTSConfig] = None):
        super().__init__()
        self.config = c = config or Qwen3TTSConfig.tiny()
        H = c.talker.hidden_size
        self.backbone = _text_lm(c.talker)                      # embed_tokens = codec embedding, lm_head = codec head
        self.text_front = _TextFrontEnd(c.text_vocab_size, c.text_hidden_size, H)
        self.speaker_front = _SpeakerFrontEnd(c, H)
        self.heads = NormedHeads(self.backbone.lm_head)
        self.code_predictor = CodePredictor(c)

    def _extra_units(self):
        return [("text_front", self.text_front), ("speaker_front", self.speaker_front), ("heads", self.heads)] + \
               [(f"code_predictor.{n}", m) for n, m in self.code_predictor.fsdp_units()]

    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: float = 0.02):
        super().init_weights(seed, std)
        self.code_predictor.init_weights(seed + 7, std)

    def embed(self, batch, run=None):
        run = run or (lambda m, *a, **k: m(*a, **k))
        dt = self.backbone.embed_tokens.weight.dtype
        x = run(self.text_front, batch["text_ids"]) * batch["text_mask"][:, None].to(dt)
        x = x + run(self.backbone.embed_tokens, batch["codec_in"]) * batch["codec_in_mask"][:, None].to(dt)
        if batch.get("speaker_embedding") is not None or batch.get("ref_mels") is not None:
            mels = batch["ref_mels"].to(dt) if batch.get("ref_mels") is not None else None
            emb = batch["speaker_embedding"].to(dt) if batch.get("speaker_embedding") is not None else None
            x = x.index_copy(0, batch["speaker_pos"], run(self.speaker_front, mels, emb).to(x.dtype))
        cm = batch["codec_mask"]
        if bool(cm.any()):
            add = run(self.code_predictor.codec_embedding, batch["codec_ids"][cm][:, 1:])
            x = x.index_add(0, cm.nonzero(as_tuple=True)[0], add.to(x.dtype))
        return x

    def forward(self, batch: dict, run=None):
        run = run or (lambda m, *a, **k: m(*a, **k))
        c = self.config
        h = self.hidden(self.embed(batch, run), batch, run)
        labels = batch.get("labels")
        if labels is None:
            return run(self.heads, h)[0]
        parts, hn = run(self.heads, h, labels, (), True)
        loss = parts[0]
        # the position that predicts code 0 of a frame also conditions that frame's remaining codebooks
        has_frame = labels != IGNORE
        if batch.get("eos_rows") is not None:
            has_frame = has_frame.index_fill(0, batch["eos_rows"].to(labels.device), False)    # eos has no frame behind it
        pred_pos = has_frame.nonzero(as_tuple=True)[0]
        frames = batch.get("label_codec_ids")
        if frames is not None and pred_pos.numel():
            code0_embed = run(self.backbone.embed_tokens, frames[:, 0])
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
