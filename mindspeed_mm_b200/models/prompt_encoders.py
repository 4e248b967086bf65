"""Prompt encoders of the HunyuanVideo family: a decoder-only language model read at an inner layer, and a byte-level T5
that encodes only the text the picture should *show* (glyphs).

* ``DecoderPromptEncoder`` -- wraps a causal LM (any model of this package that takes a packed batch and returns hidden
  states).  The prompt is put into an instruction template; the hidden state ``skip_layer`` layers before the last is
  returned and the template's instruction prefix (``crop_start`` tokens) is cut off, so the DiT sees prompt tokens only
  (mindspeed_mm/models/text_encoder/hunyuan_mllm_text_encoder.py, hunyuan15_mllm_text_encoder.py:63-121; template
  application hunyuan15_mllm_tokenizer.py:17-28, max length grown by ``crop_start`` at :60).
* ``ByteTokenizer`` -- the ByT5 vocabulary: ids 0-2 are pad / end / unknown, byte ``b`` is ``b + 3``, followed by the
  sentinel ids and by the added colour and font tokens (hunyuan15_glyph_tokenizer.py:36-84).
* ``extract_glyph_texts`` / ``format_glyph_prompt`` -- quoted spans of the prompt, de-duplicated in order, rendered as
  ``Text "<span>". `` with optional colour / font tokens (hunyuan15_glyph_tokenizer.py:92-131,
  hunyuan15_byt5/format_prompt.py:57-89).
* ``GlyphByT5Encoder`` -- a T5 encoder over those bytes; prompts without quoted text give an all-zero embedding and an
  all-zero mask (hunyuan15_glyph_text_encoder.py:36-47).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple, Union

import torch
import torch.nn as nn

from .registry import model_register
from .text_encoder import T5Config, T5Encoder

# ------------------------------------------------------------------------------------------------ templates
TEMPLATES: Dict[str, dict] = {
    # instruction prefixes of the video / image prompt encoders; ``crop_start`` is the prefix length in tokens of the
    # tokenizer the checkpoint ships with and must be re-measured (``measure_crop_start``) for any other tokenizer
    "encode-video": {
        "template": "<|start_header_id|>system<|end_header_id|>\n\nDescribe the video by detailing the following aspects: "
                    "1. The main content and theme of the video."
                    "2. The color, shape, size, texture, quantity, text, and spatial relationships of the objects."
                    "3. Actions, events, behaviors temporal relationships, physical movement changes of the objects."
                    "4. background environment, light, style and atmosphere."
                    "5. camera angles, movements, and transitions used in the video:<|eot_id|>"
                    "<|start_header_id|>user<|end_header_id|>\n\n{}<|eot_id|>",
        "crop_start": 95},
    "encode-image": {
        "template": "<|start_header_id|>system<|end_header_id|>\n\nDescribe the image by detailing the color, shape, size, "
                    "texture, quantity, text, spatial relationships of the objects and background:<|eot_id|>"
                    "<|start_header_id|>user<|end_header_id|>\n\n{}<|eot_id|>",
        "crop_start": 36},
    "encode-video-chat": {
        "template": [{"role": "system", "content": "You are a helpful assistant. Describe the video by detailing the following "
                                                   "aspects: 1. The main content and theme of the video. 2. The color, shape, "
                                                   "size, texture, quantity, text, and spatial relationships of the objects. "
                                                   "3. Actions, events, behaviors temporal relationships, physical movement "
                                                   "changes of the objects. 4. background environment, light, style and "
                                                   "atmosphere. 5. camera angles, movements, and transitions used in the video."},
                     {"role": "user", "content": "{}"}],
        "crop_start": None},                       # depends on the chat markup: measured with the tokenizer in use
}


def apply_template(text: str, template: Union[str, list], prevent_empty: bool = True):
    """A format string gets the text; a chat (list of role / content dicts) gets it in every ``content`` field."""
    if isinstance(template, str):
        return template.format(text)
    if isinstance(template, list):
        out = copy.deepcopy(template)
        for item in out:
            if isinstance(item, dict) and "content" in item:
                item["content"] = item["content"].format(text if text else (" " if prevent_empty else ""))
        return out
    raise TypeError(f"unsupported template type {type(template)}")


def render_chat(messages: Sequence[dict], add_generation_prompt: bool = True) -> str:
    """Plain ChatML rendering for tokenizers without a chat template of their own."""
    s = "".join(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n" for m in messages)
    return s + ("<|im_start|>assistant\n" if add_generation_prompt else "")


def measure_crop_start(template: Union[str, list], encode: Callable[[str], List[int]]) -> int:
    """Length in tokens of what precedes the prompt in ``template`` under ``encode``."""
    marker = "\u0001PROMPT\u0001"
    full = apply_template(marker, template)
    text = render_chat(full) if isinstance(full, list) else full
    return len(encode(text.split(marker)[0]))


def resolve_template(template: Optional[dict], encode: Callable[[str], List[int]]) -> Optional[dict]:
    """Copy of ``template`` whose ``crop_start`` is a number (measured under ``encode`` when it was left open)."""
    if template is None:
        return None
    t = dict(template)
    if t.get("crop_start") is None:
        t["crop_start"] = measure_crop_start(t["template"], encode)
    return t


def tokenize_prompts(texts: Sequence[str], encode: Callable[[str], List[int]], template: Optional[dict], max_length: int,
                     pad_id: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (ids [B, max_length + crop_start], mask) right-padded; the budget grows by the prefix length so that
    ``max_length`` prompt tokens survive the crop."""
    template = resolve_template(template, encode)
    crop = max(int(template.get("crop_start", 0)), 0) if template else 0
    L = max_length + crop
    ids = torch.full((len(texts), L), pad_id, dtype=torch.long)
    mask = torch.zeros(len(texts), L, dtype=torch.long)
    for i, t in enumerate(texts):
        if template:
            t = apply_template(t, template["template"])
            t = render_chat(t) if isinstance(t, list) else t
        e = encode(t)[:L]
        ids[i, : len(e)] = torch.tensor(e, dtype=torch.long)
        mask[i, : len(e)] = 1
    return ids, mask


class DecoderPromptEncoder(nn.Module):
    """``encode(ids [B, L], mask [B, L]) -> (hidden [B, L - crop_start, H], mask [B, L - crop_start])``.

    ``lm.hidden_states(batch)`` must take this package's packed batch (``input_ids, position_ids, cu_seqlens, max_seqlen``)
    and return the embeddings followed by every layer's output -- ``ComposableLM`` does; for any other causal LM pass
    ``hidden_fn(ids, mask) -> list of [B, L, H] hidden states`` in that order."""

    def __init__(self, lm: nn.Module, template: Optional[dict] = None, skip_layer: int = 2, apply_final_norm: bool = False,
                 hidden_fn: Optional[Callable] = None):
        super().__init__()
        self.lm, self.template, self.skip_layer, self.apply_final_norm = lm, template, skip_layer, apply_final_norm
        self.hidden_fn = hidden_fn
        for p in self.parameters():
            p.requires_grad_(False)

    def _hidden_states(self, ids, mask) -> List[torch.Tensor]:
        if self.hidden_fn is not None:
            return list(self.hidden_fn(ids, mask))
        lm = self.lm
        B, L = ids.shape
        lens = mask.sum(1).to(torch.int32)
        keep = mask.bool().reshape(-1)
        flat = ids.reshape(-1)[keep]
        pos = torch.cat([torch.arange(int(n), device=ids.device) for n in lens])
        cu = torch.nn.functional.pad(lens.cumsum(0), (1, 0)).to(torch.int32)
        if getattr(getattr(getattr(lm, "config", None), "text", None), "rope", "") == "mrope":
            pos = pos[None].expand(3, -1)
        batch = dict(input_ids=flat, position_ids=pos, cu_seqlens=cu, max_seqlen=int(lens.max()))
        hs = lm.hidden_states(batch)                                     # embeddings + one entry per layer, each [T, H]
        out = []
        for h in hs:
            full = h.new_zeros(B * L, h.shape[-1])
            full[keep] = h
            out.append(full.view(B, L, -1))
        return out

    @torch.no_grad()
    def encode(self, input_ids, attention_mask=None):
        mask = attention_mask if attention_mask is not None else torch.ones_like(input_ids)
        hs = self._hidden_states(input_ids, mask)
        h = hs[-(self.skip_layer + 1)]
        if self.skip_layer > 0 and self.apply_final_norm and hasattr(self.lm, "final_norm"):
            h = self.lm.final_norm(h)
        crop = max(int(self.template.get("crop_start") or 0), 0) if self.template else 0
        if crop:
            h, mask = h[:, crop:], mask[:, crop:]
        return h, mask


# ------------------------------------------------------------------------------------------------ glyph branch
def extract_glyph_texts(prompt: str) -> List[str]:
    """Spans between straight double quotes, then spans between curly double quotes; first occurrence of each kept."""
    found: List[str] = []
    for open_q, close_q in (('"', '"'), ("“", "”")):
        at = 0
        while True:
            a = prompt.find(open_q, at)
            if a < 0:
                break
            b = prompt.find(close_q, a + 1)
            if b < 0:
                break
            found.append(prompt[a + 1: b])
            at = b + 1
    seen, out = set(), []
    for t in found:
        if t not in seen:
            seen.add(t)
            out.append(t)
    return out


def format_glyph_prompt(texts: Sequence[str], styles: Optional[Sequence[dict]] = None, color_index: Optional[dict] = None,
                        font_index: Optional[dict] = None) -> str:
    """``Text "<t>" in <color-i>, <xx-font-j>. `` per span; a style is ``{"color": name or None, "font-family": code or None}``.
    As in the reference, the attribute list is only written when a font is given."""
    styles = styles or [{"color": None, "font-family": None}] * len(texts)
    out = ""
    for t, st in zip(texts, styles):
        s = f'Text "{t}"'
        attrs = []
        if st.get("color") is not None and color_index is not None:
            attrs.append(f"<color-{color_index[st['color']]}>")
        font = st.get("font-family")
        if font is not None and font_index is not None:
            attrs.append(f"<{font[:2]}-font-{font_index[font]}>")
            s += " in " + ", ".join(attrs)
        out += s + ". "
    return out


class ByteTokenizer:
    """UTF-8 bytes + 3, with ``extra`` named tokens appended after the sentinel block (ByT5 layout: 256 bytes, 3 specials,
    125 sentinels -> first added token is id 384)."""
    pad_id, eos_id, unk_id = 0, 1, 2

    def __init__(self, extra_tokens: Sequence[str] = (), sentinels: int = 125):
        self.base = 256 + 3 + sentinels
        self.extra = {tok: self.base + i for i, tok in enumerate(extra_tokens)}
        self._by_len = sorted(self.extra, key=len, reverse=True)

    def __len__(self):
        return self.base + len(self.extra)

    @classmethod
    def with_styles(cls, color_index: dict, font_index: dict):
        colors = [f"<color-{i}>" for i in range(len(color_index))]
        fonts = [f"<{code[:2]}-font-{font_index[code]}>" for code in font_index]
        return cls(colors + fonts)

    def encode(self, text: str, add_eos: bool = True) -> List[int]:
        ids: List[int] = []
        i = 0
        while i < len(text):
            hit = next((t for t in self._by_len if text.startswith(t, i)), None) if text[i] == "<" and self.extra else None
            if hit:
                ids.append(self.extra[hit])
                i += len(hit)
            else:
                ids += [b + 3 for b in text[i].encode("utf-8")]
                i += 1
        return ids + ([self.eos_id] if add_eos else [])

    def decode(self, ids: Sequence[int]) -> str:
        inv = {v: k for k, v in self.extra.items()}
        out, buf = "", bytearray()
        for t in ids:
            t = int(t)
            if 3 <= t < 259:
                buf.append(t - 3)
                continue
            out += buf.decode("utf-8", errors="ignore")
            buf = bytearray()
            out += inv.get(t, "")
        return out + buf.decode("utf-8", errors="ignore")

    def __call__(self, text: str, max_length: int) -> Tuple[torch.Tensor, torch.Tensor]:
        e = self.encode(text)[:max_length]
        ids = torch.full((1, max_length), self.pad_id, dtype=torch.long)
        mask = torch.zeros(1, max_length, dtype=torch.long)
        ids[0, : len(e)] = torch.tensor(e, dtype=torch.long)
        mask[0, : len(e)] = 1
        return ids, mask


@dataclass
class GlyphEncoderConfig:
    d_model: int = 1472             # ByT5-small
    d_kv: int = 64
    d_ff: int = 3584
    num_layers: int = 12
    num_heads: int = 6
    vocab_size: int = 1510          # byte vocabulary + colour and font tokens
    max_length: int = 256

    @classmethod
    def tiny(cls, **kw):
        return cls(**{**dict(d_model=32, d_kv=8, d_ff=64, num_layers=1, num_heads=4, vocab_size=400, max_length=24), **kw})


@model_register.register("hunyuan15_glyph_encoder")
class GlyphByT5Encoder(nn.Module):
    config_class = GlyphEncoderConfig

    def __init__(self, config: GlyphEncoderConfig = None, tokenizer: Optional[ByteTokenizer] = None):
        super().__init__()
        c = self.config = config or GlyphEncoderConfig()
        self.t5 = T5Encoder(T5Config(vocab_size=c.vocab_size, d_model=c.d_model, d_kv=c.d_kv, d_ff=c.d_ff,
                                     num_layers=c.num_layers, num_heads=c.num_heads, per_layer_bias=False, gated=True))
        self.tokenizer = tokenizer or ByteTokenizer()
        for p in self.parameters():
            p.requires_grad_(False)

    def tokenize(self, prompt: str, styles=None, color_index=None, font_index=None):
        """-> (ids [1, max_length], mask); all zeros when the prompt quotes nothing."""
        texts = extract_glyph_texts(prompt)
        L = self.config.max_length
        if not texts:
            return torch.zeros(1, L, dtype=torch.long), torch.zeros(1, L, dtype=torch.long)
        return self.tokenizer(format_glyph_prompt(texts, styles, color_index, font_index), L)

    @torch.no_grad()
    def encode(self, input_ids, attention_mask=None):
        mask = attention_mask if attention_mask is not None else (input_ids != 0).long()
        out = torch.zeros(*input_ids.shape, self.config.d_model, device=input_ids.device, dtype=self.t5.embed.weight.dtype)
        live = mask.sum(1) > 0
        if bool(live.any()):
            out[live] = self.t5(input_ids[live], mask[live])
        return out, mask

    def encode_prompts(self, prompts: Sequence[str], **kw):
        pairs = [self.tokenize(p, **kw) for p in prompts]
        dev = self.t5.embed.weight.device
        return self.encode(torch.cat([p[0] for p in pairs]).to(dev), torch.cat([p[1] for p in pairs]).to(dev))


# ------------------------------------------------------------------------------------------------ StepVideo text encoder
def alibi_slopes(n_heads: int) -> torch.Tensor:
    """Geometric slopes 2^(-8 i / n) for the largest power of two n <= heads, the rest interleaved from the 2n series."""
    import math
    n = 2 ** math.floor(math.log2(n_heads))
    s = torch.pow(torch.tensor(2.0 ** (-8.0 / n)), torch.arange(1, n + 1, dtype=torch.float32))
    if n < n_heads:
        extra = torch.pow(torch.tensor(2.0 ** (-4.0 / n)), torch.arange(1, 1 + 2 * (n_heads - n), 2, dtype=torch.float32))
        s = torch.cat([s, extra])
    return s


def sqrt_alibi_bias(seq_len: int, n_heads: int) -> torch.Tensor:
    """[heads, L, L] additive causal bias: ``-slope_h * sqrt(i - j)`` for j <= i, -inf above the diagonal."""
    i = torch.arange(seq_len)
    dist = (i[:, None] - i[None, :]).clamp(min=0).float().sqrt()
    bias = -dist[None] * alibi_slopes(n_heads).view(-1, 1, 1)
    return bias.masked_fill(i[None, :] > i[:, None], float("-inf"))


@dataclass
class StepLLMConfig:
    """Sizes come from the checkpoint's ``config.json`` (the reference reads them there too); the defaults only fix the
    field names and a plausible shape."""
    hidden_size: int = 6144
    num_attention_heads: int = 48
    num_attention_groups: int = 8
    num_layers: int = 48
    ffn_hidden_size: int = 16896
    vocab_size: int = 65536
    eps: float = 1e-5
    ffn_multiple_of: int = 256

    @classmethod
    def tiny(cls, **kw):
        return cls(**{**dict(hidden_size=96, num_attention_heads=6, num_attention_groups=2, num_layers=2, ffn_hidden_size=100,
                             vocab_size=128, ffn_multiple_of=16), **kw})


class _StepBlock(nn.Module):
    def __init__(self, c: StepLLMConfig):
        super().__init__()
        self.h, self.g, self.d = c.num_attention_heads, c.num_attention_groups, c.hidden_size // c.num_attention_heads
        ff = (c.ffn_hidden_size + c.ffn_multiple_of - 1) // c.ffn_multiple_of * c.ffn_multiple_of
        self.attention_norm = nn.Parameter(torch.ones(c.hidden_size))
        self.ffn_norm = nn.Parameter(torch.ones(c.hidden_size))
        self.wqkv = nn.Linear(c.hidden_size, c.hidden_size + 2 * self.d * self.g, bias=False)
        self.wo = nn.Linear(c.hidden_size, c.hidden_size, bias=False)
        self.w1 = nn.Linear(c.hidden_size, 2 * ff, bias=False)
        self.w2 = nn.Linear(ff, c.hidden_size, bias=False)
        self.eps = c.eps

    def forward(self, x, bias):
        from .. import ops
        B, L, H = x.shape
        q, kv = self.wqkv(ops.rms_norm(x, self.attention_norm, self.eps)).split([H, 2 * self.d * self.g], -1)
        k, v = kv.view(B, L, self.g, 2 * self.d).chunk(2, -1)
        rep = self.h // self.g
        q = q.view(B, L, self.h, self.d).transpose(1, 2)
        k = k.repeat_interleave(rep, 2).transpose(1, 2)
        v = v.repeat_interleave(rep, 2).transpose(1, 2)
        a = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=bias.to(q.dtype))
        x = x + self.wo(a.transpose(1, 2).reshape(B, L, H))
        g, u = self.w1(ops.rms_norm(x, self.ffn_norm, self.eps)).chunk(2, -1)
        return x + self.w2(torch.nn.functional.silu(g) * u)


@model_register.register("stepllm")
class StepLLMEncoder(nn.Module):
    """Decoder-only prompt encoder of StepVideo: no rotary or learned positions -- order comes from a causal bias that
    grows with the square root of the distance -- grouped-query attention, SwiGLU feed-forward, RMSNorm; the output is the
    last block's hidden state without a final norm (mindspeed_mm/models/text_encoder/stepllm_text_encoder.py:36-272)."""
    config_class = StepLLMConfig

    def __init__(self, config: StepLLMConfig = None):
        super().__init__()
        c = self.config = config or StepLLMConfig()
        self.tok_embeddings = nn.Embedding(c.vocab_size, c.hidden_size)
        self.layers = nn.ModuleList(_StepBlock(c) for _ in range(c.num_layers))
        for p in self.parameters():
            p.requires_grad_(False)

    def forward(self, input_ids, attention_mask=None):
        x = self.tok_embeddings(input_ids)
        bias = sqrt_alibi_bias(input_ids.shape[1], self.config.num_attention_heads).to(x.device)[None]
        for blk in self.layers:
            x = blk(x, bias)
        return x

    @torch.no_grad()
    def encode(self, input_ids, attention_mask=None):
        h = self(input_ids, attention_mask)
        return h, (attention_mask if attention_mask is not None else torch.ones_like(input_ids))
