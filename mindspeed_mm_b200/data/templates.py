"""Chat templates by name (``preprocess_parameters.template_name`` / ``template`` in a data recipe).

A template says how a conversation is laid out as text around the turns and how media markers expand:
``prefix`` once, then per turn ``system`` / ``user`` / ``assistant`` / ``observation`` slots with ``{content}``.  The user slot ends
with the assistant header, so an assistant slot is exactly what the model has to produce and is what the labels
supervise (everything else is ``ignore_index``).  Names and slot texts follow the reference's registry
(mindspeed_mm/data/data_utils/func_utils/template.py:326-505); ``{eos}`` stands for the tokenizer's end-of-sequence token.
Media: every ``<image>`` / ``<video>`` / ``<audio>`` marker becomes ``start + pad * n + end`` with the family's token names
(``n`` comes from the processor: merged patches of that item).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

_CHATML = dict(system="<|im_start|>system\n{content}<|im_end|>\n",
               user="<|im_start|>user\n{content}<|im_end|>\n<|im_start|>assistant\n",
               assistant="{content}<|im_end|>\n",
               observation="<|im_start|>tool\n{content}<|im_end|>\n<|im_start|>assistant\n")


@dataclass
class TemplateSpec:
    name: str
    prefix: str = ""
    system: str = "{content}"
    user: str = "{content}"
    assistant: str = "{content}{eos}"
    observation: Optional[str] = None
    default_system: str = ""
    stop_words: Sequence[str] = ()
    replace_eos: bool = False            # the first stop word becomes the tokenizer's eos
    efficient_eos: bool = False          # no eos after assistant turns (the next turn's header ends them)
    thought_words: Tuple[str, str] = ("<think>", "</think>")
    enable_thinking: Optional[bool] = True      # False: an empty thought block is put in front of every answer
    # media expansion: (start, pad, end) token texts per kind
    media: Dict[str, Tuple[str, str, str]] = field(default_factory=lambda: {
        "image": ("<|vision_start|>", "<|image_pad|>", "<|vision_end|>"),
        "video": ("<|vision_start|>", "<|video_pad|>", "<|vision_end|>")})


TEMPLATES: Dict[str, TemplateSpec] = {}


def register_template(spec: TemplateSpec) -> TemplateSpec:
    TEMPLATES[spec.name] = spec
    return spec


_QWEN_OMNI_MEDIA = {"image": ("<|vision_start|>", "<|image_pad|>", "<|vision_end|>"),
                    "video": ("<|vision_start|>", "<|video_pad|>", "<|vision_end|>"),
                    "audio": ("<|audio_start|>", "<|audio_pad|>", "<|audio_end|>")}
_GLM_MEDIA = {"image": ("<|begin_of_image|>", "<|image|>", "<|end_of_image|>"),
              "video": ("<|begin_of_video|>", "<|video|>", "<|end_of_video|>")}

register_template(TemplateSpec("qwen2vl", **_CHATML, default_system="You are a helpful assistant.", stop_words=("<|im_end|>",),
                               replace_eos=True))
register_template(TemplateSpec("qwen2_5_vl", **_CHATML, default_system="You are a helpful assistant.", stop_words=("<|im_end|>",),
                               replace_eos=True))
register_template(TemplateSpec("qwen3_vl", **_CHATML, stop_words=("<|im_end|>",), replace_eos=True))
register_template(TemplateSpec("qwen3_vl_nothink", **_CHATML, stop_words=("<|im_end|>",), replace_eos=True, enable_thinking=False))
register_template(TemplateSpec("qwen3_5", **_CHATML, stop_words=("<|im_end|>",), replace_eos=True))
register_template(TemplateSpec("qwen2_omni", **_CHATML, default_system="You are a helpful assistant.", stop_words=("<|im_end|>",),
                               replace_eos=True, media={"image": ("<|vision_bos|>", "<|IMAGE|>", "<|vision_eos|>"),
                                                        "video": ("<|vision_bos|>", "<|VIDEO|>", "<|vision_eos|>"),
                                                        "audio": ("<|audio_bos|>", "<|AUDIO|>", "<|audio_eos|>")}))
register_template(TemplateSpec("qwen3_omni", **_CHATML, stop_words=("<|im_end|>",), replace_eos=True, media=_QWEN_OMNI_MEDIA))
register_template(TemplateSpec("qwen3_omni_nothink", **_CHATML, stop_words=("<|im_end|>",), replace_eos=True, enable_thinking=False,
                               media=_QWEN_OMNI_MEDIA))
for _n in ("glm4.1v", "glm4v_moe"):
    register_template(TemplateSpec(_n, prefix="[gMASK]<sop>", system="<|system|>\n{content}", user="<|user|>\n{content}<|assistant|>",
                                   assistant="\n{content}", observation="<|observation|>\n{content}<|assistant|>",
                                   stop_words=("<|user|>", "<|observation|>", "</answer>"), efficient_eos=True, media=_GLM_MEDIA))
register_template(TemplateSpec("mistral", prefix="{bos}", system="[SYSTEM_PROMPT]{content}[/SYSTEM_PROMPT]", user="[INST]{content}[/INST]",
                               assistant="{content}{eos}", observation='[TOOL_RESULTS]{{"content": {content}}}[/TOOL_RESULTS]',
                               media={"image": ("", "[IMG]", "[IMG_END]")}))
for _n in ("internvl", "internvl2_5", "internvl3_5"):
    register_template(TemplateSpec(_n, **_CHATML, default_system="你是书生·万象，英文名是InternVL，是由上海人工智能实验室、清华大学及多家合作单位联合开发的多模态大语言模型。",
                                   stop_words=("<|im_end|>",), replace_eos=True,
                                   media={"image": ("<img>", "<IMG_CONTEXT>", "</img>"), "video": ("<img>", "<IMG_CONTEXT>", "</img>")}))
register_template(TemplateSpec("llava", system="{content} ", user="USER: {content} ASSISTANT:", assistant=" {content}{eos}",
                               default_system="A chat between a curious human and an artificial intelligence assistant. The assistant "
                                              "gives helpful, detailed, and polite answers to the human's questions.",
                               media={"image": ("", "<image>", ""), "video": ("", "<video>", "")}))
register_template(TemplateSpec("deepseek_vl2", user="<|User|>: {content}\n\n<|Assistant|>:", assistant=" {content}{eos}",
                               system="{content}\n\n", media={"image": ("", "<image>", "")}))
register_template(TemplateSpec("gemma", prefix="{bos}", user="<start_of_turn>user\n{content}<end_of_turn>\n<start_of_turn>model\n",
                               assistant="{content}<end_of_turn>\n", system="{content}\n\n", efficient_eos=True,
                               media={"image": ("<start_of_image>", "<image_soft_token>", "<end_of_image>")}))
register_template(TemplateSpec("default", system="System: {content}{eos}\n", user="Human: {content}{eos}\nAssistant:",
                               assistant="{content}{eos}\n"))


class TemplateRenderer:
    """Renders ``messages`` to token ids and labels with a ``TemplateSpec``.  ``tokenizer`` needs ``encode(text) -> ids`` and
    ``convert_tokens_to_ids`` (or a ``special_ids`` table) for the media tokens; pad ids may also be passed explicitly."""

    MARKERS = {"<image>": "image", "<video>": "video", "<audio>": "audio"}

    def __init__(self, spec: TemplateSpec, tokenizer, media_ids: Optional[Dict[str, Tuple[Optional[int], int, Optional[int]]]] = None):
        self.spec, self.tok = spec, tokenizer
        self.eos = getattr(tokenizer, "eos_token", None) or (spec.stop_words[0] if spec.stop_words else "")
        self.bos = getattr(tokenizer, "bos_token", None) or ""
        if media_ids is None:          # kinds whose tokens this tokenizer lacks stay out: their markers are then plain text
            media_ids = {}
            for kind, toks in spec.media.items():
                try:
                    media_ids[kind] = tuple(self._id(t) if t else None for t in toks)
                except KeyError:
                    pass
        self.media_ids = media_ids

    # the attributes the conversation dataset reads when it trims a sample to the cut-off length
    @property
    def image_token_id(self):
        return self.media_ids.get("image", (None, None, None))[1]

    @property
    def video_token_id(self):
        return self.media_ids.get("video", self.media_ids.get("image", (None, None, None)))[1]

    @property
    def vs(self):
        return self.media_ids.get("image", (None, None, None))[0]

    def _id(self, token: str) -> Optional[int]:
        table = getattr(self.tok, "special_ids", None)
        if table is not None and token in table:
            return table[token]
        conv = getattr(self.tok, "convert_tokens_to_ids", None)
        if conv is not None:
            i = conv(token)
            if i is not None and i != getattr(self.tok, "unk_token_id", None):
                return i
        raise KeyError(f"tokenizer has no id for the media token {token!r} of template {self.spec.name}")

    def _enc(self, text: str) -> List[int]:
        if not text:
            return []
        try:
            return list(self.tok.encode(text, add_special_tokens=False))
        except TypeError:
            return list(self.tok.encode(text))

    def _fill(self, slot: str, content: str) -> str:
        return slot.replace("{eos}", self.eos).replace("{bos}", self.bos).replace("{{", "{").replace("}}", "}").replace("{content}", content)

    def _expand(self, text: str, counts: List[int], kinds: List[str]) -> List[int]:
        """Token ids of ``text`` with each media marker replaced by start + n pads + end."""
        ids: List[int] = []
        rest = text
        while True:
            hits = [(rest.find(m), m) for m in self.MARKERS if rest.find(m) >= 0 and self.MARKERS[m] in self.media_ids]
            if not hits:
                return ids + self._enc(rest)
            at, marker = min(hits)
            ids += self._enc(rest[:at])
            if not counts:
                raise ValueError("more media markers in the text than media items in the sample")
            n = counts.pop(0)
            kinds.pop(0)
            start, pad, end = self.media_ids[self.MARKERS[marker]]
            ids += ([start] if start is not None else []) + [pad] * n + ([end] if end is not None else [])
            rest = rest[at + len(marker):]

    def render(self, messages: List[Dict[str, str]], media_tokens: Sequence[int] = (), media_kinds: Sequence[str] = (),
               ignore_index: int = -100) -> Tuple[List[int], List[int]]:
        sp = self.spec
        counts, kinds = list(media_tokens), list(media_kinds)
        msgs = list(messages)
        if msgs and msgs[0]["role"] != "system" and sp.default_system:
            msgs = [{"role": "system", "content": sp.default_system}] + msgs
        ids = self._enc(self._fill(sp.prefix, ""))
        labels = [ignore_index] * len(ids)
        for m in msgs:
            role, content = m["role"], m["content"]
            if role == "assistant":
                if sp.enable_thinking is False and sp.thought_words[0] not in content:
                    content = f"{sp.thought_words[0]}\n\n{sp.thought_words[1]}\n\n" + content
                slot = sp.assistant.replace("{eos}", "") if sp.efficient_eos else sp.assistant
                part = self._expand(self._fill(slot, content), counts, kinds)
                ids += part
                labels += part
                continue
            slot = {"system": sp.system, "user": sp.user, "observation": sp.observation or sp.user, "tool": sp.observation or sp.user}.get(role)
            if slot is None:
                raise ValueError(f"unknown role {role!r}")
            part = self._expand(self._fill(slot, content), counts, kinds)
            ids += part
            labels += [ignore_index] * len(part)
        if counts:
            raise ValueError("sample lists more media items than markers in its text")
        return ids, labels


def get_template(name: str, tokenizer, media_ids=None) -> TemplateRenderer:
    if name not in TEMPLATES:
        raise ValueError(f"Template {name} does not exist (known: {sorted(TEMPLATES)})")
    return TemplateRenderer(TEMPLATES[name], tokenizer, media_ids)
