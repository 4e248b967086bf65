"""File-backed datasets: multimodal conversations (images / video + chat) and pre-extracted DiT features.

* ``Qwen2VLImageProcessor`` -- ``smart_resize`` to a multiple of ``patch * merge`` within ``[min_pixels, max_pixels]``,
  bicubic resize, CLIP normalisation and flattening into ``[grid_h * grid_w, 3 * temporal * patch * patch]`` rows in
  2x2-merge order (the layout of the HF Qwen2-VL processor the reference calls through its mm_plugin:
  mindspeed_mm/data/data_utils/func_utils/mm_plugin.py, ``Qwen2vlPlugin``).
* ``ChatTemplate`` -- ChatML rendering with ``<|vision_start|><|image_pad|>*N<|vision_end|>`` expansion and label
  masking of everything but the assistant turns (mindspeed_mm/data/data_utils/func_utils/template.py, convert.py).
* ``MultimodalConversationDataset`` (``dataset_type: huggingface`` / ``multimodal``) -- reads ``.json`` / ``.jsonl`` in
  the sharegpt layout ``{"messages": [{"role", "content"}], "images": [...], "videos": [...]}`` (also
  ``conversations`` with ``from / value``), loads media relative to ``dataset_dir``, truncates to ``cutoff_len``
  (mindspeed_mm/data/datasets/qwen2vl_dataset.py:37-192).
* ``FeatureDataset`` -- ``.pt`` files with ``latents`` / ``prompt`` (+ masks) listed by a json / jsonl / txt index
  (mindspeed_mm/data/datasets/feature_dataset.py:29).
* ``read_video_frames`` -- uniform frame sampling through OpenCV (mindspeed_mm/data/data_utils/video_reader.py).
"""
from __future__ import annotations

import json
import math
import os
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
from torch.utils.data import Dataset

from ..models.registry import data_register
from .synthetic import CLIP_MEAN, CLIP_STD


# ------------------------------------------------------------------------------------------ image processor
def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56,
                 max_pixels: int = 14 * 14 * 4 * 1280) -> Tuple[int, int]:
    """Closest size with both sides divisible by ``factor``, area inside the pixel budget, aspect ratio kept."""
    if max(height, width) / min(height, width) > 200:
        raise ValueError(f"aspect ratio of {height}x{width} exceeds 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


class Qwen2VLImageProcessor:
    def __init__(self, patch_size: int = 14, temporal_patch_size: int = 2, merge_size: int = 2,
                 min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280,
                 mean: Sequence[float] = CLIP_MEAN, std: Sequence[float] = CLIP_STD):
        self.patch, self.temporal, self.merge = patch_size, temporal_patch_size, merge_size
        self.min_pixels, self.max_pixels = min_pixels, max_pixels
        self.mean = torch.tensor(mean).view(1, 3, 1, 1)
        self.std = torch.tensor(std).view(1, 3, 1, 1)

    def _to_tensor(self, img) -> torch.Tensor:
        """PIL image / uint8 HWC array / float CHW tensor -> float [3, H, W] in [0, 1]."""
        if isinstance(img, torch.Tensor):
            t = img
            if t.dtype == torch.uint8:
                t = t.float() / 255.0
            return t if t.shape[0] == 3 else t.permute(2, 0, 1)
        import numpy as np
        arr = np.asarray(img.convert("RGB") if hasattr(img, "convert") else img)
        return torch.from_numpy(arr.copy()).permute(2, 0, 1).float() / 255.0

    def frames(self, frames: torch.Tensor) -> Tuple[torch.Tensor, Tuple[int, int, int]]:
        """frames [T, 3, H, W] in [0,1] -> (patch rows, (grid_t, grid_h, grid_w))."""
        T, _, H, W = frames.shape
        h, w = smart_resize(H, W, self.patch * self.merge, self.min_pixels, self.max_pixels)
        x = torch.nn.functional.interpolate(frames, size=(h, w), mode="bicubic", align_corners=False, antialias=True)
        x = ((x.clamp(0, 1) - self.mean) / self.std)
        if T % self.temporal:
            x = torch.cat([x, x[-1:].repeat(self.temporal - T % self.temporal, 1, 1, 1)], 0)
        gt, gh, gw = x.shape[0] // self.temporal, h // self.patch, w // self.patch
        m, p = self.merge, self.patch
        x = x.view(gt, self.temporal, 3, gh // m, m, p, gw // m, m, p)
        x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)
        return x.reshape(gt * gh * gw, 3 * self.temporal * p * p), (gt, gh, gw)

    def __call__(self, img) -> Tuple[torch.Tensor, Tuple[int, int, int]]:
        if hasattr(img, "resize") and hasattr(img, "size"):      # PIL: resize on uint8 as the HF processor does
            from PIL import Image
            img = img.convert("RGB")
            h, w = smart_resize(img.size[1], img.size[0], self.patch * self.merge, self.min_pixels, self.max_pixels)
            img = img.resize((w, h), resample=Image.BICUBIC)
        return self.frames(self._to_tensor(img)[None])


def read_video_frames(path: str, num_frames: int = 8, fps: Optional[float] = None) -> torch.Tensor:
    """Uniformly sampled frames [T, 3, H, W] in [0, 1] (``fps`` given: one frame every 1/fps seconds, capped)."""
    import cv2
    cap = cv2.VideoCapture(path)
    if not cap.isOpened():
        raise IOError(f"cannot open video {path}")
    total = int(cap.get(cv2.CAP_PROP_FRAME_COUNT))
    native = cap.get(cv2.CAP_PROP_FPS) or 25.0
    n = num_frames if fps is None else max(1, min(num_frames, int(total / native * fps)))
    want = set(torch.linspace(0, max(total - 1, 0), n).round().long().tolist())
    out, i = [], 0
    while True:
        ok, frame = cap.read()
        if not ok:
            break
        if i in want:
            out.append(torch.from_numpy(cv2.cvtColor(frame, cv2.COLOR_BGR2RGB)).permute(2, 0, 1).float() / 255.0)
        i += 1
    cap.release()
    if not out:
        raise IOError(f"no frames decoded from {path}")
    return torch.stack(out)


# ------------------------------------------------------------------------------------------ chat template
class ChatTemplate:
    """ChatML with vision placeholders.  ``tokenizer`` needs ``encode(text) -> ids`` and the special-token ids."""

    IMAGE, VIDEO = "<image>", "<video>"

    def __init__(self, tokenizer, image_token_id: int, video_token_id: Optional[int] = None,
                 vision_start_id: Optional[int] = None, vision_end_id: Optional[int] = None,
                 default_system: str = "You are a helpful assistant."):
        self.tok = tokenizer
        self.image_token_id, self.video_token_id = image_token_id, video_token_id or image_token_id
        self.vs, self.ve = vision_start_id, vision_end_id
        self.system = default_system

    def _enc(self, text: str) -> List[int]:
        if not text:
            return []
        ids = self.tok.encode(text, add_special_tokens=False) if _accepts_special(self.tok) else self.tok.encode(text)
        return list(ids)

    def _content(self, text: str, counts: List[int], kinds: List[str]) -> List[int]:
        """Encode ``text`` replacing each ``<image>`` / ``<video>`` marker by start + N placeholders + end."""
        ids: List[int] = []
        rest = text
        while True:
            pos = [(rest.find(m), m) for m in (self.IMAGE, self.VIDEO) if rest.find(m) >= 0]
            if not pos:
                ids += self._enc(rest)
                return ids
            at, marker = min(pos)
            ids += self._enc(rest[:at])
            if not counts:
                raise ValueError("more media markers in the text than media items in the sample")
            n = counts.pop(0)
            kinds.pop(0)
            pad = self.image_token_id if marker == self.IMAGE else self.video_token_id
            ids += ([self.vs] if self.vs is not None else []) + [pad] * n + ([self.ve] if self.ve is not None else [])
            rest = rest[at + len(marker):]

    def render(self, messages: List[Dict[str, str]], media_tokens: List[int], media_kinds: List[str],
               ignore_index: int = -100) -> Tuple[List[int], List[int]]:
        counts, kinds = list(media_tokens), list(media_kinds)
        ids: List[int] = []
        labels: List[int] = []
        msgs = list(messages)
        if msgs and msgs[0]["role"] != "system" and self.system:
            msgs = [{"role": "system", "content": self.system}] + msgs
        for m in msgs:
            head = self._enc(f"<|im_start|>{m['role']}\n")
            body = self._content(m["content"], counts, kinds) + self._enc("<|im_end|>")
            tail = self._enc("\n")
            ids += head + body + tail
            if m["role"] == "assistant":
                labels += [ignore_index] * len(head) + body + [ignore_index] * len(tail)
            else:
                labels += [ignore_index] * (len(head) + len(body) + len(tail))
        if counts:
            raise ValueError("sample lists more media items than markers in its text")
        return ids, labels


def _accepts_special(tok) -> bool:
    import inspect
    try:
        return "add_special_tokens" in inspect.signature(tok.encode).parameters
    except (TypeError, ValueError):
        return False


class ByteTokenizer:
    """Dependency-free fallback tokenizer (UTF-8 bytes + ChatML specials) for tests and synthetic runs."""

    SPECIALS = ["<|im_start|>", "<|im_end|>", "<|vision_start|>", "<|vision_end|>", "<|image_pad|>", "<|video_pad|>"]

    def __init__(self):
        self.special_ids = {s: 256 + i for i, s in enumerate(self.SPECIALS)}
        self.vocab_size = 256 + len(self.SPECIALS)

    def encode(self, text: str) -> List[int]:
        ids: List[int] = []
        i = 0
        while i < len(text):
            for s, sid in self.special_ids.items():
                if text.startswith(s, i):
                    ids.append(sid)
                    i += len(s)
                    break
            else:
                ids += list(text[i].encode("utf-8"))
                i += 1
        return ids

    def decode(self, ids: Sequence[int]) -> str:
        inv = {v: k for k, v in self.special_ids.items()}
        out, buf = [], bytearray()
        for t in ids:
            if t in inv:
                out.append(buf.decode("utf-8", "replace"))
                buf = bytearray()
                out.append(inv[t])
            else:
                buf.append(t)
        out.append(buf.decode("utf-8", "replace"))
        return "".join(out)


# ------------------------------------------------------------------------------------------ datasets
def _read_records(path: str) -> List[dict]:
    if path.endswith(".jsonl"):
        with open(path) as f:
            return [json.loads(line) for line in f if line.strip()]
    with open(path) as f:
        data = json.load(f)
    return data if isinstance(data, list) else data["data"]


_ROLE = {"human": "user", "user": "user", "gpt": "assistant", "assistant": "assistant", "system": "system",
         "observation": "user", "function_call": "assistant"}


def normalise_messages(rec: dict) -> List[Dict[str, str]]:
    if "messages" in rec:
        return [{"role": _ROLE.get(m["role"], m["role"]), "content": m["content"]} for m in rec["messages"]]
    if "conversations" in rec:
        msgs = [{"role": _ROLE[m["from"]], "content": m["value"]} for m in rec["conversations"]]
        if rec.get("system"):
            msgs = [{"role": "system", "content": rec["system"]}] + msgs
        return msgs
    if "instruction" in rec:          # alpaca layout
        q = rec["instruction"] + ("\n" + rec["input"] if rec.get("input") else "")
        return [{"role": "user", "content": q}, {"role": "assistant", "content": rec.get("output", "")}]
    raise KeyError("record has neither 'messages', 'conversations' nor 'instruction'")


@data_register.register("huggingface")
@data_register.register("multimodal")
class MultimodalConversationDataset(Dataset):
    def __init__(self, dataset_param=None, model=None, *, files: Optional[Sequence[str]] = None, dataset_dir: str = "",
                 tokenizer=None, template: Optional[ChatTemplate] = None, processor: Optional[Qwen2VLImageProcessor] = None,
                 cutoff_len: int = 8192, video_frames: int = 8, image_loader: Optional[Callable] = None):
        if dataset_param is not None:
            basic = dict(getattr(dataset_param, "basic_parameters", None) or {})
            pre = dict(getattr(dataset_param, "preprocess_parameters", None) or {})
            files = files or basic.get("dataset") or basic.get("data_path")
            files = [files] if isinstance(files, str) else list(files)
            dataset_dir = basic.get("dataset_dir", dataset_dir)
            cutoff_len = int(basic.get("cutoff_len", cutoff_len))
            video_frames = int(basic.get("video_max_frames", video_frames))
            if tokenizer is None and pre.get("model_name_or_path") and os.path.exists(pre["model_name_or_path"]):
                from transformers import AutoTokenizer
                tokenizer = AutoTokenizer.from_pretrained(pre["model_name_or_path"])
            if processor is None:
                processor = Qwen2VLImageProcessor(min_pixels=int(pre.get("image_min_pixels", 56 * 56)),
                                                  max_pixels=int(pre.get("image_max_pixels", 14 * 14 * 4 * 1280)))
        self.records: List[dict] = []
        for f in files:
            self.records += _read_records(f if os.path.isabs(f) or not dataset_dir else os.path.join(dataset_dir, f))
        self.dir = dataset_dir
        self.proc = processor or Qwen2VLImageProcessor()
        tok = tokenizer or ByteTokenizer()
        if template is None:
            cfg = getattr(model, "config", None)
            sid = getattr(tok, "special_ids", None)
            if tokenizer is None and cfg is not None and hasattr(cfg, "image_token_id"):
                # stand-in byte tokenizer (no tokenizer files): the placeholder ids are the model's, so that the
                # vision features land where the model looks for them
                template = ChatTemplate(tok, cfg.image_token_id, getattr(cfg, "video_token_id", None),
                                        cfg.vision_start_token_id, getattr(cfg, "vision_end_token_id", None))
            elif sid is not None:
                template = ChatTemplate(tok, sid["<|image_pad|>"], sid["<|video_pad|>"], sid["<|vision_start|>"], sid["<|vision_end|>"])
            elif cfg is not None:
                template = ChatTemplate(tok, cfg.image_token_id, getattr(cfg, "video_token_id", None),
                                        cfg.vision_start_token_id, getattr(cfg, "vision_end_token_id", None))
            else:
                cv = tok.convert_tokens_to_ids
                template = ChatTemplate(tok, cv("<|image_pad|>"), cv("<|video_pad|>"), cv("<|vision_start|>"), cv("<|vision_end|>"))
        name = (pre.get("template") or pre.get("template_name")) if dataset_param is not None else None
        if name and name not in ("qwen2vl", "qwen2_5_vl") and isinstance(template, ChatTemplate):
            # another family's turn layout (``preprocess_parameters.template``) around the same placeholder ids
            from .templates import TEMPLATES, TemplateRenderer
            if name not in TEMPLATES:
                raise ValueError(f"Template {name} does not exist (known: {sorted(TEMPLATES)})")
            t0 = template
            template = TemplateRenderer(TEMPLATES[name], tok, media_ids={"image": (t0.vs, t0.image_token_id, t0.ve),
                                                                        "video": (t0.vs, t0.video_token_id, t0.ve)})
        self.template = template
        self.cutoff, self.video_frames = cutoff_len, video_frames
        self.image_loader = image_loader or self._load_image

    def _path(self, p: str) -> str:
        return p if os.path.isabs(p) or not self.dir else os.path.join(self.dir, p)

    def _load_image(self, p: str):
        from PIL import Image
        return Image.open(self._path(p))

    def __len__(self):
        return len(self.records)

    def lengths(self) -> List[int]:
        """Cheap length estimate (characters / 3 + a nominal media cost) for length-grouped sampling."""
        return [sum(len(m["content"]) for m in normalise_messages(r)) // 3 + 256 * (len(r.get("images", [])) + len(r.get("videos", [])))
                for r in self.records]

    def __getitem__(self, i: int) -> Dict[str, torch.Tensor]:
        rec = self.records[i]
        msgs = normalise_messages(rec)
        rows, grids, kinds = [], [], []
        text = "".join(m["content"] for m in msgs)
        images, videos = list(rec.get("images", [])), list(rec.get("videos", []))
        # media are consumed in the order their markers appear in the text
        order, pos = [], 0
        while True:
            a, b = text.find(ChatTemplate.IMAGE, pos), text.find(ChatTemplate.VIDEO, pos)
            cand = [(x, k) for x, k in ((a, "image"), (b, "video")) if x >= 0]
            if not cand:
                break
            at, k = min(cand)
            order.append(k)
            pos = at + 7
        if len(order) < len(images) + len(videos):       # markers missing: prepend them to the first user turn
            missing_i = len(images) - order.count("image")
            missing_v = len(videos) - order.count("video")
            for m in msgs:
                if m["role"] == "user":
                    m["content"] = ChatTemplate.IMAGE * missing_i + ChatTemplate.VIDEO * missing_v + m["content"]
                    break
            order = ["image"] * missing_i + ["video"] * missing_v + order
        for k in order:
            if k == "image":
                r, g = self.proc(self.image_loader(images.pop(0)))
            else:
                r, g = self.proc.frames(read_video_frames(self._path(videos.pop(0)), self.video_frames))
            rows.append(r)
            grids.append(g)
            kinds.append(k)
        merge2 = self.proc.merge ** 2
        counts = [g[0] * g[1] * g[2] // merge2 for g in grids]
        ids, labels = self.template.render(msgs, counts, kinds)
        if len(ids) > self.cutoff:
            ids, labels = ids[: self.cutoff], labels[: self.cutoff]
            # never cut inside a run of placeholders: drop the media whose placeholders were truncated
            kept = 0
            remaining = sum(1 for t in ids if t in (self.template.image_token_id, self.template.video_token_id))
            while kept < len(counts) and remaining >= counts[kept]:
                remaining -= counts[kept]
                kept += 1
            if remaining:
                cut = len(ids)
                while cut and ids[cut - 1] in (self.template.image_token_id, self.template.video_token_id, self.template.vs):
                    cut -= 1
                ids, labels = ids[:cut], labels[:cut]
            rows, grids = rows[:kept], grids[:kept]
        out = dict(input_ids=torch.tensor(ids, dtype=torch.long), labels=torch.tensor(labels, dtype=torch.long))
        if rows:
            out["pixel_values"] = torch.cat(rows)
            out["image_grid_thw"] = torch.tensor(grids, dtype=torch.long)
        else:
            p = self.proc
            out["pixel_values"] = p.empty() if hasattr(p, "empty") else torch.zeros(0, 3 * p.temporal * p.patch * p.patch)
            out["image_grid_thw"] = torch.zeros(0, 3, dtype=torch.long)
        return out


@data_register.register("feature")
class FeatureDataset(Dataset):
    """Index of ``.pt`` feature files; every file holds a dict with at least ``latents`` and ``prompt``."""

    def __init__(self, dataset_param=None, model=None, *, index: Optional[str] = None, data_folder: str = ""):
        if dataset_param is not None:
            basic = dict(getattr(dataset_param, "basic_parameters", None) or {})
            index = index or basic.get("data_path")
            data_folder = basic.get("data_folder", data_folder)
        self.folder = data_folder
        if index.endswith(".txt"):
            with open(index) as f:
                self.items = [{"file": line.strip()} for line in f if line.strip()]
        else:
            self.items = [r if isinstance(r, dict) else {"file": r} for r in _read_records(index)]

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        f = self.items[i]["file"]
        d = torch.load(f if os.path.isabs(f) or not self.folder else os.path.join(self.folder, f), map_location="cpu",
                       weights_only=True)
        out = {"latents": d["latents"], "prompt": d["prompt"]}
        out["prompt_mask"] = d.get("prompt_mask", torch.ones(d["prompt"].shape[0], dtype=torch.bool))
        for k in ("first_frame_latents", "clip_feature"):
            if k in d:
                out[k] = d[k]
        return out


@data_register.register("t2v")
@data_register.register("i2v")
class VideoTextDataset(Dataset):
    """Raw video (or image) + caption records for generative training without pre-extracted features
    (mindspeed_mm/data/datasets/t2v_dataset.py): ``{"path": ..., "cap": ...}`` in json / jsonl.  Frames are sampled
    uniformly, resized so that the short side covers the target, centre-cropped and scaled to [-1, 1]; the caption
    is tokenised (ids padded to ``text_len``).  The frozen VAE / text encoder of ``SoRAModel`` consume the result."""

    def __init__(self, dataset_param=None, model=None, *, files=None, data_folder: str = "", num_frames: int = 17,
                 height: int = 256, width: int = 256, tokenizer=None, text_len: int = 512):
        if dataset_param is not None:
            basic = dict(getattr(dataset_param, "basic_parameters", None) or {})
            pre = dict(getattr(dataset_param, "preprocess_parameters", None) or {})
            files = files or basic.get("data_path")
            files = [files] if isinstance(files, str) else list(files)
            data_folder = basic.get("data_folder", data_folder)
            num_frames = int(pre.get("num_frames", num_frames))
            height, width = int(pre.get("max_height", height)), int(pre.get("max_width", width))
            text_len = int(pre.get("text_len", text_len))
            tp = (pre.get("tokenizer_config") or {}).get("from_pretrained")
            if tokenizer is None and tp and os.path.exists(tp):
                from transformers import AutoTokenizer
                tokenizer = AutoTokenizer.from_pretrained(tp)
            pipeline = pre.get("train_pipeline")
        else:
            pipeline = None
        # the recipe's own transform list (``preprocess_parameters.train_pipeline``), when it has one
        from .transforms import get_transforms
        box = {"max_height": height, "max_width": width}
        self.video_tf = get_transforms(True, pipeline, transform_size=box) if pipeline and pipeline.get("video") else None
        self.image_tf = get_transforms(False, pipeline, image_size=[height, width]) if pipeline and pipeline.get("image") else None
        self.records: List[dict] = []
        for f in files:
            self.records += _read_records(f)
        self.folder, self.T, self.H, self.W, self.text_len = data_folder, num_frames, height, width, text_len
        self.tok = tokenizer or ByteTokenizer()

    def __len__(self):
        return len(self.records)

    def _frames(self, path: str) -> torch.Tensor:
        p = path if os.path.isabs(path) or not self.folder else os.path.join(self.folder, path)
        is_image = p.lower().endswith((".png", ".jpg", ".jpeg", ".bmp", ".webp"))
        if is_image:
            from PIL import Image
            import numpy as np
            img = Image.open(p).convert("RGB")
            if self.image_tf is not None:
                return self.image_tf(img).unsqueeze(1).contiguous()                  # [3, 1, H, W]
            x = torch.from_numpy(np.asarray(img).copy()).permute(2, 0, 1).float()[None] / 255.0
        else:
            x = read_video_frames(p, self.T)
        if self.video_tf is not None and not is_image:
            x = self.video_tf(x)                                                     # [T, 3, H, W], normalised by the recipe
            if 1 < x.shape[0] < self.T:
                x = torch.cat([x, x[-1:].repeat(self.T - x.shape[0], 1, 1, 1)], 0)
            return x.permute(1, 0, 2, 3).contiguous()
        _, _, h, w = x.shape
        s = max(self.H / h, self.W / w)
        nh, nw = max(self.H, round(h * s)), max(self.W, round(w * s))
        x = torch.nn.functional.interpolate(x, size=(nh, nw), mode="bilinear", align_corners=False, antialias=True)
        top, left = (nh - self.H) // 2, (nw - self.W) // 2
        x = x[:, :, top:top + self.H, left:left + self.W]
        if x.shape[0] < self.T and x.shape[0] > 1:
            x = torch.cat([x, x[-1:].repeat(self.T - x.shape[0], 1, 1, 1)], 0)
        return (x * 2 - 1).permute(1, 0, 2, 3).contiguous()           # [3, T, H, W]

    def __getitem__(self, i):
        r = self.records[i]
        cap = r.get("cap") or r.get("caption") or r.get("text") or ""
        cap = cap[0] if isinstance(cap, list) else cap
        ids = list(self.tok.encode(cap))[: self.text_len]
        mask = [1] * len(ids) + [0] * (self.text_len - len(ids))
        ids = ids + [0] * (self.text_len - len(ids))
        return dict(video=self._frames(r["path"]), prompt_ids=torch.tensor(ids), prompt_mask=torch.tensor(mask))


@data_register.register("dreambooth")
class DreamBoothDataset(VideoTextDataset):
    """Subject fine-tuning data in the layout of the diffusers DreamBooth scripts the reference's examples drive
    (examples/diffusers/{flux,sd3,sdxl}/finetune_*_dreambooth*.sh: ``--instance_data_dir`` + ``--instance_prompt``, optional
    ``--class_data_dir`` + ``--class_prompt`` for prior preservation): every image of ``instance_data_dir`` with the
    instance prompt; with a class folder each item also carries a class image and prompt (``class_video`` /
    ``class_prompt_ids`` / ``class_prompt_mask``), which the trainer weighs by ``prior_loss_weight``.  Items have the fields
    of ``VideoTextDataset`` (an image is a one-frame clip)."""

    EXT = (".png", ".jpg", ".jpeg", ".bmp", ".webp")

    def __init__(self, dataset_param=None, model=None, *, instance_data_dir: str = "", instance_prompt: str = "",
                 class_data_dir: str = "", class_prompt: str = "", repeats: int = 1, **kw):
        if dataset_param is not None:
            basic = dict(getattr(dataset_param, "basic_parameters", None) or {})
            instance_data_dir = basic.get("instance_data_dir", instance_data_dir)
            instance_prompt = basic.get("instance_prompt", instance_prompt)
            class_data_dir = basic.get("class_data_dir", class_data_dir)
            class_prompt = basic.get("class_prompt", class_prompt)
            repeats = int(basic.get("repeats", repeats))
            pre = dict(getattr(dataset_param, "preprocess_parameters", None) or {})
            kw.setdefault("height", int(pre.get("resolution", pre.get("max_height", 1024))))
            kw.setdefault("width", int(pre.get("resolution", pre.get("max_width", 1024))))
            kw.setdefault("text_len", int(pre.get("text_len", 512)))
            tp = (pre.get("tokenizer_config") or {}).get("from_pretrained")
            if kw.get("tokenizer") is None and tp and os.path.exists(tp):
                from transformers import AutoTokenizer
                kw["tokenizer"] = AutoTokenizer.from_pretrained(tp)
        if not instance_data_dir or not os.path.isdir(instance_data_dir):
            raise ValueError(f"instance_data_dir {instance_data_dir!r} is not a directory")
        super().__init__(None, model, files=[], num_frames=1, **kw)
        listing = lambda d: sorted(os.path.join(d, f) for f in os.listdir(d) if f.lower().endswith(self.EXT))
        self.records = [{"path": p, "cap": instance_prompt} for p in listing(instance_data_dir)] * max(1, repeats)
        if not self.records:
            raise ValueError(f"no images under {instance_data_dir}")
        self.class_records = [{"path": p, "cap": class_prompt} for p in listing(class_data_dir)] if class_data_dir else []
        self.folder = ""

    def __getitem__(self, i):
        item = super().__getitem__(i)
        if self.class_records:
            keep, self.records = self.records, self.class_records
            try:
                c = super().__getitem__(i % len(self.class_records))
            finally:
                self.records = keep
            item.update(class_video=c["video"], class_prompt_ids=c["prompt_ids"], class_prompt_mask=c["prompt_mask"])
        return item

