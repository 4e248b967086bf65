"""Synthetic packed VLM dataset for the reference trainer, registered through the reference's own
``data_register`` (mindspeed_mm/fsdp/data/__init__.py:9-34 resolves ``dataset_type`` by that registry).

Every item is one whole packed micro-batch of the benchmark shape: ``samples`` sequences of ``seq_len / samples``
tokens, each holding ``images`` square images of ``image_size`` pixels (448 -> 1024 patches -> 256 placeholder
tokens), concatenated to [1, seq_len].  ``position_ids`` is [4, 1, seq_len]: row 0 restarts at every packed
sequence (this is what makes the Hugging Face flash-attention path run variable-length attention), rows 1-3 are the
multimodal rotary positions.  Labels mask the image placeholders.

The dataset also carries the clock of the reference arm: ``PROBE`` records a CUDA event every time the trainer
fetches a batch (= the start of an iteration of the reference's own loop), and decides whether a batch is served
from device memory (kernel-only region) or from pinned host memory (end-to-end region).
"""
from __future__ import annotations

import os

import torch
from torch.utils.data import Dataset

from mindspeed_mm.fsdp.utils.register import data_register

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


class Probe:
    """Fetch counter + CUDA events.  ``plan(warmup, steps)`` lays out the fetch numbers:
    [0, W) warm-up from device memory, [W, W+K) timed from device memory, W+K one warm-up from host memory,
    [W+K+1, W+2K+1) timed from host memory, W+2K+1 closes the last region (that iteration is not timed)."""

    def __init__(self):
        self.n = 0
        self.marks = {}
        self.events = {}
        self.on_mark = {}

    def plan(self, warmup: int, steps: int):
        w, k = warmup, steps
        self.marks = {w: "dev0", w + k: "dev1", w + k + 1: "e2e0", w + 2 * k + 1: "e2e1"}
        self.first_host_fetch = w + k
        self.total_fetches = w + 2 * k + 2

    def fetch(self) -> bool:
        """Called at the start of every batch fetch; returns True when the batch must come from host memory."""
        name = self.marks.get(self.n)
        if name is not None:
            if torch.cuda.is_available():
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                self.events[name] = ev
            else:
                import time
                self.events[name] = time.perf_counter()
            cb = self.on_mark.get(name)
            if cb is not None:
                cb()
        host = self.n >= getattr(self, "first_host_fetch", 0)
        self.n += 1
        return host

    def elapsed_ms(self, a: str, b: str) -> float:
        ea, eb = self.events[a], self.events[b]
        if isinstance(ea, float):
            return (eb - ea) * 1e3
        return ea.elapsed_time(eb)


PROBE = Probe()


def _patchify(img, patch=14, temporal=2, merge=2):
    c, h, w = img.shape
    mean = torch.tensor(CLIP_MEAN).view(3, 1, 1)
    std = torch.tensor(CLIP_STD).view(3, 1, 1)
    x = ((img - mean) / std).unsqueeze(0).repeat(temporal, 1, 1, 1)
    gh, gw = h // patch, w // patch
    x = x.view(1, temporal, c, gh // merge, merge, patch, gw // merge, merge, patch)
    x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)
    return x.reshape(gh * gw, c * temporal * patch * patch)


def _mrope_positions(ids, image_token_id, grid_hw_merged):
    """[3, T] multimodal rotary positions of one sequence: text advances all axes; an image block holds t = 0 and
    its (h, w) grid, offset by the position where it starts; text resumes at max + 1."""
    t_len = ids.numel()
    pos = torch.zeros(3, t_len, dtype=torch.long)
    gh, gw = grid_hw_merged
    n_img = gh * gw
    hh = torch.arange(gh).view(-1, 1).expand(gh, gw).reshape(-1)
    ww = torch.arange(gw).view(1, -1).expand(gh, gw).reshape(-1)
    i, nxt = 0, 0
    is_img = (ids == image_token_id).tolist()
    while i < t_len:
        if is_img[i]:
            pos[0, i:i + n_img] = nxt
            pos[1, i:i + n_img] = nxt + hh
            pos[2, i:i + n_img] = nxt + ww
            nxt = nxt + max(gh, gw)
            i += n_img
        else:
            j = i
            while j < t_len and not is_img[j]:
                j += 1
            pos[:, i:j] = nxt + torch.arange(j - i)
            nxt += j - i
            i = j
    return pos


@data_register.register("synthetic_packed_vlm")
class SyntheticPackedVLM(Dataset):
    def __init__(self, basic_param=None, preprocess_param=None, dataset_param=None, **_):
        env = os.environ
        self.seq_len = int(env.get("MM_REF_SEQ_LEN", "8192"))
        self.samples = int(env.get("MM_REF_SAMPLES", "4"))
        self.images = int(env.get("MM_REF_IMAGES", "2"))
        self.image_size = int(env.get("MM_REF_IMAGE_SIZE", "448"))
        self.vocab = int(env.get("MM_REF_VOCAB", "152064"))
        self.image_token_id = int(env.get("MM_REF_IMAGE_TOKEN", "151655"))
        self.vision_start_id = int(env.get("MM_REF_VISION_START", "151652"))
        self.seed = 1234 + int(env.get("RANK", "0"))
        self.n_distinct = 4
        # built up front, so that no timed fetch pays for generating or uploading a batch
        self._host = {w: self._build(w) for w in range(self.n_distinct)}
        self._dev = {}
        if torch.cuda.is_available():
            self._dev = {w: {k: v.cuda() for k, v in b.items()} for w, b in self._host.items()}

    def __len__(self):
        return 1 << 20

    def _sample(self, g):
        per = self.seq_len // self.samples
        grid = self.image_size // 14
        vis = grid * grid // 4
        n_text = per - self.images * (vis + 1)
        text = torch.randint(0, min(self.vocab, self.vision_start_id) - 1, (n_text,), generator=g)
        cuts = sorted(torch.randint(0, n_text + 1, (self.images,), generator=g).tolist())
        block = torch.cat([torch.tensor([self.vision_start_id]), torch.full((vis,), self.image_token_id)])
        pieces, prev = [], 0
        for c in cuts:
            pieces += [text[prev:c], block]
            prev = c
        pieces.append(text[prev:])
        ids = torch.cat(pieces)
        labels = ids.clone()
        labels[(ids == self.image_token_id) | (ids == self.vision_start_id)] = -100
        imgs = torch.rand(self.images, 3, self.image_size, self.image_size, generator=g)
        pix = torch.cat([_patchify(im) for im in imgs])
        thw = torch.tensor([[1, grid, grid]] * self.images, dtype=torch.long)
        pos = _mrope_positions(ids, self.image_token_id, (grid // 2, grid // 2))
        return ids, labels, pix, thw, pos

    def _build(self, which):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + which)
        parts = [self._sample(g) for _ in range(self.samples)]
        ids = torch.cat([p[0] for p in parts]).unsqueeze(0)
        labels = torch.cat([p[1] for p in parts]).unsqueeze(0)
        pix = torch.cat([p[2] for p in parts]).to(torch.bfloat16)
        thw = torch.cat([p[3] for p in parts])
        text_pos = torch.cat([torch.arange(p[0].numel()) for p in parts])
        pos = torch.cat([text_pos.unsqueeze(0), torch.cat([p[4] for p in parts], dim=1)]).unsqueeze(1)
        batch = dict(input_ids=ids, labels=labels, position_ids=pos, pixel_values=pix, image_grid_thw=thw)
        if torch.cuda.is_available():
            batch = {k: v.pin_memory() for k, v in batch.items()}
        return batch

    def __getitem__(self, i):
        return i % self.n_distinct

    def nbytes(self):
        return sum(v.numel() * v.element_size() for v in self._host[0].values())

    def collate_fn(self, items):
        """The trainer's fetch: one packed micro-batch.  Host batches are pinned CPU tensors (the trainer's
        ``move_to_device`` copies them every step); device batches are already resident."""
        which = PROBE.n % self.n_distinct
        host = PROBE.fetch()
        if host or not self._dev:
            return dict(self._host[which])
        return dict(self._dev[which])
