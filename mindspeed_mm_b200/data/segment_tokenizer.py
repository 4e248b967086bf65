"""Tokenising interleaved text / image-code sequences for autoregressive image generation (Lumina-mGPT2 style).

* ``SegmentTokenizer`` -- wraps any tokenizer's ``encode`` so that a text *segment* cut out of a longer text gets the ids it
  would have had inside the full text.  Some tokenizers treat the start of a string as if a space preceded it, others
  need the space spelled out; which one is probed once with a fixed sentence.  For the first kind a segment is encoded
  behind a throw-away prefix character whose ids are then cut off
  (mindspeed_mm/models/text_encoder/lumina_mgpt2_tokenizer.py:14-64).
* ``image_token_ids`` -- a grid of VQ code indices becomes ``<start> <h> <w> row_0 <newline> row_1 <newline> ... <end>``
  with the codes shifted by ``code_offset`` into the text vocabulary (the Chameleon layout the ``lumina_mgpt2`` preset of
  ``models/composable.py`` is trained on; codes come from ``models/ae/kl_vae.py: MOVQ``).
"""
from __future__ import annotations

from typing import Callable, List, Sequence

import torch

_PROBE_PREFIXES = ("@", "\n", "\\", "=", ">", "`")


class SegmentTokenizer:
    def __init__(self, encode: Callable[[str], List[int]], bos_id: int = None, eos_id: int = None):
        self._encode = encode
        self.eos_id = eos_id
        self.bos_id = bos_id if bos_id is not None else eos_id
        full, tail = self.encode("Hi my darling"), self.encode("my darling")
        if full[-len(tail):] == tail:
            self.needs_explicit_space = False
        else:
            spaced = self.encode(" my darling")
            if full[-len(spaced):] != spaced:
                raise ValueError("tokenizer splits neither 'my darling' nor ' my darling' off 'Hi my darling' cleanly")
            self.needs_explicit_space = True

    def encode(self, s: str, bos: bool = False, eos: bool = False) -> List[int]:
        t = list(self._encode(s))
        return ([self.bos_id] if bos else []) + t + ([self.eos_id] if eos else [])

    def encode_segment(self, s: str) -> List[int]:
        """Ids of ``s`` as a continuation (no implicit leading space)."""
        if self.needs_explicit_space:
            return self.encode(s)
        for prefix in _PROBE_PREFIXES:
            p, cat = self.encode(prefix), self.encode(prefix + s)
            if cat[: len(p)] == p:
                return cat[len(p):]
        raise ValueError(f"every probe prefix merges with {s!r} under this tokenizer")


def image_token_ids(codes: torch.Tensor, code_offset: int, start_id: int, end_id: int, newline_id: int,
                    size_token_base: int = None) -> List[int]:
    """codes [h, w] (long).  ``size_token_base`` adds two tokens ``base + h`` and ``base + w`` after the start token."""
    h, w = codes.shape
    ids = [start_id]
    if size_token_base is not None:
        ids += [size_token_base + h, size_token_base + w]
    rows = (codes + code_offset).tolist()
    for r in rows:
        ids += r + [newline_id]
    return ids + [end_id]


def codes_from_token_ids(ids: Sequence[int], code_offset: int, start_id: int, end_id: int, newline_id: int,
                         size_token_base: int = None) -> torch.Tensor:
    """Inverse of ``image_token_ids`` for the first image in ``ids``; rows of unequal length are cut to the shortest."""
    ids = list(ids)
    a = ids.index(start_id) + 1 + (2 if size_token_base is not None else 0)
    b = ids.index(end_id, a)
    rows, cur = [], []
    for t in ids[a:b]:
        if t == newline_id:
            rows.append(cur)
            cur = []
        else:
            cur.append(t - code_offset)
    if cur:
        rows.append(cur)
    w = min(len(r) for r in rows)
    return torch.tensor([r[:w] for r in rows], dtype=torch.long)
