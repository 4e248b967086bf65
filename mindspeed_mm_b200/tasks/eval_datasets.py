"""Benchmark files -> prompts for the understanding benchmarks (MMMU, AI2D, DocVQA / ChartQA style VQA).

The public benchmark dumps are TSV tables with columns ``index, question, A..Z (options), hint, answer, image`` where
``image`` is one base64 picture, a list of them, or the index of another row that holds the picture (reference:
mindspeed_mm/tasks/evaluation/eval_datasets/datasets_base.py:19-103, datasets_mmmu.py:10-79, datasets_ai2d.py:10-47,
datasets_vqa.py).  A prompt is a list of ``{"type": "image" | "text", "value": ...}`` segments; MMMU questions refer to
their pictures as ``<image 1>`` inside the text and are split at those tags so that pictures sit where they are
mentioned.  ``EvalDataset.samples(rank, world)`` yields ``{"index", "messages", "answer", "category"?}`` for
``tasks/evaluation.evaluate``; results are written back as a table with a ``prediction`` column.
"""
from __future__ import annotations

import base64
import csv
import io
import json
import os
import string
import sys
from typing import Dict, Iterator, List, Optional, Sequence

csv.field_size_limit(min(sys.maxsize, 2 ** 31 - 1))


def _blank(v) -> bool:
    return v is None or (isinstance(v, float) and v != v) or (isinstance(v, str) and v.strip() in ("", "nan", "NaN"))


def read_table(path: str) -> List[Dict[str, str]]:
    with open(path, newline="", encoding="utf-8") as f:
        return list(csv.DictReader(f, delimiter="\t" if path.endswith(".tsv") else ","))


def as_list(v):
    """A cell that holds a Python / JSON list literal -> list; anything else -> [cell]."""
    if isinstance(v, (list, tuple)):
        return list(v)
    s = str(v).strip()
    if s.startswith("[") and s.endswith("]"):
        try:
            return list(json.loads(s.replace("'", '"')))
        except json.JSONDecodeError:
            return [x.strip().strip("'\"") for x in s[1:-1].split(",") if x.strip()]
    return [s]


def options_prompt(row: Dict[str, str]) -> str:
    opts = {c: row[c] for c in string.ascii_uppercase if c in row and not _blank(row[c])}
    if not opts:
        return ""
    return "Options:\n" + "".join(f"{k}. {v}\n" for k, v in opts.items()) + \
        "Please select the correct answer from the options above. \n"


def multiple_choice_text(row: Dict[str, str]) -> str:
    text = f"Hint: {row['hint']}\n" if not _blank(row.get("hint")) else ""
    return text + f"Question: {row['question']}\n" + options_prompt(row)


def split_at_image_tags(text: str, images: Sequence) -> List[dict]:
    """``... <image 2> ...`` -> text / image segments in reading order; a text without tags keeps the pictures in front."""
    parts = text.split("<image ")
    if len(parts) == 1:
        return [dict(type="image", value=p) for p in images] + [dict(type="text", value=text)]
    segs = [dict(type="text", value=parts[0])]
    for seg in parts[1:]:
        num, _, rest = seg.partition(">")
        if not num.strip().isdigit():
            raise ValueError(f"malformed image tag '<image {seg[:8]}'")
        segs.append(dict(type="image", value=images[int(num) - 1]))
        segs.append(dict(type="text", value=rest))
    return segs


class EvalDataset:
    kind = "vqa"

    def __init__(self, path: str, image_dir: Optional[str] = None, decode_images: bool = True):
        self.rows = read_table(path)
        self.by_index = {r["index"]: r for r in self.rows if "index" in r}
        self.image_dir = image_dir or os.path.join(os.path.dirname(os.path.abspath(path)), "images")
        self.decode = decode_images

    def __len__(self):
        return len(self.rows)

    # pictures ------------------------------------------------------------------------------------
    def _raw_images(self, row) -> List[str]:
        if not _blank(row.get("image_path")):
            return as_list(row["image_path"])
        cell = row.get("image")
        if _blank(cell):
            return []
        cell = str(cell)
        if len(cell) <= 64 and cell in self.by_index and cell != row.get("index"):     # a pointer to the row with the picture
            return self._raw_images(self.by_index[cell])
        return as_list(cell)

    def images(self, row) -> list:
        out = []
        for k, item in enumerate(self._raw_images(row)):
            if os.path.exists(item) or len(item) < 260 and os.path.exists(os.path.join(self.image_dir, item)):
                out.append(item if os.path.exists(item) else os.path.join(self.image_dir, item))
            elif self.decode:
                from PIL import Image
                out.append(Image.open(io.BytesIO(base64.b64decode(item))).convert("RGB"))
            else:
                out.append(item)
        return out

    # prompts -------------------------------------------------------------------------------------
    def text(self, row) -> str:
        return f"{row['question']}\nAnswer the question using a single word or phrase."

    def messages(self, row) -> List[dict]:
        return [dict(type="image", value=p) for p in self.images(row)] + [dict(type="text", value=self.text(row))]

    def answer(self, row):
        a = row.get("answer", "")
        return as_list(a) if self.kind == "vqa" and str(a).strip().startswith("[") else a

    def samples(self, rank: int = 0, world: int = 1) -> Iterator[dict]:
        for i in range(rank, len(self.rows), world):
            r = self.rows[i]
            s = {"index": r.get("index", str(i)), "messages": self.messages(r), "answer": self.answer(r)}
            if not _blank(r.get("category")):
                s["category"] = r["category"]
            yield s

    # results -------------------------------------------------------------------------------------
    def write_predictions(self, predictions: Dict[str, str], out_path: str) -> None:
        keep = [c for c in self.rows[0] if c != "image"] if self.rows else []
        with open(out_path, "w", newline="", encoding="utf-8") as f:
            w = csv.DictWriter(f, fieldnames=keep + ["prediction"], delimiter="\t")
            w.writeheader()
            for i, r in enumerate(self.rows):
                idx = r.get("index", str(i))
                w.writerow({**{c: r[c] for c in keep}, "prediction": predictions.get(idx, "")})


class AI2DDataset(EvalDataset):
    kind = "multiple_choice"

    def text(self, row) -> str:
        return multiple_choice_text(row)


class MMMUDataset(AI2DDataset):
    def messages(self, row) -> List[dict]:
        return split_at_image_tags(self.text(row), self.images(row))


DATASETS = {"mmmu": MMMUDataset, "mmmu_dev_val": MMMUDataset, "ai2d": AI2DDataset, "ai2d_test": AI2DDataset,
            "vqa": EvalDataset, "docvqa": EvalDataset, "docvqa_val": EvalDataset, "chartqa": EvalDataset,
            "chartqa_test": EvalDataset}
DEFAULT_METRIC = {"multiple_choice": "multiple_choice", "vqa": "anls"}


def build_eval_dataset(name: str, path: str, **kw) -> EvalDataset:
    key = name.lower()
    if key not in DATASETS:
        raise ValueError(f"unknown benchmark {name!r}; known: {sorted(DATASETS)}")
    return DATASETS[key](path, **kw)
