"""Dataset preparation helpers with a command line.

* ``mock``    -- writes one random picture and a JSON of identical long conversations over it, sized by picture count and
  text length: load-test data with the exact format of the real recipes
  (mindspeed_mm/fsdp/tools/data_tool/generate_mock_data_for_vlmodel.py).
* ``llava``   -- LLaVA-instruct records (``image`` + ``conversations`` with human / gpt turns) -> the ``images`` + ``messages``
  layout the conversation dataset reads; records whose picture is missing under the image root are skipped
  (mindspeed_mm/fsdp/tools/data_tool/llava_instruct_2_mllm_demo_format.py).

    python -m mindspeed_mm_b200.data.data_tools mock  --save-dir data/mock --num-pics 4 --text-length 4096 --num-samples 64
    python -m mindspeed_mm_b200.data.data_tools llava --llava-json llava_instruct_150k.json --image-root data/COCO2017 --out out.json
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Callable, List, Optional

SEED_TEXT = "A moment frozen in the flow of time"


def write_mock_dataset(save_dir: str, num_pics: int = 10, text_length: int = 16384, num_samples: int = 512, width: int = 1024,
                       height: int = 1024, count_tokens: Optional[Callable[[str], int]] = None, seed: int = 0) -> str:
    """Returns the path of the JSON.  ``count_tokens(text)`` sizes the text in tokens of the tokenizer in use (default:
    one token per four characters)."""
    import numpy as np
    from PIL import Image
    os.makedirs(save_dir, exist_ok=True)
    pic = f"test_pic_h{height}_w{width}.jpg"
    rng = np.random.default_rng(seed)
    Image.fromarray(rng.integers(0, 256, (height, width, 3), dtype=np.uint8), "RGB").save(os.path.join(save_dir, pic))
    count = count_tokens or (lambda s: max(1, len(s) // 4))
    repeats = text_length // (count(SEED_TEXT) * 2) + 1                    # question and answer share the budget
    text = (SEED_TEXT + " ") * repeats
    record = {"messages": [{"role": "user", "content": "<image>\n" * num_pics + f". Please describe the image. {text}"},
                           {"role": "assistant", "content": text}],
              "images": [pic] * num_pics}
    path = os.path.join(save_dir, f"mock_data_pic_num_{num_pics}_textlen_{text_length}.json")
    with open(path, "w") as f:
        json.dump([record] * num_samples, f)
    return path


def convert_llava_instruct(records: List[dict], image_root: Optional[str] = None, image_prefix: str = "train2017") -> List[dict]:
    out = []
    for item in records:
        new = {"images": [], "messages": []}
        if item.get("image"):
            rel = os.path.join(image_prefix, item["image"]) if image_prefix else item["image"]
            if image_root is not None and not os.path.exists(os.path.join(image_root, rel)):
                continue
            new["images"] = [rel]
        for turn in item["conversations"]:
            role = {"human": "user", "gpt": "assistant"}.get(turn["from"])
            if role is None:
                raise ValueError(f"unknown role {turn['from']!r}")
            new["messages"].append({"role": role, "content": turn["value"]})
        out.append(new)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    m = sub.add_parser("mock")
    m.add_argument("--save-dir", default="./data/mocked_vl_data")
    m.add_argument("--num-pics", type=int, default=10)
    m.add_argument("--text-length", type=int, default=16384)
    m.add_argument("--num-samples", type=int, default=512)
    m.add_argument("--pic-width", type=int, default=1024)
    m.add_argument("--pic-height", type=int, default=1024)
    m.add_argument("--tokenizer-path", default=None)
    c = sub.add_parser("llava")
    c.add_argument("--llava-json", required=True)
    c.add_argument("--image-root", default=None)
    c.add_argument("--image-prefix", default="train2017")
    c.add_argument("--out", required=True)
    a = ap.parse_args(argv)
    if a.cmd == "mock":
        count = None
        if a.tokenizer_path:
            from transformers import AutoTokenizer
            tok = AutoTokenizer.from_pretrained(a.tokenizer_path)
            count = lambda s: len(tok.encode(s))                            # noqa: E731
        print(write_mock_dataset(a.save_dir, a.num_pics, a.text_length, a.num_samples, a.pic_width, a.pic_height, count))
        return 0
    if os.path.exists(a.out):
        print(f"{a.out} already exists: rename or remove it", file=sys.stderr)
        return 1
    with open(a.llava_json) as f:
        recs = convert_llava_instruct(json.load(f), a.image_root, a.image_prefix)
    os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
    with open(a.out, "w") as f:
        json.dump(recs, f, ensure_ascii=False)
    print(f"{len(recs)} records written to {a.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
