"""Offline feature extraction for generative training: videos -> VAE latents, captions -> text-encoder states,
written as the ``.pt`` files + jsonl index that :class:`~mindspeed_mm_b200.data.multimodal.FeatureDataset` reads
(the reference's mindspeed_mm/tools/feature_extraction/get_wan_feature.py and siblings).

    python -m mindspeed_mm_b200.tasks.feature_extraction model.json data.json out_dir

Ranks of a torchrun job take disjoint strides of the dataset.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Optional

import torch


@torch.no_grad()
def extract_features(dataset, ae, text_encoder, out_dir: str, device="cpu", dtype=torch.float32, rank: int = 0, world: int = 1,
                     i2v: bool = False, chunk_frames: Optional[int] = None) -> int:
    os.makedirs(out_dir, exist_ok=True)
    index = []
    for i in range(rank, len(dataset), world):
        s = dataset[i]
        video = s["video"][None].to(device, dtype)
        rec = {"latents": ae.encode(video, chunk_frames=chunk_frames)[0].cpu(),
               "prompt": text_encoder.encode(s["prompt_ids"][None].to(device), s["prompt_mask"][None].to(device))[0].cpu(),
               "prompt_mask": s["prompt_mask"].bool()}
        if i2v:
            first = torch.zeros_like(video)
            first[:, :, :1] = video[:, :, :1]
            rec["first_frame_latents"] = ae.encode(first, chunk_frames=chunk_frames)[0][:, :1].cpu()
        name = f"{i:08d}.pt"
        torch.save(rec, os.path.join(out_dir, name))
        index.append({"file": name})
    with open(os.path.join(out_dir, f"index_rank{rank}.jsonl"), "w") as f:
        for r in index:
            f.write(json.dumps(r) + "\n")
    return len(index)


def main(argv=None):
    from types import SimpleNamespace
    from ..data.multimodal import VideoTextDataset
    from ..models.towers import build_ae, build_text_encoder
    argv = list(sys.argv[1:] if argv is None else argv)
    model = json.load(open(argv[0]))
    dp = json.load(open(argv[1])).get("dataset_param", {})
    data = SimpleNamespace(dataset_param=SimpleNamespace(basic_parameters=dp.get("basic_parameters", {}),
                                                       preprocess_parameters=dp.get("preprocess_parameters", {})))
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if dev == "cuda":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    ds = VideoTextDataset(data.dataset_param)
    n = extract_features(ds, build_ae(model.get("ae"), dev), build_text_encoder(model.get("text_encoder"), dev), argv[2], dev,
                         rank=rank, world=world, i2v=bool(model.get("i2v", False)))
    print(f"rank {rank}: wrote {n} feature files to {argv[2]}")


if __name__ == "__main__":
    main()
