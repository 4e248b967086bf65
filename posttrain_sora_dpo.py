"""Diffusion-DPO post-training of a video DiT (the reference's posttrain_sora_dpo.py).

    python posttrain_sora_dpo.py model.json pairs.jsonl [steps]

``pairs.jsonl`` lists ``.pt`` files holding ``latents_win``, ``latents_lose`` and ``prompt`` tensors.
"""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

if __name__ == "__main__":
    import torch
    from mindspeed_mm_b200.runtime import task_entry
    cfg = task_entry.load_tree(sys.argv[1])
    with open(sys.argv[2]) as f:
        files = [json.loads(l)["file"] for l in f if l.strip()]

    def it():
        while True:
            for p in files:
                yield torch.load(p, map_location="cpu", weights_only=True)
    steps = int(sys.argv[3]) if len(sys.argv) > 3 else len(files)
    for r in task_entry.posttrain_sora_dpo(cfg, it(), "cuda" if torch.cuda.is_available() else "cpu", steps):
        print(json.dumps(r))
