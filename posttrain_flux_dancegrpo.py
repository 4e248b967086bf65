"""DanceGRPO post-training of a FLUX-style MMDiT (the reference's posttrain_flux_dancegrpo.py).

    python posttrain_flux_dancegrpo.py model.json prompts.pt reward_module:function [steps]

``prompts.pt`` holds a list of ``(text_embeddings [1, L, D], pooled [1, P])`` pairs; the reward callable maps
``(final_latents, prompt) -> tensor [n]``.
"""
import importlib
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

if __name__ == "__main__":
    import torch
    from mindspeed_mm_b200.runtime import task_entry
    cfg = task_entry.load_tree(sys.argv[1])
    prompts = torch.load(sys.argv[2], map_location="cpu", weights_only=True)
    mod, fn = sys.argv[3].split(":")
    reward = getattr(importlib.import_module(mod), fn)
    steps = int(sys.argv[4]) if len(sys.argv) > 4 else len(prompts)
    for r in task_entry.posttrain_flux_dancegrpo(cfg, prompts, reward, "cuda" if torch.cuda.is_available() else "cpu", steps):
        print(json.dumps(r))
