"""Entry point with the reference's name: `python inference_vlm.py config.json` (see mindspeed_mm_b200/runtime/task_entry.py)."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from mindspeed_mm_b200.runtime import task_entry  # noqa: E402

if __name__ == "__main__":
    import torch
    cfg = task_entry.load_tree(sys.argv[1])
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    out = task_entry.inference_vlm(cfg, dev)
    print(json.dumps(out if not isinstance(out, list) or not out or not hasattr(out[0], "shape") else [list(o.shape) for o in out]))
