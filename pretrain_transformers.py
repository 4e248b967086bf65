"""Single-YAML entry point (``gpt_args`` / ``data`` / ``model`` / ``MM_TOOL_PATH``), the reference's
pretrain_transformers.py; a YAML with a ``parallel:`` block is routed to the native trainer instead.

    torchrun ... pretrain_transformers.py recipe.yaml
"""
import os
import sys

import yaml

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

if __name__ == "__main__":
    path = sys.argv[1]
    with open(path) as f:
        doc = yaml.safe_load(f)
    if "parallel" in doc and "training" in doc:
        from mindspeed_mm_b200.runtime.trainer import main
        main(sys.argv[1:])
    else:
        from mindspeed_mm_b200.runtime.legacy_entry import pretrain
        kind = "sora" if "predictor" in (doc.get("model") or {}) else "vlm"
        pretrain(kind, sys.argv[1:])
