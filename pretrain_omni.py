"""Omni-modal (text + vision + audio) pre-training entry (the reference's pretrain_omni.py): the native trainer with a
composable model preset that has an audio tower, e.g. ``model.model_id: qwen3omni``.

    torchrun ... pretrain_omni.py recipe.yaml [key=value ...]
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

if __name__ == "__main__":
    from mindspeed_mm_b200.runtime.trainer import main
    main(sys.argv[1:])
