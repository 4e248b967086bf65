"""Megatron-style entry point (same command line as the reference's pretrain_sora.py):

    torchrun ... pretrain_sora.py $GPT_ARGS --mm-data data.json --mm-model model.json --mm-tool tools.json
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from mindspeed_mm_b200.runtime.legacy_entry import pretrain  # noqa: E402

if __name__ == "__main__":
    pretrain("sora")
