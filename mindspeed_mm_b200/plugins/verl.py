"""Plugin for RL trainers that build transformers classes themselves (verl's FSDP workers): GRPO / PPO actor and
reference models of the Qwen2.5-VL / Qwen3-VL(-MoE) families run on this package's kernels.

Reference: verl_plugin/verl_npu/plugin.py:160-232 (``apply_npu_plugin``: kernel substitution on the transformers classes,
device synchronisation of TensorDict transfers, rollout-engine sleep level) and verl_plugin/setup.py:14-44 (seeding code
for reproducible runs, selected by ``DETERMINISTIC``).  On CUDA, TensorDict already synchronises its device transfers and
the rollout engine needs no sleep-level override, so what remains is the kernel substitution and the determinism
switch.  The importable shim ``verl_plugin/verl_b200`` calls ``apply_verl_plugin()`` when it is imported, which is how an
unmodified verl picks it up (``import verl_b200`` at the top of the launch script, or through ``PYTHONSTARTUP``).
"""
from __future__ import annotations

import os
import random
from typing import Dict, List, Optional

import torch

from . import hf_kernels

VLM_FAMILIES = ("qwen2", "qwen2_vl", "qwen2_5_vl", "qwen3", "qwen3_moe", "qwen3_vl", "qwen3_vl_moe")


def seed_all(seed: int = 1234) -> None:
    """Reproducible runs: seeds of every generator, deterministic algorithm selection, a fixed cuBLAS workspace and
    NCCL collectives with a fixed reduction order."""
    random.seed(seed)
    os.environ["PYTHONHASHSEED"] = str(seed)
    os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
    os.environ.setdefault("NCCL_ALGO", "Ring")
    try:
        import numpy as np
        np.random.seed(seed)
    except ImportError:
        pass
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    torch.use_deterministic_algorithms(True, warn_only=True)


def apply_verl_plugin(families=VLM_FAMILIES, attention: bool = True, deterministic: Optional[bool] = None,
                      seed: int = 1234) -> Dict[str, List[str]]:
    """Substitute the kernels into the transformers classes verl instantiates.  ``deterministic`` defaults to the
    ``DETERMINISTIC`` environment variable (``1`` / ``true``), the switch the reference's installer reads.  Models then
    select the attention kernel with ``attn_implementation="mm_b200"`` (verl: ``actor_rollout_ref.model.override_config``)."""
    if deterministic is None:
        deterministic = os.environ.get("DETERMINISTIC", "").lower() in ("1", "true", "yes")
    if deterministic:
        seed_all(seed)
    return hf_kernels.apply_kernel_plugin(families, attention=attention)
