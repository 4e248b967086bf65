"""Stand-in for the `peft` names the reference imports at module load.  LoRA is not part of the benchmark recipe;
the classes exist so that ``isinstance`` checks in the reference's collators resolve, and using them raises."""
import torch.nn as nn

__version__ = "0.0.0+standin"


class PeftModel(nn.Module):
    def __init__(self, *a, **k):
        raise ImportError("peft is not installed on this image (stand-in class)")


class LoraConfig:
    def __init__(self, *a, **k):
        raise ImportError("peft is not installed on this image (stand-in class)")


def inject_adapter_in_model(*a, **k):
    raise ImportError("peft is not installed on this image (stand-in function)")
