"""Imports every built-in model file so that its ``@model_register`` decorators run."""
from . import qwen2_5_vl  # noqa: F401
from . import wan  # noqa: F401
from .diffusion import flow_match  # noqa: F401
from . import qwen3_vl  # noqa: F401
from . import qwen3_5  # noqa: F401
from . import internvl  # noqa: F401
from ..plugins import hf_auto  # noqa: F401
from . import mmdit  # noqa: F401
from . import composable  # noqa: F401
from . import wan_variants  # noqa: F401
from . import ltx2  # noqa: F401
from . import speech_lm  # noqa: F401
from . import video_dits  # noqa: F401
from . import omni  # noqa: F401
from . import sdxl_unet  # noqa: F401
from . import prompt_encoders  # noqa: F401
