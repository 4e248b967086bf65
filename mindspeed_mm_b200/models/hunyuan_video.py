"""HunyuanVideo DiT: the dual/single-stream MMDiT with the video configuration (see ``mmdit.py``)."""
from .mmdit import HunyuanVideoDiT, MMDiTConfig  # noqa: F401

hunyuan_video_config = MMDiTConfig.hunyuan_video
