"""FLUX.1 MMDiT: the dual/single-stream MMDiT with the image configuration (see ``mmdit.py``)."""
from .mmdit import FluxDiT, MMDiTConfig  # noqa: F401

flux_dev_config = MMDiTConfig.flux_dev
