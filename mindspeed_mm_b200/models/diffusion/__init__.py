"""Diffusion / flow-matching schedulers (training targets, timestep sampling, samplers).

``build_scheduler(config)`` is the factory the generation models use: ``config["model_id"]`` selects the class, the
rest of the dict are its keyword arguments (mindspeed_mm/models/diffusion/diffusion_model.py:12).  Ids that the
reference routes to a diffusers scheduler by name (``ddim``, ``ddpm``, ``euler`` ...) map onto the equivalent class
here, since every scheduler of this package is self-contained.
"""
from .flow_match import FlowMatchScheduler  # noqa: F401
from .flows import (CogVideoDiffusion, FlowMatchDiscreteScheduler, HunyuanVideo15Scheduler, OpenSoraPlanScheduler,  # noqa: F401
                    RFlow)
from .gaussian import DDPM, IDDPM, GaussianDiffusion  # noqa: F401

SCHEDULERS = {
    "wan_flow_match_scheduler": FlowMatchScheduler,
    "flow_match": FlowMatchScheduler,
    "flow_match_discrete": FlowMatchDiscreteScheduler,
    "hunyuanvideo_diffusion": FlowMatchDiscreteScheduler,
    "hunyuanvideo_15_diffusion": HunyuanVideo15Scheduler,
    "opensoraplan_v1_5": OpenSoraPlanScheduler,
    "OpenSoraPlan": OpenSoraPlanScheduler,
    "rflow": RFlow,
    "cogvideo_diffusion": CogVideoDiffusion,
    "ddpm": DDPM,
    "DDPM": DDPM,
    "iddpm": IDDPM,
    "ddim": IDDPM,
    "DDIM": IDDPM,
}


def build_scheduler(config):
    cfg = dict(config.to_dict() if hasattr(config, "to_dict") else config)
    model_id = cfg.pop("model_id", "wan_flow_match_scheduler")
    if model_id not in SCHEDULERS:
        raise KeyError(f"unknown diffusion model_id {model_id!r}; known: {sorted(SCHEDULERS)}")
    return SCHEDULERS[model_id](**cfg)


class DiffusionModel:
    """Same two-call surface as the reference's factory object: ``DiffusionModel(config).get_model()``."""

    def __init__(self, config):
        self.diffusion = build_scheduler(config)

    def get_model(self):
        return self.diffusion
