"""Diffusion / flow-matching schedulers (training targets, timestep sampling, samplers)."""
from .flow_match import FlowMatchScheduler  # noqa: F401
