"""Task layers on top of the trainer: LoRA, inference pipelines, evaluation, preference / RL post-training."""
