"""Adapters that bring this package's kernels and sharding engine to model code it does not own: Hugging Face
``transformers`` classes (``hf_kernels``: kernel substitution; ``hf_adapter``: any ``PreTrainedModel`` under the ZeRO-3
engine) and RL trainers that build those classes themselves (``verl``: entry point of the plugin)."""
