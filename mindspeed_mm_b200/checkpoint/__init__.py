"""Checkpoint formats: HuggingFace safetensors (``hf``), sharded training checkpoints (``sharded``),
Megatron mp_rank layout and HF<->MM converters (``megatron``), operator algebra (``operators``),
``mm-convert`` CLI (``convert_cli``)."""
