"""Import this module before verl builds its workers: the transformers classes of the Qwen VLM families then run on the
sm_100a kernels of ``mindspeed_mm_b200`` (RMSNorm, rotary embedding, SwiGLU, attention ``"mm_b200"``)."""
from mindspeed_mm_b200.plugins.verl import apply_verl_plugin

PATCHED = apply_verl_plugin()
