#!/bin/bash
# GRPO of Qwen2.5-VL-7B on geo3k with verl, actor / reference on the sm_100a kernels (8 x B200, one node).
# Needs verl and a rollout engine installed; the plugin itself only needs mindspeed_mm_b200 on PYTHONPATH.
set -e
MODEL=${MODEL:-/path/to/Qwen2.5-VL-7B-Instruct}
DATA=${DATA:-/path/to/geo3k}
python - "$@" <<'PY'
import sys
import verl_b200  # noqa: F401  (substitutes the kernels before verl imports transformers models)
from verl.trainer.main_ppo import main
sys.argv = ["main_ppo"] + sys.argv[1:]
main()
PY
# typical overrides:
#   algorithm.adv_estimator=grpo data.train_files=$DATA/train.parquet data.val_files=$DATA/test.parquet
#   data.train_batch_size=512 data.max_prompt_length=1024 data.max_response_length=2048
#   actor_rollout_ref.model.path=$MODEL +actor_rollout_ref.model.override_config.attn_implementation=mm_b200
#   actor_rollout_ref.actor.use_kl_loss=True actor_rollout_ref.rollout.n=5 trainer.n_gpus_per_node=8
