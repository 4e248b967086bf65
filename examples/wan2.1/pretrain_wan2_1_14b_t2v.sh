#!/bin/bash
# Wan2.1-14B text-to-video pretraining on pre-extracted features, Ulysses sequence parallel 8 x ZeRO-3
# (the reference's examples/wan2.1/14b/t2v/pretrain.sh).
set -e
GPUS=${GPUS:-8}; MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}; MASTER_PORT=${MASTER_PORT:-29500}
GPT_ARGS="--context-parallel-size 8 --context-parallel-algo ulysses_cp_algo --micro-batch-size 1 --global-batch-size 1 \
  --train-iters 5000 --lr 1e-5 --min-lr 1e-5 --lr-decay-style constant --weight-decay 0.01 --clip-grad 1.0 --bf16 \
  --log-interval 1 --save-interval 1000 --save ./save/wan2_1_14b_t2v"
python -m torch.distributed.run --nnodes 1 --nproc-per-node $GPUS --master-addr $MASTER_ADDR --master-port $MASTER_PORT \
  pretrain_sora.py $GPT_ARGS --mm-model examples/wan2.1/pretrain_model_14b.json --mm-data examples/wan2.1/feature_data.json
