#!/bin/bash
# Qwen2.5-VL-72B, Megatron-style TP8 x PP4 (x DP) with sequence parallel, same command line as the reference's
# examples/qwen2.5vl/finetune_qwen2_5_vl_72b.sh.  One process per GPU; rendezvous through MASTER_ADDR / MASTER_PORT.
set -e
NNODES=${NNODES:-4}; NODE_RANK=${NODE_RANK:-0}; GPUS=${GPUS:-8}
MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}; MASTER_PORT=${MASTER_PORT:-29500}
GPT_ARGS="--tensor-model-parallel-size 8 --pipeline-model-parallel-size 4 --sequence-parallel \
  --micro-batch-size 1 --global-batch-size 64 --seq-length 8192 --train-iters 5000 --lr 1e-5 --min-lr 1e-6 \
  --lr-decay-style cosine --lr-warmup-fraction 0.1 --weight-decay 0.0 --clip-grad 1.0 --bf16 \
  --log-interval 1 --save-interval 500 --save ./save/qwen2_5_vl_72b --load ./ckpt/mm/Qwen2.5-VL-72B-tp8pp4"
python -m torch.distributed.run --nnodes $NNODES --node-rank $NODE_RANK --nproc-per-node $GPUS \
  --master-addr $MASTER_ADDR --master-port $MASTER_PORT pretrain_vlm.py $GPT_ARGS \
  --mm-model examples/qwen2.5vl/model_72b.json --mm-data examples/qwen2.5vl/data_72b.json
