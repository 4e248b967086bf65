#!/bin/bash
# DreamBooth LoRA fine-tuning of sd3 on a folder of subject images (the job the reference runs through the diffusers
# train_dreambooth_lora script + accelerate): this framework's own generative trainer, LoRA on the attention projections,
# ZeRO-3 over the GPUs of one node.
set -e
NPROC=${NPROC:-8}
torchrun --nnodes 1 --nproc-per-node $NPROC --master-addr 127.0.0.1 --master-port 29500 pretrain_sora.py \
    --mm-model examples/diffusers/sd3/dreambooth_lora_model.json --mm-data examples/diffusers/sd3/dreambooth_lora_data.json \
    --micro-batch-size 1 --global-batch-size $NPROC --train-iters 500 --lr 1e-4 --lr-decay-style constant \
    --weight-decay 0.0 --clip-grad 1.0 --bf16 --save ./save/sd3_dreambooth_lora --save-interval 500 --log-interval 10
