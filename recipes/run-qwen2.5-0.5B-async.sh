#!/bin/bash
# Fully asynchronous variant: 4 GPUs train, 4 GPUs generate continuously; rollout k+1 overlaps training step k and the
# trainer pushes weights every step (train_async.py with the fully-async rollout function).
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
MODEL_ARGS=($(model_args qwen2.5-0.5B))
launch train_async.py "${MODEL_ARGS[@]}" \
  --hf-checkpoint "${CKPT_DIR}/Qwen2.5-0.5B-Instruct" --ref-load "${CKPT_DIR}/Qwen2.5-0.5B-Instruct" \
  --prompt-data "${DATA_DIR}/gsm8k/train.jsonl" --input-key messages --label-key label --apply-chat-template \
  --rollout-shuffle --rm-type math --num-rollout 200 --rollout-batch-size 32 --n-samples-per-prompt 8 \
  --rollout-max-response-len 1024 --rollout-temperature 1 --global-batch-size 256 \
  --rollout-function-path slime.rollout.fully_async_rollout.generate_rollout_fully_async \
  --use-dynamic-batch-size --max-tokens-per-gpu 16384 \
  --advantage-estimator grpo --eps-clip 0.2 --eps-clip-high 0.28 --use-tis \
  --optimizer adam --lr 1e-6 --lr-decay-style constant --weight-decay 0.1 --adam-beta1 0.9 --adam-beta2 0.98 \
  --actor-num-nodes 1 --actor-num-gpus-per-node 4 --rollout-num-gpus 4 --rollout-num-gpus-per-engine 1 \
  --sglang-mem-fraction-static 0.8 --attention-dropout 0.0 --hidden-dropout 0.0 \
  --accumulate-allreduce-grads-in-fp32 --attention-softmax-in-fp32
