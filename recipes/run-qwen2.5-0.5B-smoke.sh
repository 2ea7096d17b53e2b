#!/bin/bash
# Two-rollout smoke run of the whole pipeline on one GPU (colocated trainer and engine, GSM8K, short responses).
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
MODEL_ARGS=($(model_args qwen2.5-0.5B))
launch train.py "${MODEL_ARGS[@]}" --hf-checkpoint "${CKPT_DIR}/Qwen2.5-0.5B-Instruct" --ref-load "${CKPT_DIR}/Qwen2.5-0.5B-Instruct_torch_dist" \
  --prompt-data "${DATA_DIR}/gsm8k/train.jsonl" --input-key messages --label-key label --apply-chat-template --rollout-shuffle \
  --rm-type math --num-rollout 2 --rollout-batch-size 8 --n-samples-per-prompt 4 --rollout-max-response-len 256 \
  --rollout-temperature 1 --global-batch-size 32 --use-dynamic-batch-size --max-tokens-per-gpu 4096 \
  "${GRPO_ARGS[@]}" "${ADAM_ARGS[@]}" "${MISC_ARGS[@]}" \
  --actor-num-nodes 1 --actor-num-gpus-per-node 1 --colocate --rollout-num-gpus-per-engine 1 --sglang-mem-fraction-static 0.4
