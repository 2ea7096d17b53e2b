#!/bin/bash
# GLM-Z1-9B (sandwich norms, half-rotary interleaved RoPE) on 8 GPUs: 4 for training (TP2 x CP2), 4 for rollout (2 per engine).
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
MODEL_ARGS=($(model_args glm4-9B))
launch train.py "${MODEL_ARGS[@]}" $(ckpt_args GLM-Z1-9B-0414) "${DAPO_ROLLOUT_ARGS[@]}" \
  --rollout-batch-size 32 --n-samples-per-prompt 8 --rollout-max-response-len 8192 --global-batch-size 256 \
  "${AIME_EVAL_ARGS[@]}" --n-samples-per-eval-prompt 16 --eval-max-response-len 16384 \
  --tensor-model-parallel-size 2 --sequence-parallel --context-parallel-size 1 --use-dynamic-batch-size --max-tokens-per-gpu 4608 \
  "${RECOMPUTE_ARGS[@]}" "${GRPO_ARGS[@]}" "${ADAM_ARGS[@]}" "${MISC_ARGS[@]}" \
  --actor-num-nodes 1 --actor-num-gpus-per-node 4 --rollout-num-gpus 4 --rollout-num-gpus-per-engine 2
