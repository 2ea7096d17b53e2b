#!/bin/bash
# GLM-4.7-30B-A3B (latent attention, 64 experts top-4, sigmoid router) on 8 GPUs, colocated: TP4 + SP, EP8, CPU Adam.
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
MODEL_ARGS=($(model_args glm4.7-30B-A3B))
launch train.py "${MODEL_ARGS[@]}" $(ckpt_args GLM-4.7-30B-A3B) "${DAPO_ROLLOUT_ARGS[@]}" \
  --rollout-batch-size 32 --n-samples-per-prompt 8 --rollout-max-response-len 8192 --global-batch-size 256 \
  "${AIME_EVAL_ARGS[@]}" --n-samples-per-eval-prompt 16 --eval-max-response-len 16384 \
  --tensor-model-parallel-size 4 --sequence-parallel --expert-model-parallel-size 8 --expert-tensor-parallel-size 1 --use-dynamic-batch-size --max-tokens-per-gpu 16384 \
  "${RECOMPUTE_ARGS[@]}" "${GRPO_ARGS[@]}" "${CPU_ADAM_ARGS[@]}" "${MISC_ARGS[@]}" \
  --actor-num-nodes 1 --actor-num-gpus-per-node "${NUM_GPUS}" --colocate --rollout-num-gpus-per-engine 8 --sglang-mem-fraction-static 0.7 --sglang-ep-size 8
