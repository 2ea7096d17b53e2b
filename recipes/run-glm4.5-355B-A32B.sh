#!/bin/bash
# GLM-4.5-355B-A32B on 8 nodes x 8 GPUs, colocated: TP8 + SP, PP4 (last stage 20 layers), EP16, CPU Adam; 32-GPU rollout engines.
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
MODEL_ARGS=($(model_args glm4.5-355B-A32B))
launch train.py "${MODEL_ARGS[@]}" $(ckpt_args GLM-4.5-355B-A32B) "${DAPO_ROLLOUT_ARGS[@]}" \
  --rollout-batch-size 64 --n-samples-per-prompt 8 --rollout-max-response-len 8192 --global-batch-size 512 \
  "${AIME_EVAL_ARGS[@]}" --n-samples-per-eval-prompt 16 --eval-max-response-len 16384 \
  --tensor-model-parallel-size 8 --sequence-parallel --pipeline-model-parallel-size 4 --decoder-last-pipeline-num-layers 20 --expert-model-parallel-size 16 --expert-tensor-parallel-size 1 --use-dynamic-batch-size --max-tokens-per-gpu 16384 \
  "${RECOMPUTE_ARGS[@]}" "${GRPO_ARGS[@]}" "${CPU_ADAM_ARGS[@]}" "${MISC_ARGS[@]}" \
  --actor-num-nodes "${NUM_NODES:-8}" --actor-num-gpus-per-node 8 --colocate --rollout-num-gpus-per-engine 32 --sglang-mem-fraction-static 0.7 --sglang-ep-size 32 --update-weight-buffer-size 4294967296
