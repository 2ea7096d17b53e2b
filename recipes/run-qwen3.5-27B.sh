#!/bin/bash
# Qwen3.5-27B (dense hybrid: gated delta-net + gated attention) on 2 nodes x 8 GPUs, colocated: TP4 + SP, PP2, CPU Adam.
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
MODEL_ARGS=($(model_args qwen3.5-27B))
launch train.py "${MODEL_ARGS[@]}" $(ckpt_args Qwen3.5-27B) "${DAPO_ROLLOUT_ARGS[@]}" \
  --rollout-batch-size 32 --n-samples-per-prompt 8 --rollout-max-response-len 8192 --global-batch-size 256 \
  "${AIME_EVAL_ARGS[@]}" --n-samples-per-eval-prompt 16 --eval-max-response-len 16384 \
  --tensor-model-parallel-size 4 --sequence-parallel --pipeline-model-parallel-size 2 --use-dynamic-batch-size --max-tokens-per-gpu 8192 \
  "${RECOMPUTE_ARGS[@]}" "${GRPO_ARGS[@]}" "${CPU_ADAM_ARGS[@]}" "${MISC_ARGS[@]}" \
  --actor-num-nodes "${NUM_NODES:-2}" --actor-num-gpus-per-node 8 --colocate --rollout-num-gpus-per-engine 4 --sglang-mem-fraction-static 0.7
