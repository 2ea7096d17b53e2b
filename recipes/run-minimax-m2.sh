#!/bin/bash
# MiniMax-M2 (229B, 256 experts, RMSNorm over all heads of q / k) on 8 nodes x 8 GPUs: TP8 + SP, PP2, EP32, CPU Adam.
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
MODEL_ARGS=($(model_args minimax-m2))
launch train.py "${MODEL_ARGS[@]}" $(ckpt_args MiniMax-M2) "${DAPO_ROLLOUT_ARGS[@]}" \
  --rollout-batch-size 64 --n-samples-per-prompt 8 --rollout-max-response-len 16384 --global-batch-size 512 \
  "${AIME_EVAL_ARGS[@]}" --n-samples-per-eval-prompt 16 --eval-max-response-len 16384 \
  --tensor-model-parallel-size 8 --sequence-parallel --pipeline-model-parallel-size 2 --expert-model-parallel-size 32 --expert-tensor-parallel-size 1 --use-dynamic-batch-size --max-tokens-per-gpu 16384 \
  "${RECOMPUTE_ARGS[@]}" "${GRPO_ARGS[@]}" "${CPU_ADAM_ARGS[@]}" "${MISC_ARGS[@]}" \
  --actor-num-nodes "${NUM_NODES:-8}" --actor-num-gpus-per-node 8 --colocate --rollout-num-gpus-per-engine 32 --sglang-mem-fraction-static 0.7 --sglang-ep-size 32
