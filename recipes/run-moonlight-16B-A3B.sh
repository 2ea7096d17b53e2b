#!/bin/bash
# Moonlight-16B-A3B (latent attention, 64 experts top-6) on 8 GPUs, colocated: TP4 + SP, EP8, CPU Adam, dynamic sampling
# with 4 optimizer steps per rollout.
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
MODEL_ARGS=($(model_args moonlight))
launch train.py "${MODEL_ARGS[@]}" $(ckpt_args Moonlight-16B-A3B) "${DAPO_ROLLOUT_ARGS[@]}" \
  --rollout-batch-size 128 --n-samples-per-prompt 8 --rollout-max-response-len 4096 --num-steps-per-rollout 4 "${DYNAMIC_SAMPLING_ARGS[@]}" \
  "${AIME_EVAL_ARGS[@]}" --n-samples-per-eval-prompt 8 --eval-max-response-len 4096 \
  --tensor-model-parallel-size 4 --sequence-parallel --expert-model-parallel-size 8 --expert-tensor-parallel-size 1 --use-dynamic-batch-size --max-tokens-per-gpu 8192 \
  "${RECOMPUTE_ARGS[@]}" "${GRPO_ARGS[@]}" "${CPU_ADAM_ARGS[@]}" "${MISC_ARGS[@]}" \
  --actor-num-nodes 1 --actor-num-gpus-per-node "${NUM_GPUS}" --colocate --rollout-num-gpus-per-engine 8 --sglang-mem-fraction-static 0.7 --sglang-ep-size 8
