#!/bin/bash
# Kimi-K2-Thinking (1T parameters, latent attention, 384 experts) on 32 nodes x 8 GPUs: TP8 + SP, PP8 (last stage 5 layers), CP4, EP32,
# CPU Adam, dynamic sampling with 4 optimizer steps per rollout; 64-GPU rollout engines.
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
MODEL_ARGS=($(model_args kimi-k2-thinking))
launch train.py "${MODEL_ARGS[@]}" $(ckpt_args Kimi-K2-Thinking) "${DAPO_ROLLOUT_ARGS[@]}" \
  --rollout-batch-size 128 --n-samples-per-prompt 8 --rollout-max-response-len 16384 --num-steps-per-rollout 4 "${DYNAMIC_SAMPLING_ARGS[@]}" \
  "${AIME_EVAL_ARGS[@]}" --n-samples-per-eval-prompt 8 --eval-max-response-len 16384 \
  --tensor-model-parallel-size 8 --sequence-parallel --pipeline-model-parallel-size 8 --decoder-last-pipeline-num-layers 5 --context-parallel-size 4 --expert-model-parallel-size 32 --expert-tensor-parallel-size 1 --use-dynamic-batch-size --max-tokens-per-gpu 16384 \
  "${RECOMPUTE_ARGS[@]}" "${GRPO_ARGS[@]}" "${CPU_ADAM_ARGS[@]}" "${MISC_ARGS[@]}" \
  --actor-num-nodes "${NUM_NODES:-32}" --actor-num-gpus-per-node 8 --colocate --rollout-num-gpus-per-engine 64 --sglang-mem-fraction-static 0.7 --sglang-ep-size 64 --sglang-server-concurrency 1024
