#!/bin/bash
# MiMo-7B-RL with its multi-token-prediction head kept in training (the draft loss rides along with GRPO) on 8 GPUs,
# colocated: TP2 + SP, one rollout engine per GPU; the engines speculate with the same head (chains of 3 guesses).
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
MODEL_ARGS=($(model_args mimo-7B-rl))
launch train.py "${MODEL_ARGS[@]}" $(ckpt_args MiMo-7B-RL) "${DAPO_ROLLOUT_ARGS[@]}" \
  --rollout-batch-size 32 --n-samples-per-prompt 8 --rollout-max-response-len 8192 --global-batch-size 256 \
  "${AIME_EVAL_ARGS[@]}" --n-samples-per-eval-prompt 1 --eval-max-response-len 8192 \
  --tensor-model-parallel-size 2 --sequence-parallel --use-dynamic-batch-size --max-tokens-per-gpu 9216 --enable-mtp-training --mtp-loss-scaling-factor 0.2 \
  "${RECOMPUTE_ARGS[@]}" "${GRPO_ARGS[@]}" "${ADAM_ARGS[@]}" "${MISC_ARGS[@]}" \
  --actor-num-nodes 1 --actor-num-gpus-per-node "${NUM_GPUS}" --colocate --rollout-num-gpus-per-engine 1 --sglang-mem-fraction-static 0.7 \
  --sglang-speculative-algorithm EAGLE --sglang-speculative-num-steps 3 --sglang-speculative-eagle-topk 1 --sglang-speculative-num-draft-tokens 4
