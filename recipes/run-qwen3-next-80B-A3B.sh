#!/bin/bash
# Qwen3-Next-80B-A3B (gated delta-net layers with every fourth layer gated attention, 512 experts top-10) on 4 nodes x 8 GPUs:
# TP2 + SP, PP4 (last stage 9 layers), EP8, CPU Adam, GSPO with sequence-level clipping, 32k responses.
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
MODEL_ARGS=($(model_args qwen3-next-80B-A3B))
launch train.py "${MODEL_ARGS[@]}" $(ckpt_args Qwen3-Next-80B-A3B-Thinking) "${DAPO_ROLLOUT_ARGS[@]}" \
  --rollout-batch-size 8 --n-samples-per-prompt 8 --rollout-max-response-len 32768 --global-batch-size 64 \
  "${AIME_EVAL_ARGS[@]}" --n-samples-per-eval-prompt 8 --eval-max-response-len 32768 \
  --tensor-model-parallel-size 2 --sequence-parallel --pipeline-model-parallel-size 4 --decoder-last-pipeline-num-layers 9 --expert-model-parallel-size 8 --expert-tensor-parallel-size 1 --use-dynamic-batch-size --max-tokens-per-gpu 8192 --advantage-estimator gspo --kl-loss-coef 0.0 --kl-loss-type low_var_kl --kl-coef 0.0 --entropy-coef 0.0 --eps-clip 4e-4 \
  "${RECOMPUTE_ARGS[@]}"  "${CPU_ADAM_ARGS[@]}" "${MISC_ARGS[@]}" \
  --actor-num-nodes "${NUM_NODES:-4}" --actor-num-gpus-per-node 8 --colocate --rollout-num-gpus-per-engine 8 --sglang-mem-fraction-static 0.8 --sglang-ep-size 8 --sglang-max-running-requests 256
