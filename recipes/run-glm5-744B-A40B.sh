#!/bin/bash
# GLM-5 (744B, sparse latent attention with a lightning indexer, 256 experts) on 16 nodes x 8 GPUs: TP4 + SP, PP8, EP32, all-gather
# context parallel x2, CPU Adam; 64-GPU rollout engines.
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
MODEL_ARGS=($(model_args glm5-744B-A40B))
launch train.py "${MODEL_ARGS[@]}" $(ckpt_args GLM-5) "${DAPO_ROLLOUT_ARGS[@]}" \
  --rollout-batch-size 64 --n-samples-per-prompt 8 --rollout-max-response-len 16384 --global-batch-size 512 \
  "${AIME_EVAL_ARGS[@]}" --n-samples-per-eval-prompt 16 --eval-max-response-len 16384 \
  --tensor-model-parallel-size 4 --sequence-parallel --pipeline-model-parallel-size 8 --decoder-last-pipeline-num-layers 8 --context-parallel-size 2 --allgather-cp --expert-model-parallel-size 32 --expert-tensor-parallel-size 1 --use-dynamic-batch-size --max-tokens-per-gpu 16384 \
  "${RECOMPUTE_ARGS[@]}" "${GRPO_ARGS[@]}" "${CPU_ADAM_ARGS[@]}" "${MISC_ARGS[@]}" \
  --actor-num-nodes "${NUM_NODES:-16}" --actor-num-gpus-per-node 8 --colocate --rollout-num-gpus-per-engine 64 --sglang-mem-fraction-static 0.7 --sglang-ep-size 64 --update-weight-buffer-size 4294967296
