#!/bin/bash
# Qwen3-8B on DAPO-math with a Python tool, the conversation driven by the message-level agent loop of this folder.
# No --apply-chat-template: the agent renders the conversation itself.
source "$(dirname -- "${BASH_SOURCE[0]}")/../../recipes/common.sh"
MODEL_ARGS=($(model_args qwen3-8B))
launch train.py "${MODEL_ARGS[@]}" \
  --hf-checkpoint "${CKPT_DIR}/Qwen3-8B" --ref-load "${CKPT_DIR}/Qwen3-8B_torch_dist" \
  --prompt-data "${DATA_DIR}/dapo-math-17k/dapo-math-17k.jsonl" --input-key prompt --label-key label --rollout-shuffle \
  --custom-generate-function-path examples.strands_sglang.generate_with_strands.generate \
  --custom-rm-path examples.strands_sglang.generate_with_strands.reward_func \
  --num-rollout 3000 --rollout-batch-size 32 --n-samples-per-prompt 8 --rollout-max-response-len 8192 \
  --rollout-max-context-len 16384 --rollout-temperature 1 --global-batch-size 256 --balance-data \
  --eval-interval 20 --eval-prompt-data aime "${DATA_DIR}/aime-2024/aime-2024.jsonl" --n-samples-per-eval-prompt 16 \
  --eval-max-response-len 16384 --eval-top-p 0.7 \
  --tensor-model-parallel-size 2 --sequence-parallel --use-dynamic-batch-size --max-tokens-per-gpu 9216 \
  --recompute-granularity full --recompute-method uniform --recompute-num-layers 1 \
  --advantage-estimator grpo --eps-clip 0.2 --eps-clip-high 0.28 --use-kl-loss --kl-loss-coef 0.0 --entropy-coef 0.0 \
  --optimizer adam --lr 1e-6 --lr-decay-style constant --weight-decay 0.1 --adam-beta1 0.9 --adam-beta2 0.98 \
  --actor-num-nodes 1 --actor-num-gpus-per-node "${NUM_GPUS}" --colocate --rollout-num-gpus-per-engine 2 \
  --sglang-mem-fraction-static 0.7
