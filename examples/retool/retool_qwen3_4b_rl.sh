#!/bin/bash
# RL stage of the retool example: Qwen3-4B (after the tool-use SFT stage) on DAPO-math with a Python interpreter tool.
source "$(dirname -- "${BASH_SOURCE[0]}")/../../recipes/common.sh"
MODEL_ARGS=($(model_args qwen3-4B))
launch train.py "${MODEL_ARGS[@]}" \
  --hf-checkpoint "${CKPT_DIR}/Qwen3-4B-retool-sft" --ref-load "${CKPT_DIR}/Qwen3-4B-retool-sft_torch_dist" \
  --prompt-data "${DATA_DIR}/dapo-math-17k/dapo-math-17k.jsonl" --input-key prompt --label-key label --rollout-shuffle \
  --custom-generate-function-path examples.retool.generate_with_retool.generate \
  --custom-rm-path examples.retool.generate_with_retool.reward_func \
  --num-rollout 3000 --rollout-batch-size 32 --n-samples-per-prompt 8 --rollout-max-response-len 8192 \
  --rollout-temperature 1 --global-batch-size 256 --balance-data \
  --tensor-model-parallel-size 2 --sequence-parallel --use-dynamic-batch-size --max-tokens-per-gpu 9216 \
  --advantage-estimator grpo --eps-clip 0.2 --eps-clip-high 0.28 --use-kl-loss --kl-loss-coef 0.0 \
  --optimizer adam --lr 1e-6 --lr-decay-style constant --weight-decay 0.1 --adam-beta1 0.9 --adam-beta2 0.98 \
  --actor-num-nodes 1 --actor-num-gpus-per-node "${NUM_GPUS}" --colocate --rollout-num-gpus-per-engine 2 \
  --sglang-mem-fraction-static 0.7
