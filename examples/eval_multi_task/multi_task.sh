#!/bin/bash
# Training on one prompt set while evaluating on several, each with its own reward model, sampling parameters and
# number of samples: everything about evaluation comes from multi_task.yaml (--eval-config).
HERE="$(cd -- "$(dirname -- "${BASH_SOURCE[0]}")" && pwd)"
source "${HERE}/../../recipes/common.sh"
MODEL_ARGS=($(model_args qwen3-4B))
launch train.py "${MODEL_ARGS[@]}" \
  --hf-checkpoint "${CKPT_DIR}/Qwen3-4B" --ref-load "${CKPT_DIR}/Qwen3-4B_torch_dist" \
  --prompt-data "${DATA_DIR}/dapo-math-17k/dapo-math-17k.jsonl" --input-key prompt --label-key label \
  --apply-chat-template --rollout-shuffle --rm-type deepscaler --num-rollout 3000 --rollout-batch-size 32 \
  --n-samples-per-prompt 8 --rollout-max-response-len 8192 --rollout-temperature 1 --global-batch-size 256 --balance-data \
  --eval-interval 20 --eval-config "${HERE}/multi_task.yaml" \
  --tensor-model-parallel-size 2 --sequence-parallel --use-dynamic-batch-size --max-tokens-per-gpu 9216 \
  --advantage-estimator grpo --eps-clip 0.2 --eps-clip-high 0.28 \
  --optimizer adam --lr 1e-6 --lr-decay-style constant --weight-decay 0.1 --adam-beta1 0.9 --adam-beta2 0.98 \
  --actor-num-nodes 1 --actor-num-gpus-per-node "${NUM_GPUS}" --colocate --rollout-num-gpus-per-engine 2 \
  --sglang-mem-fraction-static 0.7
