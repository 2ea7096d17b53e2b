#!/bin/bash
# Fully asynchronous rollout on one node: ACTOR_GPUS train, the rest generate without ever stopping. The only change
# against the asynchronous recipe is the rollout function: a background worker keeps the engines saturated and hands
# finished groups to the trainer as they complete, aborted partial generations are re-queued with their tokens.
source "$(dirname -- "${BASH_SOURCE[0]}")/../../recipes/common.sh"
ACTOR_GPUS="${ACTOR_GPUS:-1}"
ROLLOUT_GPUS="${ROLLOUT_GPUS:-$((NUM_GPUS - ACTOR_GPUS))}"
MODEL_ARGS=($(model_args qwen2.5-0.5B))
launch train_async.py "${MODEL_ARGS[@]}" \
  --hf-checkpoint "${CKPT_DIR}/Qwen2.5-0.5B-Instruct" --ref-load "${CKPT_DIR}/Qwen2.5-0.5B-Instruct_torch_dist" \
  --save /tmp/slime_fully_async_demo/ --save-interval 9999 \
  --rollout-function-path slime.rollout.fully_async_rollout.generate_rollout_fully_async \
  --prompt-data "${DATA_DIR}/dapo-math-17k/dapo-math-17k.jsonl" --input-key prompt --label-key label \
  --apply-chat-template --rollout-shuffle --rm-type deepscaler --num-rollout 3 --rollout-batch-size 8 \
  --n-samples-per-prompt 4 --rollout-max-response-len 1024 --rollout-temperature 1 --global-batch-size 32 --balance-data \
  --use-dynamic-batch-size --max-tokens-per-gpu 4096 \
  --advantage-estimator grpo --use-kl-loss --kl-loss-coef 0.0 --kl-loss-type low_var_kl --entropy-coef 0.0 \
  --eps-clip 0.2 --eps-clip-high 0.28 \
  --optimizer adam --lr 1e-6 --lr-decay-style constant --weight-decay 0.1 --adam-beta1 0.9 --adam-beta2 0.98 \
  --actor-num-nodes 1 --actor-num-gpus-per-node "${ACTOR_GPUS}" --rollout-num-gpus "${ROLLOUT_GPUS}" \
  --rollout-num-gpus-per-engine 1 --sglang-mem-fraction-static 0.55
