#!/bin/bash
# Qwen2.5-0.5B, colocated GRPO on one node: every GPU trains (data parallel) and serves rollouts (one engine per GPU).
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
MODEL_ARGS=($(model_args qwen2.5-0.5B))
launch train.py "${MODEL_ARGS[@]}" \
  --hf-checkpoint "${CKPT_DIR}/Qwen2.5-0.5B-Instruct" --ref-load "${CKPT_DIR}/Qwen2.5-0.5B-Instruct" \
  --save "${CKPT_DIR}/qwen2.5-0.5B-grpo" --save-interval 50 \
  --prompt-data "${DATA_DIR}/gsm8k/train.jsonl" --input-key messages --label-key label --apply-chat-template \
  --rollout-shuffle --rm-type math --num-rollout 200 --rollout-batch-size 32 --n-samples-per-prompt 8 \
  --rollout-max-response-len 1024 --rollout-temperature 1 --global-batch-size 256 \
  --eval-interval 20 --eval-prompt-data gsm8k "${DATA_DIR}/gsm8k/test.jsonl" --n-samples-per-eval-prompt 1 \
  --eval-max-response-len 1024 --eval-top-k 1 \
  --tensor-model-parallel-size 1 --use-dynamic-batch-size --max-tokens-per-gpu 16384 \
  --advantage-estimator grpo --use-kl-loss --kl-loss-coef 0.0 --kl-loss-type low_var_kl --entropy-coef 0.0 \
  --eps-clip 0.2 --eps-clip-high 0.28 \
  --optimizer adam --lr 1e-6 --lr-decay-style constant --weight-decay 0.1 --adam-beta1 0.9 --adam-beta2 0.98 \
  --actor-num-nodes 1 --actor-num-gpus-per-node "${NUM_GPUS}" --colocate --rollout-num-gpus-per-engine 1 \
  --sglang-mem-fraction-static 0.6 --attention-dropout 0.0 --hidden-dropout 0.0 \
  --accumulate-allreduce-grads-in-fp32 --attention-softmax-in-fp32
