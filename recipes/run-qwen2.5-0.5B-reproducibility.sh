#!/bin/bash
# Bit-reproducible GRPO on Qwen2.5-0.5B: fixed seeds, deterministic trainer kernels (fixed summation orders; the
# attention backward and the peer-memory collectives of this package use no atomics), deterministic engine sampling
# (per-request seeds, batch-invariant reductions), rank-order NCCL rings.
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
export NCCL_ALGO=Ring
export CUBLAS_WORKSPACE_CONFIG=:4096:8
MODEL_ARGS=($(model_args qwen2.5-0.5B))
launch train.py "${MODEL_ARGS[@]}" \
  --hf-checkpoint "${CKPT_DIR}/Qwen2.5-0.5B-Instruct" --ref-load "${CKPT_DIR}/Qwen2.5-0.5B-Instruct" \
  --prompt-data "${DATA_DIR}/gsm8k/train.jsonl" --input-key messages --label-key label --apply-chat-template \
  --rm-type math --num-rollout 100 --rollout-batch-size 32 --n-samples-per-prompt 8 --rollout-max-response-len 1024 \
  --rollout-temperature 1 --global-batch-size 256 --seed 1234 --rollout-seed 42 \
  --deterministic-mode --sglang-enable-deterministic-inference \
  --eval-interval 20 --eval-prompt-data gsm8k "${DATA_DIR}/gsm8k/test.jsonl" --n-samples-per-eval-prompt 1 \
  --eval-max-response-len 1024 --eval-top-k 1 \
  --use-dynamic-batch-size --max-tokens-per-gpu 9216 \
  --advantage-estimator grpo --use-kl-loss --kl-loss-coef 0.0 --kl-loss-type low_var_kl --entropy-coef 0.0 \
  --eps-clip 0.2 --eps-clip-high 0.28 \
  --optimizer adam --lr 1e-6 --lr-decay-style constant --weight-decay 0.1 --adam-beta1 0.9 --adam-beta2 0.98 \
  --actor-num-nodes 1 --actor-num-gpus-per-node "${NUM_GPUS}" --colocate --rollout-num-gpus-per-engine 1 \
  --sglang-mem-fraction-static 0.7 --attention-dropout 0.0 --hidden-dropout 0.0 \
  --accumulate-allreduce-grads-in-fp32 --attention-softmax-in-fp32
