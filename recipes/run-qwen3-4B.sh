#!/bin/bash
# Qwen3-4B on 8 GPUs, colocated: trainer TP2 (+ sequence parallel) x DP4 with full recomputation and token-budgeted
# micro-batches; rollout engines of 2 GPUs each; GRPO with asymmetric clipping; DAPO-math prompts, AIME evaluation.
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
MODEL_ARGS=($(model_args qwen3-4B))
launch train.py "${MODEL_ARGS[@]}" \
  --hf-checkpoint "${CKPT_DIR}/Qwen3-4B" --ref-load "${CKPT_DIR}/Qwen3-4B_torch_dist" \
  --load "${CKPT_DIR}/Qwen3-4B_slime" --save "${CKPT_DIR}/Qwen3-4B_slime" --save-interval 20 \
  --prompt-data "${DATA_DIR}/dapo-math-17k/dapo-math-17k.jsonl" --input-key prompt --label-key label \
  --apply-chat-template --rollout-shuffle --rm-type deepscaler --num-rollout 3000 --rollout-batch-size 32 \
  --n-samples-per-prompt 8 --rollout-max-response-len 8192 --rollout-temperature 1 --global-batch-size 256 --balance-data \
  --eval-interval 20 --eval-prompt-data aime "${DATA_DIR}/aime-2024/aime-2024.jsonl" --n-samples-per-eval-prompt 16 \
  --eval-max-response-len 16384 --eval-top-p 1 \
  --tensor-model-parallel-size 2 --sequence-parallel --pipeline-model-parallel-size 1 --context-parallel-size 1 \
  --recompute-granularity full --recompute-method uniform --recompute-num-layers 1 \
  --use-dynamic-batch-size --max-tokens-per-gpu 9216 \
  --advantage-estimator grpo --use-kl-loss --kl-loss-coef 0.0 --kl-loss-type low_var_kl --entropy-coef 0.0 \
  --eps-clip 0.2 --eps-clip-high 0.28 \
  --optimizer adam --lr 1e-6 --lr-decay-style constant --weight-decay 0.1 --adam-beta1 0.9 --adam-beta2 0.98 \
  --actor-num-nodes 1 --actor-num-gpus-per-node "${NUM_GPUS}" --colocate --rollout-num-gpus-per-engine 2 \
  --sglang-mem-fraction-static 0.7 --attention-dropout 0.0 --hidden-dropout 0.0 \
  --accumulate-allreduce-grads-in-fp32 --attention-softmax-in-fp32 --attention-backend flash
