#!/bin/bash
# Qwen3-32B on 8 GPUs, disaggregated and asynchronous: trainer TP4 (+ sequence parallel) on GPUs 0-3, one TP4 rollout
# engine on GPUs 4-7, rollout k+1 overlaps training step k, all 32 B parameters pushed trainer -> engine every step.
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
MODEL_ARGS=($(model_args qwen3-32B))
launch train_async.py "${MODEL_ARGS[@]}" \
  --hf-checkpoint "${CKPT_DIR}/Qwen3-32B" --ref-load "${CKPT_DIR}/Qwen3-32B_torch_dist" \
  --load "${CKPT_DIR}/Qwen3-32B_slime" --save "${CKPT_DIR}/Qwen3-32B_slime" --save-interval 20 \
  --prompt-data "${DATA_DIR}/dapo-math-17k/dapo-math-17k.jsonl" --input-key prompt --label-key label \
  --apply-chat-template --rollout-shuffle --rm-type deepscaler --num-rollout 3000 --rollout-batch-size 32 \
  --n-samples-per-prompt 8 --rollout-max-response-len 4096 --rollout-temperature 1 --global-batch-size 256 --balance-data \
  --eval-interval 20 --eval-prompt-data aime "${DATA_DIR}/aime-2024/aime-2024.jsonl" --n-samples-per-eval-prompt 16 \
  --eval-max-response-len 16384 --eval-top-p 1 \
  --tensor-model-parallel-size 4 --sequence-parallel --pipeline-model-parallel-size 1 --context-parallel-size 1 \
  --recompute-granularity full --recompute-method uniform --recompute-num-layers 1 \
  --use-dynamic-batch-size --max-tokens-per-gpu 8192 \
  --advantage-estimator grpo --use-kl-loss --kl-loss-coef 0.0 --kl-loss-type low_var_kl --entropy-coef 0.0 \
  --eps-clip 0.2 --eps-clip-high 0.28 --use-tis \
  --optimizer adam --lr 1e-6 --lr-decay-style constant --weight-decay 0.1 --adam-beta1 0.9 --adam-beta2 0.98 \
  --actor-num-nodes 1 --actor-num-gpus-per-node 4 --rollout-num-gpus 4 --rollout-num-gpus-per-engine 4 \
  --sglang-mem-fraction-static 0.8 --attention-dropout 0.0 --hidden-dropout 0.0 \
  --accumulate-allreduce-grads-in-fp32 --attention-softmax-in-fp32
