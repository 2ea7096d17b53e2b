#!/bin/bash
# Qwen3-8B on 8 GPUs, colocated, PPO with a critic of the same architecture (the critic is a second train group on the
# same GPUs; its values feed GAE), trainer TP2 + SP x DP4, engines of 2 GPUs.
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
MODEL_ARGS=($(model_args qwen3-8B))
launch train.py "${MODEL_ARGS[@]}" \
  --hf-checkpoint "${CKPT_DIR}/Qwen3-8B" --ref-load "${CKPT_DIR}/Qwen3-8B_torch_dist" \
  --num-critic-only-steps 5 \
  --load "${CKPT_DIR}/Qwen3-8B_slime" --save "${CKPT_DIR}/Qwen3-8B_slime" --save-interval 20 \
  --prompt-data "${DATA_DIR}/dapo-math-17k/dapo-math-17k.jsonl" --input-key prompt --label-key label \
  --apply-chat-template --rollout-shuffle --rm-type deepscaler --num-rollout 3000 --rollout-batch-size 32 \
  --n-samples-per-prompt 8 --rollout-max-response-len 8192 --rollout-temperature 1 --global-batch-size 256 --balance-data \
  --tensor-model-parallel-size 2 --sequence-parallel --recompute-granularity full --recompute-method uniform \
  --recompute-num-layers 1 --use-dynamic-batch-size --max-tokens-per-gpu 9216 \
  --advantage-estimator ppo --gamma 1.0 --lambd 1.0 --eps-clip 0.2 --eps-clip-high 0.28 --value-clip 0.2 \
  --kl-coef 0.0 --entropy-coef 0.0 \
  --optimizer adam --lr 1e-6 --lr-decay-style constant --weight-decay 0.1 --adam-beta1 0.9 --adam-beta2 0.98 \
  --actor-num-nodes 1 --actor-num-gpus-per-node "${NUM_GPUS}" --colocate --rollout-num-gpus-per-engine 2 \
  --sglang-mem-fraction-static 0.6 --attention-dropout 0.0 --hidden-dropout 0.0 \
  --accumulate-allreduce-grads-in-fp32 --attention-softmax-in-fp32
