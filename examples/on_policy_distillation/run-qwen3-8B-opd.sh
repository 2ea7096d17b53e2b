#!/bin/bash
# On-policy distillation: the student (Qwen3-8B) samples, a stronger teacher scores the student's own tokens, and the
# per-token reverse KL to the teacher is subtracted from the advantages (--use-opd). Two teacher placements:
#   OPD_TYPE=megatron  the teacher's weights are loaded next to the student's in the trainer and swapped in for one
#                      forward pass per step (--opd-teacher-load)
#   OPD_TYPE=sglang    the teacher runs as an engine behind --rm-url; its log-probs arrive with the reward
source "$(dirname -- "${BASH_SOURCE[0]}")/../../recipes/common.sh"
OPD_TYPE="${OPD_TYPE:-megatron}"
MODEL_ARGS=($(model_args qwen3-8B))
if [ "${OPD_TYPE}" = "megatron" ]; then
  OPD_ARGS=(--opd-type megatron --opd-teacher-load "${CKPT_DIR}/Qwen3-32B_torch_dist")
else
  OPD_ARGS=(--opd-type sglang --rm-url "${TEACHER_URL:-http://127.0.0.1:13141/generate}"
            --custom-rm-path slime_b200.rollout.on_policy_distillation.reward_func
            --custom-reward-post-process-path slime_b200.rollout.on_policy_distillation.post_process_rewards)
fi
launch train.py "${MODEL_ARGS[@]}" \
  --hf-checkpoint "${CKPT_DIR}/Qwen3-8B" --ref-load "${CKPT_DIR}/Qwen3-8B_torch_dist" \
  --load "${CKPT_DIR}/Qwen3-8B_slime" --save "${CKPT_DIR}/Qwen3-8B_slime" --save-interval 20 \
  --prompt-data "${DATA_DIR}/dapo-math-17k/dapo-math-17k.jsonl" --input-key prompt --label-key label \
  --apply-chat-template --rollout-shuffle --num-rollout 300 --rollout-batch-size 16 --n-samples-per-prompt 4 \
  --rollout-max-response-len 16384 --rollout-temperature 1 --global-batch-size 64 --balance-data \
  --use-opd "${OPD_ARGS[@]}" --opd-kl-coef 1.0 \
  --advantage-estimator grpo --use-kl-loss --kl-loss-coef 0.0 --kl-loss-type low_var_kl --entropy-coef 0.0 \
  --eps-clip 0.2 --eps-clip-high 0.28 \
  --tensor-model-parallel-size 2 --sequence-parallel --use-dynamic-batch-size --max-tokens-per-gpu 16384 \
  --recompute-granularity full \
  --optimizer adam --lr 1e-6 --lr-decay-style constant --weight-decay 0.1 --adam-beta1 0.9 --adam-beta2 0.98 \
  --actor-num-nodes 1 --actor-num-gpus-per-node "${NUM_GPUS}" --colocate --rollout-num-gpus-per-engine 2 \
  --sglang-mem-fraction-static 0.6
