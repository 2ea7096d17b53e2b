#!/bin/bash
# Shared by the run recipes: resolves paths, turns a model preset into architecture flags, launches train.py.
#   DATA_DIR      where prompt / eval sets live           (default ~/data)
#   CKPT_DIR      where checkpoints are read and written  (default ~/ckpt)
#   NUM_GPUS      GPUs of this node used by the job       (default: all visible)
#   DRY_RUN=1     print the command line instead of running it (one argument per line)
set -euo pipefail
REPO_ROOT="$(cd -- "$(dirname -- "${BASH_SOURCE[0]}")/.." && pwd)"
DATA_DIR="${DATA_DIR:-${HOME}/data}"
CKPT_DIR="${CKPT_DIR:-${HOME}/ckpt}"
if [ -z "${NUM_GPUS:-}" ]; then
  NUM_GPUS=$(python -c 'import torch; print(max(torch.cuda.device_count(), 1))')
fi
export MASTER_ADDR="${MASTER_ADDR:-127.0.0.1}"
export PYTHONPATH="${REPO_ROOT}:${PYTHONPATH:-}"

model_args() { python -m slime_b200.models.presets "$1"; }

launch() {  # launch <train.py|train_async.py> args...
  local entry="$1"; shift
  if [ "${DRY_RUN:-0}" = "1" ]; then
    printf '%s\n' "$entry" "$@"
  else
    exec python "${REPO_ROOT}/${entry}" "$@"
  fi
}

# Flag groups shared by the larger recipes (the small ones spell everything out).
DAPO_ROLLOUT_ARGS=(--prompt-data "${DATA_DIR}/dapo-math-17k/dapo-math-17k.jsonl" --input-key prompt --label-key label
  --apply-chat-template --rollout-shuffle --rm-type deepscaler --num-rollout 3000 --rollout-temperature 1 --balance-data)
AIME_EVAL_ARGS=(--eval-interval 20 --eval-prompt-data aime "${DATA_DIR}/aime-2024/aime-2024.jsonl" --eval-top-p 1)
GRPO_ARGS=(--advantage-estimator grpo --use-kl-loss --kl-loss-coef 0.0 --kl-loss-type low_var_kl --entropy-coef 0.0
  --eps-clip 0.2 --eps-clip-high 0.28)
ADAM_ARGS=(--optimizer adam --lr 1e-6 --lr-decay-style constant --weight-decay 0.1 --adam-beta1 0.9 --adam-beta2 0.98)
CPU_ADAM_ARGS=("${ADAM_ARGS[@]}" --optimizer-cpu-offload --overlap-cpu-optimizer-d2h-h2d --use-precision-aware-optimizer)
RECOMPUTE_ARGS=(--recompute-granularity full --recompute-method uniform --recompute-num-layers 1)
MISC_ARGS=(--attention-dropout 0.0 --hidden-dropout 0.0 --accumulate-allreduce-grads-in-fp32 --attention-softmax-in-fp32
  --attention-backend flash)
DYNAMIC_SAMPLING_ARGS=(--over-sampling-batch-size 256
  --dynamic-sampling-filter-path slime_b200.rollout.filter_hub.dynamic_sampling_filters.check_reward_nonzero_std)
ckpt_args() {  # ckpt_args <hf dir name>: checkpoint to start from, reference weights, where training state goes
  echo --hf-checkpoint "${CKPT_DIR}/$1" --ref-load "${CKPT_DIR}/$1_torch_dist" --load "${CKPT_DIR}/$1_slime" \
       --save "${CKPT_DIR}/$1_slime" --save-interval 20
}
