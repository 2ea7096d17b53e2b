#!/bin/bash
# Shared by the run recipes: resolves paths, turns a model preset into architecture flags, launches train.py.
#   DATA_DIR      where prompt / eval sets live           (default /root/data)
#   CKPT_DIR      where checkpoints are read and written  (default /root/ckpt)
#   NUM_GPUS      GPUs of this node used by the job       (default: all visible)
#   DRY_RUN=1     print the command line instead of running it (one argument per line)
set -euo pipefail
REPO_ROOT="$(cd -- "$(dirname -- "${BASH_SOURCE[0]}")/.." && pwd)"
DATA_DIR="${DATA_DIR:-/root/data}"
CKPT_DIR="${CKPT_DIR:-/root/ckpt}"
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
