#!/bin/bash
# Delta weight sync for disaggregated rollout: the trainer publishes, per version, only the bytes that changed (xor or
# overwrite patches, checksummed and compressed) into a shared directory; every rollout node keeps a local
# checkpoint, applies the patch chain to reach the requested version, and reloads from local disk.
#   SHARED_DIR   a filesystem every node can read (patches live here)
#   LOCAL_DIR    node-local disk holding the rollout nodes' materialised checkpoint
source "$(dirname -- "${BASH_SOURCE[0]}")/../../recipes/common.sh"
SHARED_DIR="${SHARED_DIR:-/shared/fs/slime-delta-updates}"
LOCAL_DIR="${LOCAL_DIR:-/local/nvme/slime-rollout-ckpt}"
MODEL_ARGS=($(model_args qwen3-30B-A3B))
launch train_async.py "${MODEL_ARGS[@]}" \
  --hf-checkpoint "${CKPT_DIR}/Qwen3-30B-A3B" --ref-load "${CKPT_DIR}/Qwen3-30B-A3B_torch_dist" \
  --prompt-data "${DATA_DIR}/dapo-math-17k/dapo-math-17k.jsonl" --input-key prompt --label-key label \
  --apply-chat-template --rollout-shuffle --rm-type deepscaler --num-rollout 3000 --rollout-batch-size 32 \
  --n-samples-per-prompt 8 --rollout-max-response-len 8192 --rollout-temperature 1 --global-batch-size 256 \
  --update-weight-mode delta --update-weight-transport disk --update-weight-disk-dir "${SHARED_DIR}" \
  --update-weight-local-checkpoint-dir "${LOCAL_DIR}" --update-weight-delta-encoding xor \
  --update-weight-delta-checksum xxh3-128 \
  --tensor-model-parallel-size 4 --sequence-parallel --expert-model-parallel-size 8 --expert-tensor-parallel-size 1 \
  --use-dynamic-batch-size --max-tokens-per-gpu 20480 --recompute-granularity full \
  --advantage-estimator grpo --eps-clip 0.2 --eps-clip-high 0.28 \
  --optimizer adam --lr 1e-6 --lr-decay-style constant --weight-decay 0.1 --adam-beta1 0.9 --adam-beta2 0.98 \
  --actor-num-nodes 1 --actor-num-gpus-per-node 8 --rollout-num-gpus 8 --rollout-num-gpus-per-engine 8 \
  --sglang-mem-fraction-static 0.8 --sglang-ep-size 8
