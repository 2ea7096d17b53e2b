#!/bin/bash
# Supervised fine-tuning of Qwen3-4B-Base on chat transcripts: the "rollout" only tokenises conversations and builds
# the assistant-token loss mask (sft_rollout), no engine is started (--debug-train-only), loss = token-level NLL.
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
MODEL_ARGS=($(model_args qwen3-4B))
launch train_async.py "${MODEL_ARGS[@]}" \
  --hf-checkpoint "${CKPT_DIR}/Qwen3-4B-Base" --ref-load "${CKPT_DIR}/Qwen3-4B-Base_torch_dist" \
  --load "${CKPT_DIR}/Qwen3-4B-Base_slime" --save "${CKPT_DIR}/Qwen3-4B-Base_slime" --save-interval 1000 \
  --rollout-function-path slime.rollout.sft_rollout.generate_rollout \
  --prompt-data "${DATA_DIR}/openhermes2_5/openhermes2_5.parquet" --input-key messages --rollout-shuffle --num-epoch 3 \
  --rollout-batch-size 128 --global-batch-size 128 \
  --loss-type sft_loss --calculate-per-token-loss --disable-compute-advantages-and-returns --debug-train-only \
  --tensor-model-parallel-size 1 --recompute-granularity full --recompute-method uniform --recompute-num-layers 1 \
  --use-dynamic-batch-size --max-tokens-per-gpu 9216 \
  --optimizer adam --lr 1e-5 --lr-decay-style cosine --min-lr 1e-6 --lr-warmup-fraction 0.1 --weight-decay 0.1 \
  --adam-beta1 0.9 --adam-beta2 0.95 \
  --actor-num-nodes 1 --actor-num-gpus-per-node "${NUM_GPUS}" \
  --attention-dropout 0.0 --hidden-dropout 0.0 --accumulate-allreduce-grads-in-fp32 --attention-softmax-in-fp32
