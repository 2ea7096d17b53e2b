#!/bin/bash
# Supervised fine-tuning of Qwen3-235B-A22B on OpenHermes-2.5 chat data on 4 nodes x 8 GPUs: TP4 + SP, PP4 (last stage 22 layers), EP8,
# CPU Adam. No rollout engines are started.
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
MODEL_ARGS=($(model_args qwen3-235B-A22B))
launch train_async.py "${MODEL_ARGS[@]}" --hf-checkpoint "${CKPT_DIR}/Qwen3-235B-A22B" --load "${CKPT_DIR}/Qwen3-235B-A22B_slime" --save "${CKPT_DIR}/Qwen3-235B-A22B_slime" \
  --save-interval 1000 --prompt-data "${DATA_DIR}/openhermes2_5/openhermes2_5.parquet" --input-key messages --rollout-shuffle \
  --rollout-function-path slime_b200.rollout.sft_rollout.generate_rollout --loss-type sft_loss --loss-mask-type qwen3 \
  --calculate-per-token-loss --disable-compute-advantages-and-returns --debug-train-only --num-epoch 3 \
  --rollout-batch-size 128 --global-batch-size 128 --tensor-model-parallel-size 4 --sequence-parallel --pipeline-model-parallel-size 4 --decoder-last-pipeline-num-layers 22 --expert-model-parallel-size 8 --expert-tensor-parallel-size 1 \
  "${RECOMPUTE_ARGS[@]}" --use-dynamic-batch-size --max-tokens-per-gpu 9216 \
  --optimizer adam --lr 1e-5 --lr-decay-style cosine --min-lr 1e-6 --lr-warmup-fraction 0.1 --weight-decay 0.1 --adam-beta1 0.9 \
  --adam-beta2 0.95 --optimizer-cpu-offload --overlap-cpu-optimizer-d2h-h2d --use-precision-aware-optimizer "${MISC_ARGS[@]}" \
  --actor-num-nodes "${NUM_NODES:-4}" --actor-num-gpus-per-node 8
