#!/bin/bash
# Geometry-3K with images over several turns: the model may check an answer with a scoring tool and revise it.
# The model's own vision tower is used on both sides (trainer: models/vision.py inside the model; engine: image_data).
source "$(dirname -- "${BASH_SOURCE[0]}")/../../recipes/common.sh"
HERE="$(dirname -- "${BASH_SOURCE[0]}")"
launch train.py \
  --hf-checkpoint "${CKPT_DIR}/${VLM_MODEL:-Qwen3.5-35B-A3B}" --ref-load "${CKPT_DIR}/${VLM_MODEL:-Qwen3.5-35B-A3B}" \
  --prompt-data "${DATA_DIR}/geo3k_imgurl/train.parquet" --input-key problem --label-key answer \
  --multimodal-keys '{"image": "images"}' --apply-chat-template --rollout-shuffle --rm-type math \
  --custom-generate-function-path examples.geo3k_vlm_multi_turn.rollout.generate \
  --custom-config-path "${HERE}/config.yaml" \
  --num-rollout 3000 --rollout-batch-size 64 --n-samples-per-prompt 8 --rollout-max-response-len 4096 \
  --rollout-max-context-len 8192 --rollout-temperature 1 --global-batch-size 512 \
  --eval-interval 20 --eval-prompt-data geo3k "${DATA_DIR}/geo3k_imgurl/test.parquet" --n-samples-per-eval-prompt 1 \
  --eval-max-response-len 4096 \
  --tensor-model-parallel-size "${TP:-2}" --sequence-parallel --use-dynamic-batch-size --max-tokens-per-gpu 8192 \
  --advantage-estimator grpo --eps-clip 0.2 --eps-clip-high 0.28 --use-kl-loss --kl-loss-coef 0.0 --entropy-coef 0.0 \
  --optimizer adam --lr 1e-6 --lr-decay-style constant --weight-decay 0.1 --adam-beta1 0.9 --adam-beta2 0.98 \
  --actor-num-nodes 1 --actor-num-gpus-per-node "${NUM_GPUS}" --colocate --rollout-num-gpus-per-engine 1 \
  --sglang-mem-fraction-static 0.6
