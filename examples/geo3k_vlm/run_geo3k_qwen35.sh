#!/bin/bash
# Vision-language RL on Geometry-3K: prompts carry images (`--multimodal-keys`), the processor turns them into pixel
# tensors that travel with the sample (`multimodal_inputs` for the engine, `multimodal_train_inputs` for the trainer).
# Checkpoints whose config has a `vision_config` of the Qwen3-VL / Qwen3.5 kind get the built-in vision tower on both
# sides (trainer: inside the model; engine: `image_data`); other towers come in through --custom-model-provider-path.
source "$(dirname -- "${BASH_SOURCE[0]}")/../../recipes/common.sh"
launch train.py \
  --hf-checkpoint "${CKPT_DIR}/${VLM_MODEL:-Qwen3.5-35B-A3B}" ${VLM_PROVIDER:+--custom-model-provider-path "${VLM_PROVIDER}"} \
  --prompt-data "${DATA_DIR}/geo3k/train.parquet" --input-key problem --label-key answer \
  --multimodal-keys '{"image": "images"}' --apply-chat-template --rollout-shuffle --rm-type math \
  --num-rollout 300 --rollout-batch-size 32 --n-samples-per-prompt 8 --rollout-max-response-len 4096 \
  --rollout-temperature 1 --global-batch-size 256 \
  --use-dynamic-batch-size --max-tokens-per-gpu 8192 \
  --advantage-estimator grpo --eps-clip 0.2 --eps-clip-high 0.28 \
  --optimizer adam --lr 1e-6 --lr-decay-style constant --weight-decay 0.1 --adam-beta1 0.9 --adam-beta2 0.98 \
  --actor-num-nodes 1 --actor-num-gpus-per-node "${NUM_GPUS}" --colocate --rollout-num-gpus-per-engine 1 \
  --sglang-mem-fraction-static 0.6
