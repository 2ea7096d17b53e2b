#!/bin/bash
# Qwen3-235B-A22B on 4 nodes x 8 GPUs, colocated: trainer TP4 + SP, PP4, EP8 (expert TP1), CPU-offloaded Adam;
# rollout engines of 32 GPUs with expert parallelism; fp8 rollout weights quantised during the sync.
#   NUM_NODES / NODE_RANK / MASTER_ADDR are taken from the environment of each node.
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
NUM_NODES="${NUM_NODES:-4}"
MODEL_ARGS=($(model_args qwen3-235B-A22B))
launch train.py "${MODEL_ARGS[@]}" \
  --hf-checkpoint "${CKPT_DIR}/Qwen3-235B-A22B" --ref-load "${CKPT_DIR}/Qwen3-235B-A22B_torch_dist" \
  --load "${CKPT_DIR}/Qwen3-235B-A22B_slime" --save "${CKPT_DIR}/Qwen3-235B-A22B_slime" --save-interval 20 \
  --prompt-data "${DATA_DIR}/dapo-math-17k/dapo-math-17k.jsonl" --input-key prompt --label-key label \
  --apply-chat-template --rollout-shuffle --rm-type deepscaler --num-rollout 3000 --rollout-batch-size 32 \
  --n-samples-per-prompt 8 --rollout-max-response-len 8192 --rollout-temperature 1 --global-batch-size 256 --balance-data \
  --tensor-model-parallel-size 4 --sequence-parallel --pipeline-model-parallel-size 4 --context-parallel-size 1 \
  --expert-model-parallel-size 8 --expert-tensor-parallel-size 1 \
  --decoder-last-pipeline-num-layers 22 \
  --recompute-granularity full --recompute-method uniform --recompute-num-layers 1 \
  --use-dynamic-batch-size --max-tokens-per-gpu 4096 \
  --advantage-estimator gspo --eps-clip 3e-4 --eps-clip-high 4e-4 --kl-loss-coef 0.0 --entropy-coef 0.0 \
  --optimizer adam --lr 1e-6 --lr-decay-style constant --weight-decay 0.1 --adam-beta1 0.9 --adam-beta2 0.98 \
  --optimizer-cpu-offload --overlap-cpu-optimizer-d2h-h2d --use-precision-aware-optimizer \
  --actor-num-nodes "${NUM_NODES}" --actor-num-gpus-per-node 8 --colocate --rollout-num-gpus-per-engine 32 \
  --sglang-mem-fraction-static 0.7 --sglang-ep-size 32 --sglang-quantization fp8 \
  --attention-dropout 0.0 --hidden-dropout 0.0 --accumulate-allreduce-grads-in-fp32 --attention-softmax-in-fp32
