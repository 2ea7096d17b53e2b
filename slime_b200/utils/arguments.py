"""Command-line surface: one ``argparse.Namespace`` for driver, trainer and engines.

Three flag families are merged (parity: slime/utils/arguments.py:1600-1643):
  * framework flags (cluster, rollout, data, algorithm, logging, debug, ...),
    with the names and defaults of slime/utils/arguments.py:38-1547;
  * training-backend flags with the Megatron names the shipped recipes use
    (model shape, parallel sizes, optimizer, recompute, checkpoint);
  * rollout-engine flags, every field of ``engine.server_args.ServerArgs``
    registered as ``--sglang-<field>`` plus ``--sglang-router-*``.

Flags are declared in tables (``_FLAGS``) instead of hand-written
``add_argument`` calls; ``slime_validate_args`` derives dependent settings.
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import logging
import os
from typing import Any

import yaml

logger = logging.getLogger(__name__)

B = argparse.BooleanOptionalAction
_T = "store_true"
_F = "store_false"


def _f(name, **kw):
    return (name, kw)


# fmt: off
_CLUSTER = [
    _f("--actor-num-nodes", type=int, default=1), _f("--actor-num-gpus-per-node", type=int, default=8),
    _f("--critic-num-nodes", type=int, default=None), _f("--critic-num-gpus-per-node", type=int, default=None),
    _f("--rollout-num-gpus", type=int, default=None), _f("--rollout-num-gpus-per-engine", type=int, default=1),
    _f("--num-gpus-per-node", type=int, default=8), _f("--colocate", action=_T), _f("--offload", action=_T),
    _f("--offload-train", action=B, default=None), _f("--offload-rollout", action=B, default=None),
    _f("--release-communicators-on-sleep", action=B, default=False),
]
_TRAIN = [
    _f("--train-backend", type=str, choices=["megatron", "b200"], default="megatron"),
    _f("--qwen-gdn-backend", type=str, choices=["fla", "flashqla"], default="fla"),
    _f("--train-env-vars", type=json.loads, default={}),
    _f("--update-weight-mode", choices=["full", "delta"], default="full"),
    _f("--update-weight-transport", choices=["nccl", "disk", "p2p"], default="nccl"),
    _f("--release-train", action=_T), _f("--update-weight-disk-dir", type=str, default=None),
    _f("--update-weight-disk-keep-files", action=_T),
    _f("--update-weight-delta-encoding", choices=["xor", "overwrite"], default="xor"),
    _f("--update-weight-delta-checksum", choices=["xxh3-128", "blake3", "adler32"], default="xxh3-128"),
    _f("--custom-update-weight-post-write-path", type=str, default=None),
    _f("--update-weight-local-checkpoint-dir", type=str, default=None),
    _f("--custom-model-provider-path", type=str, default=None), _f("--recompute-loss-function", action=_T),
    _f("--log-probs-chunk-size", type=int, default=-1),
    _f("--only-train-params-name-list", type=str, nargs="*", default=None),
    _f("--freeze-params-name-list", type=str, nargs="*", default=None),
    _f("--freeze-indexer", action=_T), _f("--allgather-cp", action=_T),
]
_ROLLOUT = [
    _f("--hf-checkpoint", type=str, default=None), _f("--model-name", type=str, default=None),
    _f("--rollout-function-path", type=str, default="slime.rollout.sglang_rollout.generate_rollout"),
    _f("--rollout-temperature", type=float, default=1.0), _f("--rollout-top-p", type=float, default=1.0),
    _f("--rollout-top-k", type=int, default=-1), _f("--rollout-max-context-len", type=int, default=None),
    _f("--rollout-max-prompt-len", type=int, default=None), _f("--rollout-max-response-len", type=int, default=None),
    _f("--rollout-min-new-tokens", type=int, default=None), _f("--rollout-ignore-eos", action=_T),
    _f("--rollout-skip-special-tokens", action=_T), _f("--rollout-stop", type=str, nargs="+", default=None),
    _f("--rollout-stop-token-ids", type=int, nargs="+", default=None), _f("--rollout-shuffle", action=_T),
    _f("--rollout-seed", type=int, default=42), _f("--over-sampling-batch-size", type=int, default=None),
    _f("--dynamic-sampling-filter-path", type=str, default=None), _f("--partial-rollout", action=_T),
    _f("--mask-offpolicy-in-partial-rollout", action=_T), _f("--custom-generate-function-path", type=str, default=None),
    _f("--rollout-sample-hook-path", action="append", default=[]),
    _f("--custom-rollout-log-function-path", type=str, default=None),
    _f("--custom-eval-rollout-log-function-path", type=str, default=None),
    _f("--buffer-filter-path", type=str, default=None),
    _f("--update-weight-buffer-size", type=int, default=512 * 1024**2),
    _f("--update-weights-interval", type=int, default=1), _f("--keep-old-actor", action=_T),
    _f("--rollout-data-postprocess-path", type=str, default=None),
    _f("--rollout-data-transport", type=str, choices=["object-store", "nixl"], default="object-store"),
    _f("--rollout-external-engine-addrs", type=str, nargs="+", default=None),
]
_FAULT = [
    _f("--use-fault-tolerance", action=_T), _f("--rollout-health-check-interval", type=float, default=30.0),
    _f("--rollout-health-check-timeout", type=float, default=30.0),
    _f("--rollout-health-check-first-wait", type=float, default=0),
]
_DATA = [
    _f("--num-rollout", type=int, default=None), _f("--num-epoch", type=int, default=None),
    _f("--disable-rollout-global-dataset", action=_F, dest="rollout_global_dataset"),
    _f("--data-source-path", type=str, default="slime.rollout.data_source.RolloutDataSourceWithBuffer"),
    _f("--prompt-data", type=str, default=None), _f("--apply-chat-template", action=_T),
    _f("--apply-chat-template-kwargs", type=json.loads, default={}), _f("--input-key", type=str, default="input"),
    _f("--label-key", type=str, default=None), _f("--multimodal-keys", type=json.loads, default=None),
    _f("--metadata-key", type=str, default="metadata"), _f("--tool-key", type=str, default="tools"),
    _f("--start-rollout-id", type=int, default=None), _f("--rollout-batch-size", type=int, required=True),
    _f("--n-samples-per-prompt", type=int, default=1), _f("--global-batch-size", type=int, default=None),
    _f("--num-steps-per-rollout", type=int, default=None), _f("--micro-batch-size", type=int, default=1),
    _f("--balance-data", action=_T), _f("--balance-by-flops", action=_T), _f("--use-dynamic-batch-size", action=_T),
    _f("--max-tokens-per-gpu", type=int, default=None), _f("--log-probs-max-tokens-per-gpu", type=int, default=None),
]
_EVAL = [
    _f("--eval-function-path", type=str, default=None), _f("--eval-interval", type=int, default=None),
    _f("--eval-prompt-data", type=str, nargs="+", default=None), _f("--eval-config", type=str, default=None),
    _f("--skip-eval-before-train", action=_T), _f("--eval-input-key", type=str, default=None),
    _f("--eval-label-key", type=str, default=None), _f("--eval-tool-key", type=str, default=None),
    _f("--n-samples-per-eval-prompt", type=int, default=1), _f("--eval-temperature", type=float, default=None),
    _f("--eval-top-p", type=float, default=None), _f("--eval-top-k", type=int, default=None),
    _f("--eval-max-response-len", type=int, default=None), _f("--eval-max-prompt-len", type=int, default=None),
    _f("--eval-min-new-tokens", type=int, default=None), _f("--eval-max-context-len", type=int, default=None),
]
_ALGO = [
    _f("--ref-load", type=str, default=None), _f("--ref-ckpt-step", type=int, default=None),
    _f("--load", type=str, default=None), _f("--save", type=str, default=None),
    _f("--save-interval", type=int, default=None), _f("--async-save", action=_T), _f("--no-save-optim", action=_T),
    _f("--no-load-optim", action=_T), _f("--no-load-rng", action=_T), _f("--no-save-rng", action=_T),
    _f("--finetune", action=_T), _f("--ckpt-step", type=int, default=None), _f("--ckpt-format", type=str, default="torch_dist"),
    _f("--save-hf", type=str, default=None), _f("--seed", type=int, default=1234),
    _f("--clip-grad", type=float, default=1.0), _f("--calculate-per-token-loss", action=_T),
    _f("--lr", type=float, default=1e-6), _f("--num-critic-only-steps", type=int, default=0),
    _f("--megatron-config-path", type=str, default=None), _f("--eps-clip", type=float, default=0.2),
    _f("--eps-clip-high", type=float, default=None), _f("--eps-clip-c", type=float, default=None),
    _f("--value-clip", type=float, default=0.2), _f("--kl-coef", type=float, default=0.0),
    _f("--loss-type", type=str, choices=["policy_loss", "sft_loss", "custom_loss"], default="policy_loss"),
    _f("--custom-loss-function-path", type=str, default=None),
    _f("--kl-loss-type", type=str, choices=["k1", "k2", "k3", "low_var_kl"], default="k1"),
    _f("--advantage-estimator", type=str, default="grpo",
       choices=["grpo", "gspo", "cispo", "reinforce_plus_plus", "reinforce_plus_plus_baseline", "ppo"]),
    _f("--disable-compute-advantages-and-returns", action=_F, dest="compute_advantages_and_returns"),
    _f("--custom-advantage-function-path", type=str, default=None), _f("--use-kl-loss", action=_T),
    _f("--kl-loss-coef", type=float, default=0.0), _f("--use-unbiased-kl", action=_T),
    _f("--ref-update-interval", type=int, default=None), _f("--entropy-coef", type=float, default=0.0),
    _f("--gamma", type=float, default=1.0), _f("--lambd", type=float, default=1.0),
    _f("--normalize-advantages", action=_T),
    _f("--disable-grpo-std-normalization", action=_F, dest="grpo_std_normalization"),
    _f("--disable-rewards-normalization", action=_F, dest="rewards_normalization"),
    _f("--use-rollout-entropy", action=_T), _f("--get-mismatch-metrics", action=_T),
    _f("--reset-optimizer-states", action=_T), _f("--use-stateless-adam", action=_T),
    _f("--use-rollout-logprobs", action=_T), _f("--use-tis", action=_T), _f("--tis-clip", type=float, default=2.0),
    _f("--tis-clip-low", type=float, default=0), _f("--custom-tis-function-path", type=str, default=None),
    _f("--custom-pg-loss-reducer-function-path", type=str, default=None), _f("--use-routing-replay", action=_T),
    _f("--use-rollout-routing-replay", action=_T), _f("--use-opsm", action=_T),
    _f("--opsm-delta", type=float, default=1e-4),
    _f("--use-opd", action=_T), _f("--opd-type", type=str, choices=["sglang", "megatron"], default=None),
    _f("--opd-kl-coef", type=float, default=1.0), _f("--opd-teacher-load", type=str, default=None),
    _f("--opd-teacher-ckpt-step", type=int, default=None),
]
_LOG = [
    _f("--use-wandb", action=_T), _f("--wandb-mode", type=str, default=None, choices=["online", "offline", "disabled"]),
    _f("--wandb-dir", type=str, default=None), _f("--wandb-key", type=str, default=None),
    _f("--wandb-host", type=str, default=None), _f("--wandb-team", type=str, default=None),
    _f("--wandb-group", type=str, default=None), _f("--wandb-project", type=str, default=None),
    _f("--disable-wandb-random-suffix", action=_F, dest="wandb_random_suffix"),
    _f("--wandb-always-use-train-step", action=_T), _f("--log-multi-turn", action=_T), _f("--log-passrate", action=_T),
    _f("--log-reward-category", type=str, default=None), _f("--log-correct-samples", action=_T),
    _f("--wandb-run-id", type=str, default=None), _f("--use-tensorboard", action=_T),
    _f("--tb-project-name", type=str, default=None), _f("--tb-experiment-name", type=str, default=None),
    _f("--log-interval", type=int, default=1),
]
_DEBUG = [
    _f("--save-debug-rollout-data", type=str, default=None), _f("--load-debug-rollout-data", type=str, default=None),
    _f("--load-forge-rollout-data", type=str, default=None),
    _f("--load-debug-rollout-data-subsample", type=float, default=None),
    _f("--save-debug-train-data", type=str, default=None), _f("--dump-details", type=str, default=None),
    _f("--memory-snapshot-dir", type=str, default="."), _f("--memory-snapshot-num-steps", type=int, default=None),
    _f("--memory-snapshot-path", type=str, default="snapshot.pickle"), _f("--record-memory-history", action=_T),
    _f("--profile-target", type=str, nargs="+", default=["train_overall"],
       choices=["train_overall", "train_actor", "train_log_probs"]),
    _f("--use-pytorch-profiler", action=_T), _f("--profile-step-start", type=int, default=10),
    _f("--profile-step-end", type=int, default=12), _f("--tensorboard-dir", type=str, default=None),
    _f("--memory-recorder", type=str, choices=["torch", "memray"], default="torch"),
    _f("--check-weight-update-equal", action=_T), _f("--debug-rollout-only", action=_T),
    _f("--debug-train-only", action=_T), _f("--http-proxy", type=str, default=None),
    _f("--use-distributed-post", action=_T),
]
_RM = [
    _f("--rm-type", type=str, default=None), _f("--reward-key", type=str, default=None),
    _f("--eval-reward-key", type=str, default=None), _f("--group-rm", action=_T), _f("--rm-url", type=str, default=None),
    _f("--custom-rm-path", type=str, default=None), _f("--custom-reward-post-process-path", type=str, default=None),
    _f("--custom-convert-samples-to-train-data-path", type=str, default=None),
]
_BUFFER = [
    _f("--rollout-buffer-url", type=str, default=None), _f("--fetch-trajectory-retry-times", type=int, default=-1),
    _f("--min-batch-collection-ratio", type=float, default=1), _f("--rollout-task-type", type=str, default="math"),
    _f("--loss-mask-type", type=str, default="qwen", choices=["qwen", "qwen3", "qwen3_5", "distill_qwen"]),
    _f("--data-pad-size-multiplier", type=int, default=128), _f("--rollout-sample-filter-path", type=str, default=None),
    _f("--rollout-all-samples-process-path", type=str, default=None),
]
_PLUGIN = [
    _f("--custom-megatron-init-path", type=str, default=None),
    _f("--custom-megatron-before-log-prob-hook-path", type=str, default=None),
    _f("--custom-megatron-before-train-step-hook-path", type=str, default=None),
    _f("--megatron-deepgemm-forward-layers", nargs="+", type=int, default=None),
    _f("--megatron-deepgemm-forward-modules", nargs="+", default=None),
    _f("--megatron-deepgemm-moe-forward-layers", nargs="+", type=int, default=None),
    _f("--megatron-deepgemm-moe-forward-modules", nargs="+", default=None),
    _f("--enable-mtp-training", action=_T), _f("--mtp-num-layers", type=int, default=None),
    _f("--mtp-loss-scaling-factor", type=float, default=0.2), _f("--custom-config-path", type=str, default=None),
    _f("--padded-vocab-size", type=int, default=None), _f("--runtime-env-json", type=str, default=None),
]
_CI = [
    _f("--ci-test", action=_T), _f("--ci-disable-kl-checker", action=_T), _f("--ci-check-mtp-only-grad", action=_T), _f("--numa-affinity", action=_T),
    _f("--ci-train-rollout-logprob-abs-diff-threshold", type=float, default=0.1),
    _f("--ci-save-grad-norm", type=str, default=None), _f("--ci-load-grad-norm", type=str, default=None),
]
# Training-backend flags (Megatron names).
_MODEL = [
    _f("--num-layers", type=int, default=None), _f("--hidden-size", type=int, default=None),
    _f("--ffn-hidden-size", type=int, default=None), _f("--num-attention-heads", type=int, default=None),
    _f("--group-query-attention", action=_T), _f("--num-query-groups", type=int, default=None),
    _f("--kv-channels", type=int, default=None), _f("--vocab-size", type=int, default=None),
    _f("--make-vocab-size-divisible-by", type=int, default=128),
    _f("--max-position-embeddings", type=int, default=None), _f("--seq-length", type=int, default=4096),
    _f("--swiglu", action=_T), _f("--normalization", type=str, default="RMSNorm", choices=["RMSNorm", "LayerNorm"]),
    _f("--norm-epsilon", type=float, default=1e-5), _f("--apply-layernorm-1p", action=_T),
    _f("--disable-bias-linear", action=_F, dest="add_bias_linear"), _f("--add-qkv-bias", action=_T),
    _f("--qk-layernorm", action=_T), _f("--use-rotary-position-embeddings", action=_T),
    _f("--position-embedding-type", type=str, default="rope"), _f("--no-position-embedding", action=_T),
    _f("--rotary-base", type=float, default=10000), _f("--rotary-percent", type=float, default=1.0),
    _f("--rotary-interleaved", action=_T), _f("--rotary-scaling-factor", type=float, default=1.0),
    _f("--use-rope-scaling", action=_T), _f("--no-rope-fusion", action=_T),
    _f("--untie-embeddings-and-output-weights", action=_T), _f("--attention-softmax-in-fp32", action=_T),
    _f("--attention-dropout", type=float, default=0.0), _f("--hidden-dropout", type=float, default=0.0),
    _f("--attention-backend", type=str, default="flash"), _f("--post-self-attn-layernorm", action=_T),
    _f("--post-mlp-layernorm", action=_T), _f("--use-gated-attention", action=_T), _f("--attention-output-gate", action=_T),
    _f("--multi-latent-attention", action=_T), _f("--q-lora-rank", type=int, default=None),
    _f("--kv-lora-rank", type=int, default=None), _f("--qk-head-dim", type=int, default=None),
    _f("--qk-pos-emb-head-dim", type=int, default=None), _f("--v-head-dim", type=int, default=None),
    _f("--mscale", type=float, default=1.0), _f("--mscale-all-dim", type=float, default=0.0),
    _f("--qk-layernorm-full", action=_T), _f("--softmax-sinks", action=_T),
    _f("--rotary-scaling-type", type=str, default="linear", choices=["linear", "llama3", "yarn"]),
    _f("--rope-low-freq-factor", type=float, default=1.0), _f("--rope-high-freq-factor", type=float, default=4.0),
    _f("--rotary-original-max-position", type=int, default=4096), _f("--yarn-beta-fast", type=float, default=32.0),
    _f("--yarn-beta-slow", type=float, default=1.0),
    _f("--full-attention-interval", type=int, default=None), _f("--linear-num-key-heads", type=int, default=None),
    _f("--linear-num-value-heads", type=int, default=None), _f("--linear-key-head-dim", type=int, default=None),
    _f("--linear-value-head-dim", type=int, default=None), _f("--linear-conv-kernel-dim", type=int, default=4),
    _f("--index-topk", type=int, default=None), _f("--index-n-heads", type=int, default=None),
    _f("--index-head-dim", type=int, default=None), _f("--index-topk-freq", type=int, default=1),
    _f("--index-rotary-interleaved", type=lambda v: str(v).lower() in ("1", "true", "yes"), default=None),
    _f("--index-skip-topk-offset", type=int, default=0),
    _f("--spec", type=str, nargs="*", default=None), _f("--enable-experimental", action=_T),
    _f("--no-masked-softmax-fusion", action=_T), _f("--no-gradient-accumulation-fusion", action=_T),
    _f("--init-method-std", type=float, default=0.02),
]
_MOE = [
    _f("--num-experts", type=int, default=None), _f("--moe-ffn-hidden-size", type=int, default=None),
    _f("--moe-router-topk", type=int, default=2), _f("--moe-router-score-function", type=str, default="softmax"),
    _f("--moe-router-dtype", type=str, default=None), _f("--moe-router-pre-softmax", action=_T),
    _f("--moe-router-load-balancing-type", type=str, default="aux_loss"),
    _f("--moe-router-enable-expert-bias", action=_T), _f("--moe-router-bias-update-rate", type=float, default=1e-3),
    _f("--moe-router-topk-scaling-factor", type=float, default=None),
    _f("--moe-router-num-groups", type=int, default=None), _f("--moe-router-group-topk", type=int, default=None),
    _f("--moe-aux-loss-coeff", type=float, default=0.0), _f("--moe-layer-freq", type=str, default=None),
    _f("--moe-shared-expert-intermediate-size", type=int, default=None), _f("--moe-shared-expert-gate", action=_T),
    _f("--moe-grouped-gemm", action=_T), _f("--moe-permute-fusion", action=_T),
    _f("--moe-token-dispatcher-type", type=str, default="alltoall"), _f("--moe-token-drop-policy", type=str, default="probs"),
    _f("--moe-enable-deepep", action=_T),
]
_PARALLEL = [
    _f("--tensor-model-parallel-size", type=int, default=1), _f("--pipeline-model-parallel-size", type=int, default=1),
    _f("--virtual-pipeline-model-parallel-size", type=int, default=None),
    _f("--num-layers-per-virtual-pipeline-stage", type=int, default=None),
    _f("--microbatch-group-size-per-vp-stage", type=int, default=None),
    _f("--decoder-first-pipeline-num-layers", type=int, default=None),
    _f("--decoder-last-pipeline-num-layers", type=int, default=None),
    _f("--context-parallel-size", type=int, default=1), _f("--expert-model-parallel-size", type=int, default=1),
    _f("--expert-tensor-parallel-size", type=int, default=None), _f("--sequence-parallel", action=_T),
    _f("--use-distributed-optimizer", action=_T), _f("--overlap-grad-reduce", action=_T),
    _f("--overlap-param-gather", action=_T), _f("--tp-comm-overlap", action=_T),
    _f("--distributed-backend", type=str, default="nccl"), _f("--distributed-timeout-minutes", type=int, default=10),
    _f("--ddp-bucket-size", type=int, default=None), _f("--fused-collectives", action=B, default=True),
]
_OPTIM = [
    _f("--optimizer", type=str, default="adam", choices=["adam", "sgd"]), _f("--adam-beta1", type=float, default=0.9),
    _f("--adam-beta2", type=float, default=0.999), _f("--adam-eps", type=float, default=1e-8),
    _f("--weight-decay", type=float, default=0.01), _f("--lr-decay-style", type=str, default="constant"),
    _f("--min-lr", type=float, default=0.0), _f("--lr-warmup-fraction", type=float, default=None),
    _f("--lr-warmup-iters", type=int, default=0), _f("--lr-decay-iters", type=int, default=None),
    _f("--lr-warmup-init", type=float, default=0.0), _f("--accumulate-allreduce-grads-in-fp32", action=_T),
    _f("--optimizer-cpu-offload", action=_T), _f("--overlap-cpu-optimizer-d2h-h2d", action=_T),
    _f("--use-precision-aware-optimizer", action=_T), _f("--bf16", action=B, default=True), _f("--fp16", action=_T),
    _f("--fp8-format", type=str, default=None), _f("--fp8-recipe", type=str, default=None),
    _f("--fp8-param-gather", action=_T), _f("--recompute-granularity", type=str, default=None, choices=["full", "selective"]),
    _f("--recompute-method", type=str, default=None, choices=["uniform", "block"]),
    _f("--recompute-num-layers", type=int, default=None), _f("--deterministic-mode", action=_T),
    _f("--no-check-for-nan-in-loss-and-grad", action=_F, dest="check_for_nan_in_loss_and_grad"),
    _f("--variable-seq-lengths", action=B, default=True),
]
# fmt: on

_ALL_GROUPS = [
    ("cluster", _CLUSTER), ("train", _TRAIN), ("rollout", _ROLLOUT), ("fault tolerance", _FAULT), ("data", _DATA),
    ("eval", _EVAL), ("algorithm", _ALGO), ("logging", _LOG), ("debug", _DEBUG), ("reward model", _RM),
    ("buffer", _BUFFER), ("plugins", _PLUGIN), ("ci", _CI), ("model", _MODEL), ("moe", _MOE),
    ("parallel", _PARALLEL), ("optimizer", _OPTIM),
]  # fmt: skip


def _add_table(parser: argparse.ArgumentParser, title: str, table) -> None:
    group = parser.add_argument_group(title)
    for flag, kw in table:
        kw = dict(kw)
        if isinstance(kw.get("default"), (dict, list)):
            kw["default"] = type(kw["default"])(kw["default"])  # fresh mutable per parser
        try:
            group.add_argument(flag, **kw)
        except argparse.ArgumentError:
            pass  # already registered by another family: first definition wins


def add_slime_arguments(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    for title, table in _ALL_GROUPS:
        _add_table(parser, title, table)
    return parser


def add_engine_arguments(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    """Register ``--sglang-<field>`` for every rollout-engine server argument."""
    from slime_b200.engine.server_args import ROUTER_FLAGS, ServerArgs, SKIPPED_FIELDS

    group = parser.add_argument_group("rollout engine")
    for f in dataclasses.fields(ServerArgs):
        if f.name in SKIPPED_FIELDS:
            continue
        flag = "--sglang-" + f.name.replace("_", "-")
        default = None  # None = "not given": the engine's own default applies
        if f.type in ("bool", bool):
            group.add_argument(flag, action=B, default=default)
        elif f.type in ("int", "int | None"):
            group.add_argument(flag, type=int, default=default)
        elif f.type in ("float", "float | None"):
            group.add_argument(flag, type=float, default=default)
        elif f.type.startswith("list"):
            group.add_argument(flag, nargs="+", type=(int if "int" in f.type else str), default=default)
        else:
            group.add_argument(flag, type=str, default=default)
    for flag, kw in ROUTER_FLAGS:
        group.add_argument(flag, **kw)
    return parser


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(
        "slime_b200", allow_abbrev=False, formatter_class=argparse.ArgumentDefaultsHelpFormatter
    )
    add_slime_arguments(parser)
    add_engine_arguments(parser)
    return parser


# --------------------------------------------------------------- YAML layers
def _apply_role_config(args) -> None:
    """``--megatron-config-path``: per-role overrides ``megatron: [{name, role, overrides}]``.

    CLI values are the shared baseline; the actor's overrides are applied to
    ``args``; the critic's are kept in ``args.critic_overrides`` (kl_coef forced
    to 0 and an untied output head). Resource fields are ignored.
    """
    args.critic_overrides = {"kl_coef": 0.0, "untie_embeddings_and_output_weights": True}
    path = getattr(args, "megatron_config_path", None)
    if not path:
        return
    with open(path) as f:
        doc = yaml.safe_load(f) or {}
    ignored = {"num_nodes", "num_gpus_per_node"}
    for entry in doc.get("megatron", []):
        role = entry.get("role", "actor")
        ov = {k: v for k, v in (entry.get("overrides") or entry.get("args") or {}).items() if k not in ignored}
        if role == "actor":
            for k, v in ov.items():
                setattr(args, k, v)
        elif role == "critic":
            args.critic_overrides.update(ov)
            args.critic_overrides["kl_coef"] = 0.0
        else:
            raise ValueError(f"unknown role {role!r} in {path}")


def get_role_args(args, role: str):
    """A copy of ``args`` specialised for ``role`` ('actor' or 'critic')."""
    ns = argparse.Namespace(**vars(args))
    if role == "critic":
        for k, v in getattr(args, "critic_overrides", {}).items():
            setattr(ns, k, v)
    ns.role = role
    return ns


# ---------------------------------------------------------------- validation
def _model_defaults_from_hf(args) -> None:
    """Fill unset model-shape flags from ``--hf-checkpoint``'s config.json, and
    check the ones that were given against it (parity: megatron_utils/arguments.py:97-148)."""
    path = getattr(args, "hf_checkpoint", None)
    cfg_file = os.path.join(path, "config.json") if path else None
    if path and path.startswith("preset:"):  # a named architecture with random weights, no directory on disk
        from slime_b200.models.config import get_preset

        cfg, cfg_file = get_preset(path[len("preset:") :]).to_hf_dict(), path
    elif not cfg_file or not os.path.exists(cfg_file):
        return
    else:
        with open(cfg_file) as f:
            cfg = json.load(f)
    cfg = cfg.get("text_config", cfg)
    mapping = {
        "num_layers": "num_hidden_layers", "hidden_size": "hidden_size", "ffn_hidden_size": "intermediate_size",
        "num_attention_heads": "num_attention_heads", "num_query_groups": "num_key_value_heads",
        "vocab_size": "vocab_size", "norm_epsilon": "rms_norm_eps", "rotary_base": "rope_theta",
        "kv_channels": "head_dim", "num_experts": "num_experts", "moe_ffn_hidden_size": "moe_intermediate_size",
        "moe_router_topk": "num_experts_per_tok",
    }  # fmt: skip
    explicit = getattr(args, "_explicit", set())
    for ours, theirs in mapping.items():
        if theirs not in cfg or cfg[theirs] is None:
            continue
        if ours in explicit and getattr(args, ours) is not None:
            a, b = getattr(args, ours), cfg[theirs]
            if isinstance(a, float) or isinstance(b, float):
                ok = abs(float(a) - float(b)) <= 1e-6 * max(1.0, abs(float(b)))
            else:
                ok = a == b
            if not ok:
                raise ValueError(f"--{ours.replace('_', '-')}={a} disagrees with {cfg_file} ({theirs}={b})")
        else:
            setattr(args, ours, cfg[theirs])
    if "tie_word_embeddings" in cfg and "untie_embeddings_and_output_weights" not in explicit:
        args.untie_embeddings_and_output_weights = not cfg["tie_word_embeddings"]
    arch = (cfg.get("architectures") or [""])[0]
    if "model_arch" not in explicit:
        args.model_arch = arch
    if arch.startswith("Qwen2") and "add_qkv_bias" not in explicit:
        args.add_qkv_bias = True
    if arch.startswith("Qwen3") and "qk_layernorm" not in explicit:
        args.qk_layernorm = True
    args.swiglu = True


def backend_validate_args(args) -> None:
    """Training-backend defaults (parity: megatron_utils/arguments.py:76-94,151-186)."""
    args.use_distributed_optimizer = True
    args.bf16 = not args.fp16
    args.variable_seq_lengths = True
    if args.num_experts is not None and args.moe_token_dispatcher_type == "allgather":
        args.moe_token_dispatcher_type = "alltoall"
    if args.num_query_groups is None and args.num_attention_heads is not None:
        args.num_query_groups = args.num_attention_heads
    if args.kv_channels is None and args.hidden_size and args.num_attention_heads:
        args.kv_channels = args.hidden_size // args.num_attention_heads
    if args.ffn_hidden_size is None and args.hidden_size:
        args.ffn_hidden_size = 4 * args.hidden_size
    if args.tensor_model_parallel_size == 1:
        args.sequence_parallel = False
    if isinstance(args.moe_layer_freq, str):
        try:
            args.moe_layer_freq = int(args.moe_layer_freq)
        except ValueError:
            args.moe_layer_freq = eval(args.moe_layer_freq, {"__builtins__": {}})  # "[0]*3+[1]*45" style
    if args.moe_layer_freq is None and hasattr(args, "moe_layer_freq"):
        delattr(args, "moe_layer_freq")
    if getattr(args, "use_rope_scaling", False) and args.rotary_scaling_type == "linear" and not getattr(args, "multi_latent_attention", False):
        # the Llama-3.1 frequency scaling (as in the reference's trainer), trained at 8192 positions unless said otherwise
        args.rotary_scaling_type = "llama3"
        if getattr(args, "rotary_original_max_position", None) in (None, 4096):
            args.rotary_original_max_position = 8192
    if args.vocab_size is not None and args.padded_vocab_size is None:
        mult = args.make_vocab_size_divisible_by * args.tensor_model_parallel_size
        args.padded_vocab_size = -(-args.vocab_size // mult) * mult
    if args.allgather_cp and getattr(args, "context_parallel_size", 1) > 1 and not (getattr(args, "index_topk", None)
                                  or str(getattr(args, "model_arch", "")).lower().startswith(("deepseekv32", "glmmoedsa"))):
        raise ValueError("--allgather-cp is only supported for DSA attention models (DeepSeek-V3.2 / GLM-5)")
    if args.allgather_cp and getattr(args, "context_parallel_size", 1) > 1 and (
            getattr(args, "use_rollout_routing_replay", False) or getattr(args, "enable_mtp_training", False)):
        raise ValueError("--allgather-cp: rollout routing replay and draft-head training still assume the zig-zag token layout")
    if args.virtual_pipeline_model_parallel_size is None and args.num_layers_per_virtual_pipeline_stage:
        per_stage = args.num_layers // args.pipeline_model_parallel_size
        args.virtual_pipeline_model_parallel_size = per_stage // args.num_layers_per_virtual_pipeline_stage
    if args.microbatch_group_size_per_vp_stage is None:
        args.microbatch_group_size_per_vp_stage = args.pipeline_model_parallel_size
    world = args.actor_num_nodes * args.actor_num_gpus_per_node
    mp = args.tensor_model_parallel_size * args.pipeline_model_parallel_size * args.context_parallel_size
    if world and world % mp != 0:
        raise ValueError(f"actor GPUs ({world}) not divisible by tp*pp*cp ({mp})")


def engine_validate_args(args) -> None:
    if args.rollout_num_gpus is not None and args.rollout_num_gpus > 0:
        per = args.rollout_num_gpus_per_engine
        if args.rollout_num_gpus % per != 0:
            raise ValueError(f"--rollout-num-gpus {args.rollout_num_gpus} not divisible by --rollout-num-gpus-per-engine {per}")
    if getattr(args, "sglang_config", None) and args.rollout_external_engine_addrs:
        raise ValueError("--sglang-config and --rollout-external-engine-addrs are mutually exclusive")
    if getattr(args, "sglang_server_concurrency", None) is None:
        args.sglang_server_concurrency = 512


def _resolve_eval_datasets(args):
    from slime_b200.utils.eval_config import build_eval_dataset_configs, ensure_dataset_list

    datasets_config, defaults = [], {}
    if args.eval_config:
        with open(args.eval_config) as f:
            cfg = yaml.safe_load(f) or {}
        eval_cfg = cfg.get("eval", cfg)
        defaults = dict(eval_cfg.get("defaults") or {})
        datasets_config = ensure_dataset_list(eval_cfg.get("datasets"))
        if not datasets_config:
            raise ValueError("--eval-config must define at least one dataset under `eval.datasets`.")
    elif args.eval_prompt_data:
        values = list(args.eval_prompt_data)
        if len(values) == 1:
            logger.info("[legacy] only one eval_prompt_data given; assuming it is aime")
            values = ["aime", values[0]]
        if len(values) % 2 != 0:
            raise ValueError("eval prompt data must be pairs of (name, path).")
        datasets_config = [{"name": values[i], "path": values[i + 1]} for i in range(0, len(values), 2)]
    datasets = build_eval_dataset_configs(args, datasets_config, defaults)
    args.eval_prompt_data = [x for d in datasets for x in (d.name, d.path)] if datasets else None
    return datasets


def slime_validate_args(args) -> None:
    """Cross-flag checks and derived settings (parity: slime/utils/arguments.py:1767-2075)."""
    args.eval_datasets = _resolve_eval_datasets(args)
    if args.rollout_temperature <= 0:
        raise ValueError("--rollout-temperature must be > 0; temperature 0 is greedy decoding, not a valid RL policy.")
    if (args.kl_coef != 0 or args.use_kl_loss) and not (args.ref_load and os.path.exists(args.ref_load)):
        raise FileNotFoundError(f"ref_load {args.ref_load} does not exist, please check the path.")

    if args.use_opd:
        if args.opd_type is None:
            raise ValueError("--opd-type must be specified when --use-opd is enabled. Choose 'sglang' or 'megatron'.")
        if args.opd_type == "megatron":
            if args.opd_teacher_load is None:
                raise ValueError("--opd-teacher-load is required when --opd-type=megatron.")
            if not os.path.exists(args.opd_teacher_load):
                raise FileNotFoundError(f"opd_teacher_load {args.opd_teacher_load} does not exist.")
        elif args.opd_teacher_load is not None:
            raise ValueError("--opd-teacher-load should not be set when --opd-type=sglang.")
    elif args.opd_teacher_load is not None:
        raise ValueError("--opd-teacher-load is set but --use-opd is not enabled. Please add --use-opd flag.")

    def _is_native_ckpt(p):
        return p is not None and os.path.exists(os.path.join(p, "latest_checkpointed_iteration.txt"))

    def _is_hf_dir(p):
        return p is not None and os.path.isdir(p) and os.path.exists(os.path.join(p, "config.json"))

    if not _is_native_ckpt(args.load):
        args.no_load_optim = args.no_load_rng = args.finetune = True
        if not _is_hf_dir(args.load):
            args.load = args.ref_load
        if args.ref_ckpt_step is not None:
            args.ckpt_step = args.ref_ckpt_step
        if args.start_rollout_id is None:
            args.start_rollout_id = 0

    if args.eval_interval is not None:
        assert args.eval_datasets, "Evaluation datasets must be configured when eval_interval is set."
    if args.save_interval is not None:
        assert args.save is not None, "'--save' is required when save_interval is set."
    assert not (args.kl_coef != 0 and args.kl_loss_coef != 0), "Only one of kl_coef and kl_loss_coef can be set"
    if args.advantage_estimator in ("reinforce_plus_plus", "reinforce_plus_plus_baseline"):
        assert args.normalize_advantages, f"{args.advantage_estimator} requires --normalize-advantages"
    if args.use_rollout_logprobs:
        assert not args.use_tis, "use_rollout_logprobs and use_tis cannot be set at the same time."
    if args.get_mismatch_metrics:
        assert args.custom_tis_function_path is not None, "custom_tis_function_path must be set with get_mismatch_metrics"
    if args.use_dynamic_batch_size:
        assert args.max_tokens_per_gpu is not None, "max_tokens_per_gpu must be set when use_dynamic_batch_size is set"
        if args.log_probs_max_tokens_per_gpu is None:
            args.log_probs_max_tokens_per_gpu = args.max_tokens_per_gpu
    if args.balance_by_flops:
        assert args.use_dynamic_batch_size, "--balance-by-flops requires --use-dynamic-batch-size"
        args.balance_data = True
    if args.eps_clip_high is None:
        args.eps_clip_high = args.eps_clip
    if args.advantage_estimator == "cispo" and args.eps_clip < 1.0:
        logger.warning("CISPO is canonically single-sided; --eps-clip=%s keeps a lower clip bound.", args.eps_clip)
    if args.eval_reward_key is None:
        args.eval_reward_key = args.reward_key
    if args.dump_details is not None:
        args.save_debug_rollout_data = f"{args.dump_details}/rollout_data/{{rollout_id}}.pt"
        args.save_debug_train_data = f"{args.dump_details}/train_data/{{rollout_id}}.pt"
    if args.save_debug_train_data is not None and args.save_debug_train_data == args.save_debug_rollout_data:
        raise ValueError("--save-debug-train-data must not be equal to --save-debug-rollout-data.")
    if args.load_debug_rollout_data is not None:
        args.debug_train_only = True

    args.rollout_external = args.rollout_external_engine_addrs is not None
    if args.rollout_external and not args.debug_train_only:
        from slime_b200.engine.external import apply_external_engine_info_to_args

        apply_external_engine_info_to_args(args, logger=logger)

    args.use_critic = args.advantage_estimator == "ppo"
    args.critic_num_gpus_per_node = args.actor_num_gpus_per_node
    args.critic_num_nodes = args.actor_num_nodes

    if args.offload:
        args.offload_train = args.offload_rollout = True
    del args.offload

    if args.debug_rollout_only:
        if args.rollout_external:
            pass
        elif args.colocate and args.rollout_num_gpus is None:
            args.rollout_num_gpus = args.actor_num_gpus_per_node * args.actor_num_nodes
        elif args.rollout_num_gpus == 0:
            args.actor_num_gpus_per_node = args.actor_num_nodes = 0
        else:
            args.actor_num_gpus_per_node = min(8, args.rollout_num_gpus)
            args.actor_num_nodes = args.rollout_num_gpus // args.actor_num_gpus_per_node
        args.colocate = False
        args.offload_train = args.offload_rollout = False
    assert not (args.debug_rollout_only and args.debug_train_only), "set only one of debug_rollout_only / debug_train_only"

    if args.colocate:
        if args.release_train:
            args.offload_train = False
            args.offload_rollout = True
        elif args.offload_train is None:
            args.offload_train = True
        if args.offload_rollout is None:
            args.offload_rollout = True
        if args.rollout_num_gpus is None:
            args.rollout_num_gpus = args.actor_num_gpus_per_node * args.actor_num_nodes
    args.offload_train = bool(args.offload_train)
    args.offload_rollout = bool(args.offload_rollout)
    if args.use_critic:
        args.offload_train = True
    if args.offload_train:
        args.disable_grad_buffers_cpu_backup = args.disable_param_buffers_cpu_backup = True
    if args.rollout_num_gpus is None and not args.debug_train_only:
        raise ValueError("--rollout-num-gpus is required unless --colocate or --debug-train-only is set")

    if args.eval_function_path is None:
        args.eval_function_path = args.rollout_function_path

    if args.num_steps_per_rollout is not None:
        gbs = args.rollout_batch_size * args.n_samples_per_prompt // args.num_steps_per_rollout
        if args.global_batch_size is not None:
            assert args.global_batch_size == gbs, (
                f"global_batch_size {args.global_batch_size} != rollout_batch_size {args.rollout_batch_size} * "
                f"n_samples_per_prompt {args.n_samples_per_prompt} // num_steps_per_rollout {args.num_steps_per_rollout}"
            )
        args.global_batch_size = gbs
    elif args.global_batch_size is None:
        args.global_batch_size = args.rollout_batch_size * args.n_samples_per_prompt
        args.num_steps_per_rollout = 1

    if args.n_samples_per_prompt == 1:
        args.grpo_std_normalization = False
    if args.over_sampling_batch_size is None:
        args.over_sampling_batch_size = args.rollout_batch_size
    assert args.over_sampling_batch_size >= args.rollout_batch_size, "over_sampling_batch_size must be >= rollout_batch_size"

    if args.num_epoch is not None:
        if args.num_rollout is None:
            assert args.rollout_global_dataset, "--num-epoch needs the global dataset (remove --disable-rollout-global-dataset)"
    else:
        assert args.num_rollout is not None, "please set --num-rollout or --num-epoch"
    if args.enable_mtp_training:
        assert args.mtp_num_layers, "mtp_num_layers must be set when enable_mtp_training is set"
    if args.use_rollout_routing_replay:
        args.use_routing_replay = True

    if args.custom_config_path:
        with open(args.custom_config_path) as f:
            for k, v in (yaml.safe_load(f) or {}).items():
                setattr(args, k, v)

    if args.eval_max_context_len is None:
        args.eval_max_context_len = args.rollout_max_context_len
    if args.rollout_max_context_len is not None:
        if args.rollout_max_prompt_len is None:
            args.rollout_max_prompt_len = args.rollout_max_context_len - 1
        assert args.rollout_max_prompt_len <= args.rollout_max_context_len - 1, (
            "rollout_max_prompt_len must leave room for at least one generated token"
        )
    if args.only_train_params_name_list and args.freeze_params_name_list:
        raise ValueError("You can only specify ONE of: --only-train-params-name-list, or --freeze-params-name-list.")
    if args.update_weight_transport == "disk" and not args.update_weight_disk_dir:
        raise ValueError("--update-weight-transport=disk requires --update-weight-disk-dir (shared filesystem).")
    if args.release_train:
        if args.use_critic:
            raise ValueError("--release-train does not support critic training yet.")
        if args.keep_old_actor:
            raise ValueError("--release-train does not support --keep-old-actor.")
        if args.save is None:
            raise ValueError("--release-train requires --save so the next trainer can reload.")
        if args.save_interval is None:
            args.save_interval = 1
        if args.update_weight_mode != "full" or args.update_weight_transport != "disk":
            raise ValueError("--release-train requires --update-weight-mode=full and --update-weight-transport=disk.")
    if args.update_weight_mode == "delta":
        if args.update_weight_transport != "disk":
            raise ValueError("--update-weight-mode=delta requires --update-weight-transport=disk.")
        if args.colocate:
            raise ValueError("--update-weight-mode=delta is not supported with --colocate.")
        if not args.update_weight_local_checkpoint_dir:
            raise ValueError("--update-weight-mode=delta requires --update-weight-local-checkpoint-dir.")

    # GPU budget (operational FAQ): colocated needs actor GPUs, disaggregated actor + rollout
    if not args.debug_train_only and not args.debug_rollout_only and not args.rollout_external:
        train_gpus = args.actor_num_nodes * args.actor_num_gpus_per_node
        args.total_gpus_needed = max(train_gpus, args.rollout_num_gpus) if args.colocate else train_gpus + args.rollout_num_gpus


def parse_args(argv: list[str] | None = None, add_custom_arguments=None) -> argparse.Namespace:
    parser = build_parser()
    if add_custom_arguments is not None:
        add_custom_arguments(parser)
    args = parser.parse_args(argv)
    # remember which flags were given explicitly (used for HF-config validation)
    defaults = parser.parse_args(["--rollout-batch-size", "1"])
    args._explicit = {k for k, v in vars(args).items() if k in vars(defaults) and getattr(defaults, k) != v}
    _apply_role_config(args)
    _model_defaults_from_hf(args)
    backend_validate_args(args)
    slime_validate_args(args)
    engine_validate_args(args)
    args.rank = 0
    args.world_size = args.actor_num_nodes * args.actor_num_gpus_per_node
    return args


def namespace_from_dict(d: dict[str, Any]) -> argparse.Namespace:
    """Build a fully-defaulted Namespace from a partial dict (tests, bench, tools)."""
    parser = build_parser()
    ns = parser.parse_args(["--rollout-batch-size", str(d.get("rollout_batch_size", 1))])
    for k, v in d.items():
        setattr(ns, k, v)
    return finalize_namespace(ns)


def finalize_namespace(ns: argparse.Namespace) -> argparse.Namespace:
    """Derived attributes that ``slime_validate_args`` would set, for programmatically built namespaces."""
    ns.use_critic = ns.advantage_estimator == "ppo"
    if getattr(ns, "hf_checkpoint", None):
        _model_defaults_from_hf(ns)  # model shape from config.json / a preset, as the CLI path does
    if ns.eps_clip_high is None:
        ns.eps_clip_high = ns.eps_clip
    ns.offload_train = bool(ns.offload_train)
    ns.offload_rollout = bool(ns.offload_rollout)
    ns.rollout_external = ns.rollout_external_engine_addrs is not None
    if ns.global_batch_size is None:
        ns.global_batch_size = ns.rollout_batch_size * ns.n_samples_per_prompt // (ns.num_steps_per_rollout or 1)
    if ns.over_sampling_batch_size is None:
        ns.over_sampling_batch_size = ns.rollout_batch_size
    if ns.use_rollout_routing_replay:
        ns.use_routing_replay = True
    if ns.eval_function_path is None:
        ns.eval_function_path = ns.rollout_function_path
    if ns.start_rollout_id is None and not ns.load:
        ns.start_rollout_id = 0
    if getattr(ns, "offload", None) is not None:
        del ns.offload
    if not hasattr(ns, "critic_overrides"):
        ns.critic_overrides = {"kl_coef": 0.0, "untie_embeddings_and_output_weights": True}
    if ns.microbatch_group_size_per_vp_stage is None:
        ns.microbatch_group_size_per_vp_stage = ns.pipeline_model_parallel_size
    if isinstance(getattr(ns, "moe_layer_freq", None), str):
        ns.moe_layer_freq = int(ns.moe_layer_freq)
    ns.eval_datasets = getattr(ns, "eval_datasets", [])
    return ns
