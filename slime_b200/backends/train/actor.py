"""Per-rank training actor: owns the model/optimizer, runs log-prob passes, advantage
computation, optimizer steps, checkpoints and the trainer side of weight sync.

Replaces ``MegatronTrainRayActor`` (slime/backends/megatron_utils/actor.py:58-693) and its
base ``TrainRayActor`` (slime/ray/train_actor.py:25-94). It is a plain object: the actor
runtime hosts it in a child process per GPU, and the colocated fast path
(``slime_b200.api``) instantiates it in the same process as the rollout engine so weight
sync is a device-side copy instead of an IPC + HTTP exchange.
"""

from __future__ import annotations

import logging
import os
import time
from argparse import Namespace
from datetime import timedelta

import torch
import torch.distributed as dist

from slime_b200.backends.train import checkpoint as ckpt
from slime_b200.backends.train.cp_utils import slice_log_prob_with_cp
from slime_b200.backends.train.data import DataIterator
from slime_b200.backends.train.loss import (
    compute_advantages_and_returns,
    drain_captured_log_probs,
    enable_log_prob_capture,
    get_log_probs_and_entropy,
    get_values,
)
from slime_b200.backends.train.model import TrainModel, forward_only, train
from slime_b200.observability import train_metric_utils
from slime_b200.observability.timer import Timer, inverse_timer, timer
from slime_b200.parallel import state as mpu
from slime_b200.utils import routing_replay
from slime_b200.utils.misc import load_function
from slime_b200.utils.tensor_backuper import TensorBackuper

logger = logging.getLogger(__name__)


def init_distributed(args, rank: int, world_size: int, master_addr: str, master_port: int, local_rank: int | None = None):
    """Process-group bootstrap: NCCL world (device collectives) + parallel topology."""
    os.environ.setdefault("MASTER_ADDR", str(master_addr))
    os.environ.setdefault("MASTER_PORT", str(master_port))
    os.environ["WORLD_SIZE"], os.environ["RANK"] = str(world_size), str(rank)
    if torch.cuda.is_available():
        lr = local_rank if local_rank is not None else rank % max(torch.cuda.device_count(), 1)
        os.environ["LOCAL_RANK"] = str(lr)
        torch.cuda.set_device(lr)
    backend = args.distributed_backend if torch.cuda.is_available() else "gloo"
    if not dist.is_initialized():
        dist.init_process_group(backend=backend, rank=rank, world_size=world_size,
                                timeout=timedelta(minutes=args.distributed_timeout_minutes))  # fmt: skip
    mpu.initialize_model_parallel(
        args.tensor_model_parallel_size, args.pipeline_model_parallel_size, args.virtual_pipeline_model_parallel_size,
        args.context_parallel_size, args.expert_model_parallel_size, args.expert_tensor_parallel_size,
    )  # fmt: skip


class TrainActor:
    def __init__(self, args: Namespace, role: str = "actor"):
        self.args, self.role = args, role
        self.model: TrainModel | None = None
        self.weights_backuper: TensorBackuper | None = None
        self._active_model_tag = "actor"
        self.weight_updater = None
        self.rollout_engines = []
        self.rollout_data_postprocess = (
            load_function(args.rollout_data_postprocess_path) if getattr(args, "rollout_data_postprocess_path", None) else None
        )
        self.asleep = False

    # ------------------------------------------------------------------------ init
    def init(self, with_ref: bool = False, with_opd_teacher: bool = False, device=None) -> int:
        args = self.args
        if not mpu.model_parallel_is_initialized():
            mpu.initialize_model_parallel()
        hook = getattr(args, "custom_megatron_init_path", None)
        if hook:
            load_function(hook)(args)
        if getattr(args, "deterministic_mode", False):
            torch.use_deterministic_algorithms(True, warn_only=True)
        if getattr(args, "numa_affinity", False) or os.environ.get("SLIME_B200_NUMA_AFFINITY") == "1":
            from slime_b200.utils.distributed_utils import set_numa_affinity

            cpus = set_numa_affinity(int(os.environ.get("LOCAL_RANK", "0")))
            logger.info("NUMA affinity: %s", f"{len(cpus)} CPUs" if cpus else "unchanged")
        if getattr(args, "use_routing_replay", False):
            os.environ["ENABLE_ROUTING_REPLAY"] = "1"  # read by every router (slime/utils/routing_replay.py:81 in the reference)
        self.model = TrainModel(args, role=self.role, device=device)
        start = 0
        if getattr(args, "load", None):
            loaded = ckpt.load_checkpoint(args, self.model, load_optimizer=not args.no_load_optim)
            if loaded is not None and not args.finetune:
                start = loaded + 1
        args.start_rollout_id = start if args.start_rollout_id is None else args.start_rollout_id
        if args.reset_optimizer_states and self.model.optimizer is not None:
            self.model.optimizer.reset_states()

        small = self.model.cfg.num_params() * 2 < 8e9  # keep extra weight sets on the device when they are small
        self.weights_backuper = TensorBackuper(lambda: self.model.named_parameters(), device_resident=small)
        if self.role == "actor":
            if with_ref:
                self.load_other_checkpoint("ref", args.ref_load)
            if with_opd_teacher:
                self.load_other_checkpoint("teacher", args.opd_teacher_load)
            if args.keep_old_actor:
                self.weights_backuper.backup("actor")
                self.weights_backuper.copy("actor", "old_actor")
                self.weights_backuper.copy("actor", "rollout_actor")
            elif with_ref or with_opd_teacher:
                self.weights_backuper.backup("actor")
        if getattr(args, "offload_train", False) and getattr(args, "sleep_after_init", False):
            self.sleep()
        self.prof = None
        if getattr(args, "use_pytorch_profiler", False) or getattr(args, "record_memory_history", False):
            from slime_b200.observability.profile_utils import TrainProfiler

            self.prof = TrainProfiler(args)
            self.prof.on_init_end()
        return args.start_rollout_id

    def load_other_checkpoint(self, tag: str, path: str):
        """Load another weight set (ref / teacher) through the live model, snapshot it, restore the actor."""
        self.weights_backuper.backup("actor")
        a = Namespace(**{**vars(self.args), "load": path, "no_load_optim": True, "no_load_rng": True, "finetune": True})
        if tag == "ref" and self.args.ref_ckpt_step is not None:
            a.ckpt_step = self.args.ref_ckpt_step
        if tag == "teacher" and getattr(self.args, "opd_teacher_ckpt_step", None) is not None:
            a.ckpt_step = self.args.opd_teacher_ckpt_step
        if path:
            ckpt.load_checkpoint(a, self.model, load_optimizer=False)
        self.weights_backuper.backup(tag)
        self.weights_backuper.restore("actor")

    def _switch_model(self, tag: str):
        if tag == self._active_model_tag or tag not in self.weights_backuper.backup_tags:
            self._active_model_tag = tag if tag in self.weights_backuper.backup_tags else self._active_model_tag
            if tag != self._active_model_tag:
                return
        self.weights_backuper.restore(tag)
        self._active_model_tag = tag

    # ----------------------------------------------------------------- memory choreography
    def sleep(self):
        """Colocated mode: hand the GPU to the rollout engine. Gradient and gathered-parameter
        buffers are recomputable and simply dropped; optimizer shards move to pinned host memory."""
        if self.asleep:
            return
        from slime_b200.runtime import memory

        memory.offload_train_state(self.model)
        if getattr(self.args, "release_communicators_on_sleep", False):
            mpu.release_communicators()  # NCCL buffers go too; rebuilt in wake_up
        self.asleep = True

    def wake_up(self):
        if not self.asleep:
            return
        from slime_b200.runtime import memory

        mpu.reload_communicators()  # no-op unless they were released
        memory.onload_train_state(self.model)
        self.asleep = False

    # ------------------------------------------------------------------------ data
    def _get_rollout_data(self, rollout_data_ref) -> dict:
        from slime_b200.utils.data import process_rollout_data

        if isinstance(rollout_data_ref, dict):
            data = rollout_data_ref  # in-process payload
            part = data["partition"]
            totals = data["total_lengths"]
            Timer().seq_lens = totals
            if not data.get("_localised"):
                data["total_lengths"] = [totals[i] for i in part]  # whole-batch field -> this rank's order
                data["_localised"] = True
            if "raw_reward" in data:
                data["local_raw_reward"] = [data["raw_reward"][i] for i in part]
        else:
            data = process_rollout_data(self.args, rollout_data_ref, mpu.get_data_parallel_rank(False),
                                        mpu.get_data_parallel_world_size(False))  # fmt: skip
        dev = self.model.device
        self.h2d_bytes = getattr(self, "h2d_bytes", 0) + sum(
            t.numel() * t.element_size() for k in ("tokens", "loss_masks", "rollout_log_probs") for t in data.get(k, [])
        )
        self.d2h_bytes = getattr(self, "d2h_bytes", 0) + 4 * 8  # reduced step metrics read back for logging
        data["tokens"] = [t.to(dev, torch.long, non_blocking=True) for t in data["tokens"]]
        data["loss_masks"] = [t.to(dev, torch.int, non_blocking=True) for t in data["loss_masks"]]
        if "rollout_mask_sums" in data:
            sums = torch.as_tensor([float(x) for x in data["rollout_mask_sums"]], dtype=torch.float32).to(dev, non_blocking=True)
            data["rollout_mask_sums"] = list(sums.unbind(0))  # one copy for the batch, per-sample views
        for key in ("rollout_log_probs", "teacher_log_probs"):
            if key in data:
                data[key] = [
                    slice_log_prob_with_cp(lp, tl, rl).to(dev, torch.float32, non_blocking=True)
                    for lp, tl, rl in zip(data[key], data["total_lengths"], data["response_lengths"])
                ]
        return data

    # ----------------------------------------------------------------------- train
    def train(self, rollout_id: int, rollout_data_ref, external_data=None):
        if getattr(self.args, "offload_train", False):
            self.wake_up()
        with timer("data_preprocess"):
            data = self._get_rollout_data(rollout_data_ref)
        out = self.train_critic(rollout_id, data) if self.role == "critic" else self.train_actor(rollout_id, data, external_data)
        if getattr(self, "prof", None) is not None:
            self.prof.step(rollout_id)
        return out

    def fill_routing_replay(self, iterator, data: dict):
        """R3: hand every MoE layer the experts the rollout engine picked, micro-batch by micro-batch in the order the
        passes will walk them. Rows follow the packed token stream of ``get_batch`` (CP slice per sample, padding rows
        at the end, this rank's sequence-parallel slice). Same role as slime/backends/megatron_utils/actor.py:308-355
        in the reference."""
        from slime_b200.backends.train.cp_utils import prepare_routed_experts_for_routing_replay

        a = self.args
        if "rollout_routed_experts" not in data:
            raise ValueError("rollout_routed_experts is required in the rollout data when --use-rollout-routing-replay is set")
        tp_size, tp_rank = mpu.get_tensor_model_parallel_world_size(), mpu.get_tensor_model_parallel_rank()
        layers = [i for i in range(a.num_layers) if self.model.cfg.is_moe_layer(i)]
        routing_replay.RoutingReplay.clear_all()
        iterator.reset()
        for _ in range(len(iterator)):
            batch = iterator.get_next(["rollout_routed_experts", "total_lengths"])
            rows = torch.cat([prepare_routed_experts_for_routing_replay(torch.as_tensor(r), tl)
                              for r, tl in zip(batch["rollout_routed_experts"], batch["total_lengths"])])  # fmt: skip
            pad = (-rows.shape[0]) % (tp_size * a.data_pad_size_multiplier)
            if pad:
                rows = torch.nn.functional.pad(rows, (0, 0, 0, 0, 0, pad))
            if a.sequence_parallel and tp_size > 1:
                n = rows.shape[0] // tp_size
                rows = rows[tp_rank * n : (tp_rank + 1) * n]
            routing_replay.fill_from_rollout([rows], layers)
        iterator.reset()
        del data["rollout_routed_experts"]

    def compute_log_prob(self, data_iterator, num_microbatches, store_prefix=""):
        with timer(f"{store_prefix}log_probs"):
            return forward_only(get_log_probs_and_entropy, self.args, self.model, data_iterator, num_microbatches, store_prefix)

    def can_reuse_log_probs_in_loss(self, num_microbatches) -> bool:
        """One optimizer step per rollout with plain GRPO: the training forward's own (detached)
        log-probs are the old-policy log-probs, so the separate forward pass is skipped."""
        a = self.args
        return (
            len(num_microbatches) == 1 and a.loss_type == "policy_loss" and a.kl_coef == 0 and not a.use_rollout_logprobs
            and not a.get_mismatch_metrics and not a.use_critic and not a.keep_old_actor and not a.use_opd
            and (not a.use_routing_replay or a.use_rollout_routing_replay) and a.advantage_estimator != "gspo"
        )  # fmt: skip

    def train_actor(self, rollout_id: int, data: dict, external_data=None):
        a = self.args
        it = [DataIterator(data, data["micro_batch_indices"]) for _ in self.model.chunks[:1]]
        num_mb, gbs = data["num_microbatches"], data["global_batch_sizes"]
        tags = self.weights_backuper.backup_tags
        with inverse_timer("train_wait"), timer("train"):
            if a.compute_advantages_and_returns:
                if "ref" in tags:
                    routing_replay.set_stage("fallthrough")
                    self._switch_model("ref")
                    data.update(self.compute_log_prob(it, num_mb, "ref_"))
                if "teacher" in tags:
                    routing_replay.set_stage("fallthrough")
                    self._switch_model("teacher")
                    data.update(self.compute_log_prob(it, num_mb, "teacher_"))
                if self._active_model_tag != ("old_actor" if a.keep_old_actor else "actor"):
                    self._switch_model("old_actor" if a.keep_old_actor else "actor")
                if a.use_rollout_routing_replay:
                    self.fill_routing_replay(it[0], data)
                if (not a.use_rollout_logprobs or a.get_mismatch_metrics) and not self.can_reuse_log_probs_in_loss(num_mb):
                    if a.use_routing_replay:
                        routing_replay.set_stage("replay_forward" if a.use_rollout_routing_replay else "record")
                    data.update(self.compute_log_prob(it, num_mb, ""))
                    if a.use_rollout_routing_replay:
                        routing_replay.RoutingReplay.clear_all_forward()
                if a.use_critic and external_data is not None and mpu.is_pipeline_last_stage():
                    vals = external_data.get("values")
                    if vals is not None:
                        data["values"] = [v.to(self.model.device) for v in vals]
                if self._active_model_tag != "actor" and "actor" in tags:
                    self._switch_model("actor")
                compute_advantages_and_returns(a, data)
            if self.rollout_data_postprocess is not None:
                self.rollout_data_postprocess(a, rollout_id, data)
            train_metric_utils.log_rollout_data(rollout_id, a, data)
            if a.use_routing_replay:
                routing_replay.set_stage("replay_forward")  # recomputed layers switch to the backward cursor themselves
            capture = getattr(a, "save_debug_train_data", None) is not None and "log_probs" not in data
            if capture:
                enable_log_prob_capture()
            with timer("actor_train"):
                history = train(rollout_id, self.model, it, num_mb, gbs)
            if capture:
                got = drain_captured_log_probs()
                enable_log_prob_capture(False)
                if got:
                    data["log_probs"] = [got[i] for i in data.get("sample_indices", range(len(got))) if i in got]
        self.last_metrics = train_metric_utils.log_train_steps(rollout_id, a, history, self.model)
        from slime_b200.observability import train_data_utils

        train_data_utils.save_debug_train_data(a, rollout_id=rollout_id, rollout_data=data)
        if a.use_routing_replay:
            routing_replay.RoutingReplay.clear_all()
        if "actor" in tags:
            self.weights_backuper.backup("actor")
        if a.ref_update_interval is not None and (rollout_id + 1) % a.ref_update_interval == 0 and "ref" in tags:
            with timer("ref_model_update"):
                self.weights_backuper.copy("actor", "ref")
        train_metric_utils.log_perf_data(rollout_id, a, extra_metrics=self.weight_updater.pop_metrics() if self.weight_updater else None)
        return self.last_metrics

    def train_critic(self, rollout_id: int, data: dict):
        a = self.args
        it = [DataIterator(data, data["micro_batch_indices"])]
        num_mb, gbs = data["num_microbatches"], data["global_batch_sizes"]
        data.update(forward_only(get_values, a, self.model, it, num_mb))
        if rollout_id >= a.num_critic_only_steps:
            pass  # actor consumes the values through `external_data`
        compute_advantages_and_returns(a, data)
        crit_args = Namespace(**{**vars(a), "loss_type": "value_loss"})
        self.model.args = crit_args
        history = train(rollout_id, self.model, it, num_mb, gbs)
        self.model.args = a
        self.last_metrics = train_metric_utils.log_train_steps(rollout_id, a, history, self.model, prefix="train/critic-")
        values = [v.detach().cpu() for v in data.get("values", [])] if mpu.is_pipeline_last_stage() else None
        return {"values": values}

    # ------------------------------------------------------------------------ save
    def save_model(self, rollout_id: int, force_sync: bool = False):
        a = self.args
        if a.debug_rollout_only:
            return
        ckpt.save_checkpoint(a, rollout_id, self.model, save_optimizer=not a.no_save_optim, async_save=a.async_save and not force_sync)
        if a.save_hf is not None and self.role == "actor":
            from slime_b200.checkpoint.hf_saver import save_hf_model_to_path

            save_hf_model_to_path(a, self.model, a.save_hf.format(rollout_id=rollout_id))

    # ---------------------------------------------------------------- weight sync
    def connect_rollout_engines(self, engines, lock=None):
        from slime_b200.weight_sync.updaters import make_weight_updater

        self.rollout_engines = engines
        if self.weight_updater is None:
            self.weight_updater = make_weight_updater(self.args, self.model, self.weights_backuper)
        self.weight_updater.connect_rollout_engines(engines, lock)

    def update_weights(self):
        a = self.args
        if a.debug_train_only or a.debug_rollout_only:
            return
        if getattr(a, "offload_train", False) and self.asleep:
            self.wake_up()
        with timer("update_weights"):
            self.weight_updater.update_weights()
        if a.keep_old_actor:
            # 1-step-delayed behaviour policy: rollout_actor <- old_actor <- actor
            self.weights_backuper.copy("old_actor", "rollout_actor")
            self.weights_backuper.copy("actor", "old_actor")
        if getattr(a, "offload_train", False) and getattr(a, "sleep_between_phases", False):
            self.sleep()
