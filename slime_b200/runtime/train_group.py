"""Trainer processes as an actor group: one ``TrainWorker`` per GPU, driven together by ``TrainGroup``.

    TrainGroup.create()            spawn workers, rendezvous (NCCL on GPUs, gloo on CPU), build model + optimizer
    TrainGroup.async_train(...)    every worker trains on its DP rank's payload; returns one future per worker
    TrainGroup.update_weights()    trainer -> rollout engines (tensor / distributed / disk transport)
    TrainGroup.release()/create()  ``--release-train``: free the trainer GPUs between steps, reload from the checkpoint

Parity: slime/ray/train_actor.py:25-130 (worker), slime/ray/actor_group.py:17-260 (group),
slime/ray/placement_group.py:140-253 (``create_*`` helpers).
"""

from __future__ import annotations

import copy
import logging
import os
import shutil
import time
from pathlib import Path

from slime_b200.runtime import actors
from slime_b200.utils.misc import get_current_node_ip, get_free_port

logger = logging.getLogger(__name__)

# engine calls whose result the weight updaters wait for later (they overlap with a collective on the trainer side)
_DEFERRED_ENGINE_CALLS = {"init_weights_update_group", "update_weights_from_distributed"}


class EngineProxy:
    """Gives an engine actor handle the plain-method surface the weight updaters expect.

    ``update_weights`` packs a bucket into one flat device buffer; sent through the actor channel it crosses
    the process boundary as a CUDA IPC mapping (the channel pickles with the multiprocessing reducers torch
    registers), so colocated sync never stages weights through the host."""

    weights = None  # marks a remote engine: the updaters take the bucketed path, not the same-process fused copy

    def __init__(self, handle, num_gpus: int = 1, gpu_offset: int = 0, parallel_config: dict | None = None):
        self.handle, self.num_gpus, self.gpu_offset = handle, num_gpus, gpu_offset
        self.parallel_config = parallel_config or {}

    def update_weights(self, named_tensors, version=None, flush_cache=False):
        import torch

        named = [(n, t.contiguous()) for n, t in named_tensors]
        if not named:
            return []
        meta, chunks, off = [], [], 0
        for n, t in named:
            nbytes = t.numel() * t.element_size()
            meta.append((n, str(t.dtype).replace("torch.", ""), list(t.shape), off))
            chunks.append(t.view(-1).view(torch.uint8))
            pad = (-nbytes) % 16  # keep every view 16-byte aligned inside the flat buffer
            if pad:
                chunks.append(torch.zeros(pad, dtype=torch.uint8, device=t.device))
            off += nbytes + pad
        flat = torch.cat(chunks)
        return actors.get(self.handle.update_weights_flat.remote(flat, meta, version, flush_cache))

    def __getattr__(self, name):
        if name.startswith("_"):
            raise AttributeError(name)
        method = getattr(self.handle, name)

        def call(*a, **k):
            ref = method.remote(*a, **k)
            return ref if name in _DEFERRED_ENGINE_CALLS else actors.get(ref)

        return call


class TrainWorker:
    """Hosts one ``TrainActor`` (slime_b200/backends/train/actor.py) inside an actor process."""

    def __init__(self, world_size: int, rank: int, master_addr: str, master_port: int, local_gpu: int | None = None):
        self.world_size, self.rank = world_size, rank
        self.master_addr, self.master_port, self.local_gpu = master_addr, master_port, local_gpu
        self.actor = None
        self.rollout_manager = None

    def init(self, args, role: str, with_ref: bool = False, with_opd_teacher: bool = False) -> int:
        from slime_b200.backends.train.actor import TrainActor, init_distributed
        from slime_b200.observability import logging_utils

        logging_utils.configure_logger(prefix=f"[{role} {self.rank}] ")
        self.args, self.role = args, role
        init_distributed(args, self.rank, self.world_size, self.master_addr, self.master_port, self.local_gpu)
        if self.rank == 0:
            logging_utils.init_tracking(args, primary=False)
        self.actor = TrainActor(args, role)
        return self.actor.init(with_ref=with_ref, with_opd_teacher=with_opd_teacher)

    def get_parallel_config(self) -> dict:
        from slime_b200.parallel import state as mpu

        return {"dp_size": mpu.get_data_parallel_world_size(False), "cp_size": mpu.get_context_parallel_world_size(),
                "tp_size": mpu.get_tensor_model_parallel_world_size(), "pp_size": mpu.get_pipeline_model_parallel_world_size(),
                "vpp_size": getattr(self.args, "virtual_pipeline_model_parallel_size", None) or 1,
                "microbatch_group_size_per_vp_stage": getattr(self.args, "microbatch_group_size_per_vp_stage", None) or 1}  # fmt: skip

    def set_rollout_manager(self, rollout_manager):
        """Fetch the updatable engines and the broadcast lock; rank 0 also tells the manager how the trainer is
        parallelised so it can split rollout data per DP rank."""
        self.rollout_manager = rollout_manager
        if self.rank == 0:
            actors.get(rollout_manager.set_train_parallel_config.remote(self.get_parallel_config()))
        if self.args.debug_train_only or self.role != "actor":
            return
        self._connect_engines()

    def _connect_engines(self, only_if_new: bool = False):
        engines, lock, num_new, counts, offsets, pcfgs = actors.get(self.rollout_manager.get_updatable_engines_and_lock.remote())
        if only_if_new and num_new == 0 and self.actor.weight_updater is not None:
            return
        proxies = [EngineProxy(e, n, o, c) for e, n, o, c in zip(engines, counts, offsets, pcfgs) if e is not None]
        self.actor.connect_rollout_engines(proxies, actors.LockClient(lock))

    def train(self, rollout_id: int, rollout_data_ref, external_data=None):
        return self.actor.train(rollout_id, rollout_data_ref, external_data=external_data)

    def save_model(self, rollout_id: int, force_sync: bool = False):
        return self.actor.save_model(rollout_id, force_sync=force_sync)

    def update_weights(self):
        a = self.args
        if a.debug_train_only or a.debug_rollout_only:
            return
        if self.rollout_manager is not None and (a.use_fault_tolerance or self.actor.weight_updater is None):
            if self.rank == 0 and a.use_fault_tolerance:
                actors.get(self.rollout_manager.recover_updatable_engines.remote())
            self._barrier()
            self._connect_engines(only_if_new=True)  # replaced engines: rebuild proxies / broadcast groups
        out = self.actor.update_weights()
        if self.rank == 0 and self.rollout_manager is not None:
            actors.get(self.rollout_manager.clear_updatable_num_new_engines.remote())
        return out

    def _barrier(self):
        import torch.distributed as dist

        if dist.is_initialized() and self.world_size > 1:
            dist.barrier()

    def sleep(self, tags=None):
        return self.actor.sleep()

    def wake_up(self, tags=None):
        return self.actor.wake_up()

    def clear_memory(self):
        import gc

        import torch

        gc.collect()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            torch.cuda.empty_cache()

    def pop_metrics(self) -> dict:
        u = self.actor.weight_updater
        return u.pop_metrics() if u is not None else {}

    def shutdown(self):
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()


TrainWorkerActor = actors.remote(TrainWorker)


class TrainGroup:
    """All workers of one role (actor or critic)."""

    def __init__(self, args, num_nodes: int, num_gpus_per_node: int, pg=None, role: str = "actor", with_ref: bool = False,
                 with_opd_teacher: bool = False, worker_cls=None):  # fmt: skip
        self.args, self.role, self._pg = args, role, pg
        self._num_nodes, self._num_gpus_per_node = num_nodes, num_gpus_per_node
        self._with_ref, self._with_opd_teacher = with_ref, with_opd_teacher
        self._worker_cls = worker_cls or TrainWorkerActor
        self._workers: list = []
        self._rollout_manager = None
        self._disk_weight_version = 0

    @property
    def world_size(self) -> int:
        return self._num_nodes * self._num_gpus_per_node

    def _spawn(self):
        addr, port = get_current_node_ip(), get_free_port(start_port=29500)
        env = {"NCCL_CUMEM_ENABLE": os.environ.get("NCCL_CUMEM_ENABLE", "0"),
               "NVTE_FP8_BLOCK_SCALING_FP32_SCALES": "1", "CUDA_DEVICE_MAX_CONNECTIONS": "1"}  # fmt: skip
        if getattr(self.args, "deterministic_mode", False):
            env |= {"NCCL_ALGO": "Ring", "CUBLAS_WORKSPACE_CONFIG": ":4096:8"}
        for rank in range(self.world_size):
            gpu = self._pg.gpu(rank).gpu_id if self._pg is not None and self._pg.count else None
            self._workers.append(self._worker_cls.options(name=f"{self.role}-{rank}", env=env, max_concurrency=2).remote(
                self.world_size, rank, addr, port, gpu))  # fmt: skip

    def create(self, rollout_manager=None):
        if self._workers:
            return None
        if rollout_manager is not None:
            self._rollout_manager = rollout_manager
        self.args.update_weight_start_version = self._disk_weight_version
        self._spawn()
        start_ids = actors.get([w.init.remote(self.args, self.role, with_ref=self._with_ref,
                                              with_opd_teacher=self._with_opd_teacher) for w in self._workers])  # fmt: skip
        if self._rollout_manager is not None:
            self.set_rollout_manager(self._rollout_manager)
        return start_ids

    def set_rollout_manager(self, rollout_manager):
        self._rollout_manager = rollout_manager
        return actors.get([w.set_rollout_manager.remote(rollout_manager) for w in self._workers])

    def async_train(self, rollout_id: int, rollout_data_ref, external_data=None) -> list:
        """One future per worker. Critic futures resolve to ``{"values": [...]}`` on the last pipeline stage;
        ``external_data`` is either one item per worker (critic futures) or one object for all."""
        if isinstance(external_data, list):
            assert len(external_data) == len(self._workers)
            return [w.train.remote(rollout_id, rollout_data_ref, external_data=ed) for w, ed in zip(self._workers, external_data)]
        return [w.train.remote(rollout_id, rollout_data_ref, external_data=external_data) for w in self._workers]

    def train(self, rollout_id: int, rollout_data_ref, external_data=None):
        return actors.get(self.async_train(rollout_id, rollout_data_ref, external_data))

    def save_model(self, rollout_id: int, force_sync: bool = False):
        out = actors.get([w.save_model.remote(rollout_id, force_sync=force_sync) for w in self._workers])
        if self._release_train_enabled():  # the next create() resumes from what was just written
            a = self.args
            a.load, a.ckpt_step, a.finetune = a.save, None, False
            a.no_load_optim, a.no_load_rng = a.no_save_optim, False
        return out

    def update_weights(self):
        if not self._full_disk_weight_update_enabled():
            return actors.get([w.update_weights.remote() for w in self._workers])
        version = self._disk_weight_version + 1
        vdir = Path(self.args.update_weight_disk_dir) / f"weight_v{version:06d}"
        actors.get([w.update_weights.remote() for w in self._workers])
        self._disk_weight_version = version
        if self._release_train_enabled():
            self.release()
        self._reload_rollout_weights_from_disk(vdir, str(version))

    def onload(self):
        return actors.get([w.wake_up.remote() for w in self._workers])

    def offload(self):
        return actors.get([w.sleep.remote() for w in self._workers])

    def clear_memory(self):
        return actors.get([w.clear_memory.remote() for w in self._workers])

    def release(self):
        workers, self._workers = self._workers, []
        for w in workers:
            actors.kill(w)
        if workers:
            time.sleep(0.5)  # let the driver reclaim the contexts before the engines grow back

    def _release_train_enabled(self) -> bool:
        return self.role == "actor" and bool(getattr(self.args, "release_train", False))

    def _full_disk_weight_update_enabled(self) -> bool:
        a = self.args
        return self.role == "actor" and a.update_weight_mode == "full" and a.update_weight_transport == "disk"

    def _reload_rollout_weights_from_disk(self, vdir: Path, version: str):
        """Driver-side half of the disk transport: used when the trainer processes may already be gone
        (``--release-train``), so the engines are told to reload by the driver, not by trainer rank 0."""
        rm, a = self._rollout_manager, self.args
        assert rm is not None, "disk weight update needs a rollout manager"
        if a.offload_rollout:
            actors.get(rm.onload_weights.remote())
        engines, *_ = actors.get(rm.get_updatable_engines_and_lock.remote())
        engines = [e for e in engines if e is not None]
        if not engines:
            if not a.update_weight_disk_keep_files:
                shutil.rmtree(vdir, ignore_errors=True)
            return
        model_path = str(vdir)
        if a.update_weight_local_checkpoint_dir:
            actors.get([e.pull_weights.remote(a.update_weight_local_checkpoint_dir, a.update_weight_disk_dir, int(version))
                        for e in engines])  # fmt: skip
            model_path = a.update_weight_local_checkpoint_dir
        actors.get([e.pause_generation.remote() for e in engines])
        actors.get([e.flush_cache.remote() for e in engines])
        actors.get([e.update_weights_from_disk.remote(model_path=model_path, weight_version=version) for e in engines])
        if getattr(a, "ci_test", False):
            got = actors.get([e.get_weight_version.remote() for e in engines])
            bad = [f"engine {i}: {v}" for i, v in enumerate(got) if str(v) != str(version)]
            assert not bad, f"engines did not reach weight version {version}: {bad}"
        actors.get([e.continue_generation.remote() for e in engines])
        if not a.update_weight_disk_keep_files:
            shutil.rmtree(vdir, ignore_errors=True)

    def shutdown(self):
        for w in self._workers:
            try:
                actors.get(w.shutdown.remote(), timeout=10)
            except Exception:  # noqa: BLE001
                pass
        self.release()


# ------------------------------------------------------------------------------- factories
def create_rollout_manager(args, pg):
    from slime_b200.runtime.rollout_manager import RolloutManager

    rm = RolloutManager.options(name="rollout-manager", max_concurrency=4).remote(args, pg)
    per_epoch = None
    if args.num_rollout is None:
        per_epoch = actors.get(rm.get_num_rollout_per_epoch.remote())
        args.num_rollout = per_epoch * args.num_epoch
        assert args.num_rollout > 0
    if args.check_weight_update_equal:
        actors.get(rm.check_weights.remote(action="snapshot"))
        actors.get(rm.check_weights.remote(action="reset_tensors"))
    if args.offload_rollout:
        actors.get(rm.offload.remote())
    return rm, per_epoch


def create_actor_model(args, pgs, rollout_manager, worker_cls=None):
    from slime_b200.utils.arguments import get_role_args

    actor_args = get_role_args(args, "actor")  # --megatron-config-path actor overrides are already merged into args
    g = TrainGroup(actor_args, args.actor_num_nodes, args.actor_num_gpus_per_node, pgs.get("actor"), "actor",
                   with_ref=actor_args.kl_coef != 0 or actor_args.use_kl_loss,
                   with_opd_teacher=bool(actor_args.use_opd and actor_args.opd_type == "megatron"), worker_cls=worker_cls)  # fmt: skip
    return g, g.create(rollout_manager=rollout_manager)


def create_training_models(args, pgs, rollout_manager, worker_cls=None):
    actor_model, start_ids = create_actor_model(args, pgs, rollout_manager, worker_cls)
    critic_model = None
    if args.use_critic and args.num_rollout != 0:
        from slime_b200.utils.arguments import get_role_args

        critic_args = copy.deepcopy(get_role_args(args, "critic"))
        if not getattr(args, "megatron_config_path", None):
            critic_args.disable_param_buffers_cpu_backup = False
        critic_model = TrainGroup(critic_args, args.critic_num_nodes, args.critic_num_gpus_per_node, pgs.get("critic"), "critic")
        start_ids = critic_model.create(rollout_manager=rollout_manager)
    assert len(set(start_ids)) == 1, f"workers disagree on the start rollout id: {start_ids}"
    if args.start_rollout_id is None:
        args.start_rollout_id = start_ids[0]
    if args.rollout_global_dataset:
        actors.get(rollout_manager.load.remote(args.start_rollout_id - 1))
    return actor_model, critic_model
