"""Synchronous RL training driver: generate -> train -> sync weights, one rollout at a time.

    python train.py --hf-checkpoint ... --prompt-data ... --rollout-batch-size 32 --n-samples-per-prompt 8 ...

Processes: this driver, one rollout manager, one engine per ``--rollout-num-gpus-per-engine`` GPUs and one trainer
per training GPU. With ``--colocate`` trainers and engines share GPUs and hand memory back and forth between
the phases. Same control flow and flags as the reference driver (train.py:9-99 there).
"""

from slime_b200.observability.logging_utils import configure_logger, finish_tracking, init_tracking
from slime_b200.runtime import actors
from slime_b200.runtime.placement import create_placement_groups
from slime_b200.runtime.train_group import create_rollout_manager, create_training_models
from slime_b200.utils.arguments import parse_args
from slime_b200.utils.misc import should_run_periodic_action


def train(args):
    configure_logger()
    release_train = args.release_train
    pgs = create_placement_groups(args)
    init_tracking(args)
    rollout_manager, num_rollout_per_epoch = create_rollout_manager(args, pgs["rollout"])
    actor_model, critic_model = create_training_models(args, pgs, rollout_manager)
    get = actors.get

    if args.offload_rollout and not release_train:
        get(rollout_manager.onload_weights.remote())
    actor_model.update_weights()  # engines start from the trainer's weights, not from whatever they loaded
    if args.check_weight_update_equal:
        get(rollout_manager.check_weights.remote(action="compare"))
    if args.offload_rollout:
        get(rollout_manager.onload_kv.remote())
    if args.num_rollout == 0 and args.eval_interval is not None:
        get(rollout_manager.eval.remote(rollout_id=0))

    def free_trainer_memory(actor_trained: bool):
        if args.offload_train:
            return  # the trainer goes to sleep inside update_weights instead
        (actor_model if (not args.use_critic or actor_trained) else critic_model).clear_memory()

    try:
        for rollout_id in range(args.start_rollout_id, args.num_rollout):
            if args.eval_interval is not None and rollout_id == 0 and not args.skip_eval_before_train:
                get(rollout_manager.eval.remote(rollout_id))
            rollout_data_ref = get(rollout_manager.generate.remote(rollout_id))
            if args.offload_rollout:
                get(rollout_manager.offload.remote())
            if release_train:
                actor_model.create()

            actor_trains = (not args.use_critic) or rollout_id >= args.num_critic_only_steps
            if args.use_critic:
                value_refs = critic_model.async_train(rollout_id, rollout_data_ref)
                if actor_trains:
                    get(actor_model.async_train(rollout_id, rollout_data_ref, external_data=value_refs))
                else:
                    get(value_refs)
            else:
                get(actor_model.async_train(rollout_id, rollout_data_ref))

            if release_train or should_run_periodic_action(rollout_id, args.save_interval, num_rollout_per_epoch, args.num_rollout):
                force_sync = release_train or rollout_id == args.num_rollout - 1
                if actor_trains:
                    actor_model.save_model(rollout_id, force_sync=force_sync)
                if args.use_critic:
                    critic_model.save_model(rollout_id, force_sync=force_sync)
                if args.rollout_global_dataset:
                    get(rollout_manager.save.remote(rollout_id))

            free_trainer_memory(actor_trains)
            if args.offload_rollout and not release_train:
                get(rollout_manager.onload_weights.remote())
            actor_model.update_weights()
            if args.offload_rollout:
                get(rollout_manager.onload_kv.remote())
            if should_run_periodic_action(rollout_id, args.eval_interval, num_rollout_per_epoch):
                get(rollout_manager.eval.remote(rollout_id))
    finally:
        try:
            get(rollout_manager.dispose.remote(), timeout=60)
        finally:
            actor_model.shutdown()
            if critic_model is not None:
                critic_model.shutdown()
            actors.kill(rollout_manager)
            actors.shutdown()
            finish_tracking(args)


if __name__ == "__main__":
    train(parse_args())
