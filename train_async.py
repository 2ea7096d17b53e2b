"""One-step-off-policy RL training driver: rollout N+1 is generated while the trainer works on rollout N.

Engines and trainers must be on different GPUs (no ``--colocate``). Weights are pushed every
``--update-weights-interval`` rollouts; before a push the in-flight generation is drained so no rollout mixes two
policies. Same control flow and flags as the reference driver (train_async.py:9-84 there).
"""

from slime_b200.observability.logging_utils import configure_logger, finish_tracking, init_tracking
from slime_b200.runtime import actors
from slime_b200.runtime.placement import create_placement_groups
from slime_b200.runtime.train_group import create_rollout_manager, create_training_models
from slime_b200.utils.arguments import parse_args
from slime_b200.utils.misc import should_run_periodic_action


def train(args):
    assert not args.colocate, "async training needs engines and trainers on different GPUs (drop --colocate)"
    configure_logger()
    release_train = args.release_train
    pgs = create_placement_groups(args)
    init_tracking(args)
    rollout_manager, num_rollout_per_epoch = create_rollout_manager(args, pgs["rollout"])
    actor_model, critic_model = create_training_models(args, pgs, rollout_manager)
    get = actors.get

    actor_model.update_weights()
    if args.check_weight_update_equal:
        get(rollout_manager.check_weights.remote(action="compare"))

    try:
        next_future = rollout_manager.generate.remote(args.start_rollout_id)
        current_ref = None
        for rollout_id in range(args.start_rollout_id, args.num_rollout):
            if next_future is not None:
                current_ref = get(next_future)
            if rollout_id + 1 < args.num_rollout:
                next_future = rollout_manager.generate.remote(rollout_id + 1)  # overlaps with the training below
            if release_train:
                actor_model.create()

            actor_trains = (not args.use_critic) or rollout_id >= args.num_critic_only_steps
            if args.use_critic:
                value_refs = critic_model.async_train(rollout_id, current_ref)
                if actor_trains:
                    get(actor_model.async_train(rollout_id, current_ref, external_data=value_refs))
                else:
                    get(value_refs)
            else:
                get(actor_model.async_train(rollout_id, current_ref))

            if release_train or should_run_periodic_action(rollout_id, args.save_interval, num_rollout_per_epoch, args.num_rollout):
                force_sync = release_train or rollout_id == args.num_rollout - 1
                if actor_trains:
                    actor_model.save_model(rollout_id, force_sync=force_sync)
                if args.use_critic:
                    critic_model.save_model(rollout_id, force_sync=force_sync)
                if args.rollout_global_dataset:
                    get(rollout_manager.save.remote(rollout_id))

            if release_train or (rollout_id + 1) % args.update_weights_interval == 0:
                # drain the generation in flight first: its samples must come from one policy version
                current_ref = get(next_future) if next_future is not None else None
                next_future = None
                actor_model.update_weights()

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
