"""Check that a server group's engines fit into the GPUs placed for rollout.

A group of ``num_engines`` engines starts at ``gpu_offset`` in the (node, gpu)-ordered list of rollout GPUs and takes
``num_gpus_per_engine`` consecutive entries per engine; the error names every quantity involved, because the cause is
usually a YAML offset or a per-engine size that disagrees with ``--rollout-num-gpus``. Parity:
slime/ray/rollout_validation.py:1-32.
"""

from __future__ import annotations


def validate_server_group_gpu_indices(*, worker_type: str, gpu_offset: int, num_gpus_per_engine: int, num_gpus_per_engine_on_node: int,
                                      num_engines: int, num_available_gpus: int, rollout_num_gpus: int,
                                      rollout_num_gpus_per_engine: int) -> None:  # fmt: skip
    if num_engines <= 0:
        return
    required = gpu_offset + num_engines * num_gpus_per_engine
    if gpu_offset < 0 or required > num_available_gpus:
        raise ValueError(
            "server group does not fit into the rollout GPUs: "
            f"worker_type={worker_type}, gpu_offset={gpu_offset}, num_gpus_per_engine={num_gpus_per_engine}, "
            f"num_gpus_per_engine_on_node={num_gpus_per_engine_on_node}, num_engines={num_engines}, required_gpu_slots={required}, "
            f"len(reordered_gpu_ids)={num_available_gpus}, rollout_num_gpus={rollout_num_gpus}, "
            f"rollout_num_gpus_per_engine={rollout_num_gpus_per_engine}")  # fmt: skip
