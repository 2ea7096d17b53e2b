"""Hugging Face checkpoint -> native ``torch_dist`` checkpoint (``{save}/release``).

    python -m slime_b200.tools.convert_hf_to_torch_dist --hf-checkpoint /ckpt/Qwen3-4B --save /ckpt/Qwen3-4B_torch_dist
    torchrun --nproc-per-node 8 -m slime_b200.tools.convert_hf_to_torch_dist ... --tensor-model-parallel-size 2 ...

Single process by default; under ``torchrun`` the model is built with the given parallel sizes (pipeline size defaults
to the world size, so each rank only materialises its stage) and every rank writes its shards. The result loads under
any other parallel layout because tensors are stored whole. Parity: tools/convert_hf_to_torch_dist.py:1-146.
"""

from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist


def main(argv=None):
    from slime_b200.backends.train import checkpoint as ckpt
    from slime_b200.backends.train.model import TrainModel
    from slime_b200.checkpoint.hf_loader import load_hf_weights
    from slime_b200.parallel import state as mpu
    from slime_b200.utils.arguments import namespace_from_dict

    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--hf-checkpoint", required=True)
    p.add_argument("--save", required=True)
    p.add_argument("--tensor-model-parallel-size", type=int, default=1)
    p.add_argument("--pipeline-model-parallel-size", type=int, default=None)
    p.add_argument("--expert-model-parallel-size", type=int, default=1)
    p.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = p.parse_args(argv)

    world = int(os.environ.get("WORLD_SIZE", 1))
    if world > 1:
        local = int(os.environ.get("LOCAL_RANK", 0))
        if a.device == "cuda":
            torch.cuda.set_device(local)
        dist.init_process_group("nccl" if a.device == "cuda" else "gloo")
    pp = a.pipeline_model_parallel_size or max(1, world // (a.tensor_model_parallel_size * a.expert_model_parallel_size))
    mpu.initialize_model_parallel(a.tensor_model_parallel_size, pp, None, 1, a.expert_model_parallel_size, 1)
    args = namespace_from_dict(dict(hf_checkpoint=a.hf_checkpoint, save=a.save, num_rollout=0, rollout_batch_size=1,
                                    tensor_model_parallel_size=a.tensor_model_parallel_size,
                                    pipeline_model_parallel_size=pp, expert_model_parallel_size=a.expert_model_parallel_size))  # fmt: skip
    model = TrainModel(args, device=torch.device(a.device), with_optimizer=False)
    missing = load_hf_weights(a.hf_checkpoint, model)
    if missing:
        raise SystemExit(f"the HF checkpoint has no source for: {missing}")
    ckpt.save_checkpoint(args, "release", model, save_optimizer=False, base=a.save)
    ckpt.finalize_async_saves()
    if not dist.is_initialized() or dist.get_rank() == 0:
        print(f"wrote {ckpt.checkpoint_dir(a.save, 'release')}")
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
