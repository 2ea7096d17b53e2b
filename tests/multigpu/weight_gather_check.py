"""Run under torchrun on 2 or 4 GPUs: device-side weight sync from a tensor-parallel trainer into whole (TP1) engines
(``GatherToEngine``: gather + re-layout + store in one launch) is byte-exact against the host-driven path (NCCL
all-gather per parameter -> Megatron->HF rename / split -> ``load_weights``), and its time for the model's bytes."""

import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    import faulthandler

    faulthandler.dump_traceback_later(280, exit=True)
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from slime_b200.backends.train.model import TrainModel
    from slime_b200.engine.model_runner import EngineWeights
    from slime_b200.models.config import ModelConfig, apply_to_args
    from slime_b200.ops import _lib, build
    from slime_b200.parallel import state as mpu
    from slime_b200.utils.arguments import namespace_from_dict
    from slime_b200.weight_sync import updaters
    from slime_b200.weight_sync.device_sync import GatherToEngine

    build.build()
    mpu.initialize_model_parallel(tensor_model_parallel_size=world)
    dev = torch.device("cuda", local)
    layers = int(os.environ.get("LAYERS", "4"))
    cfg = ModelConfig(num_layers=layers, hidden_size=2560, num_attention_heads=32, num_query_groups=8, kv_channels=128,
                      ffn_hidden_size=9728, vocab_size=151936, rotary_base=1e6, tie_word_embeddings=False, qk_layernorm=True,
                      padded_vocab_size=151936 + (-151936) % (128 * world))  # Qwen3-4B layers
    args = namespace_from_dict(dict(tensor_model_parallel_size=world, sequence_parallel=True, seed=3, fused_dp_step=False,
                                    untie_embeddings_and_output_weights=True, update_weight_buffer_size=512 * 1024**2))
    apply_to_args(cfg, args)
    model = TrainModel(args, device=dev, with_optimizer=False)
    with torch.no_grad():  # distinct values everywhere (norm weights start as ones)
        for i, p in enumerate(model.parameters()):
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    want = EngineWeights(cfg, torch.bfloat16, dev, 1, 0)
    t0 = time.perf_counter()
    for bucket in updaters.iter_hf_buckets(args, model):
        missing = want.load_weights(bucket)
        assert not missing, missing
    torch.cuda.synchronize()
    host_s = time.perf_counter() - t0
    got = EngineWeights(cfg, torch.bfloat16, dev, 1, 0)
    sync = GatherToEngine(model, got, mpu.get_tensor_model_parallel_group())
    moved = sync.sync()
    torch.cuda.synchronize()
    _lib.check_status(dev)
    def named(w):
        yield "embed", w.embed
        yield "lm_head", w.lm_head
        yield "final_norm", w.final_norm
        for i, L in enumerate(w.layers):
            for k, v in L.items():
                if v is not None:
                    yield f"layers.{i}.{k}", v

    bad = [n for (n, a), (_n, b) in zip(named(got), named(want)) if not torch.equal(a, b)]
    assert not bad, f"device-side weight sync differs from the host-driven path in {bad[:12]}"
    times = []
    for _ in range(3):
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        sync.sync()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    t = torch.tensor([min(times)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    _lib.check_status(dev)
    if rank == 0:
        gb = moved / 1e9
        print(f"RESULT ok world={world} layers={layers} engine_bytes={gb:.3f} GB device_sync_ms={float(t):.2f} "
              f"({gb / (float(t) / 1e3):.0f} GB/s written per GPU) host_path_s={host_s:.2f}", flush=True)
    from slime_b200.utils.distributed_utils import shutdown_distributed

    shutdown_distributed()


if __name__ == "__main__":
    main()
