"""Run under torchrun on >= 2 GPUs: the all-gather-fused GEMM against NCCL all-gather + the plain GEMM and fp32 math."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from slime_b200 import ops
    from slime_b200.ops import _lib, build
    from slime_b200.parallel.fused_tp import AllGatherGemm

    build.build()
    dev = torch.device("cuda", local)
    K, N, max_rows = 2560, 3072, 4096
    ag = AllGatherGemm(dist.group.WORLD, max_rows, K, dev)
    gw = torch.Generator(device=dev).manual_seed(5)
    w = (torch.randn(N, K, device=dev, generator=gw) * 0.05).to(torch.bfloat16)
    bias = (torch.randn(N, device=dev, generator=gw) * 0.1).to(torch.bfloat16)
    for step, (rows, dtype, use_bias) in enumerate([(128, torch.bfloat16, False), (384, torch.float32, True), (4096, torch.bfloat16, True)]):
        g = torch.Generator(device=dev).manual_seed(10 * step + rank)
        x = torch.randn(rows, K, device=dev, generator=g).to(torch.bfloat16)
        full = torch.empty(world * rows, K, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, x)
        ref = ops.gemm(full, w, bias=bias if use_bias else None, out_dtype=dtype)
        exact = full.float() @ w.float().t() + (bias.float() if use_bias else 0)
        for mode in ("direct", "staged"):
            ag.shard(rows).copy_(x)
            y = ag(rows, w, bias if use_bias else None, out_dtype=dtype, mode=mode)
            torch.cuda.synchronize()
            _lib.check_status(dev)
            assert (y.float() - exact).abs().max() <= 0.02 * exact.abs().max(), (step, mode)
            if mode == "direct":  # same kernel, same tiles: bit-identical to the unfused GEMM
                assert torch.equal(y, ref), f"step {step}: fused and unfused GEMM differ by {(y.float() - ref.float()).abs().max()}"

    rows = 4096
    x = torch.randn(rows, K, device=dev).to(torch.bfloat16)
    full = torch.empty(world * rows, K, device=dev, dtype=torch.bfloat16)

    def timed(fn, n=10):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(n):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t) * 1e3

    def nccl_path():
        dist.all_gather_into_tensor(full, x)
        ops.gemm(full, w)

    def fused_path(mode, weight):
        ag.shard(rows).copy_(x)
        ag(rows, weight, mode=mode)

    t_nccl, t_gemm = timed(nccl_path), timed(lambda: ops.gemm(full, w))
    t_direct, t_staged = timed(lambda: fused_path("direct", w)), timed(lambda: fused_path("staged", w))
    w_narrow = w[:256].contiguous()

    def nccl_narrow():
        dist.all_gather_into_tensor(full, x)
        ops.gemm(full, w_narrow)

    t_nccl_n, t_direct_n = timed(nccl_narrow), timed(lambda: fused_path("direct", w_narrow))
    _lib.check_status(dev)
    if rank == 0:
        print(f"RESULT ok world={world} M={world * rows} N={N} K={K} nccl_ag_plus_gemm_us={t_nccl:.1f} direct_us={t_direct:.1f} "
              f"staged_us={t_staged:.1f} gemm_only_us={t_gemm:.1f} | N=256: nccl_us={t_nccl_n:.1f} direct_us={t_direct_n:.1f}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
