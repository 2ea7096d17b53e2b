"""Run under torchrun on >= 2 GPUs: the fused all-reduce + residual + RMSNorm kernel against NCCL + plain PyTorch.

Checks eager calls for several token counts (with and without a residual), that all ranks hold bit-identical outputs,
and a CUDA graph that contains four calls replayed several times. Prints RESULT with device timings (max over ranks).
"""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from slime_b200.ops import _lib, build
    from slime_b200.parallel.fused_tp import FusedAllReduceNorm

    build.build()
    dev = torch.device("cuda", local)
    H, maxT, eps = 2560, 512, 1e-6
    ar = FusedAllReduceNorm(dist.group.WORLD, maxT, H, dev)
    if rank == 0:
        print(f"fused path: {'multimem' if ar.use_mc else 'p2p'} world={world}", flush=True)
    gw = torch.Generator(device=dev).manual_seed(5)
    w = (1 + 0.1 * torch.randn(H, device=dev, generator=gw)).to(torch.bfloat16)

    def reference(part, res):
        tot = part.float().clone()
        dist.all_reduce(tot)
        h = tot + (res.float() if res is not None else 0)
        y = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * w.float()
        return y, h

    for step, T in enumerate((1, 7, 148, 149, 256, 512)):
        g = torch.Generator(device=dev).manual_seed(1000 * step + rank)
        gr = torch.Generator(device=dev).manual_seed(77 + step)  # the residual is replicated: same seed everywhere
        ar.begin_forward()
        for use_res in (False, True):
            part = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
            res = torch.randn(T, H, device=dev, generator=gr).to(torch.bfloat16) if use_res else None
            ar.partial(T).copy_(part)
            y, r = ar(T, res, w, eps)
            y_ref, h_ref = reference(part, res)
            torch.cuda.synchronize()
            _lib.check_status(dev)
            # bf16 partials summed in fp32: the kernel and the reference see the same inputs, so only the output rounding differs
            torch.testing.assert_close(r.float(), h_ref, rtol=1e-2, atol=2e-2)
            torch.testing.assert_close(y.float(), y_ref, rtol=2e-2, atol=2e-2)
            both = [torch.empty_like(y) for _ in range(world)]
            dist.all_gather(both, y)
            assert all(torch.equal(both[0], b) for b in both), "ranks disagree bit-wise"
    # CUDA graph with four calls (an even count keeps the buffers alternating across replays)
    T = 256
    part = torch.randn(T, H, device=dev, generator=torch.Generator(device=dev).manual_seed(rank)).to(torch.bfloat16)
    res0 = torch.zeros(T, H, device=dev, dtype=torch.bfloat16)
    y_out, r_out = torch.empty_like(res0), torch.empty_like(res0)

    def four_calls():
        ar.begin_forward()
        res = res0
        for _ in range(4):
            ar.partial(T).copy_(part)
            y, res = ar(T, res, w, eps)
        y_out.copy_(y)
        r_out.copy_(res)

    four_calls()
    torch.cuda.synchronize()
    eager_y, eager_r = y_out.clone(), r_out.clone()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        four_calls()
        with torch.cuda.graph(graph, stream=side):
            four_calls()
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    _lib.check_status(dev)
    assert torch.equal(y_out, eager_y) and torch.equal(r_out, eager_r), "graph replay differs from eager"

    def timed(fn, n=20):
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

    from slime_b200 import ops

    def nccl_path():
        x = part.clone()
        dist.all_reduce(x)
        ops.rmsnorm(x, w, eps, res0)

    def fused_path():
        ar.partial(T).copy_(part)
        ar(T, res0, w, eps)
        ar.partial(T).copy_(part)
        ar(T, res0, w, eps)

    t_nccl, t_fused = timed(nccl_path), timed(fused_path) / 2
    _lib.check_status(dev)
    if rank == 0:
        print(f"RESULT ok T={T} H={H} nccl_us={t_nccl:.1f} fused_us={t_fused:.1f}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
