"""Run under torchrun on >= 2 GPUs: the peer-memory optimizer step against the NCCL reduce-scatter / all-gather path.

Both optimizers start from the same parameters and see the same per-rank gradients for three steps; parameters,
fp32 masters and the reported gradient norm must agree. Run once with NVSwitch multimem and once with plain P2P.
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
    from slime_b200.backends.train.buffers import FlatBuffer
    from slime_b200.backends.train.optimizer import DistributedOptimizer
    from slime_b200.ops import _lib, build

    build.build()
    dev = torch.device("cuda", local)
    torch.manual_seed(0)
    shapes = [(1024, 896), (896,), (4864, 896), (151936 // 8, 64), (7, 3)]

    def make(symmetric):
        torch.manual_seed(1)
        params = [torch.nn.Parameter(torch.randn(*s, device=dev).to(torch.bfloat16)) for s in shapes]
        buf = FlatBuffer(params, [f"p{i}" for i in range(len(params))], dist.group.WORLD, world, rank, dev, symmetric=symmetric)
        opt = DistributedOptimizer([buf], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, clip_grad=1.0)
        return params, buf, opt

    p_ref, b_ref, o_ref = make(False)
    p_fus, b_fus, o_fus = make(True)
    assert b_fus.fused is not None, "symmetric buffers were not created"
    if rank == 0:
        print(f"fused path: {'multimem' if b_fus.fused.use_mc else 'p2p'} world={world}", flush=True)
    for step in range(3):
        g = torch.Generator(device=dev).manual_seed(100 * step + rank)
        for a, b in zip(p_ref, p_fus):
            grad = torch.randn(a.shape, device=dev, generator=g)
            a.main_grad.copy_(grad)
            b.main_grad.copy_(grad)
        b_ref.reduce_scatter_grads()
        n_ref = o_ref.step(grad_scale=0.5)
        n_fus = o_fus.step(grad_scale=0.5)
        torch.cuda.synchronize()
        _lib.check_status(dev)
        torch.testing.assert_close(n_fus, n_ref, rtol=1e-4, atol=1e-6)
        # With more than two ranks the summation order differs (NCCL ring, direct sum in rank order, in-switch sum), so
        # a summed gradient that is zero to within fp32 rounding can come out with either sign, and Adam's first steps
        # move such an element by +-lr regardless of magnitude. Those elements are a few in millions: everything else
        # must agree tightly, and no element may differ by more than the two opposite updates.
        def agree(a, b, rtol, atol, what):
            diff = (a.float() - b.float()).abs()
            bad = diff > atol + rtol * b.float().abs()
            n_bad = int(bad.sum())
            assert n_bad <= max(2, a.numel() // 100000) and float(diff.max()) <= 2.5e-2 * (step + 1), (
                f"{what}: {n_bad} of {a.numel()} elements differ, max {float(diff.max()):.3e}")

        agree(o_fus.state[0]["master"], o_ref.state[0]["master"], 1e-4, 1e-5, "fp32 master")
        agree(b_fus.param_data, b_ref.param_data, 2e-2, 1e-2, "bf16 parameters")
        for a, b in zip(p_ref, p_fus):  # every rank holds every parameter after the all-gather
            agree(b.data, a.data, 2e-2, 1e-2, "gathered parameter")
        b_ref.zero_grad()
        b_fus.zero_grad()
    # timing, device events, max over ranks
    def timed(fn, n=5):
        for _ in range(2):
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
        return float(t)

    def ref_step():
        b_ref.reduce_scatter_grads()
        o_ref.step(grad_scale=0.5)

    t_ref, t_fus = timed(ref_step), timed(lambda: o_fus.step(grad_scale=0.5))
    if rank == 0:
        print(f"RESULT ok numel={b_ref.numel} nccl_ms={t_ref:.3f} fused_ms={t_fus:.3f}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
