"""Run under torchrun on >= 2 GPUs: the fused sequence-parallel linears (all-gather -> GEMM, GEMM -> reduce-scatter, one
kernel each over NVLink peer memory) against NCCL collectives around the plain GEMM, forward and backward, plus device
timings (max over ranks) at the shapes of a Qwen3-4B layer under TP = world."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    import faulthandler

    faulthandler.dump_traceback_later(280, exit=True)
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from slime_b200 import ops
    from slime_b200.ops import _lib, build
    from slime_b200.parallel import fused_tp, state as mpu, tensor_parallel as tp

    build.build()
    os.environ["SLIME_B200_FORCE_FUSED_RS"] = "1"  # this check measures the single-kernel path at every shape
    mpu.initialize_model_parallel(tensor_model_parallel_size=world)
    dev = torch.device("cuda", local)
    H = 2560
    fl = fused_tp.sequence_parallel_linears(mpu.get_tensor_model_parallel_group(), H, dev, max_tokens=9216)
    assert fl is not None, "fused linears unavailable on this box"
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    gw = torch.Generator(device=dev).manual_seed(7)

    def rnd(*shape, gen=g, s=1.0):
        return (torch.randn(*shape, device=dev, generator=gen) * s).to(torch.bfloat16)

    worst = {}
    for rows, n_col, k_row in [(128, 256, 128), (384, 3072, 1024), (1024, 9728, 4864)]:
        T = rows * world
        # ---- column-parallel: y = gather(x) W^T + b
        x = rnd(rows, H).requires_grad_()
        w = rnd(n_col, H, gen=gw, s=0.05).requires_grad_()
        b = rnd(n_col, gen=gw, s=0.1).requires_grad_()
        dy = rnd(T, n_col, s=0.5)
        y = fl.column(x, w, b)
        y.backward(dy)
        got = (y.detach(), x.grad.clone(), w.grad.clone(), b.grad.clone())
        x.grad = w.grad = b.grad = None
        y2 = ops.linear(tp.gather_from_sequence_parallel_region(x), w, b)
        y2.backward(dy)
        want = (y2.detach(), x.grad, w.grad, b.grad)
        for name, a, r in zip(("col.y", "col.dx", "col.dw", "col.db"), got, want):
            err = float((a.float() - r.float()).abs().max()) / (float(r.float().abs().max()) + 1e-6)
            worst[name] = max(worst.get(name, 0.0), err)
            assert err < 2e-2, (name, rows, err)
        assert torch.equal(got[0], want[0]), "fused and unfused forward of the column linear differ"  # same tiles, same order
        # ---- row-parallel: y_local = reduce_scatter(x W^T)
        x = rnd(T, k_row).requires_grad_()
        w = rnd(H, k_row, gen=g, s=0.05).requires_grad_()
        dy = rnd(rows, H, s=0.5)
        y = fl.row(x, w)
        y.backward(dy)
        got = (y.detach(), x.grad.clone(), w.grad.clone())
        x.grad = w.grad = None
        y2 = tp.reduce_scatter_to_sequence_parallel_region(ops.linear(x, w))
        y2.backward(dy)
        want = (y2.detach(), x.grad, w.grad)
        for name, a, r in zip(("row.y", "row.dx", "row.dw"), got, want):
            err = float((a.float() - r.float()).abs().max()) / (float(r.float().abs().max()) + 1e-6)
            worst[name] = max(worst.get(name, 0.0), err)
            assert err < 2e-2, (name, rows, err)
    torch.cuda.synchronize()
    _lib.check_status(dev)

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

    T = 9216
    rows = T // world
    res = {}
    with torch.no_grad():
        x_loc, full = rnd(rows, H), torch.empty(T, H, device=dev, dtype=torch.bfloat16)
        for name, n_col in (("qkv", 6144 // world), ("fc1", 19456 // world)):
            w = rnd(n_col, H, gen=gw, s=0.05)

            def nccl():
                dist.all_gather_into_tensor(full, x_loc)
                ops.gemm(full, w)

            res[f"ag_{name}"] = (timed(lambda: fl.ag(x_loc, w)), timed(nccl), timed(lambda: ops.gemm(full, w)))
        for name, k_row in (("proj", 4096 // world), ("fc2", 9728 // world)):
            x = rnd(T, k_row)
            w = rnd(H, k_row, gen=gw, s=0.05)
            part, out = torch.empty(T, H, device=dev, dtype=torch.bfloat16), torch.empty(rows, H, device=dev, dtype=torch.bfloat16)

            def nccl():
                ops.gemm(x, w, out=part)
                dist.reduce_scatter_tensor(out, part)

            res[f"rs_{name}"] = (timed(lambda: fl.rs(x, w)), timed(nccl), timed(lambda: ops.gemm(x, w, out=part)))
    _lib.check_status(dev)
    if rank == 0:
        tim = " ".join(f"{k}: fused {a:.0f} us / nccl+gemm {b:.0f} us / gemm only {c:.0f} us;" for k, (a, b, c) in res.items())
        print(f"RESULT ok world={world} T={T} H={H} worst_rel_err={max(worst.values()):.2e} {tim}", flush=True)
    from slime_b200.utils.distributed_utils import shutdown_distributed

    shutdown_distributed()


if __name__ == "__main__":
    main()
