"""N-sharded MLP step (BASELINE.json configs[3], the fourth config: BFloat16, batch 8192, 4096 -> 16384 -> 4096, ReLU, MSE) on the GPUs of one box.

    python -m neurotensor_b200.bench_mlp_sharded                       # 1 GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m neurotensor_b200.bench_mlp_sharded [--steps K] [--check] [--nccl]

Strong scaling: the problem is fixed, every large GEMM is split over its output columns across the ranks, and the
hidden activations and the output are gathered by the GEMMs' own epilogues (TMA stores into every rank's buffer,
partition.ShardedMLP.step_fused); `--nccl` gathers them with NCCL all-gathers instead.  Time is CUDA events around K
steps between barriers, maximum over ranks.  `--check` compares rank 0's loss and gradient shards with the same step
run unsharded on rank 0.  Prints one JSON line on rank 0.
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from neurotensor_b200 import _lib, partition  # noqa: E402


def measure(rank, world, dist=None, steps=10, batch=8192, din=4096, hidden=16384, check=False, nccl=False, warmup=3, phases=False,
            schedule="auto"):
    """Times the N-sharded step on the ranks of an initialised process group (dist = torch.distributed, or None for one
    rank) and returns the result record on every rank (`check` is filled on rank 0 only)."""
    B, D, H = batch, din, hidden
    dt = torch.bfloat16
    gen = torch.Generator(device="cuda").manual_seed(9)          # same seed on every rank: replicated tensors agree
    rn = lambda shape, s=1.0: (torch.randn(shape, generator=gen, device="cuda") * s).to(dt)
    x, t = rn((B, D)), rn((B, D))
    w1, w2 = rn((D, H), D ** -0.5), rn((H, D), H ** -0.5)
    b1, b2 = rn((H,), 0.01), rn((D,), 0.01)
    h0, hn = partition.column_shard(H, world, rank)
    mlp = partition.ShardedMLP(w1[:, h0:h0 + hn].contiguous(), b1[h0:h0 + hn].contiguous(), w2, b2, rank, world)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def all_ranks(ok):
        """True when `ok` holds on every rank (one all-reduce, so the ranks take the same branch afterwards)."""
        if dist is None:
            return bool(ok)
        flag = torch.tensor([1 if ok else 0], device="cuda", dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        return bool(flag.item())

    fused = (not nccl) and world > 1
    fused_error = None
    if fused:
        # peer mappings are made rank by rank; a rank that cannot map a peer must not leave the others waiting in the
        # first exchange, so the outcome is agreed on and every rank falls back to the NCCL gather together
        try:
            mlp.enable_fused_gather(B)
        except Exception as exc:   # noqa: BLE001 - reported in the record
            fused_error = "%s: %s" % (type(exc).__name__, exc)
        if not all_ranks(fused_error is None):
            fused_error = fused_error or "another rank could not map its peers"
            fused = False
    step = mlp.step_fused if fused else mlp.step
    schedule_ms = None
    if fused and schedule != "plain":
        # two forward schedules give the same bits: one row block, or two row blocks on two streams so that the
        # gather of one overlaps the math of the other.  Which is faster depends on how long the gather is against the
        # math (i.e. on the number of ranks): both are timed for a few steps and every rank takes the faster one (the
        # times are maxima over the ranks, so the choice is the same everywhere).
        four = lambda a, b: mlp.step_fused_pipelined(a, b, 4)
        early = lambda a, b: mlp.step_fused_pipelined(a, b, 2, True)
        variants = {"plain": mlp.step_fused, "pipelined": mlp.step_fused_pipelined, "pipelined_dw2": early, "pipelined4": four}
        if schedule in ("pipelined", "pipelined4", "pipelined_dw2"):
            step = variants[schedule]
        else:
            schedule_ms = {}
            for name, fn in list(variants.items())[:3]:   # four blocks lost on two and on eight GPUs: on request only
                for _ in range(2):
                    fn(x, t)
                barrier()
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record()
                for _ in range(5):
                    fn(x, t)
                a1.record()
                barrier()
                tt = torch.tensor([a0.elapsed_time(a1) / 5], device="cuda")
                if dist is not None:
                    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                schedule_ms[name] = float(tt.item())
            step = variants[min(schedule_ms, key=schedule_ms.get)]
    for _ in range(warmup):
        loss, grads = step(x, t)
    barrier()
    if fused and not all_ranks(_lib.lib().ntb200_check_device_status(None) == 0):
        # a bounded wait of the flag exchange ran out on some rank during the warm-up: time the NCCL gather instead
        fused_error = "flag exchange timed out during the warm-up: " + _lib.last_error()
        fused = False
        step = mlp.step
        for _ in range(warmup):
            loss, grads = step(x, t)
        barrier()
    l0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        loss, grads = step(x, t)
    e1.record()
    barrier()
    _lib.check(_lib.lib().ntb200_check_device_status(None))
    ms = e0.elapsed_time(e1) / steps
    launches = (_lib.launch_count() - l0) // steps
    if dist is not None:
        tt = torch.tensor([ms], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt.item())
    result_check = None
    if check and rank == 0:
        ref = partition.ShardedMLP(w1, b1, w2, b2, 0, 1)
        rloss, rg = ref.step(x, t)
        # the unsharded step timed on this rank's GPU in the state the sharded timing left it in: the denominator of
        # the strong-scaling efficiency (the other ranks wait at the barrier below)
        torch.cuda.synchronize()
        u0, u1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        u0.record()
        for _ in range(steps):
            ref.step(x, t)
        u1.record()
        torch.cuda.synchronize()
        unsharded_ms = u0.elapsed_time(u1) / steps
        d0, dn = partition.column_shard(D, world, rank)
        rel = lambda a, b: float(((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30)).item())
        result_check = {"loss": [float(loss.item()), float(rloss.item())],
                        "dw1": rel(grads["w1"], rg["w1"][:, h0:h0 + hn]), "dw2": rel(grads["w2"], rg["w2"][:, d0:d0 + dn]),
                        "y": rel(grads["y"], rg["y"]),
                        "unsharded_ms_per_step_same_gpu": unsharded_ms,
                        "strong_scaling_efficiency": unsharded_ms / (world * ms),
                        "bit_identical": bool(torch.equal(grads["w1"], rg["w1"][:, h0:h0 + hn]) and
                                              torch.equal(grads["w2"], rg["w2"][:, d0:d0 + dn]) and torch.equal(grads["y"], rg["y"]))}
        del ref, rg
    phase_ms = None
    if phases and fused:
        # device time of each phase of the fused step (CUDA events between the phases, averaged over the steps), and
        # the layer-1 GEMM of the same shard shape without any peer to store to, for comparison
        mlp.phase_events = []
        barrier()
        for _ in range(steps):
            step(x, t)
        barrier()
        ev, mlp.phase_events = mlp.phase_events, None
        phase_ms = {}
        for (n0, e0_), (n1, e1_) in zip(ev[:-1], ev[1:]):
            if n1 != "start":
                phase_ms[n1] = phase_ms.get(n1, 0.0) + e0_.elapsed_time(e1_) / steps
        from neurotensor_b200 import api
        h_tmp = torch.empty((B, hn), dtype=dt, device="cuda")
        a_tmp = torch.empty((B, hn), dtype=dt, device="cuda")
        for _ in range(3):
            api.gemm(x, mlp.w1, h_tmp, bias=mlp.b1, relu_out=a_tmp)
        torch.cuda.synchronize()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(steps):
            api.gemm(x, mlp.w1, h_tmp, bias=mlp.b1, relu_out=a_tmp)
        f1.record()
        torch.cuda.synchronize()
        phase_ms["layer 1 GEMM + ReLU of the same shard shape, no peers (for comparison)"] = f0.elapsed_time(f1) / steps
        es = 2
        phase_ms["bytes stored to peers per step by layer 1 / layer 2"] = [B * hn * es * (world - 1), B * mlp.dn * es * (world - 1)]
        del h_tmp, a_tmp
    flops = 5 * 2.0 * B * D * H
    record = {"config": "BFloat16 MLP %dx(%d->%d->%d) fwd+bwd step, N-sharded" % (B, D, H, D), "n_gpus": world,
              "ms_per_step": ms, "tflops": flops / (ms * 1e-3) / 1e12, "scaling": "strong", "steps": steps,
              "kernels_per_step_rank0": int(launches), "collectives_per_step": 0 if (world == 1 or fused) else 2,
              "gather": ("stores from the GEMM epilogues into peer-mapped buffers + flag exchange (ntb200_dist_gemm_allgather)" if fused
                         else ("none" if world == 1 else "NCCL all-gather + re-tile")),
              "check": result_check}
    if fused:
        record["forward_schedule"] = ("one row block" if step == mlp.step_fused else
                                      "two row blocks on two streams" if step == mlp.step_fused_pipelined else
                                      "two row blocks on two streams, dW2 alongside the output gather" if step is early else
                                      "four row blocks on four streams")
        if schedule_ms:
            record["forward_schedule_trial_ms"] = schedule_ms
    if fused_error:
        record["fused_gather_unavailable"] = fused_error
    if phase_ms is not None:
        record["phase_ms_rank%d" % rank] = phase_ms
    barrier()
    mlp.close()
    return record


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--batch", type=int, default=8192)
    ap.add_argument("--din", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=16384)
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--fused", action="store_true", help="(default) all-gathers fused into the GEMM epilogues: stores into peer buffers")
    ap.add_argument("--nccl", action="store_true", help="baseline: NCCL all-gather + re-tile kernel instead of the fused epilogues")
    ap.add_argument("--phases", action="store_true", help="also time each phase of the fused step with CUDA events (rank 0 prints them)")
    ap.add_argument("--schedule", default="auto", choices=["auto", "plain", "pipelined", "pipelined_dw2", "pipelined4"],
                    help="forward pass of the fused step: one row block, two row blocks on two streams, or whichever a short trial finds faster")
    args = ap.parse_args()
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    record = measure(rank, world, dist, args.steps, args.batch, args.din, args.hidden, args.check, args.nccl, phases=args.phases, schedule=args.schedule)
    if rank == 0:
        print(json.dumps(record), flush=True)
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
