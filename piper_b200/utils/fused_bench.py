"""Roofline numbers of the fused compute+collective kernels (run with one rank per GPU).

``python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m piper_b200.utils.fused_bench``

``python -m piper_b200.utils.fused_bench --local f1|f2|f3 [--iters n]`` runs one of the kernels in a single
process on one GPU with every "peer" buffer in that GPU's own memory (F1: a group of one; F2: two weight shards
that are both local; F3: an expert group of one), which is the form a profiler can capture: the kernels take the
same code paths, only the loads and stores that would cross NVLink stay on the device.

For each fused path the script times the kernel with CUDA events (warm-up, then the max over ranks of the
median), and prints the achieved figure next to its roofline: the slower of FLOPs / measured bf16 GEMM peak and
bytes that must cross NVLink / measured peer-copy bandwidth (770 GB/s per direction per GPU).  The NCCL
lowering of the same step is timed alongside for comparison.
"""
from __future__ import annotations

import json
import os
import statistics

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0
GEMM_TFLOPS = 1397.3
# A spin kernel of about half a millisecond goes in front of every timed region: the events then bracket device
# time only, not the host's time to build tensor maps, allocate outputs and launch.
HOST_LEAD_CYCLES = 1_000_000


def _median_ms(fn, iters=8, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ts = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(HOST_LEAD_CYCLES)      # the host enqueues fn's kernels while this spins on the device
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    t = torch.tensor([statistics.median(ts)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def local_main(which: str, iters: int) -> None:
    """Single-process variants of the three kernels (see the module docstring)."""
    from piper_b200.ops import moe as M, native
    from piper_b200.parallel.fused import FusedExpertExchange
    from piper_b200.parallel.symm import SymmetricBuffer

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = native.lib()
    st = native.status_tensor()

    def timed(fn):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(HOST_LEAD_CYCLES)  # the host enqueues fn's kernels while this spins on the device
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        return statistics.median(ts)

    if which == "f1":
        n = 128 * 1024 * 1024                      # 512 MiB of fp32 gradients: far larger than L2
        buf = SymmetricBuffer.create(n * 2 + n * 4 + 2 * 8 + 512, [0], None)
        g_off, f_off = n * 2, n * 2 + n * 4
        buf.view(torch.float32, n, g_off).normal_()
        master = torch.zeros(n, device=dev)
        m, v = torch.zeros_like(master), torch.zeros_like(master)
        counter = torch.zeros(1, dtype=torch.int32, device=dev)
        epoch = [0]

        def f1():
            epoch[0] += 1
            lib.f1_rs_adam_ag(buf.offset_ptrs(g_off), buf.offset_ptrs(0), buf.offset_ptrs(f_off), master, m, v, 0, 1,
                              epoch[0], 1e-4, 0.9, 0.95, 1e-8, 0.0, epoch[0], 1.0, counter, st, 5.0, 296)

        ms = timed(f1)
        hbm = n * (4 + 24 + 2 + 4)                 # grad read, master/m/v read+write, bf16 param write, grad clear
        print(json.dumps({"path": "F1 local (group of one)", "elements": n, "ms": ms, "hbm_GBs": hbm / ms / 1e6,
                          "fraction_of_hbm_peak": hbm / ms / 1e6 / 6549.4}))
    elif which == "f2":
        T, N, K = 4096, 6144, 4096
        w = (torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16)
        x = torch.randn(T, K, device=dev).to(torch.bfloat16)
        y = torch.empty(T, N, dtype=torch.bfloat16, device=dev)
        fl = 2.0 * T * N * K
        ms = timed(lambda: lib.gemm(x, w, y, False, False, False, st))
        print(json.dumps({"path": "plain GEMM of the same shape", "ms": ms, "tflops": fl / ms / 1e9}))
        for shards, gathered in ((2, False), (1, True), (2, True)):
            rows = N // shards
            parts = [w[p * rows:(p + 1) * rows].contiguous() for p in range(shards)]
            full = torch.zeros(N, K, dtype=torch.bfloat16, device=dev) if gathered else None
            scratch = torch.zeros((N + 255) // 256 + 2, dtype=torch.int32, device=dev) if gathered else None
            ptrs = [p.data_ptr() for p in parts]
            ms = timed(lambda: lib.ag_gemm(x, ptrs, 0, full, scratch, y, N, rows, st))
            rec = {"path": f"F2 local: {shards} local shard(s), {'gathered' if gathered else 'direct'} mode", "ms": ms,
                   "tflops": fl / ms / 1e9, "fraction_of_gemm_peak": fl / ms / 1e9 / GEMM_TFLOPS}
            if gathered:
                rec["max_abs_err_vs_full"] = float((full.float() - w.float()).abs().max())
            print(json.dumps(rec))
    else:
        T, D, E, k = 4096, 2048, 128, 8
        xt = torch.randn(T, D, device=dev).to(torch.bfloat16)
        logits = torch.randn(T, E, device=dev).to(torch.bfloat16)
        weights, idx, counts = M.moe_route(logits, k, True)
        ex = FusedExpertExchange([0], None, T, D, E, k, timeout_s=5.0, num_ctas=296)
        state = {}

        def disp():
            state["r"] = ex.dispatch(xt, idx, counts)

        ms_d = timed(disp)
        pos = state["r"][1]

        def comb():
            ex.epoch += 1
            return ex.combine(pos, weights, T)

        ms_c = timed(comb)
        moved = T * k * D * 2
        print(json.dumps({"path": "F3 local (group of one)", "dispatch_ms": ms_d, "combine_ms": ms_c,
                          "dispatch_GBs": 2 * moved / ms_d / 1e6, "combine_GBs": moved / ms_c / 1e6}))
    torch.cuda.synchronize()
    native.check_status()


def main():
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--local", choices=("f1", "f2", "f3"), default=None)
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args()
    if args.local:
        return local_main(args.local, args.iters)
    from piper_b200.ops import moe as M, native
    from piper_b200.parallel.fused import FusedExpertExchange, ShardedWeight
    from piper_b200.parallel.symm import SymmetricBuffer
    from piper_b200.runtime.layout import init_distributed

    rank, world, _ = init_distributed("cuda")
    dev = torch.device("cuda", torch.cuda.current_device())
    ranks = list(range(world))
    lib = native.lib()
    rows = []

    # ---- F1: reduce-scatter + Adam + all-gather on a 256 Mi-element bucket (1 GiB of fp32 gradients)
    n = 256 * 1024 * 1024
    shard = n // world
    buf = SymmetricBuffer.create(n * 2 + n * 4 + 2 * 8 * world + 512, ranks, None)
    g_off = n * 2
    f_off = g_off + n * 4
    grads = buf.view(torch.float32, n, g_off)
    master = torch.zeros(shard, device=dev)
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    st = native.status_tensor()
    epoch = [0]

    def f1(ctas):
        epoch[0] += 1
        lib.f1_rs_adam_ag(buf.offset_ptrs(g_off), buf.offset_ptrs(0), buf.offset_ptrs(f_off), master, m, v, rank,
                          world, epoch[0], 1e-4, 0.9, 0.95, 1e-8, 0.0, epoch[0], 1.0, counter, st, 30.0, ctas)

    for ctas in (148, 296, 592, 1184):
        grads.normal_()
        ms = _median_ms(lambda: f1(ctas))
        # bytes crossing NVLink per direction and rank: this rank reads its slice of every peer's fp32 gradients
        # (4 B/element) and every peer stores its updated bf16 slice into this rank's parameter buffer (2 B/element)
        nvlink = (world - 1) * shard * (4 + 2)
        roof_ms = nvlink / (NVLINK_GBS * 1e6)
        hbm_ms = (shard * (4 + 24 + 2) + n * 4) / (6549.4 * 1e6)
        rows.append({"path": "F1 rs+adam+ag", "ctas": ctas, "world": world, "elements": n, "ms": ms,
                     "nvlink_GBs_per_direction": nvlink / ms / 1e6, "roofline_ms": max(roof_ms, hbm_ms),
                     "fraction_of_roofline": max(roof_ms, hbm_ms) / ms})
    native.check_status()
    flat = torch.randn(n, device=dev)
    tmp = torch.empty(shard, device=dev)
    p16 = torch.empty(n, device=dev, dtype=torch.bfloat16)

    def nccl_f1():
        dist.reduce_scatter_tensor(tmp, flat)
        lib.adam_flat(master, m, v, tmp, p16[rank * shard:(rank + 1) * shard], 1e-4, 0.9, 0.95, 1e-8, 0.0, 1, 1.0)
        dist.all_gather_into_tensor(p16, p16[rank * shard:(rank + 1) * shard].clone())

    rows.append({"path": "NCCL reduce_scatter + adam kernel + all_gather", "world": world, "elements": n,
                 "ms": _median_ms(nccl_f1)})
    del buf, grads, flat, p16

    # ---- F2: all-gather fused into the QKV / FFN-up GEMMs of the Llama-3-8B shape
    for name, N, K in (("qkv", 6144, 4096), ("ffn_up", 28672, 4096)):
        T = 4096
        w = (torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16)
        x = torch.randn(T, K, device=dev).to(torch.bfloat16)
        sw = ShardedWeight(w, ranks, None, keep_full=True)
        ms = _median_ms(lambda: sw.linear(x))
        fl = 2.0 * T * N * K
        nv = (world - 1) / world * N * K * 2
        roof = max(fl / (GEMM_TFLOPS * 1e9), nv / (NVLINK_GBS * 1e6))
        y = torch.empty(T, N, device=dev, dtype=torch.bfloat16)
        full = torch.empty(N, K, device=dev, dtype=torch.bfloat16)
        shard_rows = sw.shard[: min(sw.rows_per_shard, N)].contiguous()

        def nccl_f2():
            if N % world == 0 and sw.rows_per_shard * world == N:
                dist.all_gather_into_tensor(full, sw.shard)
            lib.gemm(x, full, y, False, False, False, st)

        rows.append({"path": f"F2 ag+gemm {name}", "world": world, "ms": ms, "tflops": fl / ms / 1e9,
                     "roofline_ms": roof, "fraction_of_roofline": roof / ms, "nccl_ag_then_gemm_ms": _median_ms(nccl_f2)})
        del sw
    native.check_status()

    # ---- F3: dispatch + combine of the Qwen3-30B-A3B shape (4096 tokens, top-8 of 128 experts, D = 2048)
    T, D, E, k = 4096, 2048, 128, 8
    xt = torch.randn(T, D, device=dev).to(torch.bfloat16)
    logits = torch.randn(T, E, device=dev).to(torch.bfloat16)
    weights, idx, counts = M.moe_route(logits, k, True)
    ex = FusedExpertExchange(ranks, None, T, D, E, k)
    state = {}

    def f3_dispatch():
        state["r"] = ex.dispatch(xt, idx, counts)

    nv = (world - 1) / world * T * k * D * 2
    roof = nv / (NVLINK_GBS * 1e6)
    for ctas in (128, 296, 592):
        ex.num_ctas = ctas
        ms_d = _median_ms(f3_dispatch)
        pos = state["r"][1]

        def f3_combine():
            ex.epoch += 1          # every rank publishes and waits for the same new epoch
            return ex.combine(pos, weights, T)

        ms_c = _median_ms(f3_combine)
        rows.append({"path": "F3 dispatch push", "ctas": ctas, "world": world, "ms": ms_d, "roofline_ms": roof,
                     "fraction_of_roofline": roof / ms_d, "nvlink_GBs": nv / ms_d / 1e6})
        rows.append({"path": "F3 combine pull", "ctas": ctas, "world": world, "ms": ms_c, "roofline_ms": roof,
                     "fraction_of_roofline": roof / ms_c, "nvlink_GBs": nv / ms_c / 1e6})
    # NCCL lowering of the same exchange, without its host-side count exchange: local permutation kernel +
    # equal-split all_to_all of the routed rows, and all_to_all + local weighted combine on the way back
    routed = T * k // world * world
    a2a_in = torch.empty((routed, D), dtype=torch.bfloat16, device=dev)
    a2a_out = torch.empty_like(a2a_in)

    def nccl_dispatch():
        rws, _p, _gs, _gl, _c = M.moe_dispatch(xt, idx, counts)
        dist.all_to_all_single(a2a_out, rws[:routed])

    local = M.moe_dispatch(xt, idx, counts)

    def nccl_combine():
        dist.all_to_all_single(a2a_in, a2a_out)
        M.moe_combine(local[0], local[1], weights, local[2], local[3], counts)

    rows.append({"path": "NCCL dispatch: permute kernel + all_to_all_single", "world": world, "ms": _median_ms(nccl_dispatch)})
    rows.append({"path": "NCCL combine: all_to_all_single + combine kernel", "world": world, "ms": _median_ms(nccl_combine)})
    native.check_status()
    if rank == 0:
        for r in rows:
            print(json.dumps(r), flush=True)
        out = os.environ.get("PIPER_FUSED_BENCH_JSON")
        if out:
            with open(out, "w") as f:
                json.dump(rows, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
