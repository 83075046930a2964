"""Roofline numbers of the fused compute+collective kernels (run with one rank per GPU).

``python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m piper_b200.utils.fused_bench``

``python -m piper_b200.utils.fused_bench --local f1|f2|f3 [--iters n]`` runs one of the paths in a single
process on one GPU with every "peer" buffer in that GPU's own memory (a group of one rank; for F2 two weight
shards that are both local), which is the form a profiler can capture: the kernels take the same code paths,
only the loads and stores that would cross NVLink stay on the device.

For each fused path the script times the kernels with CUDA events (warm-up, then the max over ranks of the
median) and prints the achieved figure next to its roofline: the slower of FLOPs / measured sustained bf16 GEMM
throughput and bytes that must cross NVLink / link bandwidth.  Two link figures are used side by side: the
nominal 900 GB/s per direction per GPU (``fraction_of_link_roofline``) and the 770 GB/s that a peer copy reaches
on this pool (``fraction_of_measured_copy``).  The NCCL lowering of the same step is timed alongside.

* F1: reduce-scatter of a 256 Mi-element fp32 gradient bucket + Adam + store of the new bf16 rows into every
  rank (``zero_reduce`` with its flag kernels), against ``reduce_scatter_tensor`` + Adam kernel + ``all_gather``.
* F2: all-gather of a row-sharded weight inside the GEMM that multiplies by it (``ag_gemm``).
* F3: one mixture-of-experts layer forward of the Qwen3-30B-A3B shape as the runtime runs it: gather-push
  dispatch, group table, the two grouped GEMMs with SwiGLU on the receive region, segment return; against local
  permute + ``all_to_all_single`` + the same GEMMs + ``all_to_all_single``.
"""
from __future__ import annotations

import json
import os
import statistics

import torch
import torch.distributed as dist

LINK_GBS = 900.0            # NVLink 5, per direction per GPU (nominal)
COPY_GBS = 770.0            # peer copy measured on this pool
GEMM_TFLOPS = 1397.3        # sustained cuBLAS bf16 (MEASURED_PEAKS.json)
HBM_GBS = 6549.4
# A spin kernel of about half a millisecond goes in front of every timed region: the events then bracket device
# time only, not the host's time to build tensor maps, allocate outputs and launch.
HOST_LEAD_CYCLES = 1_000_000


def _timer(multi: bool, iters: int, warmup: int = 3):
    def run(fn) -> float:
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            if multi:
                dist.barrier()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(HOST_LEAD_CYCLES)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        t = torch.tensor([statistics.median(ts)], device="cuda")
        if multi:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return run


def _f1(rank: int, world: int, ranks: list, n: int, timed, rows: list) -> None:
    from piper_b200.ops import native
    from piper_b200.parallel.symm import SymmetricBuffer

    lib, dev = native.lib(), torch.device("cuda", torch.cuda.current_device())
    st = native.status_tensor()
    shard = n // world
    gbuf = SymmetricBuffer.create(n * 4, ranks, None)
    pbuf = SymmetricBuffer.create(n * 2, ranks, None)
    fbuf = SymmetricBuffer.create(3 * world * 8, ranks, None)
    flags_local = fbuf.view(torch.int64, 3 * world)
    grads = gbuf.view(torch.float32, n)
    master = torch.zeros(shard, device=dev)
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    shard_p = torch.zeros(shard, device=dev, dtype=torch.bfloat16)
    table = torch.tensor([[0], [0], [shard], [n]], dtype=torch.int64, device=dev)
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    abort = torch.zeros(1, dtype=torch.int32, device=dev)
    use = [0]

    def f1(ctas):
        use[0] += 1
        u = use[0]
        lib.ep_signal(fbuf.peer_ptrs, 0, rank, world, u)
        lib.ep_wait(flags_local, 0, world, u, 30.0, st, 11, abort)
        lib.zero_reduce(gbuf.peer_ptrs, None, master, m, v, shard_p, pbuf.peer_ptrs, table, rank, world, False, True,
                        1e-4, 0.9, 0.95, 1e-8, 0.0, False, u, 1.0, fbuf.peer_ptrs, world, u, counter, abort, ctas)
        lib.ep_wait(flags_local, world, world, u, 30.0, st, 12, None)
        lib.zero_clear_others(grads, table, rank, world, ctas)

    # bytes crossing NVLink per direction and rank: this rank reads its rows of every peer's fp32 gradients
    # (4 B/element) and every peer stores its updated bf16 rows into this rank's parameter buffer (2 B/element)
    nvlink = (world - 1) * shard * (4 + 2)
    hbm_ms = (shard * (4 * world + 24 + 2 + 4)) / (HBM_GBS * 1e6)
    for ctas in (148, 296, 592):
        grads.normal_()
        ms = timed(lambda: f1(ctas))
        rec = {"path": "F1 reduce-scatter + Adam + parameter store", "ctas": ctas, "world": world, "elements": n,
               "ms": ms, "hbm_floor_ms": hbm_ms}
        if world > 1:
            rec.update({"nvlink_GBs_per_direction": nvlink / ms / 1e6,
                        "fraction_of_link_roofline": max(nvlink / (LINK_GBS * 1e6), hbm_ms) / ms,
                        "fraction_of_measured_copy": max(nvlink / (COPY_GBS * 1e6), hbm_ms) / ms})
        else:
            rec["fraction_of_hbm_peak"] = hbm_ms / ms
        rows.append(rec)
    native.check_status()
    if world > 1:
        flat = torch.randn(n, device=dev)
        tmp = torch.empty(shard, device=dev)
        p16 = torch.empty(n, device=dev, dtype=torch.bfloat16)

        def nccl_f1():
            dist.reduce_scatter_tensor(tmp, flat)
            lib.adam_flat(master, m, v, tmp, p16[rank * shard:(rank + 1) * shard], 1e-4, 0.9, 0.95, 1e-8, 0.0, 1, 1.0,
                          False)
            dist.all_gather_into_tensor(p16, p16[rank * shard:(rank + 1) * shard].clone())

        rows.append({"path": "NCCL reduce_scatter + adam kernel + all_gather", "world": world, "elements": n,
                     "ms": timed(nccl_f1)})


def _f3(rank: int, world: int, ranks: list, timed, rows: list, factor: float) -> None:
    from piper_b200 import ops
    from piper_b200.ops import moe as M, native
    from piper_b200.parallel.ep_fused import FREE, READY, _Pool

    lib, dev = native.lib(), torch.device("cuda", torch.cuda.current_device())
    st = native.status_tensor()
    T, D, E, k, F = 4096, 2048, 128, 8, 768
    El = E // world
    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    xt = torch.randn(T, D, generator=g).to(torch.bfloat16).to(dev)
    logits = torch.randn(T, E, generator=g).to(torch.bfloat16).to(dev)
    w13 = (torch.randn(El, 2 * F, D, generator=g) * 0.02).to(torch.bfloat16).to(dev)
    w2 = (torch.randn(El, D, F, generator=g) * 0.02).to(torch.bfloat16).to(dev)
    weights, idx, counts = M.moe_route(logits, k, True)
    pool = _Pool(ranks, None, rank, 1, T, D, E, k, factor, dev)
    G = world * El
    b_recv, b_ret = pool.buf_id("recv", 0), pool.buf_id("ret", 0)
    state: dict = {}

    def dispatch(ctas=64, free_after=False):
        g_start = torch.empty_like(counts)
        g_len = torch.empty_like(counts)
        lib.moe_group_table(counts, E, None, g_start, g_len, torch.empty(1, dtype=torch.int32, device=dev))
        scratch = torch.zeros(2 * E + 1 + world, dtype=torch.int32, device=dev)
        pos = torch.empty(T * k, dtype=torch.int32, device=dev)
        use = pool.next_use(b_recv)
        lib.ep_dispatch_push(xt, idx, counts, g_start, scratch[:E], scratch[2 * E:], scratch[E:2 * E], pos,
                             pool.recv_ptrs[0], pool.meta_ptrs[0], pool.flags_ptrs, pool.flags_local,
                             pool.off(b_recv, FREE), use - 1, pool.off(b_recv, READY), use,
                             pool.counters[b_recv:b_recv + 1], rank, world, pool.cap_src, 30.0, st, ctas)
        gs = torch.empty(G, dtype=torch.int32, device=dev)
        gl = torch.empty(G, dtype=torch.int32, device=dev)
        rc = torch.empty(G, dtype=torch.int32, device=dev)
        lib.ep_wait_table(pool.flags_local, pool.off(b_recv, READY), pool.meta[0], gs, gl, rc, world, pool.cap_src,
                          use, 30.0, st)
        state.update(pos=pos, gs=gs, gl=gl, g_start=g_start, g_len=g_len, use=use)
        if free_after:       # timed alone: nothing reads the region, hand it back at once
            lib.ep_signal(pool.flags_ptrs, pool.off(b_recv, FREE), rank, world, use)

    def experts():
        h = M.grouped_linear(pool.recv[0], w13, state["gs"], state["gl"])
        state["out"] = M.grouped_linear(ops.swiglu(h), w2, state["gs"], state["gl"])

    def ret(ctas=64):
        # the owner is done with the receive region: hand it back so that the next dispatch may overwrite it
        lib.ep_signal(pool.flags_ptrs, pool.off(b_recv, FREE), rank, world, state["use"])
        use = pool.next_use(b_ret)
        lib.ep_block_push(state["out"], state["gs"], state["gl"], pool.meta[0][G:2 * G], El, 0, pool.cap_loc,
                          pool.ret_ptrs[0], pool.flags_ptrs, pool.flags_local, pool.off(b_ret, FREE), use - 1,
                          pool.off(b_ret, READY), use, pool.counters[b_ret:b_ret + 1], pool.aborts[b_ret:b_ret + 1],
                          rank, world, 30.0, st, ctas)
        lib.ep_wait(pool.flags_local, pool.off(b_ret, READY), world, use, 30.0, st, 4, None)
        out = M.moe_combine(pool.ret[0], state["pos"], weights, state["g_start"], state["g_len"], counts)
        lib.ep_signal(pool.flags_ptrs, pool.off(b_ret, FREE), rank, world, use)
        return out

    def layer(ctas=64):
        dispatch(ctas)
        experts()
        return ret(ctas)

    nv = (world - 1) / world * T * k * D * 2                  # bytes per leg and direction
    flops = 2.0 * T * k * (2 * F * D + D * F)
    gemm_ms = flops / (GEMM_TFLOPS * 1e9)
    for ctas in (32, 64, 128):
        layer(ctas)
        ms_d = timed(lambda: dispatch(ctas, True))
        dispatch(ctas)
        ms_e = timed(experts)
        ms_r = timed(lambda: ret(ctas))
        ms_l = timed(lambda: layer(ctas))
        roof = max(gemm_ms, 2 * nv / (LINK_GBS * 1e6))
        rec = {"path": "F3 dispatch + grouped GEMMs + return + combine (one MoE layer forward)", "ctas": ctas,
               "world": world, "capacity_factor": factor, "dispatch_ms": ms_d, "experts_ms": ms_e,
               "return_combine_ms": ms_r, "layer_ms": ms_l, "gemm_floor_ms": gemm_ms, "roofline_ms": roof,
               "fraction_of_link_roofline": roof / ms_l}
        if world > 1:
            rec.update({"dispatch_GBs": nv / ms_d / 1e6, "return_GBs": nv / ms_r / 1e6,
                        "fraction_of_measured_copy": max(gemm_ms, 2 * nv / (COPY_GBS * 1e6)) / ms_l})
        rows.append(rec)
    native.check_status()
    if world > 1:
        routed = T * k // world * world
        a2a_out = torch.empty((routed, D), dtype=torch.bfloat16, device=dev)
        a2a_back = torch.empty_like(a2a_out)
        gs_l = torch.arange(El, dtype=torch.int32, device=dev) * (routed // El // 128 * 128)
        gl_l = torch.full((El,), routed // El // 128 * 128, dtype=torch.int32, device=dev)

        def nccl_layer():
            rws, p, gs, gl, _c = M.moe_dispatch(xt, idx, counts)
            dist.all_to_all_single(a2a_out, rws[:routed])
            h = M.grouped_linear(a2a_out, w13, gs_l, gl_l)
            o = M.grouped_linear(ops.swiglu(h), w2, gs_l, gl_l)
            dist.all_to_all_single(a2a_back, o)
            return M.moe_combine(rws, p, weights, gs, gl, counts)

        rows.append({"path": "NCCL lowering of the same layer (equal-split all_to_all, no count exchange)",
                     "world": world, "layer_ms": timed(nccl_layer)})


def _f2(rank: int, world: int, ranks: list, timed, rows: list) -> None:
    from piper_b200.ops import native
    from piper_b200.parallel.fused import ShardedWeight

    lib, dev = native.lib(), torch.device("cuda", torch.cuda.current_device())
    st = native.status_tensor()
    for name, N, K in (("qkv", 6144, 4096), ("ffn_up", 28672, 4096)):
        T = 4096
        w = (torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16)
        x = torch.randn(T, K, device=dev).to(torch.bfloat16)
        sw = ShardedWeight(w, ranks, None, keep_full=True)
        ms = timed(lambda: sw.linear(x))
        fl = 2.0 * T * N * K
        nv = (world - 1) / world * N * K * 2
        y = torch.empty(T, N, device=dev, dtype=torch.bfloat16)
        full = torch.empty(N, K, device=dev, dtype=torch.bfloat16)

        def nccl_f2():
            if N % world == 0 and sw.rows_per_shard * world == N:
                dist.all_gather_into_tensor(full, sw.shard)
            lib.gemm(x, full, y, False, False, False, st)

        rows.append({"path": f"F2 all-gather inside the GEMM, {name}", "world": world, "ms": ms,
                     "tflops": fl / ms / 1e9,
                     "fraction_of_link_roofline": max(fl / (GEMM_TFLOPS * 1e9), nv / (LINK_GBS * 1e6)) / ms,
                     "fraction_of_measured_copy": max(fl / (GEMM_TFLOPS * 1e9), nv / (COPY_GBS * 1e6)) / ms,
                     "nccl_ag_then_gemm_ms": timed(nccl_f2)})
        del sw
    native.check_status()


def local_main(which: str, iters: int) -> None:
    """Single-process variants (see the module docstring)."""
    from piper_b200.ops import native

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = native.lib()
    st = native.status_tensor()
    timed = _timer(False, iters, warmup=2)
    rows: list = []
    if which == "f1":
        _f1(0, 1, [0], 128 * 1024 * 1024, timed, rows)
    elif which == "f3":
        _f3(0, 1, [0], timed, rows, 1.0)
    else:
        T, N, K = 4096, 6144, 4096
        w = (torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16)
        x = torch.randn(T, K, device=dev).to(torch.bfloat16)
        y = torch.empty(T, N, dtype=torch.bfloat16, device=dev)
        fl = 2.0 * T * N * K
        ms = timed(lambda: lib.gemm(x, w, y, False, False, False, st))
        rows.append({"path": "plain GEMM of the same shape", "ms": ms, "tflops": fl / ms / 1e9})
        for shards, gathered in ((2, False), (1, True), (2, True)):
            nrows = N // shards
            parts = [w[p * nrows:(p + 1) * nrows].contiguous() for p in range(shards)]
            full = torch.zeros(N, K, dtype=torch.bfloat16, device=dev) if gathered else None
            scratch = torch.zeros((N + 255) // 256 + 2, dtype=torch.int32, device=dev) if gathered else None
            ptrs = [p.data_ptr() for p in parts]
            ms = timed(lambda: lib.ag_gemm(x, ptrs, 0, full, scratch, y, N, nrows, st))
            rec = {"path": f"F2 local: {shards} local shard(s), {'gathered' if gathered else 'direct'} mode", "ms": ms,
                   "tflops": fl / ms / 1e9, "fraction_of_gemm_peak": fl / ms / 1e9 / GEMM_TFLOPS}
            if gathered:
                rec["max_abs_err_vs_full"] = float((full.float() - w.float()).abs().max())
            rows.append(rec)
    torch.cuda.synchronize()
    native.check_status()
    for r in rows:
        print(json.dumps(r), flush=True)


def main():
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--local", choices=("f1", "f2", "f3"), default=None)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--only", default="f1,f2,f3")
    ap.add_argument("--capacity-factor", type=float, default=1.25)
    args = ap.parse_args()
    if args.local:
        return local_main(args.local, args.iters)
    from piper_b200.runtime.layout import init_distributed

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world, _ = init_distributed("cuda")
    ranks = list(range(world))
    timed = _timer(True, args.iters)
    rows: list = []
    only = set(args.only.split(","))
    if "f1" in only:
        _f1(rank, world, ranks, 256 * 1024 * 1024, timed, rows)
    if "f2" in only:
        _f2(rank, world, ranks, timed, rows)
    if "f3" in only:
        _f3(rank, world, ranks, timed, rows, args.capacity_factor)
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
