"""Micro-benchmarks of the sm_100a kernels against measured device peaks.

``python -m piper_b200.utils.kernel_bench [--json out.json]`` times each hot
kernel on Llama-3-8B / Qwen3-30B-A3B shapes with CUDA events (warm-up, L2
flushed between iterations by writing a 256 MiB buffer) and prints achieved
TFLOP/s or GB/s.  ``torch.matmul`` (cuBLAS) is timed on the same GEMM shapes
for comparison only; it is not used by the framework.
"""
from __future__ import annotations

import argparse
import json
import math

import torch


def _time(fn, iters=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--only", default=None, help="run one family on one shape, e.g. gemm:ffn_up, attn, elementwise")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-cublas", action="store_true", help="skip the library GEMM comparison")
    ap.add_argument("--tile", type=int, default=0, choices=(0, 128, 256), help="force the GEMM CTA tile height")
    args = ap.parse_args(argv)
    global _time
    _base_time = _time
    _time = lambda fn, flush=None: _base_time(fn, iters=args.iters, warmup=args.warmup, flush=flush)  # noqa: E731
    only_family, _, only_shape = (args.only or "").partition(":")
    from piper_b200 import ops
    from piper_b200.ops import native

    dev = torch.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    st = native.status_tensor()
    rows = []
    T = 4096
    shapes = [("qkv", T, 6144, 4096), ("attn_out", T, 4096, 4096), ("ffn_up", T, 28672, 4096),
              ("ffn_down", T, 4096, 14336), ("lm_head", T, 128256, 4096), ("square8k", 8192, 8192, 8192)]
    if args.quick:
        shapes = shapes[:2]
    if only_family:
        shapes = [sh for sh in shapes if only_family == "gemm" and (not only_shape or sh[0] == only_shape)]
    for name, M, N, K in shapes:
        a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        b = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
        c = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        ms = _time(lambda: native.lib().gemm_tiled(a, b, c, False, False, False, st, args.tile), flush=flush)
        ms_ref = float("nan") if args.no_cublas else _time(lambda: torch.matmul(a, b.t(), out=c), flush=flush)
        fl = 2.0 * M * N * K
        rows.append({"kernel": f"gemm_fwd:{name}", "ms": ms, "tflops": fl / ms / 1e9, "cublas_ms": ms_ref,
                     "cublas_tflops": fl / ms_ref / 1e9})
        # dgrad and wgrad layouts
        dy = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
        dx = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
        ms = _time(lambda: native.lib().gemm_tiled(dy, b, dx, False, True, False, st, args.tile), flush=flush)
        rows.append({"kernel": f"gemm_dgrad:{name}", "ms": ms, "tflops": fl / ms / 1e9})
        dw = torch.zeros(N, K, device=dev, dtype=torch.float32)
        ms = _time(lambda: native.lib().gemm_tiled(dy, a, dw, True, True, True, st, args.tile), flush=flush)
        rows.append({"kernel": f"gemm_wgrad_f32acc:{name}", "ms": ms, "tflops": fl / ms / 1e9})
        del a, b, c, dy, dx, dw
    attn_shapes = [(1, 4096, 32, 8, 128), (1, 4096, 32, 4, 128)]
    if only_shape == "sweep":      # same token count and more, at other sequence lengths (per-CTA vs per-tile cost)
        attn_shapes = [(4, 1024, 32, 8, 128), (2, 2048, 32, 8, 128), (1, 4096, 32, 8, 128), (1, 8192, 32, 8, 128)]
    if only_family and only_family != "attn":
        attn_shapes = []
    for (B, S, Hq, Hkv, hd) in attn_shapes:
        qkv = torch.randn(B * S, (Hq + 2 * Hkv) * hd, device=dev, dtype=torch.bfloat16).requires_grad_(True)
        out = ops.attention(qkv, B, S, Hq, Hkv, hd)
        g = torch.randn_like(out)
        ms = _time(lambda: ops.attention(qkv.detach(), B, S, Hq, Hkv, hd), flush=flush)
        fl = 4.0 * B * Hq * S * S * hd / 2
        rows.append({"kernel": f"attn_fwd:B{B}S{S}Hq{Hq}kv{Hkv}", "ms": ms, "tflops": fl / ms / 1e9})

        def bwd():
            qkv.grad = None
            o = ops.attention(qkv, B, S, Hq, Hkv, hd)
            o.backward(g)
        ms_fb = _time(bwd, flush=flush)
        rows.append({"kernel": f"attn_fwd+bwd:B{B}S{S}Hq{Hq}kv{Hkv}", "ms": ms_fb, "tflops": 3.5 * fl / ms_fb / 1e9,
                     "bwd_ms": ms_fb - ms})
    if only_family and only_family != "elementwise":
        return _finish(rows, args, native)
    x = torch.randn(T, 4096, device=dev, dtype=torch.bfloat16)
    w = torch.randn(4096, device=dev, dtype=torch.bfloat16)
    ms = _time(lambda: ops.rmsnorm(x, w), flush=flush)
    rows.append({"kernel": "rmsnorm_fwd:4096x4096", "ms": ms, "gbs": 2 * x.numel() * 2 / ms / 1e6})
    res = torch.randn_like(x)
    ms_add = _time(lambda: ops.add_rmsnorm(x, res, w, 1e-6), flush=flush)
    rows.append({"kernel": "add_rmsnorm_fwd:4096x4096", "ms": ms_add, "gbs": 4 * x.numel() * 2 / ms_add / 1e6})
    xg, wg = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    gy = torch.randn_like(x)

    def norm_fb():
        xg.grad = None
        wg.grad = None
        ops.rmsnorm(xg, wg).backward(gy)
    ms_fb = _time(norm_fb, flush=flush)
    rows.append({"kernel": "rmsnorm_fwd+bwd:4096x4096", "ms": ms_fb, "bwd_ms": ms_fb - ms,
                 "bwd_gbs": 3 * x.numel() * 2 / max(ms_fb - ms, 1e-6) / 1e6})
    cos, sin = ops.rope_tables(128, T, 500000.0, device=dev)
    qkv = torch.randn(T, 48 * 128, device=dev, dtype=torch.bfloat16)
    ms = _time(lambda: ops.qk_rope(qkv, cos, sin, None, None, T, 32, 8, 128, True, 1e-6), flush=flush)
    rows.append({"kernel": "qk_rope_fwd:4096x(32+2*8)x128", "ms": ms, "gbs": 2 * qkv.numel() * 2 / ms / 1e6})
    h13 = torch.randn(T, 28672, device=dev, dtype=torch.bfloat16)
    ms = _time(lambda: ops.swiglu(h13), flush=flush)
    rows.append({"kernel": "swiglu_fwd:4096x14336", "ms": ms, "gbs": 3 * T * 14336 * 2 / ms / 1e6})
    logits = torch.randn(T, 128256, device=dev, dtype=torch.bfloat16)
    labels = torch.randint(0, 128256, (T,), device=dev)
    ms = _time(lambda: ops.cross_entropy(logits, labels), flush=flush)
    rows.append({"kernel": "ce_fwd:4096x128256", "ms": ms, "gbs": logits.numel() * 2 / ms / 1e6})
    return _finish(rows, args, native)


def _finish(rows, args, native):
    native.check_status()
    for r in rows:
        print(json.dumps(r))
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
