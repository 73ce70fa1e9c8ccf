"""Runs one kernel plugin on one shape on cuda:0 and prints a JSON line with its device time
(reference timing protocol: warm-ups, then launches each bracketed by its own event pair with
an idle spacer kernel between them, mean of the per-launch times; L2 is flushed by rotating
over enough buffer sets to exceed twice the L2 size -- reference src/common.h:21-50,
src/bench.cu:381-395).  Meant for profiling a single kernel under ncu and for quick sweeps.

    python -m sm120_gemm_b200.run_shape --kernel bf16_bm256_bn256_bk64_s6_cg2_sk1_ab0_e1 --shape 8192,8192,8192
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def time_lowp_kernel(kern, M, N, K, warmup=5, repeat=20, spacer_us=100, rotate=True, seed=0):
    """Same protocol for the fp8 / mxfp8 / w4a4 / w4a16 plugins (gemm_run_ex), random operand bits."""
    import torch

    import sm120_gemm_b200 as g

    dev = torch.device("cuda", torch.cuda.current_device())
    util = g.util_lib()
    dt = kern.config.dt
    gen = torch.Generator(device=dev); gen.manual_seed(seed)
    wbits = {"fp8": 8, "mxfp8": 8, "w4a4": 4, "w4a16": 4}[dt]
    xbits = 16 if dt == "w4a16" else wbits
    l2 = torch.cuda.get_device_properties(dev).L2_cache_size
    per_set = M * K * xbits // 8 + N * K * wbits // 8 + M * N * 2
    nbuf = min(64, max(1, -(-2 * l2 // per_set))) if rotate else 1

    def rand_bytes(rows, nbytes):
        # bytes below 0x78 in both nibbles: finite e4m3 / e2m1 codes of either sign are all fine as data
        return torch.randint(0, 0x77, (rows, nbytes), dtype=torch.uint8, device=dev, generator=gen)

    sets = []
    for _ in range(nbuf):
        W = rand_bytes(N, K * wbits // 8)
        X = torch.randn((M, K), device=dev, generator=gen).to(torch.bfloat16) if dt == "w4a16" else rand_bytes(M, K * xbits // 8)
        sets.append((X, W, torch.empty((M, N), dtype=torch.bfloat16, device=dev)))
    a = g.GemmArgs()
    a.M, a.N, a.K, a.group_size = M, N, K, 128
    a.x_scale_f = a.w_scale_f = 1.0 / 16
    keep = []
    if dt in ("mxfp8", "w4a4"):
        sx = torch.full((util.gemm_mx_tiled_scale_bytes(M, K),), 124, dtype=torch.uint8, device=dev)
        sw = torch.full((util.gemm_mx_tiled_scale_bytes(N, K),), 124, dtype=torch.uint8, device=dev)
        a.x_scale, a.w_scale = sx.data_ptr(), sw.data_ptr()
        keep += [sx, sw]
    if dt == "w4a16":
        sw = (torch.rand((N, K // 128), device=dev, generator=gen) * 0.2 + 0.05).to(torch.bfloat16)
        a.w_scale = sw.data_ptr()
        keep.append(sw)
    wsb = kern.workspace_bytes(M, N, K)
    ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)
    a.workspace, a.workspace_bytes = (ws.data_ptr() if wsb else None), wsb
    a.stream = torch.cuda.current_stream().cuda_stream
    idx = [0]

    def launch():
        X, W, Y = sets[idx[0] % nbuf]
        idx[0] += 1
        a.X, a.W, a.Y = X.data_ptr(), W.data_ptr(), Y.data_ptr()
        g.dispatch_ex(kern, a)

    for _ in range(warmup):
        launch()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(repeat)]
    for e0, e1 in ev:
        e0.record()
        launch()
        e1.record()
        util.gemm_spacer(spacer_us, a.stream)
    torch.cuda.synchronize()
    kern.check_status()
    scale_bytes = {"fp8": 8, "mxfp8": (M + N) * K // 32, "w4a4": (M + N) * K // 32, "w4a16": N * K // 128 * 2}[dt]
    return sum(e0.elapsed_time(e1) for e0, e1 in ev) / repeat, nbuf, per_set + scale_bytes


def time_kernel(kern, M, N, K, warmup=5, repeat=20, spacer_us=100, rotate=True, dist="normal", seed=0):
    import torch

    import sm120_gemm_b200 as g

    dev = torch.device("cuda", torch.cuda.current_device())
    util = g.util_lib()
    l2 = torch.cuda.get_device_properties(dev).L2_cache_size
    per_set = (M * K + N * K + M * N) * 2
    nbuf = max(1, -(-2 * l2 // per_set)) if rotate else 1
    nbuf = min(nbuf, 64)
    gen = torch.Generator(device=dev); gen.manual_seed(seed)
    scale = 1.0 / (K ** 0.5) if dist == "decode" else 1.0
    X0 = torch.randn((M, K), device=dev, generator=gen).to(torch.bfloat16)
    W0 = (torch.randn((N, K), device=dev, generator=gen) * scale).to(torch.bfloat16)
    Xs = [X0] + [X0.clone() for _ in range(nbuf - 1)]
    Ws = [W0] + [W0.clone() for _ in range(nbuf - 1)]
    Ys = [torch.empty((M, N), dtype=torch.bfloat16, device=dev) for _ in range(nbuf)]
    wsb = kern.workspace_bytes(M, N, K)
    ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    idx = [0]

    def launch():
        b = idx[0] % nbuf
        idx[0] += 1
        g.dispatch(kern, M, N, K, Xs[b].data_ptr(), Ws[b].data_ptr(), Ys[b].data_ptr(), ws.data_ptr() if wsb else 0, st)

    for _ in range(warmup):
        launch()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(repeat)]
    for a, b in ev:
        a.record()
        launch()
        b.record()
        util.gemm_spacer(spacer_us, st)
    torch.cuda.synchronize()
    kern.check_status()
    ms = sum(a.elapsed_time(b) for a, b in ev) / repeat
    return ms, nbuf


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True)
    ap.add_argument("--shape", required=True, help="M,N,K")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeat", type=int, default=20)
    ap.add_argument("--dist", default="normal", choices=["normal", "decode"])
    ap.add_argument("--no-rotate", action="store_true", help="one buffer set (small ncu captures)")
    args = ap.parse_args()
    import torch

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import sm120_gemm_b200 as g

    assert torch.cuda.is_available(), "needs a CUDA device"
    M, N, K = (int(v) for v in args.shape.split(","))
    kern = g.load_plugin(os.path.join(g.KERNEL_DIR, f"libgemm_{args.kernel}.so"))
    if not kern.can_run(M, N, K):
        sys.exit(f"{args.kernel} cannot run {M}x{N}x{K}")
    if kern.config.dt == "bf16":
        ms, nbuf = time_kernel(kern, M, N, K, args.warmup, args.repeat, rotate=not args.no_rotate, dist=args.dist)
        algo_bytes = (M * K + N * K + M * N) * 2
    else:
        ms, nbuf, algo_bytes = time_lowp_kernel(kern, M, N, K, args.warmup, args.repeat, rotate=not args.no_rotate)
    flops = 2.0 * M * N * K
    print(json.dumps({"kernel": args.kernel, "shape": [M, N, K], "ms": ms, "tflops": flops / ms / 1e9,
                      "algorithmic_gbs": algo_bytes / ms / 1e6, "buffer_sets": nbuf}))


if __name__ == "__main__":
    main()
