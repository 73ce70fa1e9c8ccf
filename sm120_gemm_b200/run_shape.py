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
    ms, nbuf = time_kernel(kern, M, N, K, args.warmup, args.repeat, rotate=not args.no_rotate, dist=args.dist)
    flops = 2.0 * M * N * K
    algo_bytes = (M * K + N * K + M * N) * 2
    print(json.dumps({"kernel": args.kernel, "shape": [M, N, K], "ms": ms, "tflops": flops / ms / 1e9,
                      "algorithmic_gbs": algo_bytes / ms / 1e6, "buffer_sets": nbuf}))


if __name__ == "__main__":
    main()
