"""Autotune: for every shape, check each valid kernel plugin against an FP32 result, time the
ones that pass, keep the fastest in the cache file, and print TFLOPS / GB/s beside cuBLAS.

Same job as the reference's ``bench --autotune`` (src/bench.cu:304-477): every candidate must
pass the correctness gate before it is timed (src/bench.cu:413-429), timing is ``bench_ms``
(src/common.h:21-50: 5 warm-ups, 20 launches each in its own event pair, spacer kernel, mean)
on rotating buffer sets that exceed twice the L2 (src/bench.cu:381-395), cuBLAS is timed the
same way, results go to ``autotune_cache.txt`` and cached shapes are skipped on a re-run.

    python -m sm120_gemm_b200.autotune                 # the reference's ten shapes + the 16384^3 family
    python -m sm120_gemm_b200.autotune --shape 128,4096,14336 --force
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
CACHE_PATH = os.path.join(HERE, "autotune_cache.txt")

# reference src/bench.cu:164-176, then the BASELINE config-3 shape and its per-rank shards
SHAPES = [(512, 512, 14336), (1024, 1024, 14336), (1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096),
          (8192, 8192, 8192), (4096, 28672, 4096), (4096, 4096, 14336), (128, 28672, 4096), (128, 4096, 14336),
          (16384, 16384, 16384), (16384, 8192, 16384), (16384, 4096, 16384), (16384, 2048, 16384)]

NOMINAL = {"bf16_tflops": 2250.0, "hbm_gbs": 8000.0}


def time_fn(fn, stream, util, warmup=5, repeat=20, spacer_us=100000):
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(repeat)]
    for a, b in ev:
        a.record()
        fn()
        b.record()
        util.gemm_spacer(spacer_us, stream)
    torch.cuda.synchronize()
    return sum(a.elapsed_time(b) for a, b in ev) / repeat


def tune_shape(reg, M, N, K, dt="bf16", verbose=True, only=None):
    """Returns (best LoadedKernel or None, best ms, cuBLAS ms, rows of per-kernel results)."""
    import torch

    import sm120_gemm_b200 as g

    dev = torch.device("cuda", torch.cuda.current_device())
    util = g.util_lib()
    st = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator(device=dev)
    gen.manual_seed(42)
    # value range of the reference's generator: uniform[-1, 1] (src/bench.cu:36-43)
    X = (torch.rand((M, K), device=dev, generator=gen) * 2 - 1).to(torch.bfloat16)
    W = (torch.rand((N, K), device=dev, generator=gen) * 2 - 1).to(torch.bfloat16)
    # FP32 check values on a row sample (all rows when the shape is small)
    rows = torch.arange(M, device=dev) if M * N <= (1 << 24) else torch.randint(0, M, (256,), device=dev, generator=gen)
    ref = X[rows].float() @ W.float().T
    l2 = torch.cuda.get_device_properties(dev).L2_cache_size
    per_set = (M * K + N * K + M * N) * 2
    nbuf = min(64, max(1, -(-2 * l2 // per_set)))
    Xs = [X] + [X.clone() for _ in range(nbuf - 1)]
    Ws = [W] + [W.clone() for _ in range(nbuf - 1)]
    Ys = [torch.empty((M, N), dtype=torch.bfloat16, device=dev) for _ in range(nbuf)]
    idx = [0]

    def cublas():
        b = idx[0] % nbuf
        idx[0] += 1
        torch.matmul(Xs[b], Ws[b].T, out=Ys[b])

    cublas_ms = time_fn(cublas, st, util)
    valid = [k for k in reg.get_valid(M, N, K, dt=dt) if k.can_run(M, N, K) and (only is None or k.config.name() in only)]
    if verbose:
        print(f"  cuBLAS: {cublas_ms:.4f} ms  {2.0 * M * N * K / cublas_ms / 1e9:.2f} TFLOPS   ({len(valid)} valid configs, {nbuf} buffer sets)")
    ws_bytes = max([k.workspace_bytes(M, N, K) for k in valid] + [16])
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    best, best_ms, results = None, 1e30, []
    for k in valid:
        wsp = ws.data_ptr() if k.workspace_bytes(M, N, K) else 0
        Ys[0].fill_(float("nan"))
        try:
            g.dispatch(k, M, N, K, X.data_ptr(), W.data_ptr(), Ys[0].data_ptr(), wsp, st)
            torch.cuda.synchronize()
            k.check_status()
        except g.GemmError as e:
            print(f"  {k.config.name():48s} LAUNCH FAIL ({e})")
            continue
        y = Ys[0][rows].float()
        rel = ((y - ref).abs() / torch.maximum(torch.maximum(y.abs(), ref.abs()), torch.ones_like(ref))).max().item()
        if not rel < 0.02:      # the reference gates at 0.1 (src/bench.cu:427); bf16 rounding alone is 0.004
            print(f"  {k.config.name():48s} FAILED check (max rel err {rel})")
            continue

        def run(k=k, wsp=wsp):
            b = idx[0] % nbuf
            idx[0] += 1
            g.dispatch(k, M, N, K, Xs[b].data_ptr(), Ws[b].data_ptr(), Ys[b].data_ptr(), wsp, st)

        ms = time_fn(run, st, util)
        k.check_status()
        results.append((k.config.name(), ms))
        if verbose:
            print(f"  {k.config.name():48s} {ms:.4f} ms  {2.0 * M * N * K / ms / 1e9:9.2f} TFLOPS  ({100.0 * cublas_ms / ms:.1f}%)")
        if ms < best_ms:
            best, best_ms = k, ms
    return best, best_ms, cublas_ms, results


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", action="append", help="M,N,K (repeatable); default: the built-in list")
    ap.add_argument("--cache", default=CACHE_PATH)
    ap.add_argument("--force", action="store_true", help="re-tune shapes already in the cache")
    ap.add_argument("--quiet", action="store_true")
    ap.add_argument("--json", default=None, help="also write per-shape results to this file")
    ap.add_argument("--match", default=None, help="only try plugins whose name matches this regular expression")
    args = ap.parse_args()
    import torch

    sys.path.insert(0, os.path.dirname(HERE))
    import sm120_gemm_b200 as g

    assert torch.cuda.is_available(), "autotune needs a GPU"
    shapes = [tuple(int(v) for v in s.split(",")) for s in args.shape] if args.shape else SHAPES
    reg = g.KernelRegistry()
    if not reg.load_dir(g.KERNEL_DIR, dt="bf16"):
        sys.exit("no kernel plugins: build them first")
    cache = g.AutotuneCache()
    cache.load(args.cache)
    peaks = dict(NOMINAL)
    mp = os.path.join(os.path.dirname(HERE), "MEASURED_PEAKS.json")
    measured = json.load(open(mp)) if os.path.exists(mp) else None
    out = []
    last_save = time.time()
    for (M, N, K) in shapes:
        print(f"\n=== Autotune M={M} N={N} K={K} ===")
        hit = cache.lookup(M, N, K)
        if hit and not args.force:
            print(f"  cached: {hit[0].name()}  {hit[1]:.4f} ms")
            continue
        only = None
        if args.match:
            import re

            only = {k.config.name() for k in reg.kernels if re.search(args.match, k.config.name())}
        best, ms, cublas_ms, results = tune_shape(reg, M, N, K, verbose=not args.quiet, only=only)
        if best is None:
            print("  NO VALID CONFIG")
            continue
        flops, nbytes = 2.0 * M * N * K, (M * K + N * K + M * N) * 2.0
        tf, gbs = flops / ms / 1e9, nbytes / ms / 1e6
        line = (f"  BEST: {best.config.name()}  {ms:.4f} ms  {tf:.2f} TFLOPS ({100.0 * cublas_ms / ms:.1f}% of cuBLAS)  "
                f"{100 * tf / peaks['bf16_tflops']:.1f}% of 2.25 PF  {gbs:.0f} GB/s = {100 * gbs / peaks['hbm_gbs']:.1f}% of 8 TB/s")
        if measured:
            line += f"  [of measured: {100 * tf / measured['bf16_tflops']:.1f}% tensor, {100 * gbs / measured['hbm_gbs']:.1f}% HBM]"
        print(line)
        cache.store(M, N, K, best.config, ms)
        out.append({"shape": [M, N, K], "best": best.config.name(), "ms": ms, "tflops": tf, "gbs": gbs, "cublas_ms": cublas_ms,
                    "all": results})
        if time.time() - last_save > 30:       # the cache doubles as the checkpoint of a long tuning run
            cache.save(args.cache)
            last_save = time.time()
    cache.save(args.cache)
    if args.json:
        json.dump(out, open(args.json, "w"), indent=1)
    print("\nAutotune complete.")


if __name__ == "__main__":
    main()
