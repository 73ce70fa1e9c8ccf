#!/usr/bin/env python
"""Benchmark of the hot path: BF16 Y = X * W^T, M = N = K = 16384 (BASELINE config 3), FP32
accumulate, on N GPUs of one node.  At N > 1 the weight rows are sharded (N/g per rank) and the
bf16 column blocks of Y are all-gathered, by default inside the GEMM epilogue (stores over NVLink
into every rank's Y) or with --gather nccl by one NCCL all-gather; total work is fixed (strong scaling).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line on rank 0.  `value` is device-timed TFLOPS with inputs resident in HBM;
`e2e` is the same metric through the plugin C ABI with HOST buffers (pinned host -> device
copies of X and W and the device -> host copy of Y inside the timed region).  The reference
arm times the CPU restatement of the reference's FP32 check loop (it has no CPU code of its
own) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M = N = K = 16384
WORKLOAD = "bf16 gemm Y=X*W^T M=N=K=16384, X,W~N(0,1) seed 2, fp32 accumulate, bf16 out (BASELINE config 3)"
# the second tile family always joins the untimed selection trial: on several GPUs the tile whose GEMM alone is
# fastest can lose once the gather rides in its epilogue
ALTERNATE_FAMILY = ["bf16_bm512_bn256_bk64_s4_cg2_sk1_ab0_e1", "bf16_bm512_bn256_bk64_s3_cg2_sk1_ab0_e1", "bf16_bm256_bn256_bk64_s6_cg2_sk1_ab0_e1"]
CHECK_ROWS = 32
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the GEMM kernel at this workload,
# from the ncu capture summarised under profiles/ (None until captured)
NCU_TRAFFIC_BYTES = {   # profiles/kernel_families_limited_metrics.md, the 16384^3 rows (read + written, with wave pacing)
    "bf16_bm512_bn256_bk64_s3_cg2_sk1_ab0_e1": 6492843520 + 527142400,
    "bf16_bm512_bn256_bk64_s4_cg2_sk1_ab0_e1": 6492905472 + 528000000,
}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                "hbm_gbs": d["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.stop_flag, self.samples, self.reasons, self.max_mhz = index, False, [], set(), None

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap", nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                     nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                     nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                     nv.nvmlClocksThrottleReasonHwPowerBrakeSlowdown: "hw_power_brake_slowdown"}
            while not self.stop_flag:
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
                time.sleep(0.004)
        except Exception as e:  # NVML missing: report it instead of inventing numbers
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def result(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


def host_threads() -> int:
    """Host hardware threads this process may use."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def load_oracle(threads: int):
    """The CPU oracle with an explicit OpenMP thread count: a launcher (torch.distributed.run) exports
    OMP_NUM_THREADS=1 to its workers, which would otherwise make the host arm a single-core run."""
    os.environ["OMP_NUM_THREADS"] = str(threads)
    from oracle import oracle as o

    o.set_threads(threads)
    return o


def cpu_baseline(seconds_target: float = 12.0):
    """Times the CPU oracle (restatement of the reference's FP32 loop, src/bench.cu:77-84) on a
    row slab of the same 16384^3 workload, all host threads."""
    import numpy as np

    o = load_oracle(host_threads())

    rng = np.random.default_rng(2)
    W = o.f32_to_bf16_bits(rng.standard_normal((N, K), dtype=np.float32))
    rows = 32
    X = o.f32_to_bf16_bits(rng.standard_normal((rows, K), dtype=np.float32))
    t0 = time.perf_counter(); o.gemm_bf16(X, W); t1 = time.perf_counter() - t0   # includes the bf16->fp32 conversion of W
    t0 = time.perf_counter(); o.gemm_bf16(X, W); t1 = min(t1, time.perf_counter() - t0)
    # grow the slab so the timed pass lasts about seconds_target
    rows2 = int(min(4096, max(64, rows * seconds_target / max(t1, 1e-3) * 0.5)))
    X = o.f32_to_bf16_bits(rng.standard_normal((rows2, K), dtype=np.float32))
    t0 = time.perf_counter(); o.gemm_bf16(X, W); dt = time.perf_counter() - t0
    tflops = 2.0 * rows2 * N * K / dt / 1e12
    return {"value": tflops, "unit": "TFLOPS", "cores": o.num_threads(), "kind": "port",
            "sample": f"{rows2} of {M} rows of Y (all {N} columns, K={K}), one timed pass of {dt:.1f} s after a warm pass"}, W


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np

    o = load_oracle(host_threads())
    base, W = cpu_baseline(4.0)
    rng = np.random.default_rng(2)
    rows = 256
    X = o.f32_to_bf16_bits(rng.standard_normal((rows, K), dtype=np.float32))
    for _ in range(min(args.warmup, 1)):
        o.gemm_bf16(X, W)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        o.gemm_bf16(X, W)
    dt = time.perf_counter() - t0
    tflops = 2.0 * rows * N * K * args.steps / dt / 1e12
    sample = f"each step = {rows} of {M} rows of Y on the host cores (CPU port of the reference's FP32 loop; the reference has no CPU implementation)"
    print(json.dumps({
        "impl": "reference", "metric": "gemm_tflops", "value": tflops, "unit": "TFLOPS", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": {"workload": WORKLOAD, "l2": "inputs larger than L2"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOPS", "cores": o.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def make_inputs(torch, dev, rank, world):
    """X (full) and this rank's rows of W, N(0,1) bf16 from fixed seeds: every rank draws the same two streams
    and keeps its own weight rows, so W never crosses GPUs.  `w_rows(r0, r1)` redraws any rows of the full W
    (for the result check)."""
    plan_rows = N // world
    gen = torch.Generator(device=dev); gen.manual_seed(2)
    X = torch.randn((M, K), device=dev, generator=gen).to(torch.bfloat16)
    chunk = 2048

    def w_blocks():
        g2 = torch.Generator(device=dev); g2.manual_seed(1002)
        for r0 in range(0, N, chunk):
            yield r0, torch.randn((chunk, K), device=dev, generator=g2).to(torch.bfloat16)

    W = torch.empty((plan_rows, K), dtype=torch.bfloat16, device=dev)
    for r0, blk in w_blocks():
        lo, hi = max(r0, rank * plan_rows), min(r0 + chunk, (rank + 1) * plan_rows)
        if lo < hi:
            W[lo - rank * plan_rows:hi - rank * plan_rows] = blk[lo - r0:hi - r0]
    return X, W, w_blocks


def check_result(torch, dist, Y, X, w_blocks, rank, world):
    """Outside the timed region: CHECK_ROWS sampled rows of this rank's full Y (its own and every other rank's
    column blocks) against the CPU oracle's FP32 rows, under the dense tolerance.  The verdict is all-reduced so
    every rank stops together.  (The oracle is used as the checker only; nothing timed touches it.)"""
    import numpy as np

    o = load_oracle(max(1, host_threads() // world))
    rows = np.unique(np.concatenate([[0, M - 1], np.random.default_rng(100 + rank).integers(0, M, CHECK_ROWS - 2)]))
    sel = torch.from_numpy(rows).to(Y.device)
    Xs = X[sel].view(torch.int16).cpu().numpy().view(np.uint16)
    Wh = np.empty((N, K), dtype=np.uint16)
    for r0, blk in w_blocks():
        Wh[r0:r0 + blk.shape[0]] = blk.view(torch.int16).cpu().numpy().view(np.uint16)
    ref = o.gemm_bf16(Xs, Wh)
    yb = Y[sel].view(torch.int16).cpu().numpy().view(np.uint16)
    r = o.check_dense(yb, ref, K, float(np.abs(o.bf16_bits_to_f32(Xs)).max()), float(np.abs(o.bf16_bits_to_f32(Wh)).max()))
    # bar (ii) at K = 16384 with unit-variance inputs sits at 99.89 % for any FP32-accumulating tensor-core GEMM
    # (cuBLAS included; tests/test_gpu_parity.py measures both against a double-precision sum), so the gate here is 99.8 %
    ok = bool(not np.isnan(o.bf16_bits_to_f32(yb)).any() and r["max_abs_err"] <= r["bound"] and r["frac_within_bf16_rounding"] >= 0.998)
    frac = r["frac_within_bf16_rounding"]
    if world > 1:
        t = torch.tensor([1.0 if ok else 0.0, frac], device=Y.device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        ok, frac = bool(t[0].item() > 0.5), float(t[1].item())
    return {"rows": int(rows.size) * world, "columns": N, "frac_within_bf16_rounding": frac, "max_abs_err": r["max_abs_err"], "bound": r["bound"],
            "against": "CPU oracle (FP32 loop of the reference's check kernel), every rank, before the timed region", "ok": ok}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kernel", default=None, help="plugin configuration name (default: autotune cache / heuristic pick, then a short trial)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-check", action="store_true", help="skip the oracle check of sampled rows before the timed region")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="N>1: fused = the epilogue stores into every rank's Y over NVLink (multimem stores to the NVSwitch multicast "
                         "address when the node offers one, else one TMA store per peer); nccl = all-gather + interleave kernel")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    import torch.distributed as dist

    import sm120_gemm_b200 as g
    from sm120_gemm_b200.host_gemm import HostGemm, ShardedHostGemm
    from sm120_gemm_b200.shard import FusedNShardedGemm, NShardedGemm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        sys.exit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    if not torch.cuda.is_available():
        sys.exit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # the fused gather stores to the NVSwitch multicast mapping of Y when symmetric memory offers one
        # (TORCH_SYMM_MEM_DISABLE_MULTICAST=1 or SM100_GEMM_MULTICAST=0 selects one TMA store per peer instead)
        dist.init_process_group("nccl", device_id=dev)

    reg = g.KernelRegistry()
    if not reg.load_dir(g.KERNEL_DIR, dt="bf16"):
        sys.exit("no kernel plugins found: run python -c 'import __graft_entry__ as e; e.build()'")
    cache = g.AutotuneCache()
    cache.load(os.path.join(ROOT, "sm120_gemm_b200", "autotune_cache.txt"))
    plan_rows = N // world
    fused_wanted = world > 1 and args.gather == "fused"
    # candidates: the dispatcher's pick for the per-rank shape (autotune cache entry, else the cost model) and one
    # plugin of each large-tile family; the fastest over a few untimed launches is used (the reference also tunes
    # before it times, src/bench.cu:304-477)
    if args.kernel:
        names = [args.kernel]
    else:
        pick = reg.select(cache, M, plan_rows, K, "bf16")
        names = ([pick.config.name()] if pick else []) + ALTERNATE_FAMILY
    cands = []
    for n in dict.fromkeys(names):
        k = reg.find(n)
        if k is None:
            sys.exit(f"plugin {n} is not built")
        if fused_wanted and not args.kernel and (k.config.epi != 1 or k.config.split_k != 1):
            continue        # the fused gather needs a TMA-store epilogue
        cands.append(k)

    X, W, w_blocks = make_inputs(torch, dev, rank, world)
    Y = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    fused_trial = fused_wanted and all(k.config.epi == 1 and k.config.split_k == 1 for k in cands)
    # on several GPUs a 256 x 256 plugin is tried both ways: sending from the epilogue, and forwarding tiles from L2
    variants = [(k, False) for k in cands]
    if fused_trial:
        variants += [(k, True) for k in cands if k.config.bm == 256 and k.config.bn == 256 and k.config.cg == 2]
    kern, forward = variants[0]
    if len(variants) > 1:
        # Untimed selection trial.  On several GPUs the candidates are tried as the whole fused step (GEMM with
        # the gather in its epilogue, then the barrier).  Each candidate runs what the timed region will run -- a short
        # idle gap, the warm-up steps, then up to 40 steps -- because under the 1 kW power cap the ranking over a few
        # launches at boost clocks differs from the ranking over a long run (measured: the four-stage 512 x 256 plugin wins
        # the first, the three-stage one the second).
        trial = []
        st = torch.cuda.current_stream().cuda_stream
        for k, fw in variants:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if fused_trial:
                f = FusedNShardedGemm(k, M, N, K, rank, world, double_buffer=False, forward=fw)
                run_once = lambda: f.run(X, W)
            else:
                ya = torch.empty((M, plan_rows), dtype=torch.bfloat16, device=dev)
                run_once = lambda: g.dispatch(k, M, plan_rows, K, X.data_ptr(), W.data_ptr(), ya.data_ptr(), 0, st)
            run_once()
            torch.cuda.synchronize()
            time.sleep(0.3)
            for _ in range(max(1, args.warmup)):
                run_once()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(max(3, min(args.steps, 40))):
                run_once()
            e1.record()
            torch.cuda.synchronize()
            trial.append(e0.elapsed_time(e1))
            if fused_trial:
                del f
            else:
                del ya
        t = torch.tensor(trial, device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)      # every rank must make the same choice
        kern, forward = variants[int(torch.argmin(t).item())]
        if rank == 0:       # the trial's table, for the record (stderr: stdout carries the one JSON line)
            n_timed = max(3, min(args.steps, 40))
            for (k, fw), ms in zip(variants, t.tolist()):
                sys.stderr.write(f"trial: {k.config.name()}{' forwarded from L2' if fw else ''}: {ms / n_timed:.4f} ms per step\n")
    fused = fused_wanted and kern.config.epi == 1 and kern.config.split_k == 1
    if fused:
        fop = FusedNShardedGemm(kern, M, N, K, rank, world, forward=forward)      # two symmetric result buffers used in turn

        class _Op:
            def run(self, X, W, Y):
                return fop.run(X, W)
        op = _Op()
        result = lambda: fop.Y
    else:
        op = NShardedGemm(kern, M, N, K, rank, world)
        result = lambda: Y

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    launches_per_step = 0
    for _ in range(args.warmup):
        launches_per_step = op.run(X, W, Y)
    if kern.config.split_k > 1:
        launches_per_step += 1
    barrier()
    kern.check_status()

    # never time a result that failed the check (the reference's rule, src/bench.cu:413-429)
    check = None
    if not args.no_check:
        check = check_result(torch, dist, result(), X, w_blocks, rank, world)
        if not check["ok"]:
            sys.exit(f"rank {rank}: result check failed before timing: {check}")

    sampler = ClockSampler(local_rank); sampler.start()
    time.sleep(0.02)
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        starts[i].record()
        op.run(X, W, Y)
        ends[i].record()
    e1.record()
    barrier()
    sampler.stop_flag = True; sampler.join(timeout=2)
    total_ms = e0.elapsed_time(e1)
    per_step = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    kern.check_status()
    if world > 1:
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())

    # ---- end to end: host buffers in, host buffer out, copies inside the timed region, plugin C ABI in the middle.
    # One GPU: X and W up, Y down, overlapped by row chunks on three streams.  N GPUs: every rank brings 1/N of the
    # rows of X and its weight rows up, the X slices are exchanged by one NCCL all-gather, and every rank takes its
    # 1/N of the rows of Y down: the host sends X and W once and receives one full Y, whatever N is.
    slice_rows = M // world
    # the host holds X once: at N > 1 each rank has the pinned rows of its own slice (the fused path exchanges them over NVLink)
    x_rows = slice_rows if (world > 1 and fused) else M
    x_row0 = rank * slice_rows if (world > 1 and fused) else 0
    Xh = torch.empty((x_rows, K), dtype=torch.bfloat16).pin_memory(); Xh.copy_(X[x_row0:x_row0 + x_rows])
    Wh = torch.empty((plan_rows, K), dtype=torch.bfloat16).pin_memory(); Wh.copy_(W)
    Yh = torch.empty((slice_rows, N), dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(2, min(args.steps, 5))
    if world == 1:
        hg = HostGemm(kern, M, N, K, chunk_rows=2048, device_X=X, device_W=W, device_Y=Y)
        e2e_step = lambda: hg.run(Xh, Wh, Yh)
        h2d, d2h = (M * K + N * K) * 2, M * N * 2
    elif fused:
        shg = ShardedHostGemm(fop, chunk_rows=2048, device_X=X, device_W=W)
        e2e_step = lambda: shg.run(Xh, Wh, Yh)
        h2d, d2h = shg.h2d_bytes, shg.d2h_bytes
    else:
        r0 = rank * slice_rows

        def e2e_step():
            X.copy_(Xh, non_blocking=True)
            W.copy_(Wh, non_blocking=True)
            op.run(X, W, Y)
            Yh.copy_(Y[r0:r0 + slice_rows], non_blocking=True)
        h2d, d2h = (M * K + plan_rows * K) * 2, slice_rows * N * 2

    e2e_step(); barrier()
    # the host-buffer path must reproduce the device-resident result bit for bit (sampled rows of this rank's slice)
    Yres = result()
    rows = torch.randint(0, slice_rows, (64,))
    same = bool(torch.equal(Yh[rows].cuda(), Yres[(rows + rank * slice_rows).cuda()]))
    if world > 1:
        t = torch.tensor([1.0 if same else 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        same = bool(t.item() > 0.5)
    assert same, "host-buffer path differs from the resident path"
    f0 = torch.cuda.Event(enable_timing=True); f1 = torch.cuda.Event(enable_timing=True)
    barrier()
    f0.record()
    for _ in range(e2e_steps):
        e2e_step()
    f1.record()
    barrier()
    e2e_ms = f0.elapsed_time(f1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())

    if rank == 0:
        flops = 2.0 * M * N * K
        peaks = load_peaks()
        value = flops * args.steps / (total_ms * 1e-3) / 1e12
        # roofline of the dominant kernel (the tcgen05 GEMM): per-launch time = the step's event time (one kernel per
        # step and rank; at N>1 the kernel also sends its tiles to the other ranks and the step ends with a barrier,
        # so the per-rank figure there is a lower bound on what the tensor pipe did)
        launch_ms = sum(per_step) / len(per_step)
        kflops = flops / world
        achieved = kflops / (launch_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": achieved / peaks["bf16_tflops"], "traffic": NCU_TRAFFIC_BYTES.get(kern.config.name()) if world == 1 else None,
                    "peak_source": f"{peaks['source']} (cuBLAS bf16 burst; sustained {peaks['bf16_tflops_sustained']})",
                    "frac_of_sustained": achieved / peaks["bf16_tflops_sustained"] if peaks["bf16_tflops_sustained"] else None,
                    "kernel": f"umma_gemm_kernel<{kern.config.name()}>", "flops_per_launch": kflops, "avg_launch_ms": launch_ms}
        clocks = sampler.result()
        ms_per_step = total_ms / args.steps
        out = {
            "metric": "gemm_tflops", "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "kernel": kern.config.name(), "l2": "inputs larger than L2 (X, W, Y = 1.5 GiB vs 126 MB L2)",
                       "parallelism": "single GPU" if world == 1 else (
                           f"N-sharded x{world}: {plan_rows} weight rows per rank, all-gather fused into the epilogue "
                           + (("(multimem stores to the NVSwitch multicast address of Y" + (", tiles forwarded from L2 by sender warps)" if (forward or kern.config.bm == 512) else ", sent from the epilogue)"))
                              if fop.multicast else "(TMA stores to every rank's Y over NVLink)") + " + barrier"
                           if fused else f"N-sharded x{world}: {plan_rows} weight rows per rank + NCCL all-gather + interleave")},
            "roofline": roofline,
            "e2e": {"value": flops * e2e_steps / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOPS", "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
                    "h2d_bytes_per_rank": h2d, "d2h_bytes_per_rank": d2h, "steps": e2e_steps,
                    "note": "pinned host X and W in (each rank its 1/N of the rows of X and its weight rows; X slices exchanged by one NCCL all-gather), one full Y back to the host (each rank its 1/N of the rows), copies overlapped with the kernels"},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            # step time in SM clock cycles (ms x median SM MHz under load x 1000): compares runs that ran at different clocks
            "sm_clock_cycles_per_step": ms_per_step * clocks["sm_mhz"] * 1e3 if clocks.get("sm_mhz") else None,
        }
        if check is not None:
            out["check"] = check
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"], _ = cpu_baseline()
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
