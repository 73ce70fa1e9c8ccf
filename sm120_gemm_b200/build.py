"""Builds the kernel plugins (one shared library per configuration) with nvcc for sm_100a.

Same job as the reference's CMake loop (CMakeLists.txt:13-60: run the generator, configure
kernel_entry.cu.in once per configuration, add_library(SHARED) each), done with direct nvcc
calls so no CMake is needed: the configuration reaches csrc/kernel_entry.cu as -D macros.

    python -m sm120_gemm_b200.build            # all configurations, in parallel
    python -m sm120_gemm_b200.build --only bf16_bm256_bn256_bk64_s6_cg2_sk1_ab0_e1
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

from .gen_configs import GemmConfig, generate_configs

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
KERNEL_DIR = os.path.join(HERE, "kernels")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
# register / spill report of every kernel is always on, as in the reference's build (CMakeLists.txt:33:
# --ptxas-options=-v,-warn-spills); build_one() fails a plugin whose kernels spill
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
              "-Xcompiler", "-fPIC,-fno-gnu-unique", "-ccbin", "/usr/bin/g++", "-diag-suppress", "177", "-Xptxas", "-v,-warn-spills"]
# -fno-gnu-unique: the function-local statics of the launch templates (per-device "attribute set" flags, cached
# occupancy) would otherwise be STB_GNU_UNIQUE symbols, which the dynamic linker shares between ALL loaded
# plugins that instantiate the same template, RTLD_LOCAL or not; two builds of one configuration in a process
# (a checked build beside the normal one) would then see each other's flags
# Test-only plugin builds (kernels/testing/): the same entry file with one extra macro each.
#   bounds:   -DGEMM_DEBUG_BOUNDS   every computed TMA coordinate / store address is checked before use
#   expiry:   a short wait limit and a producer that can be told to withhold a stage, so that a bounded wait
#             runs out and the kernel reports GEMM_ERR_DEVICE_TIMEOUT (nothing is in flight at that point)
TESTING_DIR = os.path.join(KERNEL_DIR, "testing")
TESTING_BUILDS = {
    "bounds": (["-DGEMM_DEBUG_BOUNDS"], ["bf16_bm128_bn128_bk64_s6_cg1_sk1_ab0_e1", "bf16_bm256_bn256_bk64_s6_cg2_sk1_ab0_e1",
                                         "bf16_bm512_bn256_bk64_s4_cg2_sk1_ab0_e1", "bf16_bm128_bn128_bk64_s7_cg1_sk4_ab0_e0",
                                         "bf16_bm128_bn256_bk64_s4_cg1_sk0_ab0_e0", "bf16_bm128_bn128_bk64_s7_cg1_sk1_ab0_e2"]),
    "expiry": (["-DSM100_WAIT_LIMIT_CYCLES=2000000ll", "-DSM100_TEST_WITHHOLD_STAGE"], ["bf16_bm128_bn128_bk64_s6_cg1_sk1_ab0_e1"]),
}


def entry_source(cfg: GemmConfig) -> str:
    return os.path.join(CSRC, "kernel_entry.cu")


def plugin_path(cfg: GemmConfig) -> str:
    return os.path.join(KERNEL_DIR, f"libgemm_{cfg.name()}.so")


def _deps_mtime() -> float:
    newest = 0.0
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for f in os.listdir(root):
            if f.endswith((".cu", ".cuh", ".h", ".cpp")):
                newest = max(newest, os.path.getmtime(os.path.join(root, f)))
    return newest


def build_one(cfg: GemmConfig, force: bool = False, verbose: bool = False, out: str | None = None, extra=()) -> str:
    out = out or plugin_path(cfg)
    if not force and os.path.exists(out) and os.path.getmtime(out) >= _deps_mtime():
        return out
    os.makedirs(os.path.dirname(out), exist_ok=True)
    cmd = [NVCC, *NVCC_FLAGS, *cfg.defines(), *extra, "-o", out, entry_source(cfg)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {cfg.name()}:\n{r.stdout}\n{r.stderr}")
    spills = [ln for ln in r.stderr.splitlines() if "spill" in ln and "0 bytes spill stores, 0 bytes spill loads" not in ln]
    if spills:
        os.remove(out)
        raise RuntimeError(f"{cfg.name()}: a kernel spills registers:\n" + "\n".join(spills))
    if verbose:
        sys.stderr.write(r.stderr)
    return out


def build_testing(force: bool = False) -> list[str]:
    """The test-only plugin variants, kernels/testing/<kind>/libgemm_<config>.so."""
    outs = []
    for kind, (extra, names) in TESTING_BUILDS.items():
        for n in names:
            cfg = GemmConfig.parse(n)
            outs.append(build_one(cfg, force, out=os.path.join(TESTING_DIR, kind, f"libgemm_{n}.so"), extra=extra))
    return outs


UTIL_LIB = os.path.join(KERNEL_DIR, "libsm100gemm_util.so")


def build_util(force: bool = False) -> str:
    """The utility library: quantisation kernels, weight packers and file format, block interleave for the
    N-sharded run, MX scale tiling, timing spacer."""
    srcs = [os.path.join(CSRC, f) for f in ("gemm_util.cu", "quant_kernels.cu", "weight_file.cpp")]
    if not force and os.path.exists(UTIL_LIB) and os.path.getmtime(UTIL_LIB) >= _deps_mtime():
        return UTIL_LIB
    os.makedirs(KERNEL_DIR, exist_ok=True)
    r = subprocess.run([NVCC, *NVCC_FLAGS, "-o", UTIL_LIB, *srcs], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for the utility library:\n{r.stdout}\n{r.stderr}")
    return UTIL_LIB


BENCH_BIN = os.path.join(KERNEL_DIR, "bench")


def build_bench(force: bool = False) -> str:
    """The C++ harness (csrc/bench.cu): autotune / quick / debug modes, cuBLAS beside."""
    src = os.path.join(CSRC, "bench.cu")
    if not force and os.path.exists(BENCH_BIN) and os.path.getmtime(BENCH_BIN) >= _deps_mtime():
        return BENCH_BIN
    os.makedirs(KERNEL_DIR, exist_ok=True)
    build_util()          # the harness makes its low-precision operands with the library's quantisation kernels
    cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-ccbin", "/usr/bin/g++",
           "-diag-suppress", "177", "-o", BENCH_BIN, src, "-L", KERNEL_DIR, "-lsm100gemm_util", "-Xlinker", "-rpath=$ORIGIN",
           "-lcublas", "-lcublasLt", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for bench.cu:\n{r.stdout}\n{r.stderr}")
    return BENCH_BIN


def build_all(configs=None, force: bool = False, jobs: int | None = None) -> list[str]:
    configs = list(configs) if configs is not None else generate_configs()
    jobs = jobs or max(1, (os.cpu_count() or 2))
    build_util(force)
    with ThreadPoolExecutor(jobs) as ex:
        outs = list(ex.map(lambda c: build_one(c, force), configs))
        testing = ex.submit(build_testing, force)
        bench = ex.submit(build_bench, force)
        testing.result()
        bench.result()
    return outs


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", action="append", help="configuration name (repeatable)")
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true", help="print ptxas register / spill report")
    args = ap.parse_args()
    if args.only:
        cfgs = []
        for n in args.only:
            c = GemmConfig.parse(n)
            if c is None:
                sys.exit(f"cannot parse configuration name {n!r}")
            cfgs.append(c)
        for c in cfgs:
            print(build_one(c, args.force, args.verbose))
    else:
        outs = build_all(force=args.force)
        print(f"built {len(outs)} plugins in {KERNEL_DIR}")


if __name__ == "__main__":
    main()
