"""The C++ harness (csrc/bench.cu -> kernels/bench) run as a program: the reference's three modes
(src/bench.cu:583-597) on small shapes, the data-type switch with its library comparator, the single-kernel
mode and the JSON lines."""
import json
import os
import subprocess

import pytest

import sm120_gemm_b200 as g

pytestmark = pytest.mark.gpu
BENCH = os.path.join(g.KERNEL_DIR, "bench")


def run(*args, timeout=600):
    assert os.path.exists(BENCH), "kernels/bench is missing: run __graft_entry__.build()"
    r = subprocess.run([BENCH, *args], capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return r.stdout


def test_debug_mode_calls_the_class_templates(cuda_device):
    out = run("--debug", "--shape", "1024,1024,1024", "--shape", "384,520,1088")
    assert out.count("[MMA] PASSED") == 2 and out.count("[MMA-SK] PASSED") >= 1 and "FAILED" not in out


def test_autotune_writes_cache_then_quick_reads_it(cuda_device, tmp_path):
    cache = str(tmp_path / "cache.txt")
    out = run("--autotune", "--shape", "128,4096,14336", "--cache", cache, "--peaks", os.path.join(os.path.dirname(BENCH), "..", "..", "MEASURED_PEAKS.json")
              if os.path.exists(os.path.join(os.path.dirname(BENCH), "..", "..", "MEASURED_PEAKS.json")) else "/dev/null")
    assert "BEST:" in out and "cuBLAS:" in out and "FAILED check" not in out and "LAUNCH FAIL" not in out
    lines = [ln for ln in open(cache).read().splitlines() if ln and not ln.startswith("#")]
    assert len(lines) == 1 and lines[0].startswith("bf16,1,128,4096,14336 bf16_bm")
    assert g.GemmConfig.parse(lines[0].split()[1]) is not None
    again = run("--autotune", "--shape", "128,4096,14336", "--cache", cache)
    assert "cached:" in again
    quick = run("--cache", cache)
    assert "Ours:" in quick and "cuBLAS:" in quick and lines[0].split()[1] in quick


@pytest.mark.parametrize("dt,kernel,lib", [("fp8", "fp8_bm256_bn256_bk128_s6_cg2_sk1_ab0_e1", "cuBLASLt"),
                                           ("mxfp8", "mxfp8_bm128_bn256_bk128_s3_cg1_sk1_ab0_e1", "cuBLASLt"),
                                           ("w4a4", "w4a4_bm128_bn256_bk256_s3_cg1_sk1_ab0_e1", "cuBLASLt"),
                                           ("w4a16", "w4a16_bm128_bn16_bk64_s4_cg1_sk0_ab1_e0", "cuBLASLt: unsupported")])
def test_single_kernel_mode_per_dtype_with_comparator_and_json(cuda_device, tmp_path, dt, kernel, lib):
    js = str(tmp_path / "out.jsonl")
    shape = "16,2048,2048" if dt == "w4a16" else "1024,1024,2048"
    out = run("--kernel", kernel, "--shape", shape, "--json", js)
    assert "Ours:" in out and "FAILED" not in out and "LAUNCH FAIL" not in out
    assert lib.split(":")[0] in out          # the comparator ran, or the harness says the library has none
    d = json.loads(open(js).read().splitlines()[-1])
    assert d["dtype"] == dt and d["kernel"] == kernel and d["ms"] > 0 and d["tflops"] > 0 and d["shape"] == [int(v) for v in shape.split(",")]
    assert d["comparator"].startswith("cuBLAS")


def test_uncached_shape_gets_the_heuristic_pick_and_host_reference_line(cuda_device, tmp_path):
    oracle_so = os.path.join(os.path.dirname(BENCH), "..", "..", "oracle", "liboracle.so")
    out = run("--shape", "200,1000,4096", "--cache", str(tmp_path / "none.txt"), "--host-ref", oracle_so)
    assert "heuristic pick bf16_bm" in out and "Ours:" in out and "NO VALID CONFIG" not in out
    assert "host reference (FP32 loop," in out and "GFLOP/s" in out
