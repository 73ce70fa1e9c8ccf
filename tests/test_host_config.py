"""CPU tests of the host side: configuration names, validity rules, the shared-memory model,
the autotune cache, plugin loading (every ABI symbol) and error reporting -- in the Python
mirror and, through a compiled test program, in the C++ header a C++ caller includes."""
import ctypes
import os
import re
import subprocess

import pytest

import sm120_gemm_b200 as g

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_header_checks(tmp_path, registry):
    """The C++ header on its own (names, cache, scheduler arithmetic) and on the real plugins: every symbol
    resolved (gemm_run_no_alloc included), the heuristic dispatcher, two threads in the rejection paths.
    The heuristic picks must equal the Python mirror's."""
    exe = tmp_path / "host_config_test"
    subprocess.check_call(["/usr/bin/g++", "-std=c++17", "-O1", "-pthread", "-I/usr/local/cuda/include", "-o", str(exe),
                           os.path.join(ROOT, "tests", "host_config_test.cpp"), "-ldl"])
    out = subprocess.run([str(exe), str(tmp_path / "cache.txt"), g.KERNEL_DIR], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.strip().splitlines()[-1].startswith("OK"), out.stdout + out.stderr
    picks = [ln.split() for ln in out.stdout.splitlines() if ln.startswith("PICK")]
    assert len(picks) >= 15
    for _, dt, M, N, K, name in picks:
        k = registry.heuristic(int(M), int(N), int(K), dt)
        assert k is not None and k.config.name() == name, (dt, M, N, K, name, k and k.config.name())


def test_heuristic_dispatch_needs_no_cache(registry):
    """A shape missing from the autotune cache gets a runnable plugin from the cost model (the reference skips
    such shapes, src/bench.cu:455-458); a cached shape keeps its entry."""
    cache = g.AutotuneCache()
    cache.load(os.path.join(ROOT, "sm120_gemm_b200", "autotune_cache.txt"))
    for dt, shapes in {"bf16": [(1, 8, 8), (77, 1000, 4096), (3000, 5000, 7000 // 8 * 8), (128, 4096, 14336)],
                       "fp8": [(64, 512, 1024), (8192, 8192, 8192)], "mxfp8": [(256, 512, 1024)], "w4a4": [(16, 28672, 8192)],
                       "w4a16": [(1, 128, 128), (128, 28672, 8192)]}.items():
        for (M, N, K) in shapes:
            k = registry.select(cache, M, N, K, dt)
            assert k is not None and k.config.dt == dt and k.can_run(M, N, K) and k.config.epi != 2
            hit = cache.lookup(M, N, K, dt)
            if hit:
                assert k.config.name() == hit[0].name()
    assert registry.heuristic(128, 130, 64) is None
    # large square shapes go to the large CTA-pair tiles, one-row decode shapes to a split or stream-K plugin
    assert registry.heuristic(8192, 8192, 8192).config.bm >= 256
    assert registry.heuristic(16, 4096, 14336).config.split_k != 1


def test_config_name_roundtrip_all_generated():
    cfgs = g.generate_configs()
    assert len(cfgs) == len({c.name() for c in cfgs}) > 40
    for c in cfgs:
        assert g.GemmConfig.parse(c.name()) == c
        assert c.bm in (128 * c.cg, 256 * c.cg) and c.mb == c.bm // (128 * c.cg) and c.smem_bytes() <= 232448
    assert g.GemmConfig.parse("bm128_bn64_bk64_s3_cwg2_wm32_wn32_sk1") is None
    assert g.GemmConfig.parse("bf16_bm128_bn128_bk64_s4_cg1_sk1_ab0_e1x") is None


def test_registry_loads_every_plugin_and_symbol(registry):
    names = {k.config.name() for k in registry.kernels}
    built = {f[len("libgemm_"):-3] for f in os.listdir(g.KERNEL_DIR) if f.startswith("libgemm_") and f.endswith(".so")}
    assert names == built
    header = open(os.path.join(ROOT, "include", "sm100_gemm.h")).read()
    declared = set(re.findall(r"\b(gemm_[a-z_]+)\s*\(", header))
    assert declared == set(g.ABI_SYMBOLS)
    for k in registry.kernels:
        for sym in declared:
            assert getattr(k.lib, sym) is not None
        assert k.lib.gemm_config_name().decode() == k.config.name()
        # the host-side shared-memory model must equal what the kernel was compiled with
        assert k.smem_bytes() == k.config.smem_bytes()


def test_util_library_exports_its_header():
    header = open(os.path.join(ROOT, "include", "sm100_gemm_util.h")).read()
    declared = set(re.findall(r"\b(gemm_[a-z0-9_]+)\s*\(", header))
    assert declared == set(g.UTIL_SYMBOLS)
    lib = g.util_lib()
    for sym in declared:
        assert getattr(lib, sym) is not None
    assert lib.gemm_mx_tiled_scale_bytes(100, 256) == 1 * 2 * 512      # one 128-row tile, two 4-block atoms
    assert lib.gemm_mx_tiled_scale_bytes(129, 128) == 2 * 1 * 512


def test_validity_rules_match_plugins(registry):
    shapes = [(1, 8, 8), (128, 128, 64), (100, 136, 200), (128, 130, 64), (128, 128, 60), (128, 4096, 14336),
              (128, 4096, 14400), (16, 28672, 8192), (0, 8, 8), (1024, 1024, 1000)]
    for k in registry.kernels:
        for (M, N, K) in shapes:
            assert bool(k.can_run(M, N, K)) == k.config.is_valid_for(M, N, K), (k.config.name(), M, N, K)
        if k.config.split_k > 1:
            assert k.workspace_bytes(128, 4096, 14336) == k.config.split_k * 128 * 4096 * 4
        elif k.config.dt == "w4a16":
            assert k.workspace_bytes(16, 4096, 14336) == 2 * 160 * 128 * 128 * 4
        elif k.config.split_k == 0:   # stream-K: two partial-tile slots per CTA (pair), shape-independent
            assert k.workspace_bytes(128, 4096, 14336) == 2 * (160 // k.config.cg) * k.config.bm * k.config.bn * 4
        else:
            assert k.workspace_bytes(128, 4096, 14336) == 0


def test_errors_are_reported_not_fatal(registry):
    """No launch can happen here (no GPU); argument and shape errors must come back as codes."""
    k = next(k for k in registry.kernels if k.config.dt == "bf16" and k.config.split_k == 1)
    k.lib.gemm_run(128, 130, 64, 0, 0, 0, 0, 0)          # N not a multiple of 8
    code, msg = k.last_error()
    assert code == 1 and "not supported" in msg
    k.lib.gemm_run(128, 128, 64, 0, 0, 0, 0, 0)          # null pointers
    assert k.last_error()[0] == 6
    args = g.GemmArgs()
    args.struct_size = 4
    assert k.lib.gemm_run_ex(ctypes.byref(args)) == 6    # wrong struct size
    args.struct_size = ctypes.sizeof(g.GemmArgs)
    args.dtype = 3
    assert k.lib.gemm_run_ex(ctypes.byref(args)) == 6    # dtype does not match the plugin
    sk = next(k for k in registry.kernels if k.config.dt == "bf16" and k.config.split_k == 4)
    with pytest.raises(g.GemmError) as e:
        g.dispatch(sk, 128, 128, 256, 16, 16, 16, 0, 0)  # split-K without a workspace
    assert e.value.code == 4
    fp8 = next((k for k in registry.kernels if k.config.dt == "fp8"), None)
    if fp8 is not None:
        fp8.lib.gemm_run(128, 128, 128, 16, 16, 16, 0, 0)
        assert fp8.last_error()[0] == 6                  # gemm_run is the bf16 entry point


def test_autotune_cache_roundtrip(tmp_path):
    p = tmp_path / "cache.txt"
    p.write_text("# c\n1024,1024,1024 bf16_bm128_bn128_bk64_s4_cg1_sk1_ab0_e1 0.0123\n"
                 "bf16,8,16384,16384,16384 bf16_bm256_bn256_bk64_s6_cg2_sk1_ab0_e1 1.5\nbad line\n"
                 "1,2,3 nonsense 1.0\n")
    c = g.AutotuneCache()
    assert c.load(str(p)) and len(c.entries) == 2
    assert c.lookup(1024, 1024, 1024)[1] == 0.0123
    assert c.lookup(16384, 16384, 16384, gpus=8) and not c.lookup(16384, 16384, 16384)
    cfg = g.GemmConfig.parse("bf16_bm128_bn64_bk64_s8_cg1_sk2_ab0_e0")
    c.store(128, 4096, 14336, cfg, 0.02)
    c.save(str(p))
    d = g.AutotuneCache()
    d.load(str(p))
    assert d.entries == c.entries
    assert not g.AutotuneCache().load(str(tmp_path / "missing.txt"))


def test_committed_autotune_cache_names_generated_configs():
    """Every line of the shipped cache names a configuration the generator still produces (so the plugin
    exists after a build) and that accepts the line's shape."""
    from sm120_gemm_b200.gen_configs import generate_configs

    names = {c.name(): c for c in generate_configs()}
    cache = g.AutotuneCache()
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "sm120_gemm_b200", "autotune_cache.txt")
    assert cache.load(path) and len(cache.entries) >= 10
    for (dt, gpus, M, N, K), (cfg, ms) in cache.entries.items():
        assert cfg.name() in names, f"{cfg.name()} is not generated any more"
        assert names[cfg.name()].is_valid_for(M, N, K) and ms > 0


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` runs on the host cores alone and prints one JSON line with the agreed keys."""
    import json
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "3"],
                       capture_output=True, text=True, timeout=300, cwd=root)
    assert r.returncode == 0, r.stderr[-500:]
    d = json.loads(r.stdout.strip().splitlines()[-1])
    assert d["impl"] == "reference" and d["metric"] == "gemm_tflops" and d["unit"] == "TFLOPS" and d["value"] > 0
    assert d["higher_is_better"] is True and d["cpu_baseline"]["kind"] in ("port", "reference") and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["value"] == d["value"] and d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0


def test_cmake_build_configures_and_builds_a_plugin(tmp_path):
    """The C++-only build (CMakeLists.txt at the repository root): configure for one data-type family, build one
    plugin, the utility library and the host-side unit test, run it through ctest; the plugin must load and name
    itself like its file."""
    import shutil

    if shutil.which("cmake") is None or shutil.which("ninja") is None:
        pytest.skip("cmake / ninja not installed")
    b = str(tmp_path / "build")
    subprocess.check_call(["cmake", "-S", ROOT, "-B", b, "-G", "Ninja", "-DGEMM_DTYPES=w4a16", "-DCMAKE_CUDA_COMPILER=/usr/local/cuda/bin/nvcc",
                           "-DCMAKE_CUDA_HOST_COMPILER=/usr/bin/g++"], stdout=subprocess.DEVNULL)
    name = "w4a16_bm128_bn16_bk128_s6_cg1_sk0_ab1_e0"
    subprocess.check_call(["cmake", "--build", b, "--target", f"gemm_{name}", "sm100gemm_util", "host_config_test"], stdout=subprocess.DEVNULL)
    subprocess.check_call(["ctest", "--test-dir", b], stdout=subprocess.DEVNULL)
    k = g.load_plugin(os.path.join(b, "kernels", f"libgemm_{name}.so"))
    assert k.config.name() == name and k.can_run(16, 4096, 4096) and not k.can_run(17, 4096, 4096)
    assert os.path.exists(os.path.join(b, "kernels", "libsm100gemm_util.so"))
