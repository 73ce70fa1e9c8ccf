"""Times the reference project's own mma.sync GEMM (recompiled for sm_100a into oracle/_ref/libref.so,
see Makefile.ref) next to a kernel plugin of this repo, same buffers, same protocol (5 warm-ups, 20
launches each in its own event pair, spacer kernel), and checks the two results against each other.
Comparator only: nothing in the product imports this.

    python oracle/time_ref_kernel.py 4096,4096,4096 8192,8192,8192
"""
import ctypes
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import sm120_gemm_b200 as g  # noqa: E402
from sm120_gemm_b200.autotune import time_fn  # noqa: E402


def main():
    so = os.path.join(ROOT, "oracle", "_ref", "libref.so")
    if not os.path.exists(so):
        sys.exit("oracle/_ref/libref.so is not built (needs the reference sources: make -C oracle -f Makefile.ref)")
    ref = ctypes.CDLL(so)
    ref.ref_mma_gemm.argtypes = [ctypes.c_int] * 3 + [ctypes.c_void_p] * 4
    util = g.util_lib()
    st = torch.cuda.current_stream().cuda_stream
    reg = g.KernelRegistry()
    reg.load_dir(g.KERNEL_DIR, dt="bf16")
    cache = g.AutotuneCache()
    cache.load(os.path.join(ROOT, "sm120_gemm_b200", "autotune_cache.txt"))
    for arg in sys.argv[1:] or ["4096,4096,4096"]:
        M, N, K = (int(v) for v in arg.split(","))
        X = (torch.rand((M, K), device="cuda") * 2 - 1).bfloat16()
        W = (torch.rand((N, K), device="cuda") * 2 - 1).bfloat16()
        Yr = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        Yo = torch.empty_like(Yr)
        hit = cache.lookup(M, N, K)
        k = reg.find(hit[0].name() if hit else "bf16_bm256_bn256_bk64_s6_cg2_sk1_ab0_e1")
        ws = torch.empty(max(k.workspace_bytes(M, N, K), 16), dtype=torch.uint8, device="cuda")
        assert ref.ref_mma_gemm(M, N, K, X.data_ptr(), W.data_ptr(), Yr.data_ptr(), st) == 0
        g.dispatch(k, M, N, K, X.data_ptr(), W.data_ptr(), Yo.data_ptr(), ws.data_ptr(), st)
        torch.cuda.synchronize()
        diff = (Yr.float() - Yo.float()).abs().max().item()
        # which side a difference comes from: both against an FP32 product (TF32 off), error in units of
        # the bf16 spacing at the exact value
        torch.backends.cuda.matmul.allow_tf32 = False
        rows = torch.arange(0, M, max(1, M // 1024), device="cuda")
        exact = X[rows].float() @ W.float().T
        ulp = torch.maximum(exact.abs(), torch.full_like(exact, 1e-3)).log2().floor().exp2() / 128.0
        err_ref = ((Yr[rows].float() - exact).abs() / ulp)
        err_our = ((Yo[rows].float() - exact).abs() / ulp)
        print(f"  vs FP32 on {rows.numel()} rows: reference kernel max {err_ref.max().item():.2f} ulp, >2 ulp in {(err_ref > 2).sum().item()} elements; "
              f"this repo max {err_our.max().item():.2f} ulp, >2 ulp in {(err_our > 2).sum().item()} elements")
        t_ref = time_fn(lambda: ref.ref_mma_gemm(M, N, K, X.data_ptr(), W.data_ptr(), Yr.data_ptr(), st), st, util)
        t_our = time_fn(lambda: g.dispatch(k, M, N, K, X.data_ptr(), W.data_ptr(), Yo.data_ptr(), ws.data_ptr(), st), st, util)
        fl = 2.0 * M * N * K
        print(f"{M}x{N}x{K}: reference mma.sync kernel (bm128_bn128_bk64_s2_cg2) {t_ref:.4f} ms {fl / t_ref / 1e9:.1f} TFLOPS | "
              f"{k.config.name()} {t_our:.4f} ms {fl / t_our / 1e9:.1f} TFLOPS | speed-up {t_ref / t_our:.2f}x | max |diff| {diff:.4g}")


if __name__ == "__main__":
    main()
