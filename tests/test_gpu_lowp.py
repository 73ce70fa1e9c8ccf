"""Parity of the low-precision variants against the host oracle "dequantise, then FP32 GEMM".
The reference has none of these data types; the tolerances are the task's:
  FP8 (per-tensor, MXFP8): the dense bar (max-abs bound + 99.9 % within bf16 rounding), with
  max|x|, max|w| taken over the dequantised values;
  W4A16 / W4A4: ||float(Y) - bf16_rn(ref)||_F / ||ref||_F <= 1e-3."""
import numpy as np
import pytest
import torch

from oracle import oracle as o
from tests.gpu_util import run_ex, to_bits

pytestmark = pytest.mark.gpu


def fp8_case(M, N, K, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = rng.standard_normal((N, K)).astype(np.float32)
    sx = float(np.abs(x).max() / 448.0)
    sw = float(np.abs(w).max() / 448.0)
    qx, qw = o.e4m3_quantise(x, sx), o.e4m3_quantise(w, sw)
    return qx, qw, sx, sw


@pytest.mark.parametrize("shape", [(256, 256, 256), (100, 136, 208), (1024, 1024, 1024), (128, 4096, 2048)])
def test_fp8_per_tensor(registry, cuda_device, shape):
    """BASELINE config 4(a) at sizes the host oracle finishes in seconds, every fp8 plugin."""
    M, N, K = shape
    qx, qw, sx, sw = fp8_case(M, N, K, seed=3)
    dx, dw = o.e4m3_dequantise(qx, sx), o.e4m3_dequantise(qw, sw)
    ref = o.gemm_f32(dx, dw)
    Xd, Wd = torch.from_numpy(qx).cuda(), torch.from_numpy(qw).cuda()
    ran = 0
    for k in registry.kernels:
        if k.config.dt != "fp8" or not k.can_run(M, N, K):
            continue
        Y = to_bits(run_ex(k, M, N, K, Xd, Wd, x_scale_f=sx, w_scale_f=sw))
        assert not np.isnan(o.bf16_bits_to_f32(Y)).any(), k.config.name()
        r = o.check_dense(Y, ref, K, float(np.abs(dx).max()), float(np.abs(dw).max()))
        assert r["ok"], (k.config.name(), r)
        ran += 1
    assert ran > 10


def test_fp8_8192_sampled_rows(registry, cuda_device):
    """BASELINE config 4(a) at full size: 8192^3, 40 sampled rows against the host oracle."""
    M = N = K = 8192
    qx, qw, sx, sw = fp8_case(M, N, K, seed=3)
    k = registry.find("fp8_bm256_bn256_bk128_s6_cg2_sk1_ab0_e1")
    assert k is not None
    Y = run_ex(k, M, N, K, torch.from_numpy(qx).cuda(), torch.from_numpy(qw).cuda(), x_scale_f=sx, w_scale_f=sw)
    rows = np.unique(np.concatenate([[0, 127, 128, 255, 256, M - 1], np.random.default_rng(1).integers(0, M, 34)]))
    dx, dw = o.e4m3_dequantise(qx[rows], sx), o.e4m3_dequantise(qw, sw)
    ref = o.gemm_f32(dx, dw)
    r = o.check_dense(to_bits(Y[torch.from_numpy(rows).cuda()]), ref, K, float(np.abs(dx).max()), float(np.abs(dw).max()))
    assert r["max_abs_err"] <= r["bound"] and r["frac_within_bf16_rounding"] >= 0.999, r
