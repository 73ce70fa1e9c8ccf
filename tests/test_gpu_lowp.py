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


def tiled_scales_numpy(sc: np.ndarray) -> np.ndarray:
    """The atom layout of include/sm100_gemm.h, computed independently of the device converter."""
    R, KB = sc.shape
    ka = (KB + 3) // 4
    out = np.full(((R + 127) // 128) * ka * 512, 127, np.uint8)
    r = np.arange(R)[:, None]
    kb = np.arange(KB)[None, :]
    idx = ((r // 128) * ka + kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4
    out[idx.ravel()] = sc.ravel()
    return out


def to_tiled_dev(sc: np.ndarray, K: int) -> torch.Tensor:
    import sm120_gemm_b200 as g

    util = g.util_lib()
    src = torch.from_numpy(np.ascontiguousarray(sc)).cuda()
    dst = torch.empty(util.gemm_mx_tiled_scale_bytes(sc.shape[0], K), dtype=torch.uint8, device="cuda")
    assert util.gemm_mx_scales_to_tiled(src.data_ptr(), dst.data_ptr(), sc.shape[0], K, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    return dst


def test_scale_tiling_kernel(cuda_device):
    rng = np.random.default_rng(5)
    for (R, K) in [(128, 128), (100, 256), (300, 1024), (257, 96 * 32)]:
        sc = rng.integers(100, 140, (R, K // 32)).astype(np.uint8)
        assert np.array_equal(to_tiled_dev(sc, K).cpu().numpy(), tiled_scales_numpy(sc))


def mx_case(M, N, K, kind, seed, spread=True):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = rng.standard_normal((N, K)).astype(np.float32)
    if spread:   # give the blocks different magnitudes so that wrong scale placement cannot hide
        x *= np.exp2(rng.integers(-3, 4, (M, K // 32))).repeat(32, axis=1).astype(np.float32)
        w *= np.exp2(rng.integers(-3, 4, (N, K // 32))).repeat(32, axis=1).astype(np.float32)
    qx, sx = o.mx_quantise(x, kind)
    qw, sw = o.mx_quantise(w, kind)
    return qx, sx, qw, sw


def run_mx(k, M, N, K, qx, sx, qw, sw):
    return run_ex(k, M, N, K, torch.from_numpy(qx).cuda(), torch.from_numpy(qw).cuda(), x_scale=to_tiled_dev(sx, K),
                  w_scale=to_tiled_dev(sw, K))


@pytest.mark.parametrize("shape", [(128, 128, 128), (128, 256, 256), (256, 512, 1024), (100, 136, 512), (1024, 1024, 1024)])
def test_mxfp8(registry, cuda_device, shape):
    """BASELINE config 4(b): e4m3 elements, ue8m0 scale per 32 K-elements on both operands."""
    M, N, K = shape
    qx, sx, qw, sw = mx_case(M, N, K, 8, seed=3)
    dx, dw = o.mx_dequantise(qx, sx, 8), o.mx_dequantise(qw, sw, 8)
    ref = o.gemm_f32(dx, dw)
    ran = 0
    for k in registry.kernels:
        if k.config.dt != "mxfp8" or not k.can_run(M, N, K):
            continue
        Y = to_bits(run_mx(k, M, N, K, qx, sx, qw, sw))
        assert not np.isnan(o.bf16_bits_to_f32(Y)).any(), k.config.name()
        r = o.check_dense(Y, ref, K, float(np.abs(dx).max()), float(np.abs(dw).max()))
        assert r["ok"], (k.config.name(), r)
        ran += 1
    assert ran >= 5


def test_mxfp8_8192_sampled_rows(registry, cuda_device):
    """BASELINE config 4(b) at full size: MXFP8 8192^3 with real quantised data (block magnitudes spread over
    2^-3..2^3 so a misplaced scale cannot hide), 40 sampled rows against the host oracle, dense bar.
    Runs the one-CTA and the CTA-pair tile."""
    M = N = K = 8192
    qx, sx, qw, sw = mx_case(M, N, K, 8, seed=3)
    rows = np.unique(np.concatenate([[0, 127, 128, 255, 256, M - 1], np.random.default_rng(1).integers(0, M, 34)]))
    dx, dw = o.mx_dequantise(qx[rows], sx[rows], 8), o.mx_dequantise(qw, sw, 8)
    ref = o.gemm_f32(dx, dw)
    Xd, Wd, SXd, SWd = torch.from_numpy(qx).cuda(), torch.from_numpy(qw).cuda(), to_tiled_dev(sx, K), to_tiled_dev(sw, K)
    sel = torch.from_numpy(rows).cuda()
    ran = 0
    for k in registry.kernels:
        if k.config.dt != "mxfp8" or k.config.split_k != 1 or k.config.epi != 1:
            continue
        Y = run_ex(k, M, N, K, Xd, Wd, x_scale=SXd, w_scale=SWd)
        r = o.check_dense(to_bits(Y[sel]), ref, K, float(np.abs(dx).max()), float(np.abs(dw).max()))
        assert r["max_abs_err"] <= r["bound"] and r["frac_within_bf16_rounding"] >= 0.999, (k.config.name(), r)
        ran += 1
    assert ran >= 2


@pytest.mark.parametrize("M", [1, 16, 128])
def test_w4a4_config5_shapes(registry, cuda_device, M):
    """BASELINE config 5(b) at its stated shape: M in {1, 16, 128}, N = 28672, K = 8192, MX-FP4 on both
    operands, full host oracle (dequantise, FP32 GEMM), every w4a4 plugin that takes the shape."""
    N, K = 28672, 8192
    qx, sx, qw, sw = mx_case(M, N, K, 4, seed=4)
    dx, dw = o.mx_dequantise(qx, sx, 4), o.mx_dequantise(qw, sw, 4)
    ref = o.gemm_f32(dx, dw)
    Xd, Wd, SXd, SWd = torch.from_numpy(qx).cuda(), torch.from_numpy(qw).cuda(), to_tiled_dev(sx, K), to_tiled_dev(sw, K)
    ran = 0
    for k in registry.kernels:
        if k.config.dt != "w4a4" or not k.can_run(M, N, K):
            continue
        Y = to_bits(run_ex(k, M, N, K, Xd, Wd, x_scale=SXd, w_scale=SWd))
        assert not np.isnan(o.bf16_bits_to_f32(Y)).any(), k.config.name()
        r = o.check_quantised(Y, ref)
        assert r["ok"], (k.config.name(), M, r)
        ran += 1
    assert ran >= 5


@pytest.mark.parametrize("shape", [(128, 128, 256), (128, 256, 512), (16, 512, 1024), (1, 256, 2048), (100, 136, 512), (512, 1024, 2048)])
def test_w4a4_mxfp4(registry, cuda_device, shape):
    """BASELINE config 5(b): e2m1 elements (two per byte), ue8m0 scale per 32 K-elements."""
    M, N, K = shape
    qx, sx, qw, sw = mx_case(M, N, K, 4, seed=4)
    dx, dw = o.mx_dequantise(qx, sx, 4), o.mx_dequantise(qw, sw, 4)
    ref = o.gemm_f32(dx, dw)
    ran = 0
    for k in registry.kernels:
        if k.config.dt != "w4a4" or not k.can_run(M, N, K):
            continue
        Y = to_bits(run_mx(k, M, N, K, qx, sx, qw, sw))
        assert not np.isnan(o.bf16_bits_to_f32(Y)).any(), k.config.name()
        r = o.check_quantised(Y, ref)
        assert r["ok"], (k.config.name(), r)
        ran += 1
    assert ran >= 5


def w4a16_case(M, N, K, seed):
    """BASELINE config 5(a): X ~ N(0,1) bf16; q uniform int in [-8,7]; bf16 scale = U[0.5,2]/8 per 128 K-elements."""
    rng = np.random.default_rng(seed)
    X = o.f32_to_bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    q = rng.integers(-8, 8, (N, K)).astype(np.int8)
    sc = o.f32_to_bf16_bits((rng.uniform(0.5, 2.0, (N, K // 128)) / 8).astype(np.float32))
    return X, q, sc


@pytest.mark.parametrize("shape", [(1, 128, 128), (16, 256, 256), (16, 1024, 1024), (128, 512, 2048), (7, 136, 384), (100, 4096, 1024),
                                   (1, 28672, 8192), (16, 28672, 8192), (128, 28672, 8192)])
def test_w4a16(registry, cuda_device, shape):
    M, N, K = shape
    X, q, sc = w4a16_case(M, N, K, seed=4)
    packed = o.int4_pack(q)
    ref = o.gemm_f32(o.bf16_bits_to_f32(X), o.int4_dequantise(packed, sc, 128))
    Xd = torch.from_numpy(X.view(np.int16)).cuda().view(torch.bfloat16)
    Wd = torch.from_numpy(packed).cuda()
    Sd = torch.from_numpy(sc.view(np.int16)).cuda().view(torch.bfloat16)
    ran = 0
    for k in registry.kernels:
        if k.config.dt != "w4a16" or not k.can_run(M, N, K):
            continue
        Y = to_bits(run_ex(k, M, N, K, Xd, Wd, w_scale=Sd, group_size=128))
        assert not np.isnan(o.bf16_bits_to_f32(Y)).any(), k.config.name()
        r = o.check_quantised(Y, ref)
        assert r["ok"], (k.config.name(), shape, r)
        ran += 1
    assert ran >= 1
