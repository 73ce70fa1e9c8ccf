"""The fused output transform of the `_e2` plugins, D = act(alpha * X W^T + beta * C + bias) with bf16 or
e4m3 output, the checked (-DGEMM_DEBUG_BOUNDS) builds on the ragged shapes, and the one way a bounded wait is
made to run out on a GPU.  The reference's gemm_run has no alpha/beta/bias (src/kernel_entry.cu.in:14-16)
and its waits are unbounded (src/bf16_gemm.cuh:137-148): none of this has a counterpart there."""
import ctypes
import os

import numpy as np
import pytest
import torch

import sm120_gemm_b200 as g
from oracle import oracle as o
from tests.gpu_util import to_bits, to_dev

pytestmark = pytest.mark.gpu
TESTING = os.path.join(g.KERNEL_DIR, "testing")


def _act(v: np.ndarray, act: int) -> np.ndarray:
    from scipy.special import erfc

    v = v.astype(np.float64)
    if act == g.ACT_RELU:
        v = np.maximum(v, 0)
    elif act == g.ACT_GELU:
        v = 0.5 * v * erfc(-v / np.sqrt(2))         # = v * Phi(v); 1 + erf(t) would cancel to 0 for v < -8
    elif act == g.ACT_SILU:
        v = v / (1 + np.exp(-v))
    return v.astype(np.float32)


def _run_fused(k, M, N, K, Xd, Wd, alpha=1.0, beta=0.0, C=None, bias=None, act=0, y_dtype=0, y_scale=1.0, amax=None, x_scale_f=1.0, w_scale_f=1.0):
    Y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda") if y_dtype == 0 else torch.full((M, N), 0x7F, dtype=torch.uint8, device="cuda")
    a = g.GemmArgs()
    a.M, a.N, a.K = M, N, K
    a.X, a.W, a.Y = Xd.data_ptr(), Wd.data_ptr(), Y.data_ptr()
    a.x_scale_f, a.w_scale_f = x_scale_f, w_scale_f
    a.alpha, a.beta, a.activation, a.y_dtype, a.y_scale = alpha, beta, act, y_dtype, y_scale
    a.C = C.data_ptr() if C is not None else None
    a.bias = bias.data_ptr() if bias is not None else None
    a.amax = amax.data_ptr() if amax is not None else None
    a.stream = torch.cuda.current_stream().cuda_stream
    g.dispatch_ex(k, a)
    torch.cuda.synchronize()
    k.check_status()
    return Y


@pytest.mark.parametrize("name", ["bf16_bm128_bn128_bk64_s7_cg1_sk1_ab0_e2", "bf16_bm256_bn256_bk64_s7_cg2_sk1_ab0_e2"])
@pytest.mark.parametrize("shape", [(256, 512, 512), (100, 136, 200), (300, 1032, 1088)])
def test_bias_alpha_beta_activation_bf16(registry, cuda_device, name, shape):
    k = registry.find(name)
    assert k is not None
    M, N, K = shape
    rng = np.random.default_rng(M + N)
    X, W = o.make_inputs(M, N, K, seed=3)
    Cb = o.f32_to_bf16_bits(rng.standard_normal((M, N)).astype(np.float32) * 4)
    bb = o.f32_to_bf16_bits(rng.standard_normal(N).astype(np.float32))
    acc = o.gemm_bf16(X, W)
    Xd, Wd, Cd, bd = to_dev(X), to_dev(W), to_dev(Cb), to_dev(bb)
    mx, mw = float(np.abs(o.bf16_bits_to_f32(X)).max()), float(np.abs(o.bf16_bits_to_f32(W)).max())
    for alpha, beta, use_bias, act in [(1.0, 0.0, False, 0), (0.5, 0.0, True, g.ACT_RELU), (1.0, 1.0, False, 0), (-0.25, 2.0, True, g.ACT_GELU),
                                       (1.0, 0.5, True, g.ACT_SILU), (0.0, 1.0, True, 0)]:
        pre = np.float32(alpha) * acc
        if beta != 0.0:
            pre = pre + np.float32(beta) * o.bf16_bits_to_f32(Cb)
        if use_bias:
            pre = pre + o.bf16_bits_to_f32(bb)[None, :]
        ref = _act(pre, act)
        Y = _run_fused(k, M, N, K, Xd, Wd, alpha, beta, Cd if beta != 0.0 else None, bd if use_bias else None, act)
        yb = to_bits(Y)
        assert not np.isnan(o.bf16_bits_to_f32(yb)).any()
        # same bar as the plain GEMM; the bound scales with everything that multiplies or adds to the product
        r = o.check_dense(yb, ref, K, mx, mw)
        slack = abs(alpha) * r["bound"] + 1e-2 * (abs(beta) * 16 + 4)
        assert r["frac_within_bf16_rounding"] >= 0.999 and r["max_abs_err"] <= slack, (name, shape, alpha, beta, use_bias, act, r)
    # the transform's arguments are refused by a plugin that cannot apply them
    plain = registry.find("bf16_bm128_bn128_bk64_s6_cg1_sk1_ab0_e1")
    with pytest.raises(g.GemmError):
        _run_fused(plain, M, N, K, Xd, Wd, bias=bd)
    with pytest.raises(g.GemmError):
        _run_fused(plain, M, N, K, Xd, Wd, alpha=0.5)
    with pytest.raises(g.GemmError):
        _run_fused(k, M, N, K, Xd, Wd, beta=1.0)            # beta without C


@pytest.mark.parametrize("name", ["bf16_bm128_bn128_bk64_s7_cg1_sk1_ab0_e2", "fp8_bm256_bn256_bk128_s7_cg2_sk1_ab0_e2"])
def test_e4m3_output_with_amax(registry, cuda_device, name):
    """FP8 output: Y8 = e4m3(D * y_scale), amax = max|D|.  The codes are compared with the oracle's quantiser
    applied to the oracle's D: equal except where the two FP32 sums straddle a rounding boundary, and never
    more than one code apart."""
    k = registry.find(name)
    assert k is not None
    M, N, K = 384, 520, 1024
    rng = np.random.default_rng(9)
    bb = o.f32_to_bf16_bits(rng.standard_normal(N).astype(np.float32))
    if k.config.dt == "bf16":
        X, W = o.make_inputs(M, N, K, seed=5, dist="normal")
        acc = o.gemm_bf16(X, W)
        Xd, Wd, sx, sw = to_dev(X), to_dev(W), 1.0, 1.0
    else:
        x = rng.standard_normal((M, K)).astype(np.float32); w = rng.standard_normal((N, K)).astype(np.float32)
        sx, sw = float(np.abs(x).max() / 448.0), float(np.abs(w).max() / 448.0)
        qx, qw = o.e4m3_quantise(x, sx), o.e4m3_quantise(w, sw)
        acc = o.gemm_f32(o.e4m3_dequantise(qx, sx), o.e4m3_dequantise(qw, sw))
        Xd, Wd = torch.from_numpy(qx).cuda(), torch.from_numpy(qw).cuda()
    D = _act(acc + o.bf16_bits_to_f32(bb)[None, :], g.ACT_RELU)
    y_scale = float(448.0 / np.abs(D).max()) * 0.9
    amax = torch.zeros(1, dtype=torch.float32, device="cuda")
    Y8 = _run_fused(k, M, N, K, Xd, Wd, bias=to_dev(bb), act=g.ACT_RELU, y_dtype=g.Y_E4M3, y_scale=y_scale, amax=amax, x_scale_f=sx, w_scale_f=sw)
    got = Y8.cpu().numpy()
    exp = o.e4m3_quantise(D * np.float32(y_scale), 1.0)
    same = float((got == exp).mean())
    dg, de = o.e4m3_dequantise(got, 1.0), o.e4m3_dequantise(exp, 1.0)
    step = np.maximum(np.abs(de), 2.0 ** -6) * 0.125 + 1e-6           # one e4m3 code at the value's binade (2^-9 in the subnormal range)
    assert same >= 0.99 and np.all(np.abs(dg - de) <= step), (name, same, float(np.abs(dg - de).max()))
    am = float(amax.cpu()[0])
    assert abs(am - float(np.abs(D).max())) <= 2e-3 * float(np.abs(D).max()), (am, float(np.abs(D).max()))
    # amax accumulates: a second launch with a smaller product leaves it unchanged
    _run_fused(k, M, N, K, Xd, Wd, alpha=0.5, bias=to_dev(bb), act=g.ACT_RELU, y_dtype=g.Y_E4M3, y_scale=y_scale, amax=amax, x_scale_f=sx, w_scale_f=sw)
    assert float(amax.cpu()[0]) == am


EDGE_SHAPES = [(1, 8, 8), (1, 64, 64), (16, 256, 512), (127, 264, 72), (129, 8, 8), (257, 520, 64), (128, 128, 64 * 7), (300, 72, 8), (2, 28672, 64),
               (1000, 520, 1088)]


def test_checked_builds_on_ragged_shapes(cuda_device):
    """The -DGEMM_DEBUG_BOUNDS builds check every computed TMA coordinate and store address before use and report
    the first violation through gemm_check_status: the ragged shapes must pass the check and parity."""
    d = os.path.join(TESTING, "bounds")
    libs = sorted(f for f in os.listdir(d) if f.endswith(".so"))
    assert len(libs) >= 5
    for f in libs:
        k = g.load_plugin(os.path.join(d, f))
        for (M, N, K) in EDGE_SHAPES:
            if not k.can_run(M, N, K):
                continue
            X, W = o.make_inputs(M, N, K, seed=M + N + K)
            Xd, Wd = to_dev(X), to_dev(W)
            if k.config.epi == 2:
                Y = _run_fused(k, M, N, K, Xd, Wd)
            else:
                from tests.gpu_util import run_bf16

                Y = run_bf16(k, Xd, Wd)         # check_status inside: raises if a check fired
            r = o.check_dense(to_bits(Y), o.gemm_bf16(X, W), K, 1.0, 1.0)
            assert r["ok"], (f, M, N, K, r)


def test_bounded_wait_runs_out_and_kernel_returns(cuda_device):
    """A plugin built with a short wait limit (2e6 SM cycles) whose TMA producer can be told to stop requesting
    data from a given k-block on.  Nothing is in flight at that point; the MMA issuer's wait for the next stage
    runs out, every role leaves its loop, TMEM is released and the kernel ends.  The host then sees
    GEMM_ERR_DEVICE_TIMEOUT from gemm_check_status, and the next launch on the same context is correct."""
    path = os.path.join(TESTING, "expiry", "libgemm_bf16_bm128_bn128_bk64_s6_cg1_sk1_ab0_e1.so")
    k = g.load_plugin(path)
    M, N, K = 128, 128, 1024
    X, W = o.make_inputs(M, N, K, seed=1)
    Xd, Wd = to_dev(X), to_dev(W)
    Y = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    a = g.GemmArgs()
    a.M, a.N, a.K = M, N, K
    a.X, a.W, a.Y = Xd.data_ptr(), Wd.data_ptr(), Y.data_ptr()
    a.x_scale_f = a.w_scale_f = 1.0
    a.stream = torch.cuda.current_stream().cuda_stream
    a.reserved = 3                      # the producer stops before k-block 2 of 16
    g.dispatch_ex(k, a)                 # the launch itself succeeds
    with pytest.raises(g.GemmError) as e:
        k.check_status()
    # the issuer waiting for operand data (code 2) and the epilogue waiting for the accumulator (code 4) run out together;
    # whichever records first is reported
    assert e.value.code == 5 and ("code 2" in str(e.value) or "code 4" in str(e.value))
    k.check_status()                    # reading the status cleared it
    a.reserved = 0
    Y.fill_(float("nan"))
    g.dispatch_ex(k, a)
    torch.cuda.synchronize()
    k.check_status()
    assert o.check_dense(to_bits(Y), o.gemm_bf16(X, W), K, 1.0, 1.0)["ok"]
