"""The steps in front of the low-precision GEMMs: activation / weight quantisation kernels (GPU, bit-exact
against the oracle's quantisers: this is byte work) and the offline packers + weight file (host code, CPU).
The reference has none of this (its inputs are random bf16 in memory, src/bench.cu:353-355); the layouts are
the ones include/sm100_gemm.h documents."""
import ctypes
import os

import numpy as np
import pytest

import sm120_gemm_b200 as g
from oracle import oracle as o

DT = g.DT_IDS


def _vp(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return ctypes.c_void_p(a.ctypes.data)


def tiled_scales_numpy(sc: np.ndarray) -> np.ndarray:
    """The atom layout of include/sm100_gemm.h, computed independently of the library."""
    R, KB = sc.shape
    ka = (KB + 3) // 4
    out = np.full(((R + 127) // 128) * ka * 512, 127, np.uint8)
    r = np.arange(R)[:, None]
    kb = np.arange(KB)[None, :]
    idx = ((r // 128) * ka + kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4
    out[idx.ravel()] = sc.ravel()
    return out


# ------------------------------------------------------------------------------------------ host packers (CPU)
def test_int4_and_fp4_packers_round_trip():
    lib = g.util_lib()
    rng = np.random.default_rng(0)
    N, K = 37, 256
    q = rng.integers(-8, 8, (N, K)).astype(np.int8)
    packed = np.empty((N, K // 2), np.uint8)
    assert lib.gemm_pack_int4_host(_vp(q), N, K, _vp(packed)) == 0
    assert np.array_equal(packed, o.int4_pack(q))                     # the layout the W4A16 kernel and the oracle read
    back = np.empty_like(q)
    assert lib.gemm_unpack_int4_host(_vp(packed), N, K, _vp(back)) == 0 and np.array_equal(back, q)
    bad = q.copy(); bad[3, 5] = 9
    assert lib.gemm_pack_int4_host(_vp(bad), N, K, _vp(packed)) == -5   # out of range is refused, not wrapped
    codes = rng.integers(0, 16, (N, K)).astype(np.uint8)
    p4 = np.empty((N, K // 2), np.uint8)
    assert lib.gemm_pack_fp4_host(_vp(codes), N, K, _vp(p4)) == 0
    assert np.array_equal(p4, codes[:, 0::2] | (codes[:, 1::2] << 4))
    c2 = np.empty_like(codes)
    assert lib.gemm_unpack_fp4_host(_vp(p4), N, K, _vp(c2)) == 0 and np.array_equal(c2, codes)


@pytest.mark.parametrize("shape", [(128, 128), (100, 256), (300, 1024), (257, 96 * 32), (1, 32)])
def test_host_scale_tiler_matches_layout_and_inverts(shape):
    lib = g.util_lib()
    R, K = shape
    sc = np.random.default_rng(R + K).integers(100, 140, (R, K // 32)).astype(np.uint8)
    nbytes = lib.gemm_mx_tiled_scale_bytes(R, K)
    assert nbytes == lib.gemm_packed_scale_bytes(DT["mxfp8"], R, K) == lib.gemm_packed_scale_bytes(DT["w4a4"], R, K)
    tiled = np.empty(nbytes, np.uint8)
    assert lib.gemm_mx_scales_to_tiled_host(_vp(sc), R, K, _vp(tiled)) == 0
    assert np.array_equal(tiled, tiled_scales_numpy(sc))
    back = np.empty_like(sc)
    assert lib.gemm_mx_scales_from_tiled_host(_vp(tiled), R, K, _vp(back)) == 0 and np.array_equal(back, sc)


def _quantised_weights(dt: str, N: int, K: int, seed: int):
    """(elements, scales, tensor_scale, dequantised float32 weights) in the packed layouts, made with the oracle."""
    lib = g.util_lib()
    rng = np.random.default_rng(seed)
    w = rng.standard_normal((N, K)).astype(np.float32)
    if dt == "w4a16":
        packed, sc = o.int4_quantise(w)
        return packed, sc, 1.0, o.int4_dequantise(packed, sc)
    if dt == "fp8":
        s = float(np.abs(w).max() / 448.0)
        q = o.e4m3_quantise(w, s)
        return q, None, s, o.e4m3_dequantise(q, s)
    kind = 8 if dt == "mxfp8" else 4
    q, sc = o.mx_quantise(w, kind)
    tiled = np.empty(lib.gemm_mx_tiled_scale_bytes(N, K), np.uint8)
    assert lib.gemm_mx_scales_to_tiled_host(_vp(sc), N, K, _vp(tiled)) == 0
    return q, tiled, 1.0, o.mx_dequantise(q, sc, kind)


@pytest.mark.parametrize("dt", ["fp8", "mxfp8", "w4a4", "w4a16"])
def test_weight_file_round_trip(tmp_path, dt):
    lib = g.util_lib()
    N, K = 200, 512
    elems, scales, ts, _ = _quantised_weights(dt, N, K, seed=5)
    path = str(tmp_path / f"w_{dt}.sm100qw").encode()
    assert lib.gemm_weight_file_write(path, DT[dt], N, K, ts, _vp(elems), _vp(scales) if scales is not None else None) == 0
    info = g.GemmWeightFileInfo()
    assert lib.gemm_weight_file_info(path, ctypes.byref(info)) == 0
    assert info.magic == b"SM100QW" and info.version == 1 and info.layout == 1
    assert (info.dtype, info.N, info.K) == (DT[dt], N, K)
    assert info.group == {"fp8": 0, "mxfp8": 32, "w4a4": 32, "w4a16": 128}[dt]
    assert info.elem_bytes == elems.nbytes == lib.gemm_packed_weight_bytes(DT[dt], N, K)
    assert info.scale_bytes == (scales.nbytes if scales is not None else 0)
    assert np.float32(info.tensor_scale) == np.float32(ts)
    e2 = np.empty(info.elem_bytes, np.uint8)
    s2 = np.empty(max(info.scale_bytes, 1), np.uint8)
    assert lib.gemm_weight_file_read(path, _vp(e2), e2.nbytes, _vp(s2), info.scale_bytes) == 0
    assert np.array_equal(e2, elems.view(np.uint8).ravel())
    if scales is not None:
        assert np.array_equal(s2, scales.view(np.uint8).ravel())
    # the payloads sit on 256-byte boundaries of the file
    raw = open(path, "rb").read()
    assert raw[256:256 + 16] == elems.view(np.uint8).ravel()[:16].tobytes()
    soff = 256 + (info.elem_bytes + 255) // 256 * 256
    assert len(raw) == (soff + info.scale_bytes if info.scale_bytes else 256 + info.elem_bytes)
    # failures: short buffer, flipped payload byte, foreign file, truncated file
    assert lib.gemm_weight_file_read(path, _vp(e2), e2.nbytes - 1, _vp(s2), info.scale_bytes) == -3
    bad = bytearray(raw); bad[300] ^= 0x10
    open(path, "wb").write(bytes(bad))
    assert lib.gemm_weight_file_read(path, _vp(e2), e2.nbytes, _vp(s2), info.scale_bytes) == -4
    open(path, "wb").write(b"not a weight file" * 32)
    assert lib.gemm_weight_file_info(path, ctypes.byref(info)) == -2
    open(path, "wb").write(raw[:100])
    assert lib.gemm_weight_file_info(path, ctypes.byref(info)) == 0 and lib.gemm_weight_file_read(path, _vp(e2), e2.nbytes, _vp(s2), s2.nbytes) == -2
    assert lib.gemm_weight_file_info(str(tmp_path / "missing").encode(), ctypes.byref(info)) == -1
    assert lib.gemm_weight_file_write(path, DT["w4a4"], N, 128, 1.0, _vp(elems), _vp(elems)) == -5      # K not a multiple of 256


def test_oracle_int4_quantiser_known_answers():
    w = np.zeros((2, 128), np.float32)
    w[0, :4] = [7.0, -7.0, 3.4, -3.6]              # amax 7 -> s = 1: q = 7, -7, 3, -4
    w[1, :3] = [0.5, -0.25, 0.124]                 # amax .5 -> s = bf16(.5/7) = 0.0712890625
    packed, sc = o.int4_quantise(w)
    assert o.bf16_bits_to_f32(sc)[0, 0] == 1.0
    assert list(packed[0, :2]) == [(7 & 0xf) | ((-7 & 0xf) << 4), 3 | ((-4 & 0xf) << 4)]
    s1 = float(o.bf16_bits_to_f32(sc)[1, 0])
    assert s1 == 0.0712890625
    exp = [int(np.clip(np.rint(np.float32(v) * (np.float32(1.0) / np.float32(s1))), -8, 7)) for v in (0.5, -0.25, 0.124, 0.0)]
    assert list(packed[1, :2]) == [(exp[0] & 0xf) | ((exp[1] & 0xf) << 4), (exp[2] & 0xf) | ((exp[3] & 0xf) << 4)]
    assert np.array_equal(o.int4_quantise(np.zeros((1, 128), np.float32))[1], o.f32_to_bf16_bits(np.ones((1, 1), np.float32)))


# ------------------------------------------------------------------------------------------ quantisation kernels (GPU)
def _bf16_matrix(rows, K, seed, spread=True):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, K)).astype(np.float32)
    if spread:      # block magnitudes over 2^-6 .. 2^5, some zero blocks, some huge values
        x *= np.exp2(rng.integers(-6, 6, (rows, K // 32))).repeat(32, axis=1).astype(np.float32)
        x[rng.integers(0, rows, 3), :32] = 0.0
        x[0, 0] = 3.0e38
        x[-1, -1] = -1e-38
    bits = o.f32_to_bf16_bits(x)
    return bits, o.bf16_bits_to_f32(bits)


@pytest.mark.gpu
@pytest.mark.parametrize("kind", [8, 4], ids=["mxfp8", "mxfp4"])
@pytest.mark.parametrize("shape", [(128, 128), (100, 256), (333, 1152), (1, 128), (4096, 4096)])
def test_mx_quantise_kernel_bit_exact(cuda_device, kind, shape):
    import torch

    rows, K = shape
    bits, xf = _bf16_matrix(rows, K, seed=rows + K + kind)
    q_ref, sc_ref = o.mx_quantise(xf, kind)
    lib = g.util_lib()
    xd = torch.from_numpy(bits.view(np.int16)).cuda()
    q = torch.full(q_ref.shape, 0xAA, dtype=torch.uint8, device="cuda")
    sf = torch.full((lib.gemm_mx_tiled_scale_bytes(rows, K),), 0xFF, dtype=torch.uint8, device="cuda")
    assert lib.gemm_quant_mx(xd.data_ptr(), q.data_ptr(), sf.data_ptr(), rows, K, kind, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert np.array_equal(sf.cpu().numpy(), tiled_scales_numpy(sc_ref)), "scales (atom layout, padding rows = 127)"
    assert np.array_equal(q.cpu().numpy(), q_ref), "elements"


@pytest.mark.gpu
@pytest.mark.parametrize("n", [8, 4096, 1000 * 8, 8192 * 8192 // 4])
def test_e4m3_per_tensor_quantise_kernel_bit_exact(cuda_device, n):
    import torch

    rng = np.random.default_rng(n)
    bits = o.f32_to_bf16_bits((rng.standard_normal(n) * 3).astype(np.float32))
    xf = o.bf16_bits_to_f32(bits)
    amax = np.float32(np.abs(xf).max())
    scale = np.float32(amax / np.float32(448.0))
    q_ref = o.e4m3_quantise(xf, float(scale))
    lib = g.util_lib()
    xd = torch.from_numpy(bits.view(np.int16)).cuda()
    q = torch.empty(n, dtype=torch.uint8, device="cuda")
    sc = torch.zeros(2, dtype=torch.float32, device="cuda")
    assert lib.gemm_quant_e4m3_per_tensor(xd.data_ptr(), q.data_ptr(), sc.data_ptr(), sc[1:].data_ptr(), n,
                                          torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    got = sc.cpu().numpy()
    assert got[1] == amax and got[0] == scale
    assert np.array_equal(q.cpu().numpy(), q_ref)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(16, 128), (200, 1024), (28672, 1024)])
def test_int4_quantise_kernel_bit_exact(cuda_device, shape):
    import torch

    N, K = shape
    bits, wf = _bf16_matrix(N, K, seed=N + K, spread=False)
    p_ref, s_ref = o.int4_quantise(wf)
    lib = g.util_lib()
    wd = torch.from_numpy(bits.view(np.int16)).cuda()
    p = torch.empty((N, K // 2), dtype=torch.uint8, device="cuda")
    s = torch.empty((N, K // 128), dtype=torch.int16, device="cuda")
    assert lib.gemm_quant_int4_g128(wd.data_ptr(), p.data_ptr(), s.data_ptr(), N, K, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert np.array_equal(s.cpu().numpy().view(np.uint16), s_ref)
    assert np.array_equal(p.cpu().numpy(), p_ref)


@pytest.mark.gpu
@pytest.mark.parametrize("dt", ["fp8", "mxfp8", "w4a4", "w4a16"])
def test_bf16_in_bf16_out_through_quantise_file_and_gemm(registry, cuda_device, tmp_path, dt):
    """End to end as a caller would run it: weights quantised offline and stored in a weight file; at run time
    the file's payloads go to the device as they are, the bf16 activations are quantised by the device kernel,
    and the GEMM's bf16 result must meet the variant's bar against the host oracle on the dequantised operands."""
    import torch

    from tests.gpu_util import run_ex, to_bits

    lib = g.util_lib()
    st = torch.cuda.current_stream().cuda_stream
    M, N, K = (16, 1024, 2048) if dt == "w4a16" else (256, 1024, 2048)
    elems, scales, ts, w_deq = _quantised_weights(dt, N, K, seed=11)
    path = str(tmp_path / "w.sm100qw").encode()
    assert lib.gemm_weight_file_write(path, DT[dt], N, K, ts, _vp(elems), _vp(scales) if scales is not None else None) == 0
    info = g.GemmWeightFileInfo()
    assert lib.gemm_weight_file_info(path, ctypes.byref(info)) == 0
    eh = torch.empty(info.elem_bytes, dtype=torch.uint8).pin_memory()
    sh = torch.empty(max(info.scale_bytes, 16), dtype=torch.uint8).pin_memory()
    assert lib.gemm_weight_file_read(path, eh.data_ptr(), eh.numel(), sh.data_ptr(), info.scale_bytes) == 0
    Wd, Sd = eh.cuda(), sh.cuda()
    xbits, xf = _bf16_matrix(M, K, seed=12, spread=False)
    Xd = torch.from_numpy(xbits.view(np.int16)).cuda()
    kw = {}
    if dt == "w4a16":
        Xq, x_deq = Xd.view(torch.bfloat16), xf
        kw = dict(w_scale=Sd, group_size=128)
    elif dt == "fp8":
        Xq = torch.empty((M, K), dtype=torch.uint8, device="cuda")
        sc = torch.zeros(2, dtype=torch.float32, device="cuda")
        assert lib.gemm_quant_e4m3_per_tensor(Xd.data_ptr(), Xq.data_ptr(), sc.data_ptr(), sc[1:].data_ptr(), M * K, st) == 0
        sx = float(sc.cpu()[0])
        x_deq = o.e4m3_dequantise(Xq.cpu().numpy(), sx)
        kw = dict(x_scale_f=sx, w_scale_f=float(info.tensor_scale))
    else:
        kind = 8 if dt == "mxfp8" else 4
        Xq = torch.empty((M, K if kind == 8 else K // 2), dtype=torch.uint8, device="cuda")
        SX = torch.empty(lib.gemm_mx_tiled_scale_bytes(M, K), dtype=torch.uint8, device="cuda")
        assert lib.gemm_quant_mx(Xd.data_ptr(), Xq.data_ptr(), SX.data_ptr(), M, K, kind, st) == 0
        torch.cuda.synchronize()
        sx_rows = np.empty((M, K // 32), np.uint8)
        assert lib.gemm_mx_scales_from_tiled_host(_vp(SX.cpu().numpy()), M, K, _vp(sx_rows)) == 0
        x_deq = o.mx_dequantise(Xq.cpu().numpy(), sx_rows, kind)
        kw = dict(x_scale=SX, w_scale=Sd)
    ref = o.gemm_f32(x_deq, w_deq)
    ran = 0
    for k in registry.kernels:
        if k.config.dt != dt or not k.can_run(M, N, K) or k.config.epi == 2:
            continue
        Y = to_bits(run_ex(k, M, N, K, Xq, Wd, **kw))
        if dt in ("fp8", "mxfp8"):
            r = o.check_dense(Y, ref, K, float(np.abs(x_deq).max()), float(np.abs(w_deq).max()))
        else:
            r = o.check_quantised(Y, ref)
        assert r["ok"], (k.config.name(), r)
        ran += 1
        if ran >= 4:
            break
    assert ran >= 1
