"""Python face of the CPU oracle (``oracle/host_ref.c``) plus the tolerance checks.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
benchmark's CPU-baseline leg.  The GPU library never imports this module.

The oracle restates the reference's FP32 check loop (reference src/bench.cu:77-84);
see the header of ``host_ref.c`` for how it is pinned.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` beside this file (gcc, OpenMP); returns its path."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "host_ref.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return so


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(so):
            build()
        L = ctypes.CDLL(so)
        vp, i32, sz, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_float
        L.oracle_num_threads.restype = i32
        L.oracle_gemm_bf16_rows.argtypes = [i32, i32, i32, vp, vp, vp, vp, i32, i32]
        L.oracle_gemm_bf16_rows.restype = i32
        L.oracle_gemm_f32_rows.argtypes = [i32, i32, vp, vp, vp, vp, i32, i32]
        L.oracle_gemm_bf16_rows_f64.argtypes = [i32, i32, vp, vp, vp, vp, i32]
        L.oracle_f32_to_bf16.argtypes = [vp, vp, sz]
        L.oracle_bf16_to_f32.argtypes = [vp, vp, sz]
        L.oracle_mx_quantise.argtypes = [vp, i32, i32, i32, vp, vp]
        L.oracle_mx_dequantise.argtypes = [vp, vp, i32, i32, i32, vp]
        L.oracle_e4m3_quantise.argtypes = [vp, sz, f32, vp]
        L.oracle_e4m3_dequantise.argtypes = [vp, sz, f32, vp]
        L.oracle_int4_dequantise.argtypes = [vp, vp, i32, i32, i32, vp]
        L.oracle_int4_quantise.argtypes = [vp, i32, i32, i32, vp, vp]
        L.oracle_set_threads.argtypes = [i32]
        for name in ("oracle_e4m3_to_f32", "oracle_e2m1_to_f32", "oracle_ue8m0_to_f32"):
            getattr(L, name).argtypes = [ctypes.c_uint8]
            getattr(L, name).restype = f32
        for name in ("oracle_f32_to_e4m3", "oracle_f32_to_e2m1"):
            getattr(L, name).argtypes = [f32]
            getattr(L, name).restype = ctypes.c_uint8
        L.oracle_ue8m0_for_block.argtypes = [f32, f32]
        L.oracle_ue8m0_for_block.restype = ctypes.c_uint8
        _LIB = L
    return _LIB


def _p(a: np.ndarray) -> ctypes.c_void_p:
    assert a.flags["C_CONTIGUOUS"]
    return ctypes.c_void_p(a.ctypes.data)


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_threads(n: int) -> None:
    """OpenMP threads the oracle uses from now on (torchrun exports OMP_NUM_THREADS=1 to its workers)."""
    lib().oracle_set_threads(int(n))


# ----------------------------------------------------------------------------- bf16 helpers
def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns (uint16), round-to-nearest-even."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().oracle_f32_to_bf16(_p(a), _p(out), a.size)
    return out


def bf16_bits_to_f32(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    return (a.astype(np.uint32) << 16).view(np.float32)


# ----------------------------------------------------------------------------- the GEMM oracle
def gemm_bf16(X: np.ndarray, W: np.ndarray, rows=None, strict: bool = False) -> np.ndarray:
    """FP32 ``X @ W.T`` of bf16 bit-pattern matrices X (MxK) and W (NxK).

    ``rows``: optional list of row indices of Y to compute (sampled check of large
    shapes); the result then has ``len(rows)`` rows.
    """
    X = np.ascontiguousarray(X, dtype=np.uint16)
    W = np.ascontiguousarray(W, dtype=np.uint16)
    M, K = X.shape
    N, K2 = W.shape
    assert K == K2
    if rows is None:
        r, n = None, M
    else:
        r = np.ascontiguousarray(rows, dtype=np.int32)
        n = r.size
    Y = np.empty((n, N), dtype=np.float32)
    rc = lib().oracle_gemm_bf16_rows(M, N, K, _p(X), _p(W), _p(Y), _p(r) if r is not None else None, n, int(strict))
    if rc != 0:
        raise MemoryError("oracle scratch allocation failed")
    return Y


def gemm_bf16_f64(X: np.ndarray, W: np.ndarray, rows=None) -> np.ndarray:
    """Diagnostic: ``X @ W.T`` of bf16 bit-pattern matrices with the products summed in double
    (float64 result).  Resolves what an FP32-summed reference cannot at very large K."""
    X = np.ascontiguousarray(X, dtype=np.uint16)
    W = np.ascontiguousarray(W, dtype=np.uint16)
    M, K = X.shape
    N = W.shape[0]
    r = None if rows is None else np.ascontiguousarray(rows, dtype=np.int32)
    n = M if r is None else r.size
    Y = np.empty((n, N), dtype=np.float64)
    lib().oracle_gemm_bf16_rows_f64(N, K, _p(X), _p(W), _p(Y), _p(r) if r is not None else None, n)
    return Y


def gemm_f32(X: np.ndarray, W: np.ndarray, rows=None, strict: bool = False) -> np.ndarray:
    """FP32 ``X @ W.T`` of float32 matrices (the dequantise-then-GEMM oracle's second half)."""
    X = np.ascontiguousarray(X, dtype=np.float32)
    W = np.ascontiguousarray(W, dtype=np.float32)
    M, K = X.shape
    N = W.shape[0]
    if rows is None:
        r, n = None, M
    else:
        r = np.ascontiguousarray(rows, dtype=np.int32)
        n = r.size
    Y = np.empty((n, N), dtype=np.float32)
    lib().oracle_gemm_f32_rows(N, K, _p(X), _p(W), _p(Y), _p(r) if r is not None else None, n, int(strict))
    return Y


# ----------------------------------------------------------------------------- quantisers
def mx_quantise(a: np.ndarray, kind: int):
    """Row-major RxK float32 -> (elements, ue8m0 scales[R, K/32]); kind 8 = e4m3, 4 = e2m1 (2/byte)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    R, K = a.shape
    assert K % 32 == 0
    elems = np.empty((R, K if kind == 8 else K // 2), dtype=np.uint8)
    scales = np.empty((R, K // 32), dtype=np.uint8)
    lib().oracle_mx_quantise(_p(a), R, K, kind, _p(elems), _p(scales))
    return elems, scales


def mx_dequantise(elems: np.ndarray, scales: np.ndarray, kind: int) -> np.ndarray:
    R = elems.shape[0]
    K = scales.shape[1] * 32
    out = np.empty((R, K), dtype=np.float32)
    lib().oracle_mx_dequantise(_p(np.ascontiguousarray(elems)), _p(np.ascontiguousarray(scales)), R, K, kind, _p(out))
    return out


def e4m3_quantise(a: np.ndarray, scale: float) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint8)
    lib().oracle_e4m3_quantise(_p(a), a.size, ctypes.c_float(scale), _p(out))
    return out


def e4m3_dequantise(q: np.ndarray, scale: float) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.uint8)
    out = np.empty(q.shape, dtype=np.float32)
    lib().oracle_e4m3_dequantise(_p(q), q.size, ctypes.c_float(scale), _p(out))
    return out


def int4_pack(q: np.ndarray) -> np.ndarray:
    """int8 values in [-8,7], shape (N,K) -> (N,K/2) bytes, low nibble = even k."""
    q = np.asarray(q, dtype=np.int8)
    u = (q.astype(np.int16) & 0xF).astype(np.uint8)
    return np.ascontiguousarray(u[:, 0::2] | (u[:, 1::2] << 4))


def int4_quantise(w: np.ndarray, group: int = 128):
    """float32 (N,K) -> (packed int4 (N,K/2), bf16 scale bits (N,K/group)): s = bf16(max|w|/7), q = clamp(rint(w * (1/s)))."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    N, K = w.shape
    assert K % group == 0
    packed = np.empty((N, K // 2), dtype=np.uint8)
    scales = np.empty((N, K // group), dtype=np.uint16)
    lib().oracle_int4_quantise(_p(w), N, K, group, _p(packed), _p(scales))
    return packed, scales


def int4_dequantise(packed: np.ndarray, scales_bf16: np.ndarray, group: int = 128) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    scales_bf16 = np.ascontiguousarray(scales_bf16, dtype=np.uint16)
    N, K = packed.shape[0], packed.shape[1] * 2
    out = np.empty((N, K), dtype=np.float32)
    lib().oracle_int4_dequantise(_p(packed), _p(scales_bf16), N, K, group, _p(out))
    return out


# ----------------------------------------------------------------------------- tolerances
def bf16_ulp(ref: np.ndarray) -> np.ndarray:
    """Spacing of bf16 numbers around each FP32 reference value (8 significand bits)."""
    a = np.abs(ref.astype(np.float32))
    e = np.floor(np.log2(np.maximum(a, np.float32(2.0 ** -126))))
    return np.exp2(e - 7).astype(np.float32)


def check_dense(y_bits: np.ndarray, ref: np.ndarray, K: int, max_x: float, max_w: float) -> dict:
    """The BF16 / FP8 bar: (i) max|y-ref| <= 1e-2*sqrt(K)*max|x|*max|w|;
    (ii) >= 99.9 % of outputs are one of the two bf16 neighbours of the FP32 reference."""
    y = bf16_bits_to_f32(y_bits).astype(np.float64)
    r = ref.astype(np.float64)          # an FP32 reference, or the float64 one of gemm_bf16_f64
    err = np.abs(y - r)
    bound = 1e-2 * np.sqrt(K) * max_x * max_w
    inside = err <= bf16_ulp(ref).astype(np.float64)
    frac = float(inside.mean()) if inside.size else 1.0
    return {
        "max_abs_err": float(err.max()) if err.size else 0.0,
        "bound": float(bound),
        "frac_within_bf16_rounding": frac,
        "ok": bool((err.max() if err.size else 0.0) <= bound and frac >= 0.999),
    }


def check_quantised(y_bits: np.ndarray, ref: np.ndarray) -> dict:
    """The quantised-variant bar: ||float(Y) - bf16_rn(ref)||_F / ||ref||_F <= 1e-3.
    The raw figure against the unrounded reference is returned as well; output
    rounding alone puts its floor near 1.7e-3, so it cannot be the bar."""
    y = bf16_bits_to_f32(y_bits).astype(np.float64)
    r = ref.astype(np.float64)
    rr = bf16_bits_to_f32(f32_to_bf16_bits(ref)).astype(np.float64)
    nr = np.linalg.norm(r)
    rel_rounded = float(np.linalg.norm(y - rr) / nr) if nr > 0 else 0.0
    rel_raw = float(np.linalg.norm(y - r) / nr) if nr > 0 else 0.0
    return {"rel_fro_vs_rounded_ref": rel_rounded, "rel_fro_raw": rel_raw, "ok": rel_rounded <= 1e-3}


def ref_check(y_bits: np.ndarray, ref: np.ndarray) -> float:
    """The reference's own (loose) metric: max |y-ref| / max(|y|,|ref|,1)  (src/bench.cu:97-112);
    the reference passes a kernel when this is < 0.1 (src/bench.cu:427)."""
    y = bf16_bits_to_f32(y_bits)
    d = np.abs(y - ref) / np.maximum(np.maximum(np.abs(y), np.abs(ref)), 1.0)
    return float(d.max()) if d.size else 0.0


# ----------------------------------------------------------------------------- seeded inputs
def make_inputs(M: int, N: int, K: int, seed: int, dist: str = "uniform"):
    """Seeded bf16 inputs as uint16 bit patterns.

    dist: "uniform"  X,W ~ U[-1,1]              (reference src/bench.cu:36-43 value range)
          "normal"   X,W ~ N(0,1)
          "decode"   X ~ N(0,1), W ~ N(0,1/K)
    """
    rng = np.random.default_rng(seed)
    if dist == "uniform":
        x = rng.uniform(-1, 1, (M, K)).astype(np.float32)
        w = rng.uniform(-1, 1, (N, K)).astype(np.float32)
    elif dist == "normal":
        x = rng.standard_normal((M, K), dtype=np.float32)
        w = rng.standard_normal((N, K), dtype=np.float32)
    elif dist == "decode":
        x = rng.standard_normal((M, K), dtype=np.float32)
        w = rng.standard_normal((N, K), dtype=np.float32) / np.float32(np.sqrt(K))
    else:
        raise ValueError(dist)
    return f32_to_bf16_bits(x), f32_to_bf16_bits(w)
