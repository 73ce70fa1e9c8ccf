"""Generates the committed fixtures in this directory.  Run from the repo root:

    python tests/golden/make_golden.py

The reference project has no golden vectors of its own (no tests/, no known-answer files);
what it does have is a seeded input generator and an FP32 check loop.  The fixtures therefore
hold (a) inputs produced exactly the way the reference produces them -- glibc srand(42) +
rand(), X then W, value = float(rand())/RAND_MAX*2-1 rounded to bf16 (reference
src/bench.cu:36-43, 196-198) -- and (b) expected outputs computed here WITHOUT the oracle:
exact float64 arithmetic on the bf16 values (numpy), which is the mathematically exact
result the FP32 loop approximates.  The element-format tables are computed from the format
definitions (OCP OFP8 e4m3, OCP MX e2m1 / ue8m0) with numpy only.
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def bf16_rne(a: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bits, round to nearest even, numpy only."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def bf16_to_f64(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def reference_rand_inputs(M: int, N: int, K: int):
    libc = ctypes.CDLL("libc.so.6")
    libc.srand(42)
    RAND_MAX = 2147483647

    def draw(n):
        out = np.empty(n, dtype=np.float32)
        for i in range(n):
            # float(rand()) / RAND_MAX is evaluated in float, the *2.0-1.0 in double
            v = np.float32(libc.rand()) / np.float32(RAND_MAX)
            out[i] = np.float32(np.float64(v) * 2.0 - 1.0)
        return out

    x = draw(M * K).reshape(M, K)
    w = draw(N * K).reshape(N, K)
    return bf16_rne(x), bf16_rne(w)


def e4m3_table() -> np.ndarray:
    t = np.empty(256, dtype=np.float32)
    for v in range(256):
        s, e, m = v >> 7, (v >> 3) & 15, v & 7
        if e == 15 and m == 7:
            r = np.nan
        elif e == 0:
            r = m / 8.0 * 2.0 ** -6
        else:
            r = (1 + m / 8.0) * 2.0 ** (e - 7)
        t[v] = -r if s else r
    return t


def main() -> None:
    # 1. reference-style random case, exact float64 result
    M, N, K = 48, 40, 96
    X, W = reference_rand_inputs(M, N, K)
    Y = bf16_to_f64(X) @ bf16_to_f64(W).T
    np.savez_compressed(os.path.join(HERE, "ref_rand_48x40x96.npz"), X=X, W=W, Y=Y)

    # 2. exactly representable case: small integers, every partial sum exact in FP32
    rng = np.random.default_rng(7)
    Xi = rng.integers(-4, 5, (33, 72)).astype(np.float32)
    Wi = rng.integers(-4, 5, (24, 72)).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "exact_int_33x24x72.npz"), X=bf16_rne(Xi), W=bf16_rne(Wi),
                        Y=(Xi.astype(np.float64) @ Wi.astype(np.float64).T))

    # 3. element formats
    e2m1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)
    ue8m0 = np.array([2.0 ** (v - 127) if v < 255 else np.nan for v in range(256)], dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, "formats.npz"), e4m3=e4m3_table(), e2m1=e2m1, ue8m0=ue8m0)
    print("fixtures written to", HERE)


if __name__ == "__main__":
    main()
