"""CPU tests of the oracle itself: it must agree with the committed fixtures (exact float64
results on reference-style seeded inputs), with hand-computable known answers, and its
quantisers must round-trip.  No GPU."""
import os

import numpy as np
import pytest

from oracle import oracle as o

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_golden_reference_style_inputs():
    d = np.load(os.path.join(GOLD, "ref_rand_48x40x96.npz"))
    for strict in (False, True):
        Y = o.gemm_bf16(d["X"], d["W"], strict=strict)
        # FP32 accumulation of 96 products of magnitude <= 1: error far below 96 * 2^-24 * 96
        assert np.abs(Y - d["Y"]).max() < 5e-5
    # and the reference's own loose metric (src/bench.cu:97-112) is ~0
    assert o.ref_check(o.f32_to_bf16_bits(d["Y"].astype(np.float32)), o.gemm_bf16(d["X"], d["W"])) < 0.01


def test_golden_exact_integers():
    d = np.load(os.path.join(GOLD, "exact_int_33x24x72.npz"))
    for strict in (False, True):
        Y = o.gemm_bf16(d["X"], d["W"], strict=strict)
        assert np.array_equal(Y.astype(np.float64), d["Y"])  # bit-exact: every partial sum is an integer < 2^24


def test_strict_order_matches_python_loop():
    # the reference loop (src/bench.cu:77-84), k ascending in FP32, restated in pure Python on a tiny case
    X, W = o.make_inputs(3, 4, 37, seed=5)
    xf, wf = o.bf16_bits_to_f32(X), o.bf16_bits_to_f32(W)
    exp = np.zeros((3, 4), np.float32)
    for r in range(3):
        for c in range(4):
            acc = np.float32(0)
            for k in range(37):
                acc = np.float32(acc + np.float32(xf[r, k] * wf[c, k]))
            exp[r, c] = acc
    got = o.gemm_bf16(X, W, strict=True)
    # gcc may contract a*b+c into an FMA (as nvcc does for the reference kernel under
    # --use_fast_math); allow one FP32 ulp per step of slack but demand near-equality
    assert np.abs(got - exp).max() <= 37 * np.finfo(np.float32).eps * np.abs(exp).max()


def test_rows_subset_and_empty():
    X, W = o.make_inputs(20, 16, 64, seed=1)
    full = o.gemm_bf16(X, W)
    rows = [19, 0, 7]
    assert np.array_equal(o.gemm_bf16(X, W, rows=rows), full[rows])
    assert o.gemm_bf16(X, W, rows=[]).shape == (0, 16)


def test_bf16_roundtrip_and_rne():
    a = np.array([1.0, 1.00390625, 1.01171875, -3.140625, 0.0, 65280.0], dtype=np.float32)
    b = o.f32_to_bf16_bits(a)
    back = o.bf16_bits_to_f32(b)
    assert back[0] == 1.0 and back[3] == -3.140625 and back[5] == 65280.0
    assert back[1] == 1.0            # 1 + 2^-8 is a tie: rounds to even (1.0)
    assert back[2] == 1.015625       # 1 + 3*2^-8 is a tie: rounds to even (1 + 2^-6)
    x = np.random.default_rng(0).standard_normal(10000).astype(np.float32)
    err = np.abs(o.bf16_bits_to_f32(o.f32_to_bf16_bits(x)) - x)
    assert (err <= np.abs(x) * 2.0 ** -8).all()


def test_format_tables_match_fixtures():
    f = np.load(os.path.join(GOLD, "formats.npz"))
    L = o.lib()
    got = np.array([L.oracle_e4m3_to_f32(v) for v in range(256)], dtype=np.float32)
    assert np.array_equal(np.nan_to_num(got, nan=-999), np.nan_to_num(f["e4m3"], nan=-999))
    got = np.array([L.oracle_e2m1_to_f32(v) for v in range(16)], dtype=np.float32)
    assert np.array_equal(got, f["e2m1"])
    got = np.array([L.oracle_ue8m0_to_f32(v) for v in range(256)], dtype=np.float64)
    assert np.array_equal(np.nan_to_num(got, nan=-1), np.nan_to_num(f["ue8m0"], nan=-1))


def test_e4m3_encode_is_nearest_and_saturates():
    f = np.load(os.path.join(GOLD, "formats.npz"))["e4m3"]
    L = o.lib()
    for v in range(256):                      # every finite code encodes to itself
        if not np.isnan(f[v]) and not (v == 0x80):
            assert L.oracle_f32_to_e4m3(float(f[v])) == v
    finite = np.sort(f[~np.isnan(f)])
    rng = np.random.default_rng(3)
    for x in rng.uniform(-460, 460, 2000).astype(np.float32):
        q = L.oracle_e4m3_to_f32(L.oracle_f32_to_e4m3(float(x)))
        assert abs(q - x) <= np.abs(finite - x).min() + 1e-12
    assert L.oracle_e4m3_to_f32(L.oracle_f32_to_e4m3(1e6)) == 448.0
    assert L.oracle_e4m3_to_f32(L.oracle_f32_to_e4m3(-1e6)) == -448.0


@pytest.mark.parametrize("kind,emax", [(8, 448.0), (4, 6.0)])
def test_mx_quantise_roundtrip(kind, emax):
    rng = np.random.default_rng(11)
    a = (rng.standard_normal((8, 128)) * rng.uniform(0.01, 30, (8, 1))).astype(np.float32)
    a[0, :32] = 0.0                           # an all-zero block
    elems, scales = o.mx_quantise(a, kind)
    assert scales.shape == (8, 4)
    back = o.mx_dequantise(elems, scales, kind)
    assert np.array_equal(back[0, :32], np.zeros(32, np.float32))
    # block scale is the smallest power of two that makes the block fit the element range
    for r in range(8):
        for b in range(4):
            blk = a[r, b * 32:(b + 1) * 32]
            amax = np.abs(blk).max()
            if amax == 0:
                continue
            s = 2.0 ** (int(scales[r, b]) - 127)
            assert amax / s <= emax and amax / (s / 2) > emax
    rel = np.abs(back - a).max() / np.abs(a).max()
    assert rel < (0.07 if kind == 8 else 0.3)
    # idempotence: quantising the dequantised values changes nothing
    e2, s2 = o.mx_quantise(back, kind)
    assert np.array_equal(o.mx_dequantise(e2, s2, kind), back)


def test_int4_pack_dequantise():
    rng = np.random.default_rng(2)
    q = rng.integers(-8, 8, (6, 256)).astype(np.int8)
    sc = o.f32_to_bf16_bits(rng.uniform(0.5, 2, (6, 2)).astype(np.float32) / 8)
    w = o.int4_dequantise(o.int4_pack(q), sc, group=128)
    exp = q.astype(np.float32) * np.repeat(o.bf16_bits_to_f32(sc), 128, axis=1)
    assert np.array_equal(w, exp)


def test_tolerance_checkers():
    X, W = o.make_inputs(32, 32, 512, seed=0)
    ref = o.gemm_bf16(X, W)
    good = o.f32_to_bf16_bits(ref)
    r = o.check_dense(good, ref, 512, 1.0, 1.0)
    assert r["ok"] and r["frac_within_bf16_rounding"] == 1.0
    bad = good.copy()
    bad[:4] += 3                               # 3 ulps off in 12.5 % of the outputs
    assert not o.check_dense(bad, ref, 512, 1.0, 1.0)["ok"]
    q = o.check_quantised(good, ref)
    assert q["ok"] and q["rel_fro_vs_rounded_ref"] == 0.0 and 0 < q["rel_fro_raw"] < 3e-3
