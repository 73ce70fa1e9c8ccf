"""Enumerates the kernel configurations to build, one shared library each.

Same job as the reference's scripts/gen_configs.py:7-50 (which enumerates
BM,BN in {64,128} x stages x consumer warpgroups x warp tilings x split-K under a
shared-memory cap for the mma.sync kernel), re-derived for the tcgen05 design:

  dt       bf16 | fp8 | mxfp8 | w4a16 | w4a4
  bm       rows of X per tile = 128 * cg * (row blocks per CTA): 128 (one CTA), 256 (CTA pair, cta_group::2),
           512 (CTA pair with two 128-row blocks per CTA: one B tile feeds two MMAs)
  bn       multiple of 16 up to 256  (UMMA N; two FP32 accumulator buffers need 2*bn <= 512 TMEM columns;
           the TMA-store epilogue needs a multiple of 64)
  bk       one 128-byte swizzle span of K per stage: 64 bf16, 128 fp8, 256 fp4 elements
           (w4a16: 64 = dequantised tiles in shared memory, 128 = dequantised scale groups in tensor memory)
  s        TMA ring stages, bounded by the 227 KB of shared memory one CTA may use
  cg       CTA group (1 | 2)
  sk       split-K factor (FP32 partials + reduce kernel); 0 = stream-K: the tiles x k-blocks work is
           cut into one equal contiguous range per CTA, partial tiles are summed by a fix-up kernel
  ab       operand swap for small M (W rows on the 128 accumulator lanes)
  e        epilogue: 0 = registers -> global, 1 = swizzled shared memory -> TMA store,
           2 = registers -> global with the fused output transform act(alpha*acc + beta*C + bias), bf16 or e4m3 out

Name:  <dt>_bm<bm>_bn<bn>_bk<bk>_s<s>_cg<cg>_sk<sk>_ab<ab>_e<e>

The warp-tiling fields of the reference's names (cwg, wm, wn) have no meaning for a
single-thread-issued MMA and are gone.
"""
from __future__ import annotations

import argparse
import re
from dataclasses import dataclass

MAX_SMEM = 232448  # 227 KB: cudaDevAttrMaxSharedMemoryPerBlockOptin on sm_100
DT_IDS = {"bf16": 0, "fp8": 1, "mxfp8": 2, "w4a16": 3, "w4a4": 4}
ELEM_BITS = {"bf16": 16, "fp8": 8, "mxfp8": 8, "w4a16": 16, "w4a4": 4}

_NAME_RE = re.compile(r"^(bf16|fp8|mxfp8|w4a16|w4a4)_bm(\d+)_bn(\d+)_bk(\d+)_s(\d+)_cg(\d+)_sk(\d+)_ab(\d+)_e(\d+)$")


@dataclass(frozen=True)
class GemmConfig:
    """Mirror of the reference's GemmConfig (src/gemm_config.h:24-55) for the new space."""

    dt: str
    bm: int
    bn: int
    bk: int
    num_stages: int
    cg: int
    split_k: int
    swap_ab: int
    epi: int

    @property
    def mb(self) -> int:
        """128-row blocks of X per CTA."""
        return max(1, self.bm // (128 * self.cg))

    def name(self) -> str:
        return (f"{self.dt}_bm{self.bm}_bn{self.bn}_bk{self.bk}_s{self.num_stages}_cg{self.cg}"
                f"_sk{self.split_k}_ab{self.swap_ab}_e{self.epi}")

    @staticmethod
    def parse(s: str):
        m = _NAME_RE.match(s)
        if not m:
            return None
        g = m.groups()
        return GemmConfig(g[0], *(int(v) for v in g[1:]))

    def smem_bytes(self) -> int:
        """Dynamic shared memory of the kernel; must equal the traits' SMEM_ALLOC."""
        if self.dt == "w4a16" and self.bk == 128:   # W4A16TmemTraits: load ring only (16 KB packed + 4 activation boxes per stage); s = group slots in TMEM
            load_stage = 128 * 128 + 4 * (-(-self.bn * 128 // 1024) * 1024)
            load_stages = min(8, 200 * 1024 // load_stage)
            return load_stages * load_stage + (2 * load_stages + 3 * self.num_stages) * 8 + 16 + 1024
        if self.dt == "w4a16":   # W4A16Traits: group ring (s slots of two bf16 tiles) + load ring (16 KB packed + 4 activation boxes)
            load_stage = 128 * 128 + 4 * (-(-self.bn * 128 // 1024) * 1024)
            load_stages = min(4, (224 * 1024 - self.num_stages * 2 * 128 * 128) // load_stage)
            return (self.num_stages * 2 * 128 * 128 + load_stages * load_stage
                    + (2 * load_stages + 3 * self.num_stages) * 8 + 16 + 1024)
        a = 128 * 128 * self.mb
        b = (self.bn // self.cg) * 128
        # block-scaled kinds stage one 512-byte scale atom per 128 rows and 128 K-elements
        k_atoms = self.bk // 128 if self.dt in ("mxfp8", "w4a4") else 0
        n_atoms = -(-self.bn // 128)
        sf = k_atoms * (1 + n_atoms) * 512
        epi = 0 if self.split_k > 1 else self.epi
        barriers = (2 * self.num_stages + 4 + (4 if k_atoms else 0)) * 8 + 16     # block-scaled: + scale set ready / free
        sf_ring = -(-self.num_stages * sf // 1024) * 1024
        ring = self.num_stages * (a + b) + sf_ring + barriers + 1024
        # one accumulator stage (two do not fit in the 512 TMEM columns beside the scale factors): four staging buffers if they fit
        acc_stages = 2 if 2 * self.mb * (-(-self.bn // 32) * 32) + 2 * k_atoms * (1 + n_atoms) * 4 <= 512 else 1
        bufs = 4 if acc_stages == 1 and ring + 4 * 128 * 64 * 2 <= MAX_SMEM else 2
        staging = bufs * 128 * 64 * 2 if epi == 1 else 0
        return ring + staging

    def is_valid_for(self, M: int, N: int, K: int) -> bool:
        """The plugin's own gemm_can_run, restated (reference: src/gemm_config.h:34-38)."""
        if M <= 0 or N <= 0 or K <= 0:
            return False
        if self.dt == "w4a16":   # decode kernel: M fits the padded UMMA N, whole 128-element scale groups
            return M <= self.bn and N % 8 == 0 and K % 128 == 0
        if (K * ELEM_BITS[self.dt]) % 128 != 0 or N % 8 != 0:
            return False
        if self.dt in ("mxfp8", "w4a4") and K % self.bk != 0:
            return False
        if self.split_k > 1:
            if K % self.bk != 0 or (K // self.bk) % self.split_k != 0:
                return False
        return True

    def defines(self) -> list[str]:
        return [f"-DGEMM_DT={DT_IDS[self.dt]}", f"-DGEMM_BN={self.bn}", f"-DGEMM_STAGES={self.num_stages}",
                f"-DGEMM_CG={self.cg}", f"-DGEMM_SK={self.split_k}", f"-DGEMM_AB={self.swap_ab}",
                f"-DGEMM_EPI={self.epi}", f"-DGEMM_MB={self.mb}", f"-DGEMM_BK={self.bk}", f"-DGEMM_NAME={self.name()}"]


_PEAK_TFLOPS = {"bf16": 2250.0, "fp8": 4500.0, "mxfp8": 4500.0, "w4a16": 2250.0, "w4a4": 9000.0}


def heuristic_ms(c: GemmConfig, M: int, N: int, K: int, sms: int = 148) -> float:
    """Modelled time of one launch, the same arithmetic as heuristic_ms in csrc/gemm_config.h (see there)."""
    import math

    hbm, sm_stream, launch_us = 6.5e12, 9.0e10, 4.0
    eb = ELEM_BITS[c.dt] / 8.0
    wb = 0.5 if c.dt == "w4a16" else eb
    alg_bytes = float(M) * K * eb + float(N) * K * wb + float(M) * N * 2.0
    if c.dt == "w4a16":
        return alg_bytes / hbm * 1e3 + c.bn * 1e-4 - c.num_stages * 1e-6
    slots = float(sms // c.cg)
    tiles = math.ceil(M / c.bm) * float(math.ceil(N / c.bn))
    eff_m = 1.0 if c.bm >= 512 else 0.92 if c.bm >= 256 else 0.80
    eff_n = 0.55 + 0.45 * min(c.bn, 256) / 256.0
    slot_flops = _PEAK_TFLOPS[c.dt] * 1e12 * c.cg / sms * eff_m * eff_n
    split = float(c.split_k) if c.split_k > 1 else 1.0
    unit_flops = 2.0 * c.bm * c.bn * float(K) / split
    unit_bytes = (float(c.bm) * eb + float(c.bn) * wb) * float(K) / split
    slot_bw = sm_stream * c.cg
    if c.split_k == 0:
        share = tiles / (tiles if tiles < slots else slots)
        tt, tm = share * unit_flops / slot_flops, share * unit_bytes / slot_bw
        t = (tt if tt > tm else tm) * (tiles / slots if tiles < slots else 1.0) + 4.0 * slots * c.bm * c.bn * 4.0 / 5.0e12 + 4e-6
    else:
        rounds = float(math.ceil(tiles * split / slots))
        if c.bm == 256 * c.cg and c.split_k == 1 and tiles > slots:
            rest = tiles - math.floor(tiles / slots) * slots
            if rest > 0 and 2.0 * rest <= slots:
                rounds -= 0.5
        tt, tm = unit_flops / slot_flops, unit_bytes / slot_bw
        t = rounds * (tt if tt > tm else tm)
        if c.split_k > 1:
            t += (4.0 * split + 2.0) * M * N / 5.0e12 + 3e-6
    if c.epi == 0 and M >= 1024:
        t *= 1.03
    floor_t = alg_bytes / hbm
    if t < floor_t:
        t = floor_t
    t -= c.num_stages * 1e-9
    return (t + launch_us * 1e-6) * 1e3


def heuristic_config(configs, dt: str, M: int, N: int, K: int, sms: int = 148):
    """The configuration of `configs` with the smallest modelled time for the shape, for callers that do not
    autotune (the reference skips shapes that are missing from its cache, src/bench.cu:455-458)."""
    best = None
    for c in configs:
        if c.dt != dt or c.epi == 2 or not c.is_valid_for(M, N, K):
            continue
        key = (heuristic_ms(c, M, N, K, sms), c.name())
        if best is None or key < best[0]:
            best = (key, c)
    return best[1] if best else None


def max_stages(dt: str, bn: int, cg: int, sk: int, epi: int, cap: int = MAX_SMEM) -> int:
    bk = 128 * 8 // ELEM_BITS[dt]
    s = 12
    while s >= 2 and GemmConfig(dt, 128 * cg, bn, bk, s, cg, sk, 0, epi).smem_bytes() > cap:
        s -= 1
    return s


def generate_block_scaled(dt: str, max_smem: int) -> list[GemmConfig]:
    """MXFP8 / MX-FP4: BN a multiple of the 128-row scale atom; one CTA or a CTA pair per tile."""
    bk = 128 * 8 // ELEM_BITS[dt]
    out = []
    for bn in (128, 256):
        for epi in (1, 0):
            out.append(GemmConfig(dt, 256, bn, bk, min(max_stages(dt, bn, 2, 1, epi, max_smem), 8), 2, 1, 0, epi))
    # 256 x 256 on a CTA pair has one accumulator stage: one ring stage fewer leaves room for four staging buffers,
    # so the accumulator is drained without waiting for TMA stores
    out.append(GemmConfig(dt, 256, 256, bk, 4, 2, 1, 0, 1))
    for bn in (128, 256):
        for epi in (1, 0):
            out.append(GemmConfig(dt, 128, bn, bk, min(max_stages(dt, bn, 1, 1, epi, max_smem), 8), 1, 1, 0, epi))
        for sk in (2, 4, 0):
            out.append(GemmConfig(dt, 128, bn, bk, min(max_stages(dt, bn, 1, sk, 0, max_smem), 8), 1, sk, 0, 0))
    return out


def generate_w4a16(max_smem: int) -> list[GemmConfig]:
    """W4A16 decode kernels: operands swapped (ab=1), bn = M padded to 16/32/64/128, stream-K work split.
    bk128: dequantised weights go through tensor memory (A operand of the MMA read from TMEM), s = group slots;
    bk64: dequantised weights go through shared memory, s = group ring slots."""
    out = []
    for mpad, slots in ((16, 6), (32, 5), (64, 4), (128, 2)):
        c = GemmConfig("w4a16", 128, mpad, 128, slots, 1, 0, 1, 0)
        if c.smem_bytes() <= max_smem:
            out.append(c)
    for mpad, stage_opts in ((16, (3, 4)), (32, (3, 4))):
        for st in stage_opts:
            c = GemmConfig("w4a16", 128, mpad, 64, st, 1, 0, 1, 0)
            if c.smem_bytes() <= max_smem:
                out.append(c)
    return out


def generate_configs(max_smem: int = MAX_SMEM, dts=("bf16", "fp8", "mxfp8", "w4a4", "w4a16")) -> list[GemmConfig]:
    out: list[GemmConfig] = []
    for dt in dts:
        if dt == "w4a16":
            out += generate_w4a16(max_smem)
            continue
        if dt in ("mxfp8", "w4a4"):
            out += generate_block_scaled(dt, max_smem)
            continue
        if dt not in ("bf16", "fp8"):
            continue  # W4A16 has its own kernel and generator
        bk = 128 * 8 // ELEM_BITS[dt]
        for cg in (1, 2):
            for bn in (64, 128, 192, 256):
                for epi in (1, 0):
                    top = max_stages(dt, bn, cg, 1, epi, max_smem)
                    stage_opts = sorted({min(top, 8), min(top, 4)}, reverse=True)
                    if epi == 0:
                        stage_opts = stage_opts[:1]
                    for s in stage_opts:
                        if s >= 2:
                            out.append(GemmConfig(dt, 128 * cg, bn, bk, s, cg, 1, 0, epi))
        # two row blocks per CTA (512 x 256 tiles on a CTA pair): a quarter less operand traffic per flop, for large shapes
        for s in (4, 3):
            c = GemmConfig(dt, 512, 256, bk, s, 2, 1, 0, 1)
            if c.smem_bytes() <= max_smem:
                out.append(c)
        # fused output transform (bias, alpha/beta, activation, e4m3 output with amax): one small and one large tile
        for cg, bn in ((1, 128), (2, 256)):
            out.append(GemmConfig(dt, 128 * cg, bn, bk, min(max_stages(dt, bn, cg, 1, 2, max_smem), 8), cg, 1, 0, 2))
        # split-K: for shapes with too few output tiles to fill 148 SMs (decode, M <= 128)
        for cg, bn in ((1, 64), (1, 128), (1, 256), (2, 128), (2, 256)):
            for sk in (2, 4, 7, 8, 16):
                s = min(max_stages(dt, bn, cg, sk, 0, max_smem), 8)
                out.append(GemmConfig(dt, 128 * cg, bn, bk, s, cg, sk, 0, 0))
        # tile widths that fill 148 SMs in one wave for the decode shapes (N = 4096 with 4 K slices, N = 28672)
        out.append(GemmConfig(dt, 128, 112, bk, min(max_stages(dt, 112, 1, 4, 0, max_smem), 10), 1, 4, 0, 0))
        for bn in (208, 224):
            out.append(GemmConfig(dt, 128, bn, bk, min(max_stages(dt, bn, 1, 1, 0, max_smem), 10), 1, 1, 0, 0))
        # stream-K: every SM streams the same number of bytes whatever the tile count
        for cg, bn in ((1, 64), (1, 128), (1, 192), (1, 256), (2, 128), (2, 256)):
            s = min(max_stages(dt, bn, cg, 0, 0, max_smem), 10)
            out.append(GemmConfig(dt, 128 * cg, bn, bk, s, cg, 0, 0, 0))
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--max-smem-kb", type=int, default=MAX_SMEM // 1024)
    ap.add_argument("--dt", default="bf16,fp8,mxfp8,w4a4,w4a16")
    ap.add_argument("--output", default=None,
                    help="write a CMake fragment  set(GEMM_CONFIGS \"name|DT|BN|STAGES|CG|SK|AB|EPI|MB|BK;...\")  instead of printing names "
                         "(the reference's generator does the same for its CMakeLists.txt, scripts/gen_configs.py:52-75)")
    args = ap.parse_args()
    configs = generate_configs(args.max_smem_kb * 1024, tuple(args.dt.split(",")))
    if args.output:
        import os

        os.makedirs(os.path.dirname(os.path.abspath(args.output)), exist_ok=True)
        items = [f"{c.name()}|{DT_IDS[c.dt]}|{c.bn}|{c.num_stages}|{c.cg}|{c.split_k}|{c.swap_ab}|{c.epi}|{c.mb}|{c.bk}" for c in configs]
        with open(args.output, "w") as f:
            f.write("# generated by gen_configs.py -- one entry per kernel plugin\n")
            f.write('set(GEMM_CONFIGS "' + ";".join(items) + '")\n')
        print(f"wrote {len(items)} configurations to {args.output}")
        return
    for c in configs:
        print(c.name())


if __name__ == "__main__":
    main()
