// W4A16 for decode shapes (M <= 128): Y = X * dequant(W)^T with W signed int4 (two per byte
// along K, low nibble = even k) and one bf16 scale per 128 K-elements of each weight row.
// The reference has no quantised path; this kernel has no counterpart there.
//
// Operands are swapped: the 128 weight rows of a tile are the MMA's A operand (one TMEM lane
// per weight row n) and the activations are the B operand (UMMA N = M padded to MPAD), so the
// tensor work scales with M, not with a padded 128, and -- the point of the design -- the
// group scale s[n][g] is a per-LANE scalar.  Weights are dequantised in shared memory to bf16
// holding the EXACT integers -8..7; each 128-element group is multiplied out on the tensor core
// into its own TMEM buffer and folded into per-thread FP32 totals as total[m] += s[n][g] * acc[m].
// (Folding the scale into a bf16 weight instead, bf16(q*s), rounds every weight and misses
// the 1e-3 accuracy bar.)
//
// Warps:  0 TMA producer | 1 and 3 MMA issuers (even / odd groups) | 2 TMEM alloc
//         4-7  fold + epilogue: thread r owns weight row r (TMEM lane r)
//         8..  dequantiser teams of 4 warps: thread r of a team converts row r of the tile; with two
//              teams each takes one of a group's two k-blocks
// The unit of the pipeline is one scale GROUP (128 K-elements = two 64-element bf16 tiles): a single
// thread's tcgen05 instructions cost ~60-80 cycles each to issue and these MMAs are tiny, so issuing is
// the scarce resource: 8 MMAs and one commit per group, and two issuer threads taking groups in turn.
// LOAD ring, stages of 256 K-elements (two groups): one TMA box of 128 rows x 128 bytes of packed
// int4 plus the four 64-element activation boxes of the same K range.
//   landed[p]  TMA bytes of load stage p                    -> dequantisers
//   lfree[p]   tcgen05.commit by the issuer of each of the stage's groups (2 arrivals) -> producer
// GROUP ring, slot = two bf16 tiles in shared memory + one accumulator buffer in TMEM:
//   ready[s]   both tiles of the group written              -> MMA issuer
//   gdone[s]   tcgen05.commit after the group's 8 MMAs      -> fold warps (accumulator complete) and
//              dequantisers (tiles may be overwritten)
//   gempty[s]  fold warps have read the accumulator         -> MMA issuer
//
// Work is cut stream-K fashion in units of one group: every CTA gets the same number of
// groups; a range that does not cover a tile's whole K leaves an FP32 partial [m][128] in the
// CTA's slot, summed by streamk_reduce_kernel<128,128>.
#pragma once
#include "bf16_gemm.cuh"

namespace sm100 {

struct W4A16Params {
    int M, N, K;
    int num_n_tiles;
    int num_groups;          // K / 128
    bf16 *Y;
    float *workspace;        // stream-K slots: [2 * grid][128 (m)][128 (n)] FP32
    const bf16 *scales;      // [N][K/128]
    uint32_t *status;
};

template <int MPAD_, int STAGES_>
struct W4A16Traits {
    static constexpr int MPAD = MPAD_;                 // UMMA N: M rounded up (16, 32, 64 or 128)
    static constexpr int STAGES = STAGES_;             // group ring slots
    static constexpr int TILE_N = 128;                 // weight rows per tile = TMEM lanes
    static constexpr int BK = 64;                      // K elements per bf16 tile (128 bytes)
    static constexpr int GROUP_KB = 2;                 // bf16 tiles per scale group (128 / 64)
    static constexpr int LOAD_GROUPS = 2;              // groups per load stage (256 K-elements = 128 packed bytes per row)
    static constexpr int LOAD_KB = LOAD_GROUPS * GROUP_KB;
    static constexpr int PACKED_BYTES = TILE_N * 128;  // 16 KB of int4 per load stage
    static constexpr int X_BYTES = MPAD_ * 128;        // one activation box
    static constexpr int X_STRIDE = (X_BYTES + 1023) / 1024 * 1024;
    static constexpr int LOAD_STAGE_SMEM = PACKED_BYTES + LOAD_KB * X_STRIDE;
    static constexpr int LOAD_TX_BYTES = PACKED_BYTES + LOAD_KB * X_BYTES;
    static constexpr int A_BYTES = TILE_N * 128;       // one dequantised bf16 tile
    static constexpr int SLOT_BYTES = GROUP_KB * A_BYTES;
    static constexpr int LOAD_STAGES_FIT = (224 * 1024 - STAGES_ * SLOT_BYTES) / LOAD_STAGE_SMEM;
    static constexpr int LOAD_STAGES = LOAD_STAGES_FIT > 4 ? 4 : LOAD_STAGES_FIT;
    static constexpr int NUM_BARRIERS = 2 * LOAD_STAGES + 3 * STAGES_;
    static constexpr int SMEM_BYTES = STAGES_ * SLOT_BYTES + LOAD_STAGES * LOAD_STAGE_SMEM + NUM_BARRIERS * 8 + 16;
    static constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;
    static constexpr int ACC_COLS = STAGES_ * MPAD_;   // one accumulator buffer per group slot
    static constexpr int TMEM_COLS = ACC_COLS <= 32 ? 32 : ACC_COLS <= 64 ? 64 : ACC_COLS <= 128 ? 128 : ACC_COLS <= 256 ? 256 : 512;
    static constexpr int TEAMS = MPAD_ <= 64 ? 2 : 1;   // dequantiser teams (the M = 128 fold needs the registers)
    static constexpr int THREADS = 256 + 128 * TEAMS;
    static_assert(MPAD_ == 16 || MPAD_ == 32 || MPAD_ == 64 || MPAD_ == 128, "padded M is 16, 32, 64 or 128");
    static_assert(STAGES_ >= 2 && ACC_COLS <= 512, "2 or more group slots whose accumulators fit in TMEM");
    static_assert(LOAD_STAGES >= 2, "at least two load stages must fit");
    static_assert(SMEM_ALLOC <= 232448, "exceeds the shared memory of one CTA");
};

// 8 signed int4 (two's complement nibbles, nibble j = element j) -> four bf16x2 holding the exact
// integers.  Flipping a nibble's top bit turns it into q+8 in 0..15; placed in the mantissa of 128.0
// (0x4300) that is the bf16 number 128+(q+8) exactly, and subtracting 136 leaves q.  One lop3 does the
// mask, the flip and the merge: with m = 0x000f000f and c = 0x43084308 it computes m ? (y ^ c) : c
// per bit (truth table 0x6A), where c carries both the exponent and the bit to flip.
__device__ __forceinline__ void int4x8_to_bf16x8(uint32_t w, uint32_t (&out)[4])
{
    const uint32_t w4 = w >> 4;
    const uint32_t bias = 0x43084308u;   // bf16x2 {136, 136}
#pragma unroll
    for (int j = 0; j < 4; j++) {
        // byte j of w -> bits [0,8), byte j of w4 -> bits [16,24): low halves hold nibbles 2j and 2j+1
        uint32_t sel = 0x4040u | (uint32_t)j | ((uint32_t)(4 + j) << 8);   // bytes: [j of w, filler, j of w4, filler]
        uint32_t y;
        asm("prmt.b32 %0, %1, %2, %3;" : "=r"(y) : "r"(w), "r"(w4), "r"(sel));
        asm("lop3.b32 %0, %1, 0x000f000f, 0x43084308, 0x6A;" : "=r"(y) : "r"(y));
        asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(out[j]) : "r"(y), "r"(bias));
    }
}

template <class T>
__global__ void __launch_bounds__(T::THREADS, 1)
w4a16_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, const W4A16Params p)
{
    constexpr int STAGES = T::STAGES;
    constexpr int MPAD = T::MPAD;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (smem_base - raw_addr);
    constexpr int LSTAGES = T::LOAD_STAGES;
    const uint32_t a_base = smem_base;                                   // group ring: two bf16 tiles per slot
    const uint32_t ld_base = a_base + STAGES * T::SLOT_BYTES;            // load ring: [packed 16 KB][4 activation boxes]
    const uint32_t bar_base = ld_base + LSTAGES * T::LOAD_STAGE_SMEM;
    auto landed_bar = [&](int s) { return bar_base + 8u * s; };
    auto lfree_bar = [&](int s) { return bar_base + 8u * (LSTAGES + s); };
    auto ready_bar = [&](int s) { return bar_base + 8u * (2 * LSTAGES + s); };
    auto gdone_bar = [&](int s) { return bar_base + 8u * (2 * LSTAGES + STAGES + s); };
    auto gempty_bar = [&](int s) { return bar_base + 8u * (2 * LSTAGES + 2 * STAGES + s); };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + (bar_base - smem_base) + 8u * T::NUM_BARRIERS);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    const uint8_t *ld_ptr = smem + (ld_base - smem_base);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int cta = blockIdx.x, num_ctas = gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < LSTAGES; s++) {
            mbar_init(landed_bar(s), 1);
            mbar_init(lfree_bar(s), 2);              // one commit per group of the stage (a lone group commits twice)
        }
        for (int s = 0; s < STAGES; s++) {
            mbar_init(ready_bar(s), 4 * T::TEAMS);   // one arrival per dequantiser warp
            mbar_init(gdone_bar(s), 1);
            mbar_init(gempty_bar(s), 4);             // one arrival per fold warp
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
        prefetch_tensormap(&tmap_x);
        prefetch_tensormap(&tmap_w);
    }
    if (warp == 2) {
        tmem_alloc<1>(smem_u32(tmem_slot), T::TMEM_COLS);
        tmem_relinquish<1>();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the fix-up kernel may be scheduled

    // stream-K over (tile, group) units: the schedule of bf16_gemm.cuh with one unit = one group
    GemmParams sp;
    sp.num_m_blocks = 1;
    sp.num_n_blocks = p.num_n_tiles;
    sp.num_k_blocks = p.num_groups;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int pcount = 0;                            // load stages issued so far
            WorkSched<0> sched(cta, num_ctas, sp);
            WorkItem w;
            bool ok = true;
            while (ok && sched.next(w)) {
                const int n0 = w.tile * T::TILE_N;
                for (int g = 0; g < w.kb_count; g += T::LOAD_GROUPS, pcount++) {
                    const int ps = pcount % LSTAGES;
                    if (!mbar_wait(lfree_bar(ps), (((uint32_t)(pcount / LSTAGES)) & 1u) ^ 1u, abort_flag, p.status, ST_TIMEOUT_PRODUCER, ps)) {
                        ok = false;
                        break;
                    }
                    const int k0 = (w.kb_begin + g) * 128;
                    const uint32_t dst = ld_base + ps * T::LOAD_STAGE_SMEM;
                    // always the full 256-element box: past an item's end it brings unused (or zero-filled) data
                    mbar_arrive_expect_tx(landed_bar(ps), T::LOAD_TX_BYTES);
                    tma_load_2d(dst, &tmap_w, landed_bar(ps), k0 / 2, n0);
#pragma unroll
                    for (int j = 0; j < T::LOAD_KB; j++)
                        tma_load_2d(dst + T::PACKED_BYTES + j * T::X_STRIDE, &tmap_x, landed_bar(ps), k0 + j * T::BK, 0);
                }
            }
        }
    } else if (warp == 1 || warp == 3) {
        // ------------------------------------------------------------------ MMA issuers
        if (lane == 0) {
            const int issuer = warp == 3 ? 1 : 0;
            const uint32_t instr = make_idesc(UMMA_BF16, UMMA_BF16, 128, MPAD);
            int gcount = 0;          // groups issued so far: ring slot gcount % STAGES
            int pcount = 0;          // load stages consumed so far
            WorkSched<0> sched(cta, num_ctas, sp);
            WorkItem w;
            bool ok = true;
            while (ok && sched.next(w)) {
                for (int g = 0; g < w.kb_count; g++, gcount++) {
                    const int slot = gcount % STAGES;
                    const uint32_t sphase = ((uint32_t)(gcount / STAGES)) & 1u;
                    const int ps = pcount % LSTAGES;
                    const int jg = g % T::LOAD_GROUPS;             // group inside its load stage
                    const bool stage_ends = (jg == T::LOAD_GROUPS - 1 || g == w.kb_count - 1);
                    if ((gcount & 1) != issuer) {
                        if (stage_ends) pcount++;
                        continue;
                    }
                    if (!mbar_wait(gempty_bar(slot), sphase ^ 1u, abort_flag, p.status, ST_TIMEOUT_MMA_ACC, slot)) { ok = false; break; }
                    // ready[slot] also tells that the load stage has landed: the dequantisers waited for it
                    if (!mbar_wait(ready_bar(slot), sphase, abort_flag, p.status, ST_TIMEOUT_MMA_FULL, slot)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + (uint32_t)(slot * MPAD);
                    const uint64_t a_desc = make_smem_desc_k128(a_base + slot * T::SLOT_BYTES);
                    const uint64_t b_desc = make_smem_desc_k128(ld_base + ps * T::LOAD_STAGE_SMEM + T::PACKED_BYTES + jg * T::GROUP_KB * T::X_STRIDE);
#pragma unroll
                    for (int t = 0; t < T::GROUP_KB; t++) {
                        // tile t of the group: next 16 KB of the slot, next activation box
                        const uint64_t at = a_desc + (uint64_t)((t * T::A_BYTES) >> 4), bt = b_desc + (uint64_t)((t * T::X_STRIDE) >> 4);
#pragma unroll
                        for (int k = 0; k < 4; k++)
                            umma_f16<1>(d_tmem, advance_desc_k(at, k), advance_desc_k(bt, k), instr, (t > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(gdone_bar(slot));
                    umma_commit(lfree_bar(ps));
                    if (stage_ends && jg == 0) umma_commit(lfree_bar(ps));   // the stage's only group: stand in for the missing one
                    if (stage_ends) pcount++;
                }
            }
        }
    } else if (warp >= 8) {
        // ------------------------------------------------------------------ dequantisers
        const int team = (warp - 8) >> 2;
        const int r = ((warp - 8) & 3) * 32 + lane;   // row of the tile this thread converts
        int gcount = 0, pcount = 0;
        WorkSched<0> sched(cta, num_ctas, sp);
        WorkItem w;
        bool ok = true;
        while (ok && sched.next(w)) {
            for (int g = 0; g < w.kb_count; g++, gcount++) {
                const int slot = gcount % STAGES;
                const uint32_t sphase = ((uint32_t)(gcount / STAGES)) & 1u;
                const int ps = pcount % LSTAGES;
                const uint32_t pphase = ((uint32_t)(pcount / LSTAGES)) & 1u;
                const int jg = g % T::LOAD_GROUPS;
                if (jg == T::LOAD_GROUPS - 1 || g == w.kb_count - 1) pcount++;
                if (!mbar_wait(landed_bar(ps), pphase, abort_flag, p.status, ST_TIMEOUT_DEQUANT, ps)) { ok = false; break; }
                // the slot's tiles are free once the MMAs of the group that used it last are done
                if (!mbar_wait(gdone_bar(slot), sphase ^ 1u, abort_flag, p.status, ST_TIMEOUT_DEQUANT, 16 + slot)) { ok = false; break; }
                // packed row r: 128 bytes, 128B-swizzled by the TMA; k-block j of the stage is its 16-byte chunks 2j, 2j+1
                const uint8_t *row = ld_ptr + ps * T::LOAD_STAGE_SMEM + r * 128;
#pragma unroll
                for (int t = team; t < T::GROUP_KB; t += T::TEAMS) {
                    const int j = jg * T::GROUP_KB + t;
                    const uint4 lo = *reinterpret_cast<const uint4 *>(row + (((2 * j) ^ (r & 7)) << 4));
                    const uint4 hi = *reinterpret_cast<const uint4 *>(row + (((2 * j + 1) ^ (r & 7)) << 4));
                    const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                    const uint32_t dst_row = a_base + slot * T::SLOT_BYTES + t * T::A_BYTES + r * 128;
#pragma unroll
                    for (int c = 0; c < 8; c++) {                  // 16-byte chunk c = k 8c .. 8c+7
                        uint32_t o[4];
                        int4x8_to_bf16x8(words[c], o);
                        st_shared_v4(dst_row + (uint32_t)((c ^ (r & 7)) << 4), o[0], o[1], o[2], o[3]);
                    }
                }
                fence_proxy_async_smem();                         // make the writes visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(ready_bar(slot));
            }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ fold + epilogue
        const int q = warp - 4;                        // == warp % 4: the TMEM lane quarter of this warp
        const int r = q * 32 + lane;                   // weight row inside the tile = TMEM lane
        int gcount = 0;
        WorkSched<0> sched(cta, num_ctas, sp);
        WorkItem w;
        bool ok = true;
        while (ok && sched.next(w)) {
            const int n = w.tile * T::TILE_N + r;
            const bf16 *srow = p.scales + (size_t)(n < p.N ? n : 0) * p.num_groups + w.kb_begin;
            float total[MPAD];
#pragma unroll
            for (int m = 0; m < MPAD; m++) total[m] = 0.f;
            // scales are fetched eight groups ahead of their use: a load issued where it is needed would put
            // an L2 round trip into every group and throttle the whole pipeline
            float s_cur[8], s_nxt[8];
#pragma unroll
            for (int i = 0; i < 8; i++) s_cur[i] = i < w.kb_count ? __bfloat162float(srow[i]) : 0.f;
            for (int g0 = 0; g0 < w.kb_count && ok; g0 += 8) {
#pragma unroll
                for (int i = 0; i < 8; i++) s_nxt[i] = g0 + 8 + i < w.kb_count ? __bfloat162float(srow[g0 + 8 + i]) : 0.f;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    if (g0 + i >= w.kb_count) break;
                    const int b = gcount % STAGES;
                    const float s = s_cur[i];
                    if (!mbar_wait(gdone_bar(b), (uint32_t)(gcount / STAGES) & 1u, abort_flag, p.status, ST_TIMEOUT_EPILOGUE, b)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * MPAD);
#pragma unroll
                    for (int c0 = 0; c0 < MPAD; c0 += 16) {
                        uint32_t v[16];
                        tmem_ld_32x16(t_row + (uint32_t)c0, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 16; e++) total[c0 + e] = fmaf(s, __uint_as_float(v[e]), total[c0 + e]);
                    }
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(gempty_bar(b));
                    gcount++;
                }
#pragma unroll
                for (int i = 0; i < 8; i++) s_cur[i] = s_nxt[i];
            }
            if (!ok) break;
            if (w.part < 0) {
                if (n < p.N) {
#pragma unroll
                    for (int m = 0; m < MPAD; m++)
                        if (m < p.M) p.Y[(size_t)m * p.N + n] = __float2bfloat16_rn(total[m]);
                }
            } else {
                float *slot = p.workspace + (size_t)(2 * cta + w.part) * 128 * 128 + r;
#pragma unroll
                for (int m = 0; m < MPAD; m++) slot[m * 128] = total[m];
            }
        }
    }

    __syncwarp();
    if (*abort_flag) {
        for (int i = 0; i < 64; i++) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc<1>(tmem_base, T::TMEM_COLS);
    }
}

template <class T>
struct W4A16Launcher {
    static bool can_run(int M, int N, int K)
    {
        return M >= 1 && M <= T::MPAD && N >= 8 && N % 8 == 0 && K >= 128 && K % 128 == 0;
    }
    static size_t workspace_bytes(int, int, int) { return (size_t)2 * STREAMK_MAX_CTAS * 128 * 128 * sizeof(float); }

    static int run(int M, int N, int K, const void *X, const void *Wq, void *Y, const void *scales, int group_size, float *workspace,
                   size_t workspace_bytes_given, int sm_limit, cudaStream_t stream)
    {
        if (!can_run(M, N, K)) return set_error(GEMM_ERR_SHAPE, "shape %dx%dx%d not supported (M <= %d, K a multiple of 128)", M, N, K, T::MPAD);
        if (group_size != 128) return set_error(GEMM_ERR_ARG, "W4A16 scale groups are 128 K-elements, got %d", group_size);
        if (!X || !Wq || !Y || !scales) return set_error(GEMM_ERR_ARG, "null operand or scale pointer");
        if (!workspace) return set_error(GEMM_ERR_WORKSPACE, "this configuration needs a workspace");
        if (workspace_bytes_given != 0 && workspace_bytes_given < workspace_bytes(M, N, K))
            return set_error(GEMM_ERR_WORKSPACE, "workspace has %zu bytes, %zu needed", workspace_bytes_given, workspace_bytes(M, N, K));
        DeviceInfo *dev = nullptr;
        int rc = device_info(&dev);
        if (rc != GEMM_OK) return rc;
        static std::atomic<bool> attr_set[MAX_DEVICES];
        int devid = 0;
        SM100_CUDA_TRY(cudaGetDevice(&devid));
        if (!attr_set[devid].load(std::memory_order_acquire)) {
            SM100_CUDA_TRY(cudaFuncSetAttribute(w4a16_gemm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_ALLOC));
            attr_set[devid].store(true, std::memory_order_release);
        }
        CUtensorMap tx, tw;
        rc = make_tmap_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, X, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, 64, T::MPAD, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != GEMM_OK) return rc;
        rc = make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, Wq, (uint64_t)K / 2, (uint64_t)N, (uint64_t)K / 2, 128, T::TILE_N, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != GEMM_OK) return rc;
        W4A16Params p;
        p.M = M; p.N = N; p.K = K;
        p.num_n_tiles = (N + T::TILE_N - 1) / T::TILE_N;
        p.num_groups = K / 128;
        p.Y = static_cast<bf16 *>(Y);
        p.workspace = workspace;
        p.scales = static_cast<const bf16 *>(scales);
        p.status = dev->status;
        long long units = (long long)p.num_n_tiles * p.num_groups;
        int grid = dev->sm_count;
        if (sm_limit > 0 && sm_limit < grid) grid = sm_limit;
        if (grid > STREAMK_MAX_CTAS) grid = STREAMK_MAX_CTAS;
        if (grid > units) grid = (int)units;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(T::THREADS);
        cfg.dynamicSmemBytes = T::SMEM_ALLOC;
        cfg.stream = stream;
        SM100_CUDA_TRY(cudaLaunchKernelEx(&cfg, w4a16_gemm_kernel<T>, tx, tw, p));
        int parts = 1;
        while (parts < 32 && p.num_n_tiles * parts < 2 * dev->sm_count) parts *= 2;
        cudaLaunchConfig_t rcfg = dependent_launch_config(p.num_n_tiles * parts, 256, stream);
        SM100_CUDA_TRY(cudaLaunchKernelEx(&rcfg, streamk_reduce_kernel<128, 128>, (const float *)workspace, static_cast<bf16 *>(Y), M, N, 1,
                                          p.num_n_tiles, 1, p.num_groups, grid, parts, 1.0f));
        return GEMM_OK;
    }
};

}  // namespace sm100
