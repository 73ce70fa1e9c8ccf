// W4A16 for decode shapes (M <= 128), second kernel family: the dequantised weights go from registers
// straight into TENSOR MEMORY and the MMA reads its A operand from there (tcgen05.mma with A in TMEM),
// so the only shared-memory traffic left is the packed int4 bytes coming in and the small activation tile.
//
// Why: in the shared-memory family (w4a16_gemm.cuh) every weight byte pair is written to shared memory as
// bf16 and read back by the tensor core.  At N = 28672, K = 8192 that is 2 x 6.3 MB through one SM's shared
// memory port (128 B/clk), 50 us worth, against 15 us for the HBM stream that actually bounds the problem.
// TMEM has its own write path (tcgen05.st, one lane per thread) and the tensor core reads it directly.
//
// Same mathematics as the other family (exact-integer bf16 weights, one MMA group per 128-element scale
// group into its own accumulator, FP32 fold  total[m] += s[n][g] * acc[m]), same operand swap (128 weight
// rows = TMEM lanes, UMMA N = M padded), same stream-K work split and fix-up kernel.
//
// The SM's instruction issue is the scarce resource here (the int4 -> bf16 conversion alone is ~1300 warp
// instructions per group), so every wait backs off with nanosleep instead of polling back to back: a polling
// warp takes issue slots from the dequantisers that share its scheduler.
// Warps:  0 TMA producer | 1 MMA issuer | 2 TMEM alloc | 3 idle
//         4 .. 4+4*FOLD-1   fold + epilogue: thread r of a group owns weight row r (TMEM lane r) and the group's
//                           share of the M columns
//         then TEAMS x 4    dequantiser teams: thread r converts row r of HALF a scale group (32 packed bytes ->
//                           32 registers of bf16 pairs -> one tcgen05.st into half of the group slot's A columns);
//                           teams take the half-groups in turn
// TMEM columns: SLOTS accumulators of MPAD columns, then SLOTS A buffers of 64 columns (128 bf16 per lane).
// LOAD ring, stages of 256 K-elements (two groups): one TMA box of 128 rows x 128 packed bytes plus the four
// 64-element activation boxes of the same K range.
//   landed[p]  TMA bytes of load stage p                       -> dequantisers
//   lfree[p]   tcgen05.commit after each of the stage's groups  -> producer (2 arrivals)
//   ready[s]   the group's A operand is in TMEM                 -> MMA issuer
//   gdone[s]   tcgen05.commit after the group's 8 MMAs          -> fold warps (accumulator complete) and
//              dequantisers (A columns may be overwritten)
//   gempty[s]  fold warps have read the accumulator             -> MMA issuer
#pragma once
#include "bf16_gemm.cuh"
#include "w4a16_gemm.cuh"

namespace sm100 {

// 32 lanes x 32 consecutive 32-bit columns, registers -> TMEM: thread t of the warp writes lane (base_lane + t)
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
          "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
          "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// 8 signed int4 (two's complement nibbles, nibble j = element j) -> four bf16x2 holding q / 64 exactly, with seven
// integer-pipe instructions instead of nine.  Two lop3 mask the even and the odd nibbles of the word and flip their
// sign bits (q + 8 in 0..15, one per byte); a prmt per output puts two of those bytes into the low bytes of the two
// halves and zeroes above them (selector bit 3 replicates the byte's sign bit, which is clear): as bf16 that is the
// subnormal (q + 8) * 2^-133, and fma.rn.bf16x2 with 2^127 and -1/8 turns it into (q + 8) / 64 - 8 / 64.  bf16
// arithmetic keeps subnormal inputs (no flush-to-zero for this type), and every step is exact.  The fold multiplies
// the totals by 64 at the end: a power of two, so the result is the one the integer-valued form gives, bit for bit.
__device__ __forceinline__ void int4x8_to_bf16x8_div64(uint32_t w, uint32_t (&out)[4])
{
    uint32_t even, odd;
    asm("lop3.b32 %0, %1, 0x0f0f0f0f, 0x08080808, 0x6A;" : "=r"(even) : "r"(w));
    asm("lop3.b32 %0, %1, 0x0f0f0f0f, 0x08080808, 0x6A;" : "=r"(odd) : "r"(w >> 4));
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const uint32_t sel = (uint32_t)j | ((8u | (uint32_t)j) << 4) | ((uint32_t)(4 + j) << 8) | ((8u | (uint32_t)(4 + j)) << 12);
        uint32_t y;
        asm("prmt.b32 %0, %1, %2, %3;" : "=r"(y) : "r"(even), "r"(odd), "r"(sel));
        asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(out[j]) : "r"(y), "r"(0x7f007f00u), "r"(0xbe00be00u));   // * 2^127 - 1/8
    }
}
constexpr float W4A16_TMEM_UNSCALE = 64.0f;

__device__ __forceinline__ void tmem_st_wait()
{
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// D[tmem] (+)= A[tmem] * B[smem desc]; bf16 inputs, A K-major in TMEM (lane = row, 32-bit column = two K-elements)
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

template <int MPAD_, int SLOTS_>
struct W4A16TmemTraits {
    static constexpr int MPAD = MPAD_;                 // UMMA N: M rounded up (16, 32, 64 or 128)
    static constexpr int STAGES = SLOTS_;              // group slots (accumulator + A buffer in TMEM)
    static constexpr int TILE_N = 128;                 // weight rows per tile = TMEM lanes
    static constexpr int LOAD_GROUPS = 2;              // scale groups per load stage (256 K-elements = 128 packed bytes per row)
    static constexpr int LOAD_KB = 4;                  // 64-element activation boxes per load stage
    static constexpr int PACKED_BYTES = TILE_N * 128;  // 16 KB of int4 per load stage
    static constexpr int X_BYTES = MPAD_ * 128;        // one activation box
    static constexpr int X_STRIDE = X_BYTES;           // the boxes of a stage are contiguous (one request brings all four)
    static_assert(X_BYTES % 1024 == 0, "an activation box is a whole number of 8-row swizzle groups");
    static constexpr int LOAD_STAGE_SMEM = PACKED_BYTES + LOAD_KB * X_STRIDE;
    static constexpr int LOAD_TX_BYTES = PACKED_BYTES + LOAD_KB * X_BYTES;
    static constexpr int LOAD_STAGES_FIT = (200 * 1024) / LOAD_STAGE_SMEM;
    static constexpr int LOAD_STAGES = LOAD_STAGES_FIT > 8 ? 8 : LOAD_STAGES_FIT;
    static constexpr int NUM_BARRIERS = 2 * LOAD_STAGES + 3 * SLOTS_;
    static constexpr int SMEM_BYTES = LOAD_STAGES * LOAD_STAGE_SMEM + NUM_BARRIERS * 8 + 16;
    static constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;
    static constexpr int A_COLS = 64;                  // 128 bf16 of one lane = 64 32-bit columns
    static constexpr int A_BASE = SLOTS_ * MPAD_;      // A buffers sit behind the accumulators
    static constexpr int TMEM_USED = SLOTS_ * (MPAD_ + A_COLS);
    static constexpr int TMEM_COLS = TMEM_USED <= 32 ? 32 : TMEM_USED <= 64 ? 64 : TMEM_USED <= 128 ? 128 : TMEM_USED <= 256 ? 256 : 512;
    static constexpr int FOLD = MPAD_ > 64 ? 2 : 1;    // fold groups: each keeps MPAD / FOLD running totals per thread
    static constexpr int FCOLS = MPAD_ / FOLD;
    // dequantiser teams of four warps; the unit of work is HALF a scale group (64 K-elements of 128 rows: 32 registers
    // per thread), dealt to the teams in turn.  A single warp sustains well under one instruction per clock on the
    // dependent prmt / lop3 / sub chains of the conversion, so the way to more conversion throughput is more warps.
    static constexpr int TEAMS = MPAD_ > 64 ? 2 : MPAD_ > 32 ? 3 : 4;   // fewer where the fold warps need the registers
    static constexpr int THREADS = 128 + 128 * FOLD + 128 * TEAMS;
    static constexpr int REGS_EVEN = 65536 / THREADS / 8 * 8;                      // what the launch bound gives every thread
    static constexpr int LEAN_REGS = 40;                                           // setmaxnreg target of warps 0-3
    static constexpr int DEQ_REGS = REGS_EVEN < 80 ? REGS_EVEN : 80;               // and of the dequantiser warps (32 output registers each)
    // setmaxnreg moves registers inside the CTA's own allocation (THREADS x REGS_EVEN), not the SM's whole file: an
    // increase that the decreases of the other roles do not cover would wait for ever
    static constexpr int POOL = THREADS * REGS_EVEN;
    static constexpr int FOLD_REGS_FIT = (POOL - 128 * LEAN_REGS - 128 * TEAMS * DEQ_REGS) / (128 * FOLD) / 8 * 8;
    static constexpr int FOLD_REGS = FOLD_REGS_FIT > 168 ? 168 : FOLD_REGS_FIT;    // setmaxnreg target of the fold warps
    static_assert(128 * LEAN_REGS + 128 * TEAMS * DEQ_REGS + 128 * FOLD * FOLD_REGS <= POOL && FOLD_REGS >= REGS_EVEN,
                  "the roles' register targets must fit in what the CTA was launched with");
    static_assert(MPAD_ == 16 || MPAD_ == 32 || MPAD_ == 64 || MPAD_ == 128, "padded M is 16, 32, 64 or 128");
    static_assert(SLOTS_ >= 2 && TMEM_USED <= 512, "2 or more group slots that fit in TMEM");
    static_assert(LOAD_STAGES >= 2, "at least two load stages must fit");
    static_assert(SMEM_ALLOC <= 232448, "exceeds the shared memory of one CTA");
};

template <class T>
__global__ void __launch_bounds__(T::THREADS, 1)
w4a16_tmem_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, const W4A16Params p)
{
    constexpr int SLOTS = T::STAGES;
    constexpr int MPAD = T::MPAD;
    constexpr int LSTAGES = T::LOAD_STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (smem_base - raw_addr);
    const uint32_t ld_base = smem_base;                                   // load ring: [packed 16 KB][4 activation boxes]
    const uint32_t bar_base = ld_base + LSTAGES * T::LOAD_STAGE_SMEM;
    auto landed_bar = [&](int s) { return bar_base + 8u * s; };
    auto lfree_bar = [&](int s) { return bar_base + 8u * (LSTAGES + s); };
    auto ready_bar = [&](int s) { return bar_base + 8u * (2 * LSTAGES + s); };
    auto gdone_bar = [&](int s) { return bar_base + 8u * (2 * LSTAGES + SLOTS + s); };
    auto gempty_bar = [&](int s) { return bar_base + 8u * (2 * LSTAGES + 2 * SLOTS + s); };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + (bar_base - smem_base) + 8u * T::NUM_BARRIERS);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    const uint8_t *ld_ptr = smem;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int cta = blockIdx.x, num_ctas = gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < LSTAGES; s++) {
            mbar_init(landed_bar(s), 1);
            mbar_init(lfree_bar(s), 2);              // one commit per group of the stage (a lone group commits twice)
        }
        for (int s = 0; s < SLOTS; s++) {
            mbar_init(ready_bar(s), 8);              // one arrival per warp of the two teams that converted the group's halves
            mbar_init(gdone_bar(s), 1);
            mbar_init(gempty_bar(s), 4 * T::FOLD);   // one arrival per fold warp
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

    // Registers follow the roles: the producer / issuer / allocator warps give most of theirs back, the fold warps
    // (MPAD / FOLD running totals per thread) take more than the even share.  Warps 0-3, each fold group and each
    // dequantiser team are whole warpgroups, as setmaxnreg wants.
    if (warp < 4) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(T::LEAN_REGS));
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
                    if (!mbar_wait(lfree_bar(ps), (((uint32_t)(pcount / LSTAGES)) & 1u) ^ 1u, abort_flag, p.status, ST_TIMEOUT_PRODUCER, ps, 256)) {
                        ok = false;
                        break;
                    }
                    const int k0 = (w.kb_begin + g) * 128;
                    const uint32_t dst = ld_base + ps * T::LOAD_STAGE_SMEM;
                    // always the full 256-element box: past an item's end it brings unused (or zero-filled) data
                    mbar_arrive_expect_tx(landed_bar(ps), T::LOAD_TX_BYTES);
                    tma_load_2d(dst, &tmap_w, landed_bar(ps), k0 / 2, n0);
                    // the four 64-element activation boxes of this K range in one request (chunked view of X)
                    tma_load_3d(dst + T::PACKED_BYTES, &tmap_x, landed_bar(ps), 0, 0, k0 / 64);
                }
            }
        }
      } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (all lanes run the loop, one issues)
        const uint32_t instr = make_idesc(UMMA_BF16, UMMA_BF16, 128, MPAD);
        int gcount = 0;          // groups issued so far: slot gcount % SLOTS
        int pcount = 0;          // load stages consumed so far
        WorkSched<0> sched(cta, num_ctas, sp);
        WorkItem w;
        bool ok = true;
        while (ok && sched.next(w)) {
            // (Issuing two groups at a time with their MMAs alternating, so that the two accumulation chains overlap, was
            // measured 4-10 % slower: the issuer then waits for the second group's weights before it starts the first.)
            for (int g = 0; g < w.kb_count; g++, gcount++) {
                const int slot = gcount % SLOTS;
                const uint32_t sphase = ((uint32_t)(gcount / SLOTS)) & 1u;
                const int ps = pcount % LSTAGES;
                const int jg = g % T::LOAD_GROUPS;             // group inside its load stage
                const bool stage_ends = (jg == T::LOAD_GROUPS - 1 || g == w.kb_count - 1);
                if (!__all_sync(0xffffffffu, mbar_wait(gempty_bar(slot), sphase ^ 1u, abort_flag, p.status, ST_TIMEOUT_MMA_ACC, slot, 64))) { ok = false; break; }
                // ready[slot] also tells that the load stage has landed: the dequantisers waited for it
                if (!__all_sync(0xffffffffu, mbar_wait(ready_bar(slot), sphase, abort_flag, p.status, ST_TIMEOUT_MMA_FULL, slot, 64))) { ok = false; break; }
                tc_fence_after_sync();
                if (elect_one_sync()) {
                    const uint32_t d_tmem = tmem_base + (uint32_t)(slot * MPAD);
                    const uint32_t a_tmem = tmem_base + (uint32_t)(T::A_BASE + slot * T::A_COLS);
                    const uint64_t b_desc = make_smem_desc_k128(ld_base + ps * T::LOAD_STAGE_SMEM + T::PACKED_BYTES + jg * 2 * T::X_STRIDE);
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        // K-elements 16k .. 16k+15 of the group: A columns 8k .. 8k+7; activation box k / 4, 32-byte step k % 4
                        const uint64_t bt = advance_desc_k(b_desc + (uint64_t)(((k >> 2) * T::X_STRIDE) >> 4), k & 3);
                        umma_f16_ts(d_tmem, a_tmem + (uint32_t)(8 * k), bt, instr, k > 0 ? 1u : 0u);
                    }
                    umma_commit(gdone_bar(slot));
                    umma_commit(lfree_bar(ps));
                    if (stage_ends && jg == 0) umma_commit(lfree_bar(ps));   // the stage's only group: stand in for the missing one
                }
                __syncwarp();
                if (stage_ends) pcount++;
            }
        }
      }
    } else if (warp >= 4 + 4 * T::FOLD) {
        // ------------------------------------------------------------------ dequantisers
        if constexpr (T::DEQ_REGS < T::REGS_EVEN) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(T::DEQ_REGS));
        const int team = (warp - 4 - 4 * T::FOLD) >> 2;
        const int q = warp & 3;                       // TMEM lane quarter of this warp
        const int r = q * 32 + lane;                  // row of the tile this thread converts = TMEM lane
        // Units of work are half groups, numbered 2 * (group counter) + half over the whole run of this CTA; team t converts
        // the units that are t modulo TEAMS.  The loop visits only those: all index arithmetic happens once per converted
        // unit (a warp that stepped through every group and skipped the others' spent as many instructions on the
        // stepping as on the conversion).
        int gcount0 = 0, pcount0 = 0;                  // groups and load stages before the current work item
        WorkSched<0> sched(cta, num_ctas, sp);
        WorkItem w;
        bool ok = true;
        while (ok && sched.next(w)) {
            const int u0 = 2 * gcount0, u_end = u0 + 2 * w.kb_count;
            int u = u0 + (team + T::TEAMS - u0 % T::TEAMS) % T::TEAMS;
#pragma unroll 1
            for (; u < u_end; u += T::TEAMS) {
                const int gl = (u - u0) >> 1, h = u & 1;           // group inside the work item, half of the group
                const int gc = u >> 1;                             // group counter of the run
                const int slot = gc % SLOTS;
                const uint32_t sphase = ((uint32_t)(gc / SLOTS)) & 1u;
                const int pc = pcount0 + gl / T::LOAD_GROUPS;      // load stage counter: LOAD_GROUPS groups per stage
                const int ps = pc % LSTAGES;
                const uint32_t pphase = ((uint32_t)(pc / LSTAGES)) & 1u;
                const int jg = gl % T::LOAD_GROUPS;
                if (!mbar_wait(landed_bar(ps), pphase, abort_flag, p.status, ST_TIMEOUT_DEQUANT, ps, 64)) { ok = false; break; }
                // packed row r: 128 bytes, 128B-swizzled by the TMA; group jg of the stage is its 16-byte chunks 4jg .. 4jg+3,
                // this half the chunks 4jg + 2h and 4jg + 2h + 1 (64 K-elements)
                const uint8_t *row = ld_ptr + ps * T::LOAD_STAGE_SMEM + r * 128;
                uint32_t a[32];
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(row + (((4 * jg + 2 * h + c) ^ (r & 7)) << 4));
                    const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int i = 0; i < 4; i++) {              // word i of chunk c = K-elements 32c + 8i .. +7 -> 4 column words
                        uint32_t o[4];
                        int4x8_to_bf16x8_div64(words[i], o);
                        a[16 * c + 4 * i] = o[0]; a[16 * c + 4 * i + 1] = o[1]; a[16 * c + 4 * i + 2] = o[2]; a[16 * c + 4 * i + 3] = o[3];
                    }
                }
                // the slot's A columns are free once the MMAs of the group that used them last are done
                if (!mbar_wait(gdone_bar(slot), sphase ^ 1u, abort_flag, p.status, ST_TIMEOUT_DEQUANT, 16 + slot, 64)) { ok = false; break; }
                tc_fence_after_sync();
                tmem_st_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(T::A_BASE + slot * T::A_COLS + 32 * h), a);
                tmem_st_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(ready_bar(slot));
            }
            gcount0 += w.kb_count;
            pcount0 += (w.kb_count + T::LOAD_GROUPS - 1) / T::LOAD_GROUPS;
        }
    } else {
        // ------------------------------------------------------------------ fold + epilogue
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(T::FOLD_REGS));
        constexpr int FC = T::FCOLS;
        const int fg = (warp - 4) >> 2;                // fold group: columns fg*FC .. of the accumulator
        const int q = warp & 3;                        // the TMEM lane quarter of this warp
        const int r = q * 32 + lane;                   // weight row inside the tile = TMEM lane
        int gcount = 0;
        WorkSched<0> sched(cta, num_ctas, sp);
        WorkItem w;
        bool ok = true;
        while (ok && sched.next(w)) {
            const int n = w.tile * T::TILE_N + r;
            const bf16 *srow = p.scales + (size_t)(n < p.N ? n : 0) * p.num_groups + w.kb_begin;
            float total[FC];
#pragma unroll
            for (int m = 0; m < FC; m++) total[m] = 0.f;
            // scales are fetched eight groups ahead of their use (a load issued where it is needed would put an L2
            // round trip into every group and throttle the whole pipeline) and kept as packed bf16 pairs
            const unsigned short *sraw = reinterpret_cast<const unsigned short *>(srow);
            auto fetch4 = [&](int g0, uint32_t (&dst)[4]) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t lo = g0 + 2 * i < w.kb_count ? (uint32_t)__ldg(sraw + g0 + 2 * i) : 0u;
                    const uint32_t hi = g0 + 2 * i + 1 < w.kb_count ? (uint32_t)__ldg(sraw + g0 + 2 * i + 1) : 0u;
                    dst[i] = lo | (hi << 16);
                }
            };
            uint32_t s_cur[4], s_nxt[4];
            fetch4(0, s_cur);
            for (int g0 = 0; g0 < w.kb_count && ok; g0 += 8) {
                fetch4(g0 + 8, s_nxt);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    if (g0 + i >= w.kb_count) break;
                    const int b = gcount % SLOTS;
                    const float s = __uint_as_float((i & 1) ? (s_cur[i >> 1] & 0xffff0000u) : (s_cur[i >> 1] << 16));
                    if (!mbar_wait(gdone_bar(b), (uint32_t)(gcount / SLOTS) & 1u, abort_flag, p.status, ST_TIMEOUT_EPILOGUE, b, 64)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * MPAD + fg * FC);
#pragma unroll
                    for (int c0 = 0; c0 < FC; c0 += 16) {
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
                for (int i = 0; i < 4; i++) s_cur[i] = s_nxt[i];
            }
            if (!ok) break;
            if (w.part < 0) {
                if (n < p.N) {
#pragma unroll
                    for (int m = 0; m < FC; m++)
                        if (fg * FC + m < p.M) p.Y[(size_t)(fg * FC + m) * p.N + n] = __float2bfloat16_rn(total[m] * W4A16_TMEM_UNSCALE);
                }
            } else {
                float *slot = p.workspace + (size_t)(2 * cta + w.part) * 128 * 128 + (size_t)(fg * FC) * 128 + r;
#pragma unroll
                for (int m = 0; m < FC; m++) slot[m * 128] = total[m] * W4A16_TMEM_UNSCALE;
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
struct W4A16TmemLauncher {
    static bool can_run(int M, int N, int K) { return W4A16Launcher<W4A16Traits<T::MPAD, 2>>::can_run(M, N, K); }
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
            SM100_CUDA_TRY(cudaFuncSetAttribute(w4a16_tmem_gemm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_ALLOC));
            attr_set[devid].store(true, std::memory_order_release);
        }
        CUtensorMap tx, tw;
        rc = make_tmap_chunked(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, X, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, 64, T::MPAD, T::LOAD_KB);
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
        SM100_CUDA_TRY(cudaLaunchKernelEx(&cfg, w4a16_tmem_gemm_kernel<T>, tx, tw, p));
        int parts = 1;
        while (parts < 32 && p.num_n_tiles * parts < 2 * dev->sm_count) parts *= 2;
        cudaLaunchConfig_t rcfg = dependent_launch_config(p.num_n_tiles * parts, 256, stream);
        SM100_CUDA_TRY(cudaLaunchKernelEx(&rcfg, streamk_reduce_kernel<128, 128>, (const float *)workspace, static_cast<bf16 *>(Y), M, N, 1,
                                          p.num_n_tiles, 1, p.num_groups, grid, parts, 1.0f));
        return GEMM_OK;
    }
};

}  // namespace sm100
