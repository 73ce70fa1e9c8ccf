// Y = X * W^T for sm_100a: TMA -> 128B-swizzled shared-memory ring -> tcgen05.mma with the
// accumulator in TMEM -> epilogue out of TMEM.  One persistent kernel template serves the
// direct path, split-K and stream-K (FP32 partials), the dense FP8 per-tensor variant (same
// pipeline, 1-byte elements, kind::f8f6f4) and the block-scaled MXFP8 / MX-FP4 variants.
//
// Plays the role of the reference's src/bf16_gemm.cuh (kernels :259-503 and :606-828, host
// launchers BF16GemmMMA::run :506-542 and BF16GemmMMASplitK::run :849-896), which is a
// warpgroup mma.sync design for sm_120a.  Nothing of that structure is kept except the
// class names of the entry points and the persistent static tile loop.
//
// Warp roles inside one CTA (256 threads, 384 with a second epilogue group):
//   warp 0    TMA producer (one lane)          warp 1    tcgen05.mma issuer (one lane)
//   warp 2    TMEM allocation / release        warp 3    idle
//   warps 4-7 epilogue: warp w reads TMEM lanes 32*(w-4) .. +31 (one output row per thread)
//   warps 8-11 second epilogue group, only in kernels with a single accumulator stage
//
// Barriers:  full[s]   TMA bytes landed           -> MMA issuer
//            empty[s]  tcgen05.commit of stage s  -> producer
//            tfull[a]  tcgen05.commit of a tile   -> epilogue       (a = accumulator buffer 0/1)
//            tempty[a] epilogue drained buffer a  -> MMA issuer
// Two accumulator buffers let the epilogue of tile t overlap the main loop of tile t+1.
//
// CTA pairs (CG = 2): two CTAs of a cluster compute one 256 x BN tile.  Each loads its own
// 128 rows of X and its own BN/2 rows of W (no multicast), the leader CTA issues one
// cta_group::2 MMA that reads both shared memories, and each CTA ends up with its 128 rows of
// the accumulator in its own TMEM.  full[] lives in the leader and counts both CTAs' bytes;
// empty[] / tfull[] arrivals are delivered to both CTAs by the commit.
//
// Two row blocks per CTA (MB = 2, 512 x 256 tiles on a pair): each CTA holds 256 rows of X per stage and
// every K step issues two MMAs on the same B tile, one per 128-row block, into two accumulators that
// together fill TMEM.  Shared memory then receives 96 KB of operands per 512 x 256 x 64 MACs instead of
// 128 KB, which is what bounds the 256 x 256 tile at the power cap.
#pragma once
#include <cuda_bf16.h>

#include <atomic>
#include <cstdlib>

#include "gemm_host.h"
#include "ptx_sm100.cuh"
#include "tile_order.h"
#include "umma_desc.h"

using bf16 = __nv_bfloat16;

namespace sm100 {

// -DGEMM_DEBUG_BOUNDS builds check every computed TMA coordinate and every directly computed store address
// before it is used; a violation is recorded in the device status block (code, block, offending value) and the
// access still goes ahead only where the hardware clips it anyway (TMA boxes).  Stands in for a memory checker
// on the ragged-shape tests; compiled out of the normal plugins.
#ifdef GEMM_DEBUG_BOUNDS
#define SM100_BOUNDS(cond, code, detail)                                             \
    do {                                                                             \
        if (!(cond) && p.status != nullptr && atomicCAS(p.status, 0u, (uint32_t)(code)) == 0u) { \
            p.status[1] = blockIdx.x;                                                \
            p.status[2] = (uint32_t)(detail);                                        \
        }                                                                            \
    } while (0)
#else
#define SM100_BOUNDS(cond, code, detail) do { } while (0)
#endif

// operand element kind: bf16; e4m3 with per-tensor scales; e4m3 / e2m1 with one ue8m0 scale per 32
// K-elements of both operands (block-scaled MMA, scale factors staged in TMEM)
enum : int { OPK_BF16 = 0, OPK_E4M3 = 1, OPK_MXFP8 = 2, OPK_MXFP4 = 3 };
// epilogue: register->global stores; shared memory + TMA store; register->global stores with the fused
// output transform  D = act(alpha * acc + beta * C + bias)  and an optional e4m3 output with amax
enum : int { EPI_DIRECT = 0, EPI_TMA = 1, EPI_FUSED = 2 };
enum : int { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU = 2, ACT_SILU = 3 };   // GemmArgs.activation
enum : int { YOUT_BF16 = 0, YOUT_E4M3 = 1 };                             // GemmArgs.y_dtype

// Where the bf16 result goes.  Normally one row-major M x N matrix.  In an N-sharded multi-GPU run
// each rank instead stores its M x N block into columns [col_offset, col_offset + N) of the row-major
// M x ld result on EVERY rank, which fuses the all-gather of the column blocks into the epilogue:
// either one TMA store per rank through NVLink peer mappings, or one multimem store per 16 bytes to the
// NVSwitch multicast mapping of the result.  Stores only; nothing is ever loaded from peer memory.
static constexpr int MAX_Y_PEERS = 8;
struct YMaps {
    CUtensorMap m[MAX_Y_PEERS];
};
struct YTarget {
    void *const *peers = nullptr;   // num_peers base pointers (this rank's own buffer among them); nullptr = plain Y
    int num_peers = 0;
    long long ld = 0;               // row pitch of the destination matrices in elements
    int col_offset = 0;
    void *multicast = nullptr;      // NVSwitch multicast address of the same matrix: one multimem store reaches every rank
    bool forward = false;           // with a multicast address, kernels that have sender warps: store the tile locally and let
                                    // them forward it (two-row-block kernels always do)
};

struct GemmParams {
    int M, N, K;
    int num_m_blocks, num_n_blocks;
    int num_k_blocks;     // per split (stream-K: per tile)
    int group_n;          // width (in N tiles) of a rasterisation band
    int wait_sleep_ns;    // > 0: the epilogue's wait for an accumulator and the producer's wait for a free slot back off up to this long
    void *Y;              // bf16 output (direct epilogue)
    float *workspace;     // split-K partial sums [split][M][N]
    float alpha;          // epilogue scale (FP8 per-tensor: sx*sw)
    int y_targets;        // TMA-store epilogue: destination matrices (1, or the ranks of a sharded run)
    int y_col_offset;     // column of the destination where this GEMM's column 0 lands
    bf16 *y_mc;           // non-null: multicast address of the destination (row pitch y_ld); multimem stores replace the TMA stores
    long long y_ld;
    uint32_t *status;
    // block-scaled kinds: ue8m0 scale factors in 512-byte atoms of 128 rows x 4 K-blocks,
    // atom (row/128, kblock/4) at byte ((row/128) * sf_k_atoms + kblock/4) * 512
    int sf_k_atoms;
    // fused output transform (EPI_FUSED): D = act(alpha * acc + beta * C + bias); bf16 out, or e4m3(D * y_scale) with max|D| -> amax
    const bf16 *C;        // M x N bf16, row pitch N; nullptr = no beta term
    const bf16 *bias;     // N bf16 (one per output column); nullptr = none
    float beta;
    float y_scale;
    float *amax;          // nullptr = not wanted
    int act;              // ACT_*
    int y_dtype;          // YOUT_*
    int forward;          // N-sharded run with a multicast address: 1 = tiles go to the local matrix and the sender warps forward them
    uint32_t *wave_sync;  // two-row-block kernels, many waves: arrival counter that keeps the clusters' producers in step (or nullptr)
    int tail_full;        // two-row-block kernels: whole tiles before the halved last wave (see WorkSched); < 0: no halving
    int test_withhold_kb; // wait-expiry test build only: the producer stops before this k-block (< 0: never)
};

// One piece of work for a CTA (or CTA pair): accumulate `kb_count` k-blocks of one output tile.
struct WorkItem {
    int tile;       // output tile, rasterised by tile_to_mn
    int kb_begin;   // first k-block (units of BK elements)
    int kb_count;
    int part;       // -1: the whole K range -> bf16 output; >= 0: FP32 partial (split index, or stream-K slot 0/1)
    int half;       // two-row-block kernels, last wave: -1 the whole tile, 0 / 1 only its upper / lower 256 rows (see WorkSched)
};

// Work distribution.  SPLIT_K >= 1: tiles x SPLIT_K equal K slices, dealt round-robin over the
// persistent grid (the reference's virtual-tile scheme, src/bf16_gemm.cuh:654-655).
// SPLIT_K == 0 ("stream-K"): the tiles x k-blocks units are cut into one contiguous, equally
// long range per CTA, so every SM streams the same number of bytes whatever the tile count; a
// range that does not cover a tile's whole K leaves an FP32 partial in the CTA's slot 0 (its
// first item) or slot 1 (its last item), which streamk_reduce_kernel adds up in K order.
//
// Halved last wave (SPLIT_K == 1, two-row-block kernels only; p.tail_full >= 0): when the tiles left for the last
// round of the grid are at most half as many as the clusters, every one of them is dealt as two halves of 256 rows,
// each computed like a 256 x 256 tile by a cluster of its own, so the last wave takes half as long.  Virtual
// indices below tail_full are whole tiles; index tail_full + 2i + h is half h of tile tail_full + i.
template <int SPLIT_K>
struct WorkSched {
    long long u, u_begin, u_end;   // stream-K: unit range;  fixed: virtual tile index, stride, total
    int kb_per_tile;
    int tail_full;
    __device__ WorkSched(int cluster_id, int num_clusters, const GemmParams &p)
    {
        kb_per_tile = p.num_k_blocks;
        tail_full = -1;
        if constexpr (SPLIT_K == 0) {
            const long long units = (long long)p.num_m_blocks * p.num_n_blocks * kb_per_tile;
            u_begin = units * cluster_id / num_clusters;
            u_end = units * (cluster_id + 1) / num_clusters;
            u = u_begin;
        } else {
            u = cluster_id;
            u_begin = num_clusters;
            u_end = (long long)p.num_m_blocks * p.num_n_blocks * SPLIT_K;
            if constexpr (SPLIT_K == 1) {
                tail_full = p.tail_full;
                if (tail_full >= 0) u_end = tail_full + 2 * (u_end - tail_full);
            }
        }
    }
    __device__ bool next(WorkItem &w)
    {
        if (u >= u_end) return false;
        w.half = -1;
        if constexpr (SPLIT_K == 0) {
            w.tile = (int)(u / kb_per_tile);
            w.kb_begin = (int)(u - (long long)w.tile * kb_per_tile);
            const long long left = u_end - u;
            w.kb_count = kb_per_tile - w.kb_begin < left ? kb_per_tile - w.kb_begin : (int)left;
            const bool whole = (w.kb_begin == 0 && w.kb_count == kb_per_tile);
            w.part = whole ? -1 : (u == u_begin ? 0 : 1);
            u += w.kb_count;
        } else {
            w.tile = (int)(u / SPLIT_K);
            const int split = (int)(u - (long long)w.tile * SPLIT_K);
            w.kb_begin = split * kb_per_tile;
            w.kb_count = kb_per_tile;
            w.part = SPLIT_K > 1 ? split : -1;
            if constexpr (SPLIT_K == 1) {
                if (tail_full >= 0 && u >= tail_full) {
                    const int unit = (int)(u - tail_full);
                    w.tile = tail_full + (unit >> 1);
                    w.half = unit & 1;
                }
            }
            u += u_begin;
        }
        return true;
    }
};

// MB_ = 128-row blocks of X per CTA.  With MB_ = 2 a CTA owns 256 rows: every stage holds 32 KB of X and the
// same B tile feeds two MMAs per K step, one per row block, each with its own accumulator.  Per flop that is a
// quarter less operand traffic into shared memory (and out of L2) than MB_ = 1; the two 256-column accumulators
// fill TMEM, so there is one accumulator stage and the two epilogue groups drain one row block each.
template <int OPK_, int BN_, int STAGES_, int CG_, int SPLIT_K_, int EPI_, int MB_ = 1>
struct UmmaGemmTraits {
    static constexpr int MB = MB_;
    static constexpr int EPI_ROWS = 128;                   // rows one epilogue group stages and stores at a time
    static constexpr int OPK = OPK_;
    static constexpr int BN = BN_;
    static constexpr int STAGES = STAGES_;
    static constexpr int CG = CG_;
    static constexpr int SPLIT_K = SPLIT_K_;
    static constexpr int EPI = (SPLIT_K_ > 1) ? EPI_DIRECT : EPI_;   // stream-K (0) keeps the chosen epilogue for whole tiles
    static constexpr int ELEM_BITS = (OPK_ == OPK_BF16) ? 16 : (OPK_ == OPK_MXFP4) ? 4 : 8;
    static constexpr bool BLOCK_SCALED = (OPK_ == OPK_MXFP8 || OPK_ == OPK_MXFP4);
    static constexpr int BM_CTA = 128 * MB_;               // rows of X per CTA (each accumulator covers 128 of them)
    static constexpr int BM = BM_CTA * CG_;                // rows of the tile
    static constexpr int UMMA_M = 128 * CG_;               // M extent of one MMA instruction
    static constexpr int BK_BYTES = 128;                   // one swizzle span per row
    static constexpr int BK = BK_BYTES * 8 / ELEM_BITS;    // K elements per stage
    static constexpr int BK_COORD = (OPK_ == OPK_BF16) ? BK : BK_BYTES;   // the same, in tensor-map elements (bf16, else bytes)
    static constexpr int UMMA_K_STEPS = BK_BYTES / 32;     // 4 MMAs per stage
    static constexpr int BN_CTA = BN_ / CG_;               // rows of W this CTA loads
    static constexpr int A_BYTES = BM_CTA * BK_BYTES;
    static constexpr int B_BYTES = BN_CTA * BK_BYTES;
    // block-scaled kinds: per stage, one 512-byte scale atom per 128 rows and 128 K-elements
    static constexpr int SF_K_ATOMS = BLOCK_SCALED ? BK / 128 : 0;
    static constexpr int SF_N_ATOMS = (BN_ + 127) / 128;
    static constexpr int SF_A_BYTES = SF_K_ATOMS * 512;
    static constexpr int SF_B_BYTES = SF_K_ATOMS * SF_N_ATOMS * 512;
    static constexpr int SF_BYTES = SF_A_BYTES + SF_B_BYTES;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SF_BYTES;   // bytes that arrive per stage
    static constexpr int OUT_CHUNK = 64;                   // output columns per TMA store (128 bytes of bf16)
    static constexpr int ACC_STRIDE = (BN_ + 31) / 32 * 32;  // TMEM columns between the two accumulator buffers
    static constexpr int SF_COLS_ONE = SF_K_ATOMS * (1 + SF_N_ATOMS) * 4;   // TMEM columns of one k-block's scale factors
    static constexpr int SF_COLS = 2 * SF_COLS_ONE;        // two sets: the next k-block's are copied in while this one's MMAs run
    // two FP32 accumulator buffers when they fit beside the scale factors, else one
    static constexpr int ACC_STAGE_COLS = MB_ * ACC_STRIDE;  // TMEM columns of one accumulator stage (MB_ row blocks side by side)
    static constexpr int ACC_STAGES = (2 * ACC_STAGE_COLS + SF_COLS <= 512) ? 2 : 1;
    static constexpr int SF_RING_BYTES = (STAGES_ * SF_BYTES + 1023) / 1024 * 1024;   // keeps the staging tiles 1024-byte aligned
    static constexpr int NUM_BARRIERS = 2 * STAGES_ + 4 + (BLOCK_SCALED ? 4 : 0);   // block-scaled: + scale set ready / free, two sets
    static constexpr int RING_BYTES = STAGES_ * (A_BYTES + B_BYTES) + SF_RING_BYTES + NUM_BARRIERS * 8 + 16 + 1024;
    // Staging buffers of 128 rows x 64 bf16.  Two by default (one epilogue group: used in turn; two groups: one each).
    // A kernel with a single accumulator stage stalls its MMAs until the accumulator is drained, and with two
    // buffers the drain waits for TMA stores to release them; where shared memory allows it such a kernel gets
    // four, so each of its two epilogue groups drains its pieces back to back and hands the accumulator back at once.
    static constexpr int STAGING_BUFS = (ACC_STAGES == 1 && RING_BYTES + 4 * EPI_ROWS * OUT_CHUNK * 2 <= 232448) ? 4 : 2;
    static constexpr int STAGING_BYTES = (EPI == EPI_TMA) ? STAGING_BUFS * EPI_ROWS * OUT_CHUNK * 2 : 0;
    static constexpr int SMEM_BYTES = STAGES_ * (A_BYTES + B_BYTES) + SF_RING_BYTES + STAGING_BYTES + NUM_BARRIERS * 8 + 16;
    static constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;   // slack to align the base to 1024 bytes
    static constexpr int ACC_COLS = ACC_STAGES * ACC_STAGE_COLS + SF_COLS;
    static constexpr int TMEM_COLS = ACC_COLS <= 32 ? 32 : ACC_COLS <= 64 ? 64 : ACC_COLS <= 128 ? 128 : ACC_COLS <= 256 ? 256 : 512;
    // Kernels with a single accumulator buffer cannot hide the epilogue behind the next main loop, so they
    // drain it with two epilogue groups of four warps (alternate 64- or 16-column pieces) instead of one.
    static constexpr int EPI_GROUPS = ACC_STAGES == 1 ? 2 : 1;
    // Two row blocks per CTA have a single accumulator stage, so their epilogue is on the critical path of the next
    // tile; in an N-sharded run its multicast stores would be paced by NVLink (a few GB/s per SM).  Such kernels
    // therefore store the tile to the LOCAL result with TMA stores and four more warps ("senders") forward finished
    // tiles from there to the multicast address while the next tile's MMAs run.
    // The 256 x 256 TMA-store kernels carry the sender warps too: there the caller chooses between sending 128-byte row
    // pieces from the epilogue and forwarding whole 512-byte rows from L2 (GemmParams::forward).
    static constexpr int SENDER_WARPS = (MB_ == 2 || (CG_ == 2 && BN_ == 256 && EPI == EPI_TMA && SPLIT_K_ == 1 && !BLOCK_SCALED)) ? 4 : 0;
    static constexpr int THREADS = 128 + 128 * EPI_GROUPS + 32 * SENDER_WARPS;
    static_assert(BN_ % 16 == 0 && BN_ >= 16 && BN_ <= 256, "BN (the UMMA N extent) is a multiple of 16 up to 256");
    static_assert(EPI != EPI_TMA || BN_ % 64 == 0, "the TMA-store epilogue writes 64-column boxes");
    static_assert((BN_ / CG_) % 8 == 0, "each CTA loads whole 8-row swizzle groups of W");
    static_assert(CG_ == 1 || CG_ == 2, "CTA group is 1 or 2");
    static_assert(MB_ == 1 || (MB_ == 2 && SPLIT_K_ == 1 && EPI_ == EPI_TMA && !BLOCK_SCALED && ACC_STAGES == 1),
                  "two row blocks per CTA: whole-K tiles, TMA-store epilogue, dense operand kinds, one accumulator stage");
    static_assert(EPI_ != EPI_FUSED || (SPLIT_K_ == 1 && MB_ == 1), "the fused output transform works on whole-K tiles of one row block per CTA");
    // (a 256 x 192 tile, whose scales start 64 rows into an atom on odd tiles -- two TMEM columns further on -- computes
    // correctly and leaves room for two accumulator stages, but measured 4 % (MXFP8) and 12 % (MX-FP4) slower than 256 x 256)
    static_assert(!BLOCK_SCALED || BN_ % 128 == 0, "block-scaled tiles: BN a multiple of the 128-row scale atom");
    static_assert(STAGES_ >= 2, "at least two ring stages");
    static_assert(ACC_COLS <= 512, "TMEM has 512 columns");
    static_assert(SMEM_ALLOC <= 232448, "exceeds the 227 KB of shared memory one CTA can have");
};

template <class T>
__global__ void __launch_bounds__(T::THREADS, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                 const __grid_constant__ YMaps tmap_ys, const __grid_constant__ CUtensorMap tmap_sfx,
                 const __grid_constant__ CUtensorMap tmap_sfw, const GemmParams p)
{
    constexpr int CG = T::CG;
    constexpr int BN = T::BN;
    constexpr int STAGES = T::STAGES;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (smem_base - raw_addr);

    const uint32_t a_base = smem_base;
    const uint32_t b_base = smem_base + STAGES * T::A_BYTES;
    const uint32_t sf_base = b_base + STAGES * T::B_BYTES;
    const uint32_t stg_base = sf_base + T::SF_RING_BYTES;
    const uint32_t bar_base = stg_base + T::STAGING_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    auto sfready_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 4 + s); };      // block-scaled kinds only
    auto sffree_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 6 + s); };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + (bar_base - smem_base) + 8u * T::NUM_BARRIERS);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    // epilogue -> senders: one counter per epilogue group (two words), the tiles whose row block that group has stored
    // completely, counted up for ever (a counter, not an mbarrier: the senders may fall more than one tile behind,
    // which a phase bit cannot express)
    volatile uint32_t *stored_count = tmem_slot + 2;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = (CG == 2) ? cluster_ctarank() : 0u;
    const int cluster_id = blockIdx.x / CG;
    const int num_clusters = gridDim.x / CG;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), CG * 4 * T::EPI_GROUPS);   // one arrival per epilogue warp of every CTA of the group
        }
        if constexpr (T::BLOCK_SCALED) {
            for (int s = 0; s < 2; s++) {
                mbar_init(sfready_bar(s), 1);
                mbar_init(sffree_bar(s), 1);
            }
        }
        stored_count[0] = 0;
        stored_count[1] = 0;
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
        prefetch_tensormap(&tmap_x);
        prefetch_tensormap(&tmap_w);
        if (T::EPI == EPI_TMA)
            for (int t = 0; t < p.y_targets; t++) prefetch_tensormap(&tmap_ys.m[t]);
    }
    if (warp == 2) {
        tmem_alloc<CG>(smem_u32(tmem_slot), T::TMEM_COLS);
        tmem_relinquish<CG>();
    }
    tc_fence_before_sync();
    if constexpr (CG == 2) cluster_sync_all(); else __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // split-K / stream-K: the reduce kernel that follows may be scheduled from now on (it blocks
    // in griddepcontrol.wait until this grid has finished)
    if constexpr (T::SPLIT_K != 1) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // Scale atoms of one k-block: this CTA's 128 X rows, then every 128-row group of the tile's W rows (a CTA
    // pair computes all BN columns in each CTA, so each CTA fetches all of them).  The tiled scale array is
    // mapped as rows of 256 bytes, two per 512-byte atom.
    auto load_scale_atoms = [&](int stage, int kblock, int row_x, int row_w_tile, uint32_t bar) {
        const uint32_t sf_dst = sf_base + stage * T::SF_BYTES;
        const int katom = kblock * T::SF_K_ATOMS;
#pragma unroll
        for (int a = 0; a < T::SF_K_ATOMS; a++) {
            const int ax = ((row_x / 128) * p.sf_k_atoms + katom + a) * 2;
            if constexpr (CG == 1) tma_load_2d(sf_dst + a * 512, &tmap_sfx, bar, 0, ax);
            else tma_load_2d_pair(sf_dst + a * 512, &tmap_sfx, bar, 0, ax);
#pragma unroll
            for (int j = 0; j < T::SF_N_ATOMS; j++) {
                const int aw = ((row_w_tile / 128 + j) * p.sf_k_atoms + katom + a) * 2;
                const uint32_t dst = sf_dst + T::SF_A_BYTES + (a * T::SF_N_ATOMS + j) * 512;
                if constexpr (CG == 1) tma_load_2d(dst, &tmap_sfw, bar, 0, aw);
                else tma_load_2d_pair(dst, &tmap_sfw, bar, 0, aw);
            }
        }
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            const uint32_t full_leader = (CG == 2) ? mapa_shared(full_bar(0), 0) : full_bar(0);
            bool ok = true;
            int pace_iter = 0;             // work items this producer has started
            uint32_t pace_target = 0;      // arrivals that complete the current wave's count
            WorkSched<T::SPLIT_K> sched(cluster_id, num_clusters, p);
            WorkItem w;
            while (ok && sched.next(w)) {
                int mb, nb;
                tile_to_mn(w.tile, p.num_m_blocks, p.num_n_blocks, p.group_n, mb, nb);
                // half of a tile (last wave of a two-row-block kernel): 256 consecutive rows, 128 per CTA, into row block 0
                const bool half = T::MB == 2 && w.half >= 0;
                const int row_x = half ? mb * T::BM + w.half * (T::BM / 2) + (int)cta_rank * 128 : mb * T::BM + (int)cta_rank * T::BM_CTA;
                const int row_w = nb * BN + (int)cta_rank * T::BN_CTA;
                const uint32_t stage_bytes = half ? T::STAGE_BYTES - T::A_BYTES / 2 : T::STAGE_BYTES;
                SM100_BOUNDS(row_x >= 0 && row_x < p.M + T::BM && row_w >= 0 && row_w < p.N + BN, ST_BOUNDS_LOAD_ROW, w.tile);
                if constexpr (T::MB == 2) {
                    // Wave pacing.  Clusters that share an operand panel read it from DRAM once only while they stay within
                    // the few dozen microseconds a line survives in L2; left alone they drift apart over the waves of a
                    // long launch (measured: one wave reads exactly its unique bytes, 28 waves read 1.9 times theirs).
                    // Before its second and later tiles the leader's producer therefore counts itself in and waits until
                    // every cluster that has such a tile has done so too -- or 40 microseconds have passed: the wait
                    // only paces, nothing depends on it, and a cluster that is not running cannot hold the others up.
                    if (p.wave_sync != nullptr && cta_rank == 0 && pace_iter > 0) {
                        const long long tiles = (long long)p.num_m_blocks * p.num_n_blocks;
                        const long long left = tiles - (long long)pace_iter * num_clusters;
                        pace_target += (uint32_t)(left < num_clusters ? left : num_clusters);
                        atomicAdd(p.wave_sync, 1u);
                        const long long t0 = clock64();
                        uint32_t seen;
                        do {
                            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.wave_sync) : "memory");
                            if (seen >= pace_target) break;
                            __nanosleep(200);
                        } while (clock64() - t0 < 80000);
                    }
                    pace_iter++;
                }
                for (int kb = 0; kb < w.kb_count; kb++) {
                    const int kx = (w.kb_begin + kb) * T::BK_COORD;
                    // tensor-map element = bf16, or one byte for the 8- and 4-bit kinds: the box must start inside the
                    // row (the last box may reach past its end: zero-filled) and on a 16-byte boundary
                    SM100_BOUNDS(kx >= 0 && (long long)kx < (T::OPK == OPK_BF16 ? (long long)p.K : (long long)p.K * T::ELEM_BITS / 8) &&
                                 (kx * (T::OPK == OPK_BF16 ? 2 : 1)) % 16 == 0, ST_BOUNDS_LOAD_K, kx);
#ifdef SM100_TEST_WITHHOLD_STAGE
                    // wait-expiry test build: from this k-block on nothing is requested any more, so the MMA issuer's
                    // wait for the stage runs out (nothing is in flight then: every earlier load completes by itself)
                    if (p.test_withhold_kb >= 0 && w.kb_begin + kb >= p.test_withhold_kb) { ok = false; break; }
#endif
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, ST_TIMEOUT_PRODUCER, stage, p.wait_sleep_ns > 128 ? 128 : p.wait_sleep_ns)) {
                        ok = false;
                        break;
                    }
                    if constexpr (CG == 1) {
                        mbar_arrive_expect_tx(full_bar(stage), T::STAGE_BYTES);
                        tma_load_2d(b_base + stage * T::B_BYTES, &tmap_w, full_bar(stage), kx, row_w);
                        tma_load_2d(a_base + stage * T::A_BYTES, &tmap_x, full_bar(stage), kx, row_x);
                        if constexpr (T::BLOCK_SCALED) load_scale_atoms(stage, w.kb_begin + kb, row_x, nb * BN, full_bar(stage));
                    } else {
                        if (cta_rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * stage_bytes);
                        const uint32_t fb = full_leader + 8u * stage;
                        tma_load_2d_pair(b_base + stage * T::B_BYTES, &tmap_w, fb, kx, row_w);
                        // the scale-factor map of X is free in these kernels: it carries X again, with a box of 128 rows
                        if (half) tma_load_2d_pair(a_base + stage * T::A_BYTES, &tmap_sfx, fb, kx, row_x);
                        else tma_load_2d_pair(a_base + stage * T::A_BYTES, &tmap_x, fb, kx, row_x);
                        if constexpr (T::BLOCK_SCALED) load_scale_atoms(stage, w.kb_begin + kb, row_x, nb * BN, fb);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (cta_rank == 0) {   // every lane runs the loop; one elected lane issues (see elect_one_sync)
            const uint32_t instr = (T::OPK == OPK_BF16) ? make_idesc(UMMA_BF16, UMMA_BF16, T::UMMA_M, BN)
                                                         : make_idesc(UMMA_E4M3, UMMA_E4M3, T::UMMA_M, BN);
            // Scale factors live behind the accumulator buffers, in two sets used in turn (X atoms, then W atoms).  Warp 3
            // copies them from shared memory (tcgen05.cp) one k-block ahead and publishes each set on sfready; this warp
            // hands a set back on sffree once the MMAs that read it are done.
            const uint32_t sf_tmem0 = tmem_base + (uint32_t)(T::ACC_STAGES * T::ACC_STAGE_COLS);
            uint32_t kcount = 0;       // k-blocks issued by this CTA so far: scale set kcount & 1
            int stage = 0;
            uint32_t phase = 0;
            int titer = 0;
            bool ok = true;
            WorkSched<T::SPLIT_K> sched(cluster_id, num_clusters, p);
            WorkItem w;
            for (; ok && sched.next(w); titer++) {
                const int acc = titer % T::ACC_STAGES;
                const uint32_t acc_phase = (titer / T::ACC_STAGES) & 1;
                if (!__all_sync(0xffffffffu, mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, ST_TIMEOUT_MMA_ACC, acc))) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * T::ACC_STAGE_COLS);
                for (int kb = 0; kb < w.kb_count; kb++) {
                    if (!__all_sync(0xffffffffu, mbar_wait(full_bar(stage), phase, abort_flag, p.status, ST_TIMEOUT_MMA_FULL, stage))) {
                        ok = false;
                        break;
                    }
                    if constexpr (T::BLOCK_SCALED) {
                        if (!__all_sync(0xffffffffu, mbar_wait(sfready_bar(kcount & 1u), (kcount >> 1) & 1u, abort_flag, p.status, ST_TIMEOUT_MMA_FULL, 32 + stage))) {
                            ok = false;
                            break;
                        }
                    }
                    tc_fence_after_sync();
                    if (elect_one_sync()) {
                    const uint64_t a_desc = make_smem_desc_k128(a_base + stage * T::A_BYTES);
                    const uint64_t b_desc = make_smem_desc_k128(b_base + stage * T::B_BYTES);
                    const uint32_t sfa_tmem = sf_tmem0 + (uint32_t)((kcount & 1u) * T::SF_COLS_ONE), sfb_tmem = sfa_tmem + (uint32_t)(T::SF_K_ATOMS * 4);
#pragma unroll
                    for (int k = 0; k < T::UMMA_K_STEPS; k++) {
                        const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                        if constexpr (T::OPK == OPK_MXFP8) {
                            // 4 instructions of 32 K-elements share one atom: instruction k uses scale byte k
                            umma_mxf8<CG>(d_tmem, advance_desc_k(a_desc, k), advance_desc_k(b_desc, k),
                                      make_idesc_block_scaled(UMMA_E4M3, UMMA_E4M3, T::UMMA_M, BN, k, k), sfa_tmem, sfb_tmem, accumulate);
                        } else if constexpr (T::OPK == OPK_MXFP4) {
                            // 4 instructions of 64 K-elements: two per atom, each using one half (2 scale bytes)
                            umma_mxf4<CG>(d_tmem, advance_desc_k(a_desc, k), advance_desc_k(b_desc, k),
                                      make_idesc_block_scaled(UMMA_MXF4_E2M1, UMMA_MXF4_E2M1, T::UMMA_M, BN, (k & 1) * 2, (k & 1) * 2),
                                      sfa_tmem + (k >> 1) * 4, sfb_tmem + (k >> 1) * (T::SF_N_ATOMS * 4), accumulate);
                        } else
                        if constexpr (T::OPK == OPK_BF16) {
#pragma unroll
                            for (int blk = 0; blk < T::MB; blk++)   // row block blk: X rows 128*blk.. of this CTA, 16 KB further on
                                if (blk == 0 || w.half < 0)
                                umma_f16<CG>(d_tmem + (uint32_t)(blk * T::ACC_STRIDE), advance_desc_k(a_desc + (uint64_t)(blk * 1024), k),
                                             advance_desc_k(b_desc, k), instr, accumulate);
                        } else {
#pragma unroll
                            for (int blk = 0; blk < T::MB; blk++)
                                if (blk == 0 || w.half < 0)
                                umma_f8f6f4<CG>(d_tmem + (uint32_t)(blk * T::ACC_STRIDE), advance_desc_k(a_desc + (uint64_t)(blk * 1024), k),
                                                advance_desc_k(b_desc, k), instr, accumulate);
                        }
                    }
                    if constexpr (CG == 1) umma_commit(empty_bar(stage)); else umma_commit_pair(empty_bar(stage), 3);
                    if constexpr (T::BLOCK_SCALED) {
                        if constexpr (CG == 1) umma_commit(sffree_bar(kcount & 1u)); else umma_commit_pair(sffree_bar(kcount & 1u), 1);
                    }
                    }
                    __syncwarp();
                    kcount++;
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                if (elect_one_sync()) {
                    if constexpr (CG == 1) umma_commit(tfull_bar(acc)); else umma_commit_pair(tfull_bar(acc), 3);
                }
                __syncwarp();
            }
        }
    } else if (warp == 3) {
        // ------------------------------------------------------------------ scale-factor copier (block-scaled kinds)
        if constexpr (T::BLOCK_SCALED) {
            if (cta_rank == 0) {
                const uint32_t sf_tmem0 = tmem_base + (uint32_t)(T::ACC_STAGES * T::ACC_STAGE_COLS);
                int stage = 0;
                uint32_t phase = 0, kcount = 0;
                bool ok = true;
                WorkSched<T::SPLIT_K> sched(cluster_id, num_clusters, p);
                WorkItem w;
                while (ok && sched.next(w)) {
                    for (int kb = 0; kb < w.kb_count; kb++, kcount++) {
                        const uint32_t set = kcount & 1u;
                        // the stage's scale atoms have landed, and the MMAs that read this set two k-blocks ago are done
                        if (!__all_sync(0xffffffffu, mbar_wait(full_bar(stage), phase, abort_flag, p.status, ST_TIMEOUT_MMA_FULL, 64 + stage)) ||
                            !__all_sync(0xffffffffu, mbar_wait(sffree_bar(set), ((kcount >> 1) & 1u) ^ 1u, abort_flag, p.status, ST_TIMEOUT_MMA_FULL, 96 + stage))) {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        if (elect_one_sync()) {
                            const uint32_t sfa = sf_tmem0 + set * (uint32_t)T::SF_COLS_ONE, sfb = sfa + (uint32_t)(T::SF_K_ATOMS * 4);
                            const uint32_t sf_src = sf_base + stage * T::SF_BYTES;
#pragma unroll
                            for (int a = 0; a < T::SF_K_ATOMS; a++) {
                                tmem_cp_sf_atom<CG>(sfa + a * 4, make_sf_atom_desc(sf_src + a * 512));
#pragma unroll
                                for (int j = 0; j < T::SF_N_ATOMS; j++)
                                    tmem_cp_sf_atom<CG>(sfb + (a * T::SF_N_ATOMS + j) * 4,
                                                        make_sf_atom_desc(sf_src + T::SF_A_BYTES + (a * T::SF_N_ATOMS + j) * 512));
                            }
                            // arrives once the copies above are complete (a commit tracks the issuing thread's tcgen05 operations)
                            if constexpr (CG == 1) umma_commit(sfready_bar(set)); else umma_commit_pair(sfready_bar(set), 1);
                        }
                        __syncwarp();
                        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                    }
                }
            }
        }
    } else if (warp >= 4 && warp < 4 + 4 * T::EPI_GROUPS) {
        // ------------------------------------------------------------------ epilogue
        constexpr int EG = T::EPI_GROUPS;
        const int eg = (warp - 4) >> 2;            // epilogue group of this warp
        const int q = (warp - 4) & 3;              // == warp % 4: the TMEM lane quarter this warp may read
        const int row_in_tile = q * 32 + lane;     // accumulator row = TMEM lane
        const int epi_tid = threadIdx.x - 128 - eg * 128;
        const uint32_t bar_a = 1 + 2 * eg, bar_b = 2 + 2 * eg;   // named barriers of this group
        const uint32_t tempty_leader = (CG == 2) ? mapa_shared(tempty_bar(0), 0) : tempty_bar(0);
        int titer = 0;
        int buf = 0;
        WorkSched<T::SPLIT_K> sched(cluster_id, num_clusters, p);
        WorkItem w;
        for (; sched.next(w); titer++) {
            int mb, nb;
            tile_to_mn(w.tile, p.num_m_blocks, p.num_n_blocks, p.group_n, mb, nb);
            // two row blocks per CTA: epilogue group eg drains the accumulator of row block eg
            const int blk = (T::MB == 2) ? eg : 0;
            const bool half = T::MB == 2 && w.half >= 0;     // only row block 0 holds a result: group 1 just hands the buffer back
            const int m0 = half ? mb * T::BM + w.half * (T::BM / 2) + (int)cta_rank * 128 : mb * T::BM + (int)cta_rank * T::BM_CTA + blk * 128;
            const int n0 = nb * BN;
            const int acc = titer % T::ACC_STAGES;
            const uint32_t acc_phase = (titer / T::ACC_STAGES) & 1;
            // all 128 epilogue threads must take the same decision, or the ones that go on would
            // wait at a named barrier for the ones that left
            const bool got = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, ST_TIMEOUT_EPILOGUE, acc, p.wait_sleep_ns);
            if (!named_bar_and(bar_b, 128, got)) break;
            tc_fence_after_sync();
            const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * T::ACC_STAGE_COLS + blk * T::ACC_STRIDE);
            const int grow = m0 + row_in_tile;
            // hands the drained accumulator buffer back to the MMA issuer
            auto release_acc = [&]() {
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (CG == 1) mbar_arrive(tempty_bar(acc));
                    else mbar_arrive_cluster(tempty_leader + 8u * acc);
                }
            };

            if (half && eg == 1) {
                release_acc();
                if constexpr (T::SENDER_WARPS > 0) {
                    if (p.forward && epi_tid == 0) smem_counter_add_release(smem_u32(const_cast<uint32_t *>(stored_count + eg)));
                }
            } else if (T::SPLIT_K == 0 && w.part >= 0) {
                // stream-K partial: the CTA's private slot, tile-local [BM][BN] layout, no bounds
                float *slot = p.workspace + ((size_t)(2 * cluster_id + w.part) * T::BM + cta_rank * T::BM_CTA + row_in_tile) * BN;
#pragma unroll 1
                for (int c0 = eg * 16; c0 < BN; c0 += 16 * EG) {
                    uint32_t r[16];
                    tmem_ld_32x16(t_row + (uint32_t)c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 4; c++)
                        *reinterpret_cast<uint4 *>(slot + c0 + c * 4) = make_uint4(r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]);
                }
                release_acc();
            } else if constexpr (T::SPLIT_K > 1) {
                // FP32 partial of this K slice into workspace[split][M][N]
#pragma unroll 1
                for (int c0 = eg * 16; c0 < BN; c0 += 16 * EG) {
                    uint32_t r[16];
                    tmem_ld_32x16(t_row + (uint32_t)c0, r);
                    tmem_ld_wait();
                    if (grow < p.M) {
                        float *dst = p.workspace + ((size_t)w.part * p.M + grow) * p.N + n0 + c0;
                        SM100_BOUNDS(n0 + c0 >= p.N || (((size_t)w.part * p.M + grow) * p.N + n0 + c0 + 4 <= (size_t)T::SPLIT_K * p.M * p.N && w.part < T::SPLIT_K),
                                     ST_BOUNDS_STORE, grow);
#pragma unroll
                        for (int c = 0; c < 4; c++)
                            if (n0 + c0 + c * 4 < p.N)
                                *reinterpret_cast<uint4 *>(dst + c * 4) = make_uint4(r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]);
                    }
                }
                release_acc();
            } else if constexpr (T::EPI == EPI_TMA) {
                // bf16 through swizzled shared memory and TMA stores of 128 x 64 boxes
                constexpr int J_STEP = (T::MB == 2) ? 1 : EG;     // pieces alternate between the groups unless each has its own row block
#pragma unroll 1
                for (int j = (T::MB == 2) ? 0 : eg; j < BN / 64; j += J_STEP) {
                    // the store that last read this staging buffer must have finished reading it (a group owns one
                    // buffer, or two that it uses in turn)
                    constexpr int NBUF = T::STAGING_BUFS / EG;      // buffers this group owns
                    if (epi_tid == 0) tma_store_wait_read<NBUF - 1>();
                    named_bar_sync(bar_a, 128);
                    const uint32_t stg = stg_base + (eg * NBUF + (NBUF == 2 ? buf : 0)) * (T::EPI_ROWS * 128);
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        uint32_t r[32];
                        tmem_ld_32x32(t_row + (uint32_t)(j * 64 + h * 32), r);
                        tmem_ld_wait();
                        uint32_t pk[16];
#pragma unroll
                        for (int i = 0; i < 16; i++) {
                            float lo = __uint_as_float(r[2 * i]), hi = __uint_as_float(r[2 * i + 1]);
                            if constexpr (T::OPK == OPK_E4M3) { lo *= p.alpha; hi *= p.alpha; }
                            pk[i] = pack_bf16x2(lo, hi);
                        }
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            const uint32_t chunk = (uint32_t)((h * 4 + c) ^ (row_in_tile & 7));
                            st_shared_v4(stg + row_in_tile * 128 + chunk * 16, pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
                        }
                    }
                    if (j + J_STEP >= BN / 64) release_acc();       // this group's last piece of the accumulator
                    fence_proxy_async_smem();
                    named_bar_sync(bar_a, 128);
                    if (p.y_mc != nullptr && !(T::SENDER_WARPS > 0 && p.forward)) {
                        // all-gather through NVSwitch: eight lanes read one staged 128-byte row piece and store it
                        // once to the multicast address (16 rows per pass); the barrier at the top of the next
                        // round keeps writers off this buffer until every reader is done
                        const int piece = epi_tid & 7;
                        const int ccol = n0 + j * 64 + piece * 8;
#pragma unroll 2
                        for (int r0 = 0; r0 < T::EPI_ROWS; r0 += 16) {
                            const int r = r0 + (epi_tid >> 3);
                            uint32_t a, b, c, d;
                            ld_shared_v4(stg + r * 128 + ((piece ^ (r & 7)) << 4), a, b, c, d);
                            if (m0 + r < p.M && ccol + 8 <= p.N)
                                multimem_st_v4(p.y_mc + (size_t)(m0 + r) * p.y_ld + p.y_col_offset + ccol, a, b, c, d);
                        }
                    } else if (epi_tid == 0) {
                        // stores must not start at a negative coordinate, and x must sit on a 16-byte boundary
                        SM100_BOUNDS(m0 >= 0 && p.y_col_offset + n0 + j * 64 >= 0 && ((p.y_col_offset + n0 + j * 64) * 2) % 16 == 0, ST_BOUNDS_STORE, m0);
                        for (int t = 0; t < p.y_targets; t++) tma_store_2d(&tmap_ys.m[t], stg, p.y_col_offset + n0 + j * 64, m0);
                        tma_store_commit();
                    }
                    buf ^= 1;
                }
                if constexpr (T::SENDER_WARPS > 0) {
                    // N-sharded run: this group's row block of the tile is on its way to the local result; once the
                    // stores are complete the senders may read it back (from L2) and forward it to the other ranks
                    if (p.forward && epi_tid == 0) {
                        tma_store_wait<0>();
                        fence_proxy_async_global();
                        smem_counter_add_release(smem_u32(const_cast<uint32_t *>(stored_count + eg)));
                    }
                }
            } else if constexpr (T::EPI == EPI_FUSED) {
                // D = act(alpha * acc + beta * C + bias) from registers; bf16 out (32 bytes per thread and step) or
                // e4m3(D * y_scale) (16 bytes) with the running max|D| folded into *amax once per warp and tile
                float tmax = 0.f;
#pragma unroll 1
                for (int c0 = eg * 16; c0 < BN; c0 += 16 * EG) {
                    uint32_t r[16];
                    tmem_ld_32x16(t_row + (uint32_t)c0, r);
                    tmem_ld_wait();
                    const int col = n0 + c0;
                    const bool row_ok = grow < p.M;
                    float v[16];
#pragma unroll
                    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]) * p.alpha;
                    if (p.C != nullptr && row_ok) {
                        const bf16 *cp = p.C + (size_t)grow * p.N + col;
#pragma unroll
                        for (int h = 0; h < 2; h++)
                            if (col + 8 * h < p.N) {
                                const uint4 c4 = *reinterpret_cast<const uint4 *>(cp + 8 * h);
                                const uint32_t cw[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
                                for (int i = 0; i < 4; i++) {
                                    v[8 * h + 2 * i] = fmaf(p.beta, __uint_as_float(cw[i] << 16), v[8 * h + 2 * i]);
                                    v[8 * h + 2 * i + 1] = fmaf(p.beta, __uint_as_float(cw[i] & 0xffff0000u), v[8 * h + 2 * i + 1]);
                                }
                            }
                    }
                    if (p.bias != nullptr) {
#pragma unroll
                        for (int h = 0; h < 2; h++)
                            if (col + 8 * h < p.N) {
                                const uint4 b4 = __ldg(reinterpret_cast<const uint4 *>(p.bias + col + 8 * h));
                                const uint32_t bw[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
                                for (int i = 0; i < 4; i++) {
                                    v[8 * h + 2 * i] += __uint_as_float(bw[i] << 16);
                                    v[8 * h + 2 * i + 1] += __uint_as_float(bw[i] & 0xffff0000u);
                                }
                            }
                    }
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        float x = v[i];
                        if (p.act == ACT_RELU) x = fmaxf(x, 0.f);
                        else if (p.act == ACT_GELU) x = 0.5f * x * erfcf(-x * 0.70710678118654752f);   // 1 + erf(t) = erfc(-t): no cancellation for x << 0
                        else if (p.act == ACT_SILU) x = x / (1.f + __expf(-x));
                        v[i] = x;
                        if (row_ok && col + i < p.N) tmax = fmaxf(tmax, fabsf(x));
                    }
                    if (row_ok) {
                        if (p.y_dtype == YOUT_E4M3) {
                            uint32_t q[4];
#pragma unroll
                            for (int i = 0; i < 4; i++)
                                q[i] = pack_e4m3x4(v[4 * i] * p.y_scale, v[4 * i + 1] * p.y_scale, v[4 * i + 2] * p.y_scale, v[4 * i + 3] * p.y_scale);
                            uint8_t *dst = static_cast<uint8_t *>(p.Y) + (size_t)grow * p.N + col;
                            if (col < p.N) *reinterpret_cast<uint2 *>(dst) = make_uint2(q[0], q[1]);
                            if (col + 8 < p.N) *reinterpret_cast<uint2 *>(dst + 8) = make_uint2(q[2], q[3]);
                        } else {
                            uint32_t pk[8];
#pragma unroll
                            for (int i = 0; i < 8; i++) pk[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
                            bf16 *dst = static_cast<bf16 *>(p.Y) + (size_t)grow * p.N + col;
                            if (col < p.N) *reinterpret_cast<uint4 *>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                            if (col + 8 < p.N) *reinterpret_cast<uint4 *>(dst + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                        }
                    }
                }
                release_acc();
                if (p.amax != nullptr) {
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
                    // non-negative floats order like their bit patterns
                    if (lane == 0 && tmax > 0.f) atomicMax(reinterpret_cast<unsigned int *>(p.amax), __float_as_uint(tmax));
                }
            } else {
                // bf16 straight from registers: 32 bytes per thread and step
#pragma unroll 1
                for (int c0 = eg * 16; c0 < BN; c0 += 16 * EG) {
                    uint32_t r[16];
                    tmem_ld_32x16(t_row + (uint32_t)c0, r);
                    tmem_ld_wait();
                    uint32_t pk[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        float lo = __uint_as_float(r[2 * i]), hi = __uint_as_float(r[2 * i + 1]);
                        if constexpr (T::OPK == OPK_E4M3) { lo *= p.alpha; hi *= p.alpha; }
                        pk[i] = pack_bf16x2(lo, hi);
                    }
                    if (grow < p.M) {
                        bf16 *dst = static_cast<bf16 *>(p.Y) + (size_t)grow * p.N + n0 + c0;
                        SM100_BOUNDS(n0 + c0 >= p.N || ((size_t)grow * p.N + n0 + c0 + 8 <= (size_t)p.M * p.N && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0),
                                     ST_BOUNDS_STORE, grow);
                        if (n0 + c0 < p.N) *reinterpret_cast<uint4 *>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                        if (n0 + c0 + 8 < p.N) *reinterpret_cast<uint4 *>(dst + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                    }
                }
                release_acc();
            }
        }
        if constexpr (T::EPI == EPI_TMA) {
            if (epi_tid == 0) tma_store_wait<0>();
        }
    } else if (warp >= 4 + 4 * T::EPI_GROUPS) {
        // ------------------------------------------------------------------ senders (N-sharded run, tiles forwarded from L2)
        if constexpr (T::SENDER_WARPS > 0) {
            if (p.forward) {
                const int st = threadIdx.x - (128 + 128 * T::EPI_GROUPS);    // 0 .. 127
                const int chunk = st & 31;                                    // 16-byte piece of a 512-byte tile row
                const bf16 *local = static_cast<const bf16 *>(p.Y);          // this rank's own copy of the result
                int titer = 0;
                WorkSched<T::SPLIT_K> sched(cluster_id, num_clusters, p);
                WorkItem w;
                for (; sched.next(w); titer++) {
                    int mb, nb;
                    tile_to_mn(w.tile, p.num_m_blocks, p.num_n_blocks, p.group_n, mb, nb);
                    const bool half = w.half >= 0;
                    const int m0 = half ? mb * T::BM + w.half * (T::BM / 2) + (int)cta_rank * 128 : mb * T::BM + (int)cta_rank * T::BM_CTA;
                    const int rows = half ? 128 : T::BM_CTA;
                    const int col = nb * BN + chunk * 8;
                    // work item number titer is stored once every epilogue group has counted it
                    if (!smem_counter_wait(smem_u32(const_cast<uint32_t *>(stored_count)), (uint32_t)(titer + 1), abort_flag, p.status, ST_TIMEOUT_EPILOGUE, 8) ||
                        (T::EPI_GROUPS == 2 &&
                         !smem_counter_wait(smem_u32(const_cast<uint32_t *>(stored_count + 1)), (uint32_t)(titer + 1), abort_flag, p.status, ST_TIMEOUT_EPILOGUE, 9)))
                        break;
                    if (col + 8 > p.N) continue;
                    const size_t off0 = (size_t)p.y_col_offset + col;
                    // one warp per row and pass, four rows in flight per thread: loads come from L2 (the tile was just stored),
                    // bypassing L1, which may hold this address from an earlier step
#pragma unroll 1
                    for (int r0 = st >> 5; r0 < rows; r0 += 16) {
                        uint4 v[4];
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const int r = m0 + r0 + 4 * u;
                            if (r < p.M) v[u] = __ldcg(reinterpret_cast<const uint4 *>(local + (size_t)r * p.y_ld + off0));
                        }
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const int r = m0 + r0 + 4 * u;
                            if (r < p.M) multimem_st_v4(p.y_mc + (size_t)r * p.y_ld + off0, v[u].x, v[u].y, v[u].z, v[u].w);
                        }
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    __syncwarp();
    if (*abort_flag) {
        // give copies and MMAs still in flight time to land before shared memory and TMEM go away
        for (int i = 0; i < 64; i++) __nanosleep(1000);
    }
    tc_fence_before_sync();
    if constexpr (CG == 2) cluster_sync_all(); else __syncthreads();
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc<CG>(tmem_base, T::TMEM_COLS);
    }
}

// FP32 partial sums -> bf16: Y[i] = bf16(sum_s ws[s][i]), splits added in ascending order
// (the reference's order, src/bf16_gemm.cuh:839-845).  Eight outputs per thread: two 128-bit
// loads per split, one 128-bit store; grid-stride over M*N/8 groups.  Pure HBM traffic:
// (4*SPLIT_K + 2) bytes per output.  The reference's version handles one element per thread
// with 4-byte loads and 2-byte stores (src/bf16_gemm.cuh:833-846).
template <int SPLIT_K>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float *__restrict__ ws, bf16 *__restrict__ Y, size_t mn, float alpha)
{
    // launched as a programmatic dependent of the GEMM kernel: its blocks may already sit on the
    // SMs while the GEMM drains; this waits (in hardware) until that grid is complete and visible
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const size_t groups = mn / 8;
    for (size_t g = (size_t)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += (size_t)gridDim.x * blockDim.x) {
        const float4 *src = reinterpret_cast<const float4 *>(ws + g * 8);
        float4 a = __ldcs(src), b = __ldcs(src + 1);
#pragma unroll
        for (int s = 1; s < SPLIT_K; s++) {
            const float4 *ps = reinterpret_cast<const float4 *>(ws + (size_t)s * mn + g * 8);
            float4 c = __ldcs(ps), d = __ldcs(ps + 1);
            a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w;
            b.x += d.x; b.y += d.y; b.z += d.z; b.w += d.w;
        }
        uint4 o;
        o.x = pack_bf16x2(a.x * alpha, a.y * alpha);
        o.y = pack_bf16x2(a.z * alpha, a.w * alpha);
        o.z = pack_bf16x2(b.x * alpha, b.y * alpha);
        o.w = pack_bf16x2(b.z * alpha, b.w * alpha);
        *reinterpret_cast<uint4 *>(Y + g * 8) = o;
    }
}

// Adds up the stream-K partials of every tile that more than one CTA worked on and writes the
// bf16 result; contributions are added in ascending K order (ascending CTA index).  Each tile
// is cut into `parts` row slices (one block each) so that all SMs take part; 8 outputs per
// thread, 128-bit loads and stores.  Tiles that one CTA computed whole were already written
// by the GEMM kernel and are skipped.
template <int BM, int BN>
__global__ void __launch_bounds__(256) streamk_reduce_kernel(const float *__restrict__ ws, bf16 *__restrict__ Y, int M, int N,
                                                             int num_m, int num_n, int group_n, int kb_per_tile,
                                                             int num_clusters, int parts, float alpha)
{
    asm volatile("griddepcontrol.wait;" ::: "memory");   // programmatic dependent of the GEMM kernel
    const int tile = blockIdx.x / parts, part = blockIdx.x - tile * parts;
    const long long units = (long long)num_m * num_n * kb_per_tile;
    const long long t0 = (long long)tile * kb_per_tile;
    const int c_lo = streamk_owner(units, t0, num_clusters);
    const int c_hi = streamk_owner(units, t0 + kb_per_tile - 1, num_clusters);
    if (c_lo == c_hi) return;
    int mb, nb;
    tile_to_mn(tile, num_m, num_n, group_n, mb, nb);
    const int rows_per_part = BM / parts;
    constexpr int VEC_PER_ROW = BN / 8;
    for (int it = threadIdx.x; it < rows_per_part * VEC_PER_ROW; it += blockDim.x) {
        const int r = part * rows_per_part + it / VEC_PER_ROW;
        const int c8 = (it % VEC_PER_ROW) * 8;
        const int grow = mb * BM + r, gcol = nb * BN + c8;
        if (grow >= M || gcol >= N) continue;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        for (int c = c_lo; c <= c_hi; c++) {
            const int slot = streamk_range_begin(units, c, num_clusters) >= t0 ? 0 : 1;
            const float4 *src = reinterpret_cast<const float4 *>(ws + ((size_t)(2 * c + slot) * BM + r) * BN + c8);
            const float4 x = __ldcg(src), y = __ldcg(src + 1);
            if (c == c_lo) { a = x; b = y; }
            else {
                a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
                b.x += y.x; b.y += y.y; b.z += y.z; b.w += y.w;
            }
        }
        uint4 o;
        o.x = pack_bf16x2(a.x * alpha, a.y * alpha);
        o.y = pack_bf16x2(a.z * alpha, a.w * alpha);
        o.z = pack_bf16x2(b.x * alpha, b.y * alpha);
        o.w = pack_bf16x2(b.z * alpha, b.w * alpha);
        *reinterpret_cast<uint4 *>(Y + (size_t)grow * N + gcol) = o;
    }
}

// ---------------------------------------------------------------------------------- host side
// Upper bound on resident CTAs used to size the stream-K workspace without asking a device.
static constexpr int STREAMK_MAX_CTAS = 160;

// Launch configuration of a kernel that follows the GEMM kernel on the same stream as its
// programmatic dependent (it calls griddepcontrol.wait before touching the GEMM's output).
inline cudaLaunchConfig_t dependent_launch_config(unsigned blocks, unsigned threads, cudaStream_t stream)
{
    static cudaLaunchAttribute attr = []() {
        cudaLaunchAttribute a;
        a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        a.val.programmaticStreamSerializationAllowed = 1;
        return a;
    }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return cfg;
}

// Back-off cap of the long waits, in ns: 4 ns per k-block of a tile, at most 1024, so short tiles keep
// their latency.
inline int wait_sleep_ns(int num_k_blocks)
{
    const int v = num_k_blocks * 4;
    return v > 1024 ? 1024 : v;
}

// Width of a rasterisation band in tiles.
inline int band_width(int bn, int mb = 1)
{
    // 512-row tiles: measured at 16384^3 over forty back-to-back launches (power-capped clocks), mean of six runs each:
    // 16 columns 6.53 ms (one run in six at 6.02, the others 6.55-6.74), 14 columns 6.20 ms (6.12-6.31), 12 columns
    // 6.27 ms, 10 columns 6.29 ms, 8 columns 6.85 ms, 32 columns 6.68 ms; the library GEMM took 6.01-6.06 ms beside them
    if (mb == 2) return 14;
    return bn >= 256 ? 8 : 16;
}

// Everything a launch can ask for beyond the operands; the defaults are the plain GEMM.
struct LaunchExtras {
    float alpha = 1.0f;                   // scales the accumulator (FP8 per-tensor: sx * sw, times the caller's alpha)
    int sm_limit = 0;
    const void *sf_x = nullptr, *sf_w = nullptr;   // block-scaled kinds: tiled ue8m0 scales
    const YTarget *yt = nullptr;          // N-sharded run: store into every rank's matrix
    // fused output transform (EPI_FUSED plugins only)
    const void *C = nullptr;
    const void *bias = nullptr;
    float beta = 0.0f;
    int act = ACT_NONE;
    int y_dtype = YOUT_BF16;
    float y_scale = 1.0f;
    float *amax = nullptr;
    int test_withhold_kb = -1;
};

template <class T>
struct UmmaGemmLauncher {
    static bool can_run(int M, int N, int K)
    {
        if (M <= 0 || N <= 0 || K <= 0) return false;
        if (((long long)K * T::ELEM_BITS) % 128 != 0 || N % 8 != 0) return false;   // 16-byte row pitches
        if (T::BLOCK_SCALED && K % T::BK != 0) return false;               // whole scale atoms along K
        if (T::SPLIT_K > 1) {
            int kb = (K + T::BK - 1) / T::BK;
            if (K % T::BK != 0 || kb % T::SPLIT_K != 0) return false;     // equal, non-empty K slices
        }
        return true;
    }

    static size_t workspace_bytes(int M, int N, int K)
    {
        (void)K;
        if (T::SPLIT_K == 0)   // two partial-tile slots per CTA (pair), whatever the shape
            return (size_t)2 * (STREAMK_MAX_CTAS / T::CG) * T::BM * T::BN * sizeof(float);
        return T::SPLIT_K > 1 ? (size_t)T::SPLIT_K * M * N * sizeof(float) : 0;
    }

    // persistent grid: as many CTAs (CTA pairs) as can be resident at once, capped by the
    // tile count and by `sm_limit`
    // `balance`: with a fixed work list, shrink the grid to ceil(work / waves) units, the smallest grid that
    // still finishes in the same number of waves.  Nothing waits for a half-empty last wave then, and at the
    // power cap the SMs left out pay for a higher clock on the ones that work (256 tiles on 74 CTA pairs take
    // four rounds either way; on 64 pairs no pair idles during the fourth).
    static int grid_size(const DeviceInfo &dev, int total_tiles, int sm_limit, int *out, bool balance = false)
    {
        static std::atomic<int> max_clusters[MAX_DEVICES];   // 0 = not asked yet; racing first calls compute the same value
        int devid = 0;
        SM100_CUDA_TRY(cudaGetDevice(&devid));
        int sms = dev.sm_count;
        if (T::CG == 2) {
            if (max_clusters[devid].load(std::memory_order_acquire) == 0) {
                cudaLaunchConfig_t cfg = {};
                cfg.gridDim = dim3(dev.sm_count - dev.sm_count % 2);
                cfg.blockDim = dim3(T::THREADS);
                cfg.dynamicSmemBytes = T::SMEM_ALLOC;
                cudaLaunchAttribute attr;
                attr.id = cudaLaunchAttributeClusterDimension;
                attr.val.clusterDim.x = 2;
                attr.val.clusterDim.y = 1;
                attr.val.clusterDim.z = 1;
                cfg.attrs = &attr;
                cfg.numAttrs = 1;
                int n = 0;
                SM100_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, umma_gemm_kernel<T>, &cfg));
                if (n <= 0) return set_error(GEMM_ERR_CUDA, "no CTA pair of this configuration fits on the device");
                max_clusters[devid].store(n, std::memory_order_release);
            }
            sms = 2 * max_clusters[devid].load(std::memory_order_acquire);
            if (sms > dev.sm_count) sms = dev.sm_count - dev.sm_count % 2;
        }
        if (sm_limit > 0 && sm_limit < sms) sms = sm_limit;
        int units = sms / T::CG;
        if (units < 1) units = 1;
        if (units > total_tiles) units = total_tiles;
        if (balance && T::SPLIT_K >= 1) units = balanced_units(total_tiles, units);
        *out = units * T::CG;
        return GEMM_OK;
    }

    static int run(int M, int N, int K, const void *X, const void *W, void *Y, float *workspace, size_t workspace_bytes_given,
                   cudaStream_t stream, const LaunchExtras &ex = LaunchExtras())
    {
        const float alpha = ex.alpha;
        const int sm_limit = ex.sm_limit;
        const void *sf_x = ex.sf_x, *sf_w = ex.sf_w;
        const YTarget *yt = ex.yt;
        if (!can_run(M, N, K)) return set_error(GEMM_ERR_SHAPE, "shape %dx%dx%d not supported by this configuration", M, N, K);
        const bool fused_gather = yt != nullptr && yt->num_peers > 0;
        if (fused_gather) {
            if (T::EPI != EPI_TMA) return set_error(GEMM_ERR_ARG, "storing into peer matrices needs a TMA-store configuration (e1, no split-K)");
            if (yt->num_peers > MAX_Y_PEERS || !yt->peers || yt->ld < yt->col_offset + (long long)N || yt->ld % 8 != 0 || yt->col_offset % 8 != 0)
                return set_error(GEMM_ERR_ARG, "bad peer destination: %d peers, ld %lld, column offset %d", yt->num_peers, yt->ld, yt->col_offset);
        }
        if (!X || !W || (!Y && !fused_gather)) return set_error(GEMM_ERR_ARG, "null operand pointer");
        const bool wants_transform = ex.C || ex.bias || ex.beta != 0.0f || ex.act != ACT_NONE || ex.y_dtype != YOUT_BF16 || ex.amax ||
                                     (T::OPK != OPK_E4M3 && ex.alpha != 1.0f);
        if (wants_transform && T::EPI != EPI_FUSED)
            return set_error(GEMM_ERR_ARG, "bias / beta*C / activation / e4m3 output need a fused-epilogue configuration (e2)");
        if (T::EPI == EPI_FUSED) {
            if (ex.act < ACT_NONE || ex.act > ACT_SILU || (ex.y_dtype != YOUT_BF16 && ex.y_dtype != YOUT_E4M3))
                return set_error(GEMM_ERR_ARG, "unknown activation %d or output type %d", ex.act, ex.y_dtype);
            if (ex.beta != 0.0f && !ex.C) return set_error(GEMM_ERR_ARG, "beta != 0 needs C");
            if (((reinterpret_cast<uintptr_t>(ex.C) | reinterpret_cast<uintptr_t>(ex.bias)) & 15u) != 0 || (reinterpret_cast<uintptr_t>(Y) & 15u) != 0)
                return set_error(GEMM_ERR_ARG, "C, bias and Y must be 16-byte aligned");
        }
        if (T::BLOCK_SCALED && (!sf_x || !sf_w)) return set_error(GEMM_ERR_ARG, "block-scaled configuration needs x_scale and w_scale");
        if (T::BLOCK_SCALED && ((reinterpret_cast<uintptr_t>(sf_x) | reinterpret_cast<uintptr_t>(sf_w)) & 15u))
            return set_error(GEMM_ERR_ARG, "scale arrays must be 16-byte aligned");
        if (T::SPLIT_K != 1) {
            if (!workspace) return set_error(GEMM_ERR_WORKSPACE, "split-K configuration needs a workspace");
            if (workspace_bytes_given != 0 && workspace_bytes_given < workspace_bytes(M, N, K))
                return set_error(GEMM_ERR_WORKSPACE, "workspace has %zu bytes, %zu needed", workspace_bytes_given, workspace_bytes(M, N, K));
            if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return set_error(GEMM_ERR_ARG, "workspace must be 16-byte aligned");
        }
        DeviceInfo *dev = nullptr;
        int rc = device_info(&dev);
        if (rc != GEMM_OK) return rc;
        if (T::SMEM_ALLOC > dev->max_smem_optin)
            return set_error(GEMM_ERR_CUDA, "configuration needs %d bytes of shared memory, device allows %d", T::SMEM_ALLOC, dev->max_smem_optin);

        static std::atomic<bool> attr_set[MAX_DEVICES];   // setting the attribute twice is harmless, so a flag per device is enough
        int devid = 0;
        SM100_CUDA_TRY(cudaGetDevice(&devid));
        if (!attr_set[devid].load(std::memory_order_acquire)) {
            SM100_CUDA_TRY(cudaFuncSetAttribute(umma_gemm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_ALLOC));
            attr_set[devid].store(true, std::memory_order_release);
        }

        const CUtensorMapDataType dt = (T::OPK == OPK_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
        CUtensorMap tx, tw;
        YMaps tys;
        const uint64_t row_bytes = (uint64_t)K * T::ELEM_BITS / 8;
        const uint64_t row_elems = (T::OPK == OPK_BF16) ? (uint64_t)K : row_bytes;   // fp8 / packed fp4 rows are mapped as bytes
        rc = make_tmap_2d(&tx, dt, X, row_elems, (uint64_t)M, row_bytes, T::BK_COORD, T::BM_CTA, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != GEMM_OK) return rc;
        rc = make_tmap_2d(&tw, dt, W, row_elems, (uint64_t)N, row_bytes, T::BK_COORD, T::BN_CTA, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != GEMM_OK) return rc;
        CUtensorMap tsfx = tx, tsfw = tx;   // placeholders unless block-scaled
        if (T::MB == 2) {
            // X again with a box of 128 rows, for the halves of the last wave
            rc = make_tmap_2d(&tsfx, dt, X, row_elems, (uint64_t)M, row_bytes, T::BK_COORD, 128, CU_TENSOR_MAP_SWIZZLE_128B);
            if (rc != GEMM_OK) return rc;
        }
        if (T::BLOCK_SCALED) {
            const uint64_t k_atoms = ((uint64_t)K + 127) / 128;
            rc = make_tmap_2d(&tsfx, CU_TENSOR_MAP_DATA_TYPE_UINT8, sf_x, 256, ((uint64_t)M + 127) / 128 * k_atoms * 2, 256, 256, 2,
                              CU_TENSOR_MAP_SWIZZLE_NONE);
            if (rc != GEMM_OK) return rc;
            rc = make_tmap_2d(&tsfw, CU_TENSOR_MAP_DATA_TYPE_UINT8, sf_w, 256, ((uint64_t)N + 127) / 128 * k_atoms * 2, 256, 256, 2,
                              CU_TENSOR_MAP_SWIZZLE_NONE);
            if (rc != GEMM_OK) return rc;
        }
        int y_targets = 1;
        if (fused_gather && yt->multicast) {
            if (N % 8 != 0 || (reinterpret_cast<uintptr_t>(yt->multicast) & 15u))
                return set_error(GEMM_ERR_ARG, "multicast stores need N %% 8 == 0 and a 16-byte aligned address");
            y_targets = 0;
            tys.m[0] = tx;
            if (T::SENDER_WARPS > 0 && (T::MB == 2 || yt->forward)) {
                // the tile goes to this rank's own matrix first (peers[0], by contract the local one when a multicast
                // address is given); the sender warps forward it from there
                if (!yt->peers[0]) return set_error(GEMM_ERR_ARG, "null local destination (y_peers[0])");
                y_targets = 1;
                rc = make_tmap_2d(&tys.m[0], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, yt->peers[0], (uint64_t)(yt->col_offset + N), (uint64_t)M,
                                  (uint64_t)yt->ld * 2, T::OUT_CHUNK, T::EPI_ROWS, CU_TENSOR_MAP_SWIZZLE_128B);
                if (rc != GEMM_OK) return rc;
            }
        } else if (fused_gather) {
            // one map per rank's matrix; the extent stops at this block's last column so that a partial last
            // tile is clipped there and cannot spill into the next rank's columns
            y_targets = yt->num_peers;
            for (int t = 0; t < y_targets; t++) {
                if (!yt->peers[t]) return set_error(GEMM_ERR_ARG, "null peer pointer %d", t);
                rc = make_tmap_2d(&tys.m[t], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, yt->peers[t], (uint64_t)(yt->col_offset + N), (uint64_t)M,
                                  (uint64_t)yt->ld * 2, T::OUT_CHUNK, T::EPI_ROWS, CU_TENSOR_MAP_SWIZZLE_128B);
                if (rc != GEMM_OK) return rc;
            }
        } else if (T::EPI == EPI_TMA) {
            rc = make_tmap_2d(&tys.m[0], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, Y, (uint64_t)N, (uint64_t)M, (uint64_t)N * 2, T::OUT_CHUNK, T::EPI_ROWS,
                              CU_TENSOR_MAP_SWIZZLE_128B);
            if (rc != GEMM_OK) return rc;
        } else {
            tys.m[0] = tx;
        }

        GemmParams p;
        p.M = M; p.N = N; p.K = K;
        p.num_m_blocks = (M + T::BM - 1) / T::BM;
        p.num_n_blocks = (N + T::BN - 1) / T::BN;
        p.num_k_blocks = ((K + T::BK - 1) / T::BK) / (T::SPLIT_K > 0 ? T::SPLIT_K : 1);
        p.group_n = band_width(T::BN, T::MB);
        // with a single accumulator stage the epilogue's wake-up is on the critical path of every tile
        p.wait_sleep_ns = wait_sleep_ns(T::ACC_STAGES == 1 ? (p.num_k_blocks < 16 ? p.num_k_blocks : 16) : p.num_k_blocks);
        p.forward = (fused_gather && yt->multicast && T::SENDER_WARPS > 0 && (T::MB == 2 || yt->forward)) ? 1 : 0;
        p.Y = p.forward ? yt->peers[0] : Y;
        p.workspace = workspace;
        p.alpha = alpha;
        p.status = dev->status;
        p.y_targets = y_targets;
        p.y_col_offset = fused_gather ? yt->col_offset : 0;
        p.y_mc = fused_gather ? static_cast<bf16 *>(yt->multicast) : nullptr;
        p.y_ld = fused_gather ? yt->ld : 0;
        p.sf_k_atoms = (K + 127) / 128;
        p.C = static_cast<const bf16 *>(ex.C);
        p.bias = static_cast<const bf16 *>(ex.bias);
        p.beta = ex.C ? ex.beta : 0.0f;
        p.y_scale = ex.y_scale;
        p.amax = ex.amax;
        p.act = ex.act;
        p.y_dtype = ex.y_dtype;
        p.test_withhold_kb = ex.test_withhold_kb;
        const long long work = (long long)p.num_m_blocks * p.num_n_blocks * (T::SPLIT_K > 0 ? T::SPLIT_K : p.num_k_blocks);
        int grid = 0;
        // compute-bound shapes only: a memory-bound one (M <= 128 rows) wants every SM's loads in flight
        rc = grid_size(*dev, work > (1 << 30) ? (1 << 30) : (int)work, sm_limit, &grid, M >= 512);
        if (rc != GEMM_OK) return rc;
        p.tail_full = -1;
        p.wave_sync = nullptr;
        if (T::MB == 2 && T::SPLIT_K == 1) {
            // the tiles of the last wave, when they would leave at least half of the clusters idle, go out as halves
            int full_grid = 0;
            rc = grid_size(*dev, work > (1 << 30) ? (1 << 30) : (int)work, sm_limit, &full_grid, false);
            if (rc != GEMM_OK) return rc;
            const int clusters = full_grid / T::CG;
            const int tiles = p.num_m_blocks * p.num_n_blocks;
            const int rest = tiles % clusters;
            if (tiles > clusters && rest > 0 && 2 * rest <= clusters) {
                p.tail_full = tiles - rest;
                grid = full_grid;
            }
        }
        if (T::MB == 2 && T::SPLIT_K == 1 && p.tail_full < 0 && !fused_gather && p.num_k_blocks >= 64 &&
            (long long)p.num_m_blocks * p.num_n_blocks >= 4LL * (grid / T::CG)) {
            // four waves or more of long tiles on one GPU: pace the clusters (see the producer); the counter is zeroed in
            // stream order.  (In an N-sharded run, where the sender warps' traffic shifts the clusters' timing anyway,
            // pacing measured neutral to 2 % slower on two GPUs and is left off.  Pacing the one-row-block kernels as well
            // changed none of FP8 8192^3, BF16 8192^3, 4096 x 28672 x 4096, MXFP8 and MX-FP4 8192^3: their tiles are
            // a quarter to a half as long and drift less.)
            uint32_t *slot = dev->wave_sync + dev->wave_next.fetch_add(1, std::memory_order_relaxed) % WAVE_SYNC_SLOTS;
            SM100_CUDA_TRY(cudaMemsetAsync(slot, 0, sizeof(uint32_t), stream));
            p.wave_sync = slot;
        }
        if (T::SPLIT_K == 0 && grid > STREAMK_MAX_CTAS) grid = STREAMK_MAX_CTAS - STREAMK_MAX_CTAS % T::CG;

        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(T::THREADS);
        cfg.dynamicSmemBytes = T::SMEM_ALLOC;
        cfg.stream = stream;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = T::CG;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        SM100_CUDA_TRY(cudaLaunchKernelEx(&cfg, umma_gemm_kernel<T>, tx, tw, tys, tsfx, tsfw, p));

        if (T::SPLIT_K == 0) {
            const int tiles = p.num_m_blocks * p.num_n_blocks;
            int parts = 1;
            while (parts < 32 && tiles * parts < 2 * dev->sm_count) parts *= 2;
            cudaLaunchConfig_t rc_cfg = dependent_launch_config(tiles * parts, 256, stream);
            SM100_CUDA_TRY(cudaLaunchKernelEx(&rc_cfg, streamk_reduce_kernel<T::BM, T::BN>, (const float *)workspace, static_cast<bf16 *>(Y), M, N,
                                              p.num_m_blocks, p.num_n_blocks, p.group_n, p.num_k_blocks, grid / T::CG, parts, alpha));
        }
        if (T::SPLIT_K > 1) {
            const size_t mn = (size_t)M * N;
            size_t blocks = (mn / 8 + 255) / 256;
            const size_t cap = (size_t)dev->sm_count * 8;
            if (blocks > cap) blocks = cap;
            cudaLaunchConfig_t rc_cfg = dependent_launch_config((unsigned)blocks, 256, stream);
            SM100_CUDA_TRY(cudaLaunchKernelEx(&rc_cfg, splitk_reduce_kernel<T::SPLIT_K>, (const float *)workspace, static_cast<bf16 *>(Y), mn, alpha));
        }
        return GEMM_OK;
    }
};

}  // namespace sm100

// The reference's two entry-point class templates (src/bf16_gemm.cuh:193 and :549), kept by name with a
// static run() of the same argument order; every bf16 plugin reaches its kernel through one of them (as the
// reference's entry template does, src/kernel_entry.cu.in:20-26).  The template parameters are the sm_100
// configuration space: tile rows BM = 128 x CTA_GROUP x (row blocks per CTA), BK fixed by the 128-byte swizzle
// span.  run() returns a GEMM_* status instead of exiting or throwing; run_ex() is run() with the arguments
// the reference does not have (SM limit, peer destinations, output transform).
template <int BM, int BN, int BK, int NUM_STAGES, int CTA_GROUP = 1, int EPI = sm100::EPI_TMA>
struct BF16GemmMMA {
    static constexpr int MB = BM / (128 * CTA_GROUP);
    using Traits = sm100::UmmaGemmTraits<sm100::OPK_BF16, BN, NUM_STAGES, CTA_GROUP, 1, EPI, MB>;
    using Launcher = sm100::UmmaGemmLauncher<Traits>;
    static_assert(BM == Traits::BM && BK == Traits::BK, "BM must be 128*CTA_GROUP*(1|2) and BK 64 for bf16");
    static int run(int M, int N, int K, const bf16 *X, const bf16 *W, bf16 *Y, cudaStream_t stream)
    {
        return Launcher::run(M, N, K, X, W, Y, nullptr, 0, stream);
    }
    static int run_ex(int M, int N, int K, const bf16 *X, const bf16 *W, void *Y, cudaStream_t stream, const sm100::LaunchExtras &ex)
    {
        return Launcher::run(M, N, K, X, W, Y, nullptr, 0, stream, ex);
    }
};

// SPLIT_K > 1: equal K slices, FP32 partials in `workspace`, reduce kernel; SPLIT_K == 0: stream-K.
template <int BM, int BN, int BK, int NUM_STAGES, int CTA_GROUP, int SPLIT_K>
struct BF16GemmMMASplitK {
    using Traits = sm100::UmmaGemmTraits<sm100::OPK_BF16, BN, NUM_STAGES, CTA_GROUP, SPLIT_K, sm100::EPI_DIRECT>;
    using Launcher = sm100::UmmaGemmLauncher<Traits>;
    static_assert(BM == Traits::BM && BK == Traits::BK, "BM must be 128*CTA_GROUP and BK 64 for bf16");
    // workspace: >= SPLIT_K*M*N floats, caller-owned, need not be zeroed (as src/bf16_gemm.cuh:601)
    static int run(int M, int N, int K, const bf16 *X, const bf16 *W, bf16 *Y, float *workspace, cudaStream_t stream)
    {
        return Launcher::run(M, N, K, X, W, Y, workspace, 0, stream);
    }
    static int run_ex(int M, int N, int K, const bf16 *X, const bf16 *W, void *Y, float *workspace, size_t workspace_bytes,
                      cudaStream_t stream, const sm100::LaunchExtras &ex)
    {
        return Launcher::run(M, N, K, X, W, Y, workspace, workspace_bytes, stream, ex);
    }
};
