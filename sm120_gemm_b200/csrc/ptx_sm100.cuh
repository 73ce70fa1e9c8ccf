// Thin inline-PTX wrappers for the sm_100a features the GEMM kernels use:
// mbarrier (with bounded waits), TMA tensor copies, tcgen05 (TMEM alloc, MMA, commit, ld).
//
// Same role as the PTX helper block of the reference (src/bf16_gemm.cuh:10-178), rebuilt
// for the Blackwell data-centre ISA.  Differences that matter:
//   * every wait is bounded: after WAIT_LIMIT_CYCLES without progress the waiter raises a
//     CTA-wide abort flag, records where it gave up and returns false.  The reference
//     spins forever (src/bf16_gemm.cuh:137-148).
//   * no TMA load carries a cluster-multicast qualifier anywhere in this file.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sm100 {

// A wait that sees no progress for this many SM clock cycles gives up: about 2 s at the
// 1.0-1.97 GHz the part runs at (the longest legitimate wait is one output tile's main loop,
// well under 10 ms even for K = 64k).  The SM's own cycle counter is used because it is cheap
// to read; %globaltimer is not.
#ifndef SM100_WAIT_LIMIT_CYCLES
#define SM100_WAIT_LIMIT_CYCLES 3000000000ll
#endif
static constexpr long long WAIT_LIMIT_CYCLES = SM100_WAIT_LIMIT_CYCLES;   // the wait-expiry test plugin is built with a short limit

// Codes written to the device status word by a wait that gave up.
enum : uint32_t {
    ST_OK = 0,
    ST_TIMEOUT_PRODUCER = 1,   // TMA producer waiting for a free ring slot
    ST_TIMEOUT_MMA_FULL = 2,   // MMA issuer waiting for operand data
    ST_TIMEOUT_MMA_ACC = 3,    // MMA issuer waiting for a drained accumulator
    ST_TIMEOUT_EPILOGUE = 4,   // epilogue waiting for a finished accumulator
    ST_TIMEOUT_DEQUANT = 5,    // dequantiser warps (W4A16)
    // -DGEMM_DEBUG_BOUNDS builds only: a computed coordinate or address failed its check
    ST_BOUNDS_LOAD_ROW = 16,   // TMA load: row coordinate outside the matrix (+ one tile of slack)
    ST_BOUNDS_LOAD_K = 17,     // TMA load: K coordinate outside the row or off a 16-byte boundary
    ST_BOUNDS_STORE = 18,      // store: address outside the destination or misaligned
};

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long globaltimer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// shared::cta address -> shared::cluster address of the same offset in CTA `rank`
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}

__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t nthreads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// barrier + AND-reduction of a predicate over the `nthreads` threads that use barrier `id`
__device__ __forceinline__ bool named_bar_and(uint32_t id, uint32_t nthreads, bool pred)
{
    uint32_t out;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\t"
        "bar.red.and.pred p, %2, %3, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(out)
        : "r"((uint32_t)pred), "r"(id), "r"(nthreads)
        : "memory");
    return out != 0;
}

// ---------------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_inval(uint32_t bar)
{
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// make barrier initialisation visible to the async proxy and to the other CTA of a cluster
__device__ __forceinline__ void fence_barrier_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// orders this thread's completed bulk (async-proxy) stores to global memory before what it does next in the generic proxy
__device__ __forceinline__ void fence_proxy_async_global()
{
    asm volatile("fence.proxy.async.global;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// arrive on a barrier that lives in another CTA of the cluster (address from mapa_shared)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done;
}

// Bounded wait.  Returns false when the CTA is aborting (this waiter or another one gave
// up); `abort_flag` is a word in shared memory, `status` the global status block
// (status[0] = code, [1] = blockIdx.x, [2] = detail) or nullptr.
// `sleep_cap_ns` > 0 makes a long wait cheap: between polls the thread sleeps 32 ns, then twice as long
// each time up to the cap, instead of polling back to back (warps that wait for most of a tile's main
// loop otherwise spend issue slots and power on the poll).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                          uint32_t *status, uint32_t code, uint32_t detail, uint32_t sleep_cap_ns = 0)
{
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = 0;
    uint32_t spins = 0;
    uint32_t ns = 32;
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if (sleep_cap_ns) {
            __nanosleep(ns);
            if (ns < sleep_cap_ns) ns <<= 1;
        }
        if ((++spins & (sleep_cap_ns ? 0xfu : 0xffu)) == 0) {
            if (*abort_flag) return false;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            if (now - t0 > WAIT_LIMIT_CYCLES) {
                *abort_flag = 1;
                if (status != nullptr && atomicCAS(status, 0u, code) == 0u) {
                    status[1] = blockIdx.x;
                    status[2] = detail;
                }
                return false;
            }
        }
    }
}

// A counter in shared memory as a one-way signal inside a CTA: the producer adds with release semantics, the consumer
// polls with acquire semantics until the count reaches its target.  Bounded like mbar_wait.
__device__ __forceinline__ void smem_counter_add_release(uint32_t addr)
{
    asm volatile("red.release.cta.shared::cta.add.u32 [%0], 1;" ::"r"(addr) : "memory");
}

__device__ __forceinline__ bool smem_counter_wait(uint32_t addr, uint32_t target, volatile uint32_t *abort_flag, uint32_t *status, uint32_t code,
                                                  uint32_t detail)
{
    long long t0 = 0;
    uint32_t spins = 0;
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
        if ((int32_t)(v - target) >= 0) return true;
        __nanosleep(256);
        if ((++spins & 0xfu) == 0) {
            if (*abort_flag) return false;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            if (now - t0 > WAIT_LIMIT_CYCLES) {
                *abort_flag = 1;
                if (status != nullptr && atomicCAS(status, 0u, code) == 0u) {
                    status[1] = blockIdx.x;
                    status[2] = detail;
                }
                return false;
            }
        }
    }
}

// ---------------------------------------------------------------------------------- TMA
// 2-D tile load global -> shared, completion counted on an mbarrier of this CTA.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// 3-D tile load (coordinates innermost first), completion counted on an mbarrier of this CTA.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y, int z)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// Same, for a CTA pair: the destination is this CTA's shared memory, the mbarrier may be
// the peer CTA's (a shared::cluster address).  No multicast: each CTA fetches its own tile.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t cluster_bar, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(x), "r"(y)
                 : "memory");
}

__device__ __forceinline__ void tma_store_commit()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// wait until at most N of this thread's store groups still READ shared memory
template <int N>
__device__ __forceinline__ void tma_store_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int N>
__device__ __forceinline__ void tma_store_wait()
{
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---------------------------------------------------------------------------------- tcgen05
// One lane of a fully active warp.  The tcgen05 issue loops run on ALL lanes of their warp with
// warp-uniform control flow and only the instructions themselves sit under this predicate: the
// descriptors are then warp-uniform values the compiler can keep in uniform registers, which is
// where tcgen05 instructions take their operands from.  (A loop run by a single diverged thread
// has to move every operand into uniform registers per instruction, ~60-80 cycles each.)
__device__ __forceinline__ bool elect_one_sync()
{
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

template <int CG>
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols)
{
    if constexpr (CG == 1)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
    else
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}

template <int CG>
__device__ __forceinline__ void tmem_relinquish()
{
    if constexpr (CG == 1)
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    else
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

template <int CG>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    if constexpr (CG == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
    else
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]; bf16/fp16 inputs, one thread issues.
template <int CG>
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    if constexpr (CG == 1)
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
}

// e4m3/e5m2/e2m3/e3m2/e2m1 inputs without block scaling (per-tensor FP8 path)
template <int CG>
__device__ __forceinline__ void umma_f8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    if constexpr (CG == 1)
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
}

// Block-scaled MMAs (one CTA): D (+)= (A * SFA) * (B * SFB), ue8m0 scale factors read from TMEM.
// mxf8f6f4: one scale per 32 K-elements, 32 K-elements per instruction (scale_vec::1X).
template <int CG>
__device__ __forceinline__ void umma_mxf8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                                          uint32_t sfb_tmem, uint32_t accumulate)
{
    if constexpr (CG == 1)
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
            : "memory");
}

// mxf4: e2m1 elements, one scale per 32 K-elements, 64 K-elements per instruction (scale_vec::2X).
template <int CG>
__device__ __forceinline__ void umma_mxf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                                          uint32_t sfb_tmem, uint32_t accumulate)
{
    if constexpr (CG == 1)
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
            : "memory");
}

// Shared memory -> TMEM copy of one 512-byte scale-factor atom: 32 rows x 16 bytes, written
// to 4 TMEM columns of lanes 0..31 and replicated into the other three lane quarters (the
// form the block-scaled MMA reads).  Issued by one thread, ordered with its later MMAs.  For a CTA
// pair one instruction makes each CTA copy from ITS OWN shared memory into ITS OWN TMEM.
template <int CG>
__device__ __forceinline__ void tmem_cp_sf_atom(uint32_t taddr, uint64_t smem_desc)
{
    if constexpr (CG == 1)
        asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
    else
        asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}

// Untiled bulk copy global -> shared (16-byte aligned, size a multiple of 16), completion counted
// on an mbarrier of this CTA.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// Arrive once on `bar` (this CTA) when every tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// CTA-pair form: the arrival is delivered to the barrier at the same offset in every CTA
// of `cta_mask`.  (This multicasts a barrier ARRIVAL, not a load.)
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(cta_mask)
                 : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane (base_lane + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void ld_shared_v4(uint32_t addr, uint32_t &a, uint32_t &b, uint32_t &c, uint32_t &d)
{
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr) : "memory");
}

// 16-byte store to a multicast address: NVSwitch replicates it into every GPU bound to the multicast object
// (the storing GPU included).  The .f32 type only names the lane width; the bits go through unchanged.
__device__ __forceinline__ void multimem_st_v4(void *mc_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 :: "l"(mc_addr), "f"(__uint_as_float(a)), "f"(__uint_as_float(b)), "f"(__uint_as_float(c)), "f"(__uint_as_float(d))
                 : "memory");
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// four floats -> four e4m3 bytes (round to nearest even, saturating to +-448), a in the lowest byte
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d)
{
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
    return (uint32_t)lo | ((uint32_t)hi << 16);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

}  // namespace sm100
