// Builders for the two descriptors a tcgen05.mma takes: the 64-bit shared-memory matrix
// descriptor and the 32-bit instruction descriptor.  Bit positions follow the PTX ISA
// description of tcgen05 matrix and instruction descriptors.
//
// The reference has no counterpart: its mma.sync path reads operands with ldmatrix and
// computes swizzled addresses in software (src/bf16_gemm.cuh:159-178, 371-421).
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define UMMA_HD __host__ __device__ __forceinline__
#else
#define UMMA_HD inline
#endif

namespace sm100 {

// ---- shared-memory matrix descriptor ------------------------------------------------------
//  [ 0,14)  start address >> 4          [16,30)  leading-dimension byte offset >> 4
//  [32,46)  stride-dimension byte offset >> 4      [46,48)  descriptor version (1 on sm_100)
//  [49,52)  base offset (0: tiles are 1024-byte aligned)    [61,64)  swizzle mode
enum : uint64_t { UMMA_SWIZZLE_NONE = 0, UMMA_SWIZZLE_128B = 2, UMMA_SWIZZLE_64B = 4, UMMA_SWIZZLE_32B = 6 };

// K-major operand tile whose rows are exactly one 128-byte swizzle span (64 bf16, 128 fp8
// or 256 fp4 elements), as a TMA load with SWIZZLE_128B lays it out: row r at byte r*128,
// 16-byte chunks XOR-ed with (r & 7).  Eight rows form a 1024-byte group, so the
// stride-dimension offset (distance between 8-row groups) is 1024 bytes; the
// leading-dimension offset is not used by this layout.
UMMA_HD uint64_t make_smem_desc_k128(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= UMMA_SWIZZLE_128B << 61;
    return d;
}

// One 512-byte scale-factor atom for tcgen05.cp 32x128b: 32 rows of 16 bytes, no swizzle.
// Eight 16-byte rows form a 128-byte core matrix, so 8-row groups are 128 bytes apart (SBO);
// the copy is a single 16-byte column wide, so the leading-dimension offset is unused.
UMMA_HD uint64_t make_sf_atom_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)(128u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;   // swizzle mode 0
}

// Stepping along K inside the 128-byte span: the start address moves by the byte width of
// one MMA's K extent (32 bytes for every operand type: 16 bf16 / 32 fp8 / 64 fp4).
UMMA_HD uint64_t advance_desc_k(uint64_t desc, uint32_t k_step)
{
    return desc + (uint64_t)((k_step * 32u) >> 4);
}

// ---- instruction descriptor ------------------------------------------------------------------
//  [4,6) D format (1 = F32)   [7,10) A format   [10,13) B format   [15] A major   [16] B major
//  [17,23) N >> 3             [24,29) M >> 4    (major 0 = K-major)
enum : uint32_t { UMMA_F16 = 0, UMMA_BF16 = 1, UMMA_TF32 = 2 };                        // kind::f16 / tf32
enum : uint32_t { UMMA_E4M3 = 0, UMMA_E5M2 = 1, UMMA_E2M3 = 3, UMMA_E3M2 = 4, UMMA_E2M1 = 5 };  // kind::f8f6f4 / mxf8f6f4
enum : uint32_t { UMMA_MXF4_E2M1 = 1 };                                                  // kind::mxf4

UMMA_HD uint32_t make_idesc(uint32_t a_fmt, uint32_t b_fmt, int M, int N)
{
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// Block-scaled kinds (mxf8f6f4, mxf4): bits [4,6) and [29,31) select the scale-factor slot of
// B and A inside their TMEM columns, bit 23 the scale type (1 = ue8m0).
UMMA_HD uint32_t make_idesc_block_scaled(uint32_t a_fmt, uint32_t b_fmt, int M, int N, uint32_t a_sf_id, uint32_t b_sf_id)
{
    return (b_sf_id << 4) | (a_fmt << 7) | (b_fmt << 10) | ((uint32_t)(N >> 3) << 17) | (1u << 23) |
           ((uint32_t)(M >> 4) << 24) | (a_sf_id << 29);
}

}  // namespace sm100
