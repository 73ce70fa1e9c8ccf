// Quantisation kernels: the step in front of the FP8 / MXFP8 / W4A4 / W4A16 GEMMs.  bf16 in, the
// operand layouts of include/sm100_gemm.h out (elements row-major, MX scales already in the
// 512-byte atom layout one tcgen05.cp moves into TMEM).  Exported from libsm100gemm_util.so
// (include/sm100_gemm_util.h).  No counterpart in the reference, whose inputs are random bf16
// in memory (src/bench.cu:353-355).
//
// All of it is HBM-bound byte work: 128-bit loads, 64/128-bit stores, one pass over the data
// (two for the per-tensor scale, which needs the global maximum first).  Algorithmic bytes per
// element: e4m3 per tensor 2 (absmax pass) + 2 + 1; MXFP8 2 + 1 + 1/32; MX-FP4 2 + 0.5 + 1/32;
// int4 2 + 0.5 + 2/128.
//
// The arithmetic is the oracle's, operation for operation, so results are bit-identical:
//   per-tensor:  scale = amax / 448;  q = e4m3_rne_sat(x * (1 / scale))
//   MX block:    sc = clamp(ceil(log2(amax / emax)) + 127, 0, 254) (127 for an all-zero block);
//                q = cvt(x * 2^(127 - sc)),  emax = 448 (e4m3) or 6 (e2m1)
//   int4 group:  s = bf16(amax / 7) (1 for an all-zero group);  q = clamp(rint(x * (1 / s)), -8, 7)
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stddef.h>
#include <stdint.h>

namespace {

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ void unpack8(const uint4 &v, float (&f)[8])
{
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}

// two floats -> two e4m3 bytes, round to nearest even, saturating to +-448; `a` in the low byte
__device__ __forceinline__ uint32_t e4m3x2(float a, float b)
{
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(b), "f"(a));
    return r;
}

// two floats -> two e2m1 codes in one byte (`a` in the low nibble): round to nearest, ties to the even code, saturating
__device__ __forceinline__ uint32_t e2m1x2(float a, float b)
{
    uint16_t r;
    asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u16.u8 %0, t;\n\t}" : "=h"(r) : "f"(b), "f"(a));
    return r;
}

// ue8m0 code of the smallest power of two >= amax / emax, for an amax that is a bf16 value (as every |x| here is) and
// emax = (1 + FRAC128 / 128) * 2^EMAX_EXP (448 = 1.75 * 2^8, 6 = 1.5 * 2^2).  With amax = (1 + m/128) * 2^e the quotient
// is at most 2^(e - EMAX_EXP) when m <= FRAC128 and above it otherwise, so the answer is a matter of the exponent field
// and one comparison of the 7 mantissa bits -- no division, frexp or ldexp.  (A bf16 mantissa step is 1/128, far
// coarser than the rounding of the FP32 division the host definition performs, so the two agree bit for bit.)
template <int EMAX_EXP, int FRAC128>
__device__ __forceinline__ uint32_t ue8m0_for_block(float amax)
{
    const uint32_t bits = __float_as_uint(amax) >> 16;          // bf16 bit pattern, sign clear
    if (bits == 0) return 127u;                                 // all-zero block: scale 1
    int p = (int)(bits >> 7) - EMAX_EXP + ((int)(bits & 127u) > FRAC128 ? 1 : 0);
    if ((bits >> 7) == 0) p = 0;                                // bf16 subnormal maximum: far below the smallest scale
    return (uint32_t)(p < 0 ? 0 : (p > 254 ? 254 : p));
}

// 2^(127 - sc) as a float (sc = 254 gives the subnormal 2^-127)
__device__ __forceinline__ float inv_scale_of(uint32_t sc)
{
    return __uint_as_float(sc >= 254u ? 0x00400000u : (254u - sc) << 23);
}

// byte offset of the scale of (row r, K-block kb) in the atom layout
__device__ __forceinline__ size_t sf_tiled_offset(long long r, int kb, int k_atoms)
{
    return ((size_t)(r >> 7) * k_atoms + (kb >> 2)) * 512 + (size_t)(r & 31) * 16 + (size_t)((r & 127) >> 5) * 4 + (kb & 3);
}

// ---------------------------------------------------------------------------------- per-tensor e4m3
// max |x| over n bf16 values (n a multiple of 8) into *amax_bits (float bits; non-negative floats
// order like their bit patterns, so an integer atomicMax does it).  Zeroed by the caller.
__global__ void __launch_bounds__(256) absmax_bf16_kernel(const uint4 *__restrict__ x, size_t n_vec, unsigned int *amax_bits)
{
    float m = 0.f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 v = x[i];                   // plain load: the second pass re-reads the data, keep it in L2
        float f[8];
        unpack8(v, f);
#pragma unroll
        for (int j = 0; j < 8; j++) m = fmaxf(m, fabsf(f[j]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __shared__ float wmax[8];
    if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int w = 1; w < 8; w++) m = fmaxf(m, wmax[w]);
        atomicMax(amax_bits, __float_as_uint(m));
    }
}

// q = e4m3(x / scale) with scale = amax / 448 (1 when the tensor is all zero); writes the scale too
__global__ void __launch_bounds__(256) quant_e4m3_kernel(const uint4 *__restrict__ x, uint2 *__restrict__ q, size_t n_vec,
                                                         const unsigned int *__restrict__ amax_bits, float *__restrict__ scale_out)
{
    asm volatile("griddepcontrol.wait;" ::: "memory");     // programmatic dependent of the absmax kernel
    const float amax = __uint_as_float(*amax_bits);
    const float scale = amax > 0.f ? amax / 448.0f : 1.0f;
    const float inv = 1.0f / scale;
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 v = __ldcs(x + i);
        float f[8];
        unpack8(v, f);
        uint2 o;
        o.x = e4m3x2(f[0] * inv, f[1] * inv) | (e4m3x2(f[2] * inv, f[3] * inv) << 16);
        o.y = e4m3x2(f[4] * inv, f[5] * inv) | (e4m3x2(f[6] * inv, f[7] * inv) << 16);
        q[i] = o;
    }
}

// ---------------------------------------------------------------------------------- MX formats
// One thread converts 8 consecutive K-elements (one 16-byte load); the 4 threads of a 32-element block
// agree on its maximum by shuffles; 16 threads cover the 4 blocks (128 elements) whose scales form one
// 4-byte word of the atom layout, written by the first of them.  A warp covers 256 elements of one row.
// FP4 = true: e2m1, two per byte (low nibble = even k), 4-byte stores; else e4m3, 8-byte stores.
// Rows beyond `rows` up to the next multiple of 128 get scale 1.0 (they face zero-filled operand rows).
template <bool FP4>
__global__ void __launch_bounds__(256) quant_mx_kernel(const uint4 *__restrict__ x, void *__restrict__ q, uint8_t *__restrict__ sf,
                                                       long long rows, long long rows_padded, int K, int k_atoms)
{
    const int vec_per_row = K / 8;                        // 16-byte pieces per row (K is a multiple of 128)
    const long long total = rows_padded * vec_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / vec_per_row;
        const int v = (int)(i - r * vec_per_row);
        const int lane = threadIdx.x & 31;
        float f[8];
        float m = 0.f;
        if (r < rows) {
            unpack8(__ldcs(x + i), f);
#pragma unroll
            for (int j = 0; j < 8; j++) m = fmaxf(m, fabsf(f[j]));
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++) f[j] = 0.f;
        }
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
        const uint32_t sc = FP4 ? ue8m0_for_block<2, 64>(m) : ue8m0_for_block<8, 96>(m);
        // the four scale bytes of this 128-element span, collected in the span's first lane
        const int base = lane & 16;
        uint32_t word = __shfl_sync(0xffffffffu, sc, base) | (__shfl_sync(0xffffffffu, sc, base + 4) << 8) |
                        (__shfl_sync(0xffffffffu, sc, base + 8) << 16) | (__shfl_sync(0xffffffffu, sc, base + 12) << 24);
        if ((lane & 15) == 0) *reinterpret_cast<uint32_t *>(sf + sf_tiled_offset(r, v / 4, k_atoms)) = word;
        if (r >= rows) continue;
        const float inv = inv_scale_of(sc);
        if (FP4) {
            const uint32_t o = e2m1x2(f[0] * inv, f[1] * inv) | (e2m1x2(f[2] * inv, f[3] * inv) << 8) | (e2m1x2(f[4] * inv, f[5] * inv) << 16) |
                               (e2m1x2(f[6] * inv, f[7] * inv) << 24);
            static_cast<uint32_t *>(q)[i] = o;
        } else {
            uint2 o;
            o.x = e4m3x2(f[0] * inv, f[1] * inv) | (e4m3x2(f[2] * inv, f[3] * inv) << 16);
            o.y = e4m3x2(f[4] * inv, f[5] * inv) | (e4m3x2(f[6] * inv, f[7] * inv) << 16);
            static_cast<uint2 *>(q)[i] = o;
        }
    }
}

// ---------------------------------------------------------------------------------- W4A16 weights
// Symmetric int4 per group of 128 K-elements: 16 threads of 8 elements each share one group.
__global__ void __launch_bounds__(256) quant_int4_kernel(const uint4 *__restrict__ w, uint32_t *__restrict__ q, __nv_bfloat16 *__restrict__ scales,
                                                         long long rows, int K)
{
    const int vec_per_row = K / 8;
    const long long total = rows * vec_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        float f[8];
        unpack8(__ldcs(w + i), f);
        float m = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) m = fmaxf(m, fabsf(f[j]));
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const __nv_bfloat16 sb = __float2bfloat16_rn(m > 0.f ? m / 7.0f : 1.0f);
        const float inv = 1.0f / __bfloat162float(sb);
        uint32_t o = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float t = rintf(f[j] * inv);
            t = fminf(fmaxf(t, -8.f), 7.f);
            o |= ((uint32_t)(int)t & 0xfu) << (4 * j);
        }
        q[i] = o;
        if ((threadIdx.x & 15) == 0) {
            const long long r = i / vec_per_row;
            const int g = (int)(i - r * vec_per_row) / 16;
            scales[r * (K / 128) + g] = sb;
        }
    }
}

unsigned grid_for(long long work_items, int per_block = 256)
{
    long long blocks = (work_items + per_block - 1) / per_block;
    const long long cap = 148ll * 16;        // a few waves of 148 SMs x 8 resident blocks; grid-stride does the rest
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (unsigned)blocks;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" {

// bf16 x[n] -> e4m3 q[n] with one FP32 scale for the whole tensor (scale = max|x| / 448, written to
// *scale_out on the device; x ~ q * scale).  n a multiple of 8.  `amax_ws`: one device word of scratch,
// holds max|x| (as float) afterwards.  Two kernels on `stream`.  Returns a cudaError_t.
int gemm_quant_e4m3_per_tensor(const void *x, void *q, float *scale_out, float *amax_ws, long long n, void *stream)
{
    if (n <= 0 || n % 8 != 0 || !x || !q || !scale_out || !amax_ws || !aligned16(x) || (reinterpret_cast<uintptr_t>(q) & 7u)) return (int)cudaErrorInvalidValue;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemsetAsync(amax_ws, 0, sizeof(float), st);
    if (e != cudaSuccess) return (int)e;
    const size_t n_vec = (size_t)n / 8;
    absmax_bf16_kernel<<<grid_for((long long)n_vec), 256, 0, st>>>(static_cast<const uint4 *>(x), n_vec, reinterpret_cast<unsigned int *>(amax_ws));
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid_for((long long)n_vec));
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, quant_e4m3_kernel, static_cast<const uint4 *>(x), static_cast<uint2 *>(q), n_vec,
                           reinterpret_cast<const unsigned int *>(amax_ws), scale_out);
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

// bf16 x[rows][K] -> MX elements + ue8m0 scales in the atom layout (gemm_mx_tiled_scale_bytes(rows, K) bytes).
// kind 8: e4m3, q has rows*K bytes; kind 4: e2m1, q has rows*K/2 bytes.  K a multiple of 128.
int gemm_quant_mx(const void *x, void *q, void *sf_tiled, long long rows, int K, int kind, void *stream)
{
    if (rows <= 0 || K <= 0 || K % 128 != 0 || (kind != 8 && kind != 4) || !x || !q || !sf_tiled || !aligned16(x) || !aligned16(q) || !aligned16(sf_tiled))
        return (int)cudaErrorInvalidValue;
    const long long rows_padded = (rows + 127) / 128 * 128;
    const int k_atoms = K / 128;
    const unsigned grid = grid_for(rows_padded * (K / 8));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (kind == 4)
        quant_mx_kernel<true><<<grid, 256, 0, st>>>(static_cast<const uint4 *>(x), q, static_cast<uint8_t *>(sf_tiled), rows, rows_padded, K, k_atoms);
    else
        quant_mx_kernel<false><<<grid, 256, 0, st>>>(static_cast<const uint4 *>(x), q, static_cast<uint8_t *>(sf_tiled), rows, rows_padded, K, k_atoms);
    return (int)cudaGetLastError();
}

// bf16 w[rows][K] -> signed int4, two per byte (low nibble = even k), and one bf16 scale per 128 K-elements
// ([rows][K/128]): s = bf16(max|w| / 7), q = clamp(rint(w * (1 / s)), -8, 7).  K a multiple of 128.
int gemm_quant_int4_g128(const void *w, void *q, void *scales, long long rows, int K, void *stream)
{
    if (rows <= 0 || K <= 0 || K % 128 != 0 || !w || !q || !scales || !aligned16(w) || (reinterpret_cast<uintptr_t>(q) & 3u)) return (int)cudaErrorInvalidValue;
    quant_int4_kernel<<<grid_for(rows * (K / 8)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4 *>(w), static_cast<uint32_t *>(q), static_cast<__nv_bfloat16 *>(scales), rows, K);
    return (int)cudaGetLastError();
}
}
