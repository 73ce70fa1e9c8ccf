// Small device utilities around the GEMM plugins, exported with a C ABI
// (libsm100gemm_util.so): the column-block interleave of the N-sharded multi-GPU run and
// the idle spacer kernel of the timing protocol.  No counterpart in the reference, which is
// single-GPU (device 0 is hard-coded, src/bf16_gemm.cuh:531).
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace {

// blocked[g][M][Nb] (what an all-gather of per-rank M x Nb results produces) -> row-major
// Y[M][g*Nb].  Pure HBM traffic, 16 bytes per thread per access, grid-stride.
__global__ void __launch_bounds__(256) interleave_blocks_kernel(const uint4 *__restrict__ blocked, uint4 *__restrict__ Y, int g,
                                                                 long long M, int nb_vec)
{
    const long long total = (long long)g * M * nb_vec;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int v = (int)(i % nb_vec);
        const long long t = i / nb_vec;
        const int r = (int)(t % g);
        const long long m = t / g;
        // destination index i enumerates Y row-major: (m, r, v)
        Y[i] = __ldcs(blocked + ((long long)r * M + m) * nb_vec + v);
    }
}

// Row-major ue8m0 scales [rows][kblocks] (one per 32 K-elements) -> the atom layout the
// block-scaled kernels read: 512-byte atoms of 128 rows x 4 K-blocks, atom (r/128, kb/4) at
// byte ((r/128)*k_atoms + kb/4)*512, and inside an atom byte (r%32)*16 + ((r%128)/32)*4 + kb%4
// (32 rows of 16 bytes: what one tcgen05.cp moves into TMEM).  Padding rows / K-blocks get the
// scale 1.0 (127); they only ever multiply zero-filled operand data.
__global__ void __launch_bounds__(256) mx_scales_to_tiled_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst,
                                                                  long long rows, int kblocks, int k_atoms, long long total)
{
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long atom = i >> 9;
        const int in = (int)(i & 511);
        const long long r = (atom / k_atoms) * 128 + ((in >> 2) & 3) * 32 + (in >> 4);
        const int kb = (int)(atom % k_atoms) * 4 + (in & 3);
        dst[i] = (r < rows && kb < kblocks) ? src[r * kblocks + kb] : (uint8_t)127;
    }
}

__global__ void spacer_kernel(unsigned us) { __nanosleep(us * 1000u); }

}  // namespace

extern "C" {

// elem_bytes * Nb must be a multiple of 16; pointers 16-byte aligned.  Returns a cudaError_t.
int gemm_interleave_blocks(const void *blocked, void *Y, int g, long long M, int Nb, int elem_bytes, void *stream)
{
    if (g <= 0 || M <= 0 || Nb <= 0 || ((long long)Nb * elem_bytes) % 16 != 0) return (int)cudaErrorInvalidValue;
    const int nb_vec = (int)((long long)Nb * elem_bytes / 16);
    const long long total = (long long)g * M * nb_vec;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    interleave_blocks_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4 *>(blocked), static_cast<uint4 *>(Y), g, M, nb_vec);
    return (int)cudaGetLastError();
}

// Bytes of the tiled scale array for `rows` rows and K elements (K a multiple of 32).
size_t gemm_mx_tiled_scale_bytes(long long rows, int K)
{
    const long long k_atoms = ((long long)K / 32 + 3) / 4;
    return (size_t)((rows + 127) / 128 * k_atoms * 512);
}

// src: row-major [rows][K/32] ue8m0; dst: gemm_mx_tiled_scale_bytes(rows, K) bytes, 16-byte aligned.
int gemm_mx_scales_to_tiled(const void *src, void *dst, long long rows, int K, void *stream)
{
    if (rows <= 0 || K <= 0 || K % 32 != 0) return (int)cudaErrorInvalidValue;
    const int kblocks = K / 32, k_atoms = (kblocks + 3) / 4;
    const long long total = (rows + 127) / 128 * k_atoms * 512;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    mx_scales_to_tiled_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t *>(src), static_cast<uint8_t *>(dst), rows, kblocks, k_atoms, total);
    return (int)cudaGetLastError();
}

// idle kernel between timed launches (the reference's sleep_kernel, src/common.h:16-19)
int gemm_spacer(unsigned us, void *stream)
{
    spacer_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(us);
    return (int)cudaGetLastError();
}
}
