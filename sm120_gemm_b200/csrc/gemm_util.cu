// Small device utilities around the GEMM plugins, exported with a C ABI
// (libsm100gemm_util.so): the column-block interleave of the N-sharded multi-GPU run and
// the idle spacer kernel of the timing protocol.  No counterpart in the reference, which is
// single-GPU (device 0 is hard-coded, src/bf16_gemm.cuh:531).
#include <cuda_runtime.h>
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

// idle kernel between timed launches (the reference's sleep_kernel, src/common.h:16-19)
int gemm_spacer(unsigned us, void *stream)
{
    spacer_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(us);
    return (int)cudaGetLastError();
}
}
