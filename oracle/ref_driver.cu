// Exposes the reference project's own FP32 check kernel and one of its mma.sync GEMM
// configurations through a tiny C ABI, so the CPU oracle can be validated against the real
// reference on a GPU box.  TEST INFRASTRUCTURE: built only into oracle/_ref/ (git-ignored),
// from the reference sources where they lie; none of those sources is copied here.
//
// The reference translation unit (src/bench.cu) is compiled separately with its main()
// renamed; this file only declares the two functions it uses from it:
//   naive_gemm_f32(M,N,K,X,W,Y,stream)            reference src/bench.cu:87-95
//   bench_debug()-style direct template call      reference src/bench.cu:186-188, 222
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdio>

using bf16 = __nv_bfloat16;
void naive_gemm_f32(int M, int N, int K, const bf16 *X, const bf16 *W, float *Y, cudaStream_t stream);
void ref_mma_run(int M, int N, int K, const bf16 *X, const bf16 *W, bf16 *Y, cudaStream_t stream);

extern "C" {

// device pointers in, FP32 Y out; returns the CUDA error code after synchronising
int ref_naive_gemm_f32(int M, int N, int K, const void *X, const void *W, float *Y)
{
    naive_gemm_f32(M, N, K, static_cast<const bf16 *>(X), static_cast<const bf16 *>(W), Y, nullptr);
    return (int)cudaDeviceSynchronize();
}

// the reference's mma.sync kernel (128x128x64, 2 stages, 2 consumer warpgroups), asynchronous
int ref_mma_gemm(int M, int N, int K, const void *X, const void *W, void *Y, void *stream)
{
    if (M % 128 || N % 128 || K % 64) return -1;
    ref_mma_run(M, N, K, static_cast<const bf16 *>(X), static_cast<const bf16 *>(W), static_cast<bf16 *>(Y),
                static_cast<cudaStream_t>(stream));
    return (int)cudaGetLastError();
}
}
