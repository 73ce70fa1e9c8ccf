// One translation unit = the reference's bench source (included from where it lies, with its
// main() renamed) + a linkable name for the direct template call its debug mode makes
// (reference src/bench.cu:186-188, 222).  TEST INFRASTRUCTURE; see Makefile.ref.
#define main ref_bench_main
#include "bench.cu"
#undef main

void ref_mma_run(int M, int N, int K, const bf16 *X, const bf16 *W, bf16 *Y, cudaStream_t stream)
{
    BF16GemmMMA<128, 128, 64, 2, 2, 32, 64>::run(M, N, K, X, W, Y, stream);
}
