/*
 * C ABI of libsm100gemm_util.so: small device utilities around the GEMM plugins.
 * None of them has a counterpart in the reference (single GPU, BF16 only).
 * `stream` is a cudaStream_t; the int results are cudaError_t values (0 = success).
 */
#ifndef SM100_GEMM_UTIL_H
#define SM100_GEMM_UTIL_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* N-sharded multi-GPU run: gathered [g][M][Nb] blocks -> row-major Y[M][g*Nb].
 * elem_bytes*Nb must be a multiple of 16; pointers 16-byte aligned. */
int gemm_interleave_blocks(const void *blocked, void *Y, int g, long long M, int Nb, int elem_bytes, void *stream);

/* Idle kernel of `us` microseconds: the spacer between timed launches of the reference's
 * timing protocol (sleep_kernel, src/common.h:16-19). */
int gemm_spacer(unsigned us, void *stream);

/* MX scale layout (see include/sm100_gemm.h): bytes of the tiled array for `rows` rows and K
 * elements, and the conversion of a row-major [rows][K/32] ue8m0 array into it. */
size_t gemm_mx_tiled_scale_bytes(long long rows, int K);
int gemm_mx_scales_to_tiled(const void *src, void *dst, long long rows, int K, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SM100_GEMM_UTIL_H */
