/*
 * C ABI of libsm100gemm_util.so: small device utilities around the GEMM plugins.
 * None of them has a counterpart in the reference (single GPU, BF16 only).
 * `stream` is a cudaStream_t; the int results are cudaError_t values (0 = success).
 */
#ifndef SM100_GEMM_UTIL_H
#define SM100_GEMM_UTIL_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* N-sharded multi-GPU run: gathered [g][M][Nb] blocks -> row-major Y[M][g*Nb].
 * elem_bytes*Nb must be a multiple of 16; pointers 16-byte aligned. */
int gemm_interleave_blocks(const void *blocked, void *Y, int g, long long M, int Nb, int elem_bytes, void *stream);

/* Idle kernel between timed launches of the reference's timing protocol: one thread calls
 * __nanosleep(us * 1000).  The reference passes 100 "ms" = 1e8 ns (sleep_kernel<<<1,1>>>(100),
 * src/common.h:16-19, 38), which the hardware cuts short at about a millisecond; us = 100000 asks for the
 * same thing. */
int gemm_spacer(unsigned us, void *stream);

/* MX scale layout (see include/sm100_gemm.h): bytes of the tiled array for `rows` rows and K
 * elements, and the conversion of a row-major [rows][K/32] ue8m0 array into it. */
size_t gemm_mx_tiled_scale_bytes(long long rows, int K);
int gemm_mx_scales_to_tiled(const void *src, void *dst, long long rows, int K, void *stream);

/* ---- quantisation kernels: the step in front of the low-precision GEMMs (device pointers, 16-byte aligned;
 * results are bit-identical to the host definitions given with each).  No reference counterpart: its
 * inputs are random bf16 in memory (src/bench.cu:353-355). */

/* bf16 x[n] -> e4m3 q[n] (round to nearest even, saturating) with one FP32 scale: *scale_out = max|x| / 448
 * (device float), q = e4m3(x * (1 / scale)).  n a multiple of 8.  amax_ws: one device float of scratch. */
int gemm_quant_e4m3_per_tensor(const void *x, void *q, float *scale_out, float *amax_ws, long long n, void *stream);

/* bf16 x[rows][K] -> MX elements + ue8m0 scales, one per 32 K-elements, written in the atom layout the GEMM
 * reads (gemm_mx_tiled_scale_bytes(rows, K) bytes; rows padded to 128 get the scale 1.0).
 * kind 8: e4m3 (MXFP8), q = rows*K bytes; kind 4: e2m1 (MX-FP4), q = rows*K/2 bytes, low nibble = even k.
 * scale code = clamp(ceil(log2(max|block| / emax)) + 127, 0, 254), 127 for a zero block; emax 448 / 6.
 * K a multiple of 128. */
int gemm_quant_mx(const void *x, void *q, void *sf_tiled, long long rows, int K, int kind, void *stream);

/* bf16 w[rows][K] -> signed int4 (two per byte, low nibble = even k) + bf16 scales [rows][K/128]:
 * s = bf16(max|group| / 7) (1 for a zero group), q = clamp(rint(w * (1 / s)), -8, 7).  K a multiple of 128. */
int gemm_quant_int4_g128(const void *w, void *q, void *scales, long long rows, int K, void *stream);

/* ---- offline weight packing and the weight file (host memory, host code).  No reference counterpart. */
enum {
    GEMM_FILE_ERR_ARG = -5,      /* null pointer, value out of range, K not a multiple the layout needs */
    GEMM_FILE_ERR_CHECKSUM = -4, /* payload does not match the header's checksum                         */
    GEMM_FILE_ERR_SIZE = -3,     /* caller buffer too small                                              */
    GEMM_FILE_ERR_FORMAT = -2,   /* not a weight file of this version, or truncated                      */
    GEMM_FILE_ERR_IO = -1        /* open / read / write / rename failed                                  */
};

/* First bytes of a weight file (the header block is padded to 256 bytes; payloads start on 256-byte
 * boundaries: elements at 256, scales at 256 + round_up(elem_bytes, 256)). */
typedef struct GemmWeightFileInfo {
    char magic[8];        /* "SM100QW\0"                                                    */
    uint32_t version;     /* 1                                                              */
    uint32_t dtype;       /* GEMM_DT_* of include/sm100_gemm.h                              */
    uint32_t layout;      /* version of the element / scale layouts (1 = those of sm100_gemm.h) */
    uint32_t group;       /* K-elements per scale: 32 (MX kinds), 128 (W4A16), 0 (none)     */
    uint64_t N, K;        /* weight rows (output columns) and reduction length              */
    uint64_t elem_bytes, scale_bytes;
    float tensor_scale;   /* FP8 per-tensor scale, 1 elsewhere                              */
    uint32_t checksum;    /* FNV-1a (32 bit) over the element payload, then the scale payload */
} GemmWeightFileInfo;

/* Bytes of the element / scale payload of an N x K weight matrix of the given GEMM_DT_*. */
size_t gemm_packed_weight_bytes(int dtype, long long N, int K);
size_t gemm_packed_scale_bytes(int dtype, long long N, int K);

/* int4 values in [-8, 7], one per int8, row-major -> two per byte (low nibble = even k), and back. */
int gemm_pack_int4_host(const int8_t *q, long long N, int K, uint8_t *out);
int gemm_unpack_int4_host(const uint8_t *packed, long long N, int K, int8_t *q);
/* e2m1 codes 0..15, one per byte -> two per byte (low nibble = even k), and back. */
int gemm_pack_fp4_host(const uint8_t *codes, long long N, int K, uint8_t *out);
int gemm_unpack_fp4_host(const uint8_t *packed, long long N, int K, uint8_t *codes);
/* row-major ue8m0 scales [rows][K/32] <-> the 512-byte atom layout (host version of gemm_mx_scales_to_tiled). */
int gemm_mx_scales_to_tiled_host(const uint8_t *src, long long rows, int K, uint8_t *dst);
int gemm_mx_scales_from_tiled_host(const uint8_t *src, long long rows, int K, uint8_t *dst);

/* Writes / inspects / reads a weight file.  `elems` and `scales` are already in the packed layouts (sizes
 * from the two functions above; scales NULL when the type has none).  The file is written under a temporary
 * name and renamed.  read() fills caller buffers and verifies the checksum.  0 or a GEMM_FILE_ERR_*. */
int gemm_weight_file_write(const char *path, int dtype, long long N, int K, float tensor_scale, const void *elems, const void *scales);
int gemm_weight_file_info(const char *path, GemmWeightFileInfo *out);
int gemm_weight_file_read(const char *path, void *elems, size_t elem_capacity, void *scales, size_t scale_capacity);

#ifdef __cplusplus
}
#endif
#endif /* SM100_GEMM_UTIL_H */
