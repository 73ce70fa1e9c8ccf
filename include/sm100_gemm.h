/*
 * C ABI of one kernel plugin (libgemm_<config name>.so): Y = X * W^T on one B200.
 *
 *   X  row-major M x K      W  row-major N x K      Y  row-major M x N (bf16), fully overwritten
 *   FP32 accumulation.  All pointers are DEVICE pointers, 16-byte aligned; K and N are
 *   multiples of 8 elements (16-byte row pitch).  M, N, K need not be multiples of the tile.
 *
 * Every plugin exports the same symbols; the configuration (data type, tile, stages, CTA
 * pairing, split-K, operand swap) is compiled in and encoded in the file name, which is what
 * the registry parses -- exactly the reference's scheme (src/gemm_config.h:65-120,
 * CMakeLists.txt:40-60).
 *
 * Plain C: no CUDA or C++ types in the signatures, so it binds from dlsym, ctypes, cgo, JNI...
 */
#ifndef SM100_GEMM_H
#define SM100_GEMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* cudaStream_t is `struct CUstream_st *`; spelled out so the header needs no CUDA include. */
typedef struct CUstream_st *gemm_stream_t;

/* Error codes (gemm_run_ex return value, gemm_last_error). */
enum {
    GEMM_OK = 0,
    GEMM_ERR_SHAPE = 1,          /* M/N/K not supported by this configuration              */
    GEMM_ERR_CUDA = 2,           /* a CUDA runtime call failed (message has the detail)    */
    GEMM_ERR_DRIVER = 3,         /* tensor-map encoding failed / driver entry point missing */
    GEMM_ERR_WORKSPACE = 4,      /* split-K workspace missing or too small                 */
    GEMM_ERR_DEVICE_TIMEOUT = 5, /* a bounded wait inside a kernel gave up                 */
    GEMM_ERR_ARG = 6             /* null / misaligned pointer, bad struct size, wrong dtype */
};

/* Data-type families (the `dt` prefix of a configuration name). */
enum {
    GEMM_DT_BF16 = 0,  /* X, W bf16                                                        */
    GEMM_DT_FP8 = 1,   /* X, W e4m3, one FP32 scale per tensor                             */
    GEMM_DT_MXFP8 = 2, /* X, W e4m3, one ue8m0 scale per 32 K-elements                     */
    GEMM_DT_W4A16 = 3, /* X bf16; W signed int4 (2 per byte, low nibble = even k), bf16    */
                       /* scale per `group_size` K-elements                                */
    GEMM_DT_W4A4 = 4   /* X, W e2m1 (2 per byte), one ue8m0 scale per 32 K-elements        */
};

/*
 * Replaces: extern "C" void gemm_run(...) of the reference, src/kernel_entry.cu.in:14-27
 * (typedef GemmKernelFn, src/gemm_config.h:20-22; found with dlsym "gemm_run",
 * src/gemm_config.h:93).  Same symbol, same argument list, same meaning: BF16 operands,
 * stream-ordered and asynchronous, `workspace` used only by split-K configurations
 * (>= gemm_workspace_bytes(M,N,K) bytes, need not be zeroed; the reference asks for
 * SPLIT_K*M*N floats, src/bf16_gemm.cuh:601).
 * Unlike the reference it never calls exit() and never throws: on failure nothing is
 * launched and the error is kept for gemm_last_error() on the calling thread.
 * Only plugins whose data type is bf16 accept this call; the others report GEMM_ERR_ARG.
 */
void gemm_run(int M, int N, int K, const void *X, const void *W, void *Y, float *workspace, gemm_stream_t stream);

/*
 * Extended arguments for every data type.  No counterpart in the reference (it is
 * BF16-only); gemm_run(M,N,K,X,W,Y,ws,stream) == gemm_run_ex with dtype GEMM_DT_BF16.
 */
typedef struct GemmArgs {
    uint32_t struct_size;   /* sizeof(GemmArgs), checked                                   */
    uint32_t dtype;         /* GEMM_DT_*; must match the plugin                            */
    int32_t M, N, K;
    int32_t group_size;     /* W4A16: K-elements per scale (128); others: ignored          */
    const void *X;          /* activations, layout per dtype                               */
    const void *W;          /* weights, layout per dtype                                   */
    void *Y;                /* bf16 M x N                                                  */
    const void *x_scale;    /* MXFP8 / W4A4: ue8m0 scales of X, TILED (see below); else NULL */
    const void *w_scale;    /* MXFP8 / W4A4: ue8m0 scales of W, TILED; W4A16: bf16 [N][K/group] */
    float x_scale_f;        /* FP8: per-tensor scale of X (1.0 elsewhere)                  */
    float w_scale_f;        /* FP8: per-tensor scale of W (1.0 elsewhere)                  */
    void *workspace;        /* split-K partial sums; may be NULL when not needed           */
    size_t workspace_bytes;
    int32_t sm_limit;       /* 0 = all SMs; >0 = persistent grid uses at most this many    */
    int32_t reserved;       /* set to 0                                                                    */
    gemm_stream_t stream;
    /* N-sharded multi-GPU runs (TMA-store configurations only).  When y_num_peers > 0, Y is ignored and the   */
    /* M x N result is stored into columns [y_col_offset, y_col_offset + N) of the row-major M x y_ld bf16     */
    /* matrix at each of y_peers[0 .. y_num_peers-1]: device pointers this process can write, normally the     */
    /* same symmetric buffer on every rank of the node, own rank included.  The stores are plain TMA stores    */
    /* over NVLink; the caller orders them against readers (kernel completion on every rank, then a barrier).  */
    int32_t y_num_peers;
    int32_t y_col_offset;
    int64_t y_ld;
    void *y_peers[8];
    /* Optional.  Multicast (NVSwitch) address of that same symmetric matrix: a store to it lands in every     */
    /* rank's copy.  When non-NULL the epilogue issues one multimem store per 16 bytes instead of one TMA      */
    /* store per peer, so each result byte leaves this GPU once; y_num_peers must still be > 0 and N a         */
    /* multiple of 8, and y_peers[0] must be THIS GPU's own matrix (the 512-row-tile kernels store a tile there */
    /* first and forward it).  Every process bound to the multicast object must stay alive until the stores are done. */
    void *y_multicast;
    /* Fused output transform, honoured by the fused-epilogue plugins only (`_e2` in the name; every other plugin  */
    /* answers GEMM_ERR_ARG when one of these is set):  D = act(alpha * (X * W^T) + beta * C + bias), written as   */
    /* bf16, or as e4m3(D * y_scale) (saturating, round to nearest even) with max|D| folded into *amax.  No        */
    /* counterpart in the reference, whose gemm_run has no alpha/beta/bias (src/kernel_entry.cu.in:14-16).         */
    const void *C;          /* bf16 M x N, row pitch N, 16-byte aligned; NULL = no beta term                       */
    const void *bias;       /* bf16, N values (one per output column), 16-byte aligned; NULL = none                */
    float alpha;            /* e2 plugins: scales the product (set it: 0 is taken literally); others: 0 or 1       */
    float beta;
    int32_t activation;     /* GEMM_ACT_*                                                                          */
    int32_t y_dtype;        /* GEMM_Y_BF16 (Y is bf16) or GEMM_Y_E4M3 (Y is M x N bytes)                           */
    float y_scale;          /* e4m3 output: multiplies D before the conversion                                     */
    float *amax;            /* device float, optional: atomically raised to max|D| (before y_scale); the caller    */
                            /* zeroes it before the first launch that should count                                 */
    /* With y_multicast, 256 x 256 TMA-store plugins (`_bm256_bn256_..._cg2_sk1_..._e1`, bf16 and fp8): 0 = the      */
    /* epilogue sends 128-byte row pieces to the multicast address; 1 = it stores the tile to y_peers[0] (this GPU's */
    /* own matrix) and four sender warps forward whole 512-byte rows from L2 while the next tile is computed.  The   */
    /* 512 x 256 plugins always forward; every other plugin ignores the field.                                      */
    int32_t y_forward;
} GemmArgs;

enum { GEMM_ACT_NONE = 0, GEMM_ACT_RELU = 1, GEMM_ACT_GELU = 2 /* erf form */, GEMM_ACT_SILU = 3 };
enum { GEMM_Y_BF16 = 0, GEMM_Y_E4M3 = 1 };

/*
 * Scale layout of the MX data types.  One ue8m0 byte scales 32 consecutive K-elements of one
 * row.  The kernels read the scales in 512-byte atoms of 128 rows x 4 K-blocks (what one
 * tcgen05.cp moves into TMEM): atom (r/128, kb/4) at byte ((r/128) * ceil(K/128) + kb/4) * 512,
 * and inside the atom row r, K-block kb at byte (r%32)*16 + ((r%128)/32)*4 + kb%4.  Rows are
 * padded to a multiple of 128.  libsm100gemm_util.so converts a row-major [rows][K/32] array
 * into this layout (include/sm100_gemm_util.h).  Weights are converted once; K must be a multiple of 128 (MXFP8) / 256 (W4A4).
 */
/* Returns GEMM_OK or an error code; asynchronous on success. */
int gemm_run_ex(const GemmArgs *args);

/* The configuration name compiled into this plugin ("bf16_bm256_bn256_bk64_s6_cg2_sk1_ab0_e1"):
 * <dt>_bm<tile rows>_bn<tile columns>_bk<K per stage>_s<ring stages>_cg<CTA group>_sk<split-K, 0 = stream-K>
 * _ab<operand swap>_e<epilogue: 0 direct stores, 1 TMA stores, 2 direct stores with the fused output transform>. */
const char *gemm_config_name(void);

/* Bytes of workspace the configuration needs for this shape (0 when it needs none).
 * The reference leaves this to the caller, who passes 4*M*N floats (src/bench.cu:377). */
size_t gemm_workspace_bytes(int M, int N, int K);

/* 1 when the configuration can run the shape (the reference's GemmConfig::is_valid_for,
 * src/gemm_config.h:34-38, answered by the plugin itself). */
int gemm_can_run(int M, int N, int K);

/* Dynamic shared memory the kernel asks for (the reference models this in
 * GemmConfig::smem_bytes, src/gemm_config.h:40-45). */
size_t gemm_smem_bytes(void);

/*
 * BF16 split-K GEMM for callers that must not allocate device memory.  No counterpart in the
 * reference (there the caller always brings the split-K workspace, src/bf16_gemm.cuh:601).
 *
 * Who needs it: code that runs where a device allocation is off the table -- a serving loop
 * that may not take the device-wide synchronisation cudaMalloc/cudaFree imply, a host that has
 * handed the whole GPU to its own memory pool and gives libraries no allocator, or a component
 * that is simply not allowed to own device memory.  Such a caller still passes X, W and Y; the
 * FP32 partial sums go into a fixed 16 MiB array compiled into the plugin
 * (GEMM_NO_ALLOC_SCRATCH_BYTES), so the shape must satisfy SPLIT_K*M*N*4 <= 16 MiB, else the
 * call fails with GEMM_ERR_WORKSPACE and launches nothing.  Only the bf16 split-K plugins
 * carry the array (16 MiB per loaded plugin and GPU); every other plugin answers GEMM_ERR_ARG.  The call itself performs no cudaMalloc / cudaFree.
 *
 * The first call on each device looks up the array's device address (and does the library's
 * usual one-time kernel-attribute set-up); make that first call outside any stream capture.
 * All calls on a device share the one array: two calls whose kernels can overlap on the GPU
 * (different streams, no dependency) race on it -- keep them on one stream or order them.
 * Nothing in the array needs clearing between calls: each call overwrites every partial sum
 * it later reads.  Every GPU that loads the plugin keeps the 16 MiB until the process ends.
 */
#define GEMM_NO_ALLOC_SCRATCH_BYTES ((size_t)16 << 20)
int gemm_run_no_alloc(int M, int N, int K, const void *X, const void *W, void *Y, gemm_stream_t stream);

/* Error of the last gemm_run / gemm_run_ex on this thread, and its text. */
int gemm_last_error(void);
const char *gemm_last_error_message(void);

/* Synchronises the current device and reports whether any kernel of this plugin abandoned a
 * wait (GEMM_ERR_DEVICE_TIMEOUT) since the last check.  The reference's kernels spin without
 * limit (src/bf16_gemm.cuh:137-148), so it has nothing to report. */
int gemm_check_status(void);

#ifdef __cplusplus
}
#endif
#endif /* SM100_GEMM_H */
