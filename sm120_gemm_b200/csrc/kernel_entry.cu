// One kernel plugin: compiled once per configuration with the configuration given as -D
// macros, it exports the C ABI declared in include/sm100_gemm.h.
//
// Same role as the reference's src/kernel_entry.cu.in:5-27 (a CMake-configured template with
// eight @VAR@ constants and one exported gemm_run); here the build passes
//   -DGEMM_DT=<0..4> -DGEMM_BN=<64|128|192|256> -DGEMM_STAGES=<n> -DGEMM_CG=<1|2>
//   -DGEMM_SK=<split-K> -DGEMM_AB=<0|1 operand swap> -DGEMM_EPI=<0|1|2> -DGEMM_MB=<1|2 row blocks per CTA>
//   -DGEMM_BK=<K elements per pipeline unit>
#include "bf16_gemm.cuh"
#include "w4a16_gemm.cuh"
#include "w4a16_tmem_gemm.cuh"

#ifndef GEMM_DT
#error "configuration macros missing: build through sm120_gemm_b200/build.py"
#endif

namespace {

constexpr int DT = GEMM_DT;
constexpr int BN = GEMM_BN;
constexpr int STAGES = GEMM_STAGES;
constexpr int CG = GEMM_CG;
constexpr int SK = GEMM_SK;
constexpr int AB = GEMM_AB;
constexpr int EPI = GEMM_EPI;
#ifndef GEMM_MB
#define GEMM_MB 1
#endif
#ifndef GEMM_BK
#define GEMM_BK 64
#endif
constexpr int MB = GEMM_MB;          // 128-row blocks of X per CTA
constexpr int BM = 128 * CG * MB;

#if GEMM_DT == 3
// W4A16: operands swapped (AB = 1), BN is M padded, work is always cut stream-K fashion (SK = 0)
static_assert(AB == 1 && SK == 0 && CG == 1 && EPI == 0, "W4A16 plugins are <dt>_bm128_bn<MPAD>_bk<64|128>_s<S>_cg1_sk0_ab1_e0");
#if GEMM_BK == 128   // dequantised weights through tensor memory
using Traits = sm100::W4A16TmemTraits<BN, STAGES>;
using Launcher = sm100::W4A16TmemLauncher<Traits>;
#else                // dequantised weights through shared memory
using Traits = sm100::W4A16Traits<BN, STAGES>;
using Launcher = sm100::W4A16Launcher<Traits>;
#endif
#elif GEMM_DT == 0
// BF16: through the reference's two entry-point classes, chosen at compile time exactly as its entry template
// does (src/kernel_entry.cu.in:20-26): no split -> BF16GemmMMA, split-K (or stream-K) -> BF16GemmMMASplitK
static_assert(AB == 0, "operand swap is not part of this kernel");
#if GEMM_SK == 1
using Entry = BF16GemmMMA<BM, BN, 64, STAGES, CG, EPI>;
#else
using Entry = BF16GemmMMASplitK<BM, BN, 64, STAGES, CG, SK>;
#endif
using Traits = Entry::Traits;
using Launcher = Entry::Launcher;
#else
static_assert(AB == 0, "operand swap is not part of this kernel");
constexpr int OPK = DT == GEMM_DT_FP8 ? sm100::OPK_E4M3 : DT == GEMM_DT_MXFP8 ? sm100::OPK_MXFP8 : sm100::OPK_MXFP4;
using Traits = sm100::UmmaGemmTraits<OPK, BN, STAGES, CG, SK, EPI, MB>;
using Launcher = sm100::UmmaGemmLauncher<Traits>;
#endif

#define GEMM_STR2(x) #x
#define GEMM_STR(x) GEMM_STR2(x)
const char *const kConfigName = GEMM_STR(GEMM_NAME);

// Scratch for gemm_run_no_alloc: lives in the plugin's own device image, so using it needs no
// allocation call at all.  16 MiB = room for SPLIT_K*M*N <= 4 Mi FP32 partial sums (for example
// 128 x 4096 outputs split 8 ways).  Every GPU that loads this plugin holds the array until the
// process exits.  Only the bf16 split-K configurations have the array (gemm_run_no_alloc takes bf16
// operands; compiled into the others it would be 16 MiB per loaded plugin and GPU that nothing can use).
#define GEMM_HAS_STATIC_SCRATCH (GEMM_SK > 1 && GEMM_DT == 0)
#if GEMM_HAS_STATIC_SCRATCH
constexpr size_t kStaticScratchBytes = GEMM_NO_ALLOC_SCRATCH_BYTES;
static __device__ __align__(256) float g_static_scratch[kStaticScratchBytes / sizeof(float)];
#else
constexpr size_t kStaticScratchBytes = 0;
#endif

}  // namespace

extern "C" {

void gemm_run(int M, int N, int K, const void *X, const void *W, void *Y, float *workspace, gemm_stream_t stream)
{
    sm100::clear_error();
#if GEMM_DT == 0
    auto *x = static_cast<const bf16 *>(X);
    auto *w = static_cast<const bf16 *>(W);
    auto *y = static_cast<bf16 *>(Y);
#if GEMM_SK == 1
    (void)workspace;
    Entry::run(M, N, K, x, w, y, stream);
#else
    Entry::run(M, N, K, x, w, y, workspace, stream);
#endif
#else
    (void)M; (void)N; (void)K; (void)X; (void)W; (void)Y; (void)workspace; (void)stream;
    sm100::set_error(GEMM_ERR_ARG, "gemm_run takes bf16 operands; %s needs gemm_run_ex", kConfigName);
#endif
}

int gemm_run_ex(const GemmArgs *a)
{
    sm100::clear_error();
    if (!a || a->struct_size != sizeof(GemmArgs)) return sm100::set_error(GEMM_ERR_ARG, "GemmArgs is null or has the wrong struct_size");
    if ((int)a->dtype != DT) return sm100::set_error(GEMM_ERR_ARG, "dtype %u does not match plugin %s", a->dtype, kConfigName);
#if GEMM_DT == 3
    if (a->y_num_peers > 0) return sm100::set_error(GEMM_ERR_ARG, "peer destinations are not supported by %s", kConfigName);
    if (a->C || a->bias || a->amax || a->activation || a->y_dtype) return sm100::set_error(GEMM_ERR_ARG, "%s has no fused output transform", kConfigName);
    return Launcher::run(a->M, a->N, a->K, a->X, a->W, a->Y, a->w_scale, a->group_size, static_cast<float *>(a->workspace), a->workspace_bytes,
                         a->sm_limit, a->stream);
#else
    sm100::YTarget yt;
    yt.peers = a->y_peers;
    yt.num_peers = a->y_num_peers;
    yt.multicast = a->y_multicast;
    yt.forward = a->y_forward != 0;
    yt.ld = a->y_ld;
    yt.col_offset = a->y_col_offset;
    sm100::LaunchExtras ex;
    // alpha is an argument of the fused-epilogue plugins (e2) only; the others compute the plain product
    const float user_alpha = (EPI == sm100::EPI_FUSED) ? a->alpha : 1.0f;
    if (EPI != sm100::EPI_FUSED && a->alpha != 0.0f && a->alpha != 1.0f)
        return sm100::set_error(GEMM_ERR_ARG, "alpha = %g needs a fused-epilogue configuration (e2); %s computes X*W^T as is", a->alpha, kConfigName);
    ex.alpha = (DT == GEMM_DT_FP8 ? a->x_scale_f * a->w_scale_f : 1.0f) * user_alpha;
    ex.sm_limit = a->sm_limit;
    ex.sf_x = a->x_scale;
    ex.sf_w = a->w_scale;
    ex.yt = a->y_num_peers > 0 ? &yt : nullptr;
    ex.C = a->C;
    ex.bias = a->bias;
    ex.beta = a->beta;
    ex.act = a->activation;
    ex.y_dtype = a->y_dtype;
    ex.y_scale = a->y_scale;
    ex.amax = a->amax;
#ifdef SM100_TEST_WITHHOLD_STAGE
    ex.test_withhold_kb = a->reserved - 1;      // wait-expiry test build: reserved = first withheld k-block + 1 (0 = none)
#endif
#if GEMM_DT == 0
#if GEMM_SK == 1
    return Entry::run_ex(a->M, a->N, a->K, static_cast<const bf16 *>(a->X), static_cast<const bf16 *>(a->W), a->Y, a->stream, ex);
#else
    return Entry::run_ex(a->M, a->N, a->K, static_cast<const bf16 *>(a->X), static_cast<const bf16 *>(a->W), a->Y,
                         static_cast<float *>(a->workspace), a->workspace_bytes, a->stream, ex);
#endif
#else
    return Launcher::run(a->M, a->N, a->K, a->X, a->W, a->Y, static_cast<float *>(a->workspace), a->workspace_bytes, a->stream, ex);
#endif
#endif
}

const char *gemm_config_name(void) { return kConfigName; }
size_t gemm_workspace_bytes(int M, int N, int K) { return Launcher::workspace_bytes(M, N, K); }
int gemm_can_run(int M, int N, int K) { return Launcher::can_run(M, N, K) ? 1 : 0; }
size_t gemm_smem_bytes(void) { return Traits::SMEM_ALLOC; }
int gemm_last_error(void) { return sm100::error_state().code; }
const char *gemm_last_error_message(void) { return sm100::error_state().msg; }

int gemm_run_no_alloc(int M, int N, int K, const void *X, const void *W, void *Y, gemm_stream_t stream)
{
    sm100::clear_error();
#if GEMM_HAS_STATIC_SCRATCH
    if (DT != GEMM_DT_BF16) return sm100::set_error(GEMM_ERR_ARG, "gemm_run_no_alloc takes bf16 operands; %s does not", kConfigName);
    if (!Launcher::can_run(M, N, K)) return sm100::set_error(GEMM_ERR_SHAPE, "shape %dx%dx%d not supported by %s", M, N, K, kConfigName);
    const size_t need = Launcher::workspace_bytes(M, N, K);
    if (need > kStaticScratchBytes)
        return sm100::set_error(GEMM_ERR_WORKSPACE,
                                "gemm_run_no_alloc: %s needs %zu bytes of split-K scratch for %dx%dx%d but the built-in array has %zu; "
                                "use gemm_run with a caller-owned workspace",
                                kConfigName, need, M, N, K, kStaticScratchBytes);
    // In host code `g_static_scratch` is only a handle for the symbol, not an address the GPU can
    // use: the device address is looked up once per device, with that device current.
    static float *scratch_on_device[sm100::MAX_DEVICES] = {nullptr};
    static std::mutex mu;
    int dev = 0;
    SM100_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= sm100::MAX_DEVICES) return sm100::set_error(GEMM_ERR_ARG, "device ordinal %d out of range", dev);
    float *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (scratch_on_device[dev] == nullptr) {
            void *p = nullptr;
            SM100_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
            scratch_on_device[dev] = static_cast<float *>(p);
        }
        scratch = scratch_on_device[dev];
    }
    // every partial sum the reduce kernel reads is written by this call's GEMM kernel first, so
    // nothing in the array has to start at zero and the previous call's contents do not matter
    return Launcher::run(M, N, K, X, W, Y, scratch, kStaticScratchBytes, stream);
#else
    (void)M; (void)N; (void)K; (void)X; (void)W; (void)Y; (void)stream;
    return sm100::set_error(GEMM_ERR_ARG, "gemm_run_no_alloc: %s has no built-in scratch array; call gemm_run", kConfigName);
#endif
}

int gemm_check_status(void)
{
    uint32_t st[4];
    return sm100::read_device_status(st);
}

}  // extern "C"
