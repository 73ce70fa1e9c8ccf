// bench: the C++ harness around the kernel plugins.  Three modes, as in the reference's bench
// (src/bench.cu:583-597):
//   bench --autotune   every valid plugin per shape: correctness gate, then timing; best -> cache file
//   bench              quick: re-time the cached winner of every cached shape against the library comparator
//   bench --debug      fixed configurations called through the class templates, verbose checks
// and one more for single measurements (profiling a kernel, sweeps):
//   bench --kernel <config name> --shape M,N,K      time that one plugin
//   bench --aux                                      the HBM-bound helper kernels alone (split-K reduce, quantisers, interleave) in GB/s
// Options: --dtype bf16|fp8|mxfp8|w4a4|w4a16 (default bf16)   --dir <plugin dir>   --cache <file>
//          --shape M,N,K (repeatable, replaces the built-in list)   --json <file> (one JSON object per line)
//          --peaks <MEASURED_PEAKS.json> (adds "% of measured" beside the nominal roofline fractions)
//          --host-ref <liboracle.so> (times the CPU restatement of the FP32 check loop on the host cores
//          and prints it with the thread count; the harness's CPU-baseline line, never part of a result)
//
// Kept from the reference because they define the metric: the timing protocol (bench_ms: warm-ups,
// per-launch event pairs, idle spacer, mean -- src/common.h:21-50), L2 flushing by rotating over enough
// buffer sets to exceed twice the L2 (src/bench.cu:381-395), flops = 2MNK (src/bench.cu:404), cuBLAS called
// as cublasGemmEx(OP_T, OP_N, N, M, K) on the same buffers (src/bench.cu:44-65), an FP32 GPU GEMM as the
// on-device check (src/bench.cu:68-95) and "never time a kernel that failed the check" (src/bench.cu:413-429).
// New: the low-precision families (operands made by the library's own quantisation kernels from the same
// random bf16 data, checked against the FP32 GEMM of the dequantised operands, cuBLASLt beside them where it
// has the type), roofline fractions, status codes instead of exit().
#include <cublasLt.h>
#include <cublas_v2.h>
#include <dlfcn.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <memory>
#include <string>
#include <thread>

#include "../../include/sm100_gemm_util.h"
#include "bf16_gemm.cuh"
#include "common.h"
#include "gemm_config.h"

namespace {

// nominal dense peaks per data-type family (TFLOP/s) and HBM (GB/s); "measured" comes from --peaks
constexpr double kNominalTflops[5] = {2250.0, 4500.0, 4500.0, 2250.0, 9000.0};
constexpr double kNominalHbmGbs = 8000.0;
double g_measured_bf16_tflops = 0, g_measured_hbm_gbs = 0;
FILE *g_json = nullptr;

struct Shape { int M, N, K; };
// the reference's list (src/bench.cu:164-176) plus the 16384^3 family of the N-sharded runs
std::vector<Shape> g_shapes = {{512, 512, 14336}, {1024, 1024, 14336}, {1024, 1024, 1024}, {2048, 2048, 2048}, {4096, 4096, 4096},
                               {8192, 8192, 8192}, {4096, 28672, 4096}, {4096, 4096, 14336}, {128, 28672, 4096}, {128, 4096, 14336},
                               {16384, 16384, 16384}};

template <class T>
struct DevBuf {
    T *p = nullptr;
    size_t n = 0;
    explicit DevBuf(size_t count) : n(count) { if (cudaMalloc(&p, std::max<size_t>(count, 4) * sizeof(T)) != cudaSuccess) p = nullptr; }
    ~DevBuf() { if (p) cudaFree(p); }
    DevBuf(const DevBuf &) = delete;
    DevBuf &operator=(const DevBuf &) = delete;
};

// uniform[-1,1] from srand(42)/rand(), rounded to bf16: the reference's inputs (src/bench.cu:36-43)
void fill_reference_random(std::vector<bf16> &v)
{
    for (auto &e : v) e = __float2bfloat16((float)rand() / (float)RAND_MAX * 2.0 - 1.0);
}

// FP32 check GEMM: one output per thread, k ascending (the loop of src/bench.cu:77-84) over FP32 copies
// of the operands (bf16 widened, or the quantised operands dequantised)
__global__ void check_gemm_f32_kernel(int M, int N, int K, const float *__restrict__ X, const float *__restrict__ W, float *__restrict__ Y)
{
    const int col = blockIdx.x * blockDim.x + threadIdx.x, row = blockIdx.y * blockDim.y + threadIdx.y;
    if (row >= M || col >= N) return;
    const float *x = X + (size_t)row * K, *w = W + (size_t)col * K;
    float acc = 0.f;
    for (int k = 0; k < K; k++) acc += x[k] * w[k];
    Y[(size_t)row * N + col] = acc;
}

__device__ float e4m3_to_f32(uint8_t v)
{
    const int e = (v >> 3) & 0xf, m = v & 7;
    float r = e == 0 ? ldexpf((float)m, -9) : ldexpf((float)(8 + m), e - 10);
    if (e == 0xf && m == 7) r = nanf("");
    return (v & 0x80) ? -r : r;
}
__device__ float e2m1_to_f32(uint8_t c)
{
    const float lut[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    return (c & 8) ? -lut[c & 7] : lut[c & 7];
}
__device__ size_t sf_offset(long long r, int kb, int k_atoms)
{
    return ((size_t)(r >> 7) * k_atoms + (kb >> 2)) * 512 + (size_t)(r & 31) * 16 + (size_t)((r & 127) >> 5) * 4 + (kb & 3);
}

// operand of any family -> FP32, rows x K.  kind: 0 bf16, 1 e4m3 * scale_f, 2 e4m3 * ue8m0 (tiled), 3 int4 * bf16 group scale, 4 e2m1 * ue8m0 (tiled)
__global__ void widen_kernel(int kind, const void *__restrict__ q, const void *__restrict__ sc, float scale_f, long long rows, int K, float *__restrict__ out)
{
    const long long total = rows * K;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / K;
        const int k = (int)(i - r * K);
        float v;
        if (kind == 0) v = __bfloat162float(static_cast<const bf16 *>(q)[i]);
        else if (kind == 1) v = e4m3_to_f32(static_cast<const uint8_t *>(q)[i]) * scale_f;
        else if (kind == 2) v = e4m3_to_f32(static_cast<const uint8_t *>(q)[i]) * ldexpf(1.f, (int)static_cast<const uint8_t *>(sc)[sf_offset(r, k / 32, (K + 127) / 128)] - 127);
        else if (kind == 3) {
            const uint8_t b = static_cast<const uint8_t *>(q)[i / 2];
            int n = (k & 1) ? (b >> 4) : (b & 0xf);
            if (n >= 8) n -= 16;
            v = (float)n * __bfloat162float(static_cast<const bf16 *>(sc)[r * (K / 128) + k / 128]);
        } else {
            const uint8_t b = static_cast<const uint8_t *>(q)[i / 2];
            v = e2m1_to_f32((k & 1) ? (b >> 4) : (b & 0xf)) * ldexpf(1.f, (int)static_cast<const uint8_t *>(sc)[sf_offset(r, k / 32, (K + 127) / 128)] - 127);
        }
        out[i] = v;
    }
}

struct ErrStats { float max_abs, max_rel; double fro_err, fro_ref; };
// the reference's metric: |y-ref| / max(|y|,|ref|,1)   (src/bench.cu:97-112); plus the Frobenius figures of the quantised bar
ErrStats compare(const std::vector<bf16> &y, const std::vector<float> &ref, size_t count)
{
    ErrStats s{0.f, 0.f, 0.0, 0.0};
    for (size_t i = 0; i < count; i++) {
        const float a = __bfloat162float(y[i]), d = std::fabs(a - ref[i]);
        s.max_abs = std::max(s.max_abs, std::isnan(a) ? INFINITY : d);
        s.max_rel = std::max(s.max_rel, std::isnan(a) ? INFINITY : d / std::max({std::fabs(a), std::fabs(ref[i]), 1.0f}));
        const float rr = __bfloat162float(__float2bfloat16(ref[i]));
        s.fro_err += (double)(a - rr) * (a - rr);
        s.fro_ref += (double)ref[i] * ref[i];
    }
    return s;
}

int cublas_gemm(cublasHandle_t h, int M, int N, int K, const bf16 *X, const bf16 *W, bf16 *Y)
{
    const float one = 1.f, zero = 0.f;
    // row-major Y = X W^T  ==  column-major Y^T (N x M) = W (N x K, "transposed" view) * X^T
    return (int)cublasGemmEx(h, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &one, W, CUDA_R_16BF, K, X, CUDA_R_16BF, K, &zero, Y, CUDA_R_16BF, N,
                             CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
}

// cuBLASLt comparator for the 8- and 4-bit families: D (bf16) = W^T-view * X in the library's TN form, with per-tensor FP32
// scales (fp8), ue8m0 scales per 32 (mxfp8) or -- if the library has it -- e2m1 with ue8m0 scales per 32 (w4a4).
struct LtGemm {
    cublasLtHandle_t lt = nullptr;
    cublasLtMatmulDesc_t op = nullptr;
    cublasLtMatrixLayout_t a = nullptr, b = nullptr, d = nullptr;
    cublasLtMatmulHeuristicResult_t heur{};
    DevBuf<uint8_t> ws{64u << 20};
    DevBuf<float> scalars{4};
    bool ok = false;

    LtGemm(int dt, int M, int N, int K)
    {
        if (cublasLtCreate(&lt) != CUBLAS_STATUS_SUCCESS) return;
        const cudaDataType_t et = dt == GEMM_DT_W4A4 ? CUDA_R_4F_E2M1 : CUDA_R_8F_E4M3;
        if (cublasLtMatmulDescCreate(&op, CUBLAS_COMPUTE_32F, CUDA_R_32F) != CUBLAS_STATUS_SUCCESS) return;
        const cublasOperation_t ta = CUBLAS_OP_T, tb = CUBLAS_OP_N;
        cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof(ta));
        cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof(tb));
        if (dt != GEMM_DT_FP8) {
            const cublasLtMatmulMatrixScale_t mode = CUBLASLT_MATMUL_MATRIX_SCALE_VEC32_UE8M0;
            if (cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_A_SCALE_MODE, &mode, sizeof(mode)) != CUBLAS_STATUS_SUCCESS) return;
            if (cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_B_SCALE_MODE, &mode, sizeof(mode)) != CUBLAS_STATUS_SUCCESS) return;
        }
        if (cublasLtMatrixLayoutCreate(&a, et, K, N, K) != CUBLAS_STATUS_SUCCESS) return;      // W: column-major K x N
        if (cublasLtMatrixLayoutCreate(&b, et, K, M, K) != CUBLAS_STATUS_SUCCESS) return;      // X: column-major K x M
        if (cublasLtMatrixLayoutCreate(&d, CUDA_R_16BF, N, M, N) != CUBLAS_STATUS_SUCCESS) return;
        ok = scalars.p && ws.p;
    }
    // scale pointers must be set before the heuristic query (the library checks them for the block-scaled modes)
    bool plan(const void *sa, const void *sb)
    {
        if (!ok) return false;
        if (cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_A_SCALE_POINTER, &sa, sizeof(sa)) != CUBLAS_STATUS_SUCCESS) return false;
        if (cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_B_SCALE_POINTER, &sb, sizeof(sb)) != CUBLAS_STATUS_SUCCESS) return false;
        cublasLtMatmulPreference_t pref = nullptr;
        if (cublasLtMatmulPreferenceCreate(&pref) != CUBLAS_STATUS_SUCCESS) return false;
        const size_t wsb = ws.n;
        cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &wsb, sizeof(wsb));
        int found = 0;
        const cublasStatus_t st = cublasLtMatmulAlgoGetHeuristic(lt, op, a, b, d, d, pref, 1, &heur, &found);
        cublasLtMatmulPreferenceDestroy(pref);
        return st == CUBLAS_STATUS_SUCCESS && found > 0;
    }
    int run(const void *W, const void *X, void *Y, cudaStream_t stream)
    {
        const float one = 1.f, zero = 0.f;
        return (int)cublasLtMatmul(lt, op, &one, W, a, X, b, &zero, Y, d, Y, d, &heur.algo, ws.p, ws.n, stream);
    }
    ~LtGemm()
    {
        if (a) cublasLtMatrixLayoutDestroy(a);
        if (b) cublasLtMatrixLayoutDestroy(b);
        if (d) cublasLtMatrixLayoutDestroy(d);
        if (op) cublasLtMatmulDescDestroy(op);
        if (lt) cublasLtDestroy(lt);
    }
};

size_t elem_bytes(int dt, bool weight, long long rows, int K)
{
    if (dt == GEMM_DT_BF16 || (dt == GEMM_DT_W4A16 && !weight)) return (size_t)rows * K * 2;
    if (dt == GEMM_DT_FP8 || dt == GEMM_DT_MXFP8) return (size_t)rows * K;
    return (size_t)rows * K / 2;
}
size_t scale_bytes(int dt, bool weight, long long rows, int K)
{
    if (dt == GEMM_DT_MXFP8 || dt == GEMM_DT_W4A4) return gemm_mx_tiled_scale_bytes(rows, K);
    if (dt == GEMM_DT_W4A16 && weight) return (size_t)rows * (K / 128) * 2;
    return 16;       // fp8: the per-tensor scale (a device float written by the quantiser) + its scratch word
}
int widen_kind(int dt, bool weight)
{
    if (dt == GEMM_DT_W4A16) return weight ? 3 : 0;
    return dt == GEMM_DT_BF16 ? 0 : dt == GEMM_DT_FP8 ? 1 : dt == GEMM_DT_MXFP8 ? 2 : 4;
}

// One buffer set: the operands of one launch in the family's layout, and the output.
struct OperandSet {
    std::unique_ptr<DevBuf<uint8_t>> X, W, SX, SW;
    std::unique_ptr<DevBuf<bf16>> Y;
    bool ok() const { return X && W && SX && SW && Y && X->p && W->p && SX->p && SW->p && Y->p; }
};

// Everything one shape needs on the device: inputs (rotating sets), check values for the first `check_rows` rows.
struct Problem {
    int dt, M, N, K, sets = 1, check_rows = 0;
    float sx = 1.f, sw = 1.f;         // fp8 per-tensor scales
    std::vector<OperandSet> set;
    std::vector<float> hRef;
    std::unique_ptr<DevBuf<float>> ws;
    int next = 0;
    bool ok = false;

    Problem(int dtype, int m, int n, int k, size_t ws_bytes, cudaStream_t stream) : dt(dtype), M(m), N(n), K(k)
    {
        std::vector<bf16> hX((size_t)M * K), hW((size_t)N * K);
        srand(42);
        fill_reference_random(hX);
        fill_reference_random(hW);
        int dev = 0, l2 = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev);
        const size_t per_set = elem_bytes(dt, false, M, K) + elem_bytes(dt, true, N, K) + (size_t)M * N * 2;
        sets = (int)std::min<size_t>(64, std::max<size_t>(1, (2 * (size_t)l2 + per_set - 1) / per_set));
        DevBuf<bf16> bX(hX.size()), bW(hW.size());
        if (!bX.p || !bW.p) return;
        cudaMemcpyAsync(bX.p, hX.data(), hX.size() * 2, cudaMemcpyHostToDevice, stream);
        cudaMemcpyAsync(bW.p, hW.data(), hW.size() * 2, cudaMemcpyHostToDevice, stream);
        set.resize(sets);
        for (int i = 0; i < sets; i++) {
            OperandSet &s = set[i];
            s.X.reset(new DevBuf<uint8_t>(elem_bytes(dt, false, M, K)));
            s.W.reset(new DevBuf<uint8_t>(elem_bytes(dt, true, N, K)));
            s.SX.reset(new DevBuf<uint8_t>(scale_bytes(dt, false, M, K)));
            s.SW.reset(new DevBuf<uint8_t>(scale_bytes(dt, true, N, K)));
            s.Y.reset(new DevBuf<bf16>((size_t)M * N));
            if (!s.ok()) return;
            if (i == 0) {
                if (!quantise(bX.p, bW.p, s, stream)) return;
            } else {
                cudaMemcpyAsync(s.X->p, set[0].X->p, s.X->n, cudaMemcpyDeviceToDevice, stream);
                cudaMemcpyAsync(s.W->p, set[0].W->p, s.W->n, cudaMemcpyDeviceToDevice, stream);
                cudaMemcpyAsync(s.SX->p, set[0].SX->p, s.SX->n, cudaMemcpyDeviceToDevice, stream);
                cudaMemcpyAsync(s.SW->p, set[0].SW->p, s.SW->n, cudaMemcpyDeviceToDevice, stream);
            }
        }
        ws.reset(new DevBuf<float>(std::max<size_t>(ws_bytes, 16) / sizeof(float) + 4));
        if (!ws->p) return;
        if (dt == GEMM_DT_FP8) {
            if (cudaStreamSynchronize(stream) != cudaSuccess) return;
            cudaMemcpy(&sx, set[0].SX->p, 4, cudaMemcpyDeviceToHost);
            cudaMemcpy(&sw, set[0].SW->p, 4, cudaMemcpyDeviceToHost);
        }
        // FP32 check values: the whole result when it is small, else the first 256 rows (the naive kernel is O(MNK))
        check_rows = ((double)M * N * K <= 4e10) ? M : std::min(M, 256);
        DevBuf<float> fX((size_t)check_rows * K), fW((size_t)N * K), ref((size_t)check_rows * N);
        if (!fX.p || !fW.p || !ref.p) return;
        widen_kernel<<<1024, 256, 0, stream>>>(widen_kind(dt, false), set[0].X->p, set[0].SX->p, sx, check_rows, K, fX.p);
        widen_kernel<<<1024, 256, 0, stream>>>(widen_kind(dt, true), set[0].W->p, set[0].SW->p, sw, N, K, fW.p);
        dim3 block(16, 16), grid((N + 15) / 16, (check_rows + 15) / 16);
        check_gemm_f32_kernel<<<grid, block, 0, stream>>>(check_rows, N, K, fX.p, fW.p, ref.p);
        hRef.resize((size_t)check_rows * N);
        cudaMemcpyAsync(hRef.data(), ref.p, hRef.size() * sizeof(float), cudaMemcpyDeviceToHost, stream);
        ok = cudaStreamSynchronize(stream) == cudaSuccess;
    }

    // operands of the family from the random bf16 matrices, with the library's own quantisation kernels
    bool quantise(const bf16 *bX, const bf16 *bW, OperandSet &s, cudaStream_t st)
    {
        int rc = 0;
        if (dt == GEMM_DT_BF16) {
            cudaMemcpyAsync(s.X->p, bX, s.X->n, cudaMemcpyDeviceToDevice, st);
            cudaMemcpyAsync(s.W->p, bW, s.W->n, cudaMemcpyDeviceToDevice, st);
        } else if (dt == GEMM_DT_FP8) {
            rc |= gemm_quant_e4m3_per_tensor(bX, s.X->p, reinterpret_cast<float *>(s.SX->p), reinterpret_cast<float *>(s.SX->p) + 1, (long long)M * K, st);
            rc |= gemm_quant_e4m3_per_tensor(bW, s.W->p, reinterpret_cast<float *>(s.SW->p), reinterpret_cast<float *>(s.SW->p) + 1, (long long)N * K, st);
        } else if (dt == GEMM_DT_MXFP8 || dt == GEMM_DT_W4A4) {
            rc |= gemm_quant_mx(bX, s.X->p, s.SX->p, M, K, dt == GEMM_DT_MXFP8 ? 8 : 4, st);
            rc |= gemm_quant_mx(bW, s.W->p, s.SW->p, N, K, dt == GEMM_DT_MXFP8 ? 8 : 4, st);
        } else {
            cudaMemcpyAsync(s.X->p, bX, s.X->n, cudaMemcpyDeviceToDevice, st);
            rc |= gemm_quant_int4_g128(bW, s.W->p, s.SW->p, N, K, st);
        }
        return rc == 0;
    }
    int rotate() { return next++ % sets; }
    double flops() const { return 2.0 * M * N * K; }
    // algorithmic bytes: operands, scales, bf16 result
    double bytes() const
    {
        double sc = dt == GEMM_DT_FP8 ? 8 : (dt == GEMM_DT_MXFP8 || dt == GEMM_DT_W4A4) ? ((double)M + N) * K / 32 : dt == GEMM_DT_W4A16 ? (double)N * K / 128 * 2 : 0;
        return (double)elem_bytes(dt, false, M, K) + (double)elem_bytes(dt, true, N, K) + (double)M * N * 2 + sc;
    }
};

// one launch of a plugin on buffer set b: gemm_run for bf16 (the reference's dispatch), gemm_run_ex otherwise
int launch(const LoadedKernel &k, Problem &p, int b, cudaStream_t stream)
{
    OperandSet &s = p.set[b];
    if (p.dt == GEMM_DT_BF16) return dispatch(k, p.M, p.N, p.K, s.X->p, s.W->p, s.Y->p, p.ws->p, stream);
    GemmArgs a;
    std::memset(&a, 0, sizeof(a));
    a.struct_size = sizeof(a);
    a.dtype = (uint32_t)p.dt;
    a.M = p.M; a.N = p.N; a.K = p.K;
    a.group_size = 128;
    a.X = s.X->p; a.W = s.W->p; a.Y = s.Y->p;
    if (p.dt == GEMM_DT_MXFP8 || p.dt == GEMM_DT_W4A4) { a.x_scale = s.SX->p; a.w_scale = s.SW->p; }
    if (p.dt == GEMM_DT_W4A16) a.w_scale = s.SW->p;
    a.x_scale_f = p.sx; a.w_scale_f = p.sw;
    a.alpha = 1.f; a.y_scale = 1.f;
    a.workspace = p.ws->p;
    a.workspace_bytes = 0;
    a.stream = stream;
    return k.fn_ex(&a);
}

void print_rate(const char *label, const Problem &p, double ms, double lib_ms)
{
    const double tf = p.flops() / ms / 1e9, gbs = p.bytes() / ms / 1e6, peak = kNominalTflops[p.dt];
    std::printf("  %-52s %.4f ms  %.2f TFLOPS  (", label, ms, tf);
    if (lib_ms > 0) std::printf("%.1f%% of the library, ", 100.0 * lib_ms / ms);
    std::printf("%.1f%% of %.2f PF, %.0f GB/s = %.1f%% of 8 TB/s", 100.0 * tf / peak, peak / 1000, gbs, 100.0 * gbs / kNominalHbmGbs);
    if (g_measured_hbm_gbs > 0) std::printf("; of measured: %.1f%% HBM", 100.0 * gbs / g_measured_hbm_gbs);
    if (g_measured_bf16_tflops > 0 && p.dt == GEMM_DT_BF16) std::printf(", %.1f%% tensor", 100.0 * tf / g_measured_bf16_tflops);
    std::printf(")\n");
}

void json_line(const char *mode, const Problem &p, const char *name, double ms, double lib_ms, const char *lib)
{
    if (!g_json) return;
    std::fprintf(g_json, "{\"mode\": \"%s\", \"dtype\": \"%s\", \"shape\": [%d, %d, %d], \"kernel\": \"%s\", \"ms\": %.6g, \"tflops\": %.6g, "
                         "\"algorithmic_gbs\": %.6g, \"buffer_sets\": %d, \"comparator\": \"%s\", \"comparator_ms\": %.6g}\n",
                 mode, sm100::kDtypeNames[p.dt], p.M, p.N, p.K, name, ms, p.flops() / ms / 1e9, p.bytes() / ms / 1e6, p.sets, lib, lib_ms);
    std::fflush(g_json);
}

// runs one plugin once and checks it against the FP32 values; returns whether it passed (and the figures), or -1 on launch failure
int run_and_check(const LoadedKernel &k, Problem &p, cudaStream_t stream, ErrStats *out)
{
    cudaMemsetAsync(p.set[0].Y->p, 0xff, (size_t)p.M * p.N * sizeof(bf16), stream);   // NaN pattern: unwritten outputs fail the check
    if (launch(k, p, 0, stream) != GEMM_OK) return -1;
    if (cudaStreamSynchronize(stream) != cudaSuccess || k.check_status() != GEMM_OK) return -1;
    std::vector<bf16> hY((size_t)p.check_rows * p.N);
    cudaMemcpy(hY.data(), p.set[0].Y->p, hY.size() * sizeof(bf16), cudaMemcpyDeviceToHost);
    *out = compare(hY, p.hRef, hY.size());
    // dense families: the reference's max-rel metric, tightened from 0.1 to 0.02; weight-quantised ones: the 1e-3 Frobenius bar
    if (p.dt == GEMM_DT_W4A16 || p.dt == GEMM_DT_W4A4) return std::sqrt(out->fro_err / std::max(out->fro_ref, 1e-30)) <= 1e-3 ? 1 : 0;
    return out->max_rel < 0.02f ? 1 : 0;
}

// the library comparator of a family on the same buffers, same protocol: cuBLAS (bf16) or cuBLASLt; < 0 when it has none
double time_comparator(Problem &p, cublasHandle_t handle, cudaStream_t stream, std::string *label)
{
    if (p.dt == GEMM_DT_BF16) {
        *label = "cuBLAS";
        return bench_ms([&] { OperandSet &s = p.set[p.rotate()]; cublas_gemm(handle, p.M, p.N, p.K, (const bf16 *)s.X->p, (const bf16 *)s.W->p, s.Y->p); }, stream);
    }
    if (p.dt == GEMM_DT_W4A16) { *label = "cuBLASLt: unsupported (no int4-weight GEMM)"; return -1; }
    LtGemm lt(p.dt, p.M, p.N, p.K);
    const void *sa = p.set[0].SW->p, *sb = p.set[0].SX->p;
    if (!lt.plan(sa, sb)) { *label = "cuBLASLt: unsupported"; return -1; }
    *label = "cuBLASLt";
    bool failed = false;
    const double ms = bench_ms([&] {
        OperandSet &s = p.set[p.rotate()];
        if (lt.run(s.W->p, s.X->p, s.Y->p, stream) != 0) failed = true;
    }, stream);
    if (failed) { *label = "cuBLASLt: unsupported (matmul refused)"; return -1; }
    return ms;
}

// bench --aux: the HBM-bound helper kernels on their own, as GB/s of algorithmic bytes: the split-K reduce kernel
// (decode-sized and large), the quantisation kernels and the column-block interleave.  Small cases rotate over
// enough buffer sets to exceed twice the L2, like the GEMM timings.
template <class F>
void aux_line(const char *what, double bytes, F &&launch, cudaStream_t stream)
{
    const double ms = bench_ms(launch, stream);
    const double gbs = bytes / ms / 1e6;
    std::printf("  %-64s %9.4f ms  %8.0f GB/s  (%.1f%% of 8 TB/s", what, ms, gbs, 100.0 * gbs / kNominalHbmGbs);
    if (g_measured_hbm_gbs > 0) std::printf(", %.1f%% of the measured %.0f GB/s copy rate", 100.0 * gbs / g_measured_hbm_gbs, g_measured_hbm_gbs);
    std::printf(")\n");
    if (g_json) { std::fprintf(g_json, "{\"mode\": \"aux\", \"kernel\": \"%s\", \"ms\": %.6g, \"algorithmic_gbs\": %.6g}\n", what, ms, gbs); std::fflush(g_json); }
}

template <int SK>
void aux_reduce(const char *what, size_t M, size_t N, cudaStream_t stream)
{
    const size_t mn = M * N, per_set = mn * (4 * SK + 2);
    int dev = 0, l2 = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev);
    const int sets = (int)std::min<size_t>(16, std::max<size_t>(1, (2 * (size_t)l2 + per_set - 1) / per_set));
    std::vector<std::unique_ptr<DevBuf<float>>> ws;
    std::vector<std::unique_ptr<DevBuf<bf16>>> y;
    for (int i = 0; i < sets; i++) {
        ws.emplace_back(new DevBuf<float>(mn * SK));
        y.emplace_back(new DevBuf<bf16>(mn));
        if (!ws.back()->p || !y.back()->p) { std::printf("  %s: out of memory\n", what); return; }
        cudaMemsetAsync(ws.back()->p, 0, mn * SK * 4, stream);
    }
    int next = 0;
    size_t blocks = std::min<size_t>((mn / 8 + 255) / 256, (size_t)148 * 8);
    aux_line(what, (double)per_set, [&] {
        const int b = next++ % sets;
        cudaLaunchConfig_t cfg = sm100::dependent_launch_config((unsigned)blocks, 256, stream);      // launched the way the plugins launch it
        cudaLaunchKernelEx(&cfg, sm100::splitk_reduce_kernel<SK>, (const float *)ws[b]->p, y[b]->p, mn, 1.0f);
    }, stream);
}

int aux_mode()
{
    cudaStream_t stream;
    CHECK_CUDA(cudaStreamCreate(&stream));
    std::printf("=== helper kernels: algorithmic bytes / device time ===\n");
    aux_reduce<2>("splitk_reduce<2>  128 x 28672 (decode, 36.7 MB, rotating sets)", 128, 28672, stream);
    aux_reduce<4>("splitk_reduce<4>  128 x 4096 (decode, 9.4 MB, rotating sets)", 128, 4096, stream);
    aux_reduce<2>("splitk_reduce<2>  8192 x 8192 (671 MB)", 8192, 8192, stream);
    aux_reduce<4>("splitk_reduce<4>  4096 x 8192 (604 MB)", 4096, 8192, stream);
    const long long R = 8192, K = 8192;
    DevBuf<bf16> x((size_t)R * K);
    DevBuf<uint8_t> q((size_t)R * K), sf(gemm_mx_tiled_scale_bytes(R, (int)K)), sc(64);
    DevBuf<bf16> gs((size_t)R * K / 128);
    if (!x.p || !q.p || !sf.p || !sc.p || !gs.p) return 1;
    {
        std::vector<bf16> h((size_t)R * K);
        srand(7);
        fill_reference_random(h);
        cudaMemcpy(x.p, h.data(), h.size() * 2, cudaMemcpyHostToDevice);
    }
    const double n = (double)R * K;
    aux_line("gemm_quant_mx kind 8 (bf16 -> MXFP8)  8192 x 8192", n * (2 + 1 + 1.0 / 32), [&] { gemm_quant_mx(x.p, q.p, sf.p, R, (int)K, 8, stream); }, stream);
    aux_line("gemm_quant_mx kind 4 (bf16 -> MX-FP4) 8192 x 8192", n * (2 + 0.5 + 1.0 / 32), [&] { gemm_quant_mx(x.p, q.p, sf.p, R, (int)K, 4, stream); }, stream);
    aux_line("gemm_quant_e4m3_per_tensor (absmax + quantise) 8192 x 8192", n * (2 + 2 + 1),
             [&] { gemm_quant_e4m3_per_tensor(x.p, q.p, reinterpret_cast<float *>(sc.p), reinterpret_cast<float *>(sc.p) + 1, R * K, stream); }, stream);
    aux_line("gemm_quant_int4_g128 (bf16 -> int4 + group scales) 8192 x 8192", n * (2 + 0.5 + 2.0 / 128), [&] { gemm_quant_int4_g128(x.p, q.p, gs.p, R, (int)K, stream); }, stream);
    DevBuf<bf16> blocked((size_t)R * K), y((size_t)R * K);
    if (!blocked.p || !y.p) return 1;
    aux_line("gemm_interleave_blocks 8 x [8192][1024] -> [8192][8192] bf16", n * 4, [&] { gemm_interleave_blocks(blocked.p, y.p, 8, R, (int)K / 8, 2, stream); }, stream);
    return 0;
}

struct Options {
    std::string mode, dir, cache = "autotune_cache.txt", kernel, host_ref;
    int dt = GEMM_DT_BF16;
};

int autotune(const Options &o)
{
    cudaStream_t stream;
    CHECK_CUDA(cudaStreamCreate(&stream));
    cublasHandle_t handle;
    if (cublasCreate(&handle) != CUBLAS_STATUS_SUCCESS) return 1;
    cublasSetStream(handle, stream);
    KernelRegistry registry;
    if (!registry.load_dir(o.dir, o.dt)) { std::fprintf(stderr, "No kernels found in %s\n", o.dir.c_str()); return 1; }
    AutotuneCache cache;
    cache.load(o.cache);
    int dev = 0, max_smem = 0;
    CHECK_CUDA(cudaGetDevice(&dev));
    CHECK_CUDA(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    std::printf("Device max dynamic smem: %d bytes (%.1f KB)\n", max_smem, max_smem / 1024.0);
    auto last_save = std::chrono::steady_clock::now();
    for (const Shape &s : g_shapes) {
        std::printf("\n=== Autotune %s M=%d N=%d K=%d ===\n", sm100::kDtypeNames[o.dt], s.M, s.N, s.K);
        if (auto hit = cache.lookup(s.M, s.N, s.K, o.dt)) { std::printf("  cached: %s  %.4f ms\n", hit->config.name().c_str(), hit->time_ms); continue; }
        auto valid = registry.get_valid(s.M, s.N, s.K, max_smem, o.dt);
        std::printf("  %zu valid configs\n", valid.size());
        if (valid.empty()) { std::printf("  SKIP (no valid configs)\n"); continue; }
        size_t ws_bytes = 0;
        for (auto *k : valid) ws_bytes = std::max(ws_bytes, k->workspace_bytes(s.M, s.N, s.K));
        Problem p(o.dt, s.M, s.N, s.K, ws_bytes, stream);
        if (!p.ok) { std::printf("  SKIP (could not set the problem up: out of memory?)\n"); continue; }
        std::string lib;
        const double lib_ms = time_comparator(p, handle, stream, &lib);
        if (lib_ms > 0) std::printf("  %s: %.4f ms  %.4f TFLOPS\n", lib.c_str(), lib_ms, p.flops() / lib_ms / 1e9);
        else std::printf("  %s\n", lib.c_str());
        const LoadedKernel *best = nullptr;
        double best_ms = 1e30;
        for (auto *k : valid) {
            if (k->config.epi == 2) continue;      // the fused-transform plugins compute the same product; they are not candidates for the plain GEMM
            ErrStats e;
            const int pass = run_and_check(*k, p, stream, &e);
            if (pass < 0) { std::printf("  %-52s LAUNCH FAIL (%s)\n", k->config.name().c_str(), k->last_error_message()); cudaGetLastError(); continue; }
            if (!pass) { std::printf("  %-52s FAILED check (max rel err %g, rel Frobenius %g)\n", k->config.name().c_str(), e.max_rel, std::sqrt(e.fro_err / std::max(e.fro_ref, 1e-30))); continue; }
            const double ms = bench_ms([&] { launch(*k, p, p.rotate(), stream); }, stream);
            if (ms < 0 || k->check_status() != GEMM_OK) continue;
            print_rate(k->config.name().c_str(), p, ms, lib_ms);
            json_line("autotune", p, k->config.name().c_str(), ms, lib_ms, lib.c_str());
            if (ms < best_ms) { best_ms = ms; best = k; }
        }
        if (best) {
            std::printf("  BEST:");
            print_rate(best->config.name().c_str(), p, best_ms, lib_ms);
            cache.store(s.M, s.N, s.K, best->config, best_ms, o.dt);
        } else {
            std::printf("  NO VALID CONFIG\n");
        }
        if (std::chrono::steady_clock::now() - last_save > std::chrono::seconds(30)) { cache.save(o.cache); last_save = std::chrono::steady_clock::now(); }
    }
    cache.save(o.cache);
    std::printf("\nAutotune complete.\n");
    return 0;
}

// quick mode: the cached winner of every cached shape of the family -- or, with --kernel, that plugin on the --shape list;
// a shape without a cache entry gets the heuristic pick instead of being skipped (the reference skips it, src/bench.cu:455-458)
int quick(const Options &o)
{
    AutotuneCache cache;
    cache.load(o.cache);
    KernelRegistry registry;
    if (!registry.load_dir(o.dir, o.dt)) { std::fprintf(stderr, "No kernels found in %s\n", o.dir.c_str()); return 1; }
    cudaStream_t stream;
    CHECK_CUDA(cudaStreamCreate(&stream));
    cublasHandle_t handle;
    if (cublasCreate(&handle) != CUBLAS_STATUS_SUCCESS) return 1;
    cublasSetStream(handle, stream);
    std::vector<std::pair<Shape, const LoadedKernel *>> todo;
    if (!o.kernel.empty()) {
        const LoadedKernel *k = registry.find(o.kernel);
        if (!k) { std::fprintf(stderr, "plugin %s not found in %s\n", o.kernel.c_str(), o.dir.c_str()); return 1; }
        for (const Shape &s : g_shapes) todo.push_back({s, k});
    } else if (o.mode == "--shape-list") {
        for (const Shape &s : g_shapes) {
            auto hit = cache.lookup(s.M, s.N, s.K, o.dt);
            const LoadedKernel *k = hit ? registry.find(hit->config.name()) : nullptr;
            if (!k) {
                k = heuristic_kernel(registry, o.dt, s.M, s.N, s.K);
                if (k) std::printf("M=%d N=%d K=%d: not in the cache, heuristic pick %s\n", s.M, s.N, s.K, k->config.name().c_str());
            }
            if (k) todo.push_back({s, k});
            else std::printf("M=%d N=%d K=%d: NO VALID CONFIG\n", s.M, s.N, s.K);
        }
    } else {
        if (cache.entries.empty()) { std::printf("No autotune cache found. Run with --autotune first.\n"); return 1; }
        for (const auto &[key, entry] : cache.entries) {
            const auto &[dt, gpus, M, N, K] = key;
            if (dt != o.dt || gpus != 1) continue;
            const LoadedKernel *k = registry.find(entry.config.name());
            if (!k) { std::printf("M=%d N=%d K=%d: kernel %s not found, skipping\n", M, N, K, entry.config.name().c_str()); continue; }
            todo.push_back({Shape{M, N, K}, k});
        }
    }
    for (const auto &[s, k] : todo) {
        std::printf("\n=== %s M=%d N=%d K=%d  config=%s ===\n", sm100::kDtypeNames[o.dt], s.M, s.N, s.K, k->config.name().c_str());
        if (!k->can_run(s.M, s.N, s.K)) { std::printf("  shape not supported by this configuration, skipping\n"); continue; }
        Problem p(o.dt, s.M, s.N, s.K, k->workspace_bytes(s.M, s.N, s.K), stream);
        if (!p.ok) { std::printf("  could not set the problem up, skipping\n"); continue; }
        ErrStats e;
        const int pass = run_and_check(*k, p, stream, &e);
        if (pass <= 0) { std::printf("  %s (max rel err %g)\n", pass < 0 ? "LAUNCH FAIL" : "FAILED check", e.max_rel); continue; }
        std::string lib;
        const double lib_ms = time_comparator(p, handle, stream, &lib);
        const double ms = bench_ms([&] { launch(*k, p, p.rotate(), stream); }, stream);
        if (lib_ms > 0) std::printf("  %s:  %.4f ms  %.4f TFLOPS\n", lib.c_str(), lib_ms, p.flops() / lib_ms / 1e9);
        else std::printf("  %s\n", lib.c_str());
        std::printf("  Ours:    %.4f ms  %.4f TFLOPS  (check: %d rows, max rel err %.3g)\n", ms, p.flops() / ms / 1e9, p.check_rows, e.max_rel);
        print_rate("roofline", p, ms, lib_ms);
        json_line("quick", p, k->config.name().c_str(), ms, lib_ms, lib.c_str());
    }
    return 0;
}

// fixed configurations through the class templates, as the reference's debug mode does (src/bench.cu:178-302)
int debug_mode()
{
    using Direct = BF16GemmMMA<256, 256, 64, 6, 2>;
    using Split = BF16GemmMMASplitK<128, 128, 64, 7, 1, 2>;
    cudaStream_t stream;
    CHECK_CUDA(cudaStreamCreate(&stream));
    cublasHandle_t handle;
    if (cublasCreate(&handle) != CUBLAS_STATUS_SUCCESS) return 1;
    cublasSetStream(handle, stream);
    for (const Shape &s : g_shapes) {
        std::printf("=== Testing M=%d N=%d K=%d ===\n", s.M, s.N, s.K);
        Problem p(GEMM_DT_BF16, s.M, s.N, s.K, (size_t)2 * s.M * s.N * sizeof(float), stream);
        if (!p.ok) { std::printf("  could not set the problem up\n"); return 1; }
        const size_t cnt = (size_t)p.check_rows * s.N;
        std::vector<bf16> hY(cnt), hC(cnt);
        const bf16 *X0 = (const bf16 *)p.set[0].X->p, *W0 = (const bf16 *)p.set[0].W->p;
        bf16 *Y0 = p.set[0].Y->p;
        cublas_gemm(handle, s.M, s.N, s.K, X0, W0, Y0);
        CHECK_CUDA(cudaStreamSynchronize(stream));
        cudaMemcpy(hC.data(), Y0, cnt * sizeof(bf16), cudaMemcpyDeviceToHost);
        const ErrStats ec = compare(hC, p.hRef, cnt);
        for (int variant = 0; variant < 2; variant++) {
            const char *label = variant == 0 ? "MMA" : "MMA-SK";
            cudaMemsetAsync(Y0, 0xff, (size_t)s.M * s.N * sizeof(bf16), stream);
            const int rc = variant == 0 ? Direct::run(s.M, s.N, s.K, X0, W0, Y0, stream) : Split::run(s.M, s.N, s.K, X0, W0, Y0, p.ws->p, stream);
            if (rc == GEMM_ERR_SHAPE) { std::printf("[%s] shape not supported by this configuration, skipped\n", label); continue; }
            if (rc != GEMM_OK || cudaStreamSynchronize(stream) != cudaSuccess) { std::printf("[%s] FAILED to launch\n", label); return 1; }
            cudaMemcpy(hY.data(), Y0, cnt * sizeof(bf16), cudaMemcpyDeviceToHost);
            const ErrStats e = compare(hY, p.hRef, cnt);
            std::printf("[%s] vs fp32 ref:  abs=%f rel=%f\n[%s] cuBLAS vs ref: abs=%f rel=%f\n", label, e.max_abs, e.max_rel, label, ec.max_abs, ec.max_rel);
            if (!(e.max_rel < 0.02f)) { std::printf("[%s] FAILED\n", label); return 1; }
            std::printf("[%s] PASSED\n", label);
            const double ms = bench_ms([&] {
                OperandSet &b = p.set[p.rotate()];
                if (variant == 0) Direct::run(s.M, s.N, s.K, (const bf16 *)b.X->p, (const bf16 *)b.W->p, b.Y->p, stream);
                else Split::run(s.M, s.N, s.K, (const bf16 *)b.X->p, (const bf16 *)b.W->p, b.Y->p, p.ws->p, stream);
            }, stream);
            std::printf("[%s] %.4f ms  %.4f TFLOPS\n", label, ms, p.flops() / ms / 1e9);
        }
    }
    return 0;
}

// CPU baseline line: the host restatement of the FP32 check loop (the reference has no host GEMM; its check is the GPU
// kernel of src/bench.cu:68-95), loaded from the given shared library, timed on a row slab of the first shape.
int host_reference_line(const std::string &so)
{
    void *h = dlopen(so.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!h) { std::printf("host reference: cannot load %s (%s)\n", so.c_str(), dlerror()); return 1; }
    using GemmRows = int (*)(int, int, int, const uint16_t *, const uint16_t *, float *, const int *, int, int);
    auto fn = reinterpret_cast<GemmRows>(dlsym(h, "oracle_gemm_bf16_rows"));
    auto nthreads = reinterpret_cast<int (*)()>(dlsym(h, "oracle_num_threads"));
    if (!fn || !nthreads) { std::printf("host reference: %s lacks oracle_gemm_bf16_rows\n", so.c_str()); return 1; }
    const Shape s = g_shapes.front();
    const int rows = (int)std::max<long long>(4, std::min<long long>(s.M, (long long)(2e10 / ((double)s.N * s.K))));
    std::vector<uint16_t> X((size_t)rows * s.K), W((size_t)s.N * s.K);
    std::vector<float> Y((size_t)rows * s.N);
    srand(42);
    for (auto &e : X) e = (uint16_t)(0x3c00 + rand() % 0x300);
    for (auto &e : W) e = (uint16_t)(0x3c00 + rand() % 0x300);
    fn(rows, s.N, s.K, X.data(), W.data(), Y.data(), nullptr, rows, 0);     // warm pass
    const auto t0 = std::chrono::steady_clock::now();
    fn(rows, s.N, s.K, X.data(), W.data(), Y.data(), nullptr, rows, 0);
    const double sec = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    std::printf("host reference (FP32 loop, %d OpenMP threads of %u hardware threads): %d of %d rows of M=%d N=%d K=%d in %.3f s = %.1f GFLOP/s%s\n",
                nthreads(), std::thread::hardware_concurrency(), rows, s.M, s.M, s.N, s.K, sec, 2.0 * rows * s.N * s.K / sec / 1e9,
                rows < s.M ? " (row slab; the whole shape extrapolates linearly)" : "");
    return 0;      // the library stays loaded: its OpenMP worker threads outlive the call
}

// "hbm_gbs": 6553.3, "bf16_tflops": 1628.3 out of a small JSON file, without a JSON library
void read_peaks(const std::string &path)
{
    FILE *f = std::fopen(path.c_str(), "r");
    if (!f) { std::fprintf(stderr, "cannot open %s\n", path.c_str()); return; }
    std::string text(1 << 14, 0);
    text.resize(std::fread(&text[0], 1, text.size(), f));
    std::fclose(f);
    auto number = [&](const char *key) {
        const size_t at = text.find(std::string("\"") + key + "\"");
        return at == std::string::npos ? 0.0 : std::atof(text.c_str() + text.find(':', at) + 1);
    };
    g_measured_hbm_gbs = number("hbm_gbs");
    g_measured_bf16_tflops = number("bf16_tflops");
    std::printf("measured peaks (%s): %.1f GB/s HBM copy, %.1f TFLOPS cuBLAS bf16\n", path.c_str(), g_measured_hbm_gbs, g_measured_bf16_tflops);
}

// the plugins sit beside this executable unless --dir says otherwise
std::string default_kernel_dir()
{
    char buf[4096];
    const ssize_t n = readlink("/proc/self/exe", buf, sizeof(buf) - 1);
    if (n <= 0) return ".";
    buf[n] = 0;
    std::string p(buf);
    const size_t slash = p.rfind('/');
    std::string dir = slash == std::string::npos ? "." : p.substr(0, slash);
#ifdef KERNEL_DIR
    if (access((dir + "/libsm100gemm_util.so").c_str(), R_OK) != 0) dir = KERNEL_DIR;    // a build tree that keeps the plugins elsewhere
#endif
    return dir;
}

}  // namespace

int main(int argc, char **argv)
{
    Options o;
    o.dir = default_kernel_dir();
    std::vector<Shape> shapes;
    for (int i = 1; i < argc; i++) {
        const std::string a = argv[i];
        if (a == "--debug" || a == "--autotune" || a == "--aux") o.mode = a;
        else if (a == "--dir" && i + 1 < argc) o.dir = argv[++i];
        else if (a == "--cache" && i + 1 < argc) o.cache = argv[++i];
        else if (a == "--kernel" && i + 1 < argc) o.kernel = argv[++i];
        else if (a == "--host-ref" && i + 1 < argc) o.host_ref = argv[++i];
        else if (a == "--peaks" && i + 1 < argc) read_peaks(argv[++i]);
        else if (a == "--json" && i + 1 < argc) {
            g_json = std::fopen(argv[++i], "a");
            if (!g_json) { std::fprintf(stderr, "cannot open %s\n", argv[i]); return 2; }
        } else if (a == "--dtype" && i + 1 < argc) {
            o.dt = sm100::dtype_from_name(argv[++i]);
            if (o.dt < 0) { std::fprintf(stderr, "unknown --dtype %s\n", argv[i]); return 2; }
        } else if (a == "--shape" && i + 1 < argc) {
            Shape s{};
            if (std::sscanf(argv[++i], "%d,%d,%d", &s.M, &s.N, &s.K) != 3) { std::fprintf(stderr, "bad --shape\n"); return 2; }
            shapes.push_back(s);
        } else {
            std::fprintf(stderr, "usage: bench [--debug | --autotune | --aux] [--dtype bf16|fp8|mxfp8|w4a4|w4a16] [--dir D] [--cache F] [--shape M,N,K]...\n"
                                 "             [--kernel NAME] [--json FILE] [--peaks MEASURED_PEAKS.json] [--host-ref liboracle.so]\n");
            return 2;
        }
    }
    if (!shapes.empty()) {
        g_shapes = shapes;
        if (o.mode.empty() && o.kernel.empty()) o.mode = "--shape-list";     // quick mode on the given shapes: cache entry or heuristic pick
    }
    if (!o.kernel.empty()) {
        auto cfg = GemmConfig::parse(o.kernel);
        if (!cfg) { std::fprintf(stderr, "cannot parse configuration name %s\n", o.kernel.c_str()); return 2; }
        o.dt = cfg->dt;
    }
    if (!o.host_ref.empty()) host_reference_line(o.host_ref);
    int rc;
    if (o.mode == "--aux") rc = aux_mode();
    else if (o.mode == "--debug") rc = debug_mode();
    else if (o.mode == "--autotune") rc = autotune(o);
    else rc = quick(o);
    if (g_json) std::fclose(g_json);
    return rc;
}
