// bench: the C++ harness around the kernel plugins.  Three modes, as in the reference's bench
// (src/bench.cu:583-597):
//   bench --autotune   every valid plugin per shape: correctness gate, then timing; best -> cache file
//   bench              quick: re-time the cached winner of every cached shape against cuBLAS
//   bench --debug      fixed configurations called through the class templates, verbose checks
// Options: --dir <plugin dir>  --cache <file>  --shape M,N,K (repeatable, replaces the built-in list)
//
// Kept from the reference because they define the metric: the timing protocol (bench_ms:
// warm-ups, per-launch event pairs, idle spacer, mean -- src/common.h:21-50), L2 flushing by
// rotating over enough buffer sets to exceed twice the L2 (src/bench.cu:381-395), flops = 2MNK
// (src/bench.cu:404), cuBLAS called as cublasGemmEx(OP_T, OP_N, N, M, K) on the same buffers
// (src/bench.cu:44-65), an FP32 GPU GEMM as the on-device check (src/bench.cu:68-95) and
// "never time a kernel that failed the check" (src/bench.cu:413-429).
// New: roofline fractions (2.25 PF dense bf16, 8 TB/s), status codes instead of exit().
#include <cublas_v2.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <memory>
#include <string>

#include "bf16_gemm.cuh"
#include "common.h"
#include "gemm_config.h"

#ifndef KERNEL_DIR
#define KERNEL_DIR "sm120_gemm_b200/kernels"
#endif

namespace {

constexpr double kPeakBf16Tflops = 2250.0, kPeakHbmGbs = 8000.0;

struct Shape { int M, N, K; };
// the reference's list (src/bench.cu:164-176) plus the 16384^3 family of the N-sharded runs
std::vector<Shape> g_shapes = {{512, 512, 14336}, {1024, 1024, 14336}, {1024, 1024, 1024}, {2048, 2048, 2048}, {4096, 4096, 4096},
                               {8192, 8192, 8192}, {4096, 28672, 4096}, {4096, 4096, 14336}, {128, 28672, 4096}, {128, 4096, 14336},
                               {16384, 16384, 16384}};

template <class T>
struct DevBuf {
    T *p = nullptr;
    size_t n = 0;
    explicit DevBuf(size_t count) : n(count) { if (cudaMalloc(&p, count * sizeof(T)) != cudaSuccess) p = nullptr; }
    ~DevBuf() { if (p) cudaFree(p); }
    DevBuf(const DevBuf &) = delete;
    DevBuf &operator=(const DevBuf &) = delete;
};

// uniform[-1,1] from srand(42)/rand(), rounded to bf16: the reference's inputs (src/bench.cu:36-43)
void fill_reference_random(std::vector<bf16> &v)
{
    for (auto &e : v) e = __float2bfloat16((float)rand() / (float)RAND_MAX * 2.0 - 1.0);
}

// FP32 check GEMM: one output per thread, k ascending (the loop of src/bench.cu:77-84)
__global__ void check_gemm_f32_kernel(int M, int N, int K, const bf16 *__restrict__ X, const bf16 *__restrict__ W, float *__restrict__ Y)
{
    const int col = blockIdx.x * blockDim.x + threadIdx.x, row = blockIdx.y * blockDim.y + threadIdx.y;
    if (row >= M || col >= N) return;
    const bf16 *x = X + (size_t)row * K, *w = W + (size_t)col * K;
    float acc = 0.f;
    for (int k = 0; k < K; k++) acc += __bfloat162float(x[k]) * __bfloat162float(w[k]);
    Y[(size_t)row * N + col] = acc;
}

struct ErrStats { float max_abs, max_rel; };
// the reference's metric: |y-ref| / max(|y|,|ref|,1)   (src/bench.cu:97-112)
ErrStats compare(const std::vector<bf16> &y, const std::vector<float> &ref)
{
    ErrStats s{0.f, 0.f};
    for (size_t i = 0; i < ref.size(); i++) {
        const float a = __bfloat162float(y[i]), d = std::fabs(a - ref[i]);
        s.max_abs = std::max(s.max_abs, std::isnan(a) ? INFINITY : d);
        s.max_rel = std::max(s.max_rel, std::isnan(a) ? INFINITY : d / std::max({std::fabs(a), std::fabs(ref[i]), 1.0f}));
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

// Everything one shape needs on the device: inputs, check values, rotating buffer sets.
struct Problem {
    int M, N, K, sets;
    std::vector<bf16> hX, hW;
    std::vector<float> hRef;
    std::vector<std::unique_ptr<DevBuf<bf16>>> X, W, Y;
    std::unique_ptr<DevBuf<float>> ws;
    int next = 0;
    bool ok = false;

    Problem(int m, int n, int k, size_t ws_bytes, cudaStream_t stream) : M(m), N(n), K(k)
    {
        hX.resize((size_t)M * K);
        hW.resize((size_t)N * K);
        srand(42);
        fill_reference_random(hX);
        fill_reference_random(hW);
        int dev = 0, l2 = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev);
        const size_t per_set = ((size_t)M * K + (size_t)N * K + (size_t)M * N) * sizeof(bf16);
        sets = std::min<size_t>(64, std::max<size_t>(1, (2 * (size_t)l2 + per_set - 1) / per_set));
        for (int i = 0; i < sets; i++) {
            X.emplace_back(new DevBuf<bf16>(hX.size()));
            W.emplace_back(new DevBuf<bf16>(hW.size()));
            Y.emplace_back(new DevBuf<bf16>((size_t)M * N));
            if (!X.back()->p || !W.back()->p || !Y.back()->p) return;
            cudaMemcpyAsync(X.back()->p, hX.data(), hX.size() * sizeof(bf16), cudaMemcpyHostToDevice, stream);
            cudaMemcpyAsync(W.back()->p, hW.data(), hW.size() * sizeof(bf16), cudaMemcpyHostToDevice, stream);
        }
        ws.reset(new DevBuf<float>(std::max<size_t>(ws_bytes, 16) / sizeof(float) + 4));
        DevBuf<float> ref((size_t)M * N);
        if (!ws->p || !ref.p) return;
        dim3 block(16, 16), grid((N + 15) / 16, (M + 15) / 16);
        check_gemm_f32_kernel<<<grid, block, 0, stream>>>(M, N, K, X[0]->p, W[0]->p, ref.p);
        hRef.resize((size_t)M * N);
        cudaMemcpyAsync(hRef.data(), ref.p, hRef.size() * sizeof(float), cudaMemcpyDeviceToHost, stream);
        ok = cudaStreamSynchronize(stream) == cudaSuccess;
    }
    int rotate() { return next++ % sets; }
    double flops() const { return 2.0 * M * N * K; }
    double bytes() const { return ((double)M * K + (double)N * K + (double)M * N) * 2.0; }
};

void print_rate(const char *label, const Problem &p, double ms, double cublas_ms)
{
    const double tf = p.flops() / ms / 1e9, gbs = p.bytes() / ms / 1e6;
    std::printf("  %-52s %.4f ms  %.2f TFLOPS  (%.1f%% of cuBLAS, %.1f%% of 2.25 PF, %.0f GB/s = %.1f%% of 8 TB/s)\n", label, ms, tf,
                100.0 * cublas_ms / ms, 100.0 * tf / kPeakBf16Tflops, gbs, 100.0 * gbs / kPeakHbmGbs);
}

// runs one plugin once and checks it; returns the reference's max-rel metric or a negative value on launch failure
float run_and_check(const LoadedKernel &k, Problem &p, cudaStream_t stream)
{
    cudaMemsetAsync(p.Y[0]->p, 0xff, (size_t)p.M * p.N * sizeof(bf16), stream);   // NaN pattern: unwritten outputs fail the check
    if (dispatch(k, p.M, p.N, p.K, p.X[0]->p, p.W[0]->p, p.Y[0]->p, p.ws->p, stream) != GEMM_OK) return -1.f;
    if (cudaStreamSynchronize(stream) != cudaSuccess || k.check_status() != GEMM_OK) return -1.f;
    std::vector<bf16> hY((size_t)p.M * p.N);
    cudaMemcpy(hY.data(), p.Y[0]->p, hY.size() * sizeof(bf16), cudaMemcpyDeviceToHost);
    return compare(hY, p.hRef).max_rel;
}

int autotune(const std::string &dir, const std::string &cache_path)
{
    cudaStream_t stream;
    CHECK_CUDA(cudaStreamCreate(&stream));
    cublasHandle_t handle;
    if (cublasCreate(&handle) != CUBLAS_STATUS_SUCCESS) return 1;
    cublasSetStream(handle, stream);
    KernelRegistry registry;
    if (!registry.load_dir(dir, GEMM_DT_BF16)) { std::fprintf(stderr, "No kernels found in %s\n", dir.c_str()); return 1; }
    AutotuneCache cache;
    cache.load(cache_path);
    int dev = 0, max_smem = 0;
    CHECK_CUDA(cudaGetDevice(&dev));
    CHECK_CUDA(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    std::printf("Device max dynamic smem: %d bytes (%.1f KB)\n", max_smem, max_smem / 1024.0);
    auto last_save = std::chrono::steady_clock::now();
    for (const Shape &s : g_shapes) {
        std::printf("\n=== Autotune M=%d N=%d K=%d ===\n", s.M, s.N, s.K);
        if (auto hit = cache.lookup(s.M, s.N, s.K)) { std::printf("  cached: %s  %.4f ms\n", hit->config.name().c_str(), hit->time_ms); continue; }
        auto valid = registry.get_valid(s.M, s.N, s.K, max_smem);
        std::printf("  %zu valid configs\n", valid.size());
        if (valid.empty()) { std::printf("  SKIP (no valid configs)\n"); continue; }
        size_t ws_bytes = 0;
        for (auto *k : valid) ws_bytes = std::max(ws_bytes, k->workspace_bytes(s.M, s.N, s.K));
        Problem p(s.M, s.N, s.K, ws_bytes, stream);
        if (!p.ok) { std::printf("  SKIP (could not set the problem up: out of memory?)\n"); continue; }
        const double cublas_ms = bench_ms([&] { int b = p.rotate(); cublas_gemm(handle, p.M, p.N, p.K, p.X[b]->p, p.W[b]->p, p.Y[b]->p); }, stream);
        std::printf("  cuBLAS: %.4f ms  %.4f TFLOPS\n", cublas_ms, p.flops() / cublas_ms / 1e9);
        const LoadedKernel *best = nullptr;
        double best_ms = 1e30;
        for (auto *k : valid) {
            const float rel = run_and_check(*k, p, stream);
            if (rel < 0.f) { std::printf("  %-52s LAUNCH FAIL (%s)\n", k->config.name().c_str(), k->last_error_message()); cudaGetLastError(); continue; }
            if (!(rel < 0.02f)) { std::printf("  %-52s FAILED check (max rel err %g)\n", k->config.name().c_str(), rel); continue; }
            const double ms = bench_ms([&] { int b = p.rotate(); dispatch(*k, p.M, p.N, p.K, p.X[b]->p, p.W[b]->p, p.Y[b]->p, p.ws->p, stream); }, stream);
            if (ms < 0 || k->check_status() != GEMM_OK) continue;
            print_rate(k->config.name().c_str(), p, ms, cublas_ms);
            if (ms < best_ms) { best_ms = ms; best = k; }
        }
        if (best) {
            std::printf("  BEST:");
            print_rate(best->config.name().c_str(), p, best_ms, cublas_ms);
            cache.store(s.M, s.N, s.K, best->config, best_ms);
        } else {
            std::printf("  NO VALID CONFIG\n");
        }
        if (std::chrono::steady_clock::now() - last_save > std::chrono::seconds(30)) { cache.save(cache_path); last_save = std::chrono::steady_clock::now(); }
    }
    cache.save(cache_path);
    std::printf("\nAutotune complete.\n");
    return 0;
}

int quick(const std::string &dir, const std::string &cache_path)
{
    AutotuneCache cache;
    if (!cache.load(cache_path) || cache.entries.empty()) { std::printf("No autotune cache found. Run with --autotune first.\n"); return 1; }
    KernelRegistry registry;
    if (!registry.load_dir(dir, GEMM_DT_BF16)) { std::fprintf(stderr, "No kernels found in %s\n", dir.c_str()); return 1; }
    cudaStream_t stream;
    CHECK_CUDA(cudaStreamCreate(&stream));
    cublasHandle_t handle;
    if (cublasCreate(&handle) != CUBLAS_STATUS_SUCCESS) return 1;
    cublasSetStream(handle, stream);
    for (const auto &[key, entry] : cache.entries) {
        const auto &[dt, gpus, M, N, K] = key;
        if (dt != GEMM_DT_BF16 || gpus != 1) continue;
        std::printf("\n=== M=%d N=%d K=%d  config=%s ===\n", M, N, K, entry.config.name().c_str());
        const LoadedKernel *k = registry.find(entry.config.name());
        if (!k) { std::printf("  kernel .so not found, skipping\n"); continue; }
        Problem p(M, N, K, k->workspace_bytes(M, N, K), stream);
        if (!p.ok) { std::printf("  could not set the problem up, skipping\n"); continue; }
        const double cublas_ms = bench_ms([&] { int b = p.rotate(); cublas_gemm(handle, M, N, K, p.X[b]->p, p.W[b]->p, p.Y[b]->p); }, stream);
        const double ms = bench_ms([&] { int b = p.rotate(); dispatch(*k, M, N, K, p.X[b]->p, p.W[b]->p, p.Y[b]->p, p.ws->p, stream); }, stream);
        std::printf("  cuBLAS:  %.4f ms  %.4f TFLOPS\n", cublas_ms, p.flops() / cublas_ms / 1e9);
        std::printf("  Ours:    %.4f ms  %.4f TFLOPS  (%.1f%% of cuBLAS)\n", ms, p.flops() / ms / 1e9, 100.0 * cublas_ms / ms);
        print_rate("roofline", p, ms, cublas_ms);
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
        Problem p(s.M, s.N, s.K, (size_t)2 * s.M * s.N * sizeof(float), stream);
        if (!p.ok) { std::printf("  could not set the problem up\n"); return 1; }
        std::vector<bf16> hY((size_t)s.M * s.N), hC((size_t)s.M * s.N);
        cublas_gemm(handle, s.M, s.N, s.K, p.X[0]->p, p.W[0]->p, p.Y[0]->p);
        CHECK_CUDA(cudaStreamSynchronize(stream));
        cudaMemcpy(hC.data(), p.Y[0]->p, hC.size() * sizeof(bf16), cudaMemcpyDeviceToHost);
        const ErrStats ec = compare(hC, p.hRef);
        for (int variant = 0; variant < 2; variant++) {
            const char *label = variant == 0 ? "MMA" : "MMA-SK";
            cudaMemsetAsync(p.Y[0]->p, 0xff, hY.size() * sizeof(bf16), stream);
            const int rc = variant == 0 ? Direct::run(s.M, s.N, s.K, p.X[0]->p, p.W[0]->p, p.Y[0]->p, stream)
                                        : Split::run(s.M, s.N, s.K, p.X[0]->p, p.W[0]->p, p.Y[0]->p, p.ws->p, stream);
            if (rc == GEMM_ERR_SHAPE) { std::printf("[%s] shape not supported by this configuration, skipped\n", label); continue; }
            if (rc != GEMM_OK || cudaStreamSynchronize(stream) != cudaSuccess) { std::printf("[%s] FAILED to launch\n", label); return 1; }
            cudaMemcpy(hY.data(), p.Y[0]->p, hY.size() * sizeof(bf16), cudaMemcpyDeviceToHost);
            const ErrStats e = compare(hY, p.hRef);
            std::printf("[%s] vs fp32 ref:  abs=%f rel=%f\n[%s] cuBLAS vs ref: abs=%f rel=%f\n", label, e.max_abs, e.max_rel, label, ec.max_abs, ec.max_rel);
            if (!(e.max_rel < 0.02f)) { std::printf("[%s] FAILED\n", label); return 1; }
            std::printf("[%s] PASSED\n", label);
            const double ms = bench_ms([&] {
                int b = p.rotate();
                if (variant == 0) Direct::run(s.M, s.N, s.K, p.X[b]->p, p.W[b]->p, p.Y[b]->p, stream);
                else Split::run(s.M, s.N, s.K, p.X[b]->p, p.W[b]->p, p.Y[b]->p, p.ws->p, stream);
            }, stream);
            std::printf("[%s] %.4f ms  %.4f TFLOPS\n", label, ms, p.flops() / ms / 1e9);
        }
    }
    return 0;
}

}  // namespace

int main(int argc, char **argv)
{
    std::string mode, dir = KERNEL_DIR, cache = "autotune_cache.txt";
    std::vector<Shape> shapes;
    for (int i = 1; i < argc; i++) {
        const std::string a = argv[i];
        if (a == "--debug" || a == "--autotune") mode = a;
        else if (a == "--dir" && i + 1 < argc) dir = argv[++i];
        else if (a == "--cache" && i + 1 < argc) cache = argv[++i];
        else if (a == "--shape" && i + 1 < argc) {
            Shape s{};
            if (std::sscanf(argv[++i], "%d,%d,%d", &s.M, &s.N, &s.K) != 3) { std::fprintf(stderr, "bad --shape\n"); return 2; }
            shapes.push_back(s);
        } else { std::fprintf(stderr, "usage: bench [--debug | --autotune] [--dir D] [--cache F] [--shape M,N,K]...\n"); return 2; }
    }
    if (!shapes.empty()) g_shapes = shapes;
    if (mode == "--debug") return debug_mode();
    if (mode == "--autotune") return autotune(dir, cache);
    return quick(dir, cache);
}
