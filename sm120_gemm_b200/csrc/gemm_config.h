// Host-side registry, configuration parser, autotune cache and dispatch for the sm_100a
// kernel plugins.  Header-only C++17; needs only libdl and the C ABI in include/sm100_gemm.h.
//
// It keeps the reference's host surface by name so a caller of src/gemm_config.h can switch
// over: GemmConfig (reference :24-55), LoadedKernel (:58-62), KernelRegistry (:65-120),
// AutotuneCache (:124-170), dispatch (:173-178).  What changed and why:
//   * the configuration fields are those of the tcgen05 kernels (data type, CTA group,
//     operand swap, epilogue kind) instead of warp tilings;
//   * a plugin answers can_run / workspace_bytes / smem_bytes itself, so the host-side model
//     cannot drift from the kernel (the reference keeps three copies of the smem formula);
//   * the cache key carries the data type and the GPU count, the file is replaced atomically,
//     and old three-field lines are still read as bf16 on one GPU;
//   * errors come back as status codes; nothing here calls exit().
#pragma once
#include <dlfcn.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <map>
#include <optional>
#include <string>
#include <tuple>
#include <vector>

#include "../../include/sm100_gemm.h"

namespace sm100 {
inline const char *const kDtypeNames[] = {"bf16", "fp8", "mxfp8", "w4a16", "w4a4"};
inline int dtype_from_name(const char *s)
{
    for (int i = 0; i < 5; i++)
        if (std::strcmp(s, kDtypeNames[i]) == 0) return i;
    return -1;
}
inline int elem_bits(int dt) { return dt == GEMM_DT_BF16 || dt == GEMM_DT_W4A16 ? 16 : dt == GEMM_DT_W4A4 ? 4 : 8; }
}  // namespace sm100

struct GemmConfig {
    int dt = GEMM_DT_BF16;  // GEMM_DT_*
    int bm = 128, bn = 128, bk = 64, num_stages = 4;
    int cg = 1;             // CTA group: 1, or 2 for a CTA pair sharing one 256-row tile
    int split_k = 1;        // 1: none; >1: equal K slices + reduce; 0: stream-K (equal unit ranges per CTA)
    int swap_ab = 0;        // 1: W rows on the accumulator lanes (small-M shapes)
    int epi = 1;            // 0: register->global epilogue, 1: shared memory + TMA store

    std::string name() const
    {
        char buf[160];
        std::snprintf(buf, sizeof(buf), "%s_bm%d_bn%d_bk%d_s%d_cg%d_sk%d_ab%d_e%d", sm100::kDtypeNames[dt], bm, bn, bk,
                      num_stages, cg, split_k, swap_ab, epi);
        return buf;
    }

    static std::optional<GemmConfig> parse(const std::string &s)
    {
        GemmConfig c;
        char dt_name[16] = {0};
        int consumed = 0;
        int n = std::sscanf(s.c_str(), "%15[a-z0-9]_bm%d_bn%d_bk%d_s%d_cg%d_sk%d_ab%d_e%d%n", dt_name, &c.bm, &c.bn, &c.bk,
                            &c.num_stages, &c.cg, &c.split_k, &c.swap_ab, &c.epi, &consumed);
        if (n != 9 || consumed != (int)s.size()) return std::nullopt;
        c.dt = sm100::dtype_from_name(dt_name);
        if (c.dt < 0) return std::nullopt;
        return c;
    }

    // Shapes the dense kernels accept: 16-byte row pitches; split-K needs equal, whole K slices.
    // M, N, K need not divide by the tile (TMA zero-fills and clips), unlike the reference.
    bool is_valid_for(int M, int N, int K) const
    {
        if (M <= 0 || N <= 0 || K <= 0) return false;
        if (dt == GEMM_DT_W4A16) return M <= bn && N % 8 == 0 && K % 128 == 0;   // decode kernel, bn = padded M
        if (((long long)K * sm100::elem_bits(dt)) % 128 != 0 || N % 8 != 0) return false;
        if ((dt == GEMM_DT_MXFP8 || dt == GEMM_DT_W4A4) && K % bk != 0) return false;
        if (split_k > 1 && (K % bk != 0 || (K / bk) % split_k != 0)) return false;
        return true;
    }

    // Dynamic shared memory of the dense kernel (must equal UmmaGemmTraits::SMEM_ALLOC;
    // a plugin reports the exact figure through gemm_smem_bytes()).
    size_t smem_bytes() const
    {
        if (dt == GEMM_DT_W4A16 && bk == 128) {   // tensor-memory family: load ring only (16 KB packed + 4 activation boxes per stage)
            const size_t load_stage = 128 * 128 + 4 * (((size_t)bn * 128 + 1023) / 1024 * 1024);
            const size_t fit = (200 * 1024) / load_stage;
            const size_t load_stages = fit > 8 ? 8 : fit;
            return load_stages * load_stage + (2 * load_stages + 3 * (size_t)num_stages) * 8 + 16 + 1024;
        }
        if (dt == GEMM_DT_W4A16) {   // group ring (num_stages slots of two bf16 tiles) + load ring (16 KB packed + 4 activation boxes)
            const size_t load_stage = 128 * 128 + 4 * (((size_t)bn * 128 + 1023) / 1024 * 1024);
            const size_t fit = (224 * 1024 - (size_t)num_stages * 2 * 128 * 128) / load_stage;
            const size_t load_stages = fit > 4 ? 4 : fit;
            return (size_t)num_stages * 2 * 128 * 128 + load_stages * load_stage + (2 * load_stages + 3 * (size_t)num_stages) * 8 + 16 + 1024;
        }
        const size_t k_atoms = (dt == GEMM_DT_MXFP8 || dt == GEMM_DT_W4A4) ? bk / 128 : 0;   // 512-byte scale atoms per stage
        const size_t n_atoms = (bn + 127) / 128;
        const size_t sf_ring = (num_stages * k_atoms * (1 + n_atoms) * 512 + 1023) / 1024 * 1024;
        const size_t mb = bm / (128 * cg) > 0 ? bm / (128 * cg) : 1;
        const size_t a = (size_t)128 * 128 * mb, b = (size_t)(bn / cg) * 128;
        const size_t barriers = (2 * (size_t)num_stages + 4 + (k_atoms ? 4 : 0)) * 8 + 16;   // block-scaled: + scale set ready / free
        const size_t ring = num_stages * (a + b) + sf_ring + barriers + 1024;
        // a single accumulator stage (two do not fit in TMEM) gets four staging buffers when they fit
        const bool one_acc_stage = 2 * mb * (((size_t)bn + 31) / 32 * 32) + 2 * k_atoms * (1 + n_atoms) * 4 > 512;
        const size_t bufs = (one_acc_stage && ring + 4 * 128 * 64 * 2 <= 232448) ? 4 : 2;
        const size_t staging = (split_k <= 1 && epi == 1) ? bufs * 128 * 64 * 2 : 0;
        return ring + staging;
    }
};

// Function-pointer types of the plugin ABI.
using GemmKernelFn = void (*)(int M, int N, int K, const void *X, const void *W, void *Y, float *workspace, gemm_stream_t stream);
using GemmKernelExFn = int (*)(const GemmArgs *);

struct LoadedKernel {
    GemmConfig config;
    GemmKernelFn fn = nullptr;       // gemm_run
    GemmKernelExFn fn_ex = nullptr;  // gemm_run_ex
    size_t (*workspace_bytes)(int, int, int) = nullptr;
    int (*can_run)(int, int, int) = nullptr;
    size_t (*smem_bytes)() = nullptr;
    int (*last_error)() = nullptr;
    const char *(*last_error_message)() = nullptr;
    int (*check_status)() = nullptr;
    // bf16 split-K plugins: the GEMM with its partial sums in the plugin's built-in scratch array (no allocation
    // anywhere); other plugins export the symbol too and answer GEMM_ERR_ARG
    int (*run_no_alloc)(int M, int N, int K, const void *X, const void *W, void *Y, gemm_stream_t stream) = nullptr;
    void *dl_handle = nullptr;
};

struct KernelRegistry {
    std::vector<LoadedKernel> kernels;
    bool quiet = false;

    KernelRegistry() = default;
    KernelRegistry(const KernelRegistry &) = delete;
    KernelRegistry &operator=(const KernelRegistry &) = delete;

    // Loads every libgemm_<config>.so of `dir`; files that do not parse, do not load or miss
    // a symbol are reported and skipped.  Returns whether anything was loaded.
    bool load_dir(const std::string &dir, int only_dt = -1)
    {
        namespace fs = std::filesystem;
        std::error_code ec;
        if (!fs::is_directory(dir, ec)) {
            std::fprintf(stderr, "KernelRegistry: not a directory: %s\n", dir.c_str());
            return false;
        }
        std::vector<fs::path> files;
        for (const auto &e : fs::directory_iterator(dir, ec))
            if (e.path().extension() == ".so") files.push_back(e.path());
        std::sort(files.begin(), files.end());
        static const std::string prefix = "libgemm_";
        for (const auto &path : files) {
            const std::string stem = path.stem().string();
            if (stem.compare(0, prefix.size(), prefix) != 0) continue;
            auto cfg = GemmConfig::parse(stem.substr(prefix.size()));
            if (!cfg) {
                std::fprintf(stderr, "KernelRegistry: cannot parse config from %s\n", stem.c_str());
                continue;
            }
            if (only_dt >= 0 && cfg->dt != only_dt) continue;
            void *h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
            if (!h) {
                std::fprintf(stderr, "KernelRegistry: dlopen failed for %s: %s\n", path.c_str(), dlerror());
                continue;
            }
            LoadedKernel k;
            k.config = *cfg;
            k.dl_handle = h;
            bool ok = true;
            auto sym = [&](const char *name) {
                void *p = dlsym(h, name);
                if (!p) {
                    std::fprintf(stderr, "KernelRegistry: dlsym(%s) failed for %s\n", name, path.c_str());
                    ok = false;
                }
                return p;
            };
            k.fn = reinterpret_cast<GemmKernelFn>(sym("gemm_run"));
            k.fn_ex = reinterpret_cast<GemmKernelExFn>(sym("gemm_run_ex"));
            k.workspace_bytes = reinterpret_cast<size_t (*)(int, int, int)>(sym("gemm_workspace_bytes"));
            k.can_run = reinterpret_cast<int (*)(int, int, int)>(sym("gemm_can_run"));
            k.smem_bytes = reinterpret_cast<size_t (*)()>(sym("gemm_smem_bytes"));
            k.last_error = reinterpret_cast<int (*)()>(sym("gemm_last_error"));
            k.last_error_message = reinterpret_cast<const char *(*)()>(sym("gemm_last_error_message"));
            k.check_status = reinterpret_cast<int (*)()>(sym("gemm_check_status"));
            k.run_no_alloc = reinterpret_cast<int (*)(int, int, int, const void *, const void *, void *, gemm_stream_t)>(sym("gemm_run_no_alloc"));
            auto name_fn = reinterpret_cast<const char *(*)()>(sym("gemm_config_name"));
            if (ok && cfg->name() != name_fn()) {
                std::fprintf(stderr, "KernelRegistry: %s was built as %s\n", stem.c_str(), name_fn());
                ok = false;
            }
            if (!ok) {
                dlclose(h);
                continue;
            }
            kernels.push_back(k);
        }
        if (!quiet) std::printf("KernelRegistry: loaded %zu kernels from %s\n", kernels.size(), dir.c_str());
        return !kernels.empty();
    }

    std::vector<const LoadedKernel *> get_valid(int M, int N, int K, size_t max_smem = 0, int dt = GEMM_DT_BF16) const
    {
        std::vector<const LoadedKernel *> out;
        for (const auto &k : kernels) {
            if (k.config.dt != dt || !k.can_run(M, N, K)) continue;
            if (max_smem > 0 && k.smem_bytes() > max_smem) continue;
            out.push_back(&k);
        }
        return out;
    }

    const LoadedKernel *find(const std::string &name) const
    {
        for (const auto &k : kernels)
            if (k.config.name() == name) return &k;
        return nullptr;
    }

    ~KernelRegistry()
    {
        for (auto &k : kernels)
            if (k.dl_handle) dlclose(k.dl_handle);
    }
};

// Text file, one result per line:  dt,gpus,M,N,K config_name time_ms   ('#' starts a comment).
struct AutotuneCache {
    using Key = std::tuple<int, int, int, int, int>;  // dt, gpus, M, N, K
    struct Entry {
        GemmConfig config;
        double time_ms;
    };
    std::map<Key, Entry> entries;
    bool quiet = false;

    bool load(const std::string &path)
    {
        std::ifstream f(path);
        if (!f.is_open()) return false;
        std::string line;
        size_t skipped = 0;
        while (std::getline(f, line)) {
            if (line.empty() || line[0] == '#') continue;
            char key[96], name[160];
            double ms = 0;
            if (std::sscanf(line.c_str(), "%95s %159s %lf", key, name, &ms) != 3) { skipped++; continue; }
            auto cfg = GemmConfig::parse(name);
            char dt_name[16];
            int g, M, N, K, used = 0;
            Key k;
            if (std::sscanf(key, "%15[a-z0-9],%d,%d,%d,%d%n", dt_name, &g, &M, &N, &K, &used) == 5 && key[used] == 0 &&
                sm100::dtype_from_name(dt_name) >= 0)
                k = {sm100::dtype_from_name(dt_name), g, M, N, K};
            else if (std::sscanf(key, "%d,%d,%d%n", &M, &N, &K, &used) == 3 && key[used] == 0)
                k = {GEMM_DT_BF16, 1, M, N, K};   // the reference's key format
            else { skipped++; continue; }
            if (!cfg) { skipped++; continue; }
            entries[k] = {*cfg, ms};
        }
        if (!quiet) std::printf("AutotuneCache: loaded %zu entries from %s (%zu lines skipped)\n", entries.size(), path.c_str(), skipped);
        return true;
    }

    bool save(const std::string &path) const
    {
        const std::string tmp = path + ".tmp";
        {
            std::ofstream f(tmp);
            if (!f.is_open()) return false;
            f << "# Autotune cache -- dt,gpus,M,N,K config_name time_ms\n";
            for (const auto &[key, e] : entries) {
                const auto &[dt, g, M, N, K] = key;
                f << sm100::kDtypeNames[dt] << ',' << g << ',' << M << ',' << N << ',' << K << ' ' << e.config.name() << ' ' << e.time_ms << '\n';
            }
        }
        std::error_code ec;
        std::filesystem::rename(tmp, path, ec);
        if (!quiet) std::printf("AutotuneCache: saved %zu entries to %s\n", entries.size(), path.c_str());
        return !ec;
    }

    std::optional<Entry> lookup(int M, int N, int K, int dt = GEMM_DT_BF16, int gpus = 1) const
    {
        auto it = entries.find({dt, gpus, M, N, K});
        if (it == entries.end()) return std::nullopt;
        return it->second;
    }

    void store(int M, int N, int K, const GemmConfig &config, double time_ms, int dt = GEMM_DT_BF16, int gpus = 1)
    {
        entries[{dt, gpus, M, N, K}] = {config, time_ms};
    }
};

// One indirect call into the plugin, BF16 operands (the reference's dispatch).  Returns the
// plugin's error code for the call (GEMM_OK when the launch was queued).
inline int dispatch(const LoadedKernel &kernel, int M, int N, int K, const void *X, const void *W, void *Y, float *workspace,
                    gemm_stream_t stream)
{
    kernel.fn(M, N, K, X, W, Y, workspace, stream);
    return kernel.last_error();
}

// ---------------------------------------------------------------------------------- heuristic dispatch
// A configuration for a shape that is not in the autotune cache, from a cost model instead of a measurement
// (the reference has no such path: it prints "NO VALID CONFIG" or skips the shape, src/bench.cu:345-349, 455-458).
// The model: the work is cut into tiles x split units dealt over the persistent grid in whole rounds; a unit costs
// the larger of its tensor time (peak of the data type, derated for small tiles) and its streaming time (what one
// SM can pull from memory), the whole launch cannot beat the algorithmic bytes over the HBM rate, and split-K pays
// for its reduce kernel.  Only +,-,*,/ and ceil on doubles, so the Python mirror (gen_configs.heuristic_ms)
// computes the same numbers; ties go to the name that sorts first.
inline double heuristic_ms(const GemmConfig &c, int M, int N, int K, int sms = 148)
{
    static const double peak_tflops[5] = {2250.0, 4500.0, 4500.0, 2250.0, 9000.0};
    const double hbm = 6.5e12, sm_stream = 9.0e10, launch_us = 4.0;
    const double eb = sm100::elem_bits(c.dt) / 8.0;                         // bytes per operand element
    const double wb = c.dt == GEMM_DT_W4A16 ? 0.5 : eb;
    const double alg_bytes = (double)M * K * eb + (double)N * K * wb + (double)M * N * 2.0;
    if (c.dt == GEMM_DT_W4A16)    // one kernel family: the narrowest padded M that fits, then the deeper ring
        return alg_bytes / hbm * 1e3 + c.bn * 1e-4 - c.num_stages * 1e-6;
    const double slots = (double)(sms / c.cg);
    const double tiles = std::ceil((double)M / c.bm) * std::ceil((double)N / c.bn);
    const double eff_m = c.bm >= 512 ? 1.0 : c.bm >= 256 ? 0.92 : 0.80;
    const double eff_n = 0.55 + 0.45 * (c.bn < 256 ? c.bn : 256) / 256.0;
    const double slot_flops = peak_tflops[c.dt] * 1e12 * c.cg / sms * eff_m * eff_n;
    const double split = c.split_k > 1 ? c.split_k : 1;
    const double unit_flops = 2.0 * c.bm * c.bn * (double)K / split;
    const double unit_bytes = ((double)c.bm * eb + (double)c.bn * wb) * (double)K / split;
    const double slot_bw = sm_stream * c.cg;
    double t;
    if (c.split_k == 0) {         // stream-K: every slot gets the same share
        const double share = tiles / (tiles < slots ? tiles : slots);
        const double tt = share * unit_flops / slot_flops, tm = share * unit_bytes / slot_bw;
        // + the FP32 partial tiles (two per CTA) written, read back and reduced by the fix-up kernel
        t = (tt > tm ? tt : tm) * (tiles < slots ? tiles / slots : 1.0) + 4.0 * slots * c.bm * c.bn * 4.0 / 5.0e12 + 4e-6;
    } else {
        double rounds = std::ceil(tiles * split / slots);
        if (c.bm == 256 * c.cg && c.split_k == 1 && tiles > slots) {
            // two-row-block kernels deal the tiles of a last wave that would leave half the clusters idle as halves
            const double rest = tiles - std::floor(tiles / slots) * slots;
            if (rest > 0 && 2.0 * rest <= slots) rounds -= 0.5;
        }
        const double tt = unit_flops / slot_flops, tm = unit_bytes / slot_bw;
        t = rounds * (tt > tm ? tt : tm);
        if (c.split_k > 1) t += (4.0 * split + 2.0) * M * N / 5.0e12 + 3e-6;
    }
    if (c.epi == 0 && M >= 1024) t *= 1.03;       // direct stores do not overlap the next tile as well as TMA stores
    const double floor_t = alg_bytes / hbm;
    if (t < floor_t) t = floor_t;
    t -= c.num_stages * 1e-9;                      // between otherwise equal configurations, the deeper ring
    return (t + launch_us * 1e-6) * 1e3;
}

// The loaded plugin of data type `dt` with the smallest modelled time for the shape (fused-transform plugins
// are left out: they compute the same product and are asked for by name); nullptr when none can run it.
inline const LoadedKernel *heuristic_kernel(const KernelRegistry &reg, int dt, int M, int N, int K, int sms = 148)
{
    const LoadedKernel *best = nullptr;
    double best_ms = 0;
    std::string best_name;
    for (const auto &k : reg.kernels) {
        if (k.config.dt != dt || k.config.epi == 2 || !k.can_run(M, N, K)) continue;
        const double ms = heuristic_ms(k.config, M, N, K, sms);
        const std::string name = k.config.name();
        if (!best || ms < best_ms || (ms == best_ms && name < best_name)) { best = &k; best_ms = ms; best_name = name; }
    }
    return best;
}

// dispatch for callers that do not autotune: the cache entry when there is one, else the heuristic pick
inline const LoadedKernel *select_kernel(const KernelRegistry &reg, const AutotuneCache &cache, int dt, int M, int N, int K, int gpus = 1)
{
    if (auto hit = cache.lookup(M, N, K, dt, gpus))
        if (const LoadedKernel *k = reg.find(hit->config.name())) return k;
    return heuristic_kernel(reg, dt, M, N, K);
}
