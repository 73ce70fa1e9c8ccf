// Host-only checks of csrc/gemm_config.h and csrc/tile_order.h (compiled with g++ and run by
// tests/test_host_config.py).  Prints "OK <n>" on success; any failed check prints and exits 1.
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <set>
#include <thread>

#include "../sm120_gemm_b200/csrc/gemm_config.h"
#include "../sm120_gemm_b200/csrc/tile_order.h"
#include "../sm120_gemm_b200/csrc/umma_desc.h"

static int checks = 0;
#define CHECK(cond)                                                          \
    do {                                                                     \
        checks++;                                                            \
        if (!(cond)) {                                                       \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);    \
            std::exit(1);                                                    \
        }                                                                    \
    } while (0)

int main(int argc, char **argv)
{
    // name <-> struct round trip, strictness of the parser
    GemmConfig c;
    c.dt = GEMM_DT_FP8; c.bm = 256; c.bn = 192; c.bk = 128; c.num_stages = 6; c.cg = 2; c.split_k = 4; c.swap_ab = 0; c.epi = 0;
    CHECK(c.name() == "fp8_bm256_bn192_bk128_s6_cg2_sk4_ab0_e0");
    auto p = GemmConfig::parse(c.name());
    CHECK(p && p->name() == c.name() && p->dt == GEMM_DT_FP8 && p->split_k == 4);
    CHECK(!GemmConfig::parse("bm128_bn64_bk64_s3_cwg2_wm32_wn32_sk1"));   // the reference's old names are not plugins of this build
    CHECK(!GemmConfig::parse("bf16_bm128_bn128_bk64_s4_cg1_sk1_ab0_e1_extra"));
    CHECK(!GemmConfig::parse("int8_bm128_bn128_bk64_s4_cg1_sk1_ab0_e1"));

    // validity: ragged M/N/K are fine, pitches must be 16-byte multiples, split-K needs whole equal slices
    GemmConfig b = *GemmConfig::parse("bf16_bm128_bn128_bk64_s4_cg1_sk1_ab0_e1");
    CHECK(b.is_valid_for(1, 8, 8) && b.is_valid_for(100, 136, 200));
    CHECK(!b.is_valid_for(128, 130, 64) && !b.is_valid_for(128, 128, 60) && !b.is_valid_for(0, 128, 64));
    GemmConfig sk = *GemmConfig::parse("bf16_bm128_bn128_bk64_s7_cg1_sk4_ab0_e0");
    CHECK(sk.is_valid_for(128, 4096, 14336) && !sk.is_valid_for(128, 4096, 14336 + 64) && !sk.is_valid_for(128, 128, 200));

    // the shared-memory model follows the tile family: 512-row tiles hold 32 KB of X per stage (two row blocks per
    // CTA), and with three stages four staging buffers instead of two
    GemmConfig t4 = *GemmConfig::parse("bf16_bm512_bn256_bk64_s4_cg2_sk1_ab0_e1");
    GemmConfig t3 = *GemmConfig::parse("bf16_bm512_bn256_bk64_s3_cg2_sk1_ab0_e1");
    GemmConfig p6 = *GemmConfig::parse("bf16_bm256_bn256_bk64_s6_cg2_sk1_ab0_e1");
    CHECK(t4.smem_bytes() == 4 * (32768 + 16384) + 2 * 16384 + (2 * 4 + 4) * 8 + 16 + 1024);
    CHECK(t3.smem_bytes() == 3 * (32768 + 16384) + 4 * 16384 + (2 * 3 + 4) * 8 + 16 + 1024);
    CHECK(p6.smem_bytes() == 6 * (16384 + 16384) + 2 * 16384 + (2 * 6 + 4) * 8 + 16 + 1024);
    CHECK(t4.smem_bytes() <= 232448 && t4.is_valid_for(1000, 520, 1088));

    // cache: round trip, legacy three-field keys, malformed lines skipped, atomic replace
    const std::string path = argc > 1 ? argv[1] : "/tmp/sm100_cache_test.txt";
    {
        std::ofstream f(path);
        f << "# comment\n"
          << "1024,1024,1024 bf16_bm128_bn128_bk64_s4_cg1_sk1_ab0_e1 0.0123\n"        // reference-format key
          << "fp8,1,8192,8192,8192 fp8_bm256_bn256_bk128_s6_cg2_sk1_ab0_e1 0.3\n"
          << "bf16,8,16384,16384,16384 bf16_bm256_bn256_bk64_s6_cg2_sk1_ab0_e1 1.5\n"
          << "garbage line\n"
          << "1,2 bf16_bm128_bn128_bk64_s4_cg1_sk1_ab0_e1 1.0\n"
          << "4096,4096,4096 not_a_config 1.0\n";
    }
    AutotuneCache cache;
    cache.quiet = true;
    CHECK(cache.load(path) && cache.entries.size() == 3);
    CHECK(cache.lookup(1024, 1024, 1024) && cache.lookup(1024, 1024, 1024)->time_ms == 0.0123);
    CHECK(cache.lookup(8192, 8192, 8192, GEMM_DT_FP8) && !cache.lookup(8192, 8192, 8192));
    CHECK(cache.lookup(16384, 16384, 16384, GEMM_DT_BF16, 8) && !cache.lookup(16384, 16384, 16384, GEMM_DT_BF16, 1));
    cache.store(128, 4096, 14336, sk, 0.02);
    CHECK(cache.save(path));
    AutotuneCache again;
    again.quiet = true;
    CHECK(again.load(path) && again.entries.size() == 4 && again.lookup(128, 4096, 14336)->config.name() == sk.name());
    AutotuneCache missing;
    CHECK(!missing.load(path + ".does_not_exist"));

    // registry: missing directory is reported, not fatal
    KernelRegistry none;
    none.quiet = true;
    CHECK(!none.load_dir("/nonexistent/kernel/dir"));

    // tile order is a bijection onto the grid for awkward sizes, including a narrower last band
    for (int num_m : {1, 3, 32, 64})
        for (int num_n : {1, 5, 16, 37})
            for (int group : {1, 4, 8, 16}) {
                std::set<std::pair<int, int>> seen;
                for (int t = 0; t < num_m * num_n; t++) {
                    int mb, nb;
                    sm100::tile_to_mn(t, num_m, num_n, group, mb, nb);
                    CHECK(mb >= 0 && mb < num_m && nb >= 0 && nb < num_n);
                    seen.insert({mb, nb});
                }
                CHECK((int)seen.size() == num_m * num_n);
            }

    // stream-K ranges tile the unit list and streamk_owner inverts streamk_range_begin
    for (long long units : {1LL, 7LL, 148LL, 1000LL, 74LL * 256 + 5})
        for (int nc : {1, 2, 74, 148}) {
            CHECK(sm100::streamk_range_begin(units, 0, nc) == 0 && sm100::streamk_range_begin(units, nc, nc) == units);
            for (long long u = 0; u < units; u += (units > 2000 ? 37 : 1)) {
                const int c = sm100::streamk_owner(units, u, nc);
                CHECK(c >= 0 && c < nc && sm100::streamk_range_begin(units, c, nc) <= u && u < sm100::streamk_range_begin(units, c + 1, nc));
            }
        }
    // a balanced grid is never larger and needs the same number of rounds
    for (int work : {1, 64, 74, 75, 128, 256, 512, 2048, 4097})
        for (int mx : {1, 64, 74, 148}) {
            const int b = sm100::balanced_units(work, mx);
            CHECK(b >= 1 && b <= mx && b <= work && (work + b - 1) / b == (work + mx - 1) / mx);
        }
    CHECK(sm100::balanced_units(256, 74) == 64 && sm100::balanced_units(2048, 74) == 74 && sm100::balanced_units(128, 74) == 64);

    // descriptor builders: field positions
    const uint64_t d = sm100::make_smem_desc_k128(0x12400);
    CHECK((d & 0x3fff) == (0x12400 >> 4) && ((d >> 32) & 0x3fff) == 64 && ((d >> 46) & 3) == 1 && (d >> 61) == 2);
    CHECK(sm100::advance_desc_k(d, 3) - d == 6);
    const uint32_t i = sm100::make_idesc(sm100::UMMA_BF16, sm100::UMMA_BF16, 256, 192);
    CHECK(((i >> 4) & 3) == 1 && ((i >> 7) & 7) == 1 && ((i >> 10) & 7) == 1 && ((i >> 17) & 63) == 24 && ((i >> 24) & 31) == 16);

    // with a plugin directory: the registry on real plugins, the heuristic dispatcher, two threads in the rejection paths
    if (argc > 2) {
        KernelRegistry reg;
        reg.quiet = true;
        CHECK(reg.load_dir(argv[2]) && reg.kernels.size() > 100);
        const LoadedKernel *sk4 = reg.find("bf16_bm128_bn128_bk64_s7_cg1_sk4_ab0_e0");
        const LoadedKernel *direct = reg.find("bf16_bm128_bn128_bk64_s6_cg1_sk1_ab0_e1");
        CHECK(sk4 && direct && sk4->run_no_alloc && direct->run_no_alloc);
        CHECK(sk4->run_no_alloc(2048, 2048, 1024, (void *)16, (void *)16, (void *)16, nullptr) == GEMM_ERR_WORKSPACE);   // 64 MiB of partials > 16 MiB
        CHECK(direct->run_no_alloc(128, 128, 1024, (void *)16, (void *)16, (void *)16, nullptr) == GEMM_ERR_ARG);       // no scratch in this plugin
        // one line per shape for the Python side to compare with its own model
        static const int shapes[][4] = {{0, 1024, 1024, 1024}, {0, 128, 4096, 14336}, {0, 128, 28672, 4096}, {0, 8192, 8192, 8192}, {0, 16384, 2048, 16384},
                                        {0, 512, 512, 14336}, {0, 1, 4096, 4096}, {0, 100, 136, 200}, {1, 8192, 8192, 8192}, {1, 128, 4096, 2048},
                                        {2, 8192, 8192, 8192}, {2, 256, 512, 1024}, {4, 16, 28672, 8192}, {4, 8192, 8192, 8192}, {3, 16, 28672, 8192},
                                        {3, 128, 28672, 8192}, {3, 1, 128, 128}};
        for (const auto &sh : shapes) {
            const LoadedKernel *k = heuristic_kernel(reg, sh[0], sh[1], sh[2], sh[3]);
            CHECK(k && k->can_run(sh[1], sh[2], sh[3]) && k->config.dt == sh[0] && k->config.epi != 2);
            std::printf("PICK %s %d %d %d %s\n", sm100::kDtypeNames[sh[0]], sh[1], sh[2], sh[3], k->config.name().c_str());
        }
        CHECK(heuristic_kernel(reg, GEMM_DT_BF16, 128, 130, 64) == nullptr);        // no plugin takes N % 8 != 0
        AutotuneCache empty;
        CHECK(select_kernel(reg, empty, GEMM_DT_BF16, 8192, 8192, 8192) == heuristic_kernel(reg, GEMM_DT_BF16, 8192, 8192, 8192));
        empty.store(8192, 8192, 8192, direct->config, 1.0);
        CHECK(select_kernel(reg, empty, GEMM_DT_BF16, 8192, 8192, 8192) == direct);
        // the error state is per thread and the one-time set-up paths tolerate concurrent first calls
        int codes[2] = {-1, -1};
        auto worker = [&](int t) {
            for (int i = 0; i < 200; i++) {
                if (t == 0) {
                    dispatch(*direct, 128, 130, 64, (void *)16, (void *)16, (void *)16, nullptr, nullptr);      // bad shape
                    if (direct->last_error() != GEMM_ERR_SHAPE) return;
                } else {
                    if (sk4->run_no_alloc(2048, 2048, 1024, (void *)16, (void *)16, (void *)16, nullptr) != GEMM_ERR_WORKSPACE) return;
                    if (sk4->last_error() != GEMM_ERR_WORKSPACE) return;
                }
            }
            codes[t] = 0;
        };
        std::thread a(worker, 0), b(worker, 1);
        a.join();
        b.join();
        CHECK(codes[0] == 0 && codes[1] == 0);
    }

    std::printf("OK %d\n", checks);
    return 0;
}
