// Offline side of the quantised weights: host packers into the kernel-native layouts and a small
// file format that stores a weight matrix in exactly the bytes the plugins read, so that loading
// is one read per payload straight into the buffers handed to gemm_run_ex.  Host code only (part
// of libsm100gemm_util.so, C ABI in include/sm100_gemm_util.h).  No counterpart in the reference:
// its weights are random bf16 generated in memory (src/bench.cu:353-355).
//
// File layout (little-endian):
//   [0, 256)    header (GemmWeightFileInfo at offset 0, zero padded)
//   [256, ...)  element payload: fp8 N*K bytes | mxfp8 N*K | w4a4 N*K/2 (e2m1, low nibble = even k)
//               | w4a16 N*K/2 (int4 two's complement, low nibble = even k) | bf16 N*K*2
//   next 256-byte boundary: scale payload: mx kinds: ue8m0 in 512-byte atoms (include/sm100_gemm.h),
//               w4a16: bf16 [N][K/128]; fp8: none (the per-tensor scale is in the header); bf16: none
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>

#include "../../include/sm100_gemm.h"
#include "../../include/sm100_gemm_util.h"

namespace {

constexpr char kMagic[8] = {'S', 'M', '1', '0', '0', 'Q', 'W', 0};
constexpr uint32_t kVersion = 1, kLayout = 1;
constexpr size_t kAlign = 256;

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// FNV-1a, 32 bit, continued over several buffers
uint32_t fnv1a(uint32_t h, const void *data, size_t n)
{
    const uint8_t *p = static_cast<const uint8_t *>(data);
    for (size_t i = 0; i < n; i++) {
        h ^= p[i];
        h *= 16777619u;
    }
    return h;
}

struct FileCloser {
    void operator()(FILE *f) const { if (f) std::fclose(f); }
};
using File = std::unique_ptr<FILE, FileCloser>;

size_t tiled_offset(long long r, int kb, int k_atoms)
{
    return ((size_t)(r >> 7) * k_atoms + (kb >> 2)) * 512 + (size_t)(r & 31) * 16 + (size_t)((r & 127) >> 5) * 4 + (kb & 3);
}

}  // namespace

extern "C" {

size_t gemm_packed_weight_bytes(int dtype, long long N, int K)
{
    if (N <= 0 || K <= 0) return 0;
    switch (dtype) {
    case GEMM_DT_BF16: return (size_t)N * K * 2;
    case GEMM_DT_FP8:
    case GEMM_DT_MXFP8: return (size_t)N * K;
    case GEMM_DT_W4A16:
    case GEMM_DT_W4A4: return (size_t)N * K / 2;
    default: return 0;
    }
}

size_t gemm_packed_scale_bytes(int dtype, long long N, int K)
{
    if (N <= 0 || K <= 0) return 0;
    switch (dtype) {
    case GEMM_DT_MXFP8:
    case GEMM_DT_W4A4: return (size_t)((N + 127) / 128) * (size_t)((K / 32 + 3) / 4) * 512;
    case GEMM_DT_W4A16: return (size_t)N * (K / 128) * 2;
    default: return 0;
    }
}

// values in [-8, 7], one per int8 -> two per byte, low nibble = even k (out: N*K/2 bytes)
int gemm_pack_int4_host(const int8_t *q, long long N, int K, uint8_t *out)
{
    if (!q || !out || N <= 0 || K <= 0 || K % 2 != 0) return GEMM_FILE_ERR_ARG;
    const size_t n = (size_t)N * K / 2;
    for (size_t i = 0; i < n; i++) {
        const int lo = q[2 * i], hi = q[2 * i + 1];
        if (lo < -8 || lo > 7 || hi < -8 || hi > 7) return GEMM_FILE_ERR_ARG;
        out[i] = (uint8_t)((lo & 0xf) | ((hi & 0xf) << 4));
    }
    return 0;
}

int gemm_unpack_int4_host(const uint8_t *packed, long long N, int K, int8_t *q)
{
    if (!q || !packed || N <= 0 || K <= 0 || K % 2 != 0) return GEMM_FILE_ERR_ARG;
    const size_t n = (size_t)N * K / 2;
    for (size_t i = 0; i < n; i++) {
        const int lo = packed[i] & 0xf, hi = packed[i] >> 4;
        q[2 * i] = (int8_t)(lo >= 8 ? lo - 16 : lo);
        q[2 * i + 1] = (int8_t)(hi >= 8 ? hi - 16 : hi);
    }
    return 0;
}

// e2m1 codes 0..15, one per byte -> two per byte, low nibble = even k
int gemm_pack_fp4_host(const uint8_t *codes, long long N, int K, uint8_t *out)
{
    if (!codes || !out || N <= 0 || K <= 0 || K % 2 != 0) return GEMM_FILE_ERR_ARG;
    const size_t n = (size_t)N * K / 2;
    for (size_t i = 0; i < n; i++) {
        if ((codes[2 * i] | codes[2 * i + 1]) & 0xf0) return GEMM_FILE_ERR_ARG;
        out[i] = (uint8_t)(codes[2 * i] | (codes[2 * i + 1] << 4));
    }
    return 0;
}

int gemm_unpack_fp4_host(const uint8_t *packed, long long N, int K, uint8_t *codes)
{
    if (!codes || !packed || N <= 0 || K <= 0 || K % 2 != 0) return GEMM_FILE_ERR_ARG;
    const size_t n = (size_t)N * K / 2;
    for (size_t i = 0; i < n; i++) {
        codes[2 * i] = packed[i] & 0xf;
        codes[2 * i + 1] = packed[i] >> 4;
    }
    return 0;
}

// row-major ue8m0 scales [rows][K/32] -> the 512-byte atom layout (padding bytes = 127, the scale 1.0)
int gemm_mx_scales_to_tiled_host(const uint8_t *src, long long rows, int K, uint8_t *dst)
{
    if (!src || !dst || rows <= 0 || K <= 0 || K % 32 != 0) return GEMM_FILE_ERR_ARG;
    const int kblocks = K / 32, k_atoms = (kblocks + 3) / 4;
    std::memset(dst, 127, (size_t)((rows + 127) / 128) * k_atoms * 512);
    for (long long r = 0; r < rows; r++)
        for (int kb = 0; kb < kblocks; kb++) dst[tiled_offset(r, kb, k_atoms)] = src[(size_t)r * kblocks + kb];
    return 0;
}

int gemm_mx_scales_from_tiled_host(const uint8_t *src, long long rows, int K, uint8_t *dst)
{
    if (!src || !dst || rows <= 0 || K <= 0 || K % 32 != 0) return GEMM_FILE_ERR_ARG;
    const int kblocks = K / 32, k_atoms = (kblocks + 3) / 4;
    for (long long r = 0; r < rows; r++)
        for (int kb = 0; kb < kblocks; kb++) dst[(size_t)r * kblocks + kb] = src[tiled_offset(r, kb, k_atoms)];
    return 0;
}

int gemm_weight_file_write(const char *path, int dtype, long long N, int K, float tensor_scale, const void *elems, const void *scales)
{
    const size_t eb = gemm_packed_weight_bytes(dtype, N, K), sb = gemm_packed_scale_bytes(dtype, N, K);
    if (!path || eb == 0 || !elems || (sb != 0 && !scales)) return GEMM_FILE_ERR_ARG;
    if ((dtype == GEMM_DT_MXFP8 && K % 128 != 0) || (dtype == GEMM_DT_W4A4 && K % 256 != 0) || (dtype == GEMM_DT_W4A16 && K % 128 != 0) || K % 8 != 0)
        return GEMM_FILE_ERR_ARG;
    GemmWeightFileInfo h;
    std::memset(&h, 0, sizeof(h));
    std::memcpy(h.magic, kMagic, 8);
    h.version = kVersion;
    h.dtype = (uint32_t)dtype;
    h.layout = kLayout;
    h.group = (dtype == GEMM_DT_MXFP8 || dtype == GEMM_DT_W4A4) ? 32u : dtype == GEMM_DT_W4A16 ? 128u : 0u;
    h.N = (uint64_t)N;
    h.K = (uint64_t)K;
    h.elem_bytes = eb;
    h.scale_bytes = sb;
    h.tensor_scale = dtype == GEMM_DT_FP8 ? tensor_scale : 1.0f;
    h.checksum = fnv1a(fnv1a(2166136261u, elems, eb), scales, sb);
    // written under a temporary name and renamed, so a reader never sees half a file
    const std::string tmp = std::string(path) + ".tmp";
    {
        File f(std::fopen(tmp.c_str(), "wb"));
        if (!f) return GEMM_FILE_ERR_IO;
        uint8_t pad[kAlign] = {0};
        std::memcpy(pad, &h, sizeof(h));
        if (std::fwrite(pad, 1, kAlign, f.get()) != kAlign) return GEMM_FILE_ERR_IO;
        if (std::fwrite(elems, 1, eb, f.get()) != eb) return GEMM_FILE_ERR_IO;
        std::memset(pad, 0, kAlign);
        const size_t gap = round_up(eb, kAlign) - eb;
        if (gap && std::fwrite(pad, 1, gap, f.get()) != gap) return GEMM_FILE_ERR_IO;
        if (sb && std::fwrite(scales, 1, sb, f.get()) != sb) return GEMM_FILE_ERR_IO;
        if (std::fflush(f.get()) != 0) return GEMM_FILE_ERR_IO;
    }
    if (std::rename(tmp.c_str(), path) != 0) return GEMM_FILE_ERR_IO;
    return 0;
}

int gemm_weight_file_info(const char *path, GemmWeightFileInfo *out)
{
    if (!path || !out) return GEMM_FILE_ERR_ARG;
    File f(std::fopen(path, "rb"));
    if (!f) return GEMM_FILE_ERR_IO;
    if (std::fread(out, 1, sizeof(*out), f.get()) != sizeof(*out)) return GEMM_FILE_ERR_FORMAT;
    if (std::memcmp(out->magic, kMagic, 8) != 0 || out->version != kVersion || out->layout != kLayout) return GEMM_FILE_ERR_FORMAT;
    if (out->N == 0 || out->K == 0 || out->N > (1ull << 40) || out->K > (1u << 30)) return GEMM_FILE_ERR_FORMAT;
    if (out->elem_bytes != gemm_packed_weight_bytes((int)out->dtype, (long long)out->N, (int)out->K) ||
        out->scale_bytes != gemm_packed_scale_bytes((int)out->dtype, (long long)out->N, (int)out->K) || out->elem_bytes == 0)
        return GEMM_FILE_ERR_FORMAT;
    return 0;
}

// Reads both payloads into caller buffers (pinned host memory is the natural choice) and verifies the checksum.
int gemm_weight_file_read(const char *path, void *elems, size_t elem_capacity, void *scales, size_t scale_capacity)
{
    GemmWeightFileInfo h;
    int rc = gemm_weight_file_info(path, &h);
    if (rc != 0) return rc;
    if (!elems || elem_capacity < h.elem_bytes || (h.scale_bytes && (!scales || scale_capacity < h.scale_bytes))) return GEMM_FILE_ERR_SIZE;
    File f(std::fopen(path, "rb"));
    if (!f) return GEMM_FILE_ERR_IO;
    if (std::fseek(f.get(), (long)kAlign, SEEK_SET) != 0 || std::fread(elems, 1, h.elem_bytes, f.get()) != h.elem_bytes) return GEMM_FILE_ERR_FORMAT;
    if (h.scale_bytes) {
        if (std::fseek(f.get(), (long)(kAlign + round_up(h.elem_bytes, kAlign)), SEEK_SET) != 0 ||
            std::fread(scales, 1, h.scale_bytes, f.get()) != h.scale_bytes)
            return GEMM_FILE_ERR_FORMAT;
    }
    if (fnv1a(fnv1a(2166136261u, elems, h.elem_bytes), scales, h.scale_bytes) != h.checksum) return GEMM_FILE_ERR_CHECKSUM;
    return 0;
}
}
