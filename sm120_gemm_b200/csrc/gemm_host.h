// Host-side plumbing shared by every kernel plugin: error reporting without exit(),
// tensor-map encoding through the driver entry point (no link-time libcuda dependency, so
// the plugin still loads on a machine without a driver), a small tensor-map cache, cached
// per-device attributes and the device status block that bounded waits report into.
//
// Replaces the reference's CHECK_CUDA/exit pattern (src/common.h:5-14) and its per-call
// create_tma_desc_2d (src/bf16_gemm.cuh:76-111), which re-encodes every map on every call,
// exits the process on failure and reads the SM count of device 0 whatever device is current
// (src/bf16_gemm.cuh:531).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <stdint.h>

#include "../../include/sm100_gemm.h"

namespace sm100 {

// ---------------------------------------------------------------------------------- errors
struct ErrorState {
    int code = GEMM_OK;
    char msg[256] = {0};
};

inline ErrorState &error_state()
{
    static thread_local ErrorState st;
    return st;
}

inline int set_error(int code, const char *fmt, ...)
{
    ErrorState &st = error_state();
    st.code = code;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(st.msg, sizeof(st.msg), fmt, ap);
    va_end(ap);
    fprintf(stderr, "sm100_gemm: %s\n", st.msg);
    return code;
}

inline void clear_error()
{
    error_state().code = GEMM_OK;
    error_state().msg[0] = 0;
}

#define SM100_CUDA_TRY(call)                                                                          \
    do {                                                                                              \
        cudaError_t e_ = (call);                                                                      \
        if (e_ != cudaSuccess)                                                                        \
            return ::sm100::set_error(GEMM_ERR_CUDA, "%s failed at %s:%d: %s", #call, __FILE__, __LINE__, \
                                      cudaGetErrorString(e_));                                        \
    } while (0)

// ---------------------------------------------------------------------------------- device
struct DeviceInfo {
    std::atomic<bool> ready{false};   // set (release) after every other field; readers load it (acquire) first
    int sm_count = 0;
    int max_smem_optin = 0;
    int cc_major = 0;
    uint32_t *status = nullptr;  // device address of the plugin's status block
    uint32_t *wave_sync = nullptr;        // device address of g_wave_sync
    std::atomic<unsigned> wave_next{0};   // next slot of g_wave_sync to hand to a launch
};

static constexpr int MAX_DEVICES = 32;

// the status block: [0] code, [1] blockIdx.x, [2] detail, [3] spare
__device__ uint32_t g_status_block[4];
// Arrival counters for launches whose clusters pace themselves wave by wave (one word per launch in flight, handed
// out in turn and zeroed on the launch's stream just before the kernel).
static constexpr int WAVE_SYNC_SLOTS = 64;
__device__ uint32_t g_wave_sync[WAVE_SYNC_SLOTS];

inline int device_info(DeviceInfo **out)
{
    static DeviceInfo infos[MAX_DEVICES];
    static std::mutex mu;
    int dev = 0;
    SM100_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) return set_error(GEMM_ERR_ARG, "device ordinal %d out of range", dev);
    DeviceInfo &d = infos[dev];
    if (!d.ready.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(mu);
        if (!d.ready.load(std::memory_order_relaxed)) {
            SM100_CUDA_TRY(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
            SM100_CUDA_TRY(cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
            SM100_CUDA_TRY(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
            if (d.cc_major != 10)
                return set_error(GEMM_ERR_CUDA, "device %d is compute capability %d.x; this library runs on sm_100 only", dev, d.cc_major);
            void *p = nullptr;
            SM100_CUDA_TRY(cudaGetSymbolAddress(&p, g_status_block));
            SM100_CUDA_TRY(cudaMemset(p, 0, sizeof(uint32_t) * 4));
            d.status = static_cast<uint32_t *>(p);
            SM100_CUDA_TRY(cudaGetSymbolAddress(&p, g_wave_sync));
            d.wave_sync = static_cast<uint32_t *>(p);
            d.ready.store(true, std::memory_order_release);
        }
    }
    *out = &d;
    return GEMM_OK;
}

// ---------------------------------------------------------------------------------- tensor maps
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

struct TmapKey {
    const void *ptr;
    uint64_t inner, outer, pitch;
    uint32_t box_inner, box_outer;
    int dtype, swizzle;
    bool operator==(const TmapKey &o) const
    {
        return ptr == o.ptr && inner == o.inner && outer == o.outer && pitch == o.pitch && box_inner == o.box_inner &&
               box_outer == o.box_outer && dtype == o.dtype && swizzle == o.swizzle;
    }
};

// Row-major 2-D tensor (inner = contiguous dimension, in elements; pitch in bytes).
// Out-of-range parts of a box read as zero and are clipped on store, which is what lets the
// kernels take M, N and K that are not multiples of the tile (the reference rejects those,
// src/gemm_config.h:34-38).
inline int make_tmap_2d(CUtensorMap *out, CUtensorMapDataType dtype, const void *ptr, uint64_t inner, uint64_t outer,
                        uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle)
{
    struct Slot {
        TmapKey key;
        CUtensorMap map;
        bool used;
    };
    static thread_local Slot cache[32];
    static thread_local unsigned next = 0;
    TmapKey key{ptr, inner, outer, pitch_bytes, box_inner, box_outer, (int)dtype, (int)swizzle};
    for (auto &s : cache)
        if (s.used && s.key == key) {
            *out = s.map;
            return GEMM_OK;
        }
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return set_error(GEMM_ERR_DRIVER, "cuTensorMapEncodeTiled entry point not available");
    if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0 || (pitch_bytes & 15u) != 0)
        return set_error(GEMM_ERR_ARG, "tensor base %p / pitch %llu bytes must be 16-byte aligned", ptr,
                         (unsigned long long)pitch_bytes);
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, dtype, 2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return set_error(GEMM_ERR_DRIVER, "cuTensorMapEncodeTiled failed (%d) dims=%llux%llu box=%ux%u", (int)r,
                         (unsigned long long)inner, (unsigned long long)outer, box_inner, box_outer);
    Slot &s = cache[next++ % 32];
    s.key = key;
    s.map = *out;
    s.used = true;
    return GEMM_OK;
}

// Row-major 2-D tensor seen as 3-D so that ONE copy brings several 128-byte column chunks of the same rows:
// dimension 0 = the `chunk_elems` elements of a chunk, dimension 1 = rows (pitch bytes apart), dimension 2 = chunks
// along the row (chunk bytes apart).  A box of (chunk_elems, box_rows, box_chunks) lands in shared memory as
// box_chunks consecutive [box_rows][chunk] tiles, each in the canonical 128-byte-swizzled K-major form the MMA
// descriptors expect -- what box_chunks separate 2-D copies would have produced, for one TMA request.
inline int make_tmap_chunked(CUtensorMap *out, CUtensorMapDataType dtype, int elem_bytes, const void *ptr, uint64_t row_elems, uint64_t rows,
                             uint64_t pitch_bytes, uint32_t chunk_elems, uint32_t box_rows, uint32_t box_chunks)
{
    struct Slot {
        const void *ptr;
        uint64_t row_elems, rows, pitch;
        uint32_t chunk, box_rows, box_chunks;
        int dtype;
        CUtensorMap map;
        bool used;
    };
    static thread_local Slot cache[8];
    static thread_local unsigned next = 0;
    for (auto &c : cache)
        if (c.used && c.ptr == ptr && c.row_elems == row_elems && c.rows == rows && c.pitch == pitch_bytes && c.chunk == chunk_elems &&
            c.box_rows == box_rows && c.box_chunks == box_chunks && c.dtype == (int)dtype) {
            *out = c.map;
            return GEMM_OK;
        }
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return set_error(GEMM_ERR_DRIVER, "cuTensorMapEncodeTiled entry point not available");
    if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0 || (pitch_bytes & 15u) != 0)
        return set_error(GEMM_ERR_ARG, "tensor base %p / pitch %llu bytes must be 16-byte aligned", ptr, (unsigned long long)pitch_bytes);
    cuuint64_t dims[3] = {chunk_elems, rows, (row_elems + chunk_elems - 1) / chunk_elems};
    cuuint64_t strides[2] = {pitch_bytes, (cuuint64_t)chunk_elems * elem_bytes};
    cuuint32_t box[3] = {chunk_elems, box_rows, box_chunks};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, dtype, 3, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return set_error(GEMM_ERR_DRIVER, "cuTensorMapEncodeTiled (chunked view) failed (%d) row=%llu rows=%llu box=%ux%ux%u", (int)r,
                         (unsigned long long)row_elems, (unsigned long long)rows, chunk_elems, box_rows, box_chunks);
    Slot &c = cache[next++ % 8];
    c = Slot{ptr, row_elems, rows, pitch_bytes, chunk_elems, box_rows, box_chunks, (int)dtype, *out, true};
    return GEMM_OK;
}

// Reads and clears the device status block of the current device (synchronises the device).
inline int read_device_status(uint32_t out[4])
{
    DeviceInfo *d = nullptr;
    int rc = device_info(&d);
    if (rc != GEMM_OK) return rc;
    SM100_CUDA_TRY(cudaDeviceSynchronize());
    SM100_CUDA_TRY(cudaMemcpy(out, d->status, sizeof(uint32_t) * 4, cudaMemcpyDeviceToHost));
    if (out[0] != 0) {
        SM100_CUDA_TRY(cudaMemset(d->status, 0, sizeof(uint32_t) * 4));
        return set_error(GEMM_ERR_DEVICE_TIMEOUT, "a kernel wait gave up: code %u in block %u (detail %u)", out[0], out[1], out[2]);
    }
    return GEMM_OK;
}

}  // namespace sm100
