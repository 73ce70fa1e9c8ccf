// Timing utilities of the bench harness.  The timing PROTOCOL is part of the metric and is
// kept from the reference (src/common.h:21-50): warm-up launches, then `repeat` launches
// each bracketed by its own event pair and followed by an idle spacer kernel, mean of the
// per-launch times.  CUDA failures come back as a negative time instead of exit().
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <vector>

#define CHECK_CUDA(call)                                                                                  \
    do {                                                                                                  \
        cudaError_t e_ = (call);                                                                          \
        if (e_ != cudaSuccess) {                                                                          \
            std::fprintf(stderr, "CUDA error %s at %s:%d: %s\n", #call, __FILE__, __LINE__, cudaGetErrorString(e_)); \
            return -1;                                                                                    \
        }                                                                                                 \
    } while (0)

// idle spacer between timed launches.  The reference launches sleep_kernel<<<1,1>>>(100), which asks __nanosleep for
// 100 * 10^6 ns (src/common.h:16-19, 38); the hardware cuts one __nanosleep short at about a millisecond.  The default
// here asks for the same 10^8 ns.
static __global__ void sleep_kernel(uint32_t us) { __nanosleep(us * 1000u); }

template <class F>
double bench_ms(F &&launch, cudaStream_t stream, uint32_t warmup = 5, uint32_t repeat = 20, uint32_t spacer_us = 100000)
{
    for (uint32_t i = 0; i < warmup; i++) launch();
    CHECK_CUDA(cudaStreamSynchronize(stream));
    std::vector<cudaEvent_t> ev(2 * (size_t)repeat);
    for (auto &e : ev) CHECK_CUDA(cudaEventCreate(&e));
    for (uint32_t i = 0; i < repeat; i++) {
        CHECK_CUDA(cudaEventRecord(ev[2 * i], stream));
        launch();
        CHECK_CUDA(cudaEventRecord(ev[2 * i + 1], stream));
        sleep_kernel<<<1, 1, 0, stream>>>(spacer_us);
    }
    CHECK_CUDA(cudaStreamSynchronize(stream));
    double total = 0;
    for (uint32_t i = 0; i < repeat; i++) {
        float ms = 0;
        CHECK_CUDA(cudaEventElapsedTime(&ms, ev[2 * i], ev[2 * i + 1]));
        total += ms;
    }
    for (auto &e : ev) cudaEventDestroy(e);
    return total / repeat;
}
