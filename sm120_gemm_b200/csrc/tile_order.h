// Order in which a persistent grid walks the output tiles.  Plain C++ (host and device).
#pragma once

#if defined(__CUDACC__)
#define TILE_HD __host__ __device__ __forceinline__
#else
#define TILE_HD inline
#endif

namespace sm100 {

// Bands of `group_n` tile columns, walked row by row inside a band, so the CTAs running at
// one time cover a compact block of Y and share X and W tiles through L2.  A bijection from
// [0, num_m*num_n) onto the tile grid; the last band may be narrower.
// (Same purpose as the reference's rasterize_tile, src/bf16_gemm.cuh:225-237.)
TILE_HD void tile_to_mn(int tile, int num_m, int num_n, int group_n, int &mb, int &nb)
{
    const int per_band = group_n * num_m;
    const int band = tile / per_band;
    const int rem = tile - band * per_band;
    const int n_first = band * group_n;
    const int width = num_n - n_first < group_n ? num_n - n_first : group_n;
    mb = rem / width;
    nb = n_first + (rem - mb * width);
}

}  // namespace sm100
