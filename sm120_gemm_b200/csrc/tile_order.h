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

// stream-K bookkeeping shared by the GEMM kernel and the reduce kernel: `units` (tiles x k-blocks) are cut
// into one contiguous range per CTA (pair) c, [range_begin(c), range_begin(c+1))
TILE_HD long long streamk_range_begin(long long units, int c, int num_clusters)
{
    return units * c / num_clusters;
}
TILE_HD int streamk_owner(long long units, long long u, int num_clusters)
{
    return (int)(((u + 1) * num_clusters - 1) / units);   // the c with range_begin(c) <= u < range_begin(c+1)
}

// Smallest grid that walks `work` items, dealt round-robin, in as few rounds as `max_units` would.
TILE_HD int balanced_units(int work, int max_units)
{
    const int waves = (work + max_units - 1) / max_units;
    return (work + waves - 1) / waves;
}

}  // namespace sm100
