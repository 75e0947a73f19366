// How a persistent grid of `clusters` CTA groups divides `tiles` output tiles of `k_blocks` K-blocks each when the tile
// count is not a multiple of the grid: the whole rounds go tile by tile as usual, and the K-blocks of the tiles of the last,
// partial round are spread evenly over the clusters (at most STREAM_MAX_SHARE per tile), so that nobody idles through a
// whole tile's depth.  This is the idea of
// the reference's StreamK schedule (crates/gpurs/src/gpu/tensor/schedule/stream.rs:16-113), which divides the iterations
// of every tile and combines the slices of a tile through a lock that later blocks wait on; here only the last round is
// divided, and a tile whose K-blocks went to several clusters is finished by whichever of them arrives last: nobody waits.
//
// Shared by the host (to size the scratch for the partial tiles) and the kernels (to find their work): plain integer
// arithmetic, the same on both sides.
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define GPURS_HOST_DEVICE __host__ __device__ __forceinline__
#else
#define GPURS_HOST_DEVICE inline
#endif

namespace gemm {

constexpr int STREAM_MAX_SHARE = 4;   // a split tile's K-blocks go to about this many clusters at most

struct StreamSchedule {
    int clusters;      // CTA groups that take part in the split round (the first `clusters` of the grid)
    int k_blocks;      // K-blocks per tile
    int whole_tiles;   // tiles [0, whole_tiles) are multiplied whole, tile t by cluster t % clusters
    int split_tiles;   // tiles [whole_tiles, whole_tiles + split_tiles): their K-blocks are dealt out as units
    long long units;   // split_tiles * k_blocks

    // first unit of cluster c's share; its share is [first_unit(c), first_unit(c + 1))
    GPURS_HOST_DEVICE long long first_unit(int c) const { return units * c / clusters; }

    // the cluster whose share holds unit u (0 <= u < units)
    GPURS_HOST_DEVICE int owner(long long u) const {
        int c = int(u * clusters / units);
        if (c >= clusters) c = clusters - 1;
        while (c + 1 < clusters && first_unit(c + 1) <= u) c++;
        while (c > 0 && first_unit(c) > u) c--;
        return c;
    }

    // clusters that hold K-blocks of split tile r (0-based among the split tiles), and the first of them
    GPURS_HOST_DEVICE int first_contributor(int r) const { return owner((long long)r * k_blocks); }
    GPURS_HOST_DEVICE int contributors(int r) const { return owner((long long)(r + 1) * k_blocks - 1) - first_contributor(r) + 1; }
};

// How many tiles of the last round to split (0 = none): the host's policy.  Splitting needs a whole round before it (a
// product of fewer tiles than clusters gains nothing: every tile already has a cluster to itself) and at least two
// K-blocks.  Unless forced, it must also pay: the idle share of the last round, (clusters - remainder) / clusters of a
// tile's depth, has to outweigh the partial tiles' trip through memory and the adding up, which cost about 30 K-blocks'
// time (measured: f16 4096^3, 34 of 74 left over, 64 blocks deep: +3 %; int8 1024 x 8192 x 8192, 54 of 74 left over: -11 %
// before this rule).
GPURS_HOST_DEVICE int stream_split_tiles(int tiles, int k_blocks, int clusters, bool force) {
    const int remainder = clusters > 0 ? tiles % clusters : 0;
    if (tiles <= clusters || remainder == 0 || k_blocks < 2) return 0;
    if (!force && (long long)(clusters - remainder) * k_blocks < (long long)clusters * 30) return 0;
    return remainder;
}

// The schedule for a grid of `clusters` groups when the last `split_tiles` tiles are split (the kernels get that number
// from the host and derive everything else here).
GPURS_HOST_DEVICE StreamSchedule make_stream_schedule(int tiles, int k_blocks, int clusters, int split_tiles) {
    StreamSchedule s;
    s.clusters = clusters;
    s.k_blocks = k_blocks;
    s.split_tiles = split_tiles;
    s.whole_tiles = tiles - s.split_tiles;
    s.units = (long long)s.split_tiles * k_blocks;
    // Few tiles over many clusters would cut every tile into many thin parts, and whoever adds them up reads them one
    // after the other: no more than STREAM_MAX_SHARE clusters per tile take part (the rest skip the split round).
    if (split_tiles > 0 && s.split_tiles * STREAM_MAX_SHARE < clusters) s.clusters = s.split_tiles * STREAM_MAX_SHARE;
    // Every group that takes part must get at least one unit: a group with an empty share would be counted among a tile's
    // contributors (they are numbered as a contiguous range) and never arrive.
    if (split_tiles > 0 && s.units < s.clusters) s.clusters = int(s.units);
    return s;
}

// The most clusters any split tile is shared by (what the scratch for partial tiles is sized for).
GPURS_HOST_DEVICE int max_contributors(const StreamSchedule &s) {
    int most = 0;
    for (int r = 0; r < s.split_tiles; r++) {
        const int count = s.contributors(r);
        if (count > most) most = count;
    }
    return most;
}

}  // namespace gemm
