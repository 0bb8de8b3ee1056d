// Order in which the (x tile, y tile) pairs of a scoring problem are visited.
//
// The pairs are numbered so that consecutive numbers share the x tile (the kernels keep that tile and its
// accumulators on chip) but only inside a *block* of `yb` consecutive y tiles; all x tiles are taken through one
// block of Y before the next block starts.  CTAs own consecutive number ranges and advance at about the same speed,
// so at any time they read the same few tens of MB of Y, which therefore stays in L2 instead of being streamed from
// DRAM once per x tile.
#pragma once
#include <cuda_runtime.h>

namespace dice {

struct TileMap {
  int nx, ny, yb;   // tiles along x, along y, y tiles per block
  long long full;   // pairs in a full block: nx * yb

  __host__ __device__ static TileMap make(int nx_tiles, int ny_tiles, int tile_bytes, long long l2_budget_bytes) {
    TileMap m;
    m.nx = nx_tiles;
    m.ny = ny_tiles;
    long long yb = l2_budget_bytes / (tile_bytes > 0 ? tile_bytes : 1);
    if (yb < 1) yb = 1;
    if (yb > ny_tiles) yb = ny_tiles;
    m.yb = static_cast<int>(yb);
    m.full = static_cast<long long>(nx_tiles) * m.yb;
    return m;
  }
  __host__ __device__ long long total() const { return static_cast<long long>(nx) * ny; }

  // Pair number w -> x tile, y tile, and how many following pairs (this one included) keep the same x tile.
  __host__ __device__ void locate(long long w, int& x, int& y, int& run) const {
    const long long blk = w / full;
    const long long rem = w - blk * full;
    const int y_first = static_cast<int>(blk) * yb;
    const int ybc = (ny - y_first) < yb ? (ny - y_first) : yb;
    x = static_cast<int>(rem / ybc);
    const int yi = static_cast<int>(rem % ybc);
    y = y_first + yi;
    run = ybc - yi;
  }
};

}  // namespace dice
