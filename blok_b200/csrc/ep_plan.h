// The arithmetic of the expert-parallel exchange plan, shared by the device kernel (ep.cu) and a host entry point
// (blok_ep_plan_host) so that the same code is exercised among CPU ranks.
//
// Input: the count table every rank holds after the all-gather of the histograms: table[s * experts + g] = assignments
// rank s sends to (global) expert g.  Expert g lives on rank g / per.  An owner's receive buffer is ordered by expert,
// then by source rank, then by the source's own order; every rank derives every position from the table alone.
#pragma once

#ifndef __CUDACC__
#define BLOK_HD inline
#else
#define BLOK_HD __host__ __device__ inline
#endif

namespace blok {

// A count that came from another rank is never trusted beyond the buffer: a rank whose wait timed out may have left
// anything in its row.
BLOK_HD int ep_clamped(int c, long cap) {
  if (c < 0) return 0;
  return (long)c > cap ? (int)(cap > 0x3fffffffL ? 0x3fffffffL : cap) : c;
}

// For expert g: assignments from all ranks (tot) and from the ranks below `rank` (before).
template <typename Table>
BLOK_HD void ep_expert_totals(Table table, int world, int experts, int rank, long cap, int g, int *tot, int *before) {
  int t = 0, b = 0;
  for (int s = 0; s < world; ++s) {
    const int c = ep_clamped(table[(long)s * experts + g], cap);
    if (s < rank) b += c;
    t += c;
  }
  *tot = t;
  *before = b;
}

// Owner d: the first row of each of its experts in its receive buffer (exclusive scan of tot, kept inside the buffer).
BLOK_HD void ep_owner_bases(const int *tot, int per, int d, long cap, int *base) {
  long off = 0;
  for (int e = 0; e < per; ++e) {
    const int g = d * per + e;
    base[g] = (int)off;
    off += tot[g];
    if (off > cap) off = cap;
  }
}

// This rank as owner: rows per local expert, their offsets and the tiles (at most `tile` rows of one expert) of its
// grouped GEMM.  Returns the number of tiles; *rows = rows received; *overflow = 1 if more arrived than the buffer holds.
BLOK_HD int ep_owner_tiles(const int *tot, int per, int rank, long cap, int tile, int max_tiles, int *counts, int *offsets,
                           int *tile_expert, int *tile_start, int *tile_count, long *rows, int *overflow) {
  long off = 0;
  int nt = 0;
  *overflow = 0;
  for (int e = 0; e < per; ++e) {
    int c = tot[rank * per + e];
    if (off + c > cap) {
      c = (int)(cap - off);
      *overflow = 1;
    }
    counts[e] = c;
    offsets[e] = (int)off;
    for (int s = 0; s < c && nt < max_tiles; s += tile) {
      tile_expert[nt] = e;
      tile_start[nt] = (int)off + s;
      tile_count[nt] = c - s < tile ? c - s : tile;
      ++nt;
    }
    off += c;
  }
  offsets[per] = (int)off;
  *rows = off;
  return nt;
}

}  // namespace blok
