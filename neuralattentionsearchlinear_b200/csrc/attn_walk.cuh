// Key-tile walk and visibility predicate of the chunk-masked softmax branch, shared by the
// attention kernels and the dense-mask debug kernel so that all of them realise the same mask.
// Key s is visible to query t when   sel[blk(s)] && t >= (blk(s)+1)*nbs   ||   blk(s)==blk(t) && s <= t
// (src/nats/ops/attns/attns.py:2041-2058).  A 128-query tile visits
//   1. the own span [start of the block holding the tile's first row, end of the tile), masked per element -- first,
//      because where these tiles lie follows from the query tile alone, so their loads can start before any table is read;
//   2. the first n_past selected blocks (index table, unmasked; n_past = attn_n_iters table,
//      src/nats/ops/nats_util.py:67-121).
// (The reference walks the past blocks first; the online softmax does not depend on the order.)
#pragma once
#include "common.cuh"

namespace natsl {

constexpr int ATT_BM = 128;
constexpr int ATT_BN = 64;

struct TileWalk {
    int n_past_tiles;   // unmasked tiles from selected past blocks
    int n_span;         // masked tiles of the own span (tiles 0 .. n_span-1)
    int n_tiles;        // total
    int span_start;     // first key of the own span
    int cpb;            // 64-key tiles per selection block
};

__device__ __forceinline__ TileWalk make_walk(int q0, int T, int nbs, int n_past_blocks) {
    TileWalk w;
    w.cpb = nbs / ATT_BN;
    w.n_past_tiles = n_past_blocks * w.cpb;
    w.span_start = (q0 / nbs) * nbs;
    int span_end = min(q0 + ATT_BM, T);
    w.n_span = (span_end - w.span_start + ATT_BN - 1) / ATT_BN;
    w.n_tiles = w.n_past_tiles + w.n_span;
    return w;
}

// first key of tile j and whether the tile needs the per-element mask
__device__ __forceinline__ int tile_start(const TileWalk& w, int j, const int* idx, long idx_stride, int nbs,
                                          bool& masked) {
    if (j < w.n_span) {
        masked = true;
        return w.span_start + j * ATT_BN;
    }
    masked = false;
    const int jp = j - w.n_span;
    return idx[(long)(jp / w.cpb) * idx_stride] * nbs + (jp % w.cpb) * ATT_BN;
}

__device__ __forceinline__ bool visible(int t, int s, int T, int blk_end, bool selb, bool own_chunk) {
    if (s >= T) return false;
    if (own_chunk) return s <= t && (selb || t < blk_end);
    return selb && t >= blk_end;
}

}  // namespace natsl
