// Definitions shared by the two tcgen05 attention kernels (one query tile per CTA, attn_fwd_tc.cu; persistent CTAs,
// attn_fwd_tc_persist.cu): thread roles, TMEM and shared-memory layout, the packed key-tile descriptor.
#pragma once
#include "attn_walk.cuh"
#include "tc_common.cuh"

namespace natsl {

constexpr int TC_THREADS = 320;          // TMA producer, MMA issuer, 8 softmax warps
constexpr uint32_t TC_TMEM_COLS = 256;      // score buffers of 64 columns, then O (DV columns); P_j aliases the buffer of S_j
// Score buffers of 64 columns each, then the output accumulator: two buffers when DV = 128 (2*64 + 128 = 256 columns),
// three when DV = 64 (3*64 + 64): the third one lets Q K^T run one more tile ahead of the softmax.
template <int DV> struct TcTmem {
    static constexpr int NSB = DV == 64 ? 3 : 2;
    static constexpr uint32_t o_col = NSB * 64;
    static constexpr int KST = NSB + 1;              // K ring stages
};
constexpr float LAZY_RESCALE_LOG2 = 8.0f;
constexpr int TC_LIST_CAP = 128;            // key tiles whose descriptors are kept in shared memory
constexpr int TC_VST = 2;                   // V ring stages

template <int DK, int DV>
struct TcSmem {
    static constexpr int q = 0;                                  // DK/64 sub-tiles [128][64]
    static constexpr int KST = TcTmem<DV>::KST;
    static constexpr int k = q + 128 * DK * 2;                   // KST stages x DK/64 sub-tiles [64][64]
    static constexpr int v = k + KST * 64 * DK * 2;              // TC_VST stages x DV/64 sub-tiles [64][64]
    static constexpr int list = v + TC_VST * 64 * DV * 2;        // int[TC_LIST_CAP]
    static constexpr int bars = list + TC_LIST_CAP * 4;
    static constexpr int total = bars + 256;
    static_assert(128 * DV * 2 <= 128 * DK * 2 + KST * 64 * DK * 2, "output staging must fit over Q + K");
    static_assert(total <= 115712, "two CTAs per SM");
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Where the gathered part of the key sequence lives (keys below k_split; see the kernel's comment).
struct RemoteKeys {
    int k_split;          // keys [0, k_split) are gathered keys
    const int* base;      // first pair of (segment g, this head): base[g * stride], or nullptr for the head-major layout
    int stride;
    int slots;            // virtual blocks per head and gathered segment
};

// Packed tile descriptor: bits [0,29) token coordinate of the first key in the tensor it is loaded from (own keys:
// index in k / v; gathered keys: index in k_rem / v_rem), bit 29 gathered, bit 30 masked, bit 31 block selected.
// Masked tiles always lie in the own keys, where coordinate + k_split is the position in the key sequence.
__device__ __forceinline__ int pack_tile(const TileWalk& w, int j, const int* idx, const int* selp, long tstride, int nbs,
                                         const RemoteKeys& rk) {
    bool masked;
    const int s0 = tile_start(w, j, idx, tstride, nbs, masked);
    int sel = 1;
    if (masked) sel = selp[(long)(s0 / nbs) * tstride] != 0;
    int coord = s0 - rk.k_split, rem = 0;
    if (s0 < rk.k_split) {
        rem = 1;
        coord = s0;
        if (rk.base) {
            const int vb = s0 / nbs, g = vb / rk.slots;
            coord = (rk.base[(long)g * rk.stride] + (vb - g * rk.slots)) * nbs + (s0 - vb * nbs);
        }
    }
    return coord | (rem << 29) | (masked ? (1 << 30) : 0) | (sel ? (1 << 31) : 0);
}
constexpr int TILE_COORD_MASK = 0x1FFFFFFF;

}  // namespace natsl
