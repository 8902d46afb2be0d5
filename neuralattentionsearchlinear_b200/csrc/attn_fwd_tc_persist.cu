// Chunk-masked softmax attention forward on the 5th-generation tensor cores, persistent form: two CTAs per SM stay
// resident and work through the (query tile, head, batch) items, heaviest query tiles first, so that the query load,
// the table walk and the first Q K^T of the next item run under the tail of the current one and no CTA launch,
// barrier set-up or TMEM allocation sits between two items.
// Roles, rings, TMEM layout, masks and numerics are those of attn_fwd_tc.cu (the one-item-per-CTA kernel it replaces by
// default); the differences:
//   * every ring / score-buffer / product barrier is indexed by a tile counter that runs across items;
//   * the producer loads K of tile g and V of tile g - NSB in one sequence over all items (the order in which the tensor
//     core frees the stages), the query tile of the next item as soon as the last Q K^T of the current one has completed
//     (barrier q_empty);
//   * the MMA issuer keeps the Q K^T stream up to NSB tiles ahead of the P V stream, across item boundaries; the first
//     P V of an item waits until the softmax warps have read the previous output out of TMEM (barrier o_free);
//   * the output rows go from registers straight to global memory (no staging over the query tile, which already
//     belongs to the next item by then); the key-tile descriptors live in the producer's registers, the softmax warps
//     derive the masked tiles' positions arithmetically.
// src/nats/ops/attns/attns.py:62-353 is the reference kernel this replaces.
// Every mbarrier wait has an iteration limit; on expiry the CTA records a status, stops issuing work, still frees its
// TMEM and returns.
#include "attn_tc.cuh"
#include "../../include/natsl_b200.h"
#ifdef NATSL_ATTN_TIMING
#include <cstdlib>
#endif

namespace natsl {

struct PsArgs {
    int k_split, B_rem;
    const int* rem_base;
    int rem_slots;
    const int* types_i;
    const int* indices;
    const int* attn_n_iters;
    __nv_bfloat16* o;
    float* lse;
    int B, T, Tq, q_off, HQ, HKV, HN, TN, nbs;
    float scale_log2;
    int own_chunk;
    int NTq;              // query tiles of this call
    int n_items;          // NTq * HQ * B
    int* status;
};

#ifdef NATSL_ATTN_TIMING
// scratch builds only: per CTA, cycles softmax warp 2 spent waiting for score tiles, for the item's last products, in the
// output phase, in total, and the numbers of items and tiles
__device__ long long* g_attn_ts = nullptr;
#define AT_T0() const long long at_t0 = clock64()
#define AT_ADD(slot) do { if (at_on) at_acc[slot] += clock64() - at_t0; } while (0)
#else
#define AT_T0()
#define AT_ADD(slot)
#endif

struct PsItem {
    int it, hq, b, hkv, hn, q0;
};

// item w -> (query tile, head, batch): the heaviest query tiles (the last ones) of every (head, batch) come first
__device__ __forceinline__ PsItem ps_decode(int w, const PsArgs& a) {
    const int per = a.HQ * a.B;
    const int itr = w / per, rem = w - itr * per;
    PsItem x;
    x.b = rem / a.HQ;
    x.hq = rem - x.b * a.HQ;
    x.it = a.q_off / ATT_BM + (a.NTq - 1 - itr);
    x.hkv = x.hq / (a.HQ / a.HKV);
    x.hn = x.hq / (a.HQ / a.HN);
    x.q0 = x.it * ATT_BM;
    return x;
}
__device__ __forceinline__ int ps_n_past(const PsItem& x, const PsArgs& a) {
    const int NTq_all = (a.T + ATT_BM - 1) / ATT_BM;
    return a.attn_n_iters[((long)x.b * NTq_all + x.it) * a.HN + x.hn];
}

// What the producer knows about the item one of its two load streams is in.  The table entries of the item after it
// are requested one item ahead and kept as loaded (nothing is computed from them until the cursor moves on), so that
// entering an item costs no memory round trip: a warp stalls at the first instruction that consumes a pending load.
struct PsCtx {
    PsItem x;
    int n_tiles, b_rem;
    int td[4];            // key-tile descriptors of tiles lane, lane + 32, lane + 64, lane + 96 (selection bit unused)
    TileWalk walk;
    const int* idx;
    const int* selp;
    RemoteKeys rk;
};
struct PsCursor {
    int item, j;
    bool active;
    PsCtx cur;
    int nxt_n_past;       // attn_n_iters entry of the next item, as loaded
    int nxt_blk[4];       // index-table entries of this lane's tiles of the next item, read as if all were past tiles
};

// request the table entries of the item after the current one
__device__ __forceinline__ void ps_peek(PsCursor& c, int G, const PsArgs& a, int lane) {
    const int item = c.item + G;
    if (item >= a.n_items) return;
    const PsItem y = ps_decode(item, a);
    c.nxt_n_past = ps_n_past(y, a);
    const int* idx = a.indices + ((long)y.b * a.TN * a.HN + y.hn) * 2;
    const int cpb = a.nbs / ATT_BN;
    const int n_span = make_walk(y.q0, a.T, a.nbs, 0).n_span;        // the own span comes first and needs no table
#pragma unroll
    for (int r = 0; r < 4; ++r)
        c.nxt_blk[r] = idx[(long)min(max(lane + 32 * r - n_span, 0) / cpb, a.TN - 1) * a.HN * 2];
}
// move to the next item: everything is computed from the entries requested by ps_peek
__device__ __forceinline__ void ps_next(PsCursor& c, int G, const PsArgs& a, int lane) {
    c.item += G;
    c.j = 0;
    c.active = c.item < a.n_items;
    if (!c.active) return;
    PsCtx& x = c.cur;
    x.x = ps_decode(c.item, a);
    x.walk = make_walk(x.x.q0, a.T, a.nbs, c.nxt_n_past);
    x.n_tiles = x.walk.n_tiles;
    x.idx = a.indices + ((long)x.x.b * a.TN * a.HN + x.x.hn) * 2;
    x.selp = a.types_i + ((long)x.x.b * a.TN * a.HN + x.x.hn) * 2;
    x.b_rem = x.x.b % a.B_rem;
    x.rk.k_split = a.k_split;
    x.rk.slots = a.rem_slots;
    x.rk.stride = a.HKV;
    x.rk.base = a.rem_base ? a.rem_base + ((long)x.b_rem * (a.k_split / (a.rem_slots * a.nbs))) * a.HKV + x.x.hkv : nullptr;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int j = lane + 32 * r;
        const bool past = j >= x.walk.n_span;
        const int s0 = past ? c.nxt_blk[r] * a.nbs + ((j - x.walk.n_span) % x.walk.cpb) * ATT_BN : x.walk.span_start + j * ATT_BN;
        int coord = s0 - a.k_split, rem = 0;
        if (j < x.n_tiles && s0 < a.k_split) {
            rem = 1;
            coord = s0;
            if (x.rk.base) {                              // packed gathered keys: one more table (sequence parallelism)
                const int vb = s0 / a.nbs, g = vb / x.rk.slots;
                coord = (x.rk.base[(long)g * x.rk.stride] + (vb - g * x.rk.slots)) * a.nbs + (s0 - vb * a.nbs);
            }
        }
        x.td[r] = coord | (rem << 29) | (past ? 0 : (1 << 30));
    }
    ps_peek(c, G, a, lane);
}
__device__ __forceinline__ void ps_start(PsCursor& c, int item, int G, const PsArgs& a, int lane) {
    c.item = item - G;
    ps_peek(c, G, a, lane);
    ps_next(c, G, a, lane);
}
// descriptor of tile j of the cursor's item (all lanes call; all lanes get it)
__device__ __forceinline__ int ps_tile(const PsCursor& c, int j, const PsArgs& a) {
    if (j >= 128) return pack_tile(c.cur.walk, j, c.cur.idx, c.cur.selp, (long)a.HN * 2, a.nbs, c.cur.rk);
    const int r = j >> 5;
    const int v = r == 0 ? c.cur.td[0] : (r == 1 ? c.cur.td[1] : (r == 2 ? c.cur.td[2] : c.cur.td[3]));
    return __shfl_sync(0xffffffffu, v, j & 31);
}

template <int DK, int DV>
__global__ void __launch_bounds__(TC_THREADS, 2)
attn_fwd_tc_persist_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                           const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_kr,
                           const __grid_constant__ CUtensorMap map_vr, const PsArgs a) {
    using L = TcSmem<DK, DV>;
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t sbase = smem_u32(smem);
    int* status = a.status;
    if ((sbase & 1023u) != 0) {                       // swizzled tiles need 1024-byte alignment
        if (tid == 0) atomicExch(status, 2);
        return;
    }
    const int G = gridDim.x;
    const uint32_t s_q = sbase + L::q, s_k = sbase + L::k, s_v = sbase + L::v;
    // barrier slots (8 bytes each), placed over the tile list of the one-item kernel
    const uint32_t bar0 = sbase + L::list;
    const uint32_t bar_q_full = bar0, bar_q_empty = bar0 + 8, bar_o_free = bar0 + 16, bar_pv = bar0 + 24,
                   bar_k_full = bar0 + 40, bar_k_empty = bar0 + 72, bar_v_full = bar0 + 104, bar_v_empty = bar0 + 136,
                   bar_s_full = bar0 + 168, bar_p_full = bar0 + 192;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::list + 224);
    constexpr int NSB = TcTmem<DV>::NSB, TC_KST = TcTmem<DV>::KST;
    constexpr uint32_t TC_O_COL = TcTmem<DV>::o_col;

    if (tid == 0) {
        mbar_init(bar_q_full, 1);
        mbar_init(bar_q_empty, 1);
        mbar_init(bar_o_free, 8);                        // one arrival per softmax warp
        mbar_init(bar_pv, 1);
        mbar_init(bar_pv + 8, 1);
        for (int i = 0; i < 4; ++i) {
            mbar_init(bar_k_full + 8 * i, 1);
            mbar_init(bar_k_empty + 8 * i, 1);
            mbar_init(bar_v_full + 8 * i, 1);
            mbar_init(bar_v_empty + 8 * i, 1);
        }
        for (int i = 0; i < NSB; ++i) {
            mbar_init(bar_s_full + 8 * i, 1);
            mbar_init(bar_p_full + 8 * i, 8);
        }
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TC_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            prefetch_tensormap(&map_q);
            prefetch_tensormap(&map_k);
            prefetch_tensormap(&map_v);
            if (a.k_split > 0) {
                prefetch_tensormap(&map_kr);
                prefetch_tensormap(&map_vr);
            }
        }
#ifdef NATSL_ATTN_TIMING
        const bool at_on = g_attn_ts && lane == 0;
        long long at_acc[6] = {0, 0, 0, 0, 0, 0};
        const long long at_start = clock64();
#endif
        PsCursor ck, cv;
        {
            AT_T0();
            ps_start(ck, blockIdx.x, G, a, lane);
            ps_start(cv, blockIdx.x, G, a, lane);
            AT_ADD(3);
        }
        int gk = 0, gv = 0, items_k = 0;
        bool ok = true;
        while (ok && (ck.active || cv.active)) {
            if (ck.active) {
                if (ck.j == 0) {
                    // the query tile of a new item: its place is free once the last Q K^T of the previous item is done
                    AT_T0();
                    if (items_k > 0) ok = __all_sync(0xffffffffu, mbar_wait(bar_q_empty, (items_k - 1) & 1, status));
                    AT_ADD(0);
                    if (ok && lane == 0) {
                        mbar_expect_tx(bar_q_full, 128 * DK * 2);
#pragma unroll
                        for (int sub = 0; sub < DK / 64; ++sub)
                            tma_load_4d(s_q + sub * 16384, &map_q, sub * 64, ck.cur.x.hq, ck.cur.x.q0 - a.q_off, ck.cur.x.b, bar_q_full);
                    }
                    ++items_k;
                }
                const int td = ps_tile(ck, ck.j, a);
                const int stg = gk % TC_KST;
                {
                    AT_T0();
                    if (ok && gk >= TC_KST)
                        ok = __all_sync(0xffffffffu, mbar_wait(bar_k_empty + stg * 8, ((gk / TC_KST) - 1) & 1, status));
                    AT_ADD(1);
                }
                if (ok && lane == 0) {
                    const bool rem = (td >> 29) & 1;
                    const int hh = rem ? (a.rem_base ? 0 : ck.cur.x.hkv) : ck.cur.x.hkv, bb = rem ? ck.cur.b_rem : ck.cur.x.b;
                    const uint32_t full = bar_k_full + stg * 8;
                    mbar_expect_tx(full, 64 * DK * 2);
#pragma unroll
                    for (int sub = 0; sub < DK / 64; ++sub)
                        tma_load_4d(s_k + stg * (64 * DK * 2) + sub * 8192, rem ? &map_kr : &map_k, sub * 64, hh,
                                    td & TILE_COORD_MASK, bb, full);
                    // warm L2 for the value tile that follows NSB loads later
#pragma unroll
                    for (int sub = 0; sub < DV / 64; ++sub)
                        tma_prefetch_4d(rem ? &map_vr : &map_v, sub * 64, hh, td & TILE_COORD_MASK, bb);
                }
                ++gk;
                {
                    AT_T0();
                    if (++ck.j == ck.cur.n_tiles) ps_next(ck, G, a, lane);
                    AT_ADD(3);
                }
            }
            if (ok && cv.active && (!ck.active || gv + NSB < gk)) {
                const int td = ps_tile(cv, cv.j, a);
                const int stg = gv % TC_VST;
                {
                    AT_T0();
                    if (gv >= TC_VST)
                        ok = __all_sync(0xffffffffu, mbar_wait(bar_v_empty + stg * 8, ((gv / TC_VST) - 1) & 1, status));
                    AT_ADD(2);
                }
                if (ok && lane == 0) {
                    const bool rem = (td >> 29) & 1;
                    const int hh = rem ? (a.rem_base ? 0 : cv.cur.x.hkv) : cv.cur.x.hkv, bb = rem ? cv.cur.b_rem : cv.cur.x.b;
                    const uint32_t full = bar_v_full + stg * 8;
                    mbar_expect_tx(full, 64 * DV * 2);
#pragma unroll
                    for (int sub = 0; sub < DV / 64; ++sub)
                        tma_load_4d(s_v + stg * (64 * DV * 2) + sub * 8192, rem ? &map_vr : &map_v, sub * 64, hh,
                                    td & TILE_COORD_MASK, bb, full);
                }
                ++gv;
                {
                    AT_T0();
                    if (++cv.j == cv.cur.n_tiles) ps_next(cv, G, a, lane);
                    AT_ADD(4);
                }
            }
            __syncwarp();
        }
#ifdef NATSL_ATTN_TIMING
        if (at_on) {
            at_acc[5] = clock64() - at_start;
            for (int i = 0; i < 6; ++i) g_attn_ts[blockIdx.x * 18 + 12 + i] = at_acc[i];
        }
#endif
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 64, false);
        constexpr uint32_t idesc_pv = umma_idesc_bf16(128, DV, true);
        // attn_n_iters entry of an item, as loaded; the tile count is computed from it only when the cursor gets there
        auto raw_of = [&](int item) -> int { return item < a.n_items ? ps_n_past(ps_decode(item, a), a) : 0; };
        auto tiles_of = [&](int item, int raw) -> int {
            return item < a.n_items ? make_walk(ps_decode(item, a).q0, a.T, a.nbs, raw).n_tiles : 0;
        };
        // two cursors over the same item sequence: Q K^T runs up to NSB tiles ahead of P V
        int item_q = blockIdx.x, jq = 0, nq = tiles_of(item_q, raw_of(item_q)), raw_q = raw_of(item_q + G), items_q = 0;
        int item_p = blockIdx.x, jp = 0, np = nq, raw_p = raw_of(item_p + G), items_p = 0;
        int gq = 0, gp = 0;
        bool q_active = item_q < a.n_items, p_active = q_active;
        bool ok = true;
#ifdef NATSL_ATTN_TIMING
        const bool at_on = g_attn_ts && lane == 0;
        long long at_acc[6] = {0, 0, 0, 0, 0, 0};
        const long long at_start = clock64();
#endif
        while (ok && p_active) {
            while (ok && q_active && gq < gp + NSB) {
                if (jq == 0) {
                    // a new item's first Q K^T needs its query tile; while P V work of the current item may be pending
                    // (gq > gp) do not sleep on it
                    if (gq > gp && !__all_sync(0xffffffffu, mbar_test_wait(bar_q_full, items_q & 1))) break;
                    AT_T0();
                    ok = __all_sync(0xffffffffu, mbar_wait(bar_q_full, items_q & 1, status));
                    AT_ADD(0);
                    if (!ok) break;
                }
                const int sb = gq % NSB, stg = gq % TC_KST;
                {
                    AT_T0();
                    ok = __all_sync(0xffffffffu, mbar_wait(bar_k_full + stg * 8, (gq / TC_KST) & 1, status));
                    AT_ADD(1);
                }
                if (!ok) break;
                AT_T0();
                if (lane == 0) {
                    tc_fence_after();
                    const uint32_t kt = s_k + stg * (64 * DK * 2);
#pragma unroll
                    for (int kk = 0; kk < DK / 16; ++kk) {
                        const uint64_t ad = umma_desc(s_q + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
                        const uint64_t bd = umma_desc(kt + (kk >> 2) * 8192 + (kk & 3) * 32, 16, 1024);
                        umma_ss(tmem + sb * 64, ad, bd, idesc_qk, kk > 0);
                    }
                    umma_commit(bar_s_full + sb * 8);
                    umma_commit(bar_k_empty + stg * 8);
                    if (jq == nq - 1) umma_commit(bar_q_empty);
                }
                __syncwarp();
                AT_ADD(4);
                ++gq;
                if (++jq == nq) {
                    item_q += G;
                    jq = 0;
                    ++items_q;
                    q_active = item_q < a.n_items;
                    nq = tiles_of(item_q, raw_q);
                    raw_q = raw_of(item_q + G);
                }
            }
            if (!ok) break;
            const int sb = gp % NSB, vstg = gp % TC_VST;
            {
                AT_T0();
                ok = __all_sync(0xffffffffu, mbar_wait(bar_v_full + vstg * 8, (gp / TC_VST) & 1, status));
                AT_ADD(2);
            }
            {
                AT_T0();
                if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_p_full + sb * 8, (gp / NSB) & 1, status));
                AT_ADD(3);
            }
            {
                AT_T0();
                if (ok && jp == 0 && items_p > 0)             // the previous output has left TMEM
                    ok = __all_sync(0xffffffffu, mbar_wait(bar_o_free, (items_p - 1) & 1, status));
                AT_ADD(0);
            }
            if (!ok) break;
            if (lane == 0) {
                tc_fence_after();
                const uint32_t vt = s_v + vstg * (64 * DV * 2);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint64_t bd = umma_desc(vt + kk * 2048, 8192, 1024);
                    umma_ts(tmem + TC_O_COL, tmem + sb * 64 + kk * 8, bd, idesc_pv, (jp > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(bar_v_empty + vstg * 8);
                umma_commit(bar_pv + (gp & 1) * 8);
            }
            __syncwarp();
            ++gp;
            if (++jp == np) {
                item_p += G;
                jp = 0;
                ++items_p;
                p_active = item_p < a.n_items;
                np = tiles_of(item_p, raw_p);
                raw_p = raw_of(item_p + G);
            }
        }
#ifdef NATSL_ATTN_TIMING
        if (at_on) {
            at_acc[5] = clock64() - at_start;
            for (int i = 0; i < 6; ++i) g_attn_ts[blockIdx.x * 18 + 6 + i] = at_acc[i];
        }
#endif
    } else {
        // ------------------------------------------------------------ softmax + output (8 warps)
        // Warp (quad, half) owns the 16 query rows quad*32 + half*16 ... of the tile (a warp reaches only its own
        // quarter of the TMEM lanes).  In the 16x256b layout a thread holds, of rows ra and ra + 8, the columns
        // 8k + 2(lane%4), +1 for k = 0..7: 32 scores; the four threads of a row meet through two shuffles.
        const int quad = warp & 3, half = (warp - 2) >> 2;
        const int r_a = quad * 32 + half * 16 + (lane >> 2), r_b = r_a + 8;
        const int cq = (lane & 3) * 2;
        const uint32_t t_rows = tmem + ((uint32_t)(quad * 32 + half * 16) << 16);
        const uint32_t t_o = t_rows + TC_O_COL;
        const long tstride = (long)a.HN * 2;
        const int T = a.T, nbs = a.nbs, own_chunk = a.own_chunk;
        const float scale_log2 = a.scale_log2;
        bool ok = true;
        int g = 0;                                        // tile counter across items
#ifdef NATSL_ATTN_TIMING
        const bool at_on = g_attn_ts && warp == 2 && lane == 0;
        long long at_acc[6] = {0, 0, 0, 0, 0, 0};
        const long long at_start = clock64();
#endif
        // selection bit of the block own-span tile `lane` of an item lies in (an item has at most (nbs + 128) / 64 such
        // tiles; their positions depend on the query tile only)
        auto span_sel = [&](const PsItem& y) -> int {       // the table entry as loaded (compared when it is used)
            const int s0 = (y.q0 / nbs) * nbs + lane * ATT_BN;
            if (s0 >= min(y.q0 + ATT_BM, T)) return 0;
            return a.types_i[((long)y.b * a.TN * a.HN + y.hn) * 2 + (long)(s0 / nbs) * tstride];
        };
        // both table reads of an item are issued one item ahead
        int n_past_next = 0, selb_next = 0;
        if (blockIdx.x < a.n_items) {
            const PsItem y = ps_decode(blockIdx.x, a);
            n_past_next = ps_n_past(y, a);
            selb_next = span_sel(y);
        }
        for (int item = blockIdx.x; ok && item < a.n_items; item += G) {
            const PsItem x = ps_decode(item, a);
            const TileWalk walk = make_walk(x.q0, T, nbs, n_past_next);
            const unsigned sel_mask = __ballot_sync(0xffffffffu, selb_next != 0);
            if (item + G < a.n_items) {
                const PsItem y = ps_decode(item + G, a);
                n_past_next = ps_n_past(y, a);
                selb_next = span_sel(y);
            }
            const int n_tiles = walk.n_tiles;
            const int t_a = x.q0 + r_a, t_b = x.q0 + r_b;
            float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
            for (int j = 0; j < n_tiles; ++j, ++g) {
                const int sb = g % NSB;
                const uint32_t t_s = t_rows + sb * 64;
                {
                    AT_T0();
                    ok = __all_sync(0xffffffffu, mbar_wait(bar_s_full + sb * 8, (g / NSB) & 1, status));
                    AT_ADD(0);
                }
                if (!ok) break;
                tc_fence_after();
                uint32_t sr[32];
                tmem_ld_16x256b_x8(t_s, sr);
                tmem_ld_wait();
                if (j < walk.n_span) {
                    // own-span tile: per row the visible keys are columns [0, limit] (attn_walk.cuh: visible())
                    const int ms = j;
                    const int s0 = walk.span_start + ms * ATT_BN;
                    const bool selb = (sel_mask >> ms) & 1;
                    const int blk_end = (s0 / nbs + 1) * nbs;
                    int lim_a = T - 1 - s0, lim_b = lim_a;
                    if (own_chunk) {
                        lim_a = min(lim_a, t_a - s0);
                        lim_b = min(lim_b, t_b - s0);
                        if (!(selb || t_a < blk_end)) lim_a = -1;
                        if (!(selb || t_b < blk_end)) lim_b = -1;
                    } else {
                        if (!(selb && t_a >= blk_end)) lim_a = -1;
                        if (!(selb && t_b >= blk_end)) lim_b = -1;
                    }
#pragma unroll
                    for (int k = 0; k < 8; ++k)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int c = 8 * k + cq + e;
                            sr[4 * k + e] = (c <= lim_a) ? sr[4 * k + e] : 0xff800000u;          // -inf
                            sr[4 * k + 2 + e] = (c <= lim_b) ? sr[4 * k + 2 + e] : 0xff800000u;
                        }
                }
                // row maxima of the raw scores (scale > 0, so max(scale * s) = scale * max(s))
                float xa0 = -INFINITY, xa1 = -INFINITY, xb0 = -INFINITY, xb1 = -INFINITY;
#pragma unroll
                for (int k = 0; k < 8; k += 2) {
                    xa0 = fmax3(xa0, __uint_as_float(sr[4 * k]), __uint_as_float(sr[4 * k + 1]));
                    xb0 = fmax3(xb0, __uint_as_float(sr[4 * k + 2]), __uint_as_float(sr[4 * k + 3]));
                    xa1 = fmax3(xa1, __uint_as_float(sr[4 * k + 4]), __uint_as_float(sr[4 * k + 5]));
                    xb1 = fmax3(xb1, __uint_as_float(sr[4 * k + 6]), __uint_as_float(sr[4 * k + 7]));
                }
                float xa = fmaxf(xa0, xa1), xb = fmaxf(xb0, xb1);
                xa = fmaxf(xa, __shfl_xor_sync(0xffffffffu, xa, 1));
                xb = fmaxf(xb, __shfl_xor_sync(0xffffffffu, xb, 1));
                xa = fmaxf(xa, __shfl_xor_sync(0xffffffffu, xa, 2));
                xb = fmaxf(xb, __shfl_xor_sync(0xffffffffu, xb, 2));
                const float mx_a = xa * scale_log2, mx_b = xb * scale_log2;
                const bool need_a = mx_a > m_a + LAZY_RESCALE_LOG2, need_b = mx_b > m_b + LAZY_RESCALE_LOG2;
                if (__any_sync(0xffffffffu, need_a || need_b)) {
                    const float new_a = need_a ? mx_a : m_a, new_b = need_b ? mx_b : m_b;
                    const float alpha_a = (new_a == -INFINITY) ? 1.f : ex2(m_a - new_a);
                    const float alpha_b = (new_b == -INFINITY) ? 1.f : ex2(m_b - new_b);
                    if (j > 0) {
                        // O must be at rest: P V of the previous tile has to be complete.  Even and odd tiles signal on
                        // two barriers; the score tile in hand was produced behind P V of tile g - NSB >= g - 3 (the
                        // previous phase of the barrier waited on), and P V of tile g + 1 cannot have started, so the
                        // barrier is in the phase waited for or the one after it: the parity wait is unambiguous.
                        ok = __all_sync(0xffffffffu, mbar_wait(bar_pv + ((g - 1) & 1) * 8, ((g - 1) >> 1) & 1, status));
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll 1
                        for (int c0 = 0; c0 < DV; c0 += 64) {
                            uint32_t orr[32];
                            tmem_ld_16x256b_x8(t_o + c0, orr);
                            tmem_ld_wait();
#pragma unroll
                            for (int k = 0; k < 8; ++k) {
                                orr[4 * k] = __float_as_uint(__uint_as_float(orr[4 * k]) * alpha_a);
                                orr[4 * k + 1] = __float_as_uint(__uint_as_float(orr[4 * k + 1]) * alpha_a);
                                orr[4 * k + 2] = __float_as_uint(__uint_as_float(orr[4 * k + 2]) * alpha_b);
                                orr[4 * k + 3] = __float_as_uint(__uint_as_float(orr[4 * k + 3]) * alpha_b);
                            }
                            tmem_st_16x256b_x8(t_o + c0, orr);
                        }
                    }
                    l_a *= alpha_a;
                    l_b *= alpha_b;
                    m_a = new_a;
                    m_b = new_b;
                }
                const float neg_a = (m_a == -INFINITY) ? 0.f : -m_a, neg_b = (m_b == -INFINITY) ? 0.f : -m_b;
                float la2 = 0.f, lb2 = 0.f;
                uint32_t pr[16];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float p0 = ex2(fmaf(__uint_as_float(sr[4 * k]), scale_log2, neg_a));
                    const float p1 = ex2(fmaf(__uint_as_float(sr[4 * k + 1]), scale_log2, neg_a));
                    const float p2 = ex2(fmaf(__uint_as_float(sr[4 * k + 2]), scale_log2, neg_b));
                    const float p3 = ex2(fmaf(__uint_as_float(sr[4 * k + 3]), scale_log2, neg_b));
                    if (k & 1) {
                        la2 += p0 + p1;
                        lb2 += p2 + p3;
                    } else {
                        l_a += p0 + p1;
                        l_b += p2 + p3;
                    }
                    pr[2 * k] = pack_bf16(p0, p1);                // P column 4k + lane%4 of row a
                    pr[2 * k + 1] = pack_bf16(p2, p3);            // ... of row b
                }
                l_a += la2;
                l_b += lb2;
                tmem_st_16x128b_x8(t_s, pr);                      // P over the first 32 columns of the score buffer
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_p_full + sb * 8);
            }
            if (!ok) break;
            // The item's last two products, in order (g is one past the last tile): once the one of tile g - 2 is
            // complete so is that of tile g - 3, the previous phase of the barrier of tile g - 1.
            {
                AT_T0();
                if (n_tiles >= 2)
                    ok = __all_sync(0xffffffffu, mbar_wait(bar_pv + ((g - 2) & 1) * 8, ((g - 2) >> 1) & 1, status));
                if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_pv + ((g - 1) & 1) * 8, ((g - 1) >> 1) & 1, status));
                AT_ADD(1);
            }
            if (!ok) break;
            AT_T0();
            tc_fence_after();
            l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
            l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
            l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
            l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
            const bool has_a = l_a > 0.f, has_b = l_b > 0.f;
            const float inv_a = has_a ? 1.f / l_a : 0.f, inv_b = has_b ? 1.f / l_b : 0.f;
            const int qa = t_a - a.q_off, qb = t_b - a.q_off;         // query index inside this call
            // A thread holds, per group of eight columns k, the pair 8k + 2(lane%4), +1.  Neighbouring lanes swap every
            // other pair, so that each holds four consecutive columns of half the groups: 8-byte stores, and the four
            // lanes of a row fill one 32-byte sector per instruction.
            const bool odd = lane & 1;
            const int c4 = (lane & 2) * 2;                            // 0 or 4: this lane pair's columns inside a group
            __nv_bfloat16* oa = a.o + (((long)x.b * a.Tq + qa) * a.HQ + x.hq) * DV + c4 + (odd ? 8 : 0);
            __nv_bfloat16* ob = a.o + (((long)x.b * a.Tq + qb) * a.HQ + x.hq) * DV + c4 + (odd ? 8 : 0);
#pragma unroll 1
            for (int c0 = 0; c0 < DV; c0 += 64) {
                uint32_t orr[32];
                tmem_ld_16x256b_x8(t_o + c0, orr);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    // groups k = 2i (kept by the even lane) and k = 2i + 1 (kept by the odd lane)
                    const uint32_t a0 = pack_bf16(__uint_as_float(orr[8 * i]) * inv_a, __uint_as_float(orr[8 * i + 1]) * inv_a);
                    const uint32_t a1 = pack_bf16(__uint_as_float(orr[8 * i + 4]) * inv_a, __uint_as_float(orr[8 * i + 5]) * inv_a);
                    const uint32_t b0 = pack_bf16(__uint_as_float(orr[8 * i + 2]) * inv_b, __uint_as_float(orr[8 * i + 3]) * inv_b);
                    const uint32_t b1 = pack_bf16(__uint_as_float(orr[8 * i + 6]) * inv_b, __uint_as_float(orr[8 * i + 7]) * inv_b);
                    const uint32_t ra = __shfl_xor_sync(0xffffffffu, odd ? a0 : a1, 1);
                    const uint32_t rb = __shfl_xor_sync(0xffffffffu, odd ? b0 : b1, 1);
                    if (qa < a.Tq)
                        *reinterpret_cast<uint2*>(oa + c0 + 16 * i) = odd ? make_uint2(ra, a1) : make_uint2(a0, ra);
                    if (qb < a.Tq)
                        *reinterpret_cast<uint2*>(ob + c0 + 16 * i) = odd ? make_uint2(rb, b1) : make_uint2(b0, rb);
                }
            }
            // the output accumulator may be overwritten by the next item's first product
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_o_free);
            AT_ADD(2);
#ifdef NATSL_ATTN_TIMING
            if (at_on) { at_acc[4] += 1; at_acc[5] += n_tiles; }
#endif
            if ((lane & 3) == 0) {
                if (qa < a.Tq) a.lse[((long)x.b * a.Tq + qa) * a.HQ + x.hq] = has_a ? m_a + log2f(l_a) : 0.f;
                if (qb < a.Tq) a.lse[((long)x.b * a.Tq + qb) * a.HQ + x.hq] = has_b ? m_b + log2f(l_b) : 0.f;
            }
        }
#ifdef NATSL_ATTN_TIMING
        if (at_on) {
            at_acc[3] = clock64() - at_start;
            for (int i = 0; i < 6; ++i) g_attn_ts[blockIdx.x * 18 + i] = at_acc[i];
        }
#endif
    }
    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TC_TMEM_COLS);
}

#ifdef NATSL_ATTN_TIMING
}  // namespace natsl
extern "C" int natsl_attn_set_timing(long long* p) {
    return cudaMemcpyToSymbol(natsl::g_attn_ts, &p, sizeof(p)) == cudaSuccess ? 0 : 1;
}
namespace natsl {
#endif

static int resident_ctas() {
    static int n = 0;
#ifdef NATSL_ATTN_TIMING
    if (const char* e = getenv("NATSL_ATTN_CTAS")) return atoi(e);
#endif
    if (n == 0) {
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            return 296;
        n = 2 * sms;
    }
    return n;
}

template <int DK, int DV>
int launch_attn_tc_persist(const void* q, const void* k_rem, const void* v_rem, const void* k, const void* v,
                           const int* rem_base, int rem_slots, int rem_tokens, const int* types_i, const int* indices,
                           const int* n_iters, void* o, float* lse, int B, int B_rem, int T, int Tq, int q_off, int k_split,
                           int HQ, int HKV, int HN, int nbs, float scale, int own_chunk, cudaStream_t st) {
    using L = TcSmem<DK, DV>;
    auto kern = attn_fwd_tc_persist_kernel<DK, DV>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::total);
    if (e != cudaSuccess) {
        set_error("natsl_attn_fwd: cannot reserve %d B of shared memory (%s)", L::total, cudaGetErrorString(e));
        return NATSL_ERR_CUDA;
    }
    CUtensorMap mq, mk, mv, mkr, mvr;
    int rc = encode_bthd_map(&mq, q, B, Tq, HQ, DK, 128, "natsl_attn_fwd(q)");
    if (rc == NATSL_OK) rc = encode_bthd_map(&mk, k, B, T - k_split, HKV, DK, 64, "natsl_attn_fwd(k)");
    if (rc == NATSL_OK) rc = encode_bthd_map(&mv, v, B, T - k_split, HKV, DV, 64, "natsl_attn_fwd(v)");
    if (k_split > 0) {
        const int rt = rem_base ? rem_tokens : k_split, rh = rem_base ? 1 : HKV;
        if (rc == NATSL_OK) rc = encode_bthd_map(&mkr, k_rem, B_rem, rt, rh, DK, 64, "natsl_attn_fwd(k_rem)");
        if (rc == NATSL_OK) rc = encode_bthd_map(&mvr, v_rem, B_rem, rt, rh, DV, 64, "natsl_attn_fwd(v_rem)");
    } else {
        mkr = mk;
        mvr = mv;
        B_rem = B;
    }
    PsArgs a;
    a.status = nullptr;
    if (rc == NATSL_OK) rc = status_word_ptr(&a.status);
    if (rc != NATSL_OK) return rc;
    a.k_split = k_split;
    a.B_rem = B_rem;
    a.rem_base = k_split > 0 ? rem_base : nullptr;
    a.rem_slots = rem_slots;
    a.types_i = types_i;
    a.indices = indices;
    a.attn_n_iters = n_iters;
    a.o = reinterpret_cast<__nv_bfloat16*>(o);
    a.lse = lse;
    a.B = B;
    a.T = T;
    a.Tq = Tq;
    a.q_off = q_off;
    a.HQ = HQ;
    a.HKV = HKV;
    a.HN = HN;
    a.TN = (T + nbs - 1) / nbs;
    a.nbs = nbs;
    a.scale_log2 = scale * 1.44269504f;
    a.own_chunk = own_chunk;
    a.NTq = (Tq + ATT_BM - 1) / ATT_BM;
    const long items = (long)a.NTq * HQ * B;
    if (items > 0x7fffffffL) {
        set_error("natsl_attn_fwd: too many query tiles (%ld)", items);
        return NATSL_ERR_TOO_LARGE;
    }
    a.n_items = (int)items;
    const int grid = a.n_items < resident_ctas() ? a.n_items : resident_ctas();
    kern<<<grid, TC_THREADS, L::total, st>>>(mq, mk, mv, mkr, mvr, a);
    return check_launch("natsl_attn_fwd");
}

#define NATSL_PERSIST_INST(DK, DV)                                                                                      \
    template int launch_attn_tc_persist<DK, DV>(const void*, const void*, const void*, const void*, const void*,        \
                                                const int*, int, int, const int*, const int*, const int*, void*, float*, \
                                                int, int, int, int, int, int, int, int, int, int, float, int, cudaStream_t);
NATSL_PERSIST_INST(64, 64)
NATSL_PERSIST_INST(64, 128)
NATSL_PERSIST_INST(128, 64)
NATSL_PERSIST_INST(128, 128)
#undef NATSL_PERSIST_INST

}  // namespace natsl
