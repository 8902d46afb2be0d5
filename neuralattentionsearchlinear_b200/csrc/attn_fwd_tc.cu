// Chunk-masked softmax attention forward on the 5th-generation tensor cores.
//
// One CTA = 128 queries of one softmax head; two CTAs share an SM (2 x 256 TMEM columns,
// 2 x ~113 KB shared memory).  Warp roles (320 threads):
//   warp 0    TMA producer: Q once, then the K and V tiles of the key-tile walk into a 3- or 4-stage and a
//             2-stage ring (cp.async.bulk.tensor, 128-byte swizzle, zero fill past the sequence end), in the
//             order in which the tensor core frees the stages;
//   warp 1    MMA issuer (one thread): S_j = Q K_j^T into one of two (DV = 128) or three (DV = 64) TMEM score
//             buffers, issued that many tiles ahead, and O += P_j V_j with P read straight from TMEM;
//             completion is signalled with tcgen05.commit on mbarriers;
//   warps 2-9 softmax, 16 query rows per warp, four threads per row (tcgen05.ld.16x256b fragments):
//             mask, online softmax in base 2 with a lazily updated maximum (O in TMEM is only
//             rescaled when the running maximum grows by more than 2^8), P (bf16 pairs) written back
//             with tcgen05.st over the score buffer it came from; at the end O / l -> bf16 -> shared
//             memory -> coalesced global stores.
// While the softmax warps work on tile j the tensor core runs Q K_{j+1}^T and P_{j-1} V_{j-1}.
// The key-tile list (load coordinate, gathered bit) is computed by the producer warp, its only reader; the other
// roles need just the tile count, and the softmax warps the selection bits of the blocks under the own span.
// Same key-tile walk, mask and output conventions as the mma.sync kernel (attn_walk.cuh):
// src/nats/ops/attns/attns.py:62-353 is the reference kernel this replaces.
// Every mbarrier wait has an iteration limit; on expiry the CTA records a status, stops issuing
// work, still frees its TMEM and returns.
#include "attn_tc.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

int attn_fwd_mma_sync(const void* q, const void* k, const void* v, const int32_t* types_i, const int32_t* indices,
                      const int32_t* attn_n_iters, void* o, float* lse, int B, int T, int HQ, int HKV, int HN, int DK,
                      int DV, int nbs, float scale, int own, cudaStream_t st);

// persistent form (attn_fwd_tc_persist.cu), selected by NATSL_FLAG_ATTN_PERSISTENT
template <int DK, int DV>
int launch_attn_tc_persist(const void* q, const void* k_rem, const void* v_rem, const void* k, const void* v,
                           const int* rem_base, int rem_slots, int rem_tokens, const int* types_i, const int* indices,
                           const int* n_iters, void* o, float* lse, int B, int B_rem, int T, int Tq, int q_off, int k_split,
                           int HQ, int HKV, int HN, int nbs, float scale, int own_chunk, cudaStream_t st);

template <int DK, int DV>
__global__ void __launch_bounds__(TC_THREADS, 2)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_kr,
                   const __grid_constant__ CUtensorMap map_vr, int k_split, int B_rem, const int* __restrict__ rem_base,
                   int rem_slots, const int* __restrict__ types_i,
                   const int* __restrict__ indices, const int* __restrict__ attn_n_iters,
                   __nv_bfloat16* __restrict__ o, float* __restrict__ lse, int T, int Tq, int q_off, int HQ, int HKV,
                   int HN, int TN, int nbs, float scale_log2, int own_chunk, int* status) {
    // T = number of keys (and the length the tables were built for); the Tq queries are the tokens
    // [q_off, q_off + Tq) of that sequence (q_off = 0, Tq = T except under sequence parallelism).
    // Keys [0, k_split) live in a second pair of tensors (map_kr / map_vr, batch index b % B_rem: the
    // gathered blocks of other segments, shared by the local segments), keys [k_split, T) in map_k / map_v.
    // With rem_base the gathered tensors are [B_rem, tokens, 1, D]: the selected (block, head) pairs of every
    // gathered segment packed back to back; virtual block g * rem_slots + j of head hkv is pair
    // rem_base[(b % B_rem, g, hkv)] + j.
    using L = TcSmem<DK, DV>;
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t sbase = smem_u32(smem);
    if ((sbase & 1023u) != 0) {                       // swizzled tiles need 1024-byte alignment
        if (tid == 0) atomicExch(status, 2);
        return;
    }
    const int NTq = (T + ATT_BM - 1) / ATT_BM;
    const int it = q_off / ATT_BM + ((int)gridDim.x - 1 - (int)blockIdx.x);     // heaviest tiles first
    const int hq = blockIdx.y, b = blockIdx.z;
    const int hkv = hq / (HQ / HKV), hn = hq / (HQ / HN);
    const int q0 = it * ATT_BM;
    const int* idx = indices + ((long)b * TN * HN + hn) * 2;
    const int* selp = types_i + ((long)b * TN * HN + hn) * 2;
    const long tstride = (long)HN * 2;
    const uint32_t s_q = sbase + L::q, s_k = sbase + L::k, s_v = sbase + L::v;
    int* tile_list = reinterpret_cast<int*>(smem + L::list);
    const uint32_t bar0 = sbase + L::bars;
    // barrier slots (8 bytes each)
    const uint32_t bar_q = bar0, bar_k_full = bar0 + 8, bar_k_empty = bar0 + 40, bar_v_full = bar0 + 72,
                   bar_v_empty = bar0 + 104, bar_s_full = bar0 + 136, bar_p_full = bar0 + 160, bar_pv = bar0 + 184;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::bars + 208);
    constexpr int NSB = TcTmem<DV>::NSB, TC_KST = TcTmem<DV>::KST;
    constexpr uint32_t TC_O_COL = TcTmem<DV>::o_col;

    // requested before anything else; first used after the barrier below
    const int n_past_blocks = __ldg(attn_n_iters + ((long)b * NTq + it) * HN + hn);
    if (tid == 0) {
        mbar_init(bar_q, 1);
        for (int i = 0; i < 4; ++i) {
            mbar_init(bar_k_full + 8 * i, 1);
            mbar_init(bar_k_empty + 8 * i, 1);
            mbar_init(bar_v_full + 8 * i, 1);
            mbar_init(bar_v_empty + 8 * i, 1);
        }
        for (int i = 0; i < NSB; ++i) {
            mbar_init(bar_s_full + 8 * i, 1);
            mbar_init(bar_p_full + 8 * i, 8);            // one arrival per softmax warp
        }
        mbar_init(bar_pv, 1);
        mbar_init(bar_pv + 8, 1);
        mbar_fence_init();
        // the query tile and the first own-span key / value tiles depend on no table: their loads start at once
        prefetch_tensormap(&map_q);
        mbar_expect_tx(bar_q, 128 * DK * 2);
#pragma unroll
        for (int sub = 0; sub < DK / 64; ++sub) tma_load_4d(s_q + sub * 16384, &map_q, sub * 64, hq, q0 - q_off, b, bar_q);
        const TileWalk w0 = make_walk(q0, T, nbs, 0);
        const int hkv0 = hq / (HQ / HKV);
        for (int j = 0; j < min(w0.n_span, TcTmem<DV>::KST); ++j) {
            mbar_expect_tx(bar_k_full + j * 8, 64 * DK * 2);
#pragma unroll
            for (int sub = 0; sub < DK / 64; ++sub)
                tma_load_4d(s_k + j * (64 * DK * 2) + sub * 8192, &map_k, sub * 64, hkv0, w0.span_start + j * ATT_BN - k_split, b,
                            bar_k_full + j * 8);
        }
        for (int j = 0; j < min(w0.n_span, TC_VST); ++j) {
            mbar_expect_tx(bar_v_full + j * 8, 64 * DV * 2);
#pragma unroll
            for (int sub = 0; sub < DV / 64; ++sub)
                tma_load_4d(s_v + j * (64 * DV * 2) + sub * 8192, &map_v, sub * 64, hkv0, w0.span_start + j * ATT_BN - k_split, b,
                            bar_v_full + j * 8);
        }
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TC_TMEM_COLS);
    // Nothing above waits for global memory: the barrier that publishes the mbarriers and the TMEM address comes
    // before any table is read.  Each role then fetches what it needs by itself: every warp the tile count; the
    // producer the tile list (it is the only reader of the index table); the softmax warps the selection bits of the
    // one or two blocks that the own span touches.
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const TileWalk walk = make_walk(q0, T, nbs, n_past_blocks);
    const int n_tiles = walk.n_tiles;
    const int b_rem = b % B_rem;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            prefetch_tensormap(&map_k);
            prefetch_tensormap(&map_v);
            if (k_split > 0) {
                prefetch_tensormap(&map_kr);
                prefetch_tensormap(&map_vr);
            }
        }
        RemoteKeys rk;
        rk.k_split = k_split;
        rk.slots = rem_slots;
        rk.stride = HKV;
        rk.base = rem_base ? rem_base + ((long)b_rem * (k_split / (rem_slots * nbs))) * HKV + hkv : nullptr;
        for (int j = lane; j < min(n_tiles, TC_LIST_CAP); j += 32)
            tile_list[j] = pack_tile(walk, j, idx, selp, tstride, nbs, rk);
        __syncwarp();
        auto tile_desc = [&](int j) -> int {
            return j < TC_LIST_CAP ? tile_list[j] : pack_tile(walk, j, idx, selp, tstride, nbs, rk);
        };
        const int rem_head = rem_base ? 0 : hkv;     // packed pairs have no head axis
        auto load_k = [&](int j) {                    // lane 0 only
            const int td = tile_desc(j), stg = j % TC_KST;
            const bool rem = (td >> 29) & 1;
            const uint32_t full = bar_k_full + stg * 8;
            mbar_expect_tx(full, 64 * DK * 2);
#pragma unroll
            for (int sub = 0; sub < DK / 64; ++sub)
                tma_load_4d(s_k + stg * (64 * DK * 2) + sub * 8192, rem ? &map_kr : &map_k, sub * 64, rem ? rem_head : hkv,
                            td & TILE_COORD_MASK, rem ? b_rem : b, full);
        };
        auto load_v = [&](int j) {                    // lane 0 only; also warms L2 for the tile TC_VST further on
            const int td = tile_desc(j), stg = j % TC_VST;
            const bool rem = (td >> 29) & 1;
            const uint32_t full = bar_v_full + stg * 8;
            mbar_expect_tx(full, 64 * DV * 2);
#pragma unroll
            for (int sub = 0; sub < DV / 64; ++sub)
                tma_load_4d(s_v + stg * (64 * DV * 2) + sub * 8192, rem ? &map_vr : &map_v, sub * 64, rem ? rem_head : hkv,
                            td & TILE_COORD_MASK, rem ? b_rem : b, full);
            if (j + TC_VST < n_tiles) {
                const int t1 = tile_desc(j + TC_VST);
                const bool rem1 = (t1 >> 29) & 1;
                const int c1 = t1 & TILE_COORD_MASK, b1 = rem1 ? b_rem : b, h1 = rem1 ? rem_head : hkv;
#pragma unroll
                for (int sub = 0; sub < DV / 64; ++sub) tma_prefetch_4d(rem1 ? &map_vr : &map_v, sub * 64, h1, c1, b1);
#pragma unroll
                for (int sub = 0; sub < DK / 64; ++sub) tma_prefetch_4d(rem1 ? &map_kr : &map_k, sub * 64, h1, c1, b1);
            }
        };
        // The loads follow the order in which the tensor core frees the ring stages: the K stages of the first NSB
        // tiles right after their Q K^T products, then alternately the V stage of tile i (after P_i V_i) and the
        // K stage of tile i + NSB (Q K_{i+NSB}^T is issued right behind P_i V_i).  Every wait is for the next event
        // of that sequence, so the producer sleeps in the barrier instead of polling two rings.
        int jk = min(TC_KST, n_tiles), jv = min(TC_VST, n_tiles);
        if (lane == 0) {                               // the own-span tiles among these were requested at kernel start
            for (int j = min(walk.n_span, TC_KST); j < jk; ++j) load_k(j);
            for (int j = min(walk.n_span, TC_VST); j < jv; ++j) load_v(j);
        }
        bool ok = true;
        auto next_k = [&]() {
            ok = __all_sync(0xffffffffu, mbar_wait(bar_k_empty + (jk % TC_KST) * 8, ((jk / TC_KST) - 1) & 1, status));
            if (ok && lane == 0) load_k(jk);
            ++jk;
        };
        for (int i = 0; ok && i < NSB && jk < n_tiles; ++i) next_k();
        while (ok && (jk < n_tiles || jv < n_tiles)) {
            if (jv < n_tiles) {
                ok = __all_sync(0xffffffffu, mbar_wait(bar_v_empty + (jv % TC_VST) * 8, ((jv / TC_VST) - 1) & 1, status));
                if (ok && lane == 0) load_v(jv);
                ++jv;
            }
            if (ok && jk < n_tiles) next_k();
            __syncwarp();
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 64, false);
        constexpr uint32_t idesc_pv = umma_idesc_bf16(128, DV, true);
        auto issue_qk = [&](int j) {                  // S_{j&1} = Q K_j^T   (lane 0 only)
            const int sb = j % NSB, stg = j % TC_KST;
            const uint32_t kt = s_k + stg * (64 * DK * 2);
#pragma unroll
            for (int kk = 0; kk < DK / 16; ++kk) {
                const uint64_t ad = umma_desc(s_q + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
                const uint64_t bd = umma_desc(kt + (kk >> 2) * 8192 + (kk & 3) * 32, 16, 1024);
                umma_ss(tmem + sb * 64, ad, bd, idesc_qk, kk > 0);
            }
            umma_commit(bar_s_full + sb * 8);
            umma_commit(bar_k_empty + stg * 8);
        };
        bool ok = __all_sync(0xffffffffu, mbar_wait(bar_q, 0, status));
        for (int j = 0; ok && j < min(NSB, n_tiles); ++j) {
            ok = __all_sync(0xffffffffu, mbar_wait(bar_k_full + (j % TC_KST) * 8, (j / TC_KST) & 1, status));
            if (ok && lane == 0) {
                tc_fence_after();
                issue_qk(j);
            }
            __syncwarp();
        }
        for (int j = 0; ok && j < n_tiles; ++j) {
            const int sb = j % NSB, vstg = j % TC_VST;
            ok = __all_sync(0xffffffffu, mbar_wait(bar_v_full + vstg * 8, (j / TC_VST) & 1, status));
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_p_full + sb * 8, (j / NSB) & 1, status));
            if (!ok) break;
            if (lane == 0) {
                tc_fence_after();
                const uint32_t vt = s_v + vstg * (64 * DV * 2);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint64_t bd = umma_desc(vt + kk * 2048, 8192, 1024);
                    umma_ts(tmem + TC_O_COL, tmem + sb * 64 + kk * 8, bd, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(bar_v_empty + vstg * 8);
                umma_commit(bar_pv + (j & 1) * 8);
            }
            __syncwarp();
            if (j + NSB < n_tiles) {
                const int jn = j + NSB;
                ok = __all_sync(0xffffffffu, mbar_wait(bar_k_full + (jn % TC_KST) * 8, (jn / TC_KST) & 1, status));
                if (!ok) break;
                if (lane == 0) {
                    tc_fence_after();
                    issue_qk(jn);
                }
                __syncwarp();
            }
        }
    } else {
        // ------------------------------------------------------------ softmax + epilogue (8 warps)
        // Warp (quad, half) owns the 16 query rows quad*32 + half*16 ... of the tile (a warp reaches only its own
        // quarter of the TMEM lanes).  In the 16x256b layout a thread holds, of rows ra and ra + 8, the columns
        // 8k + 2(lane%4), +1 for k = 0..7: 32 scores; the four threads of a row meet through two shuffles.
        const int quad = warp & 3, half = (warp - 2) >> 2;
        const int row_a = quad * 32 + half * 16 + (lane >> 2), row_b = row_a + 8;
        const int cq = (lane & 3) * 2;
        const int t_a = q0 + row_a, t_b = q0 + row_b;
        const uint32_t t_rows = tmem + ((uint32_t)(quad * 32 + half * 16) << 16);
        const uint32_t t_o = t_rows + TC_O_COL;
        float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
        // the own span lies in at most two selection blocks (nbs >= 64 and 64 | q0 - span_start)
        const int blk0 = walk.span_start / nbs;
        const bool sel0 = selp[(long)blk0 * tstride] != 0;
        const bool sel1 = blk0 + 1 < TN && selp[(long)(blk0 + 1) * tstride] != 0;
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            const int sb = j % NSB;
            const uint32_t t_s = t_rows + sb * 64;
            ok = __all_sync(0xffffffffu, mbar_wait(bar_s_full + sb * 8, (j / NSB) & 1, status));
            if (!ok) break;
            tc_fence_after();
            uint32_t sr[32];
            tmem_ld_16x256b_x8(t_s, sr);
            tmem_ld_wait();
            if (j < walk.n_span) {
                // own-span tile: per row the visible keys are columns [0, limit] (attn_walk.cuh: visible())
                const int s0 = walk.span_start + j * ATT_BN;
                const bool selb = (s0 / nbs == blk0) ? sel0 : sel1;
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
                    // O must be at rest: P_{j-1} V_{j-1} has to be complete.  Even and odd tiles signal on two
                    // barriers.  S_j was produced behind P_{j-NSB} V_{j-NSB}, hence behind P_{j-3} V_{j-3} (the
                    // previous phase of the barrier waited on; NSB <= 3), and P_{j+1} V_{j+1} cannot have started:
                    // the barrier is in the phase waited for or the one after it, so a parity wait without having
                    // watched the earlier phases is unambiguous.
                    ok = __all_sync(0xffffffffu, mbar_wait(bar_pv + ((j - 1) & 1) * 8, ((j - 1) >> 1) & 1, status));
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
            tmem_st_16x128b_x8(t_s, pr);                      // P_j over the first 32 columns of S_{j&1}
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p_full + sb * 8);
        }
        // The last two products, in order: S of the last tile was produced behind P V of tile n-1-NSB >= n-4, the
        // previous phase of the barrier of tile n-2; once that one is complete so is tile n-3, the previous phase
        // of the barrier of the last tile.
        if (ok && n_tiles >= 2)
            ok = __all_sync(0xffffffffu, mbar_wait(bar_pv + ((n_tiles - 2) & 1) * 8, ((n_tiles - 2) >> 1) & 1, status));
        if (ok)
            ok = __all_sync(0xffffffffu, mbar_wait(bar_pv + ((n_tiles - 1) & 1) * 8, ((n_tiles - 1) >> 1) & 1, status));
        unsigned char* stage = smem + L::q;
        if (ok) {
            tc_fence_after();
            l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
            l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
            l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
            l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
            const bool has_a = l_a > 0.f, has_b = l_b > 0.f;
            const float inv_a = has_a ? 1.f / l_a : 0.f, inv_b = has_b ? 1.f / l_b : 0.f;
#pragma unroll 1
            for (int c0 = 0; c0 < DV; c0 += 64) {
                uint32_t orr[32];
                tmem_ld_16x256b_x8(t_o + c0, orr);
                tmem_ld_wait();
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int chunk = (c0 >> 3) + k;
                    *reinterpret_cast<uint32_t*>(stage + swz<DV * 2>(row_a, chunk) + (lane & 3) * 4) =
                        pack_bf16(__uint_as_float(orr[4 * k]) * inv_a, __uint_as_float(orr[4 * k + 1]) * inv_a);
                    *reinterpret_cast<uint32_t*>(stage + swz<DV * 2>(row_b, chunk) + (lane & 3) * 4) =
                        pack_bf16(__uint_as_float(orr[4 * k + 2]) * inv_b, __uint_as_float(orr[4 * k + 3]) * inv_b);
                }
            }
            if ((lane & 3) == 0) {
                if (t_a - q_off < Tq) lse[((long)b * Tq + (t_a - q_off)) * HQ + hq] = has_a ? m_a + log2f(l_a) : 0.f;
                if (t_b - q_off < Tq) lse[((long)b * Tq + (t_b - q_off)) * HQ + hq] = has_b ? m_b + log2f(l_b) : 0.f;
            }
        }
        // every softmax warp reaches this barrier, also after a failed wait (no warp may be left behind)
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (ok) {
            constexpr int CPR = DV / 8;
            __nv_bfloat16* obase = o + (((long)b * Tq + (q0 - q_off)) * HQ + hq) * DV;
            const int st_tid = tid - 64;
            for (int i = st_tid; i < 128 * CPR; i += 256) {
                const int r = i / CPR, cch = i % CPR;
                if (q0 - q_off + r < Tq) {
                    const uint4 x = *reinterpret_cast<const uint4*>(stage + swz<DV * 2>(r, cch));
                    *reinterpret_cast<uint4*>(obase + (long)r * HQ * DV + cch * 8) = x;
                }
            }
        }
    }
    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TC_TMEM_COLS);
}

template <int DK, int DV>
static int launch_attn_tc(const void* q, const void* k_rem, const void* v_rem, const void* k, const void* v,
                          const int* rem_base, int rem_slots, int rem_tokens, const int* types_i, const int* indices,
                          const int* n_iters, void* o, float* lse, int B, int B_rem, int T, int Tq, int q_off, int k_split,
                          int HQ, int HKV, int HN, int nbs, float scale, int own_chunk, cudaStream_t st) {
    using L = TcSmem<DK, DV>;
    auto kern = attn_fwd_tc_kernel<DK, DV>;
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
    int* status = nullptr;
    if (rc == NATSL_OK) rc = status_word_ptr(&status);
    if (rc != NATSL_OK) return rc;
    const int NTq = (Tq + ATT_BM - 1) / ATT_BM, TN = (T + nbs - 1) / nbs;
    dim3 grid(NTq, HQ, B);
    kern<<<grid, TC_THREADS, L::total, st>>>(mq, mk, mv, mkr, mvr, k_split, B_rem, k_split > 0 ? rem_base : nullptr,
                                             rem_slots, types_i, indices, n_iters,
                                             reinterpret_cast<__nv_bfloat16*>(o),
                                             lse, T, Tq, q_off, HQ, HKV, HN, TN, nbs, scale * 1.44269504f, own_chunk,
                                             status);
    return check_launch("natsl_attn_fwd");
}

}  // namespace natsl

extern "C" int natsl_attn_fwd_split(const void* q, const void* k_rem, const void* v_rem, const int32_t* rem_base,
                                    int rem_slots, int rem_tokens, const void* k, const void* v, const int32_t* types_i,
                                    const int32_t* indices, const int32_t* attn_n_iters, void* o, float* lse, int B,
                                    int B_rem, int T, int Tq, int q_off, int k_split, int HQ, int HKV, int HN, int DK,
                                    int DV, int nbs, float scale, int flags, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(q && k && v && types_i && indices && attn_n_iters && o && lse, NATSL_ERR_NULL,
                  "natsl_attn_fwd: null pointer");
    NATSL_REQUIRE(B > 0 && T > 0 && HQ > 0 && HKV > 0 && HN > 0 && HQ % HKV == 0 && HQ % HN == 0, NATSL_ERR_BAD_SHAPE,
                  "natsl_attn_fwd: bad shape B=%d T=%d HQ=%d HKV=%d HN=%d", B, T, HQ, HKV, HN);
    NATSL_REQUIRE(Tq > 0 && q_off >= 0 && q_off + Tq <= T, NATSL_ERR_BAD_SHAPE,
                  "natsl_attn_fwd: queries [%d, %d) do not lie inside the %d keys", q_off, q_off + Tq, T);
    NATSL_REQUIRE(HQ <= 65535 && B <= 65535, NATSL_ERR_TOO_LARGE, "natsl_attn_fwd: B and HQ must be <= 65535");
    NATSL_REQUIRE(nbs >= 64 && nbs % 64 == 0, NATSL_ERR_UNSUPPORTED,
                  "natsl_attn_fwd: nats_block_size must be a multiple of 64 (got %d)", nbs);
    NATSL_REQUIRE(q_off % 128 == 0 && q_off % nbs == 0, NATSL_ERR_UNSUPPORTED,
                  "natsl_attn_fwd: the query offset must be a multiple of 128 and of nats_block_size (got %d)", q_off);
    NATSL_REQUIRE(k_split >= 0 && k_split <= q_off && k_split % nbs == 0, NATSL_ERR_BAD_SHAPE,
                  "natsl_attn_fwd: the key split %d must be a multiple of nats_block_size and <= the query offset %d",
                  k_split, q_off);
    NATSL_REQUIRE(k_split == 0 || (k_rem && v_rem && B_rem > 0 && B % B_rem == 0), NATSL_ERR_BAD_SHAPE,
                  "natsl_attn_fwd: a key split needs k_rem, v_rem and a batch B_rem that divides B");
    NATSL_REQUIRE(k_split == 0 || !rem_base || (rem_slots > 0 && k_split % (rem_slots * nbs) == 0 && rem_tokens > 0),
                  NATSL_ERR_BAD_SHAPE, "natsl_attn_fwd: packed gathered keys need rem_slots dividing the key split");
    const int own = (flags & NATSL_FLAG_ATTN_OWN_CHUNK) ? 1 : 0;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (flags & NATSL_FLAG_ATTN_MMA_SYNC) {
        NATSL_REQUIRE(q_off == 0 && Tq == T && k_split == 0, NATSL_ERR_UNSUPPORTED,
                      "natsl_attn_fwd: the mma.sync comparison kernel has no query offset or key split");
        return attn_fwd_mma_sync(q, k, v, types_i, indices, attn_n_iters, o, lse, B, T, HQ, HKV, HN, DK, DV, nbs, scale,
                                 own, st);
    }
#define NATSL_ATT_ARGS                                                                                                 \
    q, k_rem, v_rem, k, v, rem_base, rem_slots, rem_tokens, types_i, indices, attn_n_iters, o, lse, B, B_rem, T, Tq, q_off, \
        k_split, HQ, HKV, HN, nbs, scale, own, st
    const bool one_item = (flags & NATSL_FLAG_ATTN_PERSISTENT) == 0;
#define NATSL_ATT_CASE(KK, VV)                                                \
    if (DK == KK && DV == VV)                                                 \
        return one_item ? launch_attn_tc<KK, VV>(NATSL_ATT_ARGS) : launch_attn_tc_persist<KK, VV>(NATSL_ATT_ARGS);
    NATSL_ATT_CASE(64, 64)
    NATSL_ATT_CASE(64, 128)
    NATSL_ATT_CASE(128, 64)
    NATSL_ATT_CASE(128, 128)
#undef NATSL_ATT_CASE
#undef NATSL_ATT_ARGS
    set_error("natsl_attn_fwd: unsupported head dims DK=%d DV=%d (each 64 or 128)", DK, DV);
    return NATSL_ERR_UNSUPPORTED;
}

extern "C" int natsl_attn_fwd_ex(const void* q, const void* k, const void* v, const int32_t* types_i,
                                 const int32_t* indices, const int32_t* attn_n_iters, void* o, float* lse, int B,
                                 int T, int Tq, int q_off, int HQ, int HKV, int HN, int DK, int DV, int nbs, float scale,
                                 int flags, void* stream) {
    return natsl_attn_fwd_split(q, nullptr, nullptr, nullptr, 0, 0, k, v, types_i, indices, attn_n_iters, o, lse, B, B, T,
                                Tq, q_off, 0, HQ, HKV, HN, DK, DV, nbs, scale, flags, stream);
}

extern "C" int natsl_attn_fwd(const void* q, const void* k, const void* v, const int32_t* types_i,
                              const int32_t* indices, const int32_t* attn_n_iters, void* o, float* lse, int B, int T,
                              int HQ, int HKV, int HN, int DK, int DV, int nbs, float scale, int flags, void* stream) {
    return natsl_attn_fwd_ex(q, k, v, types_i, indices, attn_n_iters, o, lse, B, T, T, 0, HQ, HKV, HN, DK, DV, nbs, scale,
                             flags, stream);
}
