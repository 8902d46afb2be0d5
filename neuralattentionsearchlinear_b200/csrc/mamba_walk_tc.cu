// Mamba2 / SSD recurrence AND chunk output in one walk on the 5th-generation tensor cores
// (state dim K = 128, head dim V = 64, any nats_block_size that is a multiple of 64).  One CTA per (batch, head)
// walks the 64-token chunks in order; the K x V state lives in TMEM (fp32) and is never written to global memory.
// Per chunk c (S = state the chunk reads, carry = decay of the skipped blocks before it, g = chunk-local cumsum):
//     DP = q k^T                      128-row A operand [k ; q]: rows 64-127 are the q rows             (MMA 0)
//     P  = tril(DP e^{g_i - g_j})     q warps, from TMEM into shared memory (bf16)
//     o  = scale (e^{g+carry} q S + P v)                                                         (MMA 1, MMA 2 + q warps)
//     S <- e^{g_last+carry} S + k^T (v e^{min(g_last-g, 0)})                                       (MMA 3)
// which is src/nats/ops/mamba/chunk_h.py:139-218 (recurrence) fused with src/nats/ops/mamba/chunk_o.py:137-198
// (output) and the carry of src/nats/ops/utils/cumsum.py:85-133.  Only chunks of selected blocks keep their update:
// with nats_block_size > 64 the chunks of an unselected block update the state as well (their outputs read it), and
// the state saved at the start of the block (a second TMEM region) comes back at its end -- the token recurrence of
// the reference's decode kernel, src/nats/ops/mamba/fused_recurrent.py:28-322.
// The decay of an update is applied when the state is copied to shared memory for the next chunk (one TMEM pass per
// update: bf16 copy out, multiply by the next update's decay, write back), so the accumulating MMA 3 needs no
// separate rescale.  The serial chain of a chunk is MMA 3 -> that pass; it has warps of its own:
//   warp 0      TMA producer (k, q, v tiles in three stages);
//   warp 1      issuer of MMA 3 (the chain); warp 12 issuer of the output products: per chunk MMA 1 (reads the bf16
//               copy the chunk started from; the copy is double-buffered with a full / empty barrier pair, so that the
//               chain runs ahead of the output by one copy) K-step by K-step in turn with MMA 0 of the next chunk, then
//               MMA 2.  Two issuing threads because one thread issues a 128 x 64 x 16 product only every ~130 cycles;
//   warps 2-5   state warps, one per quarter of the TMEM lanes: wait for MMA 3, publish the state;
//   warps 8-9   token warps (rows 0-63): the scaled v tile of the next chunk;
//   warps 6-7, 10-11   q warps (rows 64-127, 32 columns each): P of the next chunk, then the output rows of this one.
// With o == NULL only the recurrence runs (final state only).
// All mbarrier waits are bounded (status word + clean teardown on expiry); every barrier is waited for in every one
// of its phases by each of its waiters, and no phase can complete before every waiter has seen the one before it.
#include "tc_common.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

#ifdef NATSL_MW_TIMING
// scratch build only: cycles spent per role of CTA (0, 0), summed over the chunks
__device__ long long mw_t[32];
#define MW_T0() long long t__ = clock64()
#define MW_ACC(i)                                                  \
    do {                                                           \
        const long long n__ = clock64();                           \
        if (lane == 0 && blockIdx.x == 0 && blockIdx.y == 0) mw_t[i] += n__ - t__; \
        t__ = n__;                                                 \
    } while (0)
#else
#define MW_T0()
#define MW_ACC(i)
#endif

constexpr int MW_THREADS = 416;          // 13 warps
constexpr uint32_t MW_TMEM_COLS = 512;
// TMEM column offsets: state, saved state, q S (double-buffered), P v, q k^T (double-buffered)
constexpr uint32_t MW_S = 0, MW_BK = 64, MW_D1 = 128, MW_D1B = 192, MW_D2 = 256, MW_DP = 320, MW_DPB = 384;
constexpr int MW_MAX_NT = 1024;
constexpr int MW_ACTIVE = 1, MW_RESTORE = 2, MW_SAVE = 4, MW_SEL = 8;     // per-chunk flags

struct MwSmem {
    // stage: 2 tiles [128][64] (one per half of the K dimension): rows 0-63 the k tile, rows 64-127 the q tile (32 KB),
    // then v [64][64] (8 KB).  The 128-row tile is the A operand of the q products (its first 64 result rows, k k^T and
    // k S, are never read); its first half alone is the k operand.
    static constexpr int a = 0, v = 32768, stage = 40960, nstage = 3;
    static constexpr int sbf = nstage * stage;            // 2 x S bf16 [128 k-rows][64 v-cols]              32 KB
    static constexpr int vs = sbf + 32768;                // 2 x scaled v [64 tok][64]                       16 KB
    static constexpr int pp = vs + 16384;                 // 2 x P padded to 128 rows: [128][64 tok]        32 KB
    static constexpr int gs = pp + 32768;                 // 2 x g of the chunk's 64 tokens (float)
    static constexpr int meta = gs + 512;                 // per chunk: carry, dec, g_last (float), flags (int)
    static constexpr int bars = meta + 4 * 4 * MW_MAX_NT;
    static constexpr int total = bars + 256;
};

__global__ void __launch_bounds__(MW_THREADS, 1)
mamba_walk_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const float* __restrict__ gcs,
                     const int* __restrict__ types_i, const int* __restrict__ indices, const int* __restrict__ n_blocks,
                     const float* __restrict__ h0, __nv_bfloat16* __restrict__ o, float* __restrict__ ht, int T, int H,
                     int HN, int TN, int nbs, float scale, int decay, int trailing_quirk, int* status) {
    using L = MwSmem;
    constexpr int K = 128, V = 64;
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t sbase = smem_u32(smem);
    if ((sbase & 1023u) != 0) {
        if (tid == 0) atomicExch(status, 2);
        return;
    }
    const int h = blockIdx.x, b = blockIdx.y;
    const int hn = h / (H / HN);
    const int NT = (T + 63) / 64;
    const int cpb = nbs / 64;
    const bool want_o = o != nullptr;
    float* m_carry = reinterpret_cast<float*>(smem + L::meta);
    float* m_dec = m_carry + MW_MAX_NT;
    float* m_gl = m_dec + MW_MAX_NT;
    int* m_fl = reinterpret_cast<int*>(m_gl + MW_MAX_NT);
    float* s_g = reinterpret_cast<float*>(smem + L::gs);
    const uint32_t bar0 = sbase + L::bars;
    // barriers: full[2] / empty[2] tile stages; dp (MMA 0 done); pfull (P written by the q warps); pv (scaled v of a
    // chunk written by the token warps); d2 (MMA 2, and with it MMA 1, done); s3 (MMA 3 done); sready (state copy
    // published); odone (output rows read from TMEM)
    // cfull[2] / cempty[2]: the two bf16 copies of the state (written by the state warps, read by MMA 1)
    // dp[2], pfull[2]: one per q k^T buffer / P tile.  A tile stage is released by the warps that see its last readers complete (the
    // state warps MMA 3, the q warps MMA 2) and so is a state copy (the q warps): a tcgen05.commit costs the issuing
    // thread about as much as two products.
    const uint32_t bar_full = bar0, bar_empty = bar0 + 24, bar_dp = bar0 + 48, bar_pfull = bar0 + 64, bar_pv = bar0 + 80,
                   bar_d2 = bar0 + 88, bar_s3 = bar0 + 96, bar_sready = bar0 + 104, bar_odone = bar0 + 112,
                   bar_cfull = bar0 + 120, bar_cempty = bar0 + 136;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::bars + 192);

    if (tid == 0) {
        for (int i = 0; i < L::nstage; ++i) {
            mbar_init(bar_full + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, want_o ? 256 : 128);       // state warps (+ q warps)
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_cfull + 8 * i, 128);
            mbar_init(bar_cempty + 8 * i, 128);
            mbar_init(bar_dp + 8 * i, 1);
            mbar_init(bar_pfull + 8 * i, 128);
        }
        mbar_init(bar_pv, 64);
        mbar_init(bar_d2, 1);
        mbar_init(bar_s3, 1);
        mbar_init(bar_sready, 128);
        mbar_init(bar_odone, 128);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), MW_TMEM_COLS);
    // ---- per-chunk metadata
    for (int c = tid; c < NT; c += MW_THREADS) {
        m_fl[c] = types_i[(((long)b * TN + c / cpb) * HN + hn) * 2 + 1] != 0 ? MW_SEL : 0;
        m_gl[c] = gcs[((long)b * T + min(c * 64 + 63, T - 1)) * H + h];
    }
    if (want_o) {
        // rows 0-63 of the two P tiles are never written: they stay zero (their result rows are never read)
        for (int i = tid; i < 2 * 512; i += MW_THREADS)
            reinterpret_cast<uint4*>(smem + L::pp + (i >> 9) * 16384)[i & 511] = make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
    if (tid == 0) {
        const int nsel = n_blocks[((long)b * HN + hn) * 2 + 1];
        const int last_sel = nsel > 0 ? indices[(((long)b * TN + (nsel - 1)) * HN + hn) * 2 + 1] : -1;
        float carry = 0.f, carry_save = 0.f, blk_g = 0.f;
        for (int c = 0; c < NT; ++c) {
            const int blk = c / cpb, sub = c % cpb;
            const bool sel = (m_fl[c] & MW_SEL) != 0;
            const bool active = cpb > 1 || sel;
            const bool may_carry = decay && (!trailing_quirk || blk < last_sel);
            int fl = sel ? MW_SEL : 0;
            if (cpb > 1 && sub == 0) {
                carry_save = carry;
                blk_g = 0.f;
                if (!sel) fl |= MW_SAVE;
            }
            const float gl = m_gl[c];
            m_carry[c] = carry;
            blk_g += gl;
            if (active) {
                fl |= MW_ACTIVE;
                m_dec[c] = __expf(gl + carry);
                carry = 0.f;
            } else {
                m_dec[c] = 1.f;
                if (may_carry) carry += gl;
            }
            if (cpb > 1 && (sub == cpb - 1 || c == NT - 1) && !sel) {
                fl |= MW_RESTORE;
                carry = carry_save + (may_carry ? blk_g : 0.f);
            }
            m_fl[c] = fl;
        }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    // chunk-local cumsum of token `tok` of chunk c (clamped to the last valid token of a ragged chunk)
    auto load_g = [&](int c, int tok) -> float {
        const int valid = min(64, T - c * 64);
        return gcs[((long)b * T + (long)c * 64 + min(tok, valid - 1)) * H + h];
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            prefetch_tensormap(&map_q);
            prefetch_tensormap(&map_k);
            prefetch_tensormap(&map_v);
        }
        for (int c = 0; c < NT; ++c) {
            const int stg = c % L::nstage;
            const int t0 = c * 64;
            if (c >= L::nstage) {
                bool ok = mbar_wait(bar_empty + stg * 8, ((c / L::nstage) - 1) & 1, status);
                if (!__all_sync(0xffffffffu, ok)) break;
            }
            if (lane == 0) {
                const uint32_t full = bar_full + stg * 8, base = sbase + stg * L::stage;
                mbar_expect_tx(full, (want_o ? 16384 : 0) + 16384 + 8192);
#pragma unroll
                for (int sub = 0; sub < 2; ++sub) {
                    tma_load_4d(base + L::a + sub * 16384, &map_k, sub * 64, h, t0, b, full);                       // rows 0-63
                    if (want_o) tma_load_4d(base + L::a + sub * 16384 + 8192, &map_q, sub * 64, h, t0, b, full);   // rows 64-127
                }
                tma_load_4d(base + L::v, &map_v, 0, h, t0, b, full);
                if (c + L::nstage < NT) {                           // warm L2 for the tiles this stage receives next
#pragma unroll
                    for (int sub = 0; sub < 2; ++sub) {
                        if (want_o) tma_prefetch_4d(&map_q, sub * 64, h, t0 + 64 * L::nstage, b);
                        tma_prefetch_4d(&map_k, sub * 64, h, t0 + 64 * L::nstage, b);
                    }
                    tma_prefetch_4d(&map_v, 0, h, t0 + 64 * L::nstage, b);
                }
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ issuer of the state update (the serial chain)
        constexpr uint32_t id_3 = umma_idesc_bf16(128, 64, true) | (1u << 15);          // k^T v~ (A MN-major)
        bool ok = true;
        for (int c = 0; ok && c < NT; ++c) {
            const int stg = c % L::nstage;
            const uint32_t base = sbase + stg * L::stage;
            const int fl = m_fl[c];
            MW_T0();
            ok = __all_sync(0xffffffffu, mbar_wait(bar_full + stg * 8, (c / L::nstage) & 1, status));
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_sready, c & 1, status));
            MW_ACC(0);
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_pv, c & 1, status));
            MW_ACC(1);
            if (!ok) break;
            if (lane == 0) {
                // the update of the last chunk of an unselected block would be thrown away: it is not issued
                tc_fence_after();
                if ((fl & MW_ACTIVE) && !(fl & MW_RESTORE)) {
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const uint64_t ak = umma_desc(base + L::a + kk * 2048, 16384, 1024);
                        const uint64_t bv = umma_desc(sbase + L::vs + (c & 1) * 8192 + kk * 2048, 8192, 1024);
                        umma_ss(tmem + MW_S, ak, bv, id_3, 1u);
                    }
                }
                umma_commit(bar_s3);
            }
            __syncwarp();
            MW_ACC(2);
        }
    } else if (warp == 12) {
        // ------------------------------------------------------------ issuer of the output products
        if (want_o) {
            constexpr uint32_t id_0 = umma_idesc_bf16(128, 64, false);                  // [0;q] k^T
            constexpr uint32_t id_1 = umma_idesc_bf16(128, 64, true);                   // [0;q] S
            constexpr uint32_t id_2 = umma_idesc_bf16(128, 64, true);                   // P v
            bool ok = __all_sync(0xffffffffu, mbar_wait(bar_full, 0, status));
            if (ok && lane == 0) {                     // q k^T of chunk 0
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint64_t ad = umma_desc(sbase + L::a + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
                    umma_ss(tmem + MW_DP, ad, ad, id_0, kk > 0);           // the k operand is the first half of the same tile
                }
                umma_commit(bar_dp);
            }
            __syncwarp();
            int ncopy = 0;                             // copy of the state that the current chunk reads: ncopy & 1
            bool fresh = true;                         // ... and it has not been waited for yet
            for (int c = 0; ok && c < NT; ++c) {
                const int stg = c % L::nstage, nstg = (c + 1) % L::nstage;
                const uint32_t base = sbase + stg * L::stage;
                const int fl = m_fl[c];
                const int cp = ncopy & 1;
                MW_T0();
                if (fresh) ok = __all_sync(0xffffffffu, mbar_wait(bar_cfull + cp * 8, (ncopy >> 1) & 1, status));
                fresh = false;
                MW_ACC(3);
                // q k^T of the next chunk goes to the other buffer: its last reader was P of chunk c - 1, waited for
                // before MMA 2 of that chunk
                const bool ahead = c + 1 < NT;
                if (ok && ahead) ok = __all_sync(0xffffffffu, mbar_wait(bar_full + nstg * 8, ((c + 1) / L::nstage) & 1, status));
                MW_ACC(4);
                if (ok && lane == 0) {
                    // q S of this chunk and q k^T of the next one, K-step by K-step in turn
                    tc_fence_after();
                    const uint32_t d1 = tmem + ((c & 1) ? MW_D1B : MW_D1);
                    const uint32_t nbase = sbase + nstg * L::stage;
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        const uint64_t ad = umma_desc(base + L::a + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
                        const uint64_t bs = umma_desc(sbase + L::sbf + cp * 16384 + kk * 2048, 16384, 1024);
                        umma_ss(d1, ad, bs, id_1, kk > 0);
                        if (ahead) {
                            const uint64_t an = umma_desc(nbase + L::a + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
                            umma_ss(tmem + (((c + 1) & 1) ? MW_DPB : MW_DP), an, an, id_0, kk > 0);
                        }
                    }
                    if (ahead) umma_commit(bar_dp + ((c + 1) & 1) * 8);
                }
                __syncwarp();
                if (fl & MW_ACTIVE) {
                    ++ncopy;
                    fresh = true;
                }
                MW_ACC(5);
                if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_pfull + (c & 1) * 8, (c >> 1) & 1, status));   // P of this chunk
                if (ok && c > 0) ok = __all_sync(0xffffffffu, mbar_wait(bar_odone, (c - 1) & 1, status));   // D2 is free
                MW_ACC(6);
                if (!ok) break;
                if (lane == 0) {
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const uint64_t ad = umma_desc(sbase + L::pp + (c & 1) * 16384 + kk * 32, 16, 1024);
                        const uint64_t bv = umma_desc(base + L::v + kk * 2048, 8192, 1024);
                        umma_ss(tmem + MW_D2, ad, bv, id_2, kk > 0);
                    }
                    umma_commit(bar_d2);
                }
                __syncwarp();
                MW_ACC(7);
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------ state warps: one thread per TMEM lane (= S row)
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const uint32_t t_lane = tmem + ((uint32_t)(quad * 32) << 16);
        bool ok = true;
        int pubs = 0;                                  // copies published so far; the next one goes to copy pubs & 1
        // Publishes this thread's state row: bf16 copy into shared memory, optionally a raw copy into the saved-state
        // region, and `value * mul` as the state in TMEM.  The value comes from the state in TMEM (src 0), the saved
        // state (src 1), the initial state (src 2, init_row) or is zero (src 3).
        auto publish_state = [&](float mul, int src, const float* init_row, bool save) {
            // copy pubs & 1: MMA 1 of the chunks that read its previous content must be complete
            if (want_o && pubs >= 2) {
                ok = __all_sync(0xffffffffu, mbar_wait(bar_cempty + (pubs & 1) * 8, ((pubs >> 1) - 1) & 1, status));
                if (!ok) return;
            }
            unsigned char* dst = smem + L::sbf + (pubs & 1) * 16384;
#pragma unroll 1
            for (int c0 = 0; c0 < 64; c0 += 32) {
                uint32_t r[32];
                if (src == 2) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(init_row[c0 + i]);
                } else if (src == 3) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = 0u;
                } else {
                    tmem_ld32(t_lane + (src ? MW_BK : MW_S) + c0, r);
                    tmem_ld_wait();
                }
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    uint32_t w4[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        w4[i] = pack_bf16(__uint_as_float(r[cc * 8 + 2 * i]), __uint_as_float(r[cc * 8 + 2 * i + 1]));
                    *reinterpret_cast<uint4*>(dst + swz<128>(row, (c0 >> 3) + cc)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                }
                if (save) tmem_st32(t_lane + MW_BK + c0, r);
                if (mul != 1.f || src != 0) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * mul);
                    tmem_st32(t_lane + MW_S + c0, r);
                }
            }
            tmem_st_wait();
            fence_async_smem();
            if (want_o) mbar_arrive(bar_cfull + (pubs & 1) * 8);
            ++pubs;
        };
        // decay factor of the next update at or after chunk c
        auto next_dec = [&](int c) -> float {
            for (int j = c; j < NT; ++j)
                if (m_fl[j] & MW_ACTIVE) return m_dec[j];
            return 1.f;
        };
        {   // initial state
            const float* init = h0 ? h0 + (((long)b * H + h) * K + row) * V : nullptr;
            publish_state(next_dec(0), init ? 2 : 3, init, (m_fl[0] & MW_SAVE) != 0);
            fence_async_smem();
            tc_fence_before();
            mbar_arrive(bar_sready);
        }
        for (int c = 0; c < NT; ++c) {
            const int fl = m_fl[c];
            MW_T0();
            // once the update of this chunk is complete, publish the state for the next chunk (and pre-apply the next
            // update's decay); after a failed (bounded) wait the remaining work is skipped
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_s3, c & 1, status));
            if (ok) mbar_arrive(bar_empty + (c % L::nstage) * 8);       // MMA 3 is done with the k tile
            if (warp == 2) MW_ACC(8);
            if (ok && (fl & MW_ACTIVE)) {
                tc_fence_after();
                const bool restore = (fl & MW_RESTORE) != 0;
                const bool save = !restore && c + 1 < NT && (m_fl[c + 1] & MW_SAVE) != 0;
                publish_state(next_dec(c + 1), restore ? 1 : 0, nullptr, save);
                fence_async_smem();
            }
            if (ok) {
                tc_fence_before();
                mbar_arrive(bar_sready);
            }
            if (warp == 2) MW_ACC(9);
        }
        if (ok && ht) {
            // every update's decay was pre-applied except after the last one: TMEM holds the final state
            tc_fence_after();
            float* hrow = ht + (((long)b * H + h) * K + row) * V;
#pragma unroll 1
            for (int c0 = 0; c0 < 64; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(t_lane + MW_S + c0, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    *reinterpret_cast<float4*>(hrow + c0 + i) = make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]),
                                                                           __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
            }
        }
    } else if (warp == 8 || warp == 9) {
        // ------------------------------------------------------------ token warps: v~ = v e^{min(g_last - g, 0)}
        const int tr = (warp - 8) * 32 + lane;            // token row inside the chunk
        bool ok = true;
        auto stage_v = [&](int c, float gg) {             // chunk c into buffer c & 1 (the arrival follows separately)
            const int stg = c % L::nstage;
            ok = __all_sync(0xffffffffu, mbar_wait(bar_full + stg * 8, (c / L::nstage) & 1, status));
            if (!ok) return;
            const float f2 = __expf(fminf(m_gl[c] - gg, 0.f));
            const unsigned char* vt = smem + stg * L::stage + L::v;
#pragma unroll
            for (int cc = 0; cc < 8; ++cc) {
                const uint32_t off = swz<128>(tr, cc);
                const uint4 vx = *reinterpret_cast<const uint4*>(vt + off);
                const uint32_t* vw = reinterpret_cast<const uint32_t*>(&vx);
                uint32_t b4[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 vf = unpack_bf16(vw[i]);
                    b4[i] = pack_bf16(vf.x * f2, vf.y * f2);
                }
                *reinterpret_cast<uint4*>(smem + L::vs + (c & 1) * 8192 + off) = make_uint4(b4[0], b4[1], b4[2], b4[3]);
            }
            fence_async_smem();
        };
        float g_n1 = load_g(0, tr), g_n2 = NT > 1 ? load_g(1, tr) : 0.f;
        stage_v(0, g_n1);
        if (ok) mbar_arrive(bar_pv);
        for (int c = 0; c < NT; ++c) {
            g_n1 = g_n2;                                                  // g of chunk c + 1
            if (c + 2 < NT) g_n2 = load_g(c + 2, tr);                     // consumed in the next iteration
            // The tile of the NEXT chunk, off the serial chain.  Its arrival waits until the update of this chunk is
            // complete: the MMA warp has then consumed this chunk's phase of the barrier.
            MW_T0();
            if (ok && c + 1 < NT) stage_v(c + 1, g_n1);
            if (warp == 8) MW_ACC(10);
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_s3, c & 1, status));
            if (ok && c + 1 < NT) mbar_arrive(bar_pv);
            if (warp == 8) MW_ACC(11);
        }
    } else if (want_o) {
        // ------------------------------------------------------------ q warps: rows 64-127, 32 columns each
        const int quad = warp & 3;                        // 2 or 3
        const int cb = warp >= 10 ? 32 : 0;
        const int row = quad * 32 + lane, tr = row - 64;
        const uint32_t t_lane = tmem + ((uint32_t)(quad * 32) << 16);
        bool ok = true;
        // P = tril(q k^T e^{g_i - g_j}) of chunk c as the bf16 A operand of P v, into P tile c & 1.  The 128 threads
        // first exchange the g values of the chunk's tokens (two buffers: a thread that passed the next barrier has
        // finished reading this one).
        auto build_p = [&](int c, float gg) {
            MW_T0();
            if (cb == 0) s_g[(c & 1) * 64 + tr] = gg;
            asm volatile("bar.sync 2, 128;" ::: "memory");
            if (warp == 6) MW_ACC(12);
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_dp + (c & 1) * 8, (c >> 1) & 1, status));
            if (warp == 6) MW_ACC(13);
            if (!ok) return;
            tc_fence_after();
            uint32_t r[32];
            tmem_ld32(t_lane + ((c & 1) ? MW_DPB : MW_DP) + cb, r);
            tmem_ld_wait();
            const float* sg = s_g + (c & 1) * 64;
            unsigned char* dst = smem + L::pp + (c & 1) * 16384;
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                uint32_t w4[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int j0 = cb + cc * 8 + 2 * i;
                    // no branches: the exponent is clamped (it is <= 0 wherever the mask keeps the product)
                    const float e0 = __expf(fminf(gg - sg[j0], 0.f)), e1 = __expf(fminf(gg - sg[j0 + 1], 0.f));
                    const float k0 = (j0 <= tr) ? 1.f : 0.f, k1 = (j0 + 1 <= tr) ? 1.f : 0.f;
                    w4[i] = pack_bf16(__uint_as_float(r[cc * 8 + 2 * i]) * e0 * k0, __uint_as_float(r[cc * 8 + 2 * i + 1]) * e1 * k1);
                }
                *reinterpret_cast<uint4*>(dst + swz<128>(row, (cb >> 3) + cc)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
            }
            fence_async_smem();
            tc_fence_before();
            mbar_arrive(bar_pfull + (c & 1) * 8);
            if (warp == 6) MW_ACC(14);
        };
        float g_cur = load_g(0, tr), g_n1 = NT > 1 ? load_g(1, tr) : 0.f, g_n2 = 0.f;
        int ncopy = 0;                                    // copy of the state that the current chunk reads: ncopy & 1
        build_p(0, g_cur);
        for (int c = 0; c < NT; ++c) {
            const int valid = min(64, T - c * 64);
            const long tok0 = (long)b * T + (long)c * 64;
            if (c + 2 < NT) g_n2 = load_g(c + 2, tr);                     // consumed in the next iteration
            if (c + 1 < NT) build_p(c + 1, g_n1);                         // runs to its barrier also after a failed wait
            MW_T0();
            // o = scale (e^{g+carry} q S + P v): MMA 2 complete means MMA 1 of the chunk is complete as well
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_d2, c & 1, status));
            if (warp == 6) MW_ACC(15);
            if (ok) {
                // every product that read the tile stage of this chunk, or (if an update follows) this copy of the
                // state, is complete
                mbar_arrive(bar_empty + (c % L::nstage) * 8);
                if (m_fl[c] & MW_ACTIVE) mbar_arrive(bar_cempty + (ncopy & 1) * 8);
                tc_fence_after();
                const float fq = __expf(g_cur + m_carry[c]);
                __nv_bfloat16* orow = o + ((tok0 + tr) * H + h) * V;
                uint32_t r1[32], r2[32];
                tmem_ld32(t_lane + ((c & 1) ? MW_D1B : MW_D1) + cb, r1);
                tmem_ld32(t_lane + MW_D2 + cb, r2);
                tmem_ld_wait();
                if (tr < valid) {
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        uint32_t w4[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int e = cc * 8 + 2 * i;
                            w4[i] = pack_bf16(scale * (fq * __uint_as_float(r1[e]) + __uint_as_float(r2[e])),
                                              scale * (fq * __uint_as_float(r1[e + 1]) + __uint_as_float(r2[e + 1])));
                        }
                        *reinterpret_cast<uint4*>(orow + cb + cc * 8) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                    }
                }
                tc_fence_before();
                mbar_arrive(bar_odone);
            }
            if (warp == 6) MW_ACC(16);
            if (m_fl[c] & MW_ACTIVE) ++ncopy;
            g_cur = g_n1;
            g_n1 = g_n2;
        }
    }
    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, MW_TMEM_COLS);
}

}  // namespace natsl

#ifdef NATSL_MW_TIMING
extern "C" int natsl_mw_timing(long long* out, int reset) {
    long long z[32] = {0};
    if (out && cudaMemcpyFromSymbol(out, natsl::mw_t, sizeof(z)) != cudaSuccess) return -1;
    if (reset && cudaMemcpyToSymbol(natsl::mw_t, z, sizeof(z)) != cudaSuccess) return -1;
    return 0;
}
#endif

extern "C" int natsl_mamba_walk_fused(const void* q, const void* k, const void* v, const float* gcs,
                                      const int32_t* types_i, const int32_t* indices, const int32_t* n_blocks,
                                      const float* h0, void* o, float* ht, int B, int T, int H, int HN, int K, int V,
                                      int nbs, float scale, int flags, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(k && v && gcs && types_i && indices && n_blocks, NATSL_ERR_NULL, "natsl_mamba_walk_fused: null pointer");
    NATSL_REQUIRE((o && q) || (!o && ht), NATSL_ERR_NULL,
                  "natsl_mamba_walk_fused: o needs q; without o the final state ht must be asked for");
    NATSL_REQUIRE(B > 0 && T > 0 && H > 0 && HN > 0 && H % HN == 0, NATSL_ERR_BAD_SHAPE, "natsl_mamba_walk_fused: bad shape");
    NATSL_REQUIRE(K == 128 && V == 64 && nbs >= 64 && nbs % 64 == 0, NATSL_ERR_UNSUPPORTED,
                  "natsl_mamba_walk_fused: built for K = 128, V = 64 and nats_block_size a multiple of 64 (got K=%d V=%d "
                  "nbs=%d); use natsl_linear_fwd_h + natsl_linear_fwd_o", K, V, nbs);
    NATSL_REQUIRE((T + 63) / 64 <= MW_MAX_NT, NATSL_ERR_TOO_LARGE, "natsl_mamba_walk_fused: T <= 65536");
    NATSL_REQUIRE(H <= 65535 && B <= 65535, NATSL_ERR_TOO_LARGE, "natsl_mamba_walk_fused: B, H <= 65535");
    auto kern = mamba_walk_tc_kernel;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, MwSmem::total);
    if (e != cudaSuccess) {
        set_error("natsl_mamba_walk_fused: cannot reserve %d B of shared memory (%s)", MwSmem::total, cudaGetErrorString(e));
        return NATSL_ERR_CUDA;
    }
    CUtensorMap mq, mk, mv;
    int rc = encode_bthd_map(&mk, k, B, T, H, K, 64, "natsl_mamba_walk_fused(k)");
    if (rc == NATSL_OK) rc = encode_bthd_map(&mv, v, B, T, H, V, 64, "natsl_mamba_walk_fused(v)");
    if (rc == NATSL_OK && o) rc = encode_bthd_map(&mq, q, B, T, H, K, 64, "natsl_mamba_walk_fused(q)");
    if (!o) mq = mk;
    int* status = nullptr;
    if (rc == NATSL_OK) rc = status_word_ptr(&status);
    if (rc != NATSL_OK) return rc;
    const int TN = (T + nbs - 1) / nbs;
    dim3 grid(H, B);
    kern<<<grid, MW_THREADS, MwSmem::total, reinterpret_cast<cudaStream_t>(stream)>>>(
        mq, mk, mv, gcs, types_i, indices, n_blocks, h0, reinterpret_cast<__nv_bfloat16*>(o), ht, T, H, HN, TN, nbs, scale,
        (flags & NATSL_FLAG_DECAY_SKIPPED) ? 1 : 0, (flags & NATSL_FLAG_NO_TRAILING_QUIRK) ? 0 : 1, status);
    return check_launch("natsl_mamba_walk_fused");
}
