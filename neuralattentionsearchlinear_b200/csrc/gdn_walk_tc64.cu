// Gated-delta-rule recurrence AND chunk output in one walk on the 5th-generation tensor cores, with the value
// dimension split over two CTAs (head dims K = V = 128, nats_block_size = 64): one CTA per (batch, head, half of
// the value columns) walks the 64-token chunks in order; its K x 64 slice of the state lives in TMEM (fp32) and is
// never written to global memory.  Same math as gdn_walk_tc.cu (every product is independent per value column);
// the difference is the footprint: 256 TMEM columns and about 107 KB of shared memory, so two of these CTAs -- or
// one of them and one attention CTA -- share an SM, and the serial chain of a chunk moves half the TMEM data per
// thread.  Tiles are single-buffered with one "full" barrier each: [w;q] is reloaded as soon as the first product
// of the chunk has completed, u once v' has been formed, k once the state update has completed, so the loads of
// chunk c+1 still run under the chain of chunk c.  Per chunk c
// (S = state the chunk reads, carry = decay of the skipped blocks before it):
//     [w S ; q S]       one stacked 128-row A operand [w ; q] against S (bf16 copy in shared memory)   (MMA 1)
//     v' = u - e^{carry} w S                                                                           (warps, from TMEM)
//     o  = scale (rstd_q e^{g+carry} q S + P v')      P = tril(qn kn^T e^{g_i-g_j}) from the prep kernel   (MMA 2 + warps)
//     S <- e^{g_last+carry} S + k^T (v' rstd_k e^{g_last-g})       only if the block is selected        (MMA 3)
// which is src/nats/ops/common/chunk_delta_h.py:189-324 (recurrence) fused with
// src/nats/ops/common/chunk_o.py:124-215 (output) and the carry of src/nats/ops/utils/cumsum.py:85-133.
// The decay of the state is applied when the state is copied to shared memory for the next chunk
// (one TMEM pass per update: bf16 copy out, multiply by the next update's decay, write back), so the
// accumulating MMA 3 needs no separate rescale.  P is padded to 128 rows (rows 0-63 zero) so that
// P v' lands in the TMEM lanes of the q rows.
// Warp roles: warp 0 TMA producer, warp 1 MMA issuer, warps 2-9 two threads per TMEM lane (32 columns each).  All mbarrier waits are bounded (status word +
// clean teardown on expiry).
#include "tc_common.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

constexpr int WH_THREADS = 320;
constexpr int WH_EPI = 256;
constexpr int WH_VB = 64;                                                // value columns per CTA
constexpr uint32_t WH_TMEM_COLS = 256;
constexpr uint32_t WH_S = 0, WH_D1 = 64, WH_D2 = 128, WH_D1B = 192;      // TMEM column offsets (D1 double-buffered)
constexpr int WH_MAX_NT = 128;                                          // chunks per sequence (T <= 8192)

struct WhSmem {
    static constexpr int wq = 0;                          // [w;q]: 2 sub-tiles [128][64]                  32 KB
    static constexpr int k = 32768;                       // k: 2 sub-tiles [64 tok][64]                   16 KB
    static constexpr int u = 49152;                       // u: [64 tok][64 v-cols]                          8 KB
    static constexpr int sbf = 57344;                     // S bf16: [128 k-rows][64 v-cols]                16 KB
    static constexpr int vp = sbf + 16384;                // v'  : [64 tok][64]                              8 KB
    static constexpr int vs = vp + 8192;                  // v'' : same layout                               8 KB
    static constexpr int pp = vs + 8192;                  // P padded to 128 rows: [128][64 tok]            16 KB
    static constexpr int meta = pp + 16384;               // per chunk: carry, dec, g_last (float), sel (int)
    static constexpr int bars = meta + 4 * 4 * WH_MAX_NT;
    static constexpr int total = bars + 256;
};

template <bool kDummy>
__global__ void __launch_bounds__(WH_THREADS, 2)
gdn_walk_half_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_q,
                   const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_u,
                   const __grid_constant__ CUtensorMap map_p, const float* __restrict__ gcs,
                   const float* __restrict__ krstd, const float* __restrict__ qrstd, const int* __restrict__ types_i,
                   const int* __restrict__ indices, const int* __restrict__ n_blocks, const float* __restrict__ h0,
                   __nv_bfloat16* __restrict__ o, float* __restrict__ ht, int T, int H, int HN, int TN, float scale,
                   int decay, int trailing_quirk, int* status) {
    using L = WhSmem;
    constexpr int K = 128, V = 128, VB = WH_VB;
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t sbase = smem_u32(smem);
    if ((sbase & 1023u) != 0) {
        if (tid == 0) atomicExch(status, 2);
        return;
    }
    const int h = blockIdx.x >> 1, vhalf = blockIdx.x & 1, b = blockIdx.y;
    const int v0 = vhalf * WH_VB;                         // first value column of this CTA
    const int hn = h / (H / HN);
    const int NT = (T + 63) / 64;
    float* m_carry = reinterpret_cast<float*>(smem + L::meta);
    float* m_dec = m_carry + WH_MAX_NT;
    float* m_gl = m_dec + WH_MAX_NT;
    int* m_sel = reinterpret_cast<int*>(m_gl + WH_MAX_NT);
    const uint32_t bar0 = sbase + L::bars;
    // barriers: fwq / fk / fu one "tile landed" barrier per tile; pfull / pfree the P tile; d1 (MMA 1 done: [w;q] may be
    // reloaded); pv (v', v'' written by the w lanes: u may be reloaded); d2 (MMA 2 done); s3 (MMA 3 done: k may be
    // reloaded); sready (state copy published); odone (output rows read from TMEM).  Every barrier completes one phase
    // per chunk.
    const uint32_t bar_fwq = bar0, bar_fk = bar0 + 8, bar_fu = bar0 + 16, bar_pfull = bar0 + 32, bar_pfree = bar0 + 40,
                   bar_d1 = bar0 + 48, bar_pv = bar0 + 56, bar_d2 = bar0 + 64, bar_s3 = bar0 + 72, bar_sready = bar0 + 80,
                   bar_odone = bar0 + 88;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::bars + 128);

    if (tid == 0) {
        mbar_init(bar_fwq, 1);
        mbar_init(bar_fk, 1);
        mbar_init(bar_fu, 1);
        mbar_init(bar_pfull, 1);
        mbar_init(bar_pfree, 1);
        mbar_init(bar_d1, 1);
        mbar_init(bar_pv, WH_EPI / 2);
        mbar_init(bar_d2, 1);
        mbar_init(bar_s3, 1);
        mbar_init(bar_sready, WH_EPI);
        mbar_init(bar_odone, WH_EPI / 2);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), WH_TMEM_COLS);
    // ---- per-chunk metadata: selection, carry before the chunk, decay factor of the chunk's update
    for (int c = tid; c < NT; c += WH_THREADS) {
        m_sel[c] = types_i[(((long)b * TN + c) * HN + hn) * 2 + 1] != 0;
        m_gl[c] = gcs[((long)b * T + min(c * 64 + 63, T - 1)) * H + h];
    }
    // the P operand is padded to 128 rows; rows 0-63 stay zero
    for (int i = tid; i < 8192 / 16; i += WH_THREADS) reinterpret_cast<uint4*>(smem + L::pp)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    if (tid == 0) {
        const int nsel = n_blocks[((long)b * HN + hn) * 2 + 1];
        const int last_sel = nsel > 0 ? indices[(((long)b * TN + (nsel - 1)) * HN + hn) * 2 + 1] : -1;
        float carry = 0.f;
        for (int c = 0; c < NT; ++c) {
            const float gl = m_gl[c];
            m_carry[c] = carry;
            if (m_sel[c]) {
                m_dec[c] = __expf(gl + carry);
                carry = 0.f;
            } else {
                m_dec[c] = 1.f;
                if (decay && (!trailing_quirk || c < last_sel)) carry += gl;
            }
        }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            prefetch_tensormap(&map_w); prefetch_tensormap(&map_q); prefetch_tensormap(&map_k);
            prefetch_tensormap(&map_u); prefetch_tensormap(&map_p);
        }
        for (int c = 0; c < NT; ++c) {
            const int t0 = c * 64;
            // [w;q]: free once the first product of the previous chunk has completed
            if (c >= 1) {
                bool ok = mbar_wait(bar_d1, (c - 1) & 1, status);
                if (!__all_sync(0xffffffffu, ok)) break;
            }
            if (lane == 0) {
                mbar_expect_tx(bar_fwq, 32768);
#pragma unroll
                for (int sub = 0; sub < 2; ++sub) {
                    tma_load_4d(sbase + L::wq + sub * 16384, &map_w, sub * 64, h, t0, b, bar_fwq);          // rows 0-63
                    tma_load_4d(sbase + L::wq + sub * 16384 + 8192, &map_q, sub * 64, h, t0, b, bar_fwq);   // rows 64-127
                }
            }
            // u: free once the w lanes have formed v' of the previous chunk
            if (c >= 1) {
                bool ok = mbar_wait(bar_pv, (c - 1) & 1, status);
                if (!__all_sync(0xffffffffu, ok)) break;
            }
            if (lane == 0) {
                mbar_expect_tx(bar_fu, 8192);
                tma_load_4d(sbase + L::u, &map_u, v0, h, t0, b, bar_fu);
            }
            // k: free once the state update of the previous chunk has completed
            if (c >= 1) {
                bool ok = mbar_wait(bar_s3, (c - 1) & 1, status);
                if (!__all_sync(0xffffffffu, ok)) break;
            }
            if (lane == 0) {
                mbar_expect_tx(bar_fk, 16384);
#pragma unroll
                for (int sub = 0; sub < 2; ++sub) tma_load_4d(sbase + L::k + sub * 8192, &map_k, sub * 64, h, t0, b, bar_fk);
            }
            if (c >= 1) {
                bool ok = mbar_wait(bar_pfree, (c - 1) & 1, status);       // P of the previous chunk consumed
                if (!__all_sync(0xffffffffu, ok)) break;
            }
            if (lane == 0) {
                mbar_expect_tx(bar_pfull, 8192);
                tma_load_4d(sbase + L::pp + 8192, &map_p, 0, h, t0, b, bar_pfull);                      // rows 64-127
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        constexpr uint32_t id_1 = umma_idesc_bf16(128, VB, true);                        // [w;q] S
        constexpr uint32_t id_2 = umma_idesc_bf16(128, VB, true);                        // P v'
        constexpr uint32_t id_3 = umma_idesc_bf16(128, VB, true) | (1u << 15);           // k^T v'' (A MN-major)
        bool ok = true;
        for (int c = 0; ok && c < NT; ++c) {
            const uint32_t base = sbase;
            ok = __all_sync(0xffffffffu, mbar_wait(bar_fwq, c & 1, status));
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_sready, c & 1, status));
            if (!ok) break;
            const uint32_t d1 = tmem + ((c & 1) ? WH_D1B : WH_D1);
            if (lane == 0) {
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint64_t ad = umma_desc(base + L::wq + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
                    const uint64_t bs = umma_desc(sbase + L::sbf + kk * 2048, 16384, 1024);
                    umma_ss(d1, ad, bs, id_1, kk > 0);
                }
                umma_commit(bar_d1);
            }
            __syncwarp();
            ok = __all_sync(0xffffffffu, mbar_wait(bar_pv, c & 1, status));
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_fk, c & 1, status));
            if (!ok) break;
            if (lane == 0) {
                // the state update first: the next chunk's products wait for it, the output does not
                tc_fence_after();
                if (m_sel[c]) {
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const uint64_t ak = umma_desc(base + L::k + kk * 2048, 8192, 1024);
                        const uint64_t bv = umma_desc(sbase + L::vs + kk * 2048, 8192, 1024);
                        umma_ss(tmem + WH_S, ak, bv, id_3, 1u);
                    }
                }
                umma_commit(bar_s3);
            }
            __syncwarp();
            ok = __all_sync(0xffffffffu, mbar_wait(bar_pfull, c & 1, status));
            if (ok && c > 0) ok = __all_sync(0xffffffffu, mbar_wait(bar_odone, (c - 1) & 1, status));   // D2 is free
            if (!ok) break;
            if (lane == 0) {
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint64_t ad = umma_desc(sbase + L::pp + kk * 32, 16, 1024);
                    const uint64_t bv = umma_desc(sbase + L::vp + kk * 2048, 8192, 1024);
                    umma_ss(tmem + WH_D2, ad, bv, id_2, kk > 0);
                }
                umma_commit(bar_d2);
                umma_commit(bar_pfree);
            }
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------ two threads per TMEM lane (64 columns each)
        const int quad = warp & 3;
        const int half = (warp - 2) >> 2;
        const int row = quad * 32 + lane;                 // TMEM lane: S row (k index); w row (0-63) or q row (64-127)
        const int cb = half * (VB / 2);                   // this thread's first column (of the CTA's VB)
        const uint32_t t_lane = tmem + ((uint32_t)(quad * 32) << 16);
        const bool is_q = row >= 64;
        const int tr = row & 63;                          // token row inside the chunk
        bool ok = true;

        // copies columns [cb, cb+64) of this lane's S row as bf16 into the shared copy and leaves S * mul in TMEM
        auto publish_state = [&](float mul, const float* init_row) {
#pragma unroll 1
            for (int c0 = cb; c0 < cb + VB / 2; c0 += 32) {
                uint32_t r[32];
                if (init_row) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(init_row[v0 + c0 + i]);
                } else {
                    tmem_ld32(t_lane + WH_S + c0, r);
                    tmem_ld_wait();
                }
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    uint32_t w4[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        w4[i] = pack_bf16(__uint_as_float(r[cc * 8 + 2 * i]), __uint_as_float(r[cc * 8 + 2 * i + 1]));
                    const int col = c0 + cc * 8;          // v column of this 16-byte chunk
                    *reinterpret_cast<uint4*>(smem + L::sbf + (col >> 6) * 16384 + swz<128>(row, (col & 63) >> 3)) =
                        make_uint4(w4[0], w4[1], w4[2], w4[3]);
                }
                if (mul != 1.f || init_row) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * mul);
                    tmem_st32(t_lane + WH_S + c0, r);
                }
            }
            tmem_st_wait();
        };
        // decay factor of the next update at or after chunk c
        auto next_dec = [&](int c) -> float {
            for (int j = c; j < NT; ++j)
                if (m_sel[j]) return m_dec[j];
            return 1.f;
        };
        {   // initial state
            const float* init = h0 ? h0 + (((long)b * H + h) * K + row) * V : nullptr;
            if (init) {
                publish_state(next_dec(0), init);
            } else {
#pragma unroll 1
                for (int c0 = cb; c0 < cb + VB / 2; c0 += 32) {
                    uint32_t r[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = 0u;
                    tmem_st32(t_lane + WH_S + c0, r);
                }
                tmem_st_wait();
                for (int i = 0; i < VB / 16; ++i)
                    *reinterpret_cast<uint4*>(smem + L::sbf + swz<128>(row, (cb >> 3) + i)) = make_uint4(0, 0, 0, 0);
            }
            fence_async_smem();
            tc_fence_before();
            mbar_arrive(bar_sready);
        }
        // per-row scalars of the chunk: cumsum g and the l2 norm factor (k rows for w lanes, q rows for q lanes)
        auto load_scalars = [&](int c, float& gg, float& rr) {
            const int valid = min(64, T - c * 64);
            const long tok0 = (long)b * T + (long)c * 64;
            gg = gcs[(tok0 + min(tr, valid - 1)) * H + h];
            const float* rs = is_q ? qrstd : krstd;
            rr = (tr < valid) ? rs[(tok0 + tr) * H + h] : 0.f;
        };
        float g_cur, r_cur, g_nxt = 0.f, r_nxt = 0.f;
        load_scalars(0, g_cur, r_cur);

        for (int c = 0; c < NT; ++c) {
            const int valid = min(64, T - c * 64);
            const long tok0 = (long)b * T + (long)c * 64;
            unsigned char* stage = smem;
            if (c + 1 < NT) load_scalars(c + 1, g_nxt, r_nxt);          // prefetch; consumed next iteration
            const float carry = m_carry[c];
            const float gl = m_gl[c];
            const bool sel = m_sel[c] != 0;
            const uint32_t t_d1 = t_lane + ((c & 1) ? WH_D1B : WH_D1);
            // After a failed (bounded) wait the remaining work is skipped; the loop still runs to its end.
            // Every lane first sees MMA 1 of this chunk complete: it was issued behind the previous phase of the
            // "state published" barrier, so no thread can arrive on that barrier twice within one phase.
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_d1, c & 1, status));
            if (!is_q) {
                // ---- w lanes: v' = u - e^{carry} w S ; v'' = v' rstd_k e^{g_last - g}
                if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_fu, c & 1, status));
                if (ok) {
                    tc_fence_after();
                    const float ec = __expf(carry);
                    const float f2 = r_cur * __expf(fminf(gl - g_cur, 80.f));
#pragma unroll 1
                    for (int c0 = cb; c0 < cb + VB / 2; c0 += 32) {
                        uint32_t r[32];
                        tmem_ld32(t_d1 + c0, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int cc = 0; cc < 4; ++cc) {
                            const int col = c0 + cc * 8;
                            const uint32_t off = (col >> 6) * 8192 + swz<128>(tr, (col & 63) >> 3);
                            const uint4 ux = *reinterpret_cast<const uint4*>(stage + L::u + off);
                            const uint32_t* uw = reinterpret_cast<const uint32_t*>(&ux);
                            uint32_t a4[4], b4[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float2 uf = unpack_bf16(uw[i]);
                                const float v0 = uf.x - ec * __uint_as_float(r[cc * 8 + 2 * i]);
                                const float v1 = uf.y - ec * __uint_as_float(r[cc * 8 + 2 * i + 1]);
                                a4[i] = pack_bf16(v0, v1);
                                b4[i] = pack_bf16(v0 * f2, v1 * f2);
                            }
                            *reinterpret_cast<uint4*>(smem + L::vp + off) = make_uint4(a4[0], a4[1], a4[2], a4[3]);
                            *reinterpret_cast<uint4*>(smem + L::vs + off) = make_uint4(b4[0], b4[1], b4[2], b4[3]);
                        }
                    }
                    fence_async_smem();
                    tc_fence_before();
                    mbar_arrive(bar_pv);
                }
            }
            // ---- every lane: publish the updated state for the next chunk (and pre-apply the next update's decay).
            // This is the serial chain of the walk; the output rows below are read after it.
            if (ok && sel) {
                ok = __all_sync(0xffffffffu, mbar_wait(bar_s3, c & 1, status));
                if (ok) {
                    tc_fence_after();
                    publish_state(next_dec(c + 1), nullptr);
                    fence_async_smem();
                }
            }
            if (ok) {
                tc_fence_before();
                mbar_arrive(bar_sready);
            }
            if (is_q) {
                // ---- q lanes: o = scale (rstd_q e^{g+carry} q S + P v'), off the chain (D1 is double-buffered, D2 is
                // released by the arrival below)
                if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_d2, c & 1, status));
                if (ok) {
                    tc_fence_after();
                    const float fq = r_cur * __expf(g_cur + carry);
                    __nv_bfloat16* orow = o + ((tok0 + tr) * H + h) * V + v0;
#pragma unroll 1
                    for (int c0 = cb; c0 < cb + VB / 2; c0 += 32) {
                        uint32_t r1[32], r2[32];
                        tmem_ld32(t_d1 + c0, r1);
                        tmem_ld32(t_lane + WH_D2 + c0, r2);
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
                                *reinterpret_cast<uint4*>(orow + c0 + cc * 8) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                            }
                        }
                    }
                    tc_fence_before();
                    mbar_arrive(bar_odone);
                }
            }
            g_cur = g_nxt;
            r_cur = r_nxt;
        }
        if (ok && ht) {
            // every update's decay was pre-applied except after the last one: TMEM holds the final state
            tc_fence_after();
            float* hrow = ht + (((long)b * H + h) * K + row) * V + v0;
#pragma unroll 1
            for (int c0 = cb; c0 < cb + VB / 2; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(t_lane + WH_S + c0, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    *reinterpret_cast<float4*>(hrow + c0 + i) = make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]),
                                                                           __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
            }
        }
    }
    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, WH_TMEM_COLS);
}

}  // namespace natsl

extern "C" int natsl_gdn_walk_fused_vsplit(const void* q, const void* k, const void* w, const void* u, const void* pmat,
                                    const float* gcs, const float* k_rstd, const float* q_rstd, const int32_t* types_i,
                                    const int32_t* indices, const int32_t* n_blocks, const float* h0, void* o, float* ht,
                                    int B, int T, int H, int HN, int K, int V, int nbs, float scale, int flags,
                                    void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(q && k && w && u && pmat && gcs && k_rstd && q_rstd && types_i && indices && n_blocks && o, NATSL_ERR_NULL,
                  "natsl_gdn_walk_fused_vsplit: null pointer");
    NATSL_REQUIRE(B > 0 && T > 0 && H > 0 && HN > 0 && H % HN == 0, NATSL_ERR_BAD_SHAPE, "natsl_gdn_walk_fused_vsplit: bad shape");
    NATSL_REQUIRE(K == 128 && V == 128 && nbs == 64, NATSL_ERR_UNSUPPORTED,
                  "natsl_gdn_walk_fused_vsplit: built for K = V = 128 and nats_block_size = 64 (got K=%d V=%d nbs=%d); use "
                  "natsl_linear_fwd_h + natsl_linear_fwd_o", K, V, nbs);
    NATSL_REQUIRE((T + 63) / 64 <= WH_MAX_NT, NATSL_ERR_TOO_LARGE, "natsl_gdn_walk_fused_vsplit: T <= 8192 (use natsl_gdn_walk_fused)");
    NATSL_REQUIRE(2L * H <= 2147483647L && B <= 65535, NATSL_ERR_TOO_LARGE, "natsl_gdn_walk_fused_vsplit: B <= 65535");
    auto kern = gdn_walk_half_kernel<true>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, WhSmem::total);
    if (e != cudaSuccess) {
        set_error("natsl_gdn_walk_fused_vsplit: cannot reserve %d B of shared memory (%s)", WhSmem::total, cudaGetErrorString(e));
        return NATSL_ERR_CUDA;
    }
    CUtensorMap mw, mq, mk, mu, mp;
    int rc = encode_bthd_map(&mw, w, B, T, H, K, 64, "natsl_gdn_walk_fused_vsplit(w)");
    if (rc == NATSL_OK) rc = encode_bthd_map(&mq, q, B, T, H, K, 64, "natsl_gdn_walk_fused_vsplit(q)");
    if (rc == NATSL_OK) rc = encode_bthd_map(&mk, k, B, T, H, K, 64, "natsl_gdn_walk_fused_vsplit(k)");
    if (rc == NATSL_OK) rc = encode_bthd_map(&mu, u, B, T, H, V, 64, "natsl_gdn_walk_fused_vsplit(u)");   // 64-column boxes
    if (rc == NATSL_OK) rc = encode_bthd_map(&mp, pmat, B, T, H, 64, 64, "natsl_gdn_walk_fused_vsplit(P)");
    int* status = nullptr;
    if (rc == NATSL_OK) rc = status_word_ptr(&status);
    if (rc != NATSL_OK) return rc;
    const int TN = (T + nbs - 1) / nbs;
    dim3 grid(2 * H, B);
    kern<<<grid, WH_THREADS, WhSmem::total, reinterpret_cast<cudaStream_t>(stream)>>>(
        mw, mq, mk, mu, mp, gcs, k_rstd, q_rstd, types_i, indices, n_blocks, h0, reinterpret_cast<__nv_bfloat16*>(o), ht, T, H,
        HN, TN, scale, (flags & NATSL_FLAG_DECAY_SKIPPED) ? 1 : 0, (flags & NATSL_FLAG_NO_TRAILING_QUIRK) ? 0 : 1, status);
    return check_launch("natsl_gdn_walk_fused_vsplit");
}
