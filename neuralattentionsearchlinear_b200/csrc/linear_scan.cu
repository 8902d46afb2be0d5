// Inter-chunk state recurrence of the linear branch ("fwd_h"): one CTA per (batch, head,
// value-column slice) walks the 64-token chunks of the sequence in order, keeps the K x BV
// state in fp32 registers, and for every chunk stores the state that chunk reads.
//
// Gated DeltaNet (src/nats/ops/common/chunk_delta_h.py:189-324):
//     v_new = u - e^{carry} (w S);  S <- e^{g_last+carry} S + k^T (v_new * rstd_k * e^{g_last - g})
// Mamba2/SSD (src/nats/ops/mamba/chunk_h.py:139-218):
//     S <- e^{g_last+carry} S + k^T (v * e^{min(g_last - g, 0)})
// Only chunks of selected blocks update the state; `carry` is the decay accumulated over
// skipped blocks since the last update (src/nats/ops/utils/cumsum.py:85-133), kept as a
// scalar per chunk and written out for the output kernel.  With nats_block_size > 64 the
// sub-chunks of an unselected block update a temporary state which is rolled back at the
// end of the block (the token recurrence of the reference's decode kernel,
// src/nats/ops/gated_delta_rule/fused_recurrent.py:221-228, 276-281).
//
// The two small products per step run on the tensor cores (bf16 operands, fp32 accumulate);
// everything else is a latency-bound serial walk: tiles of the next active chunk are
// prefetched with cp.async while the current one is computed.
#include "common.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

constexpr int SCAN_THREADS = 128;

template <int K, int BV, bool GDN>
struct ScanSmem {
    // Two 64xK tile buffers: [0] receives w_i, [1] receives k_i of the active chunk being processed; each is
    // refilled for the next active chunk as soon as its product is done.  Small u / vector buffers alternate.
    static constexpr int big_bytes = 64 * K * 2;
    static constexpr int u_bytes = 64 * BV * 2;
    static constexpr int vec_bytes = 2 * 64 * 4;
    static constexpr int big = 0;
    static constexpr int ubuf = 2 * big_bytes;           // 2 x ([64][BV] bf16 + gcs[64] + rstd[64])
    static constexpr int sb = ubuf + 2 * (u_bytes + vec_bytes);   // S as bf16 [K][BV]
    static constexpr int v2 = sb + K * BV * 2;           // scaled v_new [64][BV]
    static constexpr int meta = v2 + 64 * BV * 2;        // per chunk: g_last (float), active-list entry (int)
    // then (nats_block_size > 64 only) the fp32 state backup [K][BV]
    static int total(int NT, bool with_save) { return meta + NT * 8 + (with_save ? K * BV * 4 : 0); }
};

__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}

template <int K, int BV, bool GDN>
__global__ void __launch_bounds__(SCAN_THREADS)
linear_scan_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ w,
                   const __nv_bfloat16* __restrict__ u, const float* __restrict__ gcs,
                   const float* __restrict__ krstd, const int* __restrict__ types_i, const int* __restrict__ indices,
                   const int* __restrict__ n_blocks, const float* __restrict__ h0, __nv_bfloat16* __restrict__ hout,
                   float* __restrict__ carry_out, float* __restrict__ ht, int T, int H, int HN, int V, int TN, int nbs,
                   int decay, int trailing_quirk) {
    using L = ScanSmem<K, BV, GDN>;
    constexpr int MT = K / 64;          // 16-row m-tiles of the state per warp
    constexpr int NTL = BV / 8;         // n-tiles
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, q = lane & 3;
    const int vsplit = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int v0 = vsplit * BV;
    const int hn = h / (H / HN);
    const int NT = (T + 63) / 64;
    const int cpb = nbs / 64;

    const int nsel = n_blocks[((long)b * HN + hn) * 2 + 1];
    const int last_sel = nsel > 0 ? indices[(((long)b * TN + (nsel - 1)) * HN + hn) * 2 + 1] : -1;
    const int* sel_p = types_i + ((long)b * TN * HN + hn) * 2 + 1;
    const long sel_stride = (long)HN * 2;

    unsigned char* sb_p = smem + L::sb;
    unsigned char* v2_p = smem + L::v2;
    float* s_gl = reinterpret_cast<float*>(smem + L::meta);          // [NT] g_last per chunk
    int* s_act = reinterpret_cast<int*>(smem + L::meta + NT * 4);    // [NT] bit 31: block selected; low bits: active list
    float* save_p = reinterpret_cast<float*>(smem + L::meta + NT * 8);
    const uint32_t sb = smem_u32(sb_p), v2 = smem_u32(v2_p);

    // ---- per-chunk metadata: decay total, selection flag, and the list of chunks that update the state
    for (int c = tid; c < NT; c += SCAN_THREADS) {
        const int last_tok = min(c * 64 + 63, T - 1);
        s_gl[c] = gcs[((long)b * T + last_tok) * H + h];
        s_act[c] = (sel_p[(long)(c / cpb) * sel_stride] != 0) ? (1 << 31) : 0;
    }
    __syncthreads();
    __shared__ int s_nact;
    if (tid == 0) {
        int n = 0;
        for (int c = 0; c < NT; ++c)
            if (cpb > 1 || (s_act[c] < 0)) {
                s_act[n] = (s_act[n] & (1 << 31)) | c;
                ++n;
            }
        s_nact = n;
    }
    __syncthreads();
    const int n_act = s_nact;
    auto chunk_sel = [&](int c) -> bool { return s_act[c] < 0; };
    auto act_chunk = [&](int i) -> int { return s_act[i] & 0x7FFFFFFF; };

    float S[MT][NTL][4];
    const int krow0 = warp * (K / 4);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NTL; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float val = 0.f;
                if (h0) {
                    int r = krow0 + mt * 16 + gq + ((e >> 1) << 3);
                    int cidx = v0 + nt * 8 + q * 2 + (e & 1);
                    val = h0[(((long)b * H + h) * K + r) * V + cidx];
                }
                S[mt][nt][e] = val;
            }

    // group A of the i-th active chunk: w tile -> big[0], u tile + gcs/rstd rows -> small buffer i & 1;
    // group B: k tile -> big[1].  Each call commits exactly one group (possibly empty).
    auto issue_a = [&](int i) {
        if (i < n_act) {
            const int c = act_chunk(i);
            const int valid = min(64, T - c * 64);
            const long tok0 = (long)b * T + (long)c * 64;
            if (GDN) load_tile_async<64, K, SCAN_THREADS>(smem_u32(smem + L::big), w + (tok0 * H + h) * K, (long)H * K, valid, tid);
            unsigned char* ub = smem + L::ubuf + (i & 1) * (L::u_bytes + L::vec_bytes);
            load_tile_async<64, BV, SCAN_THREADS>(smem_u32(ub), u + (tok0 * H + h) * V + v0, (long)H * V, valid, tid);
            const uint32_t vec = smem_u32(ub + L::u_bytes);
            if (tid < 64) {
                const bool okr = tid < valid;
                cp_async4(vec + tid * 4, gcs + (tok0 + (okr ? tid : 0)) * H + h, okr ? 4 : 0);
            } else if (krstd) {
                const int r = tid - 64;
                const bool okr = r < valid;
                cp_async4(vec + 256 + r * 4, krstd + (tok0 + (okr ? r : 0)) * H + h, okr ? 4 : 0);
            }
        }
        cp_async_commit();
    };
    auto issue_b = [&](int i) {
        if (i < n_act) {
            const int c = act_chunk(i);
            const int valid = min(64, T - c * 64);
            const long tok0 = (long)b * T + (long)c * 64;
            load_tile_async<64, K, SCAN_THREADS>(smem_u32(smem + L::big + L::big_bytes), k + (tok0 * H + h) * K, (long)H * K,
                                                 valid, tid);
        }
        cp_async_commit();
    };
    if (!krstd) {                          // Mamba2: no key normalisation
        for (int i = tid; i < 2 * 64; i += SCAN_THREADS)
            reinterpret_cast<float*>(smem + L::ubuf + (i / 64) * (L::u_bytes + L::vec_bytes) + L::u_bytes)[64 + (i % 64)] = 1.f;
    }
    issue_a(0);
    int ia = 0;                            // index of the next active chunk
    float carry = 0.f, carry_save = 0.f, blk_g = 0.f;
    bool dirty = true;

    for (int c = 0; c < NT; ++c) {
        const int blk = c / cpb, sub = c % cpb;
        const bool sel = chunk_sel(c) ;
        const bool active = cpb > 1 || sel;
        const bool may_carry = decay && (!trailing_quirk || blk < last_sel);
        if (cpb > 1 && sub == 0) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < NTL; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) save_p[((mt * NTL + nt) * 4 + e) * SCAN_THREADS + tid] = S[mt][nt][e];
            carry_save = carry;
            blk_g = 0.f;
        }
        if (dirty) {
            __syncthreads();                   // every warp is done with the k tile of the previous active chunk
            if (GDN || hout) {                 // bf16 copy of the state: read by the w S product and the h store
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int nt = 0; nt < NTL; ++nt) {
                        int r = krow0 + mt * 16 + gq;
                        *reinterpret_cast<uint32_t*>(sb_p + swz<BV * 2>(r, nt) + q * 4) = pack_bf16(S[mt][nt][0], S[mt][nt][1]);
                        *reinterpret_cast<uint32_t*>(sb_p + swz<BV * 2>(r + 8, nt) + q * 4) =
                            pack_bf16(S[mt][nt][2], S[mt][nt][3]);
                    }
                __syncthreads();
            }
            dirty = false;
        }
        if (hout) store_tile<K, BV, SCAN_THREADS>(sb_p, hout + ((((long)b * NT + c) * H + h) * K) * V + v0, V, K, tid);
        if (carry_out && vsplit == 0 && tid == 0) carry_out[((long)b * NT + c) * H + h] = carry;
        const float gl = s_gl[c];
        blk_g += gl;

        if (active) {
            // big[1] was last read by the k^T product of the previous active chunk, before the barriers above
            issue_b(ia);
            cp_async_wait<1>();            // group A of this chunk has landed (group B may still be in flight)
            __syncthreads();
            unsigned char* ub = smem + L::ubuf + (ia & 1) * (L::u_bytes + L::vec_bytes);
            const uint32_t ws = smem_u32(smem + L::big), ks = smem_u32(smem + L::big + L::big_bytes);
            const unsigned char* us_p = ub;
            const float* vec = reinterpret_cast<const float*>(ub + L::u_bytes);
            const int r0 = warp * 16;
            float acc[NTL][4];
#pragma unroll
            for (int nt = 0; nt < NTL; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
            if (GDN) {
#pragma unroll
                for (int kk = 0; kk < K / 16; ++kk) {
                    uint32_t a[4];
                    load_a<K * 2>(ws, r0, kk * 16, lane, a);
#pragma unroll
                    for (int p = 0; p < NTL / 2; ++p) {
                        uint32_t bb[4];
                        load_b_kn<BV * 2>(sb, kk * 16, p * 16, lane, bb);
                        mma_bf16(acc[2 * p], a, bb[0], bb[1]);
                        mma_bf16(acc[2 * p + 1], a, bb[2], bb[3]);
                    }
                }
            }
            const float ec = __expf(carry);
            const int ra = r0 + gq, rb = ra + 8;
            // rows past the end of a ragged last chunk have zero k/u; their (zero-filled) cumsum only has to stay finite
            float fa, fb;
            if (GDN) {
                fa = vec[64 + ra] * __expf(fminf(gl - vec[ra], 80.f));
                fb = vec[64 + rb] * __expf(fminf(gl - vec[rb], 80.f));
            } else {
                fa = vec[64 + ra] * __expf(fminf(gl - vec[ra], 0.f));
                fb = vec[64 + rb] * __expf(fminf(gl - vec[rb], 0.f));
            }
#pragma unroll
            for (int nt = 0; nt < NTL; ++nt) {
                float2 ua = unpack_bf16(*reinterpret_cast<const uint32_t*>(us_p + swz<BV * 2>(ra, nt) + q * 4));
                float2 ub = unpack_bf16(*reinterpret_cast<const uint32_t*>(us_p + swz<BV * 2>(rb, nt) + q * 4));
                float va0 = ua.x - ec * acc[nt][0], va1 = ua.y - ec * acc[nt][1];
                float vb0 = ub.x - ec * acc[nt][2], vb1 = ub.y - ec * acc[nt][3];
                *reinterpret_cast<uint32_t*>(v2_p + swz<BV * 2>(ra, nt) + q * 4) = pack_bf16(va0 * fa, va1 * fa);
                *reinterpret_cast<uint32_t*>(v2_p + swz<BV * 2>(rb, nt) + q * 4) = pack_bf16(vb0 * fb, vb1 * fb);
            }
            cp_async_wait<0>();            // k tile of this chunk
            __syncthreads();               // v2 and k visible; every warp is done with w, u of this chunk
            issue_a(ia + 1);
            const float dec = __expf(gl + carry);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < NTL; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) S[mt][nt][e] *= dec;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                uint32_t bb[NTL / 2][4];
#pragma unroll
                for (int p = 0; p < NTL / 2; ++p) load_b_kn<BV * 2>(v2, kk * 16, p * 16, lane, bb[p]);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    uint32_t a[4];
                    load_a_t<K * 2>(ks, krow0 + mt * 16, kk * 16, lane, a);
#pragma unroll
                    for (int p = 0; p < NTL / 2; ++p) {
                        mma_bf16(S[mt][2 * p], a, bb[p][0], bb[p][1]);
                        mma_bf16(S[mt][2 * p + 1], a, bb[p][2], bb[p][3]);
                    }
                }
            }
            carry = 0.f;
            ++ia;
            dirty = true;
        } else if (may_carry) {
            carry += gl;
        }
        if (cpb > 1 && (sub == cpb - 1 || c == NT - 1) && !sel) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < NTL; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) S[mt][nt][e] = save_p[((mt * NTL + nt) * 4 + e) * SCAN_THREADS + tid];
            carry = carry_save + (may_carry ? blk_g : 0.f);
            dirty = true;
        }
    }
    cp_async_wait<0>();
    if (ht) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NTL; ++nt) {
                int r = krow0 + mt * 16 + gq;
                int cidx = v0 + nt * 8 + q * 2;
                float* p = ht + (((long)b * H + h) * K + r) * V + cidx;
                *reinterpret_cast<float2*>(p) = make_float2(S[mt][nt][0], S[mt][nt][1]);
                *reinterpret_cast<float2*>(p + 8L * V) = make_float2(S[mt][nt][2], S[mt][nt][3]);
            }
    }
}

template <int K, int BV, bool GDN>
static int launch_scan(const void* k, const void* w, const void* u, const float* gcs, const float* krstd,
                       const int* types_i, const int* indices, const int* n_blocks, const float* h0, void* hout,
                       float* carry, float* ht, int B, int T, int H, int HN, int V, int nbs, int decay, int quirk,
                       cudaStream_t st) {
    using L = ScanSmem<K, BV, GDN>;
    auto kern = linear_scan_kernel<K, BV, GDN>;
    const int NT = (T + 63) / 64;
    const int smem = L::total(NT, nbs > 64);
    if (smem > 227 * 1024) {
        set_error("natsl_linear_fwd_h: T=%d needs %d B of shared memory for the per-chunk metadata (max %d)", T, smem,
                  227 * 1024);
        return NATSL_ERR_TOO_LARGE;
    }
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
        set_error("natsl_linear_fwd_h: cannot reserve %d B of shared memory (%s)", smem, cudaGetErrorString(e));
        return NATSL_ERR_CUDA;
    }
    const int TN = (T + nbs - 1) / nbs;
    dim3 grid(V / BV, H, B);
    kern<<<grid, SCAN_THREADS, smem, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(k), reinterpret_cast<const __nv_bfloat16*>(w),
        reinterpret_cast<const __nv_bfloat16*>(u), gcs, krstd, types_i, indices, n_blocks, h0,
        reinterpret_cast<__nv_bfloat16*>(hout), carry, ht, T, H, HN, V, TN, nbs, decay, quirk);
    return check_launch("natsl_linear_fwd_h");
}

}  // namespace natsl

extern "C" int natsl_linear_fwd_h(int rule, const void* k, const void* w, const void* u, const float* gcs,
                                  const float* k_rstd, const int32_t* types_i, const int32_t* indices,
                                  const int32_t* n_blocks, const float* h0, void* h, float* carry, float* ht, int B,
                                  int T, int H, int HN, int K, int V, int nbs, int flags, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(k && u && gcs && types_i && indices && n_blocks, NATSL_ERR_NULL, "natsl_linear_fwd_h: null pointer");
    NATSL_REQUIRE((h && carry) || ((!h && !carry) && ht), NATSL_ERR_NULL,
                  "natsl_linear_fwd_h: h and carry are given together, or both NULL with ht set");
    NATSL_REQUIRE(rule == NATSL_RULE_GDN || rule == NATSL_RULE_MAMBA, NATSL_ERR_UNSUPPORTED,
                  "natsl_linear_fwd_h: unknown rule %d", rule);
    NATSL_REQUIRE(rule != NATSL_RULE_GDN || w, NATSL_ERR_NULL, "natsl_linear_fwd_h: w is required for the delta rule");
    NATSL_REQUIRE(B > 0 && T > 0 && H > 0 && HN > 0 && H % HN == 0, NATSL_ERR_BAD_SHAPE,
                  "natsl_linear_fwd_h: bad shape B=%d T=%d H=%d HN=%d", B, T, H, HN);
    NATSL_REQUIRE(H <= 65535 && B <= 65535, NATSL_ERR_TOO_LARGE, "natsl_linear_fwd_h: B and H must be <= 65535");
    NATSL_REQUIRE(nbs >= 64 && nbs % 64 == 0, NATSL_ERR_UNSUPPORTED,
                  "natsl_linear_fwd_h: nats_block_size must be a multiple of 64 (got %d)", nbs);
    NATSL_REQUIRE(V % 32 == 0, NATSL_ERR_UNSUPPORTED, "natsl_linear_fwd_h: V must be a multiple of 32 (got %d)", V);
    const int decay = (flags & NATSL_FLAG_DECAY_SKIPPED) ? 1 : 0;
    const int quirk = (flags & NATSL_FLAG_NO_TRAILING_QUIRK) ? 0 : 1;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define NATSL_SCAN_ARGS k, w, u, gcs, k_rstd, types_i, indices, n_blocks, h0, h, carry, ht, B, T, H, HN, V, nbs, decay, quirk, st
    if (rule == NATSL_RULE_GDN) {
        if (K == 64) return launch_scan<64, 32, true>(NATSL_SCAN_ARGS);
        if (K == 128) return launch_scan<128, 32, true>(NATSL_SCAN_ARGS);
    } else {
        if (K == 64) return launch_scan<64, 32, false>(NATSL_SCAN_ARGS);
        if (K == 128) return launch_scan<128, 32, false>(NATSL_SCAN_ARGS);
    }
#undef NATSL_SCAN_ARGS
    set_error("natsl_linear_fwd_h: unsupported key dim K=%d (64 or 128)", K);
    return NATSL_ERR_UNSUPPORTED;
}
