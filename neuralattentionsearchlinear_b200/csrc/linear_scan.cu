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
    static constexpr int w_bytes = GDN ? 64 * K * 2 : 0;
    static constexpr int k_bytes = 64 * K * 2;
    static constexpr int u_bytes = 64 * BV * 2;
    static constexpr int vec_bytes = 2 * 64 * 4;
    static constexpr int stage = w_bytes + k_bytes + u_bytes + vec_bytes;
    static constexpr int sb = 2 * stage;                 // S as bf16 [K][BV]
    static constexpr int v2 = sb + K * BV * 2;           // scaled v_new [64][BV]
    static constexpr int save = v2 + 64 * BV * 2;        // fp32 state backup (nats_block_size > 64 only)
    static constexpr int total = save;
    static constexpr int total_with_save = save + K * BV * 4;
};

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
    float* save_p = reinterpret_cast<float*>(smem + L::save);
    const uint32_t sb = smem_u32(sb_p), v2 = smem_u32(v2_p);

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

    auto is_active = [&](int c) -> bool { return cpb > 1 || sel_p[(long)(c / cpb) * sel_stride] != 0; };
    auto issue_loads = [&](int c, int st) {
        const int valid = min(64, T - c * 64);
        const long tok0 = (long)b * T + (long)c * 64;
        unsigned char* base = smem + st * L::stage;
        if (GDN) load_tile_async<64, K, SCAN_THREADS>(smem_u32(base), w + (tok0 * H + h) * K, (long)H * K, valid, tid);
        load_tile_async<64, K, SCAN_THREADS>(smem_u32(base + L::w_bytes), k + (tok0 * H + h) * K, (long)H * K, valid, tid);
        load_tile_async<64, BV, SCAN_THREADS>(smem_u32(base + L::w_bytes + L::k_bytes), u + (tok0 * H + h) * V + v0,
                                              (long)H * V, valid, tid);
        float* vec = reinterpret_cast<float*>(base + L::w_bytes + L::k_bytes + L::u_bytes);
        if (tid < 64) {
            // padded rows repeat the last valid cumsum (their k, u rows are zero)
            int r = min(tid, valid - 1);
            vec[tid] = gcs[(tok0 + r) * H + h];
            vec[64 + tid] = (krstd && tid < valid) ? krstd[(tok0 + tid) * H + h] : (krstd ? 0.f : 1.f);
        }
        cp_async_commit();
    };

    int next_active = 0;
    while (next_active < NT && !is_active(next_active)) ++next_active;
    if (next_active < NT) issue_loads(next_active, 0);
    int st = 0;
    float carry = 0.f, carry_save = 0.f, blk_g = 0.f;
    bool dirty = true;

    for (int c = 0; c < NT; ++c) {
        const int blk = c / cpb, sub = c % cpb;
        const bool sel = sel_p[(long)blk * sel_stride] != 0;
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
            __syncthreads();
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
            dirty = false;
        }
        store_tile<K, BV, SCAN_THREADS>(sb_p, hout + ((((long)b * NT + c) * H + h) * K) * V + v0, V, K, tid);
        if (vsplit == 0 && tid == 0) carry_out[((long)b * NT + c) * H + h] = carry;
        const int last_tok = min(c * 64 + 63, T - 1);
        const float gl = gcs[((long)b * T + last_tok) * H + h];
        blk_g += gl;

        if (active) {
            cp_async_wait<0>();
            __syncthreads();
            // prefetch the next active chunk into the other stage
            next_active = c + 1;
            while (next_active < NT && !is_active(next_active)) ++next_active;
            if (next_active < NT) issue_loads(next_active, st ^ 1);

            unsigned char* base = smem + st * L::stage;
            const uint32_t ws = smem_u32(base), ks = smem_u32(base + L::w_bytes);
            const unsigned char* us_p = base + L::w_bytes + L::k_bytes;
            const float* vec = reinterpret_cast<const float*>(base + L::w_bytes + L::k_bytes + L::u_bytes);
            const int r0 = warp * 16;
            float acc[NTL][4];
#pragma unroll
            for (int nt = 0; nt < NTL; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
            if (GDN) {
#pragma unroll 2
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
            float fa, fb;
            if (GDN) {
                fa = vec[64 + ra] * __expf(gl - vec[ra]);
                fb = vec[64 + rb] * __expf(gl - vec[rb]);
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
            __syncthreads();
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
            st ^= 1;
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
    const int smem = nbs > 64 ? L::total_with_save : L::total;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::total_with_save);
    if (e != cudaSuccess) {
        set_error("natsl_linear_fwd_h: cannot reserve %d B of shared memory (%s)", L::total_with_save,
                  cudaGetErrorString(e));
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
    NATSL_REQUIRE(k && u && gcs && types_i && indices && n_blocks && h && carry, NATSL_ERR_NULL,
                  "natsl_linear_fwd_h: null pointer");
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
