// Gated-delta-rule chunk preparation: one CTA per (batch, head, 64-token chunk) turns
// k, v, g, beta into the WY/UT representation the state recurrence consumes.
//   k_rstd = rsqrt(sum k^2 + 1e-6)                 (l2norm, src/nats/ops/mixed_ops/mixed_attn_gdn.py:119-121)
//   gcs    = chunk-local inclusive cumsum of g      (src/nats/ops/gated_delta_rule/chunk.py:52-54)
//   A      = strictLower(beta_i (kn_i . kn_j) e^{gcs_i - gcs_j})   (src/nats/ops/common/chunk_scaled_dot_kkt.py:105-126)
//   [u | w] = (I + A)^-1 [v beta | kn beta e^{gcs}]                (src/nats/ops/utils/solve_tril.py:350-447,
//                                                                  src/nats/ops/gated_delta_rule/wy_fast.py:123-153)
// The reference forms (I + A)^-1 explicitly (16x16 diagonal blocks by forward substitution, then a
// block merge) and multiplies.  Only the product is needed in the forward pass, so this kernel solves
// the block-triangular system instead: with X_ii = (I + A_ii)^-1 (fp32 forward substitution, CUDA
// cores) and G_ij = -X_ii A_ij (j < i), G_ii = X_ii (bf16),
//     U_i = G_ii Z_i + sum_{j<i} G_ij U_j          for the four 16-row blocks i = 0..3,
// where Z = [v beta | kn beta e^{gcs}] and U overwrites Z in place.  Each warp owns 64 columns of Z and
// runs its four steps on the tensor cores without block-wide synchronisation; U_j is rounded to bf16
// between steps, the same rounding the stored u, w get.
// The decay carried over skipped blocks multiplies w by one scalar per chunk (A only sees decay
// differences), so it is applied by the consumers and w here is carry-free.
#include "common.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

constexpr int PREP_THREADS = 256;          // warps 0-3 and 4-7 work on different things in most phases
constexpr int A_LD = 68;            // fp32 row pitch of A: 16-byte aligned rows for float4 reads
constexpr int X_LD = 17;            // pitch of the 16x16 diagonal-block inverses

template <int K, int V>
struct PrepSmem {
    static constexpr int ks = 0;
    static constexpr int vs = ks + 64 * K * 2;
    static constexpr int As = vs + 64 * V * 2;                 // fp32 [64][68]
    static constexpr int Xs = As + 64 * A_LD * 4;              // fp32 [4][16][17]
    static constexpr int Gs = Xs + 4 * 16 * X_LD * 4;          // bf16 [64][64] swizzled (128-byte rows)
    static constexpr int vec = Gs + 64 * 64 * 2;               // gcs, beta, rstd, wscale, q rstd: 5 x 64 floats
    static constexpr int total = vec + 5 * 64 * 4;
    static_assert(64 * K * 2 <= 64 * A_LD * 4, "the q tile is staged in the A buffer");
    static_assert(Gs % 128 == 0, "G tile alignment");
};

template <int COLS>
__device__ __forceinline__ void scale_rows_inplace(unsigned char* tile, const float* rowscale, int tid) {
    constexpr int CPR = COLS / 8;
    for (int i = tid; i < 64 * CPR; i += PREP_THREADS) {
        int r = i / CPR, c = i % CPR;
        uint4* p = reinterpret_cast<uint4*>(tile + swz<COLS * 2>(r, c));
        uint4 x = *p;
        float s = rowscale[r];
        uint32_t* xw = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float2 f = unpack_bf16(xw[j]);
            xw[j] = pack_bf16(f.x * s, f.y * s);
        }
        *p = x;
    }
}

// Block forward substitution on W columns [col0, col0+W) of a [64][COLS] tile, in place, by one warp;
// then the warp stores its 64 x W slice to global memory (row stride gstride elements).
template <int COLS, int W>
__device__ __forceinline__ void solve_group(uint32_t gtile, uint32_t ztile, unsigned char* zptr, int col0,
                                            __nv_bfloat16* gout, long gstride, int valid, int lane) {
    const int g = lane >> 2, q = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float acc[W / 8][4];
#pragma unroll
        for (int a = 0; a < W / 8; ++a)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[a][e] = 0.f;
#pragma unroll
        for (int kk = 0; kk <= i; ++kk) {
            uint32_t af[4];
            load_a<128>(gtile, 16 * i, 16 * kk, lane, af);
#pragma unroll
            for (int p = 0; p < W / 16; ++p) {
                uint32_t bf[4];
                load_b_kn<COLS * 2>(ztile, 16 * kk, col0 + 16 * p, lane, bf);
                mma_bf16(acc[2 * p], af, bf[0], bf[1]);
                mma_bf16(acc[2 * p + 1], af, bf[2], bf[3]);
            }
        }
        __syncwarp();          // all lanes have read the rows of block i before they are overwritten
#pragma unroll
        for (int nt = 0; nt < W / 8; ++nt) {
            const int ch = (col0 >> 3) + nt;
            *reinterpret_cast<uint32_t*>(zptr + swz<COLS * 2>(16 * i + g, ch) + q * 4) = pack_bf16(acc[nt][0], acc[nt][1]);
            *reinterpret_cast<uint32_t*>(zptr + swz<COLS * 2>(16 * i + g + 8, ch) + q * 4) = pack_bf16(acc[nt][2], acc[nt][3]);
        }
        __syncwarp();
    }
    constexpr int CPW = W / 8;                     // 16-byte chunks per row of the slice
    for (int it = lane; it < 64 * CPW; it += 32) {
        const int r = it / CPW, c = it % CPW;
        if (r < valid) {
            const uint4 x = *reinterpret_cast<const uint4*>(zptr + swz<COLS * 2>(r, (col0 >> 3) + c));
            *reinterpret_cast<uint4*>(gout + (long)r * gstride + col0 + c * 8) = x;
        }
    }
}

template <int K, int V>
__global__ void __launch_bounds__(PREP_THREADS, 3)
gdn_prep_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                const __nv_bfloat16* __restrict__ v, const float* __restrict__ g, const void* __restrict__ beta,
                int beta_dtype, __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ u,
                float* __restrict__ gcs_out, float* __restrict__ krstd_out, float* __restrict__ qrstd_out,
                __nv_bfloat16* __restrict__ p_out, int T, int H, int use_l2norm) {
    // q, qrstd_out, p_out may be null; when given the kernel also emits the intra-chunk score matrix
    //   P = tril(qn kn^T e^{gcs_i - gcs_j})  [B,T,H,64] bf16  (src/nats/ops/common/chunk_o.py:166,188,202-203)
    // and q's l2 norm factors, for the fused recurrence + output walk.
    using L = PrepSmem<K, V>;
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int t0 = c * 64;
    const int valid = min(64, T - t0);
    const long tok0 = (long)b * T + t0;

    unsigned char* ks_p = smem + L::ks;
    unsigned char* vs_p = smem + L::vs;
    unsigned char* gs_p = smem + L::Gs;
    float* As = reinterpret_cast<float*>(smem + L::As);
    float* Xs = reinterpret_cast<float*>(smem + L::Xs);
    float* s_gcs = reinterpret_cast<float*>(smem + L::vec);
    float* s_beta = s_gcs + 64;
    float* s_rstd = s_beta + 64;
    float* s_wsc = s_rstd + 64;
    float* s_qr = s_wsc + 64;
    unsigned char* qs_p = smem + L::As;                       // q tile, until A is written
    const uint32_t ks = smem_u32(ks_p), vs = smem_u32(vs_p), gs = smem_u32(gs_p), qs = smem_u32(qs_p);

    if (q) load_tile_async<64, K, PREP_THREADS>(qs, q + (tok0 * H + h) * K, (long)H * K, valid, tid);
    load_tile_async<64, K, PREP_THREADS>(ks, k + (tok0 * H + h) * K, (long)H * K, valid, tid);
    load_tile_async<64, V, PREP_THREADS>(vs, v + (tok0 * H + h) * V, (long)H * V, valid, tid);
    cp_async_commit();

    // ---- gcs (two-warp inclusive scan), beta
    float x = 0.f;
    if (tid < 64) {
        float bv = 0.f;
        if (tid < valid) {
            long gi = (tok0 + tid) * H + h;
            x = g[gi];
            bv = beta_dtype == NATSL_DT_F32 ? reinterpret_cast<const float*>(beta)[gi]
                                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(beta)[gi]);
        }
        s_beta[tid] = bv;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            float t = __shfl_up_sync(0xffffffffu, x, o);
            if (lane >= o) x += t;
        }
        if (tid == 31) s_wsc[0] = x;
    }
    __syncthreads();
    if (tid < 64) {
        if (tid >= 32) x += s_wsc[0];
        s_gcs[tid] = x;
        if (tid < valid) gcs_out[(tok0 + tid) * H + h] = x;
    }
    cp_async_wait<0>();
    __syncthreads();

    // ---- q row norms (read only); v rows scaled by beta (in place).  k stays raw in shared memory: its row norms
    // are the diagonal of K K^T, and 1/norm enters A, P and the right-hand side of w as row / column scales.
    if (q) {
        constexpr int CPR = K / 8;
        constexpr int RPP = 32 / CPR > 0 ? 32 / CPR : 1;
        const int sub = lane / CPR, cc = lane % CPR;
        for (int rr = 0; rr < 8; rr += RPP) {
            int r = warp * 8 + rr + sub;
            uint4 xv = *reinterpret_cast<const uint4*>(qs_p + swz<K * 2>(r, cc));
            const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xv);
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 t = unpack_bf16(xw[j]);
                ss += t.x * t.x + t.y * t.y;
            }
#pragma unroll
            for (int o = CPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (cc == 0) {
                const float rs = use_l2norm ? rsqrtf(ss + 1e-6f) : 1.0f;
                s_qr[r] = rs;
                if (r < valid && qrstd_out) qrstd_out[(tok0 + r) * H + h] = rs;
            }
        }
    }
    scale_rows_inplace<V>(vs_p, s_beta, tid);      // read again only by the substitution, many barriers from here

    // ---- products: warps 0-3 form K K^T (warp w: row block w), warps 4-7 Q K^T (warp 4+i: row block 3-i), side by side
    const int gq = lane >> 2, qd = lane & 3;
    const bool kk_warp = warp < 4;
    const int rblk = kk_warp ? warp : 7 - warp;          // 16-row block of this warp's product
    const int r0 = rblk * 16;
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    if (kk_warp || q) {
        const uint32_t atile = kk_warp ? ks : qs;
#pragma unroll 2
        for (int kk = 0; kk < K / 16; ++kk) {
            uint32_t a[4];
            load_a<K * 2>(atile, r0, kk * 16, lane, a);
            for (int p = 0; p <= rblk; ++p) {
                uint32_t bb[4];
                load_b_nk<K * 2>(ks, p * 16, kk * 16, lane, bb);
                mma_bf16(acc[2 * p], a, bb[0], bb[1]);
                mma_bf16(acc[2 * p + 1], a, bb[2], bb[3]);
            }
        }
    }
    if (kk_warp) {
        // k row norms from the diagonal of the product: the thread with gq == 2 qd + e holds (row gq, gq) in
        // acc[2 w][e] and (row gq + 8, gq + 8) in acc[2 w + 1][2 + e]
        const int e = gq - 2 * qd;
        if (e == 0 || e == 1) {
            float d0 = 0.f, d1 = 0.f;
#pragma unroll
            for (int p = 0; p < 4; ++p)
                if (p == rblk) {
                    d0 = e ? acc[2 * p][1] : acc[2 * p][0];
                    d1 = e ? acc[2 * p + 1][3] : acc[2 * p + 1][2];
                }
            const float rs0 = use_l2norm ? rsqrtf(d0 + 1e-6f) : 1.0f, rs1 = use_l2norm ? rsqrtf(d1 + 1e-6f) : 1.0f;
            const int ra = r0 + gq, rb = ra + 8;
            s_rstd[ra] = rs0;
            s_rstd[rb] = rs1;
            if (ra < valid) krstd_out[(tok0 + ra) * H + h] = rs0;
            if (rb < valid) krstd_out[(tok0 + rb) * H + h] = rs1;
        }
    }
    __syncthreads();              // every row's 1/norm is known; all products are done, so the q tile may be overwritten
    if (!kk_warp) {
        if (q) {
            // ---- P = tril(qn kn^T e^{gcs_i - gcs_j}), staged through the (still unused) G tile
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int i = r0 + gq + hh * 8;
                    const int j = nt * 8 + qd * 2;
                    float v0 = 0.f, v1 = 0.f;
                    if (j <= i && j < valid) v0 = acc[nt][hh * 2] * s_qr[i] * s_rstd[j] * __expf(s_gcs[i] - s_gcs[j]);
                    if (j + 1 <= i && j + 1 < valid)
                        v1 = acc[nt][hh * 2 + 1] * s_qr[i] * s_rstd[j + 1] * __expf(s_gcs[i] - s_gcs[j + 1]);
                    *reinterpret_cast<uint32_t*>(gs_p + swz<128>(i, nt) + qd * 4) = pack_bf16(v0, v1);
                }
            }
            __syncwarp();
            for (int it = lane; it < 16 * 8; it += 32) {
                const int r = r0 + (it >> 3), cch = it & 7;
                if (r < valid)
                    *reinterpret_cast<uint4*>(p_out + ((tok0 + r) * H + h) * 64 + cch * 8) =
                        *reinterpret_cast<const uint4*>(gs_p + swz<128>(r, cch));
            }
        }
        // right-hand side scale of w: kn beta e^{gcs}
        if (tid - 128 < 64) s_wsc[tid - 128] = s_beta[tid - 128] * s_rstd[tid - 128] * __expf(s_gcs[tid - 128]);
    } else {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            if (nt <= 2 * rblk + 1) {
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int i = r0 + gq + hh * 8;
                    const int j = nt * 8 + qd * 2;
                    const float bi = s_beta[i] * s_rstd[i];
                    float v0 = 0.f, v1 = 0.f;
                    if (i > j) v0 = bi * s_rstd[j] * acc[nt][hh * 2] * __expf(s_gcs[i] - s_gcs[j]);
                    if (i > j + 1) v1 = bi * s_rstd[j + 1] * acc[nt][hh * 2 + 1] * __expf(s_gcs[i] - s_gcs[j + 1]);
                    *reinterpret_cast<float2*>(&As[i * A_LD + j]) = make_float2(v0, v1);
                }
            }
        }
    }
    __syncthreads();              // A complete; the P staging is done, so the G tile is free; the w scale is known

    if (kk_warp) {
        // ---- X_dd = (I + A_dd)^-1 for the four 16x16 diagonal blocks: forward substitution, one warp each
        if (lane < 16) {
            const int d0 = warp * 16, cidx = lane;
            float xcol[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                // row i of the block (the same for every lane: broadcast reads), four independent partial sums
                float arow[16];
#pragma unroll
                for (int j4 = 0; j4 < 16; j4 += 4)
                    if (j4 < i)
                        *reinterpret_cast<float4*>(&arow[j4]) = *reinterpret_cast<const float4*>(&As[(d0 + i) * A_LD + d0 + j4]);
                float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
#pragma unroll
                for (int j = 0; j < i; ++j) {
                    const float t = arow[j] * xcol[j];
                    if ((j & 3) == 0) p0 += t; else if ((j & 3) == 1) p1 += t; else if ((j & 3) == 2) p2 += t; else p3 += t;
                }
                xcol[i] = ((i == cidx) ? 1.f : 0.f) - ((p0 + p1) + (p2 + p3));
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) Xs[(warp * 16 + i) * X_LD + cidx] = xcol[i];
        }
    } else {
        // ---- meanwhile: k rows -> kn beta e^{gcs} (the K K^T operand is no longer needed)
        constexpr int CPR = K / 8;
        for (int i = tid - 128; i < 64 * CPR; i += 128) {
            const int r = i / CPR, cch = i % CPR;
            uint4* ptr = reinterpret_cast<uint4*>(ks_p + swz<K * 2>(r, cch));
            uint4 x4 = *ptr;
            const float sc = s_wsc[r];
            uint32_t* xw = reinterpret_cast<uint32_t*>(&x4);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 f = unpack_bf16(xw[j]);
                xw[j] = pack_bf16(f.x * sc, f.y * sc);
            }
            *ptr = x4;
        }
    }
    __syncthreads();

    // ---- G (bf16, A-operand layout): diagonal blocks X_dd, below-diagonal blocks -X_ii A_ij
    for (int e = tid; e < 4 * 16 * 4; e += PREP_THREADS) {          // diagonal: (block, row, 4 columns)
        const int d = e >> 6, r = (e >> 2) & 15, c4 = (e & 3) * 4;
        const float* xr = &Xs[(d * 16 + r) * X_LD + c4];
        const int row = d * 16 + r, col = d * 16 + c4;
        *reinterpret_cast<uint2*>(gs_p + swz<128>(row, col >> 3) + (col & 7) * 2) =
            make_uint2(pack_bf16(xr[0], xr[1]), pack_bf16(xr[2], xr[3]));
    }
    for (int e = tid; e < 6 * 16 * 4; e += PREP_THREADS) {          // below diagonal: (block pair, row, 4 columns)
        const int blk = e >> 6, r = (e >> 2) & 15, c4 = (e & 3) * 4;
        // block pairs (i, j): (1,0) (2,0) (2,1) (3,0) (3,1) (3,2)
        const int bi = blk < 1 ? 1 : (blk < 3 ? 2 : 3);
        const int bj = blk - (bi == 1 ? 0 : (bi == 2 ? 1 : 3));
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int m = 0; m < 16; ++m) {
            const float xm = Xs[(bi * 16 + r) * X_LD + m];
            const float4 av = *reinterpret_cast<const float4*>(&As[(bi * 16 + m) * A_LD + bj * 16 + c4]);
            a0 -= xm * av.x; a1 -= xm * av.y; a2 -= xm * av.z; a3 -= xm * av.w;
        }
        const int row = bi * 16 + r, col = bj * 16 + c4;
        *reinterpret_cast<uint2*>(gs_p + swz<128>(row, col >> 3) + (col & 7) * 2) =
            make_uint2(pack_bf16(a0, a1), pack_bf16(a2, a3));
    }
    __syncthreads();

    // ---- [u | w] = block forward substitution, 32 columns per warp
    constexpr int NCG = (K + V) / 32;
    for (int cg = warp; cg < NCG; cg += 8) {
        if (cg < V / 32)
            solve_group<V, 32>(gs, vs, vs_p, cg * 32, u + (tok0 * H + h) * V, (long)H * V, valid, lane);
        else
            solve_group<K, 32>(gs, ks, ks_p, (cg - V / 32) * 32, w + (tok0 * H + h) * K, (long)H * K, valid, lane);
    }
}

template <int K, int V>
static int launch_prep(const void* q, const void* k, const void* v, const float* g, const void* beta, int beta_dtype,
                       void* w, void* u, float* gcs, float* krstd, float* qrstd, void* pmat, int B, int T, int H,
                       int use_l2norm, cudaStream_t st) {
    using L = PrepSmem<K, V>;
    auto kern = gdn_prep_kernel<K, V>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::total);
    if (e != cudaSuccess) {
        set_error("natsl_gdn_chunk_prep: cannot reserve %d B of shared memory (%s)", L::total, cudaGetErrorString(e));
        return NATSL_ERR_CUDA;
    }
    const int NT = (T + 63) / 64;
    dim3 grid(NT, H, B);
    kern<<<grid, PREP_THREADS, L::total, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(q), reinterpret_cast<const __nv_bfloat16*>(k),
        reinterpret_cast<const __nv_bfloat16*>(v), g, beta, beta_dtype, reinterpret_cast<__nv_bfloat16*>(w),
        reinterpret_cast<__nv_bfloat16*>(u), gcs, krstd, qrstd, reinterpret_cast<__nv_bfloat16*>(pmat), T, H, use_l2norm);
    return check_launch("natsl_gdn_chunk_prep");
}

}  // namespace natsl

extern "C" int natsl_gdn_chunk_prep_ex(const void* q, const void* k, const void* v, const float* g, const void* beta,
                                       int beta_dtype, void* w, void* u, float* gcs, float* k_rstd, float* q_rstd,
                                       void* pmat, int B, int T, int H, int K, int V, int use_l2norm, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(k && v && g && beta && w && u && gcs && k_rstd, NATSL_ERR_NULL, "natsl_gdn_chunk_prep: null pointer");
    NATSL_REQUIRE((q == nullptr) == (pmat == nullptr), NATSL_ERR_NULL,
                  "natsl_gdn_chunk_prep: q and the score-matrix output go together");
    NATSL_REQUIRE(B > 0 && T > 0 && H > 0, NATSL_ERR_BAD_SHAPE, "natsl_gdn_chunk_prep: empty shape");
    NATSL_REQUIRE(H <= 65535 && B <= 65535, NATSL_ERR_TOO_LARGE, "natsl_gdn_chunk_prep: B and H must be <= 65535");
    NATSL_REQUIRE(beta_dtype == NATSL_DT_BF16 || beta_dtype == NATSL_DT_F32, NATSL_ERR_UNSUPPORTED,
                  "natsl_gdn_chunk_prep: beta must be bf16 or f32");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define NATSL_PREP_CASE(KK, VV) \
    if (K == KK && V == VV)     \
        return launch_prep<KK, VV>(q, k, v, g, beta, beta_dtype, w, u, gcs, k_rstd, q_rstd, pmat, B, T, H, use_l2norm, st);
    NATSL_PREP_CASE(64, 64)
    NATSL_PREP_CASE(64, 128)
    NATSL_PREP_CASE(128, 64)
    NATSL_PREP_CASE(128, 128)
    NATSL_PREP_CASE(128, 256)
#undef NATSL_PREP_CASE
    set_error("natsl_gdn_chunk_prep: unsupported head dims K=%d V=%d (K in {64,128}, V in {64,128,256})", K, V);
    return NATSL_ERR_UNSUPPORTED;
}

extern "C" int natsl_gdn_chunk_prep(const void* k, const void* v, const float* g, const void* beta, int beta_dtype,
                                    void* w, void* u, float* gcs, float* k_rstd, int B, int T, int H, int K, int V,
                                    int use_l2norm, void* stream) {
    return natsl_gdn_chunk_prep_ex(nullptr, k, v, g, beta, beta_dtype, w, u, gcs, k_rstd, nullptr, nullptr, B, T, H, K, V,
                                   use_l2norm, stream);
}
