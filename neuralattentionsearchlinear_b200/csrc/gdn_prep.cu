// Gated-delta-rule chunk preparation: one CTA per (batch, head, 64-token chunk) turns
// k, v, g, beta into the WY/UT representation the state recurrence consumes.
//   k_rstd = rsqrt(sum k^2 + 1e-6)                 (l2norm, src/nats/ops/mixed_ops/mixed_attn_gdn.py:119-121)
//   gcs    = chunk-local inclusive cumsum of g      (src/nats/ops/gated_delta_rule/chunk.py:52-54)
//   A      = strictLower(beta_i (kn_i . kn_j) e^{gcs_i - gcs_j})   (src/nats/ops/common/chunk_scaled_dot_kkt.py:105-126)
//   Ai     = (I + A)^-1, fp32 forward substitution on the four 16x16 diagonal blocks, then
//            block merge                            (src/nats/ops/utils/solve_tril.py:350-447)
//   u = Ai (v beta),  w = Ai (kn beta e^{gcs})      (src/nats/ops/gated_delta_rule/wy_fast.py:123-153)
// The decay carried over skipped blocks multiplies w by one scalar per chunk (the inverse
// and A only see decay differences), so it is applied by the consumers and w here is
// carry-free.  KK^T, u and w run on the tensor cores (bf16 in, fp32 accumulate); the
// inverse stays in fp32 on the CUDA cores like the reference's ieee-precision default.
#include "common.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

constexpr int PREP_THREADS = 128;
constexpr int A_LD = 65;

template <int K, int V>
struct PrepSmem {
    static constexpr int ks = 0;
    static constexpr int vs = ks + 64 * K * 2;
    static constexpr int As = vs + 64 * V * 2;                 // fp32 [64][65]; later Ai bf16 [64][64]
    static constexpr int Xs = As + 64 * A_LD * 4;              // fp32 [64][65]; later output staging
    static constexpr int Tm = Xs + 64 * A_LD * 4;              // fp32 [3][16][17]
    static constexpr int vec = Tm + 3 * 16 * 17 * 4;           // gcs, beta, rstd, wscale: 4 x 64 floats
    static constexpr int total = vec + 4 * 64 * 4;
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

// out[16w.., :] = Ai[16w.., :] * B  (B = [64 tokens][COLS] bf16 tile), 64 columns at a time,
// staged per warp through `stage` and written to global with 16-byte stores.
template <int COLS>
__device__ __forceinline__ void tri_matmul_store(uint32_t ai, uint32_t bt, unsigned char* stage, __nv_bfloat16* gout,
                                                 long gstride, int valid, int warp, int lane) {
    const int r0 = warp * 16;
    const uint32_t st = smem_u32(stage);
#pragma unroll 1
    for (int cg = 0; cg < COLS / 64; ++cg) {
        float acc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
        for (int kk = 0; kk <= warp; ++kk) {
            uint32_t a[4];
            load_a<128>(ai, r0, kk * 16, lane, a);
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                uint32_t b[4];
                load_b_kn<COLS * 2>(bt, kk * 16, cg * 64 + p * 16, lane, b);
                mma_bf16(acc[2 * p], a, b[0], b[1]);
                mma_bf16(acc[2 * p + 1], a, b[2], b[3]);
            }
        }
        const int g = lane >> 2, q = lane & 3;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            // column pair (nt*8 + 2q, +1) -> chunk nt, word q
            *reinterpret_cast<uint32_t*>(stage + swz<128>(r0 + g, nt) + q * 4) = pack_bf16(acc[nt][0], acc[nt][1]);
            *reinterpret_cast<uint32_t*>(stage + swz<128>(r0 + g + 8, nt) + q * 4) = pack_bf16(acc[nt][2], acc[nt][3]);
        }
        __syncwarp();
        for (int i = lane; i < 16 * 8; i += 32) {
            int r = r0 + i / 8, c = i % 8;
            if (r < valid) {
                uint4 x = *reinterpret_cast<const uint4*>(stage + swz<128>(r, c));
                *reinterpret_cast<uint4*>(gout + (long)r * gstride + cg * 64 + c * 8) = x;
            }
        }
        __syncwarp();
        (void)st;
    }
}

template <int K, int V>
__global__ void __launch_bounds__(PREP_THREADS)
gdn_prep_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v, const float* __restrict__ g,
                const void* __restrict__ beta, int beta_dtype, __nv_bfloat16* __restrict__ w,
                __nv_bfloat16* __restrict__ u, float* __restrict__ gcs_out, float* __restrict__ krstd_out, int T, int H,
                int use_l2norm) {
    using L = PrepSmem<K, V>;
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int t0 = c * 64;
    const int valid = min(64, T - t0);
    const long tok0 = (long)b * T + t0;

    unsigned char* ks_p = smem + L::ks;
    unsigned char* vs_p = smem + L::vs;
    float* As = reinterpret_cast<float*>(smem + L::As);
    float* Xs = reinterpret_cast<float*>(smem + L::Xs);
    float* Tm = reinterpret_cast<float*>(smem + L::Tm);
    float* s_gcs = reinterpret_cast<float*>(smem + L::vec);
    float* s_beta = s_gcs + 64;
    float* s_rstd = s_beta + 64;
    float* s_wsc = s_rstd + 64;
    const uint32_t ks = smem_u32(ks_p), vs = smem_u32(vs_p);

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

    // ---- l2norm of k rows (in place), rstd out
    {
        constexpr int CPR = K / 8;                 // lanes per row
        constexpr int RPP = 32 / CPR > 0 ? 32 / CPR : 1;
        static_assert(CPR <= 32, "K <= 256");
        const int sub = lane / CPR, cc = lane % CPR;
        for (int rr = 0; rr < 16; rr += RPP) {
            int r = warp * 16 + rr + sub;
            uint4* p = reinterpret_cast<uint4*>(ks_p + swz<K * 2>(r, cc));
            uint4 xv = *p;
            uint32_t* xw = reinterpret_cast<uint32_t*>(&xv);
            float f[8];
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 t = unpack_bf16(xw[j]);
                f[2 * j] = t.x; f[2 * j + 1] = t.y;
                ss += t.x * t.x + t.y * t.y;
            }
#pragma unroll
            for (int o = CPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            float rs = use_l2norm ? rsqrtf(ss + 1e-6f) : 1.0f;
            if (use_l2norm) {
#pragma unroll
                for (int j = 0; j < 4; ++j) xw[j] = pack_bf16(f[2 * j] * rs, f[2 * j + 1] * rs);
                *p = xv;
            }
            if (cc == 0) {
                s_rstd[r] = rs;
                if (r < valid) krstd_out[(tok0 + r) * H + h] = rs;
            }
        }
    }
    __syncthreads();

    // ---- A = strictLower(beta_i (kn_i . kn_j) exp(gcs_i - gcs_j))
    {
        const int r0 = warp * 16;
        float acc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll 2
        for (int kk = 0; kk < K / 16; ++kk) {
            uint32_t a[4];
            load_a<K * 2>(ks, r0, kk * 16, lane, a);
            for (int p = 0; p <= warp; ++p) {
                uint32_t bb[4];
                load_b_nk<K * 2>(ks, p * 16, kk * 16, lane, bb);
                mma_bf16(acc[2 * p], a, bb[0], bb[1]);
                mma_bf16(acc[2 * p + 1], a, bb[2], bb[3]);
            }
        }
        const int gq = lane >> 2, q = lane & 3;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int i = r0 + gq + ((e >> 1) << 3);
                int j = nt * 8 + q * 2 + (e & 1);
                float val = 0.f;
                if (i > j) val = s_beta[i] * acc[nt][e] * __expf(s_gcs[i] - s_gcs[j]);
                As[i * A_LD + j] = val;
            }
        }
    }
    __syncthreads();

    // ---- X = (I + A)^-1 : diagonal 16x16 blocks by forward substitution (one warp each)
    if (lane < 16) {
        const int d0 = warp * 16, cidx = lane;
        float xcol[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float s = (i == cidx) ? 1.f : 0.f;
#pragma unroll
            for (int j = 0; j < i; ++j) s -= As[(d0 + i) * A_LD + d0 + j] * xcol[j];
            xcol[i] = s;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) Xs[(d0 + i) * A_LD + d0 + cidx] = xcol[i];
    }
    __syncthreads();
    // off-diagonal blocks, by distance from the diagonal: X_ij = -X_ii (sum_k A_ik X_kj)
    for (int d = 1; d <= 3; ++d) {
        const int nb = 4 - d;
        for (int e = tid; e < nb * 256; e += PREP_THREADS) {
            int blk = e >> 8, r = (e >> 4) & 15, cidx = e & 15;
            int bi = blk + d, bj = blk;
            float s = 0.f;
            for (int kb = bj; kb < bi; ++kb) {
#pragma unroll
                for (int m = 0; m < 16; ++m)
                    s += As[(bi * 16 + r) * A_LD + kb * 16 + m] * Xs[(kb * 16 + m) * A_LD + bj * 16 + cidx];
            }
            Tm[(blk * 16 + r) * 17 + cidx] = s;
        }
        __syncthreads();
        for (int e = tid; e < nb * 256; e += PREP_THREADS) {
            int blk = e >> 8, r = (e >> 4) & 15, cidx = e & 15;
            int bi = blk + d, bj = blk;
            float s = 0.f;
#pragma unroll
            for (int m = 0; m < 16; ++m) s -= Xs[(bi * 16 + r) * A_LD + bi * 16 + m] * Tm[(blk * 16 + m) * 17 + cidx];
            Xs[(bi * 16 + r) * A_LD + bj * 16 + cidx] = s;
        }
        __syncthreads();
    }

    // ---- Ai (bf16, swizzled, over the A buffer); row scales for v and k
    unsigned char* ai_p = smem + L::As;
    {
        int r = tid >> 1, half = tid & 1;
#pragma unroll
        for (int cch = 0; cch < 4; ++cch) {
            int c0 = half * 32 + cch * 8;
            uint32_t wv[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int j0 = c0 + 2 * j;
                float a0 = ((j0 >> 4) <= (r >> 4)) ? Xs[r * A_LD + j0] : 0.f;
                float a1 = (((j0 + 1) >> 4) <= (r >> 4)) ? Xs[r * A_LD + j0 + 1] : 0.f;
                if (j0 > r) a0 = 0.f;
                if (j0 + 1 > r) a1 = 0.f;
                wv[j] = pack_bf16(a0, a1);
            }
            // As and Ai alias: all reads of Xs above are from the other buffer, As itself is dead here
            *reinterpret_cast<uint4*>(ai_p + swz<128>(r, c0 >> 3)) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
        }
        if (tid < 64) s_wsc[tid] = s_beta[tid] * __expf(s_gcs[tid]);
    }
    __syncthreads();
    scale_rows_inplace<V>(vs_p, s_beta, tid);
    scale_rows_inplace<K>(ks_p, s_wsc, tid);
    __syncthreads();

    // ---- u = Ai (v beta), w = Ai (kn beta e^{gcs})
    const uint32_t ai = smem_u32(ai_p);
    unsigned char* stage = smem + L::Xs;
    tri_matmul_store<V>(ai, vs, stage, u + (tok0 * H + h) * V, (long)H * V, valid, warp, lane);
    tri_matmul_store<K>(ai, ks, stage, w + (tok0 * H + h) * K, (long)H * K, valid, warp, lane);
}

template <int K, int V>
static int launch_prep(const void* k, const void* v, const float* g, const void* beta, int beta_dtype, void* w, void* u,
                       float* gcs, float* krstd, int B, int T, int H, int use_l2norm, cudaStream_t st) {
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
        reinterpret_cast<const __nv_bfloat16*>(k), reinterpret_cast<const __nv_bfloat16*>(v), g, beta, beta_dtype,
        reinterpret_cast<__nv_bfloat16*>(w), reinterpret_cast<__nv_bfloat16*>(u), gcs, krstd, T, H, use_l2norm);
    return check_launch("natsl_gdn_chunk_prep");
}

}  // namespace natsl

extern "C" int natsl_gdn_chunk_prep(const void* k, const void* v, const float* g, const void* beta, int beta_dtype,
                                    void* w, void* u, float* gcs, float* k_rstd, int B, int T, int H, int K, int V,
                                    int use_l2norm, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(k && v && g && beta && w && u && gcs && k_rstd, NATSL_ERR_NULL, "natsl_gdn_chunk_prep: null pointer");
    NATSL_REQUIRE(B > 0 && T > 0 && H > 0, NATSL_ERR_BAD_SHAPE, "natsl_gdn_chunk_prep: empty shape");
    NATSL_REQUIRE(H <= 65535 && B <= 65535, NATSL_ERR_TOO_LARGE, "natsl_gdn_chunk_prep: B and H must be <= 65535");
    NATSL_REQUIRE(beta_dtype == NATSL_DT_BF16 || beta_dtype == NATSL_DT_F32, NATSL_ERR_UNSUPPORTED,
                  "natsl_gdn_chunk_prep: beta must be bf16 or f32");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define NATSL_PREP_CASE(KK, VV) \
    if (K == KK && V == VV) return launch_prep<KK, VV>(k, v, g, beta, beta_dtype, w, u, gcs, k_rstd, B, T, H, use_l2norm, st);
    NATSL_PREP_CASE(64, 64)
    NATSL_PREP_CASE(64, 128)
    NATSL_PREP_CASE(128, 64)
    NATSL_PREP_CASE(128, 128)
    NATSL_PREP_CASE(128, 256)
#undef NATSL_PREP_CASE
    set_error("natsl_gdn_chunk_prep: unsupported head dims K=%d V=%d (K in {64,128}, V in {64,128,256})", K, V);
    return NATSL_ERR_UNSUPPORTED;
}
