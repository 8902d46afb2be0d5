// fp32 reference-precision path: token-by-token linear recurrence with re-roll, and a plain fp32
// chunk-masked softmax attention.  These follow the reference's decode kernel
//   src/nats/ops/gated_delta_rule/fused_recurrent.py:128-358  (Mamba2 twin: src/nats/ops/mamba/fused_recurrent.py:121-322)
// per token:  S <- e^{g_t} S;  v' = beta_t (v_t - S^T k_t)  [delta rule] or v_t [Mamba2];  S <- S + k_t v'^T;
//             o_t = scale * S^T q_t;   at the end of a block that is not selected the state is rolled back to the
//             block-start state (decayed by the block's total log decay when decay over skipped blocks is on).
// They serve fp32 inputs (parity to 1e-4 against the naive recurrent form) and short sequences; the bf16
// chunked tensor-core kernels are the throughput path.  One warp per (batch, head, 8 value columns); the K rows
// of the state are spread over the lanes; CUDA-core fp32 math only.
#include "common.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

template <typename T>
__device__ __forceinline__ float ldf(const T* p, long i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, long i) { return p[i]; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long i) { return __bfloat162float(p[i]); }
template <typename T>
__device__ __forceinline__ void stf(T* p, long i, float v);
template <>
__device__ __forceinline__ void stf<float>(float* p, long i, float v) { p[i] = v; }
template <>
__device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, long i, float v) { p[i] = __float2bfloat16(v); }

constexpr int REC_BV = 8;

template <typename T, int KPL>      // KPL = K / 32 state rows per lane
__global__ void __launch_bounds__(32)
linear_recurrent_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                        const float* __restrict__ g, const T* __restrict__ beta, const int* __restrict__ types_i,
                        const float* __restrict__ h0, T* __restrict__ o, float* __restrict__ ht,
                        float* __restrict__ hstart, int Tlen, int H, int HN, int V, int TN, int nbs, float scale,
                        int gdn, int decay, int use_l2norm, const float* __restrict__ hstart_in,
                        const float* __restrict__ gsum_in, int t_off, int step_mode) {
    // step_mode (decoding): the Tlen tokens continue a block that already holds t_off tokens; h0 is the current state,
    // hstart_in the state at the start of that block, gsum_in [B,H] its log decay so far.  A block only ends where
    // (t_off + t + 1) is a multiple of nbs, and ht receives the current state instead of the state after the last
    // selected block (fused_recurrent.py:128-358 with initial_state / initial_state_current / g_cumsum).
    constexpr int K = KPL * 32;
    const int lane = threadIdx.x;
    const int v0 = blockIdx.x * REC_BV, h = blockIdx.y, b = blockIdx.z;
    const int hn = h / (H / HN);
    float S[KPL][REC_BV], S0[KPL][REC_BV], Sfin[KPL][REC_BV];
#pragma unroll
    for (int i = 0; i < KPL; ++i)
#pragma unroll
        for (int j = 0; j < REC_BV; ++j) {
            const long idx = (((long)b * H + h) * K + lane + 32 * i) * V + v0 + j;
            float x = h0 ? h0[idx] : 0.f;
            S[i][j] = Sfin[i][j] = x;
            S0[i][j] = hstart_in ? hstart_in[idx] : x;
        }
    float gsum = gsum_in ? gsum_in[(long)b * H + h] : 0.f;
    for (int t = 0; t < Tlen; ++t) {
        const long tok = (long)b * Tlen + t;
        float qk[KPL], kk[KPL];
        float sq = 0.f, sk = 0.f;
#pragma unroll
        for (int i = 0; i < KPL; ++i) {
            qk[i] = ldf(q, (tok * H + h) * K + lane + 32 * i);
            kk[i] = ldf(k, (tok * H + h) * K + lane + 32 * i);
            sq += qk[i] * qk[i];
            sk += kk[i] * kk[i];
        }
        if (use_l2norm) {
            sq = warp_sum(sq);
            sk = warp_sum(sk);
            const float rq = rsqrtf(sq + 1e-6f), rk = rsqrtf(sk + 1e-6f);
#pragma unroll
            for (int i = 0; i < KPL; ++i) { qk[i] *= rq; kk[i] *= rk; }
        }
        const float gt = g[tok * H + h];
        const float eg = __expf(gt);
        gsum += gt;
        float vv[REC_BV], dot[REC_BV];
#pragma unroll
        for (int j = 0; j < REC_BV; ++j) {
            vv[j] = ldf(v, (tok * H + h) * V + v0 + j);
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < KPL; ++i) {
                S[i][j] *= eg;
                d += S[i][j] * kk[i];
            }
            dot[j] = d;
        }
        if (gdn) {
            const float bt = ldf(beta, tok * H + h);
#pragma unroll
            for (int j = 0; j < REC_BV; ++j) vv[j] = bt * (vv[j] - warp_sum(dot[j]));
        }
#pragma unroll
        for (int j = 0; j < REC_BV; ++j) {
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < KPL; ++i) {
                S[i][j] += kk[i] * vv[j];
                d += S[i][j] * qk[i];
            }
            d = warp_sum(d) * scale;
            if (lane == 0) stf(o, (tok * H + h) * V + v0 + j, d);
        }
        if ((t_off + t + 1) % nbs == 0 || (!step_mode && t == Tlen - 1)) {
            const int sel = types_i[(((long)b * TN + (t_off + t) / nbs) * HN + hn) * 2 + 1];
            const float roll = decay ? __expf(gsum) : 1.f;
#pragma unroll
            for (int i = 0; i < KPL; ++i)
#pragma unroll
                for (int j = 0; j < REC_BV; ++j) {
                    if (sel) Sfin[i][j] = S[i][j]; else S[i][j] = S0[i][j] * roll;
                    S0[i][j] = S[i][j];
                }
            gsum = 0.f;
        }
    }
#pragma unroll
    for (int i = 0; i < KPL; ++i)
#pragma unroll
        for (int j = 0; j < REC_BV; ++j) {
            const long idx = (((long)b * H + h) * K + lane + 32 * i) * V + v0 + j;
            if (ht) ht[idx] = step_mode ? S[i][j] : Sfin[i][j];
            if (hstart) hstart[idx] = S0[i][j];
        }
}

// fp32 attention: one warp per (batch, head, query); lanes stride over the visible keys.
template <typename T, int DK, int DV>
__global__ void __launch_bounds__(128)
attn_fp32_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                 const int* __restrict__ types_i, T* __restrict__ o, float* __restrict__ lse, int Tlen, int HQ, int HKV,
                 int HN, int TN, int nbs, float scale, int own_chunk) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int hq = blockIdx.y, b = blockIdx.z;
    if (t >= Tlen) return;
    const int hkv = hq / (HQ / HKV), hn = hq / (HQ / HN);
    float qr[DK];
#pragma unroll
    for (int d = 0; d < DK; ++d) qr[d] = ldf(q, (((long)b * Tlen + t) * HQ + hq) * DK + d) * scale;
    float m = -INFINITY, l = 0.f, acc[DV];
#pragma unroll
    for (int d = 0; d < DV; ++d) acc[d] = 0.f;
    const int tb = t / nbs;
    for (int s = lane; s <= t; s += 32) {
        const int sb = s / nbs;
        const bool sel = types_i[(((long)b * TN + sb) * HN + hn) * 2] != 0;
        const bool vis = (sel && t >= (sb + 1) * nbs) || (own_chunk && sb == tb);
        if (!vis) continue;
        const long kb = (((long)b * Tlen + s) * HKV + hkv);
        float sc = 0.f;
#pragma unroll
        for (int d = 0; d < DK; ++d) sc += qr[d] * ldf(k, kb * DK + d);
        const float mn = fmaxf(m, sc);
        const float al = __expf(m - mn), p = __expf(sc - mn);
        l = l * al + p;
#pragma unroll
        for (int d = 0; d < DV; ++d) acc[d] = acc[d] * al + p * ldf(v, kb * DV + d);
        m = mn;
    }
    // merge the lanes
    float mg = m;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mg = fmaxf(mg, __shfl_xor_sync(0xffffffffu, mg, off));
    const float f = (m == -INFINITY) ? 0.f : __expf(m - mg);
    float lt = warp_sum(l * f);
    const bool has = mg != -INFINITY && lt > 0.f;
#pragma unroll
    for (int d = 0; d < DV; ++d) {
        const float x = warp_sum(acc[d] * f);
        if (lane == 0) stf(o, (((long)b * Tlen + t) * HQ + hq) * DV + d, has ? x / lt : 0.f);
    }
    if (lane == 0) lse[((long)b * Tlen + t) * HQ + hq] = has ? (mg + logf(lt)) * 1.44269504f : 0.f;
}

template <typename T>
static int launch_recurrent(const void* q, const void* k, const void* v, const float* g, const void* beta,
                            const int* types_i, const float* h0, void* o, float* ht, float* hstart, int B, int T_, int H,
                            int HN, int K, int V, int nbs, float scale, int gdn, int decay, int l2, cudaStream_t st,
                            const float* hstart_in = nullptr, const float* gsum_in = nullptr, int t_off = 0,
                            int step_mode = 0) {
    const int TN = (t_off + T_ + nbs - 1) / nbs;
    dim3 grid(V / REC_BV, H, B);
#define NATSL_REC(KPL) linear_recurrent_kernel<T, KPL><<<grid, 32, 0, st>>>( \
        reinterpret_cast<const T*>(q), reinterpret_cast<const T*>(k), reinterpret_cast<const T*>(v), g, \
        reinterpret_cast<const T*>(beta), types_i, h0, reinterpret_cast<T*>(o), ht, hstart, T_, H, HN, V, TN, nbs, scale, gdn, decay, l2, \
        hstart_in, gsum_in, t_off, step_mode)
    if (K == 32) NATSL_REC(1);
    else if (K == 64) NATSL_REC(2);
    else if (K == 96) NATSL_REC(3);
    else if (K == 128) NATSL_REC(4);
    else if (K == 192) NATSL_REC(6);
    else if (K == 256) NATSL_REC(8);
    else {
        set_error("natsl_linear_recurrent_fwd: unsupported key dim K=%d (32, 64, 96, 128, 192 or 256)", K);
        return NATSL_ERR_UNSUPPORTED;
    }
#undef NATSL_REC
    return check_launch("natsl_linear_recurrent_fwd");
}

template <typename T>
static int launch_attn_fp32(const void* q, const void* k, const void* v, const int* types_i, void* o, float* lse, int B,
                            int T_, int HQ, int HKV, int HN, int DK, int DV, int nbs, float scale, int own,
                            cudaStream_t st) {
    const int TN = (T_ + nbs - 1) / nbs;
    dim3 grid((T_ + 3) / 4, HQ, B);
#define NATSL_AF(DKK, DVV) attn_fp32_kernel<T, DKK, DVV><<<grid, 128, 0, st>>>( \
        reinterpret_cast<const T*>(q), reinterpret_cast<const T*>(k), reinterpret_cast<const T*>(v), types_i, \
        reinterpret_cast<T*>(o), lse, T_, HQ, HKV, HN, TN, nbs, scale, own)
    if (DK == 64 && DV == 64) NATSL_AF(64, 64);
    else if (DK == 32 && DV == 32) NATSL_AF(32, 32);
    else if (DK == 128 && DV == 64) NATSL_AF(128, 64);
    else if (DK == 64 && DV == 128) NATSL_AF(64, 128);
    else if (DK == 128 && DV == 128) NATSL_AF(128, 128);
    else {
        set_error("natsl_attn_fwd_fp32: unsupported head dims DK=%d DV=%d", DK, DV);
        return NATSL_ERR_UNSUPPORTED;
    }
#undef NATSL_AF
    return check_launch("natsl_attn_fwd_fp32");
}

}  // namespace natsl

extern "C" int natsl_linear_recurrent_fwd(int rule, int dtype, const void* q, const void* k, const void* v,
                                          const float* g, const void* beta, const int32_t* types_i, const float* h0,
                                          void* o, float* ht, float* hstart, int B, int T, int H, int HN, int K, int V,
                                          int nbs, float scale, int flags, int use_l2norm, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(q && k && v && g && types_i && o, NATSL_ERR_NULL, "natsl_linear_recurrent_fwd: null pointer");
    NATSL_REQUIRE(rule == NATSL_RULE_GDN || rule == NATSL_RULE_MAMBA, NATSL_ERR_UNSUPPORTED, "natsl_linear_recurrent_fwd: bad rule");
    NATSL_REQUIRE(rule != NATSL_RULE_GDN || beta, NATSL_ERR_NULL, "natsl_linear_recurrent_fwd: beta is required for the delta rule");
    NATSL_REQUIRE(B > 0 && T > 0 && H > 0 && HN > 0 && H % HN == 0 && V % REC_BV == 0 && nbs > 0, NATSL_ERR_BAD_SHAPE,
                  "natsl_linear_recurrent_fwd: bad shape (V must be a multiple of 8)");
    NATSL_REQUIRE(H <= 65535 && B <= 65535, NATSL_ERR_TOO_LARGE, "natsl_linear_recurrent_fwd: B, H <= 65535");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int gdn = rule == NATSL_RULE_GDN, decay = (flags & NATSL_FLAG_DECAY_SKIPPED) ? 1 : 0;
    if (dtype == NATSL_DT_F32)
        return launch_recurrent<float>(q, k, v, g, beta, types_i, h0, o, ht, hstart, B, T, H, HN, K, V, nbs, scale, gdn, decay, use_l2norm, st);
    if (dtype == NATSL_DT_BF16)
        return launch_recurrent<__nv_bfloat16>(q, k, v, g, beta, types_i, h0, o, ht, hstart, B, T, H, HN, K, V, nbs, scale, gdn, decay, use_l2norm, st);
    set_error("natsl_linear_recurrent_fwd: dtype must be f32 or bf16");
    return NATSL_ERR_UNSUPPORTED;
}

extern "C" int natsl_linear_recurrent_step(int rule, int dtype, const void* q, const void* k, const void* v, const float* g,
                                           const void* beta, const int32_t* types_i, const float* h_cur,
                                           const float* h_start, const float* gsum, int t_off, void* o, float* h_cur_out,
                                           float* h_start_out, int B, int T, int H, int HN, int K, int V, int nbs,
                                           float scale, int flags, int use_l2norm, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(q && k && v && g && types_i && h_cur && h_start && gsum && o && h_cur_out && h_start_out, NATSL_ERR_NULL,
                  "natsl_linear_recurrent_step: null pointer");
    NATSL_REQUIRE(rule == NATSL_RULE_GDN || rule == NATSL_RULE_MAMBA, NATSL_ERR_UNSUPPORTED, "natsl_linear_recurrent_step: bad rule");
    NATSL_REQUIRE(rule != NATSL_RULE_GDN || beta, NATSL_ERR_NULL, "natsl_linear_recurrent_step: beta is required for the delta rule");
    NATSL_REQUIRE(B > 0 && T > 0 && H > 0 && HN > 0 && H % HN == 0 && V % REC_BV == 0 && nbs > 0 && t_off >= 0 && t_off < nbs,
                  NATSL_ERR_BAD_SHAPE, "natsl_linear_recurrent_step: bad shape (V a multiple of 8, 0 <= t_off < nbs)");
    NATSL_REQUIRE(H <= 65535 && B <= 65535, NATSL_ERR_TOO_LARGE, "natsl_linear_recurrent_step: B, H <= 65535");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int gdn = rule == NATSL_RULE_GDN, decay = (flags & NATSL_FLAG_DECAY_SKIPPED) ? 1 : 0;
    if (dtype == NATSL_DT_F32)
        return launch_recurrent<float>(q, k, v, g, beta, types_i, h_cur, o, h_cur_out, h_start_out, B, T, H, HN, K, V, nbs, scale,
                                       gdn, decay, use_l2norm, st, h_start, gsum, t_off, 1);
    if (dtype == NATSL_DT_BF16)
        return launch_recurrent<__nv_bfloat16>(q, k, v, g, beta, types_i, h_cur, o, h_cur_out, h_start_out, B, T, H, HN, K, V, nbs,
                                               scale, gdn, decay, use_l2norm, st, h_start, gsum, t_off, 1);
    set_error("natsl_linear_recurrent_step: dtype must be f32 or bf16");
    return NATSL_ERR_UNSUPPORTED;
}

extern "C" int natsl_attn_fwd_fp32(int dtype, const void* q, const void* k, const void* v, const int32_t* types_i, void* o,
                                   float* lse, int B, int T, int HQ, int HKV, int HN, int DK, int DV, int nbs, float scale,
                                   int flags, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(q && k && v && types_i && o && lse, NATSL_ERR_NULL, "natsl_attn_fwd_fp32: null pointer");
    NATSL_REQUIRE(B > 0 && T > 0 && HQ > 0 && HKV > 0 && HN > 0 && HQ % HKV == 0 && HQ % HN == 0 && nbs > 0,
                  NATSL_ERR_BAD_SHAPE, "natsl_attn_fwd_fp32: bad shape");
    NATSL_REQUIRE(HQ <= 65535 && B <= 65535, NATSL_ERR_TOO_LARGE, "natsl_attn_fwd_fp32: B, HQ <= 65535");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int own = (flags & NATSL_FLAG_ATTN_OWN_CHUNK) ? 1 : 0;
    if (dtype == NATSL_DT_F32) return launch_attn_fp32<float>(q, k, v, types_i, o, lse, B, T, HQ, HKV, HN, DK, DV, nbs, scale, own, st);
    if (dtype == NATSL_DT_BF16)
        return launch_attn_fp32<__nv_bfloat16>(q, k, v, types_i, o, lse, B, T, HQ, HKV, HN, DK, DV, nbs, scale, own, st);
    set_error("natsl_attn_fwd_fp32: dtype must be f32 or bf16");
    return NATSL_ERR_UNSUPPORTED;
}
