// Output of the linear branch for every 64-token chunk ("fwd_o"): one CTA per (chunk, batch,
// head, value-column block).
//   o = scale * [ e^{g + carry} * rstd_q * (q S)  +  tril(qn kn^T * e^{g_i - g_j}) v' ],
//   v' = u - e^{carry} (w S)          (gated delta rule; src/nats/ops/common/chunk_o.py:124-215)
//   v' = v                            (Mamba2/SSD;       src/nats/ops/mamba/chunk_o.py:137-198)
// S is the state the chunk reads (written per chunk by the recurrence kernel), `carry` the decay
// of the skipped blocks before it.  q and k are read raw; their l2 normalisation is folded in as
// row / column scales of the fp32 tiles.  All four products run on the tensor cores with bf16
// operands and fp32 accumulation; P stays in registers between QK^T and P v'.
#include "common.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

constexpr int OUT_THREADS = 256;

template <int K, int VB, bool GDN>
struct OutSmem {
    static constexpr int qs = 0;
    static constexpr int ks = qs + 64 * K * 2;
    static constexpr int ws = ks + 64 * K * 2;
    static constexpr int us = ws + (GDN ? 64 * K * 2 : 0);
    static constexpr int hs = us + 64 * VB * 2;
    static constexpr int vec = hs + K * VB * 2;     // gcs, k_rstd, q_rstd
    static constexpr int total = vec + 3 * 64 * 4;
};

template <int K, int VB, bool GDN>
__global__ void __launch_bounds__(OUT_THREADS)
linear_out_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                  const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ u,
                  const float* __restrict__ gcs, const float* __restrict__ krstd, const __nv_bfloat16* __restrict__ hin,
                  const float* __restrict__ carry_in, __nv_bfloat16* __restrict__ o, int T, int H, int V, float scale,
                  int mode) {
    // mode bit 0: l2-normalise q (and k through k_rstd); bit 1: no own-chunk term (P = 0), the mode in which only
    // the softmax branch covers the current chunk (chunk_o.py:210-211)
    const int use_l2norm = mode & 1;
    const bool own = !(mode & 2);
    using L = OutSmem<K, VB, GDN>;
    constexpr int NH = VB / 16;          // n-tiles per warp (half of the block's columns)
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, qd = lane & 3;
    const int NT = (T + 63) / 64;
    const int c = blockIdx.x;
    const int vblk = blockIdx.y % (V / VB), h = blockIdx.y / (V / VB), b = blockIdx.z;
    const int v0 = vblk * VB;
    const int valid = min(64, T - c * 64);
    const long tok0 = (long)b * T + (long)c * 64;
    const int rw = warp & 3, cgp = warp >> 2;
    const int r0 = rw * 16, n_base = cgp * (VB / 2);

    unsigned char* qs_p = smem + L::qs;
    unsigned char* us_p = smem + L::us;
    unsigned char* hs_p = smem + L::hs;
    float* s_g = reinterpret_cast<float*>(smem + L::vec);
    float* s_kr = s_g + 64;
    float* s_qr = s_kr + 64;
    const uint32_t qs = smem_u32(qs_p), ks = smem_u32(smem + L::ks), ws = smem_u32(smem + L::ws), us = smem_u32(us_p),
                   hs = smem_u32(hs_p);

    load_tile_async<64, K, OUT_THREADS>(qs, q + (tok0 * H + h) * K, (long)H * K, valid, tid);
    load_tile_async<64, K, OUT_THREADS>(ks, k + (tok0 * H + h) * K, (long)H * K, valid, tid);
    cp_async_commit();
    if (GDN) load_tile_async<64, K, OUT_THREADS>(ws, w + (tok0 * H + h) * K, (long)H * K, valid, tid);
    load_tile_async<64, VB, OUT_THREADS>(us, u + (tok0 * H + h) * V + v0, (long)H * V, valid, tid);
    load_tile_async<K, VB, OUT_THREADS>(hs, hin + ((((long)b * NT + c) * H + h) * K) * V + v0, V, K, tid);
    cp_async_commit();
    if (tid < 64) {
        int r = min(tid, valid - 1);
        s_g[tid] = gcs[(tok0 + r) * H + h];
        s_kr[tid] = (krstd && tid < valid) ? krstd[(tok0 + tid) * H + h] : (krstd ? 0.f : 1.f);
    }
    const float carry = carry_in[((long)b * NT + c) * H + h];
    cp_async_wait<1>();
    __syncthreads();

    // ---- q row norms
    {
        constexpr int CPR = K / 8;
        constexpr int RPP = 32 / CPR;
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
            for (int off = CPR / 2; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
            if (cc == 0) s_qr[r] = use_l2norm ? rsqrtf(ss + 1e-6f) : 1.0f;
        }
    }
    __syncthreads();

    // ---- P = tril(qn kn^T * e^{g_i - g_j}) as bf16 A fragments
    uint32_t pa[4][4];
    {
        float acc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll 2
        for (int kk = 0; kk < K / 16; ++kk) {
            uint32_t a[4];
            load_a<K * 2>(qs, r0, kk * 16, lane, a);
            for (int p = 0; p <= rw; ++p) {
                uint32_t bb[4];
                load_b_nk<K * 2>(ks, p * 16, kk * 16, lane, bb);
                mma_bf16(acc[2 * p], a, bb[0], bb[1]);
                mma_bf16(acc[2 * p + 1], a, bb[2], bb[3]);
            }
        }
        const int ia = r0 + gq, ib = ia + 8;
        const float qa = s_qr[ia], qb = s_qr[ib], ga = s_g[ia], gb = s_g[ib];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            float pv[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int i = (e >> 1) ? ib : ia;
                int j = nt * 8 + qd * 2 + (e & 1);
                float val = 0.f;
                if (own && i >= j && j < valid)
                    val = acc[nt][e] * ((e >> 1) ? qb : qa) * s_kr[j] * __expf(((e >> 1) ? gb : ga) - s_g[j]);
                pv[e] = val;
            }
            pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(pv[0], pv[1]);
            pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(pv[2], pv[3]);
        }
    }
    cp_async_wait<0>();
    __syncthreads();

    // ---- q S and w S
    float accq[NH][4], accw[GDN ? NH : 1][4];
#pragma unroll
    for (int i = 0; i < NH; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            accq[i][j] = 0.f;
            if (GDN) accw[i][j] = 0.f;
        }
#pragma unroll 2
    for (int kk = 0; kk < K / 16; ++kk) {
        uint32_t aq[4], aw[4];
        load_a<K * 2>(qs, r0, kk * 16, lane, aq);
        if (GDN) load_a<K * 2>(ws, r0, kk * 16, lane, aw);
#pragma unroll
        for (int p = 0; p < NH / 2; ++p) {
            uint32_t bb[4];
            load_b_kn<VB * 2>(hs, kk * 16, n_base + p * 16, lane, bb);
            mma_bf16(accq[2 * p], aq, bb[0], bb[1]);
            mma_bf16(accq[2 * p + 1], aq, bb[2], bb[3]);
            if (GDN) {
                mma_bf16(accw[2 * p], aw, bb[0], bb[1]);
                mma_bf16(accw[2 * p + 1], aw, bb[2], bb[3]);
            }
        }
    }
    const int ia = r0 + gq, ib = ia + 8;
    if (GDN) {
        // v' = u - e^{carry} (w S), written over u
        const float ec = __expf(carry);
#pragma unroll
        for (int nt = 0; nt < NH; ++nt) {
            int ch = (n_base >> 3) + nt;
            uint32_t* pa_ = reinterpret_cast<uint32_t*>(us_p + swz<VB * 2>(ia, ch) + qd * 4);
            uint32_t* pb_ = reinterpret_cast<uint32_t*>(us_p + swz<VB * 2>(ib, ch) + qd * 4);
            float2 ua = unpack_bf16(*pa_), ub = unpack_bf16(*pb_);
            *pa_ = pack_bf16(ua.x - ec * accw[nt][0], ua.y - ec * accw[nt][1]);
            *pb_ = pack_bf16(ub.x - ec * accw[nt][2], ub.y - ec * accw[nt][3]);
        }
    }
    {
        const float fa = s_qr[ia] * __expf(s_g[ia] + carry), fb = s_qr[ib] * __expf(s_g[ib] + carry);
#pragma unroll
        for (int nt = 0; nt < NH; ++nt) {
            accq[nt][0] *= fa; accq[nt][1] *= fa;
            accq[nt][2] *= fb; accq[nt][3] *= fb;
        }
    }
    __syncthreads();

    // ---- + P v'
    for (int kk = 0; kk <= rw; ++kk) {
#pragma unroll
        for (int p = 0; p < NH / 2; ++p) {
            uint32_t bb[4];
            load_b_kn<VB * 2>(us, kk * 16, n_base + p * 16, lane, bb);
            mma_bf16(accq[2 * p], pa[kk], bb[0], bb[1]);
            mma_bf16(accq[2 * p + 1], pa[kk], bb[2], bb[3]);
        }
    }
    // ---- stage over the (now idle) state tile and store
#pragma unroll
    for (int nt = 0; nt < NH; ++nt) {
        int ch = (n_base >> 3) + nt;
        *reinterpret_cast<uint32_t*>(hs_p + swz<VB * 2>(ia, ch) + qd * 4) = pack_bf16(accq[nt][0] * scale, accq[nt][1] * scale);
        *reinterpret_cast<uint32_t*>(hs_p + swz<VB * 2>(ib, ch) + qd * 4) = pack_bf16(accq[nt][2] * scale, accq[nt][3] * scale);
    }
    __syncthreads();
    store_tile<64, VB, OUT_THREADS>(hs_p, o + (tok0 * H + h) * V + v0, (long)H * V, valid, tid);
}

template <int K, int VB, bool GDN>
static int launch_out(const void* q, const void* k, const void* w, const void* u, const float* gcs, const float* krstd,
                      const void* hin, const float* carry, void* o, int B, int T, int H, int V, float scale,
                      int mode, cudaStream_t st) {
    using L = OutSmem<K, VB, GDN>;
    auto kern = linear_out_kernel<K, VB, GDN>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::total);
    if (e != cudaSuccess) {
        set_error("natsl_linear_fwd_o: cannot reserve %d B of shared memory (%s)", L::total, cudaGetErrorString(e));
        return NATSL_ERR_CUDA;
    }
    const int NT = (T + 63) / 64;
    dim3 grid(NT, H * (V / VB), B);
    kern<<<grid, OUT_THREADS, L::total, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(q), reinterpret_cast<const __nv_bfloat16*>(k),
        reinterpret_cast<const __nv_bfloat16*>(w), reinterpret_cast<const __nv_bfloat16*>(u), gcs, krstd,
        reinterpret_cast<const __nv_bfloat16*>(hin), carry, reinterpret_cast<__nv_bfloat16*>(o), T, H, V, scale,
        mode);
    return check_launch("natsl_linear_fwd_o");
}

}  // namespace natsl

extern "C" int natsl_linear_fwd_o(int rule, const void* q, const void* k, const void* w, const void* u,
                                  const float* gcs, const float* k_rstd, const void* h, const float* carry, void* o,
                                  int B, int T, int H, int K, int V, float scale, int mode, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(q && k && u && gcs && h && carry && o, NATSL_ERR_NULL, "natsl_linear_fwd_o: null pointer");
    NATSL_REQUIRE(rule == NATSL_RULE_GDN || rule == NATSL_RULE_MAMBA, NATSL_ERR_UNSUPPORTED,
                  "natsl_linear_fwd_o: unknown rule %d", rule);
    NATSL_REQUIRE(rule != NATSL_RULE_GDN || w, NATSL_ERR_NULL, "natsl_linear_fwd_o: w is required for the delta rule");
    NATSL_REQUIRE(B > 0 && T > 0 && H > 0, NATSL_ERR_BAD_SHAPE, "natsl_linear_fwd_o: empty shape");
    NATSL_REQUIRE(B <= 65535 && (long)H * (V / 64 + 1) <= 65535, NATSL_ERR_TOO_LARGE,
                  "natsl_linear_fwd_o: grid too large (B=%d H=%d)", B, H);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define NATSL_OUT_ARGS q, k, w, u, gcs, k_rstd, h, carry, o, B, T, H, V, scale, mode, st
    const bool gdn = rule == NATSL_RULE_GDN;
    if (K == 128 && V % 128 == 0) return gdn ? launch_out<128, 128, true>(NATSL_OUT_ARGS) : launch_out<128, 128, false>(NATSL_OUT_ARGS);
    if (K == 128 && V % 64 == 0) return gdn ? launch_out<128, 64, true>(NATSL_OUT_ARGS) : launch_out<128, 64, false>(NATSL_OUT_ARGS);
    if (K == 64 && V % 128 == 0) return gdn ? launch_out<64, 128, true>(NATSL_OUT_ARGS) : launch_out<64, 128, false>(NATSL_OUT_ARGS);
    if (K == 64 && V % 64 == 0) return gdn ? launch_out<64, 64, true>(NATSL_OUT_ARGS) : launch_out<64, 64, false>(NATSL_OUT_ARGS);
#undef NATSL_OUT_ARGS
    set_error("natsl_linear_fwd_o: unsupported head dims K=%d V=%d (K in {64,128}, V multiple of 64)", K, V);
    return NATSL_ERR_UNSUPPORTED;
}
