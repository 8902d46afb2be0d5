// Bandwidth kernels for the steps of the NAtSL layer directly before the hybrid attention op, forward and backward:
//   short causal depthwise convolution + SiLU   (fla ShortConvolution at src/nats/layers/natsl_attn_gdn.py:329-348, 430-447)
//   RMSNorm, optionally fused with the residual add in front of it
//                                               (fla RMSNorm: per-head q/k norms natsl_attn_gdn.py:233-235, 504-505; block
//                                                norms src/nats/models/natsl_attn_gdn/modeling_natsl_attn_gdn.py:62, 110, 138-139)
//   SwiGLU  silu(a) * b                          (fla GatedMLP, modeling_natsl_attn_gdn.py:111-117)
//   mean over each block of tokens               (fla mean_pooling, natsl_attn_gdn.py:412-416; src/nats/ops/utils/pooling.py:26-57)
// All tensors bf16, math in fp32, 16-byte accesses where the row width allows.  Reductions over rows (weight gradients)
// are written as per-CTA partial sums and added up by the caller: no atomics, reproducible results.
#include "common.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t* u = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = unpack_bf16(u[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&f)[8]) {
    *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// ------------------------------------------------------------------------------------------------ short conv + SiLU
constexpr int CONV_W = 4;
constexpr int CONV_TT = 32;          // tokens per thread (forward)

// y[b,t,d] = act(bias[d] + sum_j w[d,j] x[b, t-(W-1)+j, d]); one thread = 8 channels x CONV_TT tokens.
__global__ void __launch_bounds__(128)
short_conv_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                      const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y, int T, int D, int silu) {
    const int cg = blockIdx.x * blockDim.x + threadIdx.x;          // group of 8 channels
    if (cg * 8 >= D) return;
    const int d0 = cg * 8;
    const int t0 = blockIdx.y * CONV_TT, b = blockIdx.z;
    float wt[8][CONV_W], bs[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        bs[c] = bias ? __bfloat162float(bias[d0 + c]) : 0.f;
#pragma unroll
        for (int j = 0; j < CONV_W; ++j) wt[c][j] = __bfloat162float(w[(d0 + c) * CONV_W + j]);
    }
    float win[CONV_W][8];                                           // sliding window: win[j] = x[t-(W-1)+j]
#pragma unroll
    for (int j = 0; j < CONV_W - 1; ++j) {
        const int t = t0 - (CONV_W - 1) + j;
        if (t >= 0) ld8(x + ((long)b * T + t) * D + d0, win[j + 1]);
        else {
#pragma unroll
            for (int c = 0; c < 8; ++c) win[j + 1][c] = 0.f;
        }
    }
    const int t_end = min(T, t0 + CONV_TT);
    for (int t = t0; t < t_end; ++t) {
#pragma unroll
        for (int j = 0; j < CONV_W - 1; ++j)
#pragma unroll
            for (int c = 0; c < 8; ++c) win[j][c] = win[j + 1][c];
        ld8(x + ((long)b * T + t) * D + d0, win[CONV_W - 1]);
        float out[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            float a = bs[c];
#pragma unroll
            for (int j = 0; j < CONV_W; ++j) a += wt[c][j] * win[j][c];
            out[c] = silu ? a * sigmoidf_(a) : a;
        }
        st8(y + ((long)b * T + t) * D + d0, out);
    }
}

// Backward: dpre = dy * act'(pre) with pre recomputed; dx[t] = sum_j w[j] dpre[t+(W-1)-j];
// dw[d,j] = sum_{b,t} dpre[t] x[t-(W-1)+j], dbias[d] = sum dpre: per-(batch, token range) partial sums
// dw_part [B * gridDim.y, D, W + 1] (column W = bias).  One thread = 8 channels x `span` tokens.
__global__ void __launch_bounds__(128)
short_conv_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                      const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ dy,
                      __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_part, int T, int D, int silu, int span) {
    const int cg = blockIdx.x * blockDim.x + threadIdx.x;
    if (cg * 8 >= D) return;
    const int d0 = cg * 8;
    const int t0 = blockIdx.y * span, b = blockIdx.z;
    constexpr int W = CONV_W;
    float wt[8][W], bs[8], dwa[8][W + 1];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        bs[c] = bias ? __bfloat162float(bias[d0 + c]) : 0.f;
#pragma unroll
        for (int j = 0; j < W; ++j) wt[c][j] = __bfloat162float(w[(d0 + c) * W + j]);
#pragma unroll
        for (int j = 0; j <= W; ++j) dwa[c][j] = 0.f;
    }
    auto loadx = [&](int t, float (&f)[8]) {
        if (t >= 0 && t < T) ld8(x + ((long)b * T + t) * D + d0, f);
        else {
#pragma unroll
            for (int c = 0; c < 8; ++c) f[c] = 0.f;
        }
    };
    // dpre at token t (zero outside [0, T)); xw = x[t-(W-1) .. t]
    auto dpre_at = [&](int t, const float (&xw)[W][8], float (&dp)[8]) {
        if (t < 0 || t >= T) {
#pragma unroll
            for (int c = 0; c < 8; ++c) dp[c] = 0.f;
            return;
        }
        float g[8];
        ld8(dy + ((long)b * T + t) * D + d0, g);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            float a = bs[c];
#pragma unroll
            for (int j = 0; j < W; ++j) a += wt[c][j] * xw[j][c];
            if (silu) {
                const float s = sigmoidf_(a);
                dp[c] = g[c] * s * (1.f + a * (1.f - s));
            } else {
                dp[c] = g[c];
            }
        }
    };
    // xs holds x[tt-(W-1) .. tt+(W-1)] (2W-1 rows) for the current tt; dps holds dpre[tt .. tt+(W-1)]
    float xs[2 * W - 1][8], dps[W][8];
#pragma unroll
    for (int i = 0; i < 2 * W - 1; ++i) loadx(t0 - (W - 1) + i, xs[i]);
#pragma unroll
    for (int i = 0; i < W; ++i) {
        float xw[W][8];
#pragma unroll
        for (int j = 0; j < W; ++j)
#pragma unroll
            for (int c = 0; c < 8; ++c) xw[j][c] = xs[i + j][c];
        dpre_at(t0 + i, xw, dps[i]);
    }
    const int t_end = min(T, t0 + span);
    for (int tt = t0; tt < t_end; ++tt) {
        // weight gradient of token tt (tokens of this thread's own range only: each token counted once)
#pragma unroll
        for (int c = 0; c < 8; ++c) {
#pragma unroll
            for (int j = 0; j < W; ++j) dwa[c][j] += dps[0][c] * xs[j][c];
            dwa[c][W] += dps[0][c];
        }
        // dx[tt] = sum_j w[j] dpre[tt + (W-1) - j]
        float o[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            float a = 0.f;
#pragma unroll
            for (int j = 0; j < W; ++j) a += wt[c][j] * dps[W - 1 - j][c];
            o[c] = a;
        }
        st8(dx + ((long)b * T + tt) * D + d0, o);
        // slide by one token
#pragma unroll
        for (int i = 0; i < 2 * W - 2; ++i)
#pragma unroll
            for (int c = 0; c < 8; ++c) xs[i][c] = xs[i + 1][c];
        loadx(tt + W, xs[2 * W - 2]);
#pragma unroll
        for (int i = 0; i < W - 1; ++i)
#pragma unroll
            for (int c = 0; c < 8; ++c) dps[i][c] = dps[i + 1][c];
        {
            float xw[W][8];
#pragma unroll
            for (int j = 0; j < W; ++j)
#pragma unroll
                for (int c = 0; c < 8; ++c) xw[j][c] = xs[W - 1 + j][c];
            dpre_at(tt + W, xw, dps[W - 1]);
        }
    }
    float* out = dw_part + (((long)b * gridDim.y + blockIdx.y) * D + d0) * (W + 1);
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
        for (int j = 0; j <= W; ++j) out[c * (W + 1) + j] = dwa[c][j];
}

// ------------------------------------------------------------------------------------------------ RMSNorm
// One warp per row of D elements; lane owns NV vectors of VEC elements: element (j*32 + lane)*VEC + e.
template <int D>
struct RowShape {
    static constexpr int VEC = (D >= 256) ? 8 : D / 32;
    static constexpr int NV = D / (32 * VEC);
};

// Loads vector j of a row (VEC elements of this lane) as floats.
template <int D>
__device__ __forceinline__ void vec_load(const __nv_bfloat16* row, int lane, int j, float (&f)[RowShape<D>::VEC]) {
    constexpr int VEC = RowShape<D>::VEC;
    const __nv_bfloat16* q = row + (j * 32 + lane) * VEC;
    if constexpr (VEC == 8) {
        ld8(q, f);
    } else {
#pragma unroll
        for (int e = 0; e < VEC; e += 2) {
            const float2 t = unpack_bf16(*reinterpret_cast<const uint32_t*>(q + e));
            f[e] = t.x;
            f[e + 1] = t.y;
        }
    }
}
template <int D>
__device__ __forceinline__ void vec_store(__nv_bfloat16* row, int lane, int j, const float (&f)[RowShape<D>::VEC]) {
    constexpr int VEC = RowShape<D>::VEC;
    __nv_bfloat16* q = row + (j * 32 + lane) * VEC;
    if constexpr (VEC == 8) {
        st8(q, f);
    } else {
#pragma unroll
        for (int e = 0; e < VEC; e += 2) *reinterpret_cast<uint32_t*>(q + e) = pack_bf16(f[e], f[e + 1]);
    }
}
template <int D>
__device__ __forceinline__ void vec_weight(const void* w, int w_f32, int lane, int j, float (&f)[RowShape<D>::VEC]) {
    constexpr int VEC = RowShape<D>::VEC;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
        const int col = (j * 32 + lane) * VEC + e;
        f[e] = w ? (w_f32 ? reinterpret_cast<const float*>(w)[col] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[col])) : 1.f;
    }
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16(x)); }

// s = x (+ res, rounded to bf16: the stored sum is what is normalised);  y = s * rsqrt(mean(s^2) + eps) * w.
// sum_out (may be NULL) receives s.  Two passes over the row (the second one hits the L1 / L2 cache).
template <int D>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res, const void* __restrict__ w,
                   int w_f32, __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ sum_out, long rows, float eps) {
    constexpr int VEC = RowShape<D>::VEC, NV = RowShape<D>::NV;
    const int lane = threadIdx.x & 31;
    const long row = (long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const __nv_bfloat16* xr = x + row * D;
    const __nv_bfloat16* rr = res ? res + row * D : nullptr;
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        float a[VEC];
        vec_load<D>(xr, lane, j, a);
        if (rr) {
            float r[VEC];
            vec_load<D>(rr, lane, j, r);
#pragma unroll
            for (int e = 0; e < VEC; ++e) a[e] = round_bf16(a[e] + r[e]);
            if (sum_out) vec_store<D>(sum_out + row * D, lane, j, a);
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) ss += a[e] * a[e];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / D + eps);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        float a[VEC], ww[VEC];
        vec_load<D>(xr, lane, j, a);
        if (rr) {
            float r[VEC];
            vec_load<D>(rr, lane, j, r);
#pragma unroll
            for (int e = 0; e < VEC; ++e) a[e] = round_bf16(a[e] + r[e]);
        }
        vec_weight<D>(w, w_f32, lane, j, ww);
#pragma unroll
        for (int e = 0; e < VEC; ++e) a[e] = a[e] * rstd * ww[e];
        vec_store<D>(y + row * D, lane, j, a);
    }
}

// Narrow rows (D = 64, 128, 256: the per-head norms): D / 8 lanes per row with 16 bytes each, 32 / (D / 8) rows per warp,
// one pass with the row in registers -- a warp per 128-byte row moves too few bytes per instruction.
template <int D>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_narrow_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                          const void* __restrict__ w, int w_f32, __nv_bfloat16* __restrict__ y,
                          __nv_bfloat16* __restrict__ sum_out, long rows, float eps) {
    constexpr int LPR = D / 8, RPW = 32 / LPR;
    const int lane = threadIdx.x & 31, sub = lane % LPR;
    const long row_raw = ((long)blockIdx.x * 8 + (threadIdx.x >> 5)) * RPW + lane / LPR;
    const bool ok = row_raw < rows;
    const long row = ok ? row_raw : rows - 1;                 // keep every lane in the shuffles
    float a[8], ww[8];
    ld8(x + row * D + sub * 8, a);
    if (res) {
        float r[8];
        ld8(res + row * D + sub * 8, r);
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = round_bf16(a[e] + r[e]);
        if (sum_out && ok) st8(sum_out + row * D + sub * 8, a);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const int col = sub * 8 + e;
        ww[e] = w ? (w_f32 ? reinterpret_cast<const float*>(w)[col] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[col])) : 1.f;
    }
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += a[e] * a[e];
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss / D + eps);
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = a[e] * rstd * ww[e];
    if (ok) st8(y + row * D + sub * 8, a);
}

// dx = rstd (dy w - xhat mean(dy w xhat)) (+ dadd);  dw_part [gridDim.x, D] = per-CTA sums of dy xhat.
template <int D>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ s, const void* __restrict__ w, int w_f32,
                   const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ dadd,
                   __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_part, long rows, float eps) {
    constexpr int VEC = RowShape<D>::VEC, NV = RowShape<D>::NV;
    __shared__ float s_dw[D];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float dwa[NV][VEC];
#pragma unroll
    for (int j = 0; j < NV; ++j)
#pragma unroll
        for (int e = 0; e < VEC; ++e) dwa[j][e] = 0.f;
    for (long row = (long)blockIdx.x * 8 + warp; row < rows; row += (long)gridDim.x * 8) {
        const __nv_bfloat16* sr = s + row * D;
        const __nv_bfloat16* gr = dy + row * D;
        float ss = 0.f, c = 0.f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            float a[VEC], g[VEC], ww[VEC];
            vec_load<D>(sr, lane, j, a);
            vec_load<D>(gr, lane, j, g);
            vec_weight<D>(w, w_f32, lane, j, ww);
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                ss += a[e] * a[e];
                c += g[e] * ww[e] * a[e];
            }
        }
        ss = warp_sum(ss);
        const float rstd = rsqrtf(ss / D + eps);
        c = warp_sum(c) * rstd / D;                       // mean(dy w xhat)
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            float a[VEC], g[VEC], ww[VEC];
            vec_load<D>(sr, lane, j, a);
            vec_load<D>(gr, lane, j, g);
            vec_weight<D>(w, w_f32, lane, j, ww);
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                const float xh = a[e] * rstd;
                dwa[j][e] += g[e] * xh;
                g[e] = rstd * (g[e] * ww[e] - xh * c);
            }
            if (dadd) {
                float r[VEC];
                vec_load<D>(dadd + row * D, lane, j, r);
#pragma unroll
                for (int e = 0; e < VEC; ++e) g[e] += r[e];
            }
            vec_store<D>(dx + row * D, lane, j, g);
        }
    }
    // warps add their sums one after the other: fixed order, one row of shared memory
    for (int wv = 0; wv < 8; ++wv) {
        if (warp == wv) {
#pragma unroll
            for (int j = 0; j < NV; ++j)
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    const int col = (j * 32 + lane) * VEC + e;
                    s_dw[col] = (wv == 0 ? 0.f : s_dw[col]) + dwa[j][e];
                }
        }
        __syncthreads();
    }
    for (int i = threadIdx.x; i < D; i += 256) dw_part[(long)blockIdx.x * D + i] = s_dw[i];
}

// ------------------------------------------------------------------------------------------------ SwiGLU
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y, long n8) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
        float fa[8], fb[8], o[8];
        ld8(a + i * 8, fa);
        ld8(b + i * 8, fb);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = fa[e] * sigmoidf_(fa[e]) * fb[e];
        st8(y + i * 8, o);
    }
}
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b, const __nv_bfloat16* __restrict__ dy,
                  __nv_bfloat16* __restrict__ da, __nv_bfloat16* __restrict__ db, long n8) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
        float fa[8], fb[8], g[8], oa[8], ob[8];
        ld8(a + i * 8, fa);
        ld8(b + i * 8, fb);
        ld8(dy + i * 8, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float s = sigmoidf_(fa[e]);
            oa[e] = g[e] * fb[e] * s * (1.f + fa[e] * (1.f - s));
            ob[e] = g[e] * fa[e] * s;
        }
        st8(da + i * 8, oa);
        st8(db + i * 8, ob);
    }
}

// ------------------------------------------------------------------------------------------------ block mean
// y[b, c, d] = mean over the tokens of block c (the last block may be shorter); one thread = 8 channels of one block.
__global__ void __launch_bounds__(128)
block_mean_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int T, int D, int nbs, int NB) {
    const int cg = blockIdx.x * blockDim.x + threadIdx.x;
    if (cg * 8 >= D) return;
    const int c = blockIdx.y, b = blockIdx.z;
    const int t0 = c * nbs, t1 = min(T, t0 + nbs);
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int t = t0; t < t1; ++t) {
        float f[8];
        ld8(x + ((long)b * T + t) * D + cg * 8, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += f[e];
    }
    const float inv = 1.f / (float)(t1 - t0);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] *= inv;
    st8(y + ((long)b * NB + c) * D + cg * 8, acc);
}

static inline const __nv_bfloat16* bfc(const void* p) { return reinterpret_cast<const __nv_bfloat16*>(p); }
static inline __nv_bfloat16* bfm(void* p) { return reinterpret_cast<__nv_bfloat16*>(p); }

}  // namespace natsl

using namespace natsl;

// Forward with the input tile staged in shared memory: one CTA = 128 channels x 64 tokens (+ 3 halo rows), every load
// issued at once with cp.async; warp s computes the tokens 8 s .. 8 s + 7, a lane four channels.
constexpr int CF_TT = 64, CF_L = 32, CF_CH = 4;
__global__ void __launch_bounds__(256)
short_conv_fwd_tile_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                           const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y, int T, int D, int silu) {
    constexpr int W = CONV_W, XR = CF_TT + W - 1, ROWB = CF_L * CF_CH * 2, CPR = ROWB / 16;
    __shared__ __align__(16) unsigned char xs[XR * ROWB];
    const int tid = threadIdx.x, lane = tid & 31, sr = tid >> 5;
    const int d_cta = blockIdx.x * CF_L * CF_CH, d0 = d_cta + lane * CF_CH;
    const int t0 = blockIdx.y * CF_TT, b = blockIdx.z;
    const bool ch_ok = d0 < D;
    const uint32_t xs_a = smem_u32(xs);
    for (int i = tid; i < XR * CPR; i += 256) {
        const int r = i / CPR, c = i % CPR;
        const int t = t0 - (W - 1) + r, dd = d_cta + c * 8;
        const bool ok = t >= 0 && t < T && dd < D;
        cp_async16(xs_a + r * ROWB + c * 16, ok ? (const void*)(x + ((long)b * T + t) * D + dd) : (const void*)x, ok ? 16 : 0);
    }
    cp_async_commit();
    float wt[CF_CH][W], bs[CF_CH];
#pragma unroll
    for (int c = 0; c < CF_CH; ++c) {
        bs[c] = (bias && ch_ok) ? __bfloat162float(bias[d0 + c]) : 0.f;
#pragma unroll
        for (int j = 0; j < W; ++j) wt[c][j] = ch_ok ? __bfloat162float(w[(d0 + c) * W + j]) : 0.f;
    }
    cp_async_wait<0>();
    __syncthreads();
    static_assert(CF_CH == 4, "a thread reads 8 bytes per row");
    float win[W][CF_CH];
    auto row = [&](int r, float (&f)[CF_CH]) {
        const uint2 v = *reinterpret_cast<const uint2*>(xs + r * ROWB + lane * 8);
        const float2 a = unpack_bf16(v.x), c = unpack_bf16(v.y);
        f[0] = a.x; f[1] = a.y; f[2] = c.x; f[3] = c.y;
    };
    const int ts = sr * 8;
#pragma unroll
    for (int j = 0; j < W - 1; ++j) row(ts + j, win[j + 1]);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
        for (int j = 0; j < W - 1; ++j)
#pragma unroll
            for (int c = 0; c < CF_CH; ++c) win[j][c] = win[j + 1][c];
        row(ts + i + W - 1, win[W - 1]);
        float o[CF_CH];
#pragma unroll
        for (int c = 0; c < CF_CH; ++c) {
            float a = bs[c];
#pragma unroll
            for (int j = 0; j < W; ++j) a += wt[c][j] * win[j][c];
            o[c] = silu ? a * sigmoidf_(a) : a;
        }
        if (ch_ok && t0 + ts + i < T)
            *reinterpret_cast<uint2*>(y + ((long)b * T + t0 + ts + i) * D + d0) = make_uint2(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]));
    }
}

extern "C" int natsl_short_conv_fwd(const void* x, const void* w, const void* bias, void* y, int B, int T, int D, int W,
                                    int silu, void* stream) {
    NATSL_REQUIRE(x && w && y, NATSL_ERR_NULL, "natsl_short_conv_fwd: null pointer");
    NATSL_REQUIRE(B > 0 && T > 0 && D > 0 && D % 8 == 0 && B <= 65535, NATSL_ERR_BAD_SHAPE,
                  "natsl_short_conv_fwd: bad shape (D a multiple of 8)");
    NATSL_REQUIRE(W == CONV_W, NATSL_ERR_UNSUPPORTED, "natsl_short_conv_fwd: kernel size %d is not built (4)", W);
    dim3 grid((D + CF_L * CF_CH - 1) / (CF_L * CF_CH), (T + CF_TT - 1) / CF_TT, B);
    short_conv_fwd_tile_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(bfc(x), bfc(w), bfc(bias), bfm(y), T, D, silu);
    return check_launch("natsl_short_conv_fwd");
}

// The same backward for span = 64 with the tiles staged in shared memory: one CTA = 128 channels x 64 tokens, all loads
// of the x tile (64 + 6 halo rows) and the dy tile (64 + 3) are issued at once with cp.async (the sliding-window form
// above has two loads in flight per thread and is bound by their latency), warp s computes the tokens 8 s .. 8 s + 7 for
// 32 groups of 8 channels, and the eight warps' weight-gradient partials are summed in shared memory in a fixed order:
// one partial per CTA.
constexpr int CB_TT = 64, CB_CG = 32, CB_CH = 4;      // tokens per CTA, threads across channels, channels per thread
__global__ void __launch_bounds__(256, 3)
short_conv_bwd_tile_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                           const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ dy,
                           __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_part, int T, int D, int silu) {
    constexpr int W = CONV_W;
    constexpr int XR = CB_TT + 2 * (W - 1), YR = CB_TT + (W - 1);            // rows of the two tiles
    constexpr int ROWB = CB_CG * CB_CH * 2;                                  // bytes per tile row
    constexpr int CPR = ROWB / 16;                                          // 16-byte chunks per tile row
    extern __shared__ __align__(16) unsigned char smem_cb[];
    unsigned char* xs = smem_cb;
    unsigned char* ys = smem_cb + XR * ROWB;
    const int tid = threadIdx.x, lane = tid & 31, sr = tid >> 5;
    const int d_cta = blockIdx.x * CB_CG * CB_CH;
    const int t0 = blockIdx.y * CB_TT, b = blockIdx.z;
    const int d0 = d_cta + lane * CB_CH;
    const bool ch_ok = d0 < D;
    {
        const uint32_t xs_a = smem_u32(xs), ys_a = smem_u32(ys);
        for (int i = tid; i < XR * CPR; i += 256) {
            const int r = i / CPR, c = i % CPR;
            const int t = t0 - (W - 1) + r, dd = d_cta + c * 8;
            const bool ok = t >= 0 && t < T && dd < D;
            cp_async16(xs_a + r * ROWB + c * 16, ok ? (const void*)(x + ((long)b * T + t) * D + dd) : (const void*)x, ok ? 16 : 0);
        }
        for (int i = tid; i < YR * CPR; i += 256) {
            const int r = i / CPR, c = i % CPR;
            const int t = t0 + r, dd = d_cta + c * 8;
            const bool ok = t < T && dd < D;
            cp_async16(ys_a + r * ROWB + c * 16, ok ? (const void*)(dy + ((long)b * T + t) * D + dd) : (const void*)dy, ok ? 16 : 0);
        }
        cp_async_commit();
    }
    float wt[CB_CH][W], bs[CB_CH], dwa[CB_CH][W + 1];
#pragma unroll
    for (int c = 0; c < CB_CH; ++c) {
        bs[c] = (bias && ch_ok) ? __bfloat162float(bias[d0 + c]) : 0.f;
#pragma unroll
        for (int j = 0; j < W; ++j) wt[c][j] = ch_ok ? __bfloat162float(w[(d0 + c) * W + j]) : 0.f;
#pragma unroll
        for (int j = 0; j <= W; ++j) dwa[c][j] = 0.f;
    }
    cp_async_wait<0>();
    __syncthreads();
    static_assert(CB_CH == 4, "a thread reads 8 bytes per row");
    auto row8 = [&](const unsigned char* tile, int r, float (&f)[CB_CH]) {
        const uint2 v = *reinterpret_cast<const uint2*>(tile + r * ROWB + lane * 8);
        const float2 t0_ = unpack_bf16(v.x), t1_ = unpack_bf16(v.y);
        f[0] = t0_.x; f[1] = t0_.y; f[2] = t1_.x; f[3] = t1_.y;
    };
    // token tt of the tile (0 .. 63 + halo): x rows tt .. tt + 3 of the x tile are its window, dy row tt its gradient.
    // With `own` (a token of this warp's range, inside the sequence) its weight-gradient terms are added while the
    // window is in registers.
    auto dpre_at = [&](int tt, bool own, float (&dp)[CB_CH]) {
        float xw[W][CB_CH];
#pragma unroll
        for (int j = 0; j < W; ++j) row8(xs, tt + j, xw[j]);
        float g[CB_CH];
        row8(ys, tt, g);                                   // zero outside the sequence
#pragma unroll
        for (int c = 0; c < CB_CH; ++c) {
            float a = bs[c];
#pragma unroll
            for (int j = 0; j < W; ++j) a += wt[c][j] * xw[j][c];
            if (silu) {
                const float sg = sigmoidf_(a);
                dp[c] = g[c] * sg * (1.f + a * (1.f - sg));
            } else {
                dp[c] = g[c];
            }
            if (own) {
#pragma unroll
                for (int j = 0; j < W; ++j) dwa[c][j] += dp[c] * xw[j][c];
                dwa[c][W] += dp[c];
            }
        }
    };
    const int ts = sr * 8;                                  // first token of this warp inside the tile
    float dps[W][CB_CH];                                        // dpre[tt .. tt + 3]
#pragma unroll
    for (int i = 1; i < W; ++i) dpre_at(ts + i - 1, true, dps[i]);        // dps[1..3] = dpre[ts .. ts+2] (dy = 0 past T)
#pragma unroll 1
    for (int i = 0; i < 8; ++i) {
        const int tt = ts + i;
#pragma unroll
        for (int k = 0; k < W - 1; ++k)
#pragma unroll
            for (int c = 0; c < CB_CH; ++c) dps[k][c] = dps[k + 1][c];
        dpre_at(tt + W - 1, i + W - 1 < 8, dps[W - 1]);
        if (t0 + tt < T) {
            float o[CB_CH];
#pragma unroll
            for (int c = 0; c < CB_CH; ++c) {
                float a = 0.f;
#pragma unroll
                for (int j = 0; j < W; ++j) a += wt[c][j] * dps[W - 1 - j][c];
                o[c] = a;
            }
            if (ch_ok)
                *reinterpret_cast<uint2*>(dx + ((long)b * T + t0 + tt) * D + d0) = make_uint2(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]));
        }
    }
    // ---- the eight warps' partials -> one per CTA (fixed order)
    __syncthreads();
    float* red = reinterpret_cast<float*>(smem_cb);          // [8 warps][CB_CH * (W + 1)][32 lanes]
#pragma unroll
    for (int c = 0; c < CB_CH; ++c)
#pragma unroll
        for (int j = 0; j <= W; ++j) red[(sr * CB_CH * (W + 1) + c * (W + 1) + j) * CB_CG + lane] = dwa[c][j];
    __syncthreads();
    for (int o = tid; o < CB_CH * (W + 1) * CB_CG; o += 256) {
        float a = 0.f;
#pragma unroll
        for (int s8 = 0; s8 < 8; ++s8) a += red[s8 * CB_CH * (W + 1) * CB_CG + o];
        const int i = o / CB_CG, cgp = o % CB_CG;
        const int dd = d_cta + cgp * CB_CH + i / (W + 1);
        if (dd < D) dw_part[(((long)b * gridDim.y + blockIdx.y) * D + dd) * (W + 1) + i % (W + 1)] = a;
    }
}

extern "C" int natsl_short_conv_bwd(const void* x, const void* w, const void* bias, const void* dy, void* dx, float* dw_part,
                                    int B, int T, int D, int W, int silu, int span, void* stream) {
    NATSL_REQUIRE(x && w && dy && dx && dw_part, NATSL_ERR_NULL, "natsl_short_conv_bwd: null pointer");
    NATSL_REQUIRE(B > 0 && T > 0 && D > 0 && D % 8 == 0 && B <= 65535 && span > 0, NATSL_ERR_BAD_SHAPE,
                  "natsl_short_conv_bwd: bad shape (D a multiple of 8)");
    NATSL_REQUIRE(W == CONV_W, NATSL_ERR_UNSUPPORTED, "natsl_short_conv_bwd: kernel size %d is not built (4)", W);
    const int groups = D / 8;
    if (span == CB_TT) {
        constexpr int smem = ((CB_TT + 2 * (CONV_W - 1)) + (CB_TT + CONV_W - 1)) * CB_CG * CB_CH * 2;
        static_assert(smem >= 8 * CB_CH * (CONV_W + 1) * CB_CG * 4, "the partial sums are reduced over the tiles");
        cudaError_t e = cudaFuncSetAttribute(short_conv_bwd_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) {
            set_error("natsl_short_conv_bwd: cannot reserve %d B of shared memory (%s)", smem, cudaGetErrorString(e));
            return NATSL_ERR_CUDA;
        }
        dim3 grid((D + CB_CG * CB_CH - 1) / (CB_CG * CB_CH), (T + CB_TT - 1) / CB_TT, B);
        short_conv_bwd_tile_kernel<<<grid, 256, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
            bfc(x), bfc(w), bfc(bias), bfc(dy), bfm(dx), dw_part, T, D, silu);
        return check_launch("natsl_short_conv_bwd");
    }
    dim3 grid((groups + 127) / 128, (T + span - 1) / span, B);
    short_conv_bwd_kernel<<<grid, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(bfc(x), bfc(w), bfc(bias), bfc(dy), bfm(dx),
                                                                                   dw_part, T, D, silu, span);
    return check_launch("natsl_short_conv_bwd");
}

#define NATSL_ROW_DISPATCH(CALL)                                                               \
    switch (D) {                                                                               \
        case 64: CALL(64); break;                                                              \
        case 128: CALL(128); break;                                                            \
        case 256: CALL(256); break;                                                            \
        case 512: CALL(512); break;                                                            \
        case 1024: CALL(1024); break;                                                          \
        case 2048: CALL(2048); break;                                                          \
        default:                                                                               \
            set_error("unsupported row width D=%d (64, 128, 256, 512, 1024 or 2048)", D);      \
            return NATSL_ERR_UNSUPPORTED;                                                      \
    }

extern "C" int natsl_rmsnorm_fwd(const void* x, const void* res, const void* w, int w_dtype, void* y, void* sum_out, long rows,
                                 int D, float eps, void* stream) {
    NATSL_REQUIRE(x && y, NATSL_ERR_NULL, "natsl_rmsnorm_fwd: null pointer");
    NATSL_REQUIRE(rows > 0, NATSL_ERR_BAD_SHAPE, "natsl_rmsnorm_fwd: empty input");
    NATSL_REQUIRE(w_dtype == NATSL_DT_BF16 || w_dtype == NATSL_DT_F32, NATSL_ERR_UNSUPPORTED, "natsl_rmsnorm_fwd: weight must be bf16 or f32");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (D == 64 || D == 128 || D == 256) {
        const int rpc = 8 * (32 / (D / 8));                  // rows per CTA
        const unsigned gridn = (unsigned)((rows + rpc - 1) / rpc);
#define NATSL_NARROW(DD) rmsnorm_fwd_narrow_kernel<DD><<<gridn, 256, 0, st>>>(bfc(x), bfc(res), w, w_dtype == NATSL_DT_F32, bfm(y), bfm(sum_out), rows, eps)
        if (D == 64) NATSL_NARROW(64);
        else if (D == 128) NATSL_NARROW(128);
        else NATSL_NARROW(256);
#undef NATSL_NARROW
        return check_launch("natsl_rmsnorm_fwd");
    }
    const unsigned grid = (unsigned)((rows + 7) / 8);
#define NATSL_CALL(DD) rmsnorm_fwd_kernel<DD><<<grid, 256, 0, st>>>(bfc(x), bfc(res), w, w_dtype == NATSL_DT_F32, bfm(y), bfm(sum_out), rows, eps)
    NATSL_ROW_DISPATCH(NATSL_CALL)
#undef NATSL_CALL
    return check_launch("natsl_rmsnorm_fwd");
}

extern "C" int natsl_rmsnorm_bwd(const void* s, const void* w, int w_dtype, const void* dy, const void* dadd, void* dx,
                                 float* dw_part, int n_part, long rows, int D, float eps, void* stream) {
    NATSL_REQUIRE(s && dy && dx && dw_part, NATSL_ERR_NULL, "natsl_rmsnorm_bwd: null pointer");
    NATSL_REQUIRE(rows > 0 && n_part > 0, NATSL_ERR_BAD_SHAPE, "natsl_rmsnorm_bwd: empty input");
    NATSL_REQUIRE(w_dtype == NATSL_DT_BF16 || w_dtype == NATSL_DT_F32, NATSL_ERR_UNSUPPORTED, "natsl_rmsnorm_bwd: weight must be bf16 or f32");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define NATSL_CALL(DD) rmsnorm_bwd_kernel<DD><<<n_part, 256, 0, st>>>(bfc(s), w, w_dtype == NATSL_DT_F32, bfc(dy), bfc(dadd), bfm(dx), dw_part, rows, eps)
    NATSL_ROW_DISPATCH(NATSL_CALL)
#undef NATSL_CALL
    return check_launch("natsl_rmsnorm_bwd");
}

extern "C" int natsl_swiglu_fwd(const void* a, const void* b, void* y, long n, void* stream) {
    NATSL_REQUIRE(a && b && y, NATSL_ERR_NULL, "natsl_swiglu_fwd: null pointer");
    NATSL_REQUIRE(n > 0 && n % 8 == 0, NATSL_ERR_BAD_SHAPE, "natsl_swiglu_fwd: element count must be a positive multiple of 8");
    const long n8 = n / 8;
    const unsigned grid = (unsigned)((n8 + 255) / 256 < 148 * 16 ? (n8 + 255) / 256 : 148 * 16);
    swiglu_fwd_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(bfc(a), bfc(b), bfm(y), n8);
    return check_launch("natsl_swiglu_fwd");
}

extern "C" int natsl_swiglu_bwd(const void* a, const void* b, const void* dy, void* da, void* db, long n, void* stream) {
    NATSL_REQUIRE(a && b && dy && da && db, NATSL_ERR_NULL, "natsl_swiglu_bwd: null pointer");
    NATSL_REQUIRE(n > 0 && n % 8 == 0, NATSL_ERR_BAD_SHAPE, "natsl_swiglu_bwd: element count must be a positive multiple of 8");
    const long n8 = n / 8;
    const unsigned grid = (unsigned)((n8 + 255) / 256 < 148 * 16 ? (n8 + 255) / 256 : 148 * 16);
    swiglu_bwd_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(bfc(a), bfc(b), bfc(dy), bfm(da), bfm(db), n8);
    return check_launch("natsl_swiglu_bwd");
}

extern "C" int natsl_block_mean(const void* x, void* y, int B, int T, int D, int nbs, void* stream) {
    NATSL_REQUIRE(x && y, NATSL_ERR_NULL, "natsl_block_mean: null pointer");
    NATSL_REQUIRE(B > 0 && T > 0 && D > 0 && D % 8 == 0 && nbs > 0 && B <= 65535, NATSL_ERR_BAD_SHAPE,
                  "natsl_block_mean: bad shape (D a multiple of 8)");
    const int NB = (T + nbs - 1) / nbs;
    NATSL_REQUIRE(NB <= 65535, NATSL_ERR_TOO_LARGE, "natsl_block_mean: too many blocks");
    dim3 grid((D / 8 + 127) / 128, NB, B);
    block_mean_kernel<<<grid, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(bfc(x), bfm(y), T, D, nbs, NB);
    return check_launch("natsl_block_mean");
}

// ------------------------------------------------------------------------------------------------ cross entropy rows
// One CTA per row of bf16 logits [rows, vocab]: loss_rows[r] = (logsumexp(l) - l[y]) if y != ignore else 0, and the
// logits are overwritten with their gradient (softmax(l) - onehot(y)) * inv_denom (zero for ignored rows), bf16.
// Two passes over the row: maximum and sum of exponentials (online, fp32), then the gradient.
__global__ void __launch_bounds__(256)
xent_rows_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels, float* __restrict__ loss_rows,
                 int vocab, long long ignore_index, float inv_denom) {
    __shared__ float s_m[8], s_s[8];
    const long row = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    __nv_bfloat16* lr = logits + row * (long)vocab;
    const long long y = labels[row];
    const bool ok = y != ignore_index;
    const int n8 = vocab / 8;
    float m = -INFINITY, s = 0.f;
    for (int i = tid; i < n8; i += 256) {
        float f[8];
        natsl::ld8(lr + i * 8, f);
        float mx = f[0];
#pragma unroll
        for (int e = 1; e < 8; ++e) mx = fmaxf(mx, f[e]);
        const float mn = fmaxf(m, mx);
        float acc = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc += __expf(f[e] - mn);
        s = s * __expf(m - mn) + acc;
        m = mn;
    }
    for (int i = n8 * 8 + tid; i < vocab; i += 256) {          // tail (vocab not a multiple of 8)
        const float f = __bfloat162float(lr[i]);
        const float mn = fmaxf(m, f);
        s = s * __expf(m - mn) + __expf(f - mn);
        m = mn;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
        const float mn = fmaxf(m, m2);
        s = (mn == -INFINITY) ? 0.f : s * __expf(m - mn) + s2 * __expf(m2 - mn);
        m = mn;
    }
    if (lane == 0) {
        s_m[warp] = m;
        s_s[warp] = s;
    }
    __syncthreads();
    float M = s_m[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) M = fmaxf(M, s_m[w]);
    float S = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) S += (s_m[w] == -INFINITY) ? 0.f : s_s[w] * __expf(s_m[w] - M);
    const float lse = M + __logf(S);
    if (tid == 0) loss_rows[row] = ok ? lse - __bfloat162float(lr[ok ? y : 0]) : 0.f;
    __syncthreads();                                           // the target logit is read before the row is overwritten
    const float sc = ok ? inv_denom : 0.f;
    for (int i = tid; i < n8; i += 256) {
        float f[8];
        natsl::ld8(lr + i * 8, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float p = __expf(f[e] - lse) - ((long long)(i * 8 + e) == y ? 1.f : 0.f);
            f[e] = p * sc;
        }
        natsl::st8(lr + i * 8, f);
    }
    for (int i = n8 * 8 + tid; i < vocab; i += 256) {
        const float p = __expf(__bfloat162float(lr[i]) - lse) - ((long long)i == y ? 1.f : 0.f);
        lr[i] = __float2bfloat16(p * sc);
    }
}

extern "C" int natsl_xent_rows(void* logits, const void* labels, float* loss_rows, long rows, int vocab, long ignore_index,
                               float inv_denom, void* stream) {
    NATSL_REQUIRE(logits && labels && loss_rows, NATSL_ERR_NULL, "natsl_xent_rows: null pointer");
    NATSL_REQUIRE(rows > 0 && rows <= 0x7fffffffL && vocab > 0, NATSL_ERR_BAD_SHAPE, "natsl_xent_rows: bad shape");
    NATSL_REQUIRE((reinterpret_cast<uintptr_t>(logits) & 15) == 0 && vocab % 8 == 0, NATSL_ERR_UNSUPPORTED,
                  "natsl_xent_rows: rows must be 16-byte aligned (vocab a multiple of 8)");
    xent_rows_kernel<<<(unsigned)rows, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<__nv_bfloat16*>(logits), reinterpret_cast<const long long*>(labels), loss_rows, vocab,
        (long long)ignore_index, inv_denom);
    return check_launch("natsl_xent_rows");
}
