// Output mixing of the hybrid layer: two-input RMSNorm with per-row mixing weights and a swish gate,
//   y = (x1 * rstd1 * w1 * a + x2 * rstd2 * w2 * b) * g * sigmoid(g),   rstd = 1 / sqrt(mean(x^2) + eps)
// (x1 = linear-branch output, x2 = softmax-branch output, (a, b) = learned per-(token, head) weights).
// Replaces the forward of FusedMultiInputRMSNormGated, src/nats/modules/fused_norm_gate.py:38-182
// (module :1354-1429).  Pure bandwidth: one warp per row of D elements, 16-byte loads and stores, fp32 math.
#include "common.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

__device__ __forceinline__ float load_scalar(const void* p, int dtype, long i) {
    return dtype == NATSL_DT_F32 ? reinterpret_cast<const float*>(p)[i]
                                 : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// D / 8 lanes per row with 16 bytes each (32 / (D / 8) rows per warp): one pass, the three rows in registers.
template <int D>
__global__ void __launch_bounds__(256)
norm_gate_mix_kernel(const __nv_bfloat16* __restrict__ x1, const __nv_bfloat16* __restrict__ x2,
                     const __nv_bfloat16* __restrict__ g, const void* __restrict__ xw, int xw_dtype,
                     const void* __restrict__ w1, const void* __restrict__ w2, int w_dtype,
                     __nv_bfloat16* __restrict__ y, long rows, float eps, int activation) {
    constexpr int LPR = D / 8, RPW = 32 / LPR;
    const int lane = threadIdx.x & 31, sub = lane % LPR;
    const long row_raw = ((long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * RPW + lane / LPR;
    const bool ok = row_raw < rows;
    const long row = ok ? row_raw : rows - 1;                 // keep every lane in the shuffles
    const long base = row * D + sub * 8;
    float a[8], b[8], gg[8];
    auto load = [&](const __nv_bfloat16* p, float* out) {
        const uint4 v = *reinterpret_cast<const uint4*>(p + base);
        const uint32_t* u = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) { float2 f = unpack_bf16(u[i]); out[2 * i] = f.x; out[2 * i + 1] = f.y; }
    };
    load(x1, a);
    load(x2, b);
    load(g, gg);
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) { s1 += a[i] * a[i]; s2 += b[i] * b[i]; }
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) {
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    const float r1 = rsqrtf(s1 / D + eps), r2 = rsqrtf(s2 / D + eps);
    float m1 = 1.f, m2 = 1.f;
    if (xw) { m1 = load_scalar(xw, xw_dtype, row * 2); m2 = load_scalar(xw, xw_dtype, row * 2 + 1); }
    float out[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int d = sub * 8 + i;
        const float ww1 = w1 ? load_scalar(w1, w_dtype, d) : 1.f, ww2 = w2 ? load_scalar(w2, w_dtype, d) : 1.f;
        const float v = a[i] * r1 * ww1 * m1 + b[i] * r2 * ww2 * m2;
        const float sg = 1.f / (1.f + __expf(-gg[i]));
        out[i] = activation == 1 ? v * sg : v * gg[i] * sg;
    }
    if (ok)
        *reinterpret_cast<uint4*>(y + base) = make_uint4(pack_bf16(out[0], out[1]), pack_bf16(out[2], out[3]),
                                                         pack_bf16(out[4], out[5]), pack_bf16(out[6], out[7]));
}


// Backward of the output mixing (src/nats/modules/fused_norm_gate.py:353, :657).  With n = x * rstd and
// v = n1 w1 a + n2 w2 b,  y = v * s(g):   dv = dy s(g),  dg = dy v s'(g),  da = <dv, n1 w1>,  db = <dv, n2 w2>,
// dx = rstd (dn - n mean(dn n)) with dn1 = dv w1 a (dn2 likewise), and the weight gradients dw1 = sum_rows dv n1 a,
// dw2 = sum_rows dv n2 b.  One warp per row, rows strided over a fixed grid; every CTA writes one partial sum of the
// weight gradients (dw_part [grid, 2, D] fp32; the caller adds the CTAs up), so nothing is accumulated atomically.
template <int D>
__global__ void __launch_bounds__(256)
norm_gate_mix_bwd_kernel(const __nv_bfloat16* __restrict__ x1, const __nv_bfloat16* __restrict__ x2,
                         const __nv_bfloat16* __restrict__ g, const void* __restrict__ xw, int xw_dtype,
                         const void* __restrict__ w1, const void* __restrict__ w2, int w_dtype,
                         const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx1,
                         __nv_bfloat16* __restrict__ dx2, __nv_bfloat16* __restrict__ dg, float* __restrict__ dxw,
                         float* __restrict__ dw_part, long rows, float eps, int activation) {
    constexpr int EPL = D / 32;
    __shared__ float s_dw[8][2][D];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float ww1[EPL], ww2[EPL], dw1[EPL], dw2[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        const int d = lane * EPL + i;
        ww1[i] = w1 ? load_scalar(w1, w_dtype, d) : 1.f;
        ww2[i] = w2 ? load_scalar(w2, w_dtype, d) : 1.f;
        dw1[i] = 0.f;
        dw2[i] = 0.f;
    }
    auto load = [&](const __nv_bfloat16* p, long base, float* out) {
#pragma unroll
        for (int i = 0; i < EPL; i += 2) {
            const float2 f = unpack_bf16(*reinterpret_cast<const uint32_t*>(p + base + i));
            out[i] = f.x;
            out[i + 1] = f.y;
        }
    };
    auto store = [&](__nv_bfloat16* p, long base, const float* v) {
#pragma unroll
        for (int i = 0; i < EPL; i += 2) *reinterpret_cast<uint32_t*>(p + base + i) = pack_bf16(v[i], v[i + 1]);
    };
    for (long row = (long)blockIdx.x * 8 + warp; row < rows; row += (long)gridDim.x * 8) {
        const long base = row * D + lane * EPL;
        float a[EPL], b[EPL], gg[EPL], d[EPL];
        load(x1, base, a);
        load(x2, base, b);
        load(g, base, gg);
        load(dy, base, d);
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) { s1 += a[i] * a[i]; s2 += b[i] * b[i]; }
        s1 = warp_sum(s1);
        s2 = warp_sum(s2);
        const float r1 = rsqrtf(s1 / D + eps), r2 = rsqrtf(s2 / D + eps);
        float m1 = 1.f, m2 = 1.f;
        if (xw) { m1 = load_scalar(xw, xw_dtype, row * 2); m2 = load_scalar(xw, xw_dtype, row * 2 + 1); }
        float da = 0.f, db = 0.f, c1 = 0.f, c2 = 0.f;
        float dgo[EPL], dn1[EPL], dn2[EPL];
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const float n1 = a[i] * r1, n2 = b[i] * r2;
            const float v = n1 * ww1[i] * m1 + n2 * ww2[i] * m2;
            const float sg = 1.f / (1.f + __expf(-gg[i]));
            const float s = activation == 1 ? sg : gg[i] * sg;
            const float sp = activation == 1 ? sg * (1.f - sg) : sg * (1.f + gg[i] * (1.f - sg));
            const float dv = d[i] * s;
            dgo[i] = d[i] * v * sp;
            da += dv * n1 * ww1[i];
            db += dv * n2 * ww2[i];
            dw1[i] += dv * n1 * m1;
            dw2[i] += dv * n2 * m2;
            dn1[i] = dv * ww1[i] * m1;
            dn2[i] = dv * ww2[i] * m2;
            c1 += dn1[i] * n1;
            c2 += dn2[i] * n2;
            a[i] = n1;
            b[i] = n2;
        }
        da = warp_sum(da); db = warp_sum(db); c1 = warp_sum(c1) / D; c2 = warp_sum(c2) / D;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            dn1[i] = r1 * (dn1[i] - a[i] * c1);
            dn2[i] = r2 * (dn2[i] - b[i] * c2);
        }
        store(dx1, base, dn1);
        store(dx2, base, dn2);
        store(dg, base, dgo);
        if (dxw && lane == 0) { dxw[row * 2] = da; dxw[row * 2 + 1] = db; }
    }
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        s_dw[warp][0][lane * EPL + i] = dw1[i];
        s_dw[warp][1][lane * EPL + i] = dw2[i];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * D; i += 256) {
        float s = 0.f;
#pragma unroll
        for (int wv = 0; wv < 8; ++wv) s += s_dw[wv][i / D][i % D];
        dw_part[(long)blockIdx.x * 2 * D + i] = s;
    }
}

}  // namespace natsl

extern "C" int natsl_norm_gate_mix(const void* x1, const void* x2, const void* g, const void* xw, int xw_dtype,
                                   const void* w1, const void* w2, int w_dtype, void* y, long rows, int D, float eps,
                                   int activation, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(x1 && x2 && g && y, NATSL_ERR_NULL, "natsl_norm_gate_mix: null pointer");
    NATSL_REQUIRE(rows > 0, NATSL_ERR_BAD_SHAPE, "natsl_norm_gate_mix: empty input");
    NATSL_REQUIRE(activation == 0 || activation == 1, NATSL_ERR_UNSUPPORTED, "natsl_norm_gate_mix: activation 0 (swish) or 1 (sigmoid)");
    NATSL_REQUIRE((xw_dtype == NATSL_DT_BF16 || xw_dtype == NATSL_DT_F32) && (w_dtype == NATSL_DT_BF16 || w_dtype == NATSL_DT_F32),
                  NATSL_ERR_UNSUPPORTED, "natsl_norm_gate_mix: weights must be bf16 or f32");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int wpb = 8;
    const long rpc = (long)wpb * (32 / (D > 0 ? (D / 8 > 0 ? D / 8 : 1) : 1));      // rows per CTA
    const unsigned grid = (unsigned)((rows + rpc - 1) / rpc);
#define NATSL_NG(DD) norm_gate_mix_kernel<DD><<<grid, wpb * 32, 0, st>>>( \
        reinterpret_cast<const __nv_bfloat16*>(x1), reinterpret_cast<const __nv_bfloat16*>(x2), \
        reinterpret_cast<const __nv_bfloat16*>(g), xw, xw_dtype, w1, w2, w_dtype, reinterpret_cast<__nv_bfloat16*>(y), rows, eps, activation)
    if (D == 64) NATSL_NG(64);
    else if (D == 128) NATSL_NG(128);
    else if (D == 256) NATSL_NG(256);
    else {
        set_error("natsl_norm_gate_mix: unsupported row width D=%d (64, 128 or 256)", D);
        return NATSL_ERR_UNSUPPORTED;
    }
#undef NATSL_NG
    return check_launch("natsl_norm_gate_mix");
}

extern "C" int natsl_norm_gate_mix_bwd(const void* x1, const void* x2, const void* g, const void* xw, int xw_dtype,
                                       const void* w1, const void* w2, int w_dtype, const void* dy, void* dx1, void* dx2,
                                       void* dg, float* dxw, float* dw_part, int n_part, long rows, int D, float eps,
                                       int activation, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(x1 && x2 && g && dy && dx1 && dx2 && dg && dw_part, NATSL_ERR_NULL, "natsl_norm_gate_mix_bwd: null pointer");
    NATSL_REQUIRE((xw == nullptr) == (dxw == nullptr), NATSL_ERR_NULL,
                  "natsl_norm_gate_mix_bwd: the mixing weights and their gradient go together");
    NATSL_REQUIRE(rows > 0 && n_part > 0 && n_part <= 65535, NATSL_ERR_BAD_SHAPE, "natsl_norm_gate_mix_bwd: bad sizes");
    NATSL_REQUIRE(activation == 0 || activation == 1, NATSL_ERR_UNSUPPORTED, "natsl_norm_gate_mix_bwd: activation 0 (swish) or 1 (sigmoid)");
    NATSL_REQUIRE((xw_dtype == NATSL_DT_BF16 || xw_dtype == NATSL_DT_F32) && (w_dtype == NATSL_DT_BF16 || w_dtype == NATSL_DT_F32),
                  NATSL_ERR_UNSUPPORTED, "natsl_norm_gate_mix_bwd: weights must be bf16 or f32");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    auto bf = [](const void* p) { return reinterpret_cast<const __nv_bfloat16*>(p); };
    auto bm = [](void* p) { return reinterpret_cast<__nv_bfloat16*>(p); };
#define NATSL_NGB(DD) norm_gate_mix_bwd_kernel<DD><<<n_part, 256, 0, st>>>(bf(x1), bf(x2), bf(g), xw, xw_dtype, w1, w2, w_dtype, \
        bf(dy), bm(dx1), bm(dx2), bm(dg), dxw, dw_part, rows, eps, activation)
    if (D == 64) NATSL_NGB(64);
    else if (D == 128) NATSL_NGB(128);
    else if (D == 256) NATSL_NGB(256);
    else {
        set_error("natsl_norm_gate_mix_bwd: unsupported row width D=%d (64, 128 or 256)", D);
        return NATSL_ERR_UNSUPPORTED;
    }
#undef NATSL_NGB
    return check_launch("natsl_norm_gate_mix_bwd");
}
