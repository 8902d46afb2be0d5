// Gated-delta-rule chunk preparation on the 5th-generation tensor cores (head dims K = V = 128).
// Same inputs, outputs and conventions as gdn_prep.cu (the mma.sync kernel, kept for the other head dims):
//   k_rstd, q_rstd, gcs, A = strictLower(beta_i (kn_i . kn_j) e^{gcs_i - gcs_j}),
//   [u | w] = (I + A)^-1 [v beta | kn beta e^{gcs}],  P = tril(qn kn^T e^{gcs_i - gcs_j})
// (src/nats/ops/common/chunk_scaled_dot_kkt.py:105-126, src/nats/ops/utils/solve_tril.py:350-447,
//  src/nats/ops/gated_delta_rule/wy_fast.py:123-153, src/nats/ops/common/chunk_o.py:166,188,202-203).
//
// One CTA per (batch, head, 64-token chunk), 160 threads, 128 TMEM columns, ~52 KB of shared memory (four CTAs per SM):
//   warp 4      TMA producer (k, q tiles at the start, the v tile once A is no longer needed; 128-byte swizzle)
//               and single-thread MMA issuer;
//   warps 0-3   one thread per TMEM lane.
// Steps:
//   1. D1 = [k ; q] k^T            one stacked 128 x 64 x 128 product into TMEM (rows 0-63: K K^T, rows 64-127: Q K^T);
//   2. row norms of k from the diagonal of D1, A (fp32, shared memory) from rows 0-63, P (bf16, global memory,
//      one 128-byte row per thread) from rows 64-127;
//   3. Ai = (I + A)^-1 like the reference does it: the four 16 x 16 diagonal blocks by forward substitution in fp32,
//      the blocks below by the block recursion Ai_ij = -X_ii sum_{j<=m<i} A_im Ai_mj, evaluated per panel of eight
//      columns (the columns of an inverse are independent of one another) with tf32 mma.sync products, fp32
//      accumulation; Ai diag(beta) and Ai diag(beta rstd e^{gcs}) are written as two bf16 operand tiles, so the
//      right-hand sides never have to be scaled in shared memory;
//   4. D2 = [v^T (Ai diag beta)^T | k^T (Ai diag(..))^T]: the raw v and k tiles are the (MN-major) A operands,
//      features in the TMEM lanes, tokens in the columns: no accumulator row is wasted;
//   5. w, then u, go from TMEM through a [token][feature] staging tile (written feature by feature, which is
//      conflict-free) to global memory with TMA stores; P leaves the same way.
// The decay carried over skipped blocks multiplies w by one scalar per chunk and is applied by the consumers.
// Every mbarrier wait is bounded: on expiry the status word is set and the CTA runs on to its teardown.
#include "tc_common.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

constexpr int PT_THREADS = 160;
constexpr int PT_EPI = 128;
constexpr uint32_t PT_TMEM_COLS = 128;
constexpr int PT_A_LD = 68;                  // fp32 row pitch of A: conflict-free 16-byte row stores and fragment loads

struct PtSmem {
    // [k sub-tile 0][q sub-tile 0][k sub-tile 1][q sub-tile 1], each [64 tokens][64 features] = 8 KB: the stacked
    // [k ; q] operand of the first product.  The q sub-tiles are reused: first sub-tile 0 for staging P, then both for
    // the two Ai operand tiles.
    static constexpr int kq = 0;
    // fp32 A [64][68] (diagonal blocks replaced by their inverses); once Ai is formed the v tile (2 sub-tiles, 16 KB)
    // is loaded over it -- it is needed by the last product only, and this is what lets four CTAs share an SM
    static constexpr int As = 32768;
    static constexpr int v = As;
    static constexpr int scr = As + 64 * PT_A_LD * 4;        // per warp [16][8] fp32: accumulator -> B-fragment exchange
    static constexpr int vec = scr + 4 * 512;                // gcs, beta, k rstd, w scale, q rstd: 5 x 64 floats
    static constexpr int bars = vec + 5 * 64 * 4;
    static constexpr int total = bars + 64;
    static constexpr int aiu = kq + 8192, aiw = kq + 24576;  // Ai diag(beta), Ai diag(beta rstd e^{gcs}): [64][64] bf16
    static constexpr int pst = kq + 8192;                    // P staging [64][64] bf16
    static_assert(As % 1024 == 0 && 64 * PT_A_LD * 4 >= 16384, "the v tile must fit over A, 1024-byte aligned");
    static_assert(4 * (total + 1024) <= 232448, "four CTAs per SM");
};

__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

#ifdef NATSL_PREP_TIMING
// scratch builds only: cycle stamps of thread 0 (slots 0-9) and thread 64 (slots 10-19) of every CTA
__device__ long long* g_prep_ts = nullptr;
#define PT_STAMP(slot)                                                                                        \
    do {                                                                                                      \
        if (g_prep_ts && (tid == 0 || tid == 64))                                                             \
            g_prep_ts[(((long)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 20 + (tid ? 10 : 0) + (slot)] = clock64(); \
    } while (0)
#else
#define PT_STAMP(slot)
#endif

__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}
// D (16 x 8, fp32) += A (16 x 8, tf32, row) * B (8 x 8, tf32, col)
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// A fragments (two k-steps of 8) of the 16 x 16 block at (row0, col0) of the fp32 matrix As
__device__ __forceinline__ void load_a_tf32(const float* As, int row0, int col0, int lane, uint32_t (&a)[2][4]) {
    const int g = lane >> 2, q = lane & 3;
#pragma unroll
    for (int s = 0; s < 2; ++s) {
        const float* p = As + (row0 + g) * PT_A_LD + col0 + 8 * s + q;
        a[s][0] = to_tf32(p[0]);
        a[s][1] = to_tf32(p[8 * PT_A_LD]);
        a[s][2] = to_tf32(p[4]);
        a[s][3] = to_tf32(p[8 * PT_A_LD + 4]);
    }
}
// A 16 x 8 accumulator (rows g, g+8; columns 2q, 2q+1) -> the B fragments of the same matrix used as a right factor
__device__ __forceinline__ void acc_to_b(float* scr, const float (&c)[4], int lane, uint32_t (&b)[2][2]) {
    const int g = lane >> 2, q = lane & 3;
    *reinterpret_cast<float2*>(scr + g * 8 + 2 * q) = make_float2(c[0], c[1]);
    *reinterpret_cast<float2*>(scr + (g + 8) * 8 + 2 * q) = make_float2(c[2], c[3]);
    __syncwarp();
#pragma unroll
    for (int s = 0; s < 2; ++s) {
        b[s][0] = to_tf32(scr[(8 * s + q) * 8 + g]);
        b[s][1] = to_tf32(scr[(8 * s + q + 4) * 8 + g]);
    }
    __syncwarp();
}

// One panel of eight columns [c0, c0+8) of Ai (c0 = 16 j + 8 half), by one warp: zero above block row j, X_jj's half,
// then block rows j+1..3 by the recursion; every 16 x 8 block is written, scaled per column, into both operand tiles.
__device__ __forceinline__ void inverse_panel(const float* As, float* scr, unsigned char* aiu, unsigned char* aiw,
                                              const float* s_beta, const float* s_wsc, int j, int half, int lane) {
    const int g = lane >> 2, q = lane & 3;
    const int c0 = 16 * j + 8 * half;
    const int chunk = c0 >> 3;
    const int ca = c0 + 2 * q;
    const float bu0 = s_beta[ca], bu1 = s_beta[ca + 1], bw0 = s_wsc[ca], bw1 = s_wsc[ca + 1];
    for (int r = lane; r < 16 * j; r += 32) {
        *reinterpret_cast<uint4*>(aiu + swz<128>(r, chunk)) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(aiw + swz<128>(r, chunk)) = make_uint4(0, 0, 0, 0);
    }
    auto put = [&](int blk, const float (&y)[4]) {
        const int ra = 16 * blk + g, rb = ra + 8;
        *reinterpret_cast<uint32_t*>(aiu + swz<128>(ra, chunk) + q * 4) = pack_bf16(y[0] * bu0, y[1] * bu1);
        *reinterpret_cast<uint32_t*>(aiu + swz<128>(rb, chunk) + q * 4) = pack_bf16(y[2] * bu0, y[3] * bu1);
        *reinterpret_cast<uint32_t*>(aiw + swz<128>(ra, chunk) + q * 4) = pack_bf16(y[0] * bw0, y[1] * bw1);
        *reinterpret_cast<uint32_t*>(aiw + swz<128>(rb, chunk) + q * 4) = pack_bf16(y[2] * bw0, y[3] * bw1);
    };
    uint32_t yb[4][2][2];                        // B fragments of the panel's blocks, by block row
    {
        float y[4];
        const float* p = As + (16 * j + g) * PT_A_LD + c0 + 2 * q;
        y[0] = p[0]; y[1] = p[1]; y[2] = p[8 * PT_A_LD]; y[3] = p[8 * PT_A_LD + 1];
        put(j, y);
#pragma unroll
        for (int m = 0; m < 3; ++m)
            if (m == j) acc_to_b(scr, y, lane, yb[m]);
    }
#pragma unroll
    for (int i = 1; i < 4; ++i) {
        if (i > j) {
            float t[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int m = 0; m < 3; ++m) {
                if (m >= j && m < i) {
                    uint32_t a[2][4];
                    load_a_tf32(As, 16 * i, 16 * m, lane, a);
                    mma_tf32(t, a[0], yb[m][0][0], yb[m][0][1]);
                    mma_tf32(t, a[1], yb[m][1][0], yb[m][1][1]);
                }
            }
            uint32_t tb[2][2];
            acc_to_b(scr, t, lane, tb);
            uint32_t x[2][4];
            load_a_tf32(As, 16 * i, 16 * i, lane, x);
            float y[4] = {0.f, 0.f, 0.f, 0.f};
            mma_tf32(y, x[0], tb[0][0], tb[0][1]);
            mma_tf32(y, x[1], tb[1][0], tb[1][1]);
#pragma unroll
            for (int e = 0; e < 4; ++e) y[e] = -y[e];
            put(i, y);
            if (i < 3) acc_to_b(scr, y, lane, yb[i]);
        }
    }
}

__global__ void __launch_bounds__(PT_THREADS, 4)
gdn_prep_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_w,
                   const __grid_constant__ CUtensorMap map_u, const __grid_constant__ CUtensorMap map_p, int has_q,
                   const float* __restrict__ g, const void* __restrict__ beta, int beta_dtype,
                   float* __restrict__ gcs_out, float* __restrict__ krstd_out, float* __restrict__ qrstd_out, int T,
                   int H, int use_l2norm, int* status) {
    using L = PtSmem;
    constexpr int K = 128;
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t sbase = smem_u32(smem);
    if ((sbase & 1023u) != 0) {
        if (tid == 0) atomicExch(status, 2);
        return;
    }
    const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int t0 = c * 64;
    const int valid = min(64, T - t0);
    const long tok0 = (long)b * T + t0;

    float* As = reinterpret_cast<float*>(smem + L::As);
    float* s_gcs = reinterpret_cast<float*>(smem + L::vec);
    float* s_beta = s_gcs + 64;
    float* s_rstd = s_beta + 64;
    float* s_wsc = s_rstd + 64;
    float* s_qr = s_wsc + 64;
    const uint32_t bar_load = sbase + L::bars, bar_d1 = bar_load + 8, bar_ai = bar_load + 16, bar_d2w = bar_load + 24,
                   bar_v = bar_load + 32, bar_d2u = bar_load + 40;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::bars + 48);

    PT_STAMP(0);
    if (tid == 0) {
        mbar_init(bar_load, 1);
        mbar_init(bar_d1, 1);
        mbar_init(bar_ai, PT_EPI);
        mbar_init(bar_d2w, 1);
        mbar_init(bar_v, 1);
        mbar_init(bar_d2u, 1);
        mbar_fence_init();
    }
    if (warp == 4) tmem_alloc(smem_u32(tmem_slot), PT_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    PT_STAMP(1);

    if (warp == 4) {
        // ------------------------------------------------------------ TMA producer + MMA issuer
        if (lane == 0) {
            mbar_expect_tx(bar_load, has_q ? 32768 : 16384);
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
                tma_load_4d(sbase + L::kq + sub * 16384, &map_k, sub * 64, h, t0, b, bar_load);
                if (has_q) tma_load_4d(sbase + L::kq + sub * 16384 + 8192, &map_q, sub * 64, h, t0, b, bar_load);
            }
            // v is only needed at the very end: warm L2 now, load it when A is dead
            tma_prefetch_4d(&map_v, 0, h, t0, b);
            tma_prefetch_4d(&map_v, 64, h, t0, b);
        }
        __syncwarp();
        mbar_wait(bar_load, 0, status);
        if (lane == 0) {
            constexpr uint32_t id_1 = umma_idesc_bf16(128, 64, false);
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < K / 16; ++kk) {
                const uint64_t d = umma_desc(sbase + L::kq + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
                umma_ss(tmem, d, d, id_1, kk > 0);
            }
            umma_commit(bar_d1);
        }
        __syncwarp();
        mbar_wait(bar_ai, 0, status);
        if (lane == 0) {
            constexpr uint32_t id_2 = umma_idesc_bf16(128, 64, false) | (1u << 15);      // A MN-major (features x tokens)
            // every thread has finished with A (and fenced): the v tile may land on it
            mbar_expect_tx(bar_v, 16384);
            tma_load_4d(sbase + L::v, &map_v, 0, h, t0, b, bar_v);
            tma_load_4d(sbase + L::v + 8192, &map_v, 64, h, t0, b, bar_v);
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const uint64_t ak = umma_desc(sbase + L::kq + kk * 2048, 16384, 1024);
                const uint64_t bw = umma_desc(sbase + L::aiw + kk * 32, 16, 1024);
                umma_ss(tmem + 64, ak, bw, id_2, kk > 0);
            }
            umma_commit(bar_d2w);
        }
        __syncwarp();
        mbar_wait(bar_v, 0, status);
        if (lane == 0) {
            constexpr uint32_t id_2 = umma_idesc_bf16(128, 64, false) | (1u << 15);
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const uint64_t av = umma_desc(sbase + L::v + kk * 2048, 8192, 1024);
                const uint64_t bu = umma_desc(sbase + L::aiu + kk * 32, 16, 1024);
                umma_ss(tmem, av, bu, id_2, kk > 0);
            }
            umma_commit(bar_d2u);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ one thread per TMEM lane
        const int row = tid;                                   // D1: k row (0-63) or q row (64-127); D2: feature
        const uint32_t t_lane = tmem + ((uint32_t)(warp * 32) << 16);
        if (warp == 0) {
            // gcs = inclusive cumsum of g over the chunk (two elements per lane), beta
            float x0 = 0.f, x1 = 0.f, b0 = 0.f, b1 = 0.f;
            const long g0 = (tok0 + lane) * H + h, g1 = (tok0 + lane + 32) * H + h;
            if (lane < valid) {
                x0 = g[g0];
                b0 = beta_dtype == NATSL_DT_F32 ? reinterpret_cast<const float*>(beta)[g0]
                                                : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(beta)[g0]);
            }
            if (lane + 32 < valid) {
                x1 = g[g1];
                b1 = beta_dtype == NATSL_DT_F32 ? reinterpret_cast<const float*>(beta)[g1]
                                                : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(beta)[g1]);
            }
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float a0 = __shfl_up_sync(0xffffffffu, x0, o), a1 = __shfl_up_sync(0xffffffffu, x1, o);
                if (lane >= o) {
                    x0 += a0;
                    x1 += a1;
                }
            }
            x1 += __shfl_sync(0xffffffffu, x0, 31);
            s_gcs[lane] = x0;
            s_gcs[lane + 32] = x1;
            s_beta[lane] = b0;
            s_beta[lane + 32] = b1;
            if (lane < valid) gcs_out[g0] = x0;
            if (lane + 32 < valid) gcs_out[g1] = x1;
        }
        mbar_wait(bar_load, 0, status);
        PT_STAMP(2);
        if (warp >= 2 && has_q) {
            // q row norms (one row per thread; the swizzle makes the 16-byte reads of eight rows conflict-free)
            const int r = row - 64;
            float ss = 0.f;
#pragma unroll
            for (int sub = 0; sub < 2; ++sub)
#pragma unroll
                for (int cc = 0; cc < 8; ++cc) {
                    const uint4 xv = *reinterpret_cast<const uint4*>(smem + L::kq + sub * 16384 + 8192 + swz<128>(r, cc));
                    const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xv);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = unpack_bf16(xw[e]);
                        ss += f.x * f.x + f.y * f.y;
                    }
                }
            const float rs = use_l2norm ? rsqrtf(ss + 1e-6f) : 1.0f;
            s_qr[r] = rs;
            if (r < valid && qrstd_out) qrstd_out[(tok0 + r) * H + h] = rs;
        }
        mbar_wait(bar_d1, 0, status);
        tc_fence_after();
        PT_STAMP(3);
        if (warp < 2) {
            // k row norms from the diagonal of K K^T: row i of warp w has its diagonal in columns [32 w, 32 w + 32)
            uint32_t r[32];
            tmem_ld32(t_lane + 32 * warp, r);
            tmem_ld_wait();
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (i == lane) d = __uint_as_float(r[i]);
            const float rs = use_l2norm ? rsqrtf(d + 1e-6f) : 1.0f;
            s_rstd[row] = rs;
            if (row < valid) krstd_out[(tok0 + row) * H + h] = rs;
        }
        epi_barrier();                      // gcs, beta, both row norms are known; the q tile has been read for the last time
        PT_STAMP(4);
        if (warp < 2) {
            const float gi = s_gcs[row];
            const float bi = s_beta[row] * s_rstd[row];
            s_wsc[row] = bi * __expf(gi);
#pragma unroll 1
            for (int hh = 0; hh <= warp; ++hh) {           // columns above the row's 32-column group are never read
                uint32_t r[32];
                tmem_ld32(t_lane + 32 * hh, r);
                tmem_ld_wait();
#pragma unroll
                for (int j4 = 0; j4 < 32; j4 += 4) {
                    const int j = 32 * hh + j4;
                    const float4 gj = *reinterpret_cast<const float4*>(s_gcs + j);
                    const float4 rj = *reinterpret_cast<const float4*>(s_rstd + j);
                    // strictly below the diagonal; the exponent is clamped so that the masked entries stay finite
                    float4 a;
                    a.x = (row > j ? bi : 0.f) * rj.x * __uint_as_float(r[j4]) * __expf(fminf(gi - gj.x, 0.f));
                    a.y = (row > j + 1 ? bi : 0.f) * rj.y * __uint_as_float(r[j4 + 1]) * __expf(fminf(gi - gj.y, 0.f));
                    a.z = (row > j + 2 ? bi : 0.f) * rj.z * __uint_as_float(r[j4 + 2]) * __expf(fminf(gi - gj.z, 0.f));
                    a.w = (row > j + 3 ? bi : 0.f) * rj.w * __uint_as_float(r[j4 + 3]) * __expf(fminf(gi - gj.w, 0.f));
                    *reinterpret_cast<float4*>(As + row * PT_A_LD + j) = a;
                }
            }
        } else if (has_q) {
            // P = tril(qn kn^T e^{gcs_i - gcs_j}): one row per thread into the staging tile (the q sub-tile is free);
            // one TMA store writes the tile after the next barrier
            const int i = row - 64;
            const float gi = s_gcs[i], qi = s_qr[i];
            unsigned char* pst = smem + L::pst;
#pragma unroll 1
            for (int hh = 0; hh < 2; ++hh) {
                uint32_t r[32];
                tmem_ld32(t_lane + 32 * hh, r);
                tmem_ld_wait();
#pragma unroll
                for (int j8 = 0; j8 < 32; j8 += 8) {
                    const int j = 32 * hh + j8;
                    float pv[8];
#pragma unroll
                    for (int e4 = 0; e4 < 8; e4 += 4) {
                        const float4 gj = *reinterpret_cast<const float4*>(s_gcs + j + e4);
                        const float4 rj = *reinterpret_cast<const float4*>(s_rstd + j + e4);
                        pv[e4] = (i >= j + e4 ? qi : 0.f) * rj.x * __uint_as_float(r[j8 + e4]) * __expf(fminf(gi - gj.x, 0.f));
                        pv[e4 + 1] = (i >= j + e4 + 1 ? qi : 0.f) * rj.y * __uint_as_float(r[j8 + e4 + 1]) * __expf(fminf(gi - gj.y, 0.f));
                        pv[e4 + 2] = (i >= j + e4 + 2 ? qi : 0.f) * rj.z * __uint_as_float(r[j8 + e4 + 2]) * __expf(fminf(gi - gj.z, 0.f));
                        pv[e4 + 3] = (i >= j + e4 + 3 ? qi : 0.f) * rj.w * __uint_as_float(r[j8 + e4 + 3]) * __expf(fminf(gi - gj.w, 0.f));
                    }
                    *reinterpret_cast<uint4*>(pst + swz<128>(i, j >> 3)) =
                        make_uint4(pack_bf16(pv[0], pv[1]), pack_bf16(pv[2], pv[3]), pack_bf16(pv[4], pv[5]), pack_bf16(pv[6], pv[7]));
                }
            }
            fence_async_smem();
        }
        PT_STAMP(5);
        epi_barrier();                      // A complete, the w scale known, D1 read for the last time, P staged
        if (tid == 64 && has_q) {
            tma_store_4d(&map_p, sbase + L::pst, 0, h, t0, b);
            tma_store_commit();
        }
        if (lane < 16) {
            // X_dd = (I + A_dd)^-1 by forward substitution, lane = column; written over A_dd
            const int d0 = warp * 16, cidx = lane;
            float xcol[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float arow[16];
#pragma unroll
                for (int j4 = 0; j4 < 16; j4 += 4)
                    if (j4 < i)
                        *reinterpret_cast<float4*>(&arow[j4]) =
                            *reinterpret_cast<const float4*>(&As[(d0 + i) * PT_A_LD + d0 + j4]);
                float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
#pragma unroll
                for (int j = 0; j < i; ++j) {
                    const float t = arow[j] * xcol[j];
                    if ((j & 3) == 0) p0 += t; else if ((j & 3) == 1) p1 += t; else if ((j & 3) == 2) p2 += t; else p3 += t;
                }
                xcol[i] = ((i == cidx) ? 1.f : 0.f) - ((p0 + p1) + (p2 + p3));
            }
            __syncwarp(0x0000ffffu);
#pragma unroll
            for (int i = 0; i < 16; ++i) As[(d0 + i) * PT_A_LD + d0 + cidx] = xcol[i];
        }
        PT_STAMP(6);
        if (tid == 64 && has_q) tma_store_wait_read();      // the P tile has been read: its place becomes Ai diag(beta)
        epi_barrier();
        {
            float* scr = reinterpret_cast<float*>(smem + L::scr) + warp * 128;
            unsigned char* aiu = smem + L::aiu;
            unsigned char* aiw = smem + L::aiw;
            if (warp < 2) {
                inverse_panel(As, scr, aiu, aiw, s_beta, s_wsc, 0, warp, lane);
            } else {
#pragma unroll
                for (int j = 1; j < 4; ++j) inverse_panel(As, scr, aiu, aiw, s_beta, s_wsc, j, warp - 2, lane);
            }
        }
        PT_STAMP(7);
        fence_async_smem();
        tc_fence_before();
        mbar_arrive(bar_ai);
        PT_STAMP(8);
        // ---- w (columns 64-127, its product does not wait for the v tile) then u (columns 0-63): lane = feature,
        // column = token.  Each thread writes its feature's 64 values as single bf16 into a [token][feature] staging
        // tile (32 lanes = 64 contiguous bytes of one row: conflict-free), then one thread stores the tiles with TMA.
        // Staging: w over the k sub-tiles (dead once its product is done), u over the two Ai tiles.
        {
            const int sub = row >> 6, cf = row & 63;
            uint32_t off[8];                             // byte offset of this feature inside a row, by (token & 7)
#pragma unroll
            for (int x = 0; x < 8; ++x) off[x] = (uint32_t)((((cf >> 3) ^ x) << 4) + (cf & 7) * 2);
#pragma unroll 1
            for (int arr = 0; arr < 2; ++arr) {          // 0: w, 1: u
                mbar_wait(arr == 0 ? bar_d2w : bar_d2u, 0, status);
                tc_fence_after();
                unsigned char* stg = smem + L::kq + sub * 16384 + (arr == 0 ? 0 : 8192);
#pragma unroll 1
                for (int hh = 0; hh < 2; ++hh) {
                    uint32_t r[32];
                    tmem_ld32(t_lane + (arr == 0 ? 64 : 0) + 32 * hh, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int tt = 0; tt < 32; ++tt)
                        *reinterpret_cast<__nv_bfloat16*>(stg + (32 * hh + tt) * 128 + off[tt & 7]) =
                            __float2bfloat16(__uint_as_float(r[tt]));
                }
                fence_async_smem();
                epi_barrier();
                if (tid == 0) {
                    const CUtensorMap* mp = arr == 0 ? &map_w : &map_u;
                    tma_store_4d(mp, sbase + L::kq + (arr == 0 ? 0 : 8192), 0, h, t0, b);
                    tma_store_4d(mp, sbase + L::kq + 16384 + (arr == 0 ? 0 : 8192), 64, h, t0, b);
                    tma_store_commit();
                }
            }
            if (tid == 0) tma_store_wait_read();
        }
        PT_STAMP(9);
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 4) tmem_dealloc(tmem, PT_TMEM_COLS);
}

}  // namespace natsl

#ifdef NATSL_PREP_TIMING
extern "C" int natsl_prep_tc_set_timing(long long* p) {
    return cudaMemcpyToSymbol(natsl::g_prep_ts, &p, sizeof(p)) == cudaSuccess ? 0 : 1;
}
#endif

extern "C" int natsl_gdn_chunk_prep_tc(const void* q, const void* k, const void* v, const float* g, const void* beta,
                                       int beta_dtype, void* w, void* u, float* gcs, float* k_rstd, float* q_rstd,
                                       void* pmat, int B, int T, int H, int K, int V, int use_l2norm, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(k && v && g && beta && w && u && gcs && k_rstd, NATSL_ERR_NULL, "natsl_gdn_chunk_prep_tc: null pointer");
    NATSL_REQUIRE((q == nullptr) == (pmat == nullptr), NATSL_ERR_NULL,
                  "natsl_gdn_chunk_prep_tc: q and the score-matrix output go together");
    NATSL_REQUIRE(B > 0 && T > 0 && H > 0, NATSL_ERR_BAD_SHAPE, "natsl_gdn_chunk_prep_tc: empty shape");
    NATSL_REQUIRE(H <= 65535 && B <= 65535, NATSL_ERR_TOO_LARGE, "natsl_gdn_chunk_prep_tc: B and H must be <= 65535");
    NATSL_REQUIRE(beta_dtype == NATSL_DT_BF16 || beta_dtype == NATSL_DT_F32, NATSL_ERR_UNSUPPORTED,
                  "natsl_gdn_chunk_prep_tc: beta must be bf16 or f32");
    NATSL_REQUIRE(K == 128 && V == 128, NATSL_ERR_UNSUPPORTED,
                  "natsl_gdn_chunk_prep_tc: built for K = V = 128 (got K=%d V=%d); use natsl_gdn_chunk_prep_ex", K, V);
    auto kern = gdn_prep_tc_kernel;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PtSmem::total);
    if (e != cudaSuccess) {
        set_error("natsl_gdn_chunk_prep_tc: cannot reserve %d B of shared memory (%s)", PtSmem::total, cudaGetErrorString(e));
        return NATSL_ERR_CUDA;
    }
    CUtensorMap mq, mk, mv, mw, mu, mp;
    int rc = encode_bthd_map(&mk, k, B, T, H, K, 64, "natsl_gdn_chunk_prep_tc(k)");
    if (rc == NATSL_OK) rc = encode_bthd_map(&mv, v, B, T, H, V, 64, "natsl_gdn_chunk_prep_tc(v)");
    if (rc == NATSL_OK) rc = encode_bthd_map(&mq, q ? q : k, B, T, H, K, 64, "natsl_gdn_chunk_prep_tc(q)");
    if (rc == NATSL_OK) rc = encode_bthd_map(&mw, w, B, T, H, K, 64, "natsl_gdn_chunk_prep_tc(w)");
    if (rc == NATSL_OK) rc = encode_bthd_map(&mu, u, B, T, H, V, 64, "natsl_gdn_chunk_prep_tc(u)");
    if (rc == NATSL_OK) rc = pmat ? encode_bthd_map(&mp, pmat, B, T, H, 64, 64, "natsl_gdn_chunk_prep_tc(P)") : NATSL_OK;
    if (!pmat) mp = mk;
    int* status = nullptr;
    if (rc == NATSL_OK) rc = status_word_ptr(&status);
    if (rc != NATSL_OK) return rc;
    const int NT = (T + 63) / 64;
    dim3 grid(NT, H, B);
    kern<<<grid, PT_THREADS, PtSmem::total, reinterpret_cast<cudaStream_t>(stream)>>>(
        mq, mk, mv, mw, mu, mp, q ? 1 : 0, g, beta, beta_dtype, gcs, k_rstd, q_rstd, T, H, use_l2norm, status);
    return check_launch("natsl_gdn_chunk_prep_tc");
}
