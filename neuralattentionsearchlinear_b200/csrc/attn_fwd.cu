// Chunk-masked softmax attention forward (the softmax branch of the hybrid layer).
// Key s is visible to query t when the key's block is softmax-selected and ends at or before t's
// block start..., precisely:   sel[blk(s)] && t >= (blk(s)+1)*nbs   ||   blk(s)==blk(t) && s <= t
// (mask of the reference's own check, src/nats/ops/attns/attns.py:2041-2058; kernel stages
// src/nats/ops/attns/attns.py:173-217 for selected past blocks and :271-340 for the own span).
// One CTA per (128-query tile, softmax head, batch).  The key tiles it visits are
//   1. the first n_past selected blocks (index table, unmasked; n_past is the
//      `attn_n_iters` table = compute_attn_n_iters_per_block, src/nats/ops/nats_util.py:67-121),
//   2. the own span [block start of the tile's first row, end of the tile), masked per element.
// Flash-attention style online softmax in base 2 (attns.py:158-159, 205-212): Q K^T and P V on the
// tensor cores (bf16 operands, fp32 accumulate), K/V tiles double-buffered with cp.async.
// Rows that see no key give o = 0, lse = 0 (attns.py:343-350).
// The same tile walk and visibility predicate also drive a debug kernel that writes the dense
// 0/1 mask, which is what the bit-exact mask check compares.
#include "common.cuh"
#include "attn_walk.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

constexpr int ATT_THREADS = 256;

template <int DK, int DV>
struct AttSmem {
    static constexpr int qs = 0;
    static constexpr int ks = qs + ATT_BM * DK * 2;
    static constexpr int vs = ks + 2 * ATT_BN * DK * 2;
    static constexpr int total = vs + 2 * ATT_BN * DV * 2;
};

template <int DK, int DV>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                const __nv_bfloat16* __restrict__ v, const int* __restrict__ types_i, const int* __restrict__ indices,
                const int* __restrict__ attn_n_iters, __nv_bfloat16* __restrict__ o, float* __restrict__ lse, int T,
                int HQ, int HKV, int HN, int TN, int nbs, float scale_log2, int own_chunk) {
    using L = AttSmem<DK, DV>;
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, qd = lane & 3;
    const int NTq = gridDim.x;
    const int it = NTq - 1 - blockIdx.x;          // heaviest tiles first
    const int hq = blockIdx.y, b = blockIdx.z;
    const int hkv = hq / (HQ / HKV), hn = hq / (HQ / HN);
    const int q0 = it * ATT_BM;
    const int* idx = indices + ((long)b * TN * HN + hn) * 2;          // attention column
    const int* selp = types_i + ((long)b * TN * HN + hn) * 2;
    const long tstride = (long)HN * 2;
    const TileWalk walk = make_walk(q0, T, nbs, attn_n_iters[((long)b * NTq + it) * HN + hn]);

    const uint32_t qs = smem_u32(smem + L::qs), ks = smem_u32(smem + L::ks), vs = smem_u32(smem + L::vs);
    const __nv_bfloat16* kbase = k + ((long)b * T * HKV + hkv) * DK;
    const __nv_bfloat16* vbase = v + ((long)b * T * HKV + hkv) * DV;

    auto load_kv = [&](int j, int stg) {
        bool m;
        int s = tile_start(walk, j, idx, tstride, nbs, m);
        int valid = min(ATT_BN, T - s);
        load_tile_async<ATT_BN, DK, ATT_THREADS>(ks + stg * ATT_BN * DK * 2, kbase + (long)s * HKV * DK, (long)HKV * DK,
                                                 valid, tid);
        load_tile_async<ATT_BN, DV, ATT_THREADS>(vs + stg * ATT_BN * DV * 2, vbase + (long)s * HKV * DV, (long)HKV * DV,
                                                 valid, tid);
    };

    load_tile_async<ATT_BM, DK, ATT_THREADS>(qs, q + (((long)b * T + q0) * HQ + hq) * DK, (long)HQ * DK,
                                             min(ATT_BM, T - q0), tid);
    load_kv(0, 0);
    cp_async_commit();

    const int r0 = warp * 16;
    const int ta = q0 + r0 + gq, tb = ta + 8;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    float oacc[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) oacc[i][j] = 0.f;

    for (int j = 0; j < walk.n_tiles; ++j) {
        const int stg = j & 1;
        if (j + 1 < walk.n_tiles) {
            load_kv(j + 1, stg ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        bool masked;
        const int s0 = tile_start(walk, j, idx, tstride, nbs, masked);
        bool skip = false;
        bool selb = true;
        int blk_end = 0;
        if (masked) {
            const int blk = s0 / nbs;
            selb = selp[(long)blk * tstride] != 0;
            blk_end = (blk + 1) * nbs;
            if (own_chunk) skip = s0 > q0 + r0 + 15;               // keys entirely after this warp's rows
            else skip = !selb || (q0 + r0 + 15 < blk_end);
        }
        if (!skip) {
            const uint32_t kt = ks + stg * ATT_BN * DK * 2, vt = vs + stg * ATT_BN * DV * 2;
            float sacc[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) sacc[i][e] = 0.f;
#pragma unroll
            for (int kk = 0; kk < DK / 16; ++kk) {
                uint32_t a[4];
                load_a<DK * 2>(qs, r0, kk * 16, lane, a);
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                    uint32_t bb[4];
                    load_b_nk<DK * 2>(kt, p * 16, kk * 16, lane, bb);
                    mma_bf16(sacc[2 * p], a, bb[0], bb[1]);
                    mma_bf16(sacc[2 * p + 1], a, bb[2], bb[3]);
                }
            }
            float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float sv = sacc[nt][e] * scale_log2;
                    if (masked) {
                        int t = (e >> 1) ? tb : ta;
                        int s = s0 + nt * 8 + qd * 2 + (e & 1);
                        if (!visible(t, s, T, blk_end, selb, own_chunk != 0)) sv = -INFINITY;
                    }
                    sacc[nt][e] = sv;
                    if (e >> 1) mx_b = fmaxf(mx_b, sv); else mx_a = fmaxf(mx_a, sv);
                }
            }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
            const float mu_a = (mn_a == -INFINITY) ? 0.f : mn_a, mu_b = (mn_b == -INFINITY) ? 0.f : mn_b;
            const float al_a = exp2f(m_a - mu_a), al_b = exp2f(m_b - mu_b);
            m_a = mn_a; m_b = mn_b;
            float rs_a = 0.f, rs_b = 0.f;
            uint32_t pa[4][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                float p0 = exp2f(sacc[nt][0] - mu_a), p1 = exp2f(sacc[nt][1] - mu_a);
                float p2 = exp2f(sacc[nt][2] - mu_b), p3 = exp2f(sacc[nt][3] - mu_b);
                rs_a += p0 + p1;
                rs_b += p2 + p3;
                pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(p0, p1);
                pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
            }
            l_a = l_a * al_a + rs_a;
            l_b = l_b * al_b + rs_b;
#pragma unroll
            for (int i = 0; i < DV / 8; ++i) {
                oacc[i][0] *= al_a; oacc[i][1] *= al_a;
                oacc[i][2] *= al_b; oacc[i][3] *= al_b;
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                for (int p = 0; p < DV / 16; ++p) {
                    uint32_t bb[4];
                    load_b_kn<DV * 2>(vt, kk * 16, p * 16, lane, bb);
                    mma_bf16(oacc[2 * p], pa[kk], bb[0], bb[1]);
                    mma_bf16(oacc[2 * p + 1], pa[kk], bb[2], bb[3]);
                }
            }
        }
        __syncthreads();
    }

    // ---- epilogue: normalise, stage this warp's 16 rows over the value buffers, store
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    const bool ok_a = m_a != -INFINITY && l_a > 0.f, ok_b = m_b != -INFINITY && l_b > 0.f;
    const float inv_a = ok_a ? 1.f / l_a : 0.f, inv_b = ok_b ? 1.f / l_b : 0.f;
    unsigned char* stage = smem + L::vs;
#pragma unroll
    for (int nt = 0; nt < DV / 8; ++nt) {
        *reinterpret_cast<uint32_t*>(stage + swz<DV * 2>(r0 + gq, nt) + qd * 4) =
            pack_bf16(oacc[nt][0] * inv_a, oacc[nt][1] * inv_a);
        *reinterpret_cast<uint32_t*>(stage + swz<DV * 2>(r0 + gq + 8, nt) + qd * 4) =
            pack_bf16(oacc[nt][2] * inv_b, oacc[nt][3] * inv_b);
    }
    if (qd == 0) {
        if (ta < T) lse[((long)b * T + ta) * HQ + hq] = ok_a ? m_a + log2f(l_a) : 0.f;
        if (tb < T) lse[((long)b * T + tb) * HQ + hq] = ok_b ? m_b + log2f(l_b) : 0.f;
    }
    __syncwarp();
    constexpr int CPR = DV / 8;
    __nv_bfloat16* obase = o + (((long)b * T + q0) * HQ + hq) * DV;
    for (int i = lane; i < 16 * CPR; i += 32) {
        int r = r0 + i / CPR, cch = i % CPR;
        if (q0 + r < T) {
            uint4 x = *reinterpret_cast<const uint4*>(stage + swz<DV * 2>(r, cch));
            *reinterpret_cast<uint4*>(obase + (long)r * HQ * DV + cch * 8) = x;
        }
    }
}

// Dense 0/1 mask [B, HQ, T, T] produced by the same tile walk and predicate (debug / parity).
__global__ void __launch_bounds__(ATT_THREADS)
attn_mask_kernel(const int* __restrict__ types_i, const int* __restrict__ indices, const int* __restrict__ attn_n_iters,
                 unsigned char* __restrict__ mask, int T, int HQ, int HN, int TN, int nbs, int own_chunk) {
    const int NTq = gridDim.x;
    const int it = blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
    const int hn = hq / (HQ / HN);
    const int q0 = it * ATT_BM;
    const int* idx = indices + ((long)b * TN * HN + hn) * 2;
    const int* selp = types_i + ((long)b * TN * HN + hn) * 2;
    const long tstride = (long)HN * 2;
    const TileWalk walk = make_walk(q0, T, nbs, attn_n_iters[((long)b * NTq + it) * HN + hn]);
    unsigned char* mb = mask + ((long)b * HQ + hq) * T * T;
    for (int j = 0; j < walk.n_tiles; ++j) {
        bool masked;
        const int s0 = tile_start(walk, j, idx, tstride, nbs, masked);
        bool selb = true;
        int blk_end = 0;
        if (masked) {
            const int blk = s0 / nbs;
            selb = selp[(long)blk * tstride] != 0;
            blk_end = (blk + 1) * nbs;
        }
        for (int e = threadIdx.x; e < ATT_BM * ATT_BN; e += ATT_THREADS) {
            int t = q0 + e / ATT_BN, s = s0 + e % ATT_BN;
            if (t >= T || s >= T) continue;
            bool vis = masked ? visible(t, s, T, blk_end, selb, own_chunk != 0) : true;
            if (vis) mb[(long)t * T + s] = 1;
        }
    }
}

template <int DK, int DV>
static int launch_attn(const void* q, const void* k, const void* v, const int* types_i, const int* indices,
                       const int* n_iters, void* o, float* lse, int B, int T, int HQ, int HKV, int HN, int nbs,
                       float scale, int own_chunk, cudaStream_t st) {
    using L = AttSmem<DK, DV>;
    auto kern = attn_fwd_kernel<DK, DV>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::total);
    if (e != cudaSuccess) {
        set_error("natsl_attn_fwd: cannot reserve %d B of shared memory (%s)", L::total, cudaGetErrorString(e));
        return NATSL_ERR_CUDA;
    }
    const int NTq = (T + ATT_BM - 1) / ATT_BM, TN = (T + nbs - 1) / nbs;
    dim3 grid(NTq, HQ, B);
    kern<<<grid, ATT_THREADS, L::total, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(q), reinterpret_cast<const __nv_bfloat16*>(k),
        reinterpret_cast<const __nv_bfloat16*>(v), types_i, indices, n_iters, reinterpret_cast<__nv_bfloat16*>(o), lse,
        T, HQ, HKV, HN, TN, nbs, scale * 1.44269504f, own_chunk);
    return check_launch("natsl_attn_fwd");
}

}  // namespace natsl

namespace natsl {
// mma.sync implementation (kept as the comparison / debug path; selected with NATSL_FLAG_ATTN_MMA_SYNC)
int attn_fwd_mma_sync(const void* q, const void* k, const void* v, const int32_t* types_i, const int32_t* indices,
                      const int32_t* attn_n_iters, void* o, float* lse, int B, int T, int HQ, int HKV, int HN, int DK,
                      int DV, int nbs, float scale, int own, cudaStream_t st) {
#define NATSL_ATT_ARGS q, k, v, types_i, indices, attn_n_iters, o, lse, B, T, HQ, HKV, HN, nbs, scale, own, st
    if (DK == 64 && DV == 64) return launch_attn<64, 64>(NATSL_ATT_ARGS);
    if (DK == 64 && DV == 128) return launch_attn<64, 128>(NATSL_ATT_ARGS);
    if (DK == 128 && DV == 64) return launch_attn<128, 64>(NATSL_ATT_ARGS);
    if (DK == 128 && DV == 128) return launch_attn<128, 128>(NATSL_ATT_ARGS);
#undef NATSL_ATT_ARGS
    set_error("natsl_attn_fwd: unsupported head dims DK=%d DV=%d (each 64 or 128)", DK, DV);
    return NATSL_ERR_UNSUPPORTED;
}
}  // namespace natsl

extern "C" int natsl_attn_dense_mask(const int32_t* types_i, const int32_t* indices, const int32_t* attn_n_iters,
                                     uint8_t* mask, int B, int T, int HQ, int HN, int nbs, int flags, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(types_i && indices && attn_n_iters && mask, NATSL_ERR_NULL, "natsl_attn_dense_mask: null pointer");
    NATSL_REQUIRE(B > 0 && T > 0 && HQ > 0 && HN > 0 && HQ % HN == 0, NATSL_ERR_BAD_SHAPE,
                  "natsl_attn_dense_mask: bad shape");
    NATSL_REQUIRE((long)B * HQ * T * T <= (1L << 32), NATSL_ERR_TOO_LARGE,
                  "natsl_attn_dense_mask: dense mask of %ld bytes refused (debug entry, <= 4 GiB)", (long)B * HQ * T * T);
    NATSL_REQUIRE(nbs >= 64 && nbs % 64 == 0, NATSL_ERR_UNSUPPORTED, "natsl_attn_dense_mask: bad nats_block_size");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemsetAsync(mask, 0, (size_t)B * HQ * T * T, st);
    if (e != cudaSuccess) {
        set_error("natsl_attn_dense_mask: memset failed (%s)", cudaGetErrorString(e));
        return NATSL_ERR_CUDA;
    }
    const int NTq = (T + ATT_BM - 1) / ATT_BM, TN = (T + nbs - 1) / nbs;
    dim3 grid(NTq, HQ, B);
    attn_mask_kernel<<<grid, ATT_THREADS, 0, st>>>(types_i, indices, attn_n_iters, mask, T, HQ, HN, TN, nbs,
                                                   (flags & NATSL_FLAG_ATTN_OWN_CHUNK) ? 1 : 0);
    return check_launch("natsl_attn_dense_mask");
}
