// Backward of the chunk-masked softmax branch (src/nats/ops/attns/attns.py:1562-1759; preprocess :357-372,
// dq :383-708, dk/dv :719-982).  Key s is visible to query t when its block is softmax-selected and lies
// entirely before t, or when both are in the same block and s <= t (the forward's mask).  With
//     p = exp2(scale*log2(e) * q.k - lse),   delta = rowsum(o * do),   ds = p * (do.v - delta)
// the gradients are dq = scale * ds k, dk = scale * ds^T q, dv = p^T do.
//
// Two kernels, both on mma.sync with bf16 operands and fp32 accumulation, both deterministic (no atomics; every
// reduction has a fixed order):
//   attn_bwd_dq_kernel    one CTA per (64 queries, query head): walks the visible 64-key tiles, keeps dq in
//                         registers; also writes delta (the preprocess kernel of the reference folded in).
//   attn_bwd_dkdv_kernel  one CTA per (64 keys, key/value head): walks the query tiles that see these keys
//                         (rest of the own block, and every later block when the keys' block is selected) for
//                         every query head of the group, keeps dk and dv in registers, and sums ds over the
//                         later blocks' queries: the reference's `dnats` column for the softmax branch
//                         (attns.py:922, 975-978), written per (64-key tile, query head).
// `compat` reproduces the reference's default backward, which drops every own-block entry of ds and p
// (attns.py:590-591, 631-633, 842, 884 with the flag passed at mixed_attn_gdn.py:237) while lse and delta still
// come from the full forward.
#include "warp_gemm.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

constexpr int AB_THREADS = 128;
constexpr float kLog2e = 1.4426950408889634f;

template <int DK, int DV>
struct AttnBwdSmem {
    static constexpr int fixed_a = 0;                         // dq: Q tile     dkdv: K tile
    static constexpr int fixed_b = fixed_a + 64 * DK * 2;     // dq: dO tile    dkdv: V tile
    static constexpr int ring_a = fixed_b + 64 * DV * 2;      // 2 x [64][DK]   dq: K tiles   dkdv: Q tiles
    static constexpr int ring_b = ring_a + 2 * 64 * DK * 2;   // 2 x [64][DV]   dq: V tiles   dkdv: dO tiles
    static constexpr int vec = ring_b + 2 * 64 * DV * 2;      // lse, delta: 2 x 2 x 64 floats
    static constexpr int list = vec + 4 * 64 * 4;             // dq: visible key tiles (ints), NT entries
    static int total(int NT) { return list + NT * 4; }
};

// ------------------------------------------------------------------------------------------------- dq
template <int DK, int DV>
__global__ void __launch_bounds__(AB_THREADS)
attn_bwd_dq_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                   const __nv_bfloat16* __restrict__ v, const __nv_bfloat16* __restrict__ o,
                   const __nv_bfloat16* __restrict__ d_o, const float* __restrict__ lse, const int* __restrict__ types_i,
                   __nv_bfloat16* __restrict__ dq, float* __restrict__ delta_out, int T, int HQ, int HKV, int HN, int TN,
                   int nbs, float scale, int own_chunk, int compat) {
    using L = AttnBwdSmem<DK, DV>;
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, qd = lane & 3;
    const int NT = (T + 63) / 64;
    const int qt = NT - 1 - blockIdx.x;                      // heavy (late) query tiles first
    const int hq = blockIdx.y, b = blockIdx.z;
    const int hkv = hq / (HQ / HKV), hn = hq / (HQ / HN);
    const int cpb = nbs / 64;
    const int bq = qt / cpb;                                 // block of the queries
    const int valid_q = min(64, T - qt * 64);
    const long tokq = (long)b * T + (long)qt * 64;

    unsigned char* qs_p = smem + L::fixed_a;
    unsigned char* dos_p = smem + L::fixed_b;
    const uint32_t qs = smem_u32(qs_p), dos = smem_u32(dos_p);
    const uint32_t kring = smem_u32(smem + L::ring_a), vring = smem_u32(smem + L::ring_b);
    float* s_lse = reinterpret_cast<float*>(smem + L::vec);
    float* s_delta = s_lse + 64;
    int* s_list = reinterpret_cast<int*>(smem + L::list);
    __shared__ int s_count;

    // ---- Q, dO, and O (staged in the first V buffer) of the query tile
    load_tile_async<64, DK, AB_THREADS>(qs, q + (tokq * HQ + hq) * DK, (long)HQ * DK, valid_q, tid);
    load_tile_async<64, DV, AB_THREADS>(dos, d_o + (tokq * HQ + hq) * DV, (long)HQ * DV, valid_q, tid);
    load_tile_async<64, DV, AB_THREADS>(vring, o + (tokq * HQ + hq) * DV, (long)HQ * DV, valid_q, tid);
    cp_async_commit();
    if (tid < 64) s_lse[tid] = tid < valid_q ? lse[(tokq + tid) * HQ + hq] : 0.f;

    // ---- visible key tiles: sub-tiles of the selected blocks before the query's block, then the own block's
    // sub-tiles up to the query tile (warp 0 compacts with ballots)
    if (warp == 0) {
        const int* sel_p = types_i + ((long)b * TN * HN + hn) * 2;           // column 0, stride HN * 2 per block
        int count = 0;
        const int n_cand = qt + 1;
        for (int base = 0; base < n_cand; base += 32) {
            const int kt = base + lane;
            bool vis = false;
            if (kt < n_cand) {
                const int c = kt / cpb;
                vis = (c == bq) ? (own_chunk && !compat) : (sel_p[(long)c * HN * 2] != 0);
            }
            const unsigned m = __ballot_sync(0xffffffffu, vis);
            if (vis) s_list[count + __popc(m & ((1u << lane) - 1))] = kt;
            count += __popc(m);
        }
        if (lane == 0) s_count = count;
    }
    cp_async_wait<0>();
    __syncthreads();
    const int n_tiles = s_count;

    // ---- delta = rowsum(o * do)
    {
        const unsigned char* os_p = smem + L::ring_b;
        constexpr int CPR = DV / 8;
        for (int r = warp * 16; r < warp * 16 + 16; ++r) {
            float s = 0.f;
            for (int cc = lane; cc < CPR; cc += 32) {
                const uint4 a = *reinterpret_cast<const uint4*>(os_p + swz<DV * 2>(r, cc));
                const uint4 d = *reinterpret_cast<const uint4*>(dos_p + swz<DV * 2>(r, cc));
                const uint32_t* aw = reinterpret_cast<const uint32_t*>(&a);
                const uint32_t* dw = reinterpret_cast<const uint32_t*>(&d);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 x = unpack_bf16(aw[j]), y = unpack_bf16(dw[j]);
                    s += x.x * y.x + x.y * y.y;
                }
            }
            s = warp_sum(s);
            if (lane == 0) {
                s_delta[r] = s;
                if (r < valid_q) delta_out[(tokq + r) * HQ + hq] = s;
            }
        }
    }
    __syncthreads();                                          // the O staging buffer is free again

    auto issue = [&](int i) {
        if (i < n_tiles) {
            const int kt = s_list[i];
            const int valid_k = min(64, T - kt * 64);
            const long tokk = (long)b * T + (long)kt * 64;
            load_tile_async<64, DK, AB_THREADS>(kring + (i & 1) * 64 * DK * 2, k + (tokk * HKV + hkv) * DK, (long)HKV * DK,
                                                valid_k, tid);
            load_tile_async<64, DV, AB_THREADS>(vring + (i & 1) * 64 * DV * 2, v + (tokk * HKV + hkv) * DV, (long)HKV * DV,
                                                valid_k, tid);
        }
        cp_async_commit();
    };

    float acc_dq[DK / 8][4];
    zero_acc(acc_dq);
    const int r0 = warp * 16;
    const int ia = r0 + gq, ib = ia + 8;
    const float lse_a = s_lse[ia], lse_b = s_lse[ib], del_a = s_delta[ia], del_b = s_delta[ib];
    const float sl2 = scale * kLog2e;

    issue(0);
    for (int i = 0; i < n_tiles; ++i) {
        issue(i + 1);
        cp_async_wait<1>();
        __syncthreads();
        const int kt = s_list[i];
        const uint32_t ks = kring + (i & 1) * 64 * DK * 2, vs = vring + (i & 1) * 64 * DV * 2;
        float acc_s[8][4], acc_p[8][4];
        zero_acc(acc_s);
        zero_acc(acc_p);
        warp_gemm<DK * 2, A_ROW, DK * 2, B_NK, 8>(acc_s, qs, r0, ks, 0, 0, DK, lane);
        warp_gemm<DV * 2, A_ROW, DV * 2, B_NK, 8>(acc_p, dos, r0, vs, 0, 0, DV, lane);
        const bool diag = kt == qt;
        const int kmax = T - kt * 64;                         // keys j >= kmax do not exist
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i_row = (e >> 1) ? ib : ia;
                const int j = nt * 8 + qd * 2 + (e & 1);
                const bool ok = j < kmax && (!diag || j <= i_row);
                const float p = exp2f(acc_s[nt][e] * sl2 - ((e >> 1) ? lse_b : lse_a));
                acc_s[nt][e] = ok ? p * (acc_p[nt][e] - ((e >> 1) ? del_b : del_a)) : 0.f;
            }
        uint32_t dsf[4][4];
        acc_to_afrag<8>(acc_s, dsf);
        warp_gemm_ra<4, DK * 2, B_KN, DK / 8>(acc_dq, dsf, ks, 0, 0, lane);
        __syncthreads();                                      // every warp is done with this stage before it is refilled
    }
    cp_async_wait<0>();

    // ---- dq = scale * acc, staged through the Q tile
#pragma unroll
    for (int nt = 0; nt < DK / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc_dq[nt][e] *= scale;
    store_acc_bf16<DK * 2, DK / 8>(qs_p, acc_dq, r0, 0, lane);
    __syncthreads();
    store_tile<64, DK, AB_THREADS>(qs_p, dq + (tokq * HQ + hq) * DK, (long)HQ * DK, valid_q, tid);
}

// ------------------------------------------------------------------------------------------------- dk, dv
template <int DK, int DV>
__global__ void __launch_bounds__(AB_THREADS)
attn_bwd_dkdv_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                     const __nv_bfloat16* __restrict__ v, const __nv_bfloat16* __restrict__ d_o,
                     const float* __restrict__ lse, const float* __restrict__ delta, const int* __restrict__ types_i,
                     __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv, float* __restrict__ dnats_part, int T,
                     int HQ, int HKV, int HN, int TN, int nbs, float scale, int own_chunk, int compat) {
    using L = AttnBwdSmem<DK, DV>;
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, qd = lane & 3;
    const int NT = (T + 63) / 64;
    const int kt = blockIdx.x;                               // early key tiles are seen by the most queries: first
    const int hkv = blockIdx.y, b = blockIdx.z;
    const int G = HQ / HKV;
    const int cpb = nbs / 64;
    const int c = kt / cpb;                                  // block of the keys
    const int valid_k = min(64, T - kt * 64);
    const long tokk = (long)b * T + (long)kt * 64;
    const int own_end = min((c + 1) * cpb, NT);              // query tiles [kt, own_end) share the keys' block
    const int n_own = (own_chunk && !compat) ? own_end - kt : 0;

    unsigned char* ks_p = smem + L::fixed_a;
    unsigned char* vs_p = smem + L::fixed_b;
    const uint32_t ks = smem_u32(ks_p), vs = smem_u32(vs_p);
    const uint32_t qring = smem_u32(smem + L::ring_a), doring = smem_u32(smem + L::ring_b);
    float* s_vec = reinterpret_cast<float*>(smem + L::vec);  // [stage][lse 64 | delta 64]
    __shared__ float s_dn[16][4];                            // per query head of the group and warp: fixed summation order
    __shared__ int s_npast[16];

    load_tile_async<64, DK, AB_THREADS>(ks, k + (tokk * HKV + hkv) * DK, (long)HKV * DK, valid_k, tid);
    load_tile_async<64, DV, AB_THREADS>(vs, v + (tokk * HKV + hkv) * DV, (long)HKV * DV, valid_k, tid);
    cp_async_commit();
    if (tid < 16) {
#pragma unroll
        for (int wv = 0; wv < 4; ++wv) s_dn[tid][wv] = 0.f;
        int np = 0;
        if (tid < G) {
            const int hq = hkv * G + tid;
            const int hn = hq / (HQ / HN);
            const bool sel = types_i[(((long)b * TN + c) * HN + hn) * 2] != 0;
            np = sel ? max(0, NT - own_end) : 0;
        }
        s_npast[tid] = np;
    }
    __syncthreads();
    int total = 0;
    for (int gi = 0; gi < G; ++gi) total += n_own + s_npast[gi];

    // flat iteration index -> (query head of the group, query tile, own-block flag)
    auto decode = [&](int idx, int& gi, int& qt, bool& own) {
        gi = 0;
        while (true) {
            const int n = n_own + s_npast[gi];
            if (idx < n) break;
            idx -= n;
            ++gi;
        }
        own = idx < n_own;
        qt = own ? kt + idx : own_end + (idx - n_own);
    };
    auto issue = [&](int i) {
        if (i < total) {
            int gi, qt;
            bool own;
            decode(i, gi, qt, own);
            const int hq = hkv * G + gi;
            const int valid_q = min(64, T - qt * 64);
            const long tokq = (long)b * T + (long)qt * 64;
            load_tile_async<64, DK, AB_THREADS>(qring + (i & 1) * 64 * DK * 2, q + (tokq * HQ + hq) * DK, (long)HQ * DK,
                                                valid_q, tid);
            load_tile_async<64, DV, AB_THREADS>(doring + (i & 1) * 64 * DV * 2, d_o + (tokq * HQ + hq) * DV, (long)HQ * DV,
                                                valid_q, tid);
            if (tid < 64) {
                const bool okr = tid < valid_q;
                const long gi_ = (tokq + (okr ? tid : 0)) * HQ + hq;
                float* dst = s_vec + (i & 1) * 128;
                dst[tid] = okr ? lse[gi_] : 0.f;
                dst[64 + tid] = okr ? delta[gi_] : 0.f;
            }
        }
        cp_async_commit();
    };

    float acc_dk[DK / 8][4], acc_dv[DV / 8][4];
    zero_acc(acc_dk);
    zero_acc(acc_dv);
    const int r0 = warp * 16;
    const int ja = r0 + gq, jb = ja + 8;                      // key rows of this lane
    const float sl2 = scale * kLog2e;
    float dn_acc = 0.f;
    int dn_gi = 0;

    issue(0);
    for (int i = 0; i < total; ++i) {
        issue(i + 1);
        cp_async_wait<1>();
        __syncthreads();
        int gi, qt;
        bool own;
        decode(i, gi, qt, own);
        if (gi != dn_gi) {                                    // uniform over the CTA
            dn_acc = warp_sum(dn_acc);
            if (lane == 0) s_dn[dn_gi][warp] += dn_acc;
            dn_acc = 0.f;
            dn_gi = gi;
        }
        const uint32_t qs = qring + (i & 1) * 64 * DK * 2, dos = doring + (i & 1) * 64 * DV * 2;
        const float* v_lse = s_vec + (i & 1) * 128;
        const float* v_del = v_lse + 64;
        // transposed score tile: rows = keys, columns = queries
        float acc_s[8][4], acc_p[8][4];
        zero_acc(acc_s);
        zero_acc(acc_p);
        warp_gemm<DK * 2, A_ROW, DK * 2, B_NK, 8>(acc_s, ks, r0, qs, 0, 0, DK, lane);
        warp_gemm<DV * 2, A_ROW, DV * 2, B_NK, 8>(acc_p, vs, r0, dos, 0, 0, DV, lane);
        const bool diag = qt == kt;
        const int qmax = T - qt * 64;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = (e >> 1) ? jb : ja;             // key
                const int iq = nt * 8 + qd * 2 + (e & 1);     // query
                const bool ok = iq < qmax && j < valid_k && (!diag || j <= iq);
                const float p = ok ? exp2f(acc_s[nt][e] * sl2 - v_lse[iq]) : 0.f;
                const float ds = p * (acc_p[nt][e] - v_del[iq]);
                acc_s[nt][e] = p;
                acc_p[nt][e] = ds;
                if (!own) dn_acc += ds;
            }
        uint32_t pf[4][4], dsf[4][4];
        acc_to_afrag<8>(acc_s, pf);
        acc_to_afrag<8>(acc_p, dsf);
        warp_gemm_ra<4, DV * 2, B_KN, DV / 8>(acc_dv, pf, dos, 0, 0, lane);
        warp_gemm_ra<4, DK * 2, B_KN, DK / 8>(acc_dk, dsf, qs, 0, 0, lane);
        __syncthreads();
    }
    cp_async_wait<0>();
    dn_acc = warp_sum(dn_acc);
    if (lane == 0 && total > 0) s_dn[dn_gi][warp] += dn_acc;

    // ---- stores: dk = scale * acc, dv; staged through the (idle) ring buffers
    unsigned char* st_k = smem + L::ring_a;
    unsigned char* st_v = smem + L::ring_b;
#pragma unroll
    for (int nt = 0; nt < DK / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc_dk[nt][e] *= scale;
    store_acc_bf16<DK * 2, DK / 8>(st_k, acc_dk, r0, 0, lane);
    store_acc_bf16<DV * 2, DV / 8>(st_v, acc_dv, r0, 0, lane);
    __syncthreads();
    store_tile<64, DK, AB_THREADS>(st_k, dk + (tokk * HKV + hkv) * DK, (long)HKV * DK, valid_k, tid);
    store_tile<64, DV, AB_THREADS>(st_v, dv + (tokk * HKV + hkv) * DV, (long)HKV * DV, valid_k, tid);
    if (tid < G) dnats_part[((long)b * NT + kt) * HQ + hkv * G + tid] = (s_dn[tid][0] + s_dn[tid][1]) + (s_dn[tid][2] + s_dn[tid][3]);
}

template <int DK, int DV>
static int launch_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                           const int* types_i, void* dq, void* dk, void* dv, float* delta, float* dnats_part, int B, int T,
                           int HQ, int HKV, int HN, int nbs, float scale, int own_chunk, int compat, cudaStream_t st) {
    using L = AttnBwdSmem<DK, DV>;
    const int NT = (T + 63) / 64;
    const int TN = (T + nbs - 1) / nbs;
    const int smem = L::total(NT);
    if (smem > 227 * 1024) {
        set_error("natsl_attn_bwd: T=%d needs %d B of shared memory (max %d)", T, smem, 227 * 1024);
        return NATSL_ERR_TOO_LARGE;
    }
    auto k1 = attn_bwd_dq_kernel<DK, DV>;
    auto k2 = attn_bwd_dkdv_kernel<DK, DV>;
    cudaError_t e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
        set_error("natsl_attn_bwd: cannot reserve %d B of shared memory (%s)", smem, cudaGetErrorString(e));
        return NATSL_ERR_CUDA;
    }
    auto bf = [](const void* p) { return reinterpret_cast<const __nv_bfloat16*>(p); };
    k1<<<dim3(NT, HQ, B), AB_THREADS, smem, st>>>(bf(q), bf(k), bf(v), bf(o), bf(d_o), lse, types_i,
                                                 reinterpret_cast<__nv_bfloat16*>(dq), delta, T, HQ, HKV, HN, TN, nbs, scale,
                                                 own_chunk, compat);
    int rc = check_launch("natsl_attn_bwd (dq)");
    if (rc != NATSL_OK) return rc;
    k2<<<dim3(NT, HKV, B), AB_THREADS, smem, st>>>(bf(q), bf(k), bf(v), bf(d_o), lse, delta, types_i,
                                                  reinterpret_cast<__nv_bfloat16*>(dk), reinterpret_cast<__nv_bfloat16*>(dv),
                                                  dnats_part, T, HQ, HKV, HN, TN, nbs, scale, own_chunk, compat);
    return check_launch("natsl_attn_bwd (dk, dv)");
}

}  // namespace natsl

extern "C" int natsl_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                              const int32_t* types_i, void* dq, void* dk, void* dv, float* delta, float* dnats_part, int B,
                              int T, int HQ, int HKV, int HN, int DK, int DV, int nbs, float scale, int flags,
                              void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(q && k && v && o && d_o && lse && types_i && dq && dk && dv && delta && dnats_part, NATSL_ERR_NULL,
                  "natsl_attn_bwd: null pointer");
    NATSL_REQUIRE(B > 0 && T > 0 && HQ > 0 && HKV > 0 && HN > 0 && HQ % HKV == 0 && HQ % HN == 0, NATSL_ERR_BAD_SHAPE,
                  "natsl_attn_bwd: bad shape B=%d T=%d HQ=%d HKV=%d HN=%d", B, T, HQ, HKV, HN);
    NATSL_REQUIRE(HQ / HKV <= 16, NATSL_ERR_UNSUPPORTED, "natsl_attn_bwd: at most 16 query heads per key/value head");
    NATSL_REQUIRE(nbs >= 64 && nbs % 64 == 0, NATSL_ERR_UNSUPPORTED,
                  "natsl_attn_bwd: nats_block_size must be a multiple of 64 (got %d)", nbs);
    NATSL_REQUIRE(HQ <= 65535 && B <= 65535, NATSL_ERR_TOO_LARGE, "natsl_attn_bwd: B and HQ must be <= 65535");
    const int own = (flags & NATSL_FLAG_ATTN_OWN_CHUNK) ? 1 : 0;
    const int compat = (flags & NATSL_FLAG_BWD_REFERENCE_COMPAT) ? 1 : 0;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define NATSL_AB_CASE(KK, VV) \
    if (DK == KK && DV == VV) \
        return launch_attn_bwd<KK, VV>(q, k, v, o, d_o, lse, types_i, dq, dk, dv, delta, dnats_part, B, T, HQ, HKV, HN, nbs, \
                                       scale, own, compat, st);
    NATSL_AB_CASE(64, 64)
    NATSL_AB_CASE(64, 128)
    NATSL_AB_CASE(128, 64)
    NATSL_AB_CASE(128, 128)
#undef NATSL_AB_CASE
    set_error("natsl_attn_bwd: unsupported head dims DK=%d DV=%d (64 or 128 each)", DK, DV);
    return NATSL_ERR_UNSUPPORTED;
}
