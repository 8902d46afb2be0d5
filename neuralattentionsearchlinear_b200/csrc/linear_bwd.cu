// Backward of the linear branch (Gated DeltaNet and Mamba2/SSD) in the 64-token chunk form, block size 64
// (src/nats/ops/gated_delta_rule/chunk.py:170-332, src/nats/ops/mamba/chunk.py:112-240).
//
// Per chunk c of one (batch, head): g = chunk-local cumsum, Gam_ij = e^{g_i - g_j}, S = the state the chunk reads,
// car = decay of the skipped chunks before it, act = "this chunk updates the state".  The forward is
//     v' = u - e^{car} w S,   o = s [ (e^{g+car} qn) S + P v' ],   P = tril(qn kn^T Gam),
//     act:  S+ = e^{g_L+car} S + kn^T (v' kd),   kd = e^{g_L - g}   (Mamba2: u = v, w = 0, kd = e^{min(g_L - g, 0)}).
// Five kernels, in this order, after the forward's own preparation (w, u, gcs) and recurrence (S, car per chunk):
//   linear_bwd_pre_kernel    per chunk: qn, kn (l2 norm, bf16, with the 1/norm factors), dv'_loc = s P^T do
//                            (fla chunk_bwd_dv_local, call src/nats/ops/common/chunk_o.py:1339).
//   linear_bwd_dh_kernel     the serial part: one CTA per (batch, head, value-column slice) walks the chunks in
//                            reverse with dS in registers (src/nats/ops/common/chunk_delta_h.py:346-635):
//                                dv' = act (kn dS) kd + dv'_loc;   dS <- (act ? e^{g_L+car} : 1) dS + s (e^{g+car} qn)^T do
//                                - e^{car} w^T dv'.   Stores dS after every updating chunk and dv' of every chunk.
//   linear_bwd_state_kernel  per chunk, everything that contracts with S or dS: v', kd-weighted k dS (the decay
//                            gradients and `dnats`, chunk_o.py:440-443, 459-492), dkn += (v' kd) dS^T,
//                            dqn += s e^{g+car} do S^T, dw = -e^{car} dv' S^T (chunk_o.py:393-571).
//   linear_bwd_intra_kernel  per chunk, the 64x64 part: dP = s tril(do v'^T), through P to qn, kn and the decays;
//                            through the WY transform by two triangular solves with (I + A)^T
//                            (src/nats/ops/gated_delta_rule/wy_fast.py:169-334):
//                                [dzu | dzw] = (I + A)^-T [dv' | dw],  dA = -strictLower(dzu u^T + dzw w^T);
//                            then the l2-norm backward (mixed_attn_gdn.py:273-275).
//   linear_bwd_dg_kernel     per (batch, head): the scalar chain of the carried decay over skipped chunks and the
//                            reverse chunk-local cumsum (chunk.py:318-331, src/nats/ops/utils/cumsum.py REVERSED).
// All products run on mma.sync with bf16 operands and fp32 accumulation.  No atomics on global memory; shared-memory
// sums either have one writer per slot or exactly two terms, so results are reproducible bit for bit.
#include "warp_gemm.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

constexpr int LB_THREADS = 256;
constexpr int LB_A_LD = 68;
constexpr int LB_X_LD = 17;

__device__ __forceinline__ float kdecay(float gl, float g, bool gdn) {
    const float d = gl - g;
    return __expf(gdn ? fminf(d, 80.f) : fminf(d, 0.f));
}

// Row sums of squares of a [64][COLS] bf16 tile -> rstd[64] (1 when !use), 8 warps.
template <int COLS>
__device__ __forceinline__ void row_rstd(const unsigned char* tile, float* rstd, int use, int warp, int lane) {
    constexpr int CPR = COLS / 8;
    constexpr int RPP = 32 / CPR;
    const int sub = lane / CPR, cc = lane % CPR;
    for (int rr = 0; rr < 8; rr += RPP) {
        const int r = warp * 8 + rr + sub;
        const uint4 xv = *reinterpret_cast<const uint4*>(tile + swz<COLS * 2>(r, cc));
        const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xv);
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 t = unpack_bf16(xw[j]);
            ss += t.x * t.x + t.y * t.y;
        }
#pragma unroll
        for (int o = CPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (cc == 0) rstd[r] = use ? rsqrtf(ss + 1e-6f) : 1.0f;
    }
}

template <int COLS>
__device__ __forceinline__ void scale_rows(unsigned char* tile, const float* rowscale, int tid) {
    constexpr int CPR = COLS / 8;
    for (int i = tid; i < 64 * CPR; i += LB_THREADS) {
        const int r = i / CPR, c = i % CPR;
        uint4* p = reinterpret_cast<uint4*>(tile + swz<COLS * 2>(r, c));
        uint4 x = *p;
        const float s = rowscale[r];
        uint32_t* xw = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = unpack_bf16(xw[j]);
            xw[j] = pack_bf16(f.x * s, f.y * s);
        }
        *p = x;
    }
}

// ================================================================================================ pre
template <int K, int V>
struct PreSmem {
    static constexpr int qs = 0;
    static constexpr int ks = qs + 64 * K * 2;
    static constexpr int dos = ks + 64 * K * 2;
    static constexpr int ps = dos + 64 * V * 2;
    static constexpr int vec = ps + 64 * 64 * 2;          // g, q rstd, k rstd
    static constexpr int total = vec + 3 * 64 * 4;
};

template <int K, int V>
__global__ void __launch_bounds__(LB_THREADS)
linear_bwd_pre_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                      const __nv_bfloat16* __restrict__ d_o, const float* __restrict__ gcs, __nv_bfloat16* __restrict__ qn,
                      __nv_bfloat16* __restrict__ kn, float* __restrict__ q_rstd, float* __restrict__ k_rstd,
                      __nv_bfloat16* __restrict__ dvl, int T, int H, float scale, int use_l2norm) {
    using L = PreSmem<K, V>;
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, qd = lane & 3;
    const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int valid = min(64, T - c * 64);
    const long tok0 = (long)b * T + (long)c * 64;
    unsigned char* qs_p = smem + L::qs;
    unsigned char* ks_p = smem + L::ks;
    unsigned char* dos_p = smem + L::dos;
    unsigned char* ps_p = smem + L::ps;
    const uint32_t qs = smem_u32(qs_p), ks = smem_u32(ks_p), dos = smem_u32(dos_p), ps = smem_u32(ps_p);
    float* s_g = reinterpret_cast<float*>(smem + L::vec);
    float* s_qr = s_g + 64;
    float* s_kr = s_qr + 64;

    load_tile_async<64, K, LB_THREADS>(qs, q + (tok0 * H + h) * K, (long)H * K, valid, tid);
    load_tile_async<64, K, LB_THREADS>(ks, k + (tok0 * H + h) * K, (long)H * K, valid, tid);
    load_tile_async<64, V, LB_THREADS>(dos, d_o + (tok0 * H + h) * V, (long)H * V, valid, tid);
    cp_async_commit();
    if (tid < 64) s_g[tid] = gcs[(tok0 + min(tid, valid - 1)) * H + h];
    cp_async_wait<0>();
    __syncthreads();
    row_rstd<K>(qs_p, s_qr, use_l2norm, warp, lane);
    row_rstd<K>(ks_p, s_kr, use_l2norm, warp, lane);
    __syncthreads();
    if (use_l2norm) {
        scale_rows<K>(qs_p, s_qr, tid);
        scale_rows<K>(ks_p, s_kr, tid);
        if (tid < valid) {
            q_rstd[(tok0 + tid) * H + h] = s_qr[tid];
            k_rstd[(tok0 + tid) * H + h] = s_kr[tid];
        }
        __syncthreads();
        store_tile<64, K, LB_THREADS>(qs_p, qn + (tok0 * H + h) * K, (long)H * K, valid, tid);
        store_tile<64, K, LB_THREADS>(ks_p, kn + (tok0 * H + h) * K, (long)H * K, valid, tid);
    }
    // ---- P = tril(qn kn^T Gam)
    const int rw = warp & 3, half = warp >> 2;
    const int r0 = rw * 16;
    {
        float acc[4][4];
        zero_acc(acc);
        warp_gemm<K * 2, A_ROW, K * 2, B_NK, 4>(acc, qs, r0, ks, 32 * half, 0, K, lane);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = r0 + gq + ((e >> 1) << 3);
                const int j = 32 * half + nt * 8 + qd * 2 + (e & 1);
                acc[nt][e] = (j <= i && i < valid) ? acc[nt][e] * __expf(s_g[i] - s_g[j]) : 0.f;
            }
        store_acc_bf16<128, 4>(ps_p, acc, r0, 32 * half, lane);
    }
    __syncthreads();
    // ---- dv'_loc = s P^T do
    {
        constexpr int NT8 = V / 16;
        float acc[NT8][4];
        zero_acc(acc);
        warp_gemm<128, A_TRANS, V * 2, B_KN, NT8>(acc, ps, r0, dos, half * (V / 2), 0, 64, lane);
#pragma unroll
        for (int nt = 0; nt < NT8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[nt][e] *= scale;
        __syncthreads();                                   // every warp has read do
        store_acc_bf16<V * 2, NT8>(dos_p, acc, r0, half * (V / 2), lane);
    }
    __syncthreads();
    store_tile<64, V, LB_THREADS>(dos_p, dvl + (tok0 * H + h) * V, (long)H * V, valid, tid);
}

// ================================================================================================ dh (reverse walk)
constexpr int DH_THREADS = 128;

template <int K, int BV, bool GDN>
struct DhSmem {
    static constexpr int ks = 0;
    static constexpr int qs = ks + 64 * K * 2;
    static constexpr int ws = qs + 64 * K * 2;
    static constexpr int dob = ws + (GDN ? 64 * K * 2 : 0);   // do slice
    static constexpr int dvl = dob + 64 * BV * 2;             // dv'_loc slice
    static constexpr int dsb = dvl + 64 * BV * 2;             // dS as bf16 [K][BV]
    static constexpr int dos = dsb + K * BV * 2;              // s e^{g+car} do
    static constexpr int dvs = dos + 64 * BV * 2;             // -e^{car} dv'
    static constexpr int dvo = dvs + 64 * BV * 2;             // dv' (store staging)
    static constexpr int vec = dvo + 64 * BV * 2;             // g[64]
    static constexpr int meta = vec + 64 * 4;                 // per chunk: g_last, carry, act
    static int total(int NT) { return meta + NT * 12; }
};

template <int K, int BV, bool GDN>
__global__ void __launch_bounds__(DH_THREADS)
linear_bwd_dh_kernel(const __nv_bfloat16* __restrict__ qn, const __nv_bfloat16* __restrict__ kn,
                     const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ d_o,
                     const __nv_bfloat16* __restrict__ dvl_in, const float* __restrict__ gcs,
                     const float* __restrict__ carry_in, const int* __restrict__ types_i, const int* __restrict__ indices,
                     const int* __restrict__ n_blocks, const float* __restrict__ dht, __nv_bfloat16* __restrict__ dS_all,
                     __nv_bfloat16* __restrict__ dvp_out, float* __restrict__ dh0, int T, int H, int HN, int V, float scale) {
    using L = DhSmem<K, BV, GDN>;
    constexpr int MT = K / 64;
    constexpr int NTL = BV / 8;
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, qd = lane & 3;
    const int vsplit = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int v0 = vsplit * BV;
    const int hn = h / (H / HN);
    const int NT = (T + 63) / 64;
    const int TN = NT;
    const int nsel = n_blocks[((long)b * HN + hn) * 2 + 1];
    const int last_sel = nsel > 0 ? indices[(((long)b * TN + (nsel - 1)) * HN + hn) * 2 + 1] : -1;

    unsigned char* dsb_p = smem + L::dsb;
    unsigned char* dos_p = smem + L::dos;
    unsigned char* dvs_p = smem + L::dvs;
    unsigned char* dvo_p = smem + L::dvo;
    const unsigned char* dob_p = smem + L::dob;
    const unsigned char* dvl_p = smem + L::dvl;
    const uint32_t ks = smem_u32(smem + L::ks), qs = smem_u32(smem + L::qs), ws = smem_u32(smem + L::ws);
    const uint32_t dsb = smem_u32(dsb_p), dos = smem_u32(dos_p), dvs = smem_u32(dvs_p);
    float* s_g = reinterpret_cast<float*>(smem + L::vec);
    float* s_gl = reinterpret_cast<float*>(smem + L::meta);
    float* s_car = s_gl + NT;
    int* s_act = reinterpret_cast<int*>(s_car + NT);

    for (int c = tid; c < NT; c += DH_THREADS) {
        const int last_tok = min(c * 64 + 63, T - 1);
        s_gl[c] = gcs[((long)b * T + last_tok) * H + h];
        s_car[c] = carry_in[((long)b * NT + c) * H + h];
        s_act[c] = types_i[(((long)b * TN + c) * HN + hn) * 2 + 1] != 0;
    }
    __syncthreads();

    float dS[MT][NTL][4];
    const int krow0 = warp * (K / 4);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) zero_acc(dS[mt]);

    auto add_dht = [&]() {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NTL; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = krow0 + mt * 16 + gq + ((e >> 1) << 3);
                    const int cidx = v0 + nt * 8 + qd * 2 + (e & 1);
                    dS[mt][nt][e] += dht[(((long)b * H + h) * K + r) * V + cidx];
                }
    };

    const int r0 = warp * 16;
    const int ia = r0 + gq, ib = ia + 8;
    for (int c = NT - 1; c >= 0; --c) {
        const int valid = min(64, T - c * 64);
        const long tok0 = (long)b * T + (long)c * 64;
        const bool act = s_act[c] != 0;
        const float gl = s_gl[c], car = s_car[c];
        if (act) load_tile_async<64, K, DH_THREADS>(ks, kn + (tok0 * H + h) * K, (long)H * K, valid, tid);
        load_tile_async<64, K, DH_THREADS>(qs, qn + (tok0 * H + h) * K, (long)H * K, valid, tid);
        if (GDN) load_tile_async<64, K, DH_THREADS>(ws, w + (tok0 * H + h) * K, (long)H * K, valid, tid);
        load_tile_async<64, BV, DH_THREADS>(smem_u32(smem + L::dob), d_o + (tok0 * H + h) * V + v0, (long)H * V, valid, tid);
        load_tile_async<64, BV, DH_THREADS>(smem_u32(smem + L::dvl), dvl_in + (tok0 * H + h) * V + v0, (long)H * V, valid, tid);
        cp_async_commit();
        if (tid < 64) s_g[tid] = gcs[(tok0 + min(tid, valid - 1)) * H + h];
        if (dht && c == last_sel) add_dht();
        if (act) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) store_acc_bf16<BV * 2, NTL>(dsb_p, dS[mt], krow0 + mt * 16, 0, lane);
        }
        cp_async_wait<0>();
        __syncthreads();
        if (act) store_tile<K, BV, DH_THREADS>(dsb_p, dS_all + ((((long)b * NT + c) * H + h) * K) * V + v0, V, K, tid);

        // ---- dv' = act (kn dS) kd + dv'_loc
        float acc[NTL][4];
        zero_acc(acc);
        if (act) warp_gemm<K * 2, A_ROW, BV * 2, B_KN, NTL>(acc, ks, r0, dsb, 0, 0, K, lane);
        const float kda = kdecay(gl, s_g[ia], GDN), kdb = kdecay(gl, s_g[ib], GDN);
        const float ec = __expf(car);
        const float ea = scale * __expf(s_g[ia] + car), eb = scale * __expf(s_g[ib] + car);
#pragma unroll
        for (int nt = 0; nt < NTL; ++nt) {
            const int col = nt * 8 + qd * 2;
            const float2 la = load_pair_bf16<BV * 2>(dvl_p, ia, col), lb = load_pair_bf16<BV * 2>(dvl_p, ib, col);
            const float2 da = load_pair_bf16<BV * 2>(dob_p, ia, col), db = load_pair_bf16<BV * 2>(dob_p, ib, col);
            const float a0 = acc[nt][0] * kda + la.x, a1 = acc[nt][1] * kda + la.y;
            const float b0 = acc[nt][2] * kdb + lb.x, b1 = acc[nt][3] * kdb + lb.y;
            const uint32_t offa = swz<BV * 2>(ia, nt) + qd * 4, offb = swz<BV * 2>(ib, nt) + qd * 4;
            *reinterpret_cast<uint32_t*>(dvo_p + offa) = pack_bf16(a0, a1);
            *reinterpret_cast<uint32_t*>(dvo_p + offb) = pack_bf16(b0, b1);
            if (GDN) {
                // the rounded dv' is what the other kernels read: use it here too
                const float2 ra = unpack_bf16(pack_bf16(a0, a1)), rb = unpack_bf16(pack_bf16(b0, b1));
                *reinterpret_cast<uint32_t*>(dvs_p + offa) = pack_bf16(-ec * ra.x, -ec * ra.y);
                *reinterpret_cast<uint32_t*>(dvs_p + offb) = pack_bf16(-ec * rb.x, -ec * rb.y);
            }
            *reinterpret_cast<uint32_t*>(dos_p + offa) = pack_bf16(ea * da.x, ea * da.y);
            *reinterpret_cast<uint32_t*>(dos_p + offb) = pack_bf16(eb * db.x, eb * db.y);
        }
        __syncthreads();
        store_tile<64, BV, DH_THREADS>(dvo_p, dvp_out + (tok0 * H + h) * V + v0, (long)H * V, valid, tid);

        // ---- dS <- (act ? e^{g_L+car} : 1) dS + qn^T (s e^{g+car} do) + w^T (-e^{car} dv')
        if (act) {
            const float dec = __expf(gl + car);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < NTL; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) dS[mt][nt][e] *= dec;
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            warp_gemm<K * 2, A_TRANS, BV * 2, B_KN, NTL>(dS[mt], qs, krow0 + mt * 16, dos, 0, 0, 64, lane);
            if (GDN) warp_gemm<K * 2, A_TRANS, BV * 2, B_KN, NTL>(dS[mt], ws, krow0 + mt * 16, dvs, 0, 0, 64, lane);
        }
        __syncthreads();                                    // tiles are overwritten by the next chunk's loads
    }
    if (dht && last_sel < 0) add_dht();                     // no chunk updated the state: the final state is h0
    if (dh0) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NTL; ++nt) {
                const int r = krow0 + mt * 16 + gq;
                const int cidx = v0 + nt * 8 + qd * 2;
                float* p = dh0 + (((long)b * H + h) * K + r) * V + cidx;
                *reinterpret_cast<float2*>(p) = make_float2(dS[mt][nt][0], dS[mt][nt][1]);
                *reinterpret_cast<float2*>(p + 8L * V) = make_float2(dS[mt][nt][2], dS[mt][nt][3]);
            }
    }
}

// ================================================================================================ state
template <int K, int V, bool GDN>
struct StSmem {
    static constexpr int Ss = 0;                              // S [K][V]
    static constexpr int dSs = Ss + K * V * 2;                // dS [K][V]
    static constexpr int ks = dSs + K * V * 2;
    static constexpr int ws = ks + 64 * K * 2;
    static constexpr int us = ws + 64 * K * 2;                // u, then v'
    static constexpr int dvs = us + 64 * V * 2;               // dv'
    static constexpr int dos = dvs + 64 * V * 2;
    static constexpr int vs = dos + 64 * V * 2;               // raw v (chunks that do not update the state, GDN)
    static constexpr int vec = vs + (GDN ? 64 * V * 2 : 0);   // g[64], r[64], red[8 warps][2] + red2[2]
    static constexpr int total = vec + (64 + 64 + 32) * 4;
    static_assert(K * V * 2 >= 64 * K * 2, "the dS tile doubles as an output staging buffer");
};

template <int K, int V, bool GDN>
__global__ void __launch_bounds__(LB_THREADS)
linear_bwd_state_kernel(const __nv_bfloat16* __restrict__ kn, const __nv_bfloat16* __restrict__ v,
                        const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ u,
                        const __nv_bfloat16* __restrict__ d_o, const __nv_bfloat16* __restrict__ dvp,
                        const float* __restrict__ gcs, const __nv_bfloat16* __restrict__ hS,
                        const float* __restrict__ carry_in, const __nv_bfloat16* __restrict__ dS_all,
                        const int* __restrict__ types_i, const int* __restrict__ indices, const int* __restrict__ n_blocks,
                        const int* __restrict__ starting_h_idx, __nv_bfloat16* __restrict__ vp_out,
                        __nv_bfloat16* __restrict__ dw_out, __nv_bfloat16* __restrict__ dq1_out,
                        __nv_bfloat16* __restrict__ dk1_out, float* __restrict__ dkd_out, float* __restrict__ scal,
                        float* __restrict__ dnats_lin, int T, int H, int HN, float scale, int invalid_dnats) {
    using L = StSmem<K, V, GDN>;
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, qd = lane & 3;
    const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int hn = h / (H / HN);
    const int NT = (T + 63) / 64;
    const int TN = NT;
    const int valid = min(64, T - c * 64);
    const long tok0 = (long)b * T + (long)c * 64;
    const bool act = types_i[(((long)b * TN + c) * HN + hn) * 2 + 1] != 0;
    int slot = c;
    if (!act) {
        slot = -1;
        if (invalid_dnats) {
            const int nsel = n_blocks[((long)b * HN + hn) * 2 + 1];
            const int j = starting_h_idx[((long)b * NT + c) * HN + hn];      // updating chunks before this one
            if (j < nsel) slot = indices[(((long)b * TN + j) * HN + hn) * 2 + 1];
        }
    }
    unsigned char* Ss_p = smem + L::Ss;
    unsigned char* dSs_p = smem + L::dSs;
    unsigned char* ks_p = smem + L::ks;
    unsigned char* ws_p = smem + L::ws;
    unsigned char* us_p = smem + L::us;
    const unsigned char* dvs_p = smem + L::dvs;
    const unsigned char* vs_p = smem + L::vs;
    const uint32_t Ss = smem_u32(Ss_p), dSs = smem_u32(dSs_p), ks = smem_u32(ks_p), ws = smem_u32(ws_p), us = smem_u32(us_p),
                   dvs = smem_u32(smem + L::dvs), dos = smem_u32(smem + L::dos), vs = smem_u32(smem + L::vs);
    float* s_g = reinterpret_cast<float*>(smem + L::vec);
    float* s_r = s_g + 64;
    float* s_red = s_r + 64;

    const long st_off = (((long)b * NT + c) * H + h) * (long)K * V;
    load_tile_async<K, V, LB_THREADS>(Ss, hS + st_off, V, K, tid);
    if (GDN) load_tile_async<64, K, LB_THREADS>(ws, w + (tok0 * H + h) * K, (long)H * K, valid, tid);
    load_tile_async<64, V, LB_THREADS>(us, u + (tok0 * H + h) * V, (long)H * V, valid, tid);
    load_tile_async<64, V, LB_THREADS>(dvs, dvp + (tok0 * H + h) * V, (long)H * V, valid, tid);
    load_tile_async<64, V, LB_THREADS>(dos, d_o + (tok0 * H + h) * V, (long)H * V, valid, tid);
    if (slot >= 0) {
        load_tile_async<K, V, LB_THREADS>(dSs, dS_all + (((long)b * NT + slot) * H + h) * (long)K * V, V, K, tid);
        load_tile_async<64, K, LB_THREADS>(ks, kn + (tok0 * H + h) * K, (long)H * K, valid, tid);
        if (GDN && !act) load_tile_async<64, V, LB_THREADS>(vs, v + (tok0 * H + h) * V, (long)H * V, valid, tid);
    }
    cp_async_commit();
    if (tid < 64) {
        s_g[tid] = gcs[(tok0 + min(tid, valid - 1)) * H + h];
        s_r[tid] = 0.f;
    }
    if (tid < 32) s_red[tid] = 0.f;
    const float car = carry_in[((long)b * NT + c) * H + h];
    const float ec = __expf(car);
    cp_async_wait<0>();
    __syncthreads();
    const float gl = s_g[valid - 1];

    const int rw = warp & 3, half = warp >> 2;
    const int r0 = rw * 16;
    const int ia = r0 + gq, ib = ia + 8;
    constexpr int NV = V / 16, NK = K / 16;
    const int nv0 = half * (V / 2), nk0 = half * (K / 2);

    // ---- v' = u - e^{car} w S (over u, in place);  t1 = sum (w S) * dv'
    float t1 = 0.f;
    if (GDN) {
        float acc[NV][4];
        zero_acc(acc);
        warp_gemm<K * 2, A_ROW, V * 2, B_KN, NV>(acc, ws, r0, Ss, nv0, 0, K, lane);
#pragma unroll
        for (int nt = 0; nt < NV; ++nt) {
            const int col = nv0 + nt * 8 + qd * 2;
            uint32_t* pa = reinterpret_cast<uint32_t*>(us_p + swz<V * 2>(ia, col >> 3) + qd * 4);
            uint32_t* pb = reinterpret_cast<uint32_t*>(us_p + swz<V * 2>(ib, col >> 3) + qd * 4);
            const float2 ua = unpack_bf16(*pa), ub = unpack_bf16(*pb);
            const float2 da = load_pair_bf16<V * 2>(dvs_p, ia, col), db = load_pair_bf16<V * 2>(dvs_p, ib, col);
            t1 += acc[nt][0] * da.x + acc[nt][1] * da.y + acc[nt][2] * db.x + acc[nt][3] * db.y;
            *pa = pack_bf16(ua.x - ec * acc[nt][0], ua.y - ec * acc[nt][1]);
            *pb = pack_bf16(ub.x - ec * acc[nt][2], ub.y - ec * acc[nt][3]);
        }
    }
    __syncthreads();                                         // v' complete (rows are shared by two warps)

    // ---- r_i = sum_v (kn dS)_iv x_iv,  x = v' (updating chunk) or the raw values (other chunks, for dnats)
    if (slot >= 0) {
        float acc[NV][4];
        zero_acc(acc);
        warp_gemm<K * 2, A_ROW, V * 2, B_KN, NV>(acc, ks, r0, dSs, nv0, 0, K, lane);
        const unsigned char* x_p = (GDN && !act) ? vs_p : us_p;
        float ra = 0.f, rb = 0.f;
#pragma unroll
        for (int nt = 0; nt < NV; ++nt) {
            const int col = nv0 + nt * 8 + qd * 2;
            const float2 xa = load_pair_bf16<V * 2>(x_p, ia, col), xb = load_pair_bf16<V * 2>(x_p, ib, col);
            ra += acc[nt][0] * xa.x + acc[nt][1] * xa.y;
            rb += acc[nt][2] * xb.x + acc[nt][3] * xb.y;
        }
        ra = quad_sum(ra);
        rb = quad_sum(rb);
        if (qd == 0) {
            atomicAdd(&s_r[ia], ra);
            atomicAdd(&s_r[ib], rb);
        }
    }
    // ---- products with S and dS over the value dim: dkn1 = kd (v' dS^T), dqn1 = s e^{g+car} do S^T, dw = -e^{car} dv' S^T
    float acc_k[NK][4], acc_q[NK][4], acc_w[GDN ? NK : 2][4];
    zero_acc(acc_k);
    zero_acc(acc_q);
    if (act) warp_gemm<V * 2, A_ROW, V * 2, B_NK, NK>(acc_k, us, r0, dSs, nk0, 0, V, lane);
    warp_gemm<V * 2, A_ROW, V * 2, B_NK, NK>(acc_q, dos, r0, Ss, nk0, 0, V, lane);
    if constexpr (GDN) {
        zero_acc(acc_w);
        warp_gemm<V * 2, A_ROW, V * 2, B_NK, NK>(acc_w, dvs, r0, Ss, nk0, 0, V, lane);
    }
    {
        const float kda = kdecay(gl, s_g[ia], GDN), kdb = kdecay(gl, s_g[ib], GDN);
        const float ea = scale * __expf(s_g[ia] + car), eb = scale * __expf(s_g[ib] + car);
#pragma unroll
        for (int nt = 0; nt < NK; ++nt) {
            acc_k[nt][0] *= kda; acc_k[nt][1] *= kda; acc_k[nt][2] *= kdb; acc_k[nt][3] *= kdb;
            acc_q[nt][0] *= ea; acc_q[nt][1] *= ea; acc_q[nt][2] *= eb; acc_q[nt][3] *= eb;
            if constexpr (GDN) {
#pragma unroll
                for (int e = 0; e < 4; ++e) acc_w[nt][e] *= -ec;
            }
        }
    }
    // ---- ddec = e^{g_L+car} <dS, S>
    float dd = 0.f;
    if (act) {
        constexpr int CPR = V / 8;
        for (int i = tid; i < K * CPR; i += LB_THREADS) {
            const int r = i / CPR, cc = i % CPR;
            const uint4 a = *reinterpret_cast<const uint4*>(Ss_p + swz<V * 2>(r, cc));
            const uint4 d = *reinterpret_cast<const uint4*>(dSs_p + swz<V * 2>(r, cc));
            const uint32_t* aw = reinterpret_cast<const uint32_t*>(&a);
            const uint32_t* dw = reinterpret_cast<const uint32_t*>(&d);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 x = unpack_bf16(aw[j]), y = unpack_bf16(dw[j]);
                dd += x.x * y.x + x.y * y.y;
            }
        }
    }
    dd = warp_sum(dd);
    t1 = warp_sum(t1);
    if (lane == 0) {                                         // one slot per warp: the sums below have a fixed order
        s_red[2 * warp] = dd;
        s_red[2 * warp + 1] = t1;
    }
    __syncthreads();                                         // all products done: k, w, dS tiles become staging buffers
    // ---- per-token decay gradient of the state write, dnats
    if (tid < 64) {
        const float kd = kdecay(gl, s_g[tid], GDN);
        float val = (tid < valid) ? s_r[tid] * kd : 0.f;
        if (!GDN && gl - s_g[tid] > 0.f) val = 0.f;          // the clamp passes no gradient (never taken: g <= 0)
        if (tid < valid) dkd_out[(tok0 + tid) * H + h] = act ? val : 0.f;
        float dn = (tid < valid) ? s_r[tid] * kd : 0.f;
        dn = warp_sum(dn);
        if (lane == 0) s_red[16 + warp] = dn;
    }
    store_acc_bf16<K * 2, NK>(ks_p, acc_k, r0, nk0, lane);
    store_acc_bf16<K * 2, NK>(ws_p, acc_q, r0, nk0, lane);
    if constexpr (GDN) store_acc_bf16<K * 2, NK>(dSs_p, acc_w, r0, nk0, lane);
    __syncthreads();
    if (act) store_tile<64, K, LB_THREADS>(ks_p, dk1_out + (tok0 * H + h) * K, (long)H * K, valid, tid);
    store_tile<64, K, LB_THREADS>(ws_p, dq1_out + (tok0 * H + h) * K, (long)H * K, valid, tid);
    if (GDN) {
        store_tile<64, K, LB_THREADS>(dSs_p, dw_out + (tok0 * H + h) * K, (long)H * K, valid, tid);
        store_tile<64, V, LB_THREADS>(us_p, vp_out + (tok0 * H + h) * V, (long)H * V, valid, tid);
    }
    if (tid == 0) {
        float* sc = scal + (((long)b * NT + c) * H + h) * 4;
        const float dn = s_red[16] + s_red[17];
        float dd_tot = 0.f, t1_tot = 0.f;
        for (int wv = 0; wv < 8; ++wv) {
            dd_tot += s_red[2 * wv];
            t1_tot += s_red[2 * wv + 1];
        }
        sc[0] = act ? dd_tot * __expf(gl + car) : 0.f;       // ddec
        sc[1] = act ? dn : 0.f;                              // sum of the per-token decay gradients of the write
        sc[2] = ec * t1_tot;                                 // e^{car} <w S, dv'>
        dnats_lin[((long)b * NT + c) * H + h] = (slot >= 0) ? dn : 0.f;
    }
}

// ================================================================================================ intra
template <int K, int V, bool GDN>
struct InSmem {
    static constexpr int qns = 0;
    static constexpr int kns = qns + 64 * K * 2;
    static constexpr int ws = kns + 64 * K * 2;               // w; later dq staging
    static constexpr int dws = ws + 64 * K * 2;               // dw -> dzw; later dk staging
    static constexpr int vps = dws + 64 * K * 2;              // v'
    static constexpr int dos = vps + 64 * V * 2;
    static constexpr int m1 = dos + 64 * V * 2;               // dqk (bf16 64x64)
    static constexpr int us = m1 + 64 * 64 * 2;
    static constexpr int dvs = us + (GDN ? 64 * V * 2 : 0);   // dv' -> dzu -> dv
    static constexpr int vs = dvs + (GDN ? 64 * V * 2 : 0);
    static constexpr int m2 = vs + (GDN ? 64 * V * 2 : 0);    // dkk (bf16 64x64)
    static constexpr int hs = m2 + (GDN ? 64 * 64 * 2 : 0);   // H (bf16 64x64)
    static constexpr int As = hs + (GDN ? 64 * 64 * 2 : 0);   // A fp32 [64][68]
    static constexpr int Xs = As + (GDN ? 64 * LB_A_LD * 4 : 0);
    static constexpr int vec = Xs + (GDN ? 4 * 16 * LB_X_LD * 4 : 0);
    // g, beta, zk, dE, dotq, dotk (6 x 64); decay-gradient row sums [2 phases][2 halves][64] and column sums
    // [2 phases][4 row blocks][64]; dbeta parts [2 halves + value part][64]; + 16
    static constexpr int total = vec + ((6 + 4 + 8 + 3) * 64 + 16) * 4;
};

// In-place solve of (I + A)^T X = R for 32 columns [col0, col0+32) of a [64][COLS] bf16 tile by one warp:
// block back substitution with H_ii = (I + A_ii)^-1, H_ji = -A_ji H_ii (j > i):  X_i = sum_{j >= i} H_ji^T Y_j,
// Y_j = R_i for j = i and the already solved X_j for j > i.
template <int COLS>
__device__ __forceinline__ void solve_t_group(uint32_t htile, uint32_t ztile, unsigned char* zptr, int col0, int lane) {
#pragma unroll
    for (int i = 3; i >= 0; --i) {
        float acc[4][4];
        zero_acc(acc);
#pragma unroll
        for (int j = i; j < 4; ++j) {
            uint32_t af[4];
            load_a_t<128>(htile, 16 * i, 16 * j, lane, af);
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                uint32_t bf[4];
                load_b_kn<COLS * 2>(ztile, 16 * j, col0 + 16 * p, lane, bf);
                mma_bf16(acc[2 * p], af, bf[0], bf[1]);
                mma_bf16(acc[2 * p + 1], af, bf[2], bf[3]);
            }
        }
        __syncwarp();
        store_acc_bf16<COLS * 2, 4>(zptr, acc, 16 * i, col0, lane);
        __syncwarp();
    }
}

template <int K, int V, bool GDN>
__global__ void __launch_bounds__(LB_THREADS)
linear_bwd_intra_kernel(const __nv_bfloat16* __restrict__ qn, const __nv_bfloat16* __restrict__ kn,
                        const __nv_bfloat16* __restrict__ v, const __nv_bfloat16* __restrict__ w,
                        const __nv_bfloat16* __restrict__ u, const __nv_bfloat16* __restrict__ vp,
                        const __nv_bfloat16* __restrict__ dvp, const __nv_bfloat16* __restrict__ dw_in,
                        const __nv_bfloat16* __restrict__ d_o, const __nv_bfloat16* __restrict__ dq1,
                        const __nv_bfloat16* __restrict__ dk1, const float* __restrict__ gcs, const void* __restrict__ beta,
                        int beta_dtype, const float* __restrict__ q_rstd, const float* __restrict__ k_rstd,
                        const float* __restrict__ dkd, const int* __restrict__ types_i, __nv_bfloat16* __restrict__ dq,
                        __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv, float* __restrict__ dbeta,
                        float* __restrict__ dg_tok, float* __restrict__ scal, int T, int H, int HN, float scale,
                        int use_l2norm) {
    using L = InSmem<K, V, GDN>;
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, qd = lane & 3;
    const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int hn = h / (H / HN);
    const int NT = (T + 63) / 64;
    const int valid = min(64, T - c * 64);
    const long tok0 = (long)b * T + (long)c * 64;
    const bool act = types_i[(((long)b * NT + c) * HN + hn) * 2 + 1] != 0;

    unsigned char* qns_p = smem + L::qns;
    unsigned char* kns_p = smem + L::kns;
    unsigned char* ws_p = smem + L::ws;
    unsigned char* dws_p = smem + L::dws;
    unsigned char* m1_p = smem + L::m1;
    unsigned char* m2_p = smem + L::m2;
    unsigned char* hs_p = smem + L::hs;
    unsigned char* dvs_p = smem + L::dvs;
    const unsigned char* vs_p = smem + L::vs;
    const uint32_t qns = smem_u32(qns_p), kns = smem_u32(kns_p), ws = smem_u32(ws_p), dws = smem_u32(dws_p),
                   vps = smem_u32(smem + L::vps), dos = smem_u32(smem + L::dos), m1 = smem_u32(m1_p), us = smem_u32(smem + L::us),
                   dvs = smem_u32(dvs_p), m2 = smem_u32(m2_p), hs = smem_u32(hs_p);
    float* As = reinterpret_cast<float*>(smem + L::As);
    float* Xs = reinterpret_cast<float*>(smem + L::Xs);
    float* s_g = reinterpret_cast<float*>(smem + L::vec);
    float* s_b = s_g + 64;
    float* s_zk = s_b + 64;
    float* s_dE = s_zk + 64;
    float* s_dotq = s_dE + 64;
    float* s_dotk = s_dotq + 64;
    float* s_dgr = s_dotk + 64;                              // [phase][half][64]: one writer per slot, fixed summation order
    float* s_dgc = s_dgr + 4 * 64;                           // [phase][row block][64]
    float* s_dbp = s_dgc + 8 * 64;                           // [half 0 | half 1 | value part][64]
    float* s_red = s_dbp + 3 * 64;

    load_tile_async<64, K, LB_THREADS>(qns, qn + (tok0 * H + h) * K, (long)H * K, valid, tid);
    load_tile_async<64, K, LB_THREADS>(kns, kn + (tok0 * H + h) * K, (long)H * K, valid, tid);
    load_tile_async<64, V, LB_THREADS>(vps, vp + (tok0 * H + h) * V, (long)H * V, valid, tid);
    load_tile_async<64, V, LB_THREADS>(dos, d_o + (tok0 * H + h) * V, (long)H * V, valid, tid);
    if (GDN) {
        load_tile_async<64, K, LB_THREADS>(ws, w + (tok0 * H + h) * K, (long)H * K, valid, tid);
        load_tile_async<64, K, LB_THREADS>(dws, dw_in + (tok0 * H + h) * K, (long)H * K, valid, tid);
        load_tile_async<64, V, LB_THREADS>(us, u + (tok0 * H + h) * V, (long)H * V, valid, tid);
        load_tile_async<64, V, LB_THREADS>(dvs, dvp + (tok0 * H + h) * V, (long)H * V, valid, tid);
        load_tile_async<64, V, LB_THREADS>(smem_u32(smem + L::vs), v + (tok0 * H + h) * V, (long)H * V, valid, tid);
    }
    cp_async_commit();
    if (tid < 64) {
        const long gi = (tok0 + min(tid, valid - 1)) * H + h;
        s_g[tid] = gcs[gi];
        float bv = 0.f;
        if (GDN && tid < valid)
            bv = beta_dtype == NATSL_DT_F32 ? reinterpret_cast<const float*>(beta)[gi]
                                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(beta)[gi]);
        s_b[tid] = bv;
        s_zk[tid] = 0.f; s_dE[tid] = 0.f; s_dotq[tid] = 0.f; s_dotk[tid] = 0.f;
        for (int i = 0; i < 15; ++i) s_dgr[i * 64 + tid] = 0.f;
    }
    if (tid < 16) s_red[tid] = 0.f;
    cp_async_wait<0>();
    __syncthreads();

    const int rw = warp & 3, half = warp >> 2;
    const int r0 = rw * 16;
    const int ia = r0 + gq, ib = ia + 8;
    const int c0 = 32 * half;

    // ---- phase 1: qk, kk, dP;  dqk = s dP Gam (tril), A = strictLower(beta kk Gam), decay gradients of P
    float kk[4][4];
    zero_acc(kk);
    {
        float qk[4][4], dpr[4][4];
        zero_acc(qk);
        zero_acc(dpr);
        warp_gemm<K * 2, A_ROW, K * 2, B_NK, 4>(qk, qns, r0, kns, c0, 0, K, lane);
        if (GDN) warp_gemm<K * 2, A_ROW, K * 2, B_NK, 4>(kk, kns, r0, kns, c0, 0, K, lane);
        warp_gemm<V * 2, A_ROW, V * 2, B_NK, 4>(dpr, dos, r0, vps, c0, 0, V, lane);
        float rs_a = 0.f, rs_b = 0.f;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            float cs0 = 0.f, cs1 = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = (e >> 1) ? ib : ia;
                const int j = c0 + nt * 8 + qd * 2 + (e & 1);
                const bool low = j <= i && i < valid;
                const float gam = low ? __expf(s_g[i] - s_g[j]) : 0.f;
                const float dqk = scale * dpr[nt][e] * gam;
                const float dgam = dqk * qk[nt][e];
                if (e >> 1) rs_b += dgam; else rs_a += dgam;
                if (e & 1) cs1 += dgam; else cs0 += dgam;
                dpr[nt][e] = dqk;
                if (GDN) As[i * LB_A_LD + j] = (j < i && i < valid) ? s_b[i] * kk[nt][e] * gam : 0.f;
            }
            cs0 = colgroup_sum(cs0);
            cs1 = colgroup_sum(cs1);
            if (gq == 0) {
                s_dgc[(0 * 4 + rw) * 64 + c0 + nt * 8 + qd * 2] = -cs0;
                s_dgc[(0 * 4 + rw) * 64 + c0 + nt * 8 + qd * 2 + 1] = -cs1;
            }
        }
        rs_a = quad_sum(rs_a);
        rs_b = quad_sum(rs_b);
        if (qd == 0) {
            s_dgr[(0 * 2 + half) * 64 + ia] = rs_a;
            s_dgr[(0 * 2 + half) * 64 + ib] = rs_b;
        }
        store_acc_bf16<128, 4>(m1_p, dpr, r0, c0, lane);
    }
    __syncthreads();

    // ---- phase 2: dqn = dqk kn, dkn = dqk^T qn
    constexpr int NK = K / 16;
    const int nk0 = half * (K / 2);
    float acc_q[NK][4], acc_k[NK][4];
    zero_acc(acc_q);
    zero_acc(acc_k);
    warp_gemm<128, A_ROW, K * 2, B_KN, NK>(acc_q, m1, r0, kns, nk0, 0, 64, lane);
    warp_gemm<128, A_TRANS, K * 2, B_KN, NK>(acc_k, m1, r0, qns, nk0, 0, 64, lane);

    if (GDN) {
        // ---- phase 3: X_dd = (I + A_dd)^-1 (forward substitution, one warp per diagonal block), then H
        if (warp < 4 && lane < 16) {
            const int d0 = warp * 16, cidx = lane;
            float xcol[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float s = 0.f;
#pragma unroll
                for (int j = 0; j < i; ++j) s += As[(d0 + i) * LB_A_LD + d0 + j] * xcol[j];
                xcol[i] = ((i == cidx) ? 1.f : 0.f) - s;
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) Xs[(warp * 16 + i) * LB_X_LD + cidx] = xcol[i];
        }
        __syncthreads();
        for (int e = tid; e < 4 * 16 * 16; e += LB_THREADS) {          // diagonal blocks: H_dd = X_dd
            const int d = e >> 8, r = (e >> 4) & 15, cc = e & 15;
            const int row = d * 16 + r, col = d * 16 + cc;
            reinterpret_cast<__nv_bfloat16*>(hs_p + swz<128>(row, col >> 3))[col & 7] =
                __float2bfloat16(Xs[(d * 16 + r) * LB_X_LD + cc]);
        }
        for (int e = tid; e < 6 * 16 * 16; e += LB_THREADS) {          // below the diagonal: H_ji = -A_ji X_ii
            const int blk = e >> 8, r = (e >> 4) & 15, cc = e & 15;
            // block pairs (j, i): (1,0) (2,0) (2,1) (3,0) (3,1) (3,2)
            const int bj = blk < 1 ? 1 : (blk < 3 ? 2 : 3);
            const int bi = blk - (bj == 1 ? 0 : (bj == 2 ? 1 : 3));
            float a = 0.f;
#pragma unroll
            for (int m = 0; m < 16; ++m) a -= As[(bj * 16 + r) * LB_A_LD + bi * 16 + m] * Xs[(bi * 16 + m) * LB_X_LD + cc];
            const int row = bj * 16 + r, col = bi * 16 + cc;
            reinterpret_cast<__nv_bfloat16*>(hs_p + swz<128>(row, col >> 3))[col & 7] = __float2bfloat16(a);
        }
        __syncthreads();
        // ---- phase 4: [dzu | dzw] = (I + A)^-T [dv' | dw], in place, 32 columns per warp
        constexpr int NCG = (K + V) / 32;
        for (int cg = warp; cg < NCG; cg += 8) {
            if (cg < V / 32) solve_t_group<V>(hs, dvs, dvs_p, cg * 32, lane);
            else solve_t_group<K>(hs, dws, dws_p, (cg - V / 32) * 32, lane);
        }
        __syncthreads();
        // ---- phase 5: dA = -strictLower(dzu u^T + dzw w^T); dkk = dA beta Gam; gradients of beta and the decays
        {
            float dar[4][4];
            zero_acc(dar);
            warp_gemm<V * 2, A_ROW, V * 2, B_NK, 4>(dar, dvs, r0, us, c0, 0, V, lane);
            warp_gemm<K * 2, A_ROW, K * 2, B_NK, 4>(dar, dws, r0, ws, c0, 0, K, lane);
            float rs_a = 0.f, rs_b = 0.f, db_a = 0.f, db_b = 0.f;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                float cs0 = 0.f, cs1 = 0.f;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = (e >> 1) ? ib : ia;
                    const int j = c0 + nt * 8 + qd * 2 + (e & 1);
                    const bool low = j < i && i < valid;
                    const float gam = low ? __expf(s_g[i] - s_g[j]) : 0.f;
                    const float dA = low ? -dar[nt][e] : 0.f;
                    const float kg = kk[nt][e] * gam;
                    const float dgam = dA * s_b[i] * kg;                 // dA * A
                    if (e >> 1) { rs_b += dgam; db_b += dA * kg; } else { rs_a += dgam; db_a += dA * kg; }
                    if (e & 1) cs1 += dgam; else cs0 += dgam;
                    dar[nt][e] = dA * s_b[i] * gam;                      // dkk
                }
                cs0 = colgroup_sum(cs0);
                cs1 = colgroup_sum(cs1);
                if (gq == 0) {
                    s_dgc[(1 * 4 + rw) * 64 + c0 + nt * 8 + qd * 2] = -cs0;
                    s_dgc[(1 * 4 + rw) * 64 + c0 + nt * 8 + qd * 2 + 1] = -cs1;
                }
            }
            rs_a = quad_sum(rs_a); rs_b = quad_sum(rs_b);
            db_a = quad_sum(db_a); db_b = quad_sum(db_b);
            if (qd == 0) {
                s_dgr[(1 * 2 + half) * 64 + ia] = rs_a;
                s_dgr[(1 * 2 + half) * 64 + ib] = rs_b;
                s_dbp[half * 64 + ia] = db_a;
                s_dbp[half * 64 + ib] = db_b;
            }
            store_acc_bf16<128, 4>(m2_p, dar, r0, c0, lane);
        }
        __syncthreads();
        // ---- phase 6: dkn += dkk kn + dkk^T kn
        warp_gemm<128, A_ROW, K * 2, B_KN, NK>(acc_k, m2, r0, kns, nk0, 0, 64, lane);
        warp_gemm<128, A_TRANS, K * 2, B_KN, NK>(acc_k, m2, r0, kns, nk0, 0, 64, lane);
        // ---- dv = dzu beta (in place), dbeta += <dzu, v>
        {
            constexpr int CPR = V / 8;
            constexpr int RPP = 32 / CPR > 0 ? 32 / CPR : 1;
            static_assert(CPR <= 32, "value rows wider than 256 are not handled");
            const int sub = lane / CPR, cc = lane % CPR;
            for (int rr = 0; rr < 8; rr += RPP) {
                const int r = warp * 8 + rr + sub;
                uint4* pz = reinterpret_cast<uint4*>(dvs_p + swz<V * 2>(r, cc));
                uint4 z = *pz;
                const uint4 vv = *reinterpret_cast<const uint4*>(vs_p + swz<V * 2>(r, cc));
                uint32_t* zw = reinterpret_cast<uint32_t*>(&z);
                const uint32_t* vw = reinterpret_cast<const uint32_t*>(&vv);
                const float bt = s_b[r];
                float s = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 a = unpack_bf16(zw[j]), x = unpack_bf16(vw[j]);
                    s += a.x * x.x + a.y * x.y;
                    zw[j] = pack_bf16(a.x * bt, a.y * bt);
                }
                *pz = z;
#pragma unroll
                for (int o = CPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (cc == 0) s_dbp[2 * 64 + r] = s;
            }
        }
    }
    // ---- phase 7: per-element epilogue in the accumulator layout of dqn / dkn
    {
        const float ega = __expf(s_g[ia]), egb = __expf(s_g[ib]);
        const float fa = s_b[ia] * ega, fb = s_b[ib] * egb;
        float zk_a = 0.f, zk_b = 0.f, dE_a = 0.f, dE_b = 0.f;
        const __nv_bfloat16* dq1_a = dq1 + ((tok0 + ia) * H + h) * K;
        const __nv_bfloat16* dq1_b = dq1 + ((tok0 + ib) * H + h) * K;
        const __nv_bfloat16* dk1_a = dk1 + ((tok0 + ia) * H + h) * K;
        const __nv_bfloat16* dk1_b = dk1 + ((tok0 + ib) * H + h) * K;
#pragma unroll
        for (int nt = 0; nt < NK; ++nt) {
            const int col = nk0 + nt * 8 + qd * 2;
            const float2 kna = load_pair_bf16<K * 2>(kns_p, ia, col), knb = load_pair_bf16<K * 2>(kns_p, ib, col);
            const float2 qna = load_pair_bf16<K * 2>(qns_p, ia, col), qnb = load_pair_bf16<K * 2>(qns_p, ib, col);
            if (GDN) {
                const float2 za = load_pair_bf16<K * 2>(dws_p, ia, col), zb = load_pair_bf16<K * 2>(dws_p, ib, col);
                zk_a += za.x * kna.x + za.y * kna.y;
                zk_b += zb.x * knb.x + zb.y * knb.y;
                acc_k[nt][0] += za.x * fa; acc_k[nt][1] += za.y * fa;
                acc_k[nt][2] += zb.x * fb; acc_k[nt][3] += zb.y * fb;
            }
            if (ia < valid) {
                const float2 x = unpack_bf16(*reinterpret_cast<const uint32_t*>(dq1_a + col));
                acc_q[nt][0] += x.x; acc_q[nt][1] += x.y;
                dE_a += x.x * qna.x + x.y * qna.y;
                if (act) {
                    const float2 y = unpack_bf16(*reinterpret_cast<const uint32_t*>(dk1_a + col));
                    acc_k[nt][0] += y.x; acc_k[nt][1] += y.y;
                }
            }
            if (ib < valid) {
                const float2 x = unpack_bf16(*reinterpret_cast<const uint32_t*>(dq1_b + col));
                acc_q[nt][2] += x.x; acc_q[nt][3] += x.y;
                dE_b += x.x * qnb.x + x.y * qnb.y;
                if (act) {
                    const float2 y = unpack_bf16(*reinterpret_cast<const uint32_t*>(dk1_b + col));
                    acc_k[nt][2] += y.x; acc_k[nt][3] += y.y;
                }
            }
        }
        // dot products of the l2-norm backward, over the finished dqn / dkn
        float dq_a = 0.f, dq_b = 0.f, dk_a = 0.f, dk_b = 0.f;
#pragma unroll
        for (int nt = 0; nt < NK; ++nt) {
            const int col = nk0 + nt * 8 + qd * 2;
            const float2 kna = load_pair_bf16<K * 2>(kns_p, ia, col), knb = load_pair_bf16<K * 2>(kns_p, ib, col);
            const float2 qna = load_pair_bf16<K * 2>(qns_p, ia, col), qnb = load_pair_bf16<K * 2>(qns_p, ib, col);
            dq_a += acc_q[nt][0] * qna.x + acc_q[nt][1] * qna.y;
            dq_b += acc_q[nt][2] * qnb.x + acc_q[nt][3] * qnb.y;
            dk_a += acc_k[nt][0] * kna.x + acc_k[nt][1] * kna.y;
            dk_b += acc_k[nt][2] * knb.x + acc_k[nt][3] * knb.y;
        }
        zk_a = quad_sum(zk_a); zk_b = quad_sum(zk_b);
        dE_a = quad_sum(dE_a); dE_b = quad_sum(dE_b);
        dq_a = quad_sum(dq_a); dq_b = quad_sum(dq_b);
        dk_a = quad_sum(dk_a); dk_b = quad_sum(dk_b);
        if (qd == 0) {
            atomicAdd(&s_zk[ia], zk_a); atomicAdd(&s_zk[ib], zk_b);
            atomicAdd(&s_dE[ia], dE_a); atomicAdd(&s_dE[ib], dE_b);
            atomicAdd(&s_dotq[ia], dq_a); atomicAdd(&s_dotq[ib], dq_b);
            atomicAdd(&s_dotk[ia], dk_a); atomicAdd(&s_dotk[ib], dk_b);
        }
    }
    __syncthreads();                                         // row sums complete; w and dzw tiles are free
    // ---- phase 8: l2-norm backward, staging, stores
    {
        float qra = 1.f, qrb = 1.f, kra = 1.f, krb = 1.f;
        if (use_l2norm) {
            qra = ia < valid ? q_rstd[(tok0 + ia) * H + h] : 0.f;
            qrb = ib < valid ? q_rstd[(tok0 + ib) * H + h] : 0.f;
            kra = ia < valid ? k_rstd[(tok0 + ia) * H + h] : 0.f;
            krb = ib < valid ? k_rstd[(tok0 + ib) * H + h] : 0.f;
        }
        const float pq_a = use_l2norm ? s_dotq[ia] : 0.f, pq_b = use_l2norm ? s_dotq[ib] : 0.f;
        const float pk_a = use_l2norm ? s_dotk[ia] : 0.f, pk_b = use_l2norm ? s_dotk[ib] : 0.f;
#pragma unroll
        for (int nt = 0; nt < NK; ++nt) {
            const int col = nk0 + nt * 8 + qd * 2;
            const float2 kna = load_pair_bf16<K * 2>(kns_p, ia, col), knb = load_pair_bf16<K * 2>(kns_p, ib, col);
            const float2 qna = load_pair_bf16<K * 2>(qns_p, ia, col), qnb = load_pair_bf16<K * 2>(qns_p, ib, col);
            acc_q[nt][0] = qra * (acc_q[nt][0] - qna.x * pq_a); acc_q[nt][1] = qra * (acc_q[nt][1] - qna.y * pq_a);
            acc_q[nt][2] = qrb * (acc_q[nt][2] - qnb.x * pq_b); acc_q[nt][3] = qrb * (acc_q[nt][3] - qnb.y * pq_b);
            acc_k[nt][0] = kra * (acc_k[nt][0] - kna.x * pk_a); acc_k[nt][1] = kra * (acc_k[nt][1] - kna.y * pk_a);
            acc_k[nt][2] = krb * (acc_k[nt][2] - knb.x * pk_b); acc_k[nt][3] = krb * (acc_k[nt][3] - knb.y * pk_b);
        }
        store_acc_bf16<K * 2, NK>(ws_p, acc_q, r0, nk0, lane);
        store_acc_bf16<K * 2, NK>(dws_p, acc_k, r0, nk0, lane);
    }
    if (tid < 64) {
        const float eg = __expf(s_g[tid]);
        const float dE = s_dE[tid];
        if (tid < valid) {
            const long gi = (tok0 + tid) * H + h;
            float dgt = (s_dgr[tid] + s_dgr[64 + tid]) +
                        ((s_dgc[tid] + s_dgc[64 + tid]) + (s_dgc[128 + tid] + s_dgc[192 + tid])) + dE - dkd[gi];
            if (GDN) {
                dgt += (s_dgr[128 + tid] + s_dgr[192 + tid]) +
                       ((s_dgc[256 + tid] + s_dgc[320 + tid]) + (s_dgc[384 + tid] + s_dgc[448 + tid]));
                dgt += s_zk[tid] * s_b[tid] * eg;
                dbeta[gi] = (s_dbp[tid] + s_dbp[64 + tid]) + s_dbp[128 + tid] + eg * s_zk[tid];
            }
            dg_tok[gi] = dgt;
        }
        float se = (tid < valid) ? dE : 0.f;
        se = warp_sum(se);
        if (lane == 0) atomicAdd(&s_red[0], se);
    }
    __syncthreads();
    store_tile<64, K, LB_THREADS>(ws_p, dq + (tok0 * H + h) * K, (long)H * K, valid, tid);
    store_tile<64, K, LB_THREADS>(dws_p, dk + (tok0 * H + h) * K, (long)H * K, valid, tid);
    if (GDN) store_tile<64, V, LB_THREADS>(dvs_p, dv + (tok0 * H + h) * V, (long)H * V, valid, tid);
    if (tid == 0) scal[(((long)b * NT + c) * H + h) * 4 + 3] = s_red[0];
}

// ================================================================================================ dg
// One CTA per (batch, head): the carried-decay chain over the chunks in reverse, then the reverse
// cumsum inside every chunk.  scal [B,NT,H,4] = (ddec, sum dkd, e^{car} <w S, dv'>, sum dE) per chunk.
constexpr int DG_THREADS = 256;
__global__ void __launch_bounds__(DG_THREADS)
linear_bwd_dg_kernel(const float* __restrict__ dg_tok, const float* __restrict__ scal, const int* __restrict__ types_i,
                     const int* __restrict__ indices, const int* __restrict__ n_blocks, float* __restrict__ dg, int T, int H,
                     int HN, int decay, int trailing_quirk) {
    extern __shared__ float s_dgl[];
    const int tid = threadIdx.x, lane = tid & 31;
    const int h = blockIdx.x, b = blockIdx.y;
    const int hn = h / (H / HN);
    const int NT = (T + 63) / 64;
    const int TN = NT;
    // stage the per-chunk scalars in shared memory (parallel loads), then one thread walks the chain
    float* s_sc = s_dgl + NT;                               // [NT][4]
    int* s_act = reinterpret_cast<int*>(s_sc + 4 * NT);     // [NT]
    for (int i = tid; i < 4 * NT; i += DG_THREADS) s_sc[i] = scal[((long)b * NT + i / 4) * H * 4 + (long)h * 4 + (i & 3)];
    for (int c = tid; c < NT; c += DG_THREADS) s_act[c] = types_i[(((long)b * TN + c) * HN + hn) * 2 + 1] != 0;
    __syncthreads();
    if (tid == 0) {
        const int nsel = n_blocks[((long)b * HN + hn) * 2 + 1];
        const int last_sel = nsel > 0 ? indices[(((long)b * TN + (nsel - 1)) * HN + hn) * 2 + 1] : -1;
        float dcar = 0.f;                                    // gradient w.r.t. the carry after the chunk
        for (int c = NT - 1; c >= 0; --c) {
            const float* sc = s_sc + 4 * c;
            const bool act = s_act[c] != 0;
            const bool may_carry = decay && (!trailing_quirk || c < last_sel);
            float dgl;
            if (act) dgl = sc[0] + sc[1];
            else dgl = may_carry ? dcar : 0.f;
            s_dgl[c] = dgl;
            dcar = (act ? sc[0] : dcar) + (sc[3] - sc[2]);
        }
    }
    __syncthreads();
    // reverse cumsum inside every chunk: one warp per chunk, two tokens per lane
    const int warp = tid >> 5;
    for (int c = warp; c < NT; c += DG_THREADS / 32) {
        const int valid = min(64, T - c * 64);
        const long tok0 = (long)b * T + (long)c * 64;
        const int ta = 2 * lane, tb2 = 2 * lane + 1;
        float x0 = ta < valid ? dg_tok[(tok0 + ta) * H + h] : 0.f;
        float x1 = tb2 < valid ? dg_tok[(tok0 + tb2) * H + h] : 0.f;
        if (ta == valid - 1) x0 += s_dgl[c];
        if (tb2 == valid - 1) x1 += s_dgl[c];
        float sfx = x0 + x1;                                 // inclusive suffix sum of the lanes' pair sums
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_down_sync(0xffffffffu, sfx, o);
            if (lane + o < 32) sfx += t;
        }
        const float after = sfx - (x0 + x1);                 // everything behind this lane's pair
        if (ta < valid) dg[(tok0 + ta) * H + h] = x0 + x1 + after;
        if (tb2 < valid) dg[(tok0 + tb2) * H + h] = x1 + after;
    }
}

// ================================================================================================ launchers
static inline const __nv_bfloat16* bfc(const void* p) { return reinterpret_cast<const __nv_bfloat16*>(p); }
static inline __nv_bfloat16* bfm(void* p) { return reinterpret_cast<__nv_bfloat16*>(p); }

template <typename Kern>
static int reserve_smem(Kern kern, int bytes, const char* who) {
    if (bytes > 227 * 1024) {
        set_error("%s: needs %d B of shared memory (max %d)", who, bytes, 227 * 1024);
        return NATSL_ERR_TOO_LARGE;
    }
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) {
        set_error("%s: cannot reserve %d B of shared memory (%s)", who, bytes, cudaGetErrorString(e));
        return NATSL_ERR_CUDA;
    }
    return NATSL_OK;
}

template <int K, int V>
static int launch_pre(const void* q, const void* k, const void* d_o, const float* gcs, void* qn, void* kn, float* q_rstd,
                      float* k_rstd, void* dvl, int B, int T, int H, float scale, int use_l2norm, cudaStream_t st) {
    auto kern = linear_bwd_pre_kernel<K, V>;
    int rc = reserve_smem(kern, PreSmem<K, V>::total, "natsl_linear_bwd_pre");
    if (rc != NATSL_OK) return rc;
    kern<<<dim3((T + 63) / 64, H, B), LB_THREADS, PreSmem<K, V>::total, st>>>(bfc(q), bfc(k), bfc(d_o), gcs, bfm(qn), bfm(kn),
                                                                              q_rstd, k_rstd, bfm(dvl), T, H, scale, use_l2norm);
    return check_launch("natsl_linear_bwd_pre");
}

template <int K, int BV, bool GDN>
static int launch_dh(const void* qn, const void* kn, const void* w, const void* d_o, const void* dvl, const float* gcs,
                     const float* carry, const int* types_i, const int* indices, const int* n_blocks, const float* dht,
                     void* dS_all, void* dvp, float* dh0, int B, int T, int H, int HN, int V, float scale, cudaStream_t st) {
    auto kern = linear_bwd_dh_kernel<K, BV, GDN>;
    const int NT = (T + 63) / 64;
    const int smem = DhSmem<K, BV, GDN>::total(NT);
    int rc = reserve_smem(kern, smem, "natsl_linear_bwd_dh");
    if (rc != NATSL_OK) return rc;
    kern<<<dim3(V / BV, H, B), DH_THREADS, smem, st>>>(bfc(qn), bfc(kn), bfc(w), bfc(d_o), bfc(dvl), gcs, carry, types_i,
                                                       indices, n_blocks, dht, bfm(dS_all), bfm(dvp), dh0, T, H, HN, V, scale);
    return check_launch("natsl_linear_bwd_dh");
}

template <int K, int V, bool GDN>
static int launch_state(const void* kn, const void* v, const void* w, const void* u, const void* d_o, const void* dvp,
                        const float* gcs, const void* hS, const float* carry, const void* dS_all, const int* types_i,
                        const int* indices, const int* n_blocks, const int* shi, void* vp, void* dw, void* dq1, void* dk1,
                        float* dkd, float* scal, float* dnats_lin, int B, int T, int H, int HN, float scale, int invalid,
                        cudaStream_t st) {
    auto kern = linear_bwd_state_kernel<K, V, GDN>;
    int rc = reserve_smem(kern, StSmem<K, V, GDN>::total, "natsl_linear_bwd_state");
    if (rc != NATSL_OK) return rc;
    kern<<<dim3((T + 63) / 64, H, B), LB_THREADS, StSmem<K, V, GDN>::total, st>>>(
        bfc(kn), bfc(v), bfc(w), bfc(u), bfc(d_o), bfc(dvp), gcs, bfc(hS), carry, bfc(dS_all), types_i, indices, n_blocks, shi,
        bfm(vp), bfm(dw), bfm(dq1), bfm(dk1), dkd, scal, dnats_lin, T, H, HN, scale, invalid);
    return check_launch("natsl_linear_bwd_state");
}

template <int K, int V, bool GDN>
static int launch_intra(const void* qn, const void* kn, const void* v, const void* w, const void* u, const void* vp,
                        const void* dvp, const void* dw, const void* d_o, const void* dq1, const void* dk1, const float* gcs,
                        const void* beta, int beta_dtype, const float* q_rstd, const float* k_rstd, const float* dkd,
                        const int* types_i, void* dq, void* dk, void* dv, float* dbeta, float* dg_tok, float* scal, int B,
                        int T, int H, int HN, float scale, int use_l2norm, cudaStream_t st) {
    auto kern = linear_bwd_intra_kernel<K, V, GDN>;
    int rc = reserve_smem(kern, InSmem<K, V, GDN>::total, "natsl_linear_bwd_intra");
    if (rc != NATSL_OK) return rc;
    kern<<<dim3((T + 63) / 64, H, B), LB_THREADS, InSmem<K, V, GDN>::total, st>>>(
        bfc(qn), bfc(kn), bfc(v), bfc(w), bfc(u), bfc(vp), bfc(dvp), bfc(dw), bfc(d_o), bfc(dq1), bfc(dk1), gcs, beta,
        beta_dtype, q_rstd, k_rstd, dkd, types_i, bfm(dq), bfm(dk), bfm(dv), dbeta, dg_tok, scal, T, H, HN, scale, use_l2norm);
    return check_launch("natsl_linear_bwd_intra");
}

}  // namespace natsl

// ------------------------------------------------------------------------------------------------ C ABI
extern "C" int natsl_linear_bwd_pre(const void* q, const void* k, const void* d_o, const float* gcs, void* qn, void* kn,
                                    float* q_rstd, float* k_rstd, void* dvl, int B, int T, int H, int K, int V, float scale,
                                    int use_l2norm, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(q && k && d_o && gcs && dvl, NATSL_ERR_NULL, "natsl_linear_bwd_pre: null pointer");
    NATSL_REQUIRE(!use_l2norm || (qn && kn && q_rstd && k_rstd), NATSL_ERR_NULL,
                  "natsl_linear_bwd_pre: the normalised copies and 1/norm outputs are required with use_l2norm");
    NATSL_REQUIRE(B > 0 && T > 0 && H > 0 && B <= 65535 && H <= 65535, NATSL_ERR_BAD_SHAPE, "natsl_linear_bwd_pre: bad shape");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define NATSL_CASE(KK, VV) \
    if (K == KK && V == VV) return launch_pre<KK, VV>(q, k, d_o, gcs, qn, kn, q_rstd, k_rstd, dvl, B, T, H, scale, use_l2norm, st);
    NATSL_CASE(64, 64) NATSL_CASE(64, 128) NATSL_CASE(128, 64) NATSL_CASE(128, 128)
#undef NATSL_CASE
    set_error("natsl_linear_bwd_pre: unsupported head dims K=%d V=%d (64 or 128 each)", K, V);
    return NATSL_ERR_UNSUPPORTED;
}

extern "C" int natsl_linear_bwd_dh(int rule, const void* qn, const void* kn, const void* w, const void* d_o, const void* dvl,
                                   const float* gcs, const float* carry, const int32_t* types_i, const int32_t* indices,
                                   const int32_t* n_blocks, const float* dht, void* dS_all, void* dvp, float* dh0, int B,
                                   int T, int H, int HN, int K, int V, float scale, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(qn && kn && d_o && dvl && gcs && carry && types_i && indices && n_blocks && dS_all && dvp, NATSL_ERR_NULL,
                  "natsl_linear_bwd_dh: null pointer");
    NATSL_REQUIRE(rule == NATSL_RULE_GDN || rule == NATSL_RULE_MAMBA, NATSL_ERR_UNSUPPORTED, "natsl_linear_bwd_dh: unknown rule");
    NATSL_REQUIRE(rule != NATSL_RULE_GDN || w, NATSL_ERR_NULL, "natsl_linear_bwd_dh: w is required for the delta rule");
    NATSL_REQUIRE(B > 0 && T > 0 && H > 0 && HN > 0 && H % HN == 0 && B <= 65535 && H <= 65535, NATSL_ERR_BAD_SHAPE,
                  "natsl_linear_bwd_dh: bad shape");
    NATSL_REQUIRE(V % 32 == 0, NATSL_ERR_UNSUPPORTED, "natsl_linear_bwd_dh: V must be a multiple of 32");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define NATSL_ARGS qn, kn, w, d_o, dvl, gcs, carry, types_i, indices, n_blocks, dht, dS_all, dvp, dh0, B, T, H, HN, V, scale, st
    if (rule == NATSL_RULE_GDN) {
        if (K == 64) return launch_dh<64, 32, true>(NATSL_ARGS);
        if (K == 128) return launch_dh<128, 32, true>(NATSL_ARGS);
    } else {
        if (K == 64) return launch_dh<64, 32, false>(NATSL_ARGS);
        if (K == 128) return launch_dh<128, 32, false>(NATSL_ARGS);
    }
#undef NATSL_ARGS
    set_error("natsl_linear_bwd_dh: unsupported key dim K=%d (64 or 128)", K);
    return NATSL_ERR_UNSUPPORTED;
}

extern "C" int natsl_linear_bwd_state(int rule, const void* kn, const void* v, const void* w, const void* u, const void* d_o,
                                      const void* dvp, const float* gcs, const void* h, const float* carry, const void* dS_all,
                                      const int32_t* types_i, const int32_t* indices, const int32_t* n_blocks,
                                      const int32_t* starting_h_idx, void* vp, void* dw, void* dq1, void* dk1, float* dkd,
                                      float* scal, float* dnats_lin, int B, int T, int H, int HN, int K, int V, float scale,
                                      int invalid_dnats, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(kn && u && d_o && dvp && gcs && h && carry && dS_all && types_i && indices && n_blocks && starting_h_idx &&
                      dq1 && dk1 && dkd && scal && dnats_lin,
                  NATSL_ERR_NULL, "natsl_linear_bwd_state: null pointer");
    NATSL_REQUIRE(rule == NATSL_RULE_GDN || rule == NATSL_RULE_MAMBA, NATSL_ERR_UNSUPPORTED, "natsl_linear_bwd_state: unknown rule");
    NATSL_REQUIRE(rule != NATSL_RULE_GDN || (v && w && vp && dw), NATSL_ERR_NULL,
                  "natsl_linear_bwd_state: v, w, vp and dw are required for the delta rule");
    NATSL_REQUIRE(B > 0 && T > 0 && H > 0 && HN > 0 && H % HN == 0 && B <= 65535 && H <= 65535, NATSL_ERR_BAD_SHAPE,
                  "natsl_linear_bwd_state: bad shape");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define NATSL_ARGS kn, v, w, u, d_o, dvp, gcs, h, carry, dS_all, types_i, indices, n_blocks, starting_h_idx, vp, dw, dq1, dk1, dkd, scal, dnats_lin, B, T, H, HN, scale, invalid_dnats, st
#define NATSL_CASE(KK, VV)                                                             \
    if (K == KK && V == VV)                                                            \
        return rule == NATSL_RULE_GDN ? launch_state<KK, VV, true>(NATSL_ARGS) : launch_state<KK, VV, false>(NATSL_ARGS);
    NATSL_CASE(64, 64) NATSL_CASE(64, 128) NATSL_CASE(128, 64) NATSL_CASE(128, 128)
#undef NATSL_CASE
#undef NATSL_ARGS
    set_error("natsl_linear_bwd_state: unsupported head dims K=%d V=%d (64 or 128 each)", K, V);
    return NATSL_ERR_UNSUPPORTED;
}

extern "C" int natsl_linear_bwd_intra(int rule, const void* qn, const void* kn, const void* v, const void* w, const void* u,
                                      const void* vp, const void* dvp, const void* dw, const void* d_o, const void* dq1,
                                      const void* dk1, const float* gcs, const void* beta, int beta_dtype, const float* q_rstd,
                                      const float* k_rstd, const float* dkd, const int32_t* types_i, void* dq, void* dk,
                                      void* dv, float* dbeta, float* dg_tok, float* scal, int B, int T, int H, int HN, int K,
                                      int V, float scale, int use_l2norm, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(qn && kn && vp && d_o && dq1 && dk1 && gcs && dkd && types_i && dq && dk && dg_tok && scal, NATSL_ERR_NULL,
                  "natsl_linear_bwd_intra: null pointer");
    NATSL_REQUIRE(rule == NATSL_RULE_GDN || rule == NATSL_RULE_MAMBA, NATSL_ERR_UNSUPPORTED, "natsl_linear_bwd_intra: unknown rule");
    NATSL_REQUIRE(rule != NATSL_RULE_GDN || (v && w && u && dvp && dw && beta && dv && dbeta), NATSL_ERR_NULL,
                  "natsl_linear_bwd_intra: v, w, u, dvp, dw, beta, dv and dbeta are required for the delta rule");
    NATSL_REQUIRE(!use_l2norm || (q_rstd && k_rstd), NATSL_ERR_NULL, "natsl_linear_bwd_intra: 1/norm factors are required");
    NATSL_REQUIRE(B > 0 && T > 0 && H > 0 && HN > 0 && H % HN == 0 && B <= 65535 && H <= 65535, NATSL_ERR_BAD_SHAPE,
                  "natsl_linear_bwd_intra: bad shape");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define NATSL_ARGS qn, kn, v, w, u, vp, dvp, dw, d_o, dq1, dk1, gcs, beta, beta_dtype, q_rstd, k_rstd, dkd, types_i, dq, dk, dv, dbeta, dg_tok, scal, B, T, H, HN, scale, use_l2norm, st
#define NATSL_CASE(KK, VV)                                                             \
    if (K == KK && V == VV)                                                            \
        return rule == NATSL_RULE_GDN ? launch_intra<KK, VV, true>(NATSL_ARGS) : launch_intra<KK, VV, false>(NATSL_ARGS);
    NATSL_CASE(64, 64) NATSL_CASE(64, 128) NATSL_CASE(128, 64) NATSL_CASE(128, 128)
#undef NATSL_CASE
#undef NATSL_ARGS
    set_error("natsl_linear_bwd_intra: unsupported head dims K=%d V=%d (64 or 128 each)", K, V);
    return NATSL_ERR_UNSUPPORTED;
}

extern "C" int natsl_linear_bwd_dg(const float* dg_tok, const float* scal, const int32_t* types_i, const int32_t* indices,
                                   const int32_t* n_blocks, float* dg, int B, int T, int H, int HN, int flags, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(dg_tok && scal && types_i && indices && n_blocks && dg, NATSL_ERR_NULL, "natsl_linear_bwd_dg: null pointer");
    NATSL_REQUIRE(B > 0 && T > 0 && H > 0 && HN > 0 && H % HN == 0 && B <= 65535, NATSL_ERR_BAD_SHAPE,
                  "natsl_linear_bwd_dg: bad shape");
    const int NT = (T + 63) / 64;
    NATSL_REQUIRE(NT * 24 <= 48 * 1024, NATSL_ERR_TOO_LARGE, "natsl_linear_bwd_dg: T=%d is too long", T);
    const int decay = (flags & NATSL_FLAG_DECAY_SKIPPED) ? 1 : 0;
    const int quirk = (flags & NATSL_FLAG_NO_TRAILING_QUIRK) ? 0 : 1;
    linear_bwd_dg_kernel<<<dim3(H, B), DG_THREADS, NT * 24, reinterpret_cast<cudaStream_t>(stream)>>>(dg_tok, scal, types_i, indices,
                                                                                           n_blocks, dg, T, H, HN, decay, quirk);
    return check_launch("natsl_linear_bwd_dg");
}
