// Warp-level tile products on mma.sync for the backward kernels: one warp accumulates a 16-row strip
//     acc[16 x 8*NT8] += A[16 x k] * B[k x 8*NT8]
// from bf16 operand tiles in XOR-swizzled shared memory (swz<ROW_BYTES>() of common.cuh).  The four storage
// combinations cover every product of the backward pass without a transposed copy of any tile:
//     A_ROW   : A stored row-major [m][k]            A_TRANS : A = M^T with M stored row-major [k][m]
//     B_NK    : B^T stored row-major [n][k]          B_KN    : B stored row-major [k][n]
// Accumulator element acc[nt][e] of lane (gq = lane >> 2, qd = lane & 3) is
//     row = m0 + gq + 8 * (e >> 1),   column = n0 + 8 * nt + 2 * qd + (e & 1).
#pragma once
#include "common.cuh"

namespace natsl {

enum : int { A_ROW = 0, A_TRANS = 1 };
enum : int { B_NK = 0, B_KN = 1 };

template <int NT8>
__device__ __forceinline__ void zero_acc(float (&acc)[NT8][4]) {
#pragma unroll
    for (int i = 0; i < NT8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
}

// acc += A[m0.., k_begin..k_end) * B[k_begin..k_end), n0..)   (k range a multiple of 16)
template <int A_RB, int A_MODE, int B_RB, int B_MODE, int NT8>
__device__ __forceinline__ void warp_gemm(float (&acc)[NT8][4], uint32_t atile, int m0, uint32_t btile, int n0, int k_begin,
                                          int k_end, int lane) {
    static_assert(NT8 % 2 == 0, "n-tiles come in pairs");
#pragma unroll 2
    for (int k0 = k_begin; k0 < k_end; k0 += 16) {
        uint32_t a[4];
        if (A_MODE == A_ROW) load_a<A_RB>(atile, m0, k0, lane, a);
        else load_a_t<A_RB>(atile, m0, k0, lane, a);
#pragma unroll
        for (int p = 0; p < NT8 / 2; ++p) {
            uint32_t b[4];
            if (B_MODE == B_NK) load_b_nk<B_RB>(btile, n0 + 16 * p, k0, lane, b);
            else load_b_kn<B_RB>(btile, k0, n0 + 16 * p, lane, b);
            mma_bf16(acc[2 * p], a, b[0], b[1]);
            mma_bf16(acc[2 * p + 1], a, b[2], b[3]);
        }
    }
}

// Same with A taken from registers: afrag[j] is the A fragment of contraction step j (16 values of k each),
// typically made from an accumulator strip with acc_to_afrag().  B rows start at kb0.
template <int KSTEPS, int B_RB, int B_MODE, int NT8>
__device__ __forceinline__ void warp_gemm_ra(float (&acc)[NT8][4], const uint32_t (&afrag)[KSTEPS][4], uint32_t btile, int n0,
                                             int kb0, int lane) {
#pragma unroll
    for (int j = 0; j < KSTEPS; ++j) {
#pragma unroll
        for (int p = 0; p < NT8 / 2; ++p) {
            uint32_t b[4];
            if (B_MODE == B_NK) load_b_nk<B_RB>(btile, n0 + 16 * p, kb0 + 16 * j, lane, b);
            else load_b_kn<B_RB>(btile, kb0 + 16 * j, n0 + 16 * p, lane, b);
            mma_bf16(acc[2 * p], afrag[j], b[0], b[1]);
            mma_bf16(acc[2 * p + 1], afrag[j], b[2], b[3]);
        }
    }
}

// A 16 x (8*NT8) accumulator strip, rounded to bf16, is the A operand of a product that contracts over its columns.
template <int NT8>
__device__ __forceinline__ void acc_to_afrag(const float (&acc)[NT8][4], uint32_t (&afrag)[NT8 / 2][4]) {
#pragma unroll
    for (int j = 0; j < NT8 / 2; ++j) {
        afrag[j][0] = pack_bf16(acc[2 * j][0], acc[2 * j][1]);
        afrag[j][1] = pack_bf16(acc[2 * j][2], acc[2 * j][3]);
        afrag[j][2] = pack_bf16(acc[2 * j + 1][0], acc[2 * j + 1][1]);
        afrag[j][3] = pack_bf16(acc[2 * j + 1][2], acc[2 * j + 1][3]);
    }
}

// Write a strip (rows m0.., columns n0..) into a swizzled bf16 tile with ROW_BYTES-long rows.
template <int RB, int NT8>
__device__ __forceinline__ void store_acc_bf16(unsigned char* tile, const float (&acc)[NT8][4], int m0, int n0, int lane) {
    const int gq = lane >> 2, qd = lane & 3;
#pragma unroll
    for (int nt = 0; nt < NT8; ++nt) {
        const int ch = (n0 >> 3) + nt;
        *reinterpret_cast<uint32_t*>(tile + swz<RB>(m0 + gq, ch) + qd * 4) = pack_bf16(acc[nt][0], acc[nt][1]);
        *reinterpret_cast<uint32_t*>(tile + swz<RB>(m0 + gq + 8, ch) + qd * 4) = pack_bf16(acc[nt][2], acc[nt][3]);
    }
}

// The two bf16 values at (row, column n0 + 8*nt + 2*qd, +1) of a swizzled tile (the positions acc[nt][0..1] or
// acc[nt][2..3] of the lane address).
template <int RB>
__device__ __forceinline__ float2 load_pair_bf16(const unsigned char* tile, int row, int col) {
    return unpack_bf16(*reinterpret_cast<const uint32_t*>(tile + swz<RB>(row, col >> 3) + (col & 7) * 2));
}

// Sum over the four lanes that share an accumulator row.
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v;
}
// Sum over the eight lanes (gq = 0..7) that share an accumulator column pair.
__device__ __forceinline__ float colgroup_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    v += __shfl_xor_sync(0xffffffffu, v, 16);
    return v;
}

}  // namespace natsl
