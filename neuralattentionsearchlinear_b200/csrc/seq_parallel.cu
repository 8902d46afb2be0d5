// Kernels of the sequence-parallel path (long sequences split into contiguous segments over GPUs).
//
// Linear branch (Mamba2/SSD, scalar decay): over one segment the carried state obeys
//     h_out = a * h_in + S_loc,    a = exp(sum of the log decays the carried state sees in the segment)
// (all tokens with decay over skipped blocks, else only tokens of selected blocks), so every rank
// runs its recurrence from a zero state, the (a, S_loc) pairs are all-gathered, and
// natsl_sp_state_combine folds the ranks before it into the state the segment really starts from.
// The reference has no sequence-parallel code; the recurrence these follow is
// src/nats/ops/mamba/chunk_h.py:139-218.
//
// Softmax branch: a rank only needs the *selected* key/value blocks of earlier ranks.
// natsl_pack_selected_blocks compacts them per head (index table order) into a token-major buffer
// that is all-gathered and placed in front of the rank's own keys.
#include "tc_common.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

// a[b,h]     = exp(sum over blocks of the segment that decay the carried state of that block's total log decay)
// trail[b,h] = exp(sum over the skipped blocks after the last selected block) (1 without decay over skipped blocks):
//              the recurrence kernel returns the state right after the last selected block; times trail it is the
//              state at the end of the segment.
__global__ void segment_decay_kernel(const float* __restrict__ gcs, const int* __restrict__ types_i,
                                     float* __restrict__ a_out, float* __restrict__ trail_out, int B, int T, int H,
                                     int HN, int TN, int nbs, int decay) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= B * H) return;
    const int b = i / H, h = i % H, hn = h / (H / HN);
    const int NT = (T + 63) / 64, cpb = nbs / 64;
    float acc = 0.f, tr = 0.f;
    for (int c = 0; c < NT; ++c) {
        const int sel = types_i[(((long)b * TN + c / cpb) * HN + hn) * 2 + 1];
        const float gl = gcs[((long)b * T + min(c * 64 + 63, T - 1)) * H + h];
        if (decay || sel) acc += gl;
        if (sel) tr = 0.f; else if (decay) tr += gl;
    }
    a_out[i] = __expf(acc);
    trail_out[i] = __expf(tr);
}

// h_in[b,h,:,:] = sum_{r < rank} (prod_{r < r' < rank} a[r',b,h]) * S[r,b,h,:,:]
__global__ void state_combine_kernel(const float* __restrict__ a, const float* __restrict__ S, float* __restrict__ h_in,
                                     int rank, long bh, long kv) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= bh * kv) return;
    const long g = i / kv;
    float acc = 0.f, f = 1.f;
    for (int r = rank - 1; r >= 0; --r) {
        acc += f * S[(long)r * bh * kv + i];
        f *= a[(long)r * bh + g];
    }
    h_in[i] = acc;
}

// P[0] = h0 (or 0), P[i+1] = a[i] * P[i] + S[i]: exclusive prefixes, the total state and the total decay.
__global__ void prefix_states_kernel(const float* __restrict__ a, const float* __restrict__ S, const float* __restrict__ h0,
                                     float* __restrict__ prefix, float* __restrict__ total_S, float* __restrict__ total_a,
                                     int N, long bh, long kv) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= bh * kv) return;
    const long g = i / kv;
    float p = h0 ? h0[i] : 0.f, f = 1.f;
    for (int n = 0; n < N; ++n) {
        if (prefix) prefix[(long)n * bh * kv + i] = p;
        const float an = a[(long)n * bh + g];
        p = an * p + S[(long)n * bh * kv + i];
        f *= an;
    }
    if (total_S) total_S[i] = p;
    if (total_a && i % kv == 0) total_a[g] = f;
}

// packed[b, j*nbs + i, h, :] = x[b, idx[b,j,hn,op]*nbs + i, h, :]   for j < min(n_sel, cap)
__global__ void __launch_bounds__(256)
pack_blocks_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ indices, const int* __restrict__ n_blocks,
                   __nv_bfloat16* __restrict__ packed, int T, int H, int HN, int TN, int D, int nbs, int op, int cap) {
    const int j = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int hn = h / (H / HN);
    const int n = n_blocks[((long)b * HN + hn) * 2 + op];
    if (j >= n) return;
    const int blk = indices[(((long)b * TN + j) * HN + hn) * 2 + op];
    const int cpr = D / 8;                          // 16-byte chunks per row
    for (int e = threadIdx.x; e < nbs * cpr; e += blockDim.x) {
        const int i = e / cpr, c = e % cpr;
        const long t = (long)blk * nbs + i;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t < T) v = *reinterpret_cast<const uint4*>(x + (((long)b * T + t) * H + h) * D + c * 8);
        *reinterpret_cast<uint4*>(packed + (((long)b * cap * nbs + (long)j * nbs + i) * H + h) * D + c * 8) = v;
    }
}

// Same blocks, no padding: pair p = (sum of the counts of the heads before h) + j of batch entry b goes to
// packed[b, p*nbs + i, :].
__global__ void __launch_bounds__(256)
pack_pairs_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ indices, const int* __restrict__ n_blocks,
                  __nv_bfloat16* __restrict__ packed, int T, int H, int HN, int TN, int D, int nbs, int op, int cap,
                  int max_per_head, int* status) {
    const int j = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int G = H / HN, hn = h / G;
    const int n = n_blocks[((long)b * HN + hn) * 2 + op];
    if (j >= n) return;
    if (max_per_head > 0 && n > max_per_head && threadIdx.x == 0) atomicExch(status, NATSL_DEV_CAPACITY);
    int base = 0;
    for (int g = 0; g < hn; ++g) base += n_blocks[((long)b * HN + g) * 2 + op];
    base = base * G + (h - hn * G) * n;
    const int pidx = base + j;
    if (pidx >= cap) {
        if (threadIdx.x == 0) atomicExch(status, NATSL_DEV_CAPACITY);
        return;
    }
    const int blk = indices[(((long)b * TN + j) * HN + hn) * 2 + op];
    const int cpr = D / 8;                          // 16-byte chunks per row
    for (int e = threadIdx.x; e < nbs * cpr; e += blockDim.x) {
        const int i = e / cpr, c = e % cpr;
        const long t = (long)blk * nbs + i;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t < T) v = *reinterpret_cast<const uint4*>(x + (((long)b * T + t) * H + h) * D + c * 8);
        *reinterpret_cast<uint4*>(packed + (((long)b * cap + pidx) * nbs + i) * D + c * 8) = v;
    }
}

}  // namespace natsl

extern "C" int natsl_sp_segment_decay(const float* gcs, const int32_t* types_i, float* a, float* trail, int B, int T,
                                      int H, int HN, int nbs, int flags, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(gcs && types_i && a && trail, NATSL_ERR_NULL, "natsl_sp_segment_decay: null pointer");
    NATSL_REQUIRE(B > 0 && T > 0 && H > 0 && HN > 0 && H % HN == 0 && nbs >= 64 && nbs % 64 == 0, NATSL_ERR_BAD_SHAPE,
                  "natsl_sp_segment_decay: bad shape");
    const int TN = (T + nbs - 1) / nbs;
    segment_decay_kernel<<<(B * H + 127) / 128, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        gcs, types_i, a, trail, B, T, H, HN, TN, nbs, (flags & NATSL_FLAG_DECAY_SKIPPED) ? 1 : 0);
    return check_launch("natsl_sp_segment_decay");
}

extern "C" int natsl_sp_state_combine(const float* a, const float* S, float* h_in, int rank, int world, int B, int H,
                                      int K, int V, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(a && S && h_in, NATSL_ERR_NULL, "natsl_sp_state_combine: null pointer");
    NATSL_REQUIRE(world > 0 && rank >= 0 && rank < world && B > 0 && H > 0 && K > 0 && V > 0, NATSL_ERR_BAD_SHAPE,
                  "natsl_sp_state_combine: bad rank/shape");
    const long bh = (long)B * H, kv = (long)K * V;
    state_combine_kernel<<<(unsigned)((bh * kv + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        a, S, h_in, rank, bh, kv);
    return check_launch("natsl_sp_state_combine");
}

extern "C" int natsl_sp_prefix_states(const float* a, const float* S, const float* h0, float* prefix, float* total_S,
                                      float* total_a, int N, int B, int H, int K, int V, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(a && S, NATSL_ERR_NULL, "natsl_sp_prefix_states: null pointer");
    NATSL_REQUIRE(N > 0 && B > 0 && H > 0 && K > 0 && V > 0, NATSL_ERR_BAD_SHAPE, "natsl_sp_prefix_states: bad shape");
    const long bh = (long)B * H, kv = (long)K * V;
    prefix_states_kernel<<<(unsigned)((bh * kv + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        a, S, h0, prefix, total_S, total_a, N, bh, kv);
    return check_launch("natsl_sp_prefix_states");
}

extern "C" int natsl_pack_selected_blocks(const void* x, const int32_t* indices, const int32_t* n_blocks, void* packed,
                                          int B, int T, int H, int HN, int D, int nbs, int op, int cap_blocks,
                                          void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(x && indices && n_blocks && packed, NATSL_ERR_NULL, "natsl_pack_selected_blocks: null pointer");
    NATSL_REQUIRE(B > 0 && T > 0 && H > 0 && HN > 0 && H % HN == 0 && D % 8 == 0 && (op == 0 || op == 1),
                  NATSL_ERR_BAD_SHAPE, "natsl_pack_selected_blocks: bad shape");
    NATSL_REQUIRE(H <= 65535 && B <= 65535, NATSL_ERR_TOO_LARGE, "natsl_pack_selected_blocks: B, H <= 65535");
    if (cap_blocks <= 0) return NATSL_OK;
    const int TN = (T + nbs - 1) / nbs;
    dim3 grid(cap_blocks, H, B);
    pack_blocks_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const __nv_bfloat16*>(x), indices, n_blocks, reinterpret_cast<__nv_bfloat16*>(packed), T, H, HN,
        TN, D, nbs, op, cap_blocks);
    return check_launch("natsl_pack_selected_blocks");
}

extern "C" int natsl_pack_selected_pairs(const void* x, const int32_t* indices, const int32_t* n_blocks, void* packed,
                                         int B, int T, int H, int HN, int D, int nbs, int op, int cap_pairs,
                                         int max_per_head, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(x && indices && n_blocks && packed, NATSL_ERR_NULL, "natsl_pack_selected_pairs: null pointer");
    NATSL_REQUIRE(B > 0 && T > 0 && H > 0 && HN > 0 && H % HN == 0 && D % 8 == 0 && (op == 0 || op == 1),
                  NATSL_ERR_BAD_SHAPE, "natsl_pack_selected_pairs: bad shape");
    NATSL_REQUIRE(H <= 65535 && B <= 65535, NATSL_ERR_TOO_LARGE, "natsl_pack_selected_pairs: B, H <= 65535");
    if (cap_pairs <= 0) return NATSL_OK;
    int* status = nullptr;
    int rc = status_word_ptr(&status);
    if (rc != NATSL_OK) return rc;
    const int TN = (T + nbs - 1) / nbs;
    dim3 grid(TN, H, B);
    pack_pairs_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const __nv_bfloat16*>(x), indices, n_blocks, reinterpret_cast<__nv_bfloat16*>(packed), T, H, HN,
        TN, D, nbs, op, cap_pairs, max_per_head, status);
    return check_launch("natsl_pack_selected_pairs");
}
