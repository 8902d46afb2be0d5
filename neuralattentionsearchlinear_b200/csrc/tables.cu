// Selection tables.  One launch turns the per-(block, head) op types into every
// integer table of the path, on the device, without the host round trip the
// reference takes (a Python loop over a device tensor).  All outputs are int32 and
// equal, value for value, to what the reference computes with
//   src/nats/ops/mixed_ops/mixed_attn_gdn.py:88-100  (round, index sort, block counts)
//   src/nats/ops/nats_util.py:6-32    prepare_nats_block_indices
//   src/nats/ops/nats_util.py:35-64   prepare_nats_chunk_offsets
//   src/nats/ops/nats_util.py:67-121  compute_attn_n_iters_per_block
//   src/nats/ops/nats_util.py:124-162 compute_starting_idx_for_chunks
// Pure integer / byte work, HBM- and latency-bound: one CTA per (batch, selection
// head) compacts the selected block ids with a block-wide prefix sum; the "sort" of
// the reference is that compaction (selected ids are already ascending).
#include "common.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

constexpr int TBL_THREADS = 256;

__device__ __forceinline__ float load_type(const void* p, int dtype, long i) {
    switch (dtype) {
        case NATSL_DT_BF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
        case NATSL_DT_F32: return reinterpret_cast<const float*>(p)[i];
        case NATSL_DT_F16: return __half2float(reinterpret_cast<const __half*>(p)[i]);
        default: return (float)reinterpret_cast<const int*>(p)[i];
    }
}

// number of entries of the ascending list idx[0..n) (stride elements apart) that are < x
__device__ __forceinline__ int count_below(const int* idx, long stride, int n, int x) {
    int lo = 0, hi = n;
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (idx[(long)mid * stride] < x) lo = mid + 1; else hi = mid;
    }
    return lo;
}

__global__ void __launch_bounds__(TBL_THREADS)
tables_kernel(const void* __restrict__ types, int dtype, int B, int TN, int HN, int T, int nbs, int attn_bt,
              int* __restrict__ types_i, int* __restrict__ indices, int* __restrict__ n_blocks,
              int* __restrict__ n_chunks_lin, int* __restrict__ starting_h_idx, int* __restrict__ attn_n_iters) {
    __shared__ int warp_tot[TBL_THREADS / 32];
    __shared__ int s_n[2];
    const int bh = blockIdx.x, b = bh / HN, hn = bh % HN;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const long stride = (long)HN * 2;                       // between consecutive blocks of one (b, hn, op)
    for (int op = 0; op < 2; ++op) {
        const long base = ((long)b * TN * HN + hn) * 2 + op;
        int running = 0;
        for (int i0 = 0; i0 < TN; i0 += TBL_THREADS) {
            int i = i0 + tid;
            int flag = 0;
            if (i < TN) {
                flag = (rintf(load_type(types, dtype, base + (long)i * stride)) == 1.0f) ? 1 : 0;
                types_i[base + (long)i * stride] = flag;
            }
            unsigned bal = __ballot_sync(0xffffffffu, flag);
            int excl = __popc(bal & ((1u << lane) - 1));
            if (lane == 0) warp_tot[wid] = __popc(bal);
            __syncthreads();
            int off = 0, tot = 0;
#pragma unroll
            for (int w = 0; w < TBL_THREADS / 32; ++w) {
                int v = warp_tot[w];
                if (w < wid) off += v;
                tot += v;
            }
            if (flag) indices[base + (long)(running + off + excl) * stride] = i;
            running += tot;
            __syncthreads();
        }
        for (int j = running + tid; j < TN; j += TBL_THREADS) indices[base + (long)j * stride] = TN;
        if (tid == 0) {
            n_blocks[(long)bh * 2 + op] = running;
            s_n[op] = running;
            if (op == 1) n_chunks_lin[bh] = running * (nbs / NATSL_CHUNK);
        }
    }
    __syncthreads();   // indices written by this CTA are visible to it from here on
    const int NT = (T + NATSL_CHUNK - 1) / NATSL_CHUNK;
    const int* lin = indices + ((long)b * TN * HN + hn) * 2 + 1;
    for (int i = tid; i < NT; i += TBL_THREADS) {
        // #selected linear blocks with idx*nbs < i*64  <=>  idx < ceil(i*64 / nbs)
        int x = (i * NATSL_CHUNK + nbs - 1) / nbs;
        starting_h_idx[((long)b * NT + i) * HN + hn] = count_below(lin, stride, s_n[1], x);
    }
    const int NTq = (T + attn_bt - 1) / attn_bt;
    const int* att = indices + ((long)b * TN * HN + hn) * 2;
    for (int i = tid; i < NTq; i += TBL_THREADS) {
        // #selected attention blocks with (idx+1)*nbs <= i*attn_bt  <=>  idx < floor(i*attn_bt / nbs)
        int x = (i * attn_bt) / nbs;
        attn_n_iters[((long)b * NTq + i) * HN + hn] = count_below(att, stride, s_n[0], x);
    }
}

// offsets = exclusive prefix sum of the per-(b, hn) selected compute-chunk counts (single CTA),
// then the (flat b*HN+hn, local j) list.
__global__ void __launch_bounds__(TBL_THREADS)
offsets_kernel(const int* __restrict__ n_chunks_lin, int n, int* __restrict__ offsets) {
    __shared__ int warp_tot[TBL_THREADS / 32];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    int running = 0;
    if (tid == 0) offsets[0] = 0;
    for (int i0 = 0; i0 < n; i0 += TBL_THREADS) {
        int i = i0 + tid;
        int v = i < n ? n_chunks_lin[i] : 0;
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warp_tot[wid] = incl;
        __syncthreads();
        int off = 0, tot = 0;
#pragma unroll
        for (int w = 0; w < TBL_THREADS / 32; ++w) {
            int t = warp_tot[w];
            if (w < wid) off += t;
            tot += t;
        }
        if (i < n) offsets[i + 1] = running + off + incl;
        running += tot;
        __syncthreads();
    }
}

__global__ void chunk_indices_kernel(const int* __restrict__ offsets, int* __restrict__ chunk_indices) {
    const int bh = blockIdx.x;
    const int lo = offsets[bh], hi = offsets[bh + 1];
    for (int j = lo + threadIdx.x; j < hi; j += blockDim.x) {
        chunk_indices[2 * (long)j] = bh;
        chunk_indices[2 * (long)j + 1] = j - lo;
    }
}

}  // namespace natsl

extern "C" int natsl_build_tables(const void* types, int types_dtype, int B, int TN, int HN, int T, int nbs,
                                  int attn_bt, int32_t* types_i, int32_t* indices, int32_t* n_blocks,
                                  int32_t* n_chunks_lin, int32_t* offsets, int32_t* chunk_indices,
                                  int32_t* starting_h_idx, int32_t* attn_n_iters, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(types && types_i && indices && n_blocks && n_chunks_lin && offsets && starting_h_idx && attn_n_iters,
                  NATSL_ERR_NULL, "natsl_build_tables: null pointer");
    NATSL_REQUIRE(B > 0 && TN > 0 && HN > 0 && T > 0, NATSL_ERR_BAD_SHAPE, "natsl_build_tables: empty shape");
    NATSL_REQUIRE(nbs >= NATSL_CHUNK && nbs % NATSL_CHUNK == 0, NATSL_ERR_UNSUPPORTED,
                  "natsl_build_tables: nats_block_size must be a multiple of 64 (got %d)", nbs);
    NATSL_REQUIRE(TN == (T + nbs - 1) / nbs, NATSL_ERR_BAD_SHAPE,
                  "natsl_build_tables: TN=%d does not match cdiv(T=%d, nbs=%d)", TN, T, nbs);
    NATSL_REQUIRE(attn_bt > 0 && types_dtype >= 0 && types_dtype <= NATSL_DT_I32, NATSL_ERR_UNSUPPORTED,
                  "natsl_build_tables: bad attn_bt/dtype");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    tables_kernel<<<B * HN, TBL_THREADS, 0, st>>>(types, types_dtype, B, TN, HN, T, nbs, attn_bt, types_i, indices,
                                                  n_blocks, n_chunks_lin, starting_h_idx, attn_n_iters);
    offsets_kernel<<<1, TBL_THREADS, 0, st>>>(n_chunks_lin, B * HN, offsets);
    if (chunk_indices) chunk_indices_kernel<<<B * HN, 128, 0, st>>>(offsets, chunk_indices);
    return check_launch("natsl_build_tables");
}
