// Chunk-local inclusive cumsum of the per-token log decay over 64-token chunks
// (what the reference gets from flash-linear-attention's chunk_local_cumsum, called at
// src/nats/ops/mamba/chunk.py:49-51 and src/nats/ops/gated_delta_rule/chunk.py:52-54).
// Pure bandwidth: consecutive threads take consecutive heads so every load/store is coalesced.
#include "common.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

__global__ void chunk_cumsum_kernel(const float* __restrict__ g, float* __restrict__ gcs, int T, int H, long n_units) {
    const long unit = (long)blockIdx.x * blockDim.x + threadIdx.x;      // (b, chunk, h)
    if (unit >= n_units) return;
    const int NT = (T + 63) / 64;
    const int h = unit % H;
    const long bc = unit / H;
    const int c = bc % NT;
    const long b = bc / NT;
    const int t0 = c * 64, t1 = min(T, t0 + 64);
    float acc = 0.f;
    for (int t = t0; t < t1; ++t) {
        long i = (b * T + t) * H + h;
        acc += g[i];
        gcs[i] = acc;
    }
}

}  // namespace natsl

extern "C" int natsl_chunk_local_cumsum(const float* g, float* gcs, int B, int T, int H, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(g && gcs, NATSL_ERR_NULL, "natsl_chunk_local_cumsum: null pointer");
    NATSL_REQUIRE(B > 0 && T > 0 && H > 0, NATSL_ERR_BAD_SHAPE, "natsl_chunk_local_cumsum: empty shape");
    const long n = (long)B * ((T + 63) / 64) * H;
    const int threads = 128;
    chunk_cumsum_kernel<<<(unsigned)((n + threads - 1) / threads), threads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        g, gcs, T, H, n);
    return check_launch("natsl_chunk_local_cumsum");
}
