// natsl_gdn_fwd_noalloc: the gated-delta-rule branch forward (chunk preparation -> state
// recurrence -> chunk output) for callers that are not allowed to allocate device memory.
//
// Who that is: host code that runs where a device allocation is off limits — a serving loop whose
// memory plan is fixed at start-up and whose allocator belongs to another runtime, a plugin invoked
// from inside another framework's execution callback (where cudaMalloc may synchronise the whole
// device or is simply forbidden), or a worker that is handed only its input and output buffers.
// The regular entry points need six intermediate buffers from the caller (w, u, gcs, k_rstd, the
// per-chunk states h and the carry); this one takes them from a fixed array that lives in the
// library image instead, so the caller passes inputs and outputs only.
//
// Limits and rules:
//  * The array is NATSL_NOALLOC_SCRATCH_BYTES (32 MiB) per GPU that loads the library, held until
//    the process exits.  A call whose intermediates need more is rejected with NATSL_ERR_TOO_LARGE
//    and a message that states both numbers; nothing is launched.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current) and caches it.  Make that first call outside any stream capture.
//  * No cudaMalloc / cudaFree / allocating library routine is called here or in the kernels' launchers.
//  * All calls on a device share the one array and it keeps the previous call's contents.  Every
//    element a call reads it has written earlier in the same call (rows past the end of a ragged
//    last chunk are zero-filled on load, never read from the array), so nothing has to be cleared.
//    Two calls that overlap in time on the same GPU (different streams or threads) race on the
//    array: serialise them.
#include <mutex>

#include "common.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

static __device__ __align__(256) unsigned char g_noalloc_scratch[NATSL_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
static std::mutex g_setup_mutex;
static unsigned char* g_scratch_addr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device (looked up once per device).
static int scratch_for_current_device(unsigned char** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_error("natsl_gdn_fwd_noalloc: cannot identify the current device (%s)", cudaGetErrorString(e));
        return NATSL_ERR_CUDA;
    }
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_addr[dev] == nullptr) {
        unsigned char* p = nullptr;
        // In host code the array's name is only a handle; the kernels need its address on this device.
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr) {
            set_error("natsl_gdn_fwd_noalloc: cudaGetSymbolAddress failed on device %d (%s)", dev,
                      cudaGetErrorString(e));
            return NATSL_ERR_CUDA;
        }
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return NATSL_OK;
}

static inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

}  // namespace natsl

extern "C" int natsl_gdn_fwd_noalloc(const void* q, const void* k, const void* v, const float* g, const void* beta,
                                     int beta_dtype, const int32_t* types_i, const int32_t* indices,
                                     const int32_t* n_blocks, const float* h0, void* o, float* ht, int B, int T, int H,
                                     int HN, int K, int V, int nbs, float scale, int flags, int use_l2norm,
                                     void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(q && k && v && g && beta && types_i && indices && n_blocks && o, NATSL_ERR_NULL,
                  "natsl_gdn_fwd_noalloc: null pointer");
    NATSL_REQUIRE(B > 0 && T > 0 && H > 0 && K > 0 && V > 0, NATSL_ERR_BAD_SHAPE, "natsl_gdn_fwd_noalloc: empty shape");
    // Everything the three stages would reject is rejected here, before the first launch: a refused call
    // must leave the shared array (and the outputs) untouched.
    NATSL_REQUIRE(HN > 0 && H % HN == 0, NATSL_ERR_BAD_SHAPE, "natsl_gdn_fwd_noalloc: %d heads over %d selection heads", H,
                  HN);
    NATSL_REQUIRE(nbs >= 64 && nbs % 64 == 0, NATSL_ERR_UNSUPPORTED,
                  "natsl_gdn_fwd_noalloc: nats_block_size must be a multiple of 64 (got %d)", nbs);
    NATSL_REQUIRE((K == 64 && (V == 64 || V == 128)) || (K == 128 && (V == 64 || V == 128 || V == 256)),
                  NATSL_ERR_UNSUPPORTED,
                  "natsl_gdn_fwd_noalloc: unsupported head dims K=%d V=%d (K in {64,128}, V in {64,128,256})", K, V);
    NATSL_REQUIRE(beta_dtype == NATSL_DT_BF16 || beta_dtype == NATSL_DT_F32, NATSL_ERR_UNSUPPORTED,
                  "natsl_gdn_fwd_noalloc: beta must be bf16 or f32");
    NATSL_REQUIRE(B <= 65535 && (long)H * (V / 64 + 1) <= 65535, NATSL_ERR_TOO_LARGE,
                  "natsl_gdn_fwd_noalloc: grid too large (B=%d H=%d)", B, H);
    const size_t NT = (size_t)(T + 63) / 64;
    const size_t n_tok = (size_t)B * T * H;
    const size_t sz_w = align256(n_tok * K * 2), sz_u = align256(n_tok * V * 2), sz_f = align256(n_tok * 4);
    const size_t sz_h = align256((size_t)B * NT * H * K * V * 2), sz_c = align256((size_t)B * NT * H * 4);
    const size_t need = sz_w + sz_u + 2 * sz_f + sz_h + sz_c;
    NATSL_REQUIRE(need <= (size_t)NATSL_NOALLOC_SCRATCH_BYTES, NATSL_ERR_TOO_LARGE,
                  "natsl_gdn_fwd_noalloc: B=%d T=%d H=%d K=%d V=%d needs %zu bytes of intermediates, the built-in "
                  "scratch holds %zu; use the regular entry points with caller-provided buffers",
                  B, T, H, K, V, need, (size_t)NATSL_NOALLOC_SCRATCH_BYTES);
    unsigned char* base = nullptr;
    int rc = scratch_for_current_device(&base);
    if (rc != NATSL_OK) return rc;
    unsigned char* p = base;
    void* w = p; p += sz_w;
    void* u = p; p += sz_u;
    float* gcs = reinterpret_cast<float*>(p); p += sz_f;
    float* krstd = reinterpret_cast<float*>(p); p += sz_f;
    void* h = p; p += sz_h;
    float* carry = reinterpret_cast<float*>(p);
    rc = natsl_gdn_chunk_prep(k, v, g, beta, beta_dtype, w, u, gcs, krstd, B, T, H, K, V, use_l2norm, stream);
    if (rc != NATSL_OK) return rc;
    rc = natsl_linear_fwd_h(NATSL_RULE_GDN, k, w, u, gcs, krstd, types_i, indices, n_blocks, h0, h, carry, ht, B, T, H,
                            HN, K, V, nbs, flags, stream);
    if (rc != NATSL_OK) return rc;
    return natsl_linear_fwd_o(NATSL_RULE_GDN, q, k, w, u, gcs, krstd, h, carry, o, B, T, H, K, V, scale, use_l2norm ? 1 : 0,
                              stream);
}
