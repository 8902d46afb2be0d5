// Shared device helpers for the NAtSL sm_100a kernels: cp.async staging, swizzled
// shared-memory tiles, ldmatrix / mma.sync fragments, small numeric helpers, and
// the host-side error plumbing of the C-ABI.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define NATSL_CHUNK 64

namespace natsl {

// ------------------------------------------------------------------ host-side errors
void set_error(const char* fmt, ...);
int check_launch(const char* what);

#define NATSL_REQUIRE(cond, code, ...)          \
    do {                                        \
        if (!(cond)) {                          \
            ::natsl::set_error(__VA_ARGS__);    \
            return (code);                      \
        }                                       \
    } while (0)

enum : int {
    NATSL_OK = 0,
    NATSL_ERR_BAD_SHAPE = -1,
    NATSL_ERR_UNSUPPORTED = -2,
    NATSL_ERR_NULL = -3,
    NATSL_ERR_CUDA = -4,
    NATSL_ERR_TOO_LARGE = -5,
};

// ------------------------------------------------------------------ device helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte async copy global -> shared; bytes beyond src_bytes (0 or 16) are zero-filled.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a swizzled tile whose rows are
// ROW_BYTES long (64, 128 or 256).  The XOR keeps the eight rows touched by one
// ldmatrix 8x8 load in eight different 16-byte bank groups.
template <int ROW_BYTES>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    static_assert(ROW_BYTES == 64 || ROW_BYTES == 128 || ROW_BYTES == 256 || ROW_BYTES == 512, "row size");
    if (ROW_BYTES == 64) return row * 64 + ((chunk ^ ((row >> 1) & 3)) << 4);
    return row * ROW_BYTES + ((chunk ^ (row & 7)) << 4);
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t u) {
    __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
    return __bfloat1622float2(v);
}

// ---- fragment loaders over swizzled bf16 tiles ------------------------------------
// A fragment (16 rows x 16 k) of a row-major [rows][k] tile.
template <int ROW_BYTES>
__device__ __forceinline__ void load_a(uint32_t tile, int row0, int k0, int lane, uint32_t (&a)[4]) {
    int r = row0 + (lane & 15);
    int c = (k0 >> 3) + (lane >> 4);
    ldsm_x4(tile + swz<ROW_BYTES>(r, c), a[0], a[1], a[2], a[3]);
}
// A fragment (16 m x 16 k) of A = M^T where M is stored row-major [k][m].
template <int ROW_BYTES>
__device__ __forceinline__ void load_a_t(uint32_t tile, int m0, int k0, int lane, uint32_t (&a)[4]) {
    int i = lane >> 3;
    int r = k0 + (lane & 7) + ((i >> 1) << 3);
    int c = (m0 >> 3) + (i & 1);
    ldsm_x4_t(tile + swz<ROW_BYTES>(r, c), a[0], a[1], a[2], a[3]);
}
// B fragments for two adjacent n-tiles (16 n x 16 k) when B^T is stored row-major [n][k]
// (e.g. keys [key][d] for Q K^T): b[0],b[1] -> n-tile n0, b[2],b[3] -> n-tile n0+8.
template <int ROW_BYTES>
__device__ __forceinline__ void load_b_nk(uint32_t tile, int n0, int k0, int lane, uint32_t (&b)[4]) {
    int r = n0 + (lane & 7) + ((lane >> 4) << 3);
    int c = (k0 >> 3) + ((lane >> 3) & 1);
    ldsm_x4(tile + swz<ROW_BYTES>(r, c), b[0], b[1], b[2], b[3]);
}
// B fragments for two adjacent n-tiles when B is stored row-major [k][n]
// (e.g. values [key][dv] for P V): b[0],b[1] -> n-tile n0, b[2],b[3] -> n-tile n0+8.
template <int ROW_BYTES>
__device__ __forceinline__ void load_b_kn(uint32_t tile, int k0, int n0, int lane, uint32_t (&b)[4]) {
    int r = k0 + (lane & 7) + (((lane >> 3) & 1) << 3);
    int c = (n0 >> 3) + (lane >> 4);
    ldsm_x4_t(tile + swz<ROW_BYTES>(r, c), b[0], b[1], b[2], b[3]);
}

// Copy a [ROWS][COLS] bf16 tile from global (row stride `gstride` elements) into a swizzled
// shared tile with cp.async; rows >= valid_rows are zero-filled.  NT = threads taking part.
template <int ROWS, int COLS, int NT>
__device__ __forceinline__ void load_tile_async(uint32_t tile, const __nv_bfloat16* g, long gstride, int valid_rows,
                                                int tid) {
    constexpr int CPR = COLS / 8;  // 16-byte chunks per row
    constexpr int TOTAL = ROWS * CPR;
#pragma unroll
    for (int i = tid; i < TOTAL; i += NT) {
        int r = i / CPR, c = i % CPR;
        bool ok = r < valid_rows;
        const __nv_bfloat16* src = g + (ok ? (long)r * gstride + c * 8 : 0);
        cp_async16(tile + swz<COLS * 2>(r, c), src, ok ? 16 : 0);
    }
}

// Store a swizzled [ROWS][COLS] bf16 shared tile to global with 16-byte coalesced stores.
template <int ROWS, int COLS, int NT>
__device__ __forceinline__ void store_tile(const unsigned char* tile, __nv_bfloat16* g, long gstride, int valid_rows,
                                           int tid) {
    constexpr int CPR = COLS / 8;
    constexpr int TOTAL = ROWS * CPR;
#pragma unroll
    for (int i = tid; i < TOTAL; i += NT) {
        int r = i / CPR, c = i % CPR;
        if (r < valid_rows) {
            uint4 v = *reinterpret_cast<const uint4*>(tile + swz<COLS * 2>(r, c));
            *reinterpret_cast<uint4*>(g + (long)r * gstride + c * 8) = v;
        }
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace natsl
