// Host side of the tensor-core kernels' shared plumbing: the per-device status word that bounded
// waits write when they give up, and TMA tensor-map encoding through the driver entry point
// (resolved at run time, so the library does not link against libcuda).
#include <mutex>

#include "tc_common.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

static __device__ int g_status_word = 0;

constexpr int kMaxDev = 64;
static std::mutex g_mu;
static int* g_status_addr[kMaxDev] = {nullptr};

int status_word_ptr(int** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDev) {
        set_error("cannot identify the current device (%s)", cudaGetErrorString(e));
        return NATSL_ERR_CUDA;
    }
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_status_addr[dev]) {
        int* p = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_status_word);
        if (e != cudaSuccess || !p) {
            set_error("cudaGetSymbolAddress(status word) failed on device %d (%s)", dev, cudaGetErrorString(e));
            return NATSL_ERR_CUDA;
        }
        g_status_addr[dev] = p;
    }
    *out = g_status_addr[dev];
    return NATSL_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

int encode_bthd_map(CUtensorMap* out, const void* base, int B, int T, int H, int D, int box_rows, const char* who) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) {
        set_error("%s: the driver does not provide cuTensorMapEncodeTiled", who);
        return NATSL_ERR_CUDA;
    }
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || D % 64 != 0) {
        set_error("%s: TMA needs a 16-byte aligned base and a head dim multiple of 64 (D=%d)", who, D);
        return NATSL_ERR_UNSUPPORTED;
    }
    cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)T, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)H * D * 2, (cuuint64_t)T * H * D * 2};
    cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("%s: cuTensorMapEncodeTiled failed (%d) for [B=%d,T=%d,H=%d,D=%d]", who, (int)r, B, T, H, D);
        return NATSL_ERR_CUDA;
    }
    return NATSL_OK;
}

// Self-test of the bounded-wait path: one warp waits on an mbarrier that nobody arrives at, with the same wait loop
// the tensor-core kernels use but a caller-given (short) poll limit.  The wait runs out, the status word is set and
// the kernel returns normally: the context stays usable.
__global__ void bounded_wait_selftest_kernel(int polls, int* status) {
    __shared__ __align__(8) unsigned long long bar;
    const uint32_t b = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(b, 1);
        mbar_fence_init();
    }
    __syncthreads();
    bool ok = false;
    for (int i = 0; i < polls && !ok; ++i) ok = mbar_try_wait(b, 0);
    if (!ok && threadIdx.x == 0) atomicExch(status, NATSL_DEV_WAIT_TIMEOUT);
}

}  // namespace natsl

extern "C" int natsl_bounded_wait_selftest(int polls, void* stream) {
    using namespace natsl;
    NATSL_REQUIRE(polls > 0 && polls <= (1 << 20), NATSL_ERR_BAD_SHAPE, "natsl_bounded_wait_selftest: 1 <= polls <= 2^20");
    int* status = nullptr;
    int rc = status_word_ptr(&status);
    if (rc != NATSL_OK) return rc;
    bounded_wait_selftest_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(polls, status);
    return check_launch("natsl_bounded_wait_selftest");
}

extern "C" int natsl_device_status(void) {
    using namespace natsl;
    int* p = nullptr;
    int rc = status_word_ptr(&p);
    if (rc != NATSL_OK) return rc;
    int v = 0;
    cudaError_t e = cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);     // synchronises the device
    if (e != cudaSuccess) {
        set_error("natsl_device_status: %s", cudaGetErrorString(e));
        return NATSL_ERR_CUDA;
    }
    if (v != 0) {
        cudaMemset(p, 0, sizeof(int));
        set_error(v == NATSL_DEV_CAPACITY
                      ? "a caller-given capacity was too small (device status %d); the outputs are invalid"
                      : "a kernel gave up a bounded wait (device status %d); its outputs are invalid", v);
    }
    return v;
}
