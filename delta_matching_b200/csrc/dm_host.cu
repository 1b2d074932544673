// Host-side plumbing of libdm_b200: pointer checks, TMA tensor maps, the per-device status word, build identity.
#include <stdarg.h>
#include <atomic>
#include <mutex>

#include "dm_host.h"

namespace dmh {

// Pointers that have been verified once are remembered by the 2 MiB segment of the address space they lie in (with the device
// that owns them): CUDA reserves device address ranges in units of at least that size and never hands parts of them to host
// allocations, so a later pointer in the same segment needs no driver query.  Eight to fourteen queries per entry point were
// most of the host time of the small kernels.  A direct-mapped table of atomics: a stale or colliding entry only costs a query.
static std::atomic<uint64_t> g_seg_cache[512];

static bool seg_cached(const void* p, int dev) {
    const uint64_t seg = reinterpret_cast<uintptr_t>(p) >> 21;
    const uint64_t want = (seg << 8) | (uint64_t)(dev + 1);
    return g_seg_cache[(seg ^ (seg >> 9)) & 511].load(std::memory_order_relaxed) == want;
}
static void seg_remember(const void* p, int dev) {
    const uint64_t seg = reinterpret_cast<uintptr_t>(p) >> 21;
    g_seg_cache[(seg ^ (seg >> 9)) & 511].store((seg << 8) | (uint64_t)(dev + 1), std::memory_order_relaxed);
}

int check_device_ptr(const void* p, const char* name, char* err, size_t errlen) {
    DM_REQUIRE(p != nullptr, DM_ERR_ARG, "%s is NULL", name);
    int dev = -1;
    DM_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 255 && seg_cached(p, dev)) return DM_OK;
    cudaPointerAttributes a;
    cudaError_t e = cudaPointerGetAttributes(&a, p);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(err, errlen, DM_ERR_ARG, "%s is not a CUDA device pointer (%s)", name, cudaGetErrorString(e));
    }
    DM_REQUIRE(a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged, DM_ERR_ARG,
               "%s must be CUDA device memory (got a host pointer)", name);
    DM_REQUIRE(a.type == cudaMemoryTypeManaged || a.device == dev, DM_ERR_ARG,
               "%s lives on device %d but the current device is %d: every tensor must be on the same device", name, a.device, dev);
    if (a.type == cudaMemoryTypeDevice && dev >= 0 && dev < 255) seg_remember(p, dev);
    return DM_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

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

int make_tmap_u8(CUtensorMap* out, const void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_rows, char* err,
                 size_t errlen) {
    EncodeTiledFn fn = encode_fn();
    DM_REQUIRE(fn != nullptr, DM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the CUDA driver");
    DM_REQUIRE(aligned16(base), DM_ERR_ARG, "tensor base %p is not 16-byte aligned", base);
    DM_REQUIRE(row_bytes % 128 == 0 && box_rows >= 1 && box_rows <= 256, DM_ERR_ARG, "bad tensor-map geometry");
    cuuint64_t dims[2] = {row_bytes, rows};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {128, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    DM_REQUIRE(r == CUDA_SUCCESS, DM_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return DM_OK;
}

bool register_pool_ok(int compiled_regs_per_thread, int threads, int regs_needed) {
    return compiled_regs_per_thread > 0 && threads > 0 && (int64_t)compiled_regs_per_thread * threads >= (int64_t)regs_needed;
}

int check_register_pool(const void* kernel, int threads, int regs_needed, char* err, size_t errlen) {
    cudaFuncAttributes a;
    DM_CUDA(cudaFuncGetAttributes(&a, kernel));
    DM_REQUIRE(register_pool_ok(a.numRegs, threads, regs_needed), DM_ERR_UNSUPPORTED,
               "this build of the kernel was compiled with %d registers per thread (%d threads), but its roles request %d in "
               "all: refusing to launch (a setmaxnreg.inc would never be satisfied)", a.numRegs, threads, regs_needed);
    return DM_OK;
}

int sm_count(int* sms, char* err, size_t errlen) {
    static std::mutex mu;
    static int cached[64] = {0};
    int dev = 0;
    DM_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(mu);
    if (dev >= 0 && dev < 64 && cached[dev]) {
        *sms = cached[dev];
        return DM_OK;
    }
    DM_CUDA(cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev));
    if (dev >= 0 && dev < 64) cached[dev] = *sms;
    return DM_OK;
}

static std::mutex g_status_mu;
static int* g_status[64] = {nullptr};

int* device_status_word(char* err, size_t errlen) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        fail(err, errlen, DM_ERR_CUDA, "cudaGetDevice failed");
        return nullptr;
    }
    std::lock_guard<std::mutex> lk(g_status_mu);
    if (!g_status[dev]) {
        int* p = nullptr;
        if (cudaMalloc(&p, sizeof(int)) != cudaSuccess || cudaMemset(p, 0, sizeof(int)) != cudaSuccess) {
            fail(err, errlen, DM_ERR_CUDA, "cannot allocate the device status word");
            return nullptr;
        }
        g_status[dev] = p;
    }
    return g_status[dev];
}

}  // namespace dmh

extern "C" const char* dm_build_info(void) {
    return "libdm_b200 0.1.0; arch=sm_100a; numerics=Delta-Matching-128 v3 / Delta-Matching-256 v1 (tcgen05 realization); "
           "twins=none; bf16_dp=0; dbg=1";
}

extern "C" int dm_register_pool_ok(int32_t compiled_regs_per_thread, int32_t threads, int32_t regs_needed) {
    return dmh::register_pool_ok(compiled_regs_per_thread, threads, regs_needed) ? 1 : 0;
}

extern "C" int dm_init(char* err, size_t errlen) {
    if (!dmh::device_status_word(err, errlen)) return DM_ERR_CUDA;
    int rc, sms = 0;
    if ((rc = dmh::sm_count(&sms, err, errlen))) return rc;
    if ((rc = dmh::prepare_fwd(err, errlen))) return rc;
    if ((rc = dmh::prepare_fwd256(err, errlen))) return rc;
    if ((rc = dmh::prepare_delta(err, errlen))) return rc;
    if ((rc = dmh::prepare_bwd1(err, errlen))) return rc;
    return dmh::prepare_bwd2(err, errlen);
}

extern "C" int dm_device_status(int32_t* status, char* err, size_t errlen) {
    DM_REQUIRE(status != nullptr, DM_ERR_ARG, "status is NULL");
    int* w = dmh::device_status_word(err, errlen);
    if (!w) return DM_ERR_CUDA;
    DM_CUDA(cudaDeviceSynchronize());
    int v = 0;
    DM_CUDA(cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost));
    DM_CUDA(cudaMemset(w, 0, sizeof(int)));
    *status = v;
    return DM_OK;
}
