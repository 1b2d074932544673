// Host-side helpers shared by the C-ABI entry points: error reporting, argument checks, TMA tensor-map construction,
// and the per-device status word the kernels' bounded waits report into.
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>
#include <stddef.h>
#include <stdio.h>
#include <stdarg.h>
#include <string.h>
#include <mutex>

#include "../../include/dm_b200.h"

namespace dmh {

inline int fail(char* err, size_t errlen, int code, const char* fmt, ...) __attribute__((format(printf, 4, 5)));
inline int fail(char* err, size_t errlen, int code, const char* fmt, ...) {
    if (err && errlen) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(err, errlen, fmt, ap);
        va_end(ap);
    }
    return code;
}

#define DM_REQUIRE(cond, code, ...)                                   \
    do {                                                              \
        if (!(cond)) return dmh::fail(err, errlen, (code), __VA_ARGS__); \
    } while (0)

#define DM_CUDA(call)                                                                                           \
    do {                                                                                                        \
        cudaError_t e_ = (call);                                                                                \
        if (e_ != cudaSuccess)                                                                                  \
            return dmh::fail(err, errlen, DM_ERR_CUDA, "CUDA error %s at %s:%d", cudaGetErrorString(e_), __FILE__, __LINE__); \
    } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Requires the pointer to be device-accessible memory on the current device (rejects host pointers before any launch).
int check_device_ptr(const void* p, const char* name, char* err, size_t errlen);

// 2-D uint8 tensor map: `rows` rows of `row_bytes` bytes (pitch = row_bytes), boxes of box_rows x 128 bytes, 128-byte swizzle.
int make_tmap_u8(CUtensorMap* out, const void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_rows, char* err, size_t errlen);

// Kernels that move registers between their roles with setmaxnreg only work if the CTA was launched with the pool the
// roles' requests add up to: `threads` x the compiled register count must be at least `regs_needed` (the sum over the
// roles of threads x requested registers), otherwise a setmaxnreg.inc would wait for registers that never come.  Refuses
// with DM_ERR_UNSUPPORTED instead of launching.
int check_register_pool(const void* kernel, int threads, int regs_needed, char* err, size_t errlen);
// The same rule on plain numbers (the part a host test can reach).
bool register_pool_ok(int compiled_regs_per_thread, int threads, int regs_needed);

// Per-device one-time set-up (function attributes, register-pool checks) behind a mutex: `f` runs once per device, with
// that device current, the first time an entry point that needs it is called there (or from dm_init).
struct DeviceOnce {
    std::mutex mu;
    bool done[64] = {};
};
template <class F>
int device_once(DeviceOnce& o, char* err, size_t errlen, F&& f) {
    int dev = 0;
    DM_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(o.mu);
    if (dev >= 0 && dev < 64 && o.done[dev]) return DM_OK;
    if (int rc = f()) return rc;
    if (dev >= 0 && dev < 64) o.done[dev] = true;
    return DM_OK;
}
// Number of SMs of the current device (cached per device).
int sm_count(int* sms, char* err, size_t errlen);

// One-time set-up of each kernel family on the current device (also reached lazily from the entry points).
int prepare_fwd(char* err, size_t errlen);
int prepare_fwd256(char* err, size_t errlen);
int launch_kmean_fold_quant_k(const void* k, DmStrides ks, const float* partials, DmShape s, float* km, void* k8, float* k8s, void* stream,
                              char* err, size_t errlen);
int launch_gqa_fold(const void* x0, void* out0, const void* x1, void* out1, int B, int N, int H, int Hk, int D, void* stream, char* err,
                    size_t errlen);
int prepare_delta(char* err, size_t errlen);
int prepare_bwd1(char* err, size_t errlen);
int prepare_bwd2(char* err, size_t errlen);

// One int per device, zero-initialised: kernels write a non-zero value when a bounded wait gives up.
int* device_status_word(char* err, size_t errlen);

}  // namespace dmh
