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

// One int per device, zero-initialised: kernels write a non-zero value when a bounded wait gives up.
int* device_status_word(char* err, size_t errlen);

}  // namespace dmh
