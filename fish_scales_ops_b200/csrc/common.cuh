// Shared host-side helpers of the library: error reporting, argument checks, per-device facts.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/fso_b200.h"

namespace fso {

// Thread-local text of the last failure on this host thread.
void set_error(const char* fmt, ...);

// Device-side status word (one per device; the library is a single translation unit, so this is the only copy).
// 0 = fine; otherwise the code of the first bounded wait that ran out inside a kernel (FSO_DEV_* below).
static __device__ int g_dev_status = 0;

constexpr int FSO_DEV_WAIT_PRODUCER = 0x100;   // TMA producer waited for a free stage
constexpr int FSO_DEV_WAIT_MMA_FULL = 0x200;   // MMA issuer waited for a filled stage
constexpr int FSO_DEV_WAIT_MMA_TMEM = 0x300;   // MMA issuer waited for a drained accumulator
constexpr int FSO_DEV_WAIT_EPILOGUE = 0x400;   // epilogue waited for a finished accumulator
constexpr int FSO_DEV_SELFTEST_WAIT = 0x700;   // the self-test's wait on a barrier nothing arrives at ran out

int sm_count();                                 // SMs of the current device (cached per device)
int current_device();

#define FSO_REQUIRE(cond, ...)                                                                                      \
    do {                                                                                                            \
        if (!(cond)) {                                                                                              \
            ::fso::set_error(__VA_ARGS__);                                                                          \
            return FSO_ERR_INVALID;                                                                                 \
        }                                                                                                           \
    } while (0)

#define FSO_CUDA(expr)                                                                                              \
    do {                                                                                                            \
        cudaError_t e__ = (expr);                                                                                   \
        if (e__ != cudaSuccess) {                                                                                   \
            ::fso::set_error("%s failed: %s", #expr, cudaGetErrorString(e__));                                      \
            (void)cudaGetLastError(); /* the failure is reported here: later calls must not see it again */        \
            return static_cast<int>(e__);                                                                           \
        }                                                                                                           \
    } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Result of the launches just made. cudaGetLastError() also clears the error, so that a failed launch is reported by
// the call that caused it and by no later one.
inline int launch_status(const char* what)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: launch failed: %s", what, cudaGetErrorString(e));
        return static_cast<int>(e);
    }
    return 0;
}

}  // namespace fso
