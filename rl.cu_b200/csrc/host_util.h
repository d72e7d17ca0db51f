// Host-side helpers shared by the translation units of the library: the
// per-thread error message behind rlcu_last_error() and status-returning
// wrappers for CUDA / NCCL calls.  Nothing here exits or throws.
#pragma once

#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include <cstdarg>
#include <cstdio>

#include "rlcu_adamw.h"

namespace rlcu {

inline char* error_buffer() {
    static thread_local char buf[512] = "";
    return buf;
}

inline const char* last_error() { return error_buffer(); }

inline int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

// NVTX range around the host-side enqueue of one phase of the step (header-only NVTX v3:
// nothing is linked, and without a profiler attached a range costs one pointer test).
struct NvtxRange {
    explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
    NvtxRange(const NvtxRange&) = delete;
    NvtxRange& operator=(const NvtxRange&) = delete;
};

}  // namespace rlcu

#define RLCU_CUDA(call)                                                                    \
    do {                                                                                   \
        cudaError_t rlcu_e_ = (call);                                                      \
        if (rlcu_e_ != cudaSuccess)                                                        \
            return ::rlcu::set_error(RLCU_ERR_CUDA, "%s: %s (%s:%d)", #call,               \
                                     cudaGetErrorString(rlcu_e_), __FILE__, __LINE__);     \
    } while (0)
