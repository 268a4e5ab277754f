// Shared host/device helpers of libnats_b200 (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/nats_b200.h"

namespace nats {

constexpr int kTile = 128;           // query rows / key columns per MMA tile of the prefill
constexpr int kMaxTiles = 4096;      // prefill: N <= kMaxTiles * kTile
constexpr int32_t kNoLimit = 0x7fffffff;

// ---- host-side error text (thread local) ----------------------------------------------------
char* last_error_buf();
int fail(int code, const char* fmt, ...);

#define NATS_CHECK_ARG(cond, ...)                                   \
    do {                                                            \
        if (!(cond)) return ::nats::fail(NATS_ERR_INVALID_ARG, __VA_ARGS__); \
    } while (0)

#define NATS_CHECK_CUDA(expr)                                                                     \
    do {                                                                                          \
        cudaError_t e_ = (expr);                                                                  \
        if (e_ != cudaSuccess)                                                                    \
            return ::nats::fail(NATS_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_));   \
    } while (0)

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline int cdiv(int a, int b) { return (a + b - 1) / b; }

// ---- device helpers --------------------------------------------------------------------------
__device__ __forceinline__ int warp_incl_scan(int v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
    }
    return v;
}

// 16-byte global accesses
__device__ __forceinline__ uint4 ld16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void st16(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }
// streaming variants: data that is touched once should not displace the L2 working set
__device__ __forceinline__ uint4 ld16_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

}  // namespace nats
