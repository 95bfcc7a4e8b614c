// Shared helpers for the sm_100a kernels and the C-ABI layer: error capture,
// cache-hinted loads/stores, small device utilities.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/ra_spmm_b200.h"

namespace ra {

using i64 = long long;

// B200: 148 SMs. Grids of persistent kernels are sized from the device
// attribute at run time; this constant only seeds defaults.
constexpr int kDefaultSMs = 148;

// ---- thread-local error text --------------------------------------------
void set_error(const char* fmt, ...);
const char* get_error();
int sm_count();   // cached cudaDevAttrMultiProcessorCount of the current device

#define RA_CUDA_TRY(expr)                                                     \
    do {                                                                      \
        cudaError_t _e = (expr);                                              \
        if (_e != cudaSuccess) {                                              \
            ::ra::set_error("%s failed at %s:%d: %s", #expr, __FILE__,        \
                            __LINE__, cudaGetErrorString(_e));                \
            return RA_ERR_CUDA;                                               \
        }                                                                     \
    } while (0)

#define RA_KERNEL_CHECK()                                                     \
    do {                                                                      \
        cudaError_t _e = cudaGetLastError();                                  \
        if (_e != cudaSuccess) {                                              \
            ::ra::set_error("kernel launch failed at %s:%d: %s", __FILE__,    \
                            __LINE__, cudaGetErrorString(_e));                \
            return RA_ERR_CUDA;                                               \
        }                                                                     \
    } while (0)

#define RA_REQUIRE(cond, code, ...)                                           \
    do {                                                                      \
        if (!(cond)) {                                                        \
            ::ra::set_error(__VA_ARGS__);                                     \
            return (code);                                                    \
        }                                                                     \
    } while (0)

// Function attributes (dynamic shared-memory limit, carve-out) belong to a (kernel, device)
// pair, so a launcher keeps one bit per device ordinal and configures the kernel the first
// time it runs on each device. Two host threads may both configure (the calls are
// idempotent); neither can launch before its own configure call returned.
template <typename F>
inline cudaError_t configure_once_per_device(std::atomic<unsigned long long>& done, F&& configure) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const unsigned long long bit = (dev >= 0 && dev < 64) ? (1ull << dev) : 0ull;   // ordinals >= 64: always configure
    if (bit && (done.load(std::memory_order_acquire) & bit)) return cudaSuccess;
    e = configure();
    if (e != cudaSuccess) return e;
    if (bit) done.fetch_or(bit, std::memory_order_release);
    return cudaSuccess;
}

inline bool aligned16(const void* p) {
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0u;
}

// ---- device helpers -------------------------------------------------------
#ifdef __CUDACC__

// Streaming (read-once) 128-bit load: col/val streams must not displace the
// dense B rows that the gathers want to keep in L1/L2.
__device__ __forceinline__ int4 ld_stream_int4(const int4* p) { return __ldcs(p); }
__device__ __forceinline__ int ld_stream_int(const int* p) { return __ldcs(p); }
__device__ __forceinline__ float ld_stream_float(const float* p) { return __ldcs(p); }
// Gather load of a dense-B fragment: read-only path, default (keep) policy.
__device__ __forceinline__ float4 ld_gather_float4(const float4* p) { return __ldg(p); }
// Write-once output: streaming store so C does not evict B from L2.
__device__ __forceinline__ void st_stream_float4(float4* p, const float4& v) {
    asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};"
                 :: "l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void st_stream_float(float* p, float v) {
    asm volatile("st.global.cs.f32 [%0], %1;" :: "l"(p), "f"(v) : "memory");
}

// acc += a * b on four lanes of a float4. sm_100 has a packed two-wide fp32 FMA
// (same rounding as two scalar FMAs), which halves the issue slots of the
// multiply-accumulate stream.
__device__ __forceinline__ void fma4(float4& acc, float a, const float4& b) {
#if defined(__CUDA_ARCH__) && __CUDA_ARCH__ >= 1000
    const float2 aa = make_float2(a, a);
    const float2 lo = __ffma2_rn(aa, make_float2(b.x, b.y), make_float2(acc.x, acc.y));
    const float2 hi = __ffma2_rn(aa, make_float2(b.z, b.w), make_float2(acc.z, acc.w));
    acc.x = lo.x; acc.y = lo.y; acc.z = hi.x; acc.w = hi.y;
#else
    acc.x = fmaf(a, b.x, acc.x);
    acc.y = fmaf(a, b.y, acc.y);
    acc.z = fmaf(a, b.z, acc.z);
    acc.w = fmaf(a, b.w, acc.w);
#endif
}

#endif  // __CUDACC__

}  // namespace ra
