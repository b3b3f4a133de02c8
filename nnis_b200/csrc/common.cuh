// Shared helpers of the sm_100a kernels: element types, loads that widen to
// float, stores that round once, warp reductions, and the status codes that
// the C entry points return.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define NNIS_OK 0
// Negative codes are argument errors found on the host before any launch;
// positive codes are cudaError_t values of the launch itself.
#define NNIS_ERR_ARGUMENT (-1)
#define NNIS_ERR_UNSUPPORTED (-2)
#define NNIS_ERR_ALIGNMENT (-3)
#define NNIS_ERR_DEVICE_STATUS (-4)

#define NNIS_DTYPE_F32 0
#define NNIS_DTYPE_BF16 1

#define NNIS_API extern "C" __attribute__((visibility("default")))

#define NNIS_RETURN_LAUNCH() \
    do { cudaError_t e__ = cudaGetLastError(); return e__ == cudaSuccess ? NNIS_OK : (int)e__; } while (0)

namespace nnis {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(bf16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float x) { return __float2bfloat16_rn(x); }

// Four consecutive elements widened to float; the address must be aligned to
// four elements (16 bytes for float, 8 for bfloat16).
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    uint2 raw = *reinterpret_cast<const uint2*>(p);
    float4 r;
    r.x = __uint_as_float(raw.x << 16);
    r.y = __uint_as_float(raw.x & 0xffff0000u);
    r.z = __uint_as_float(raw.y << 16);
    r.w = __uint_as_float(raw.y & 0xffff0000u);
    return r;
}

// Two consecutive elements widened to float; the address must be aligned to two
// elements (8 bytes for float, 4 for bfloat16).
__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load2(const bf16* p) {
    uint32_t raw = *reinterpret_cast<const uint32_t*>(p);
    return make_float2(__uint_as_float(raw << 16), __uint_as_float(raw & 0xffff0000u));
}

__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y);
    __nv_bfloat162 hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&lo);
    raw.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// The sum over each half of a warp (lanes 0-15, 16-31); every lane calls it.
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// The timeline of a step (trace.cu): the next slot of the trace buffer for a launch
// of the named kernel, or null when no trace is being taken.
unsigned long long* trace_slot(const char* name);

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// the same from a thread that the caller picks (one per CTA)
__device__ __forceinline__ void trace_mark_here(unsigned long long* slot, int word) {
    if (slot) {
        if (word & 1) atomicMax(slot + word, global_ns());
        else atomicMin(slot + word, global_ns());
    }
}

// even words: the earliest CTA; odd words: the latest
__device__ __forceinline__ void trace_mark(unsigned long long* slot, int word) {
    if (slot && threadIdx.x == 0) {
        if (word & 1) atomicMax(slot + word, global_ns());
        else atomicMin(slot + word, global_ns());
    }
}

}  // namespace nnis
