// Shared device helpers for the sm_100a kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

#define MM_API extern "C" __attribute__((visibility("default")))

// Status word written by kernels whose bounded waits ran out (read by the host; never traps).
enum MmStatus : int { MM_OK = 0, MM_TIMEOUT_TMA = 1, MM_TIMEOUT_MMA = 2, MM_TIMEOUT_EPI = 3, MM_TIMEOUT_PEER = 4 };

struct alignas(16) Vec8 {
    bf162 v[4];
};

__device__ __forceinline__ void unpack8(const Vec8& p, float* f) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __bfloat1622float2(p.v[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

__device__ __forceinline__ Vec8 pack8(const float* f) {
    Vec8 p;
#pragma unroll
    for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return p;
}

// Streaming accesses for kernels that run beside a GEMM (optimizer update, gradient reduction): their data is touched
// once, so it is marked evict-first in L2 and bypasses L1; the GEMM's operand tiles, which many CTAs re-read from L2, stay.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ float4 ld_stream_f4(const float4* p, uint64_t pol) {
    float4 v;
    asm volatile("ld.global.L1::no_allocate.L2::cache_hint.v4.f32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p), "l"(pol));
    return v;
}
__device__ __forceinline__ void st_stream_f4(float4* p, const float4& v, uint64_t pol) {
    asm volatile("st.global.L2::cache_hint.v4.f32 [%0], {%1,%2,%3,%4}, %5;" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z),
                 "f"(v.w), "l"(pol)
                 : "memory");
}
__device__ __forceinline__ uint4 ld_stream_u4(const uint4* p, uint64_t pol) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p), "l"(pol));
    return v;
}
__device__ __forceinline__ uint2 ld_stream_u2(const uint2* p, uint64_t pol) {
    uint2 v;
    asm volatile("ld.global.L1::no_allocate.L2::cache_hint.v2.u32 {%0,%1}, [%2], %3;" : "=r"(v.x), "=r"(v.y) : "l"(p), "l"(pol));
    return v;
}

// 32-byte global accesses (sm_100: ld / st .v8.b32): 16 bf16 per instruction, half the load-store instructions of the
// 16-byte form for the same bytes.  Addresses must be 32-byte aligned.
struct Vec16 {
    uint32_t r[8];
};
__device__ __forceinline__ Vec16 ld_v16(const void* p) {
    Vec16 v;
    asm volatile("ld.global.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v.r[0]), "=r"(v.r[1]), "=r"(v.r[2]), "=r"(v.r[3]), "=r"(v.r[4]), "=r"(v.r[5]), "=r"(v.r[6]), "=r"(v.r[7])
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void st_v16(void* p, const Vec16& v) {
    asm volatile("st.global.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v.r[0]), "r"(v.r[1]), "r"(v.r[2]), "r"(v.r[3]),
                 "r"(v.r[4]), "r"(v.r[5]), "r"(v.r[6]), "r"(v.r[7])
                 : "memory");
}
__device__ __forceinline__ void unpack16(const Vec16& v, float* f) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.r[i]));
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ Vec16 pack16(const float* f) {
    Vec16 v;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        v.r[i] = *reinterpret_cast<uint32_t*>(&t);
    }
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over the whole block; every thread gets the result.  `red` holds >= 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__device__ __forceinline__ void block_sum2(float& a, float& b, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    a = warp_sum(a);
    b = warp_sum(b);
    __syncthreads();
    if (lane == 0) {
        red[wid] = a;
        red[34 + wid] = b;
    }
    __syncthreads();
    if (wid == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        float u = lane < nw ? red[34 + lane] : 0.f;
        t = warp_sum(t);
        u = warp_sum(u);
        if (lane == 0) {
            red[32] = t;
            red[33] = u;
        }
    }
    __syncthreads();
    a = red[32];
    b = red[33];
}
