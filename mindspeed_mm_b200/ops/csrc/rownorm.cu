// Row normalisations of SHORT rows (8 .. 256 elements: per-head q/k RMSNorm, the L2 norm of gated-delta-net heads, small
// LayerNorms), forward: RMSNorm, LayerNorm-modulate (adaLN / affine LayerNorm) and L2 norm.
//
// A thread block per row wastes most of its lanes on such rows.  Here G lanes (4..32, a power of two) own a row: one
// 16-byte vector each, a shuffle reduction inside the group (no shared memory, no block barrier), the result written
// from registers.  A 256-thread block carries 256 / G rows at once and every warp proceeds on its own.  Measured on
// 65536 x 32 rows of 128: 0.94 of the copy bandwidth against 0.45 for the block-per-row kernel.  Longer rows stay with
// the block-per-row kernels of elementwise.cu: the same scheme with NV vectors per lane measured slower there (0.45
// against 0.67 of the copy bandwidth at 3584 elements), so only NV = 1 is instantiated.
#include "common.cuh"

namespace {

constexpr int kBlock = 256;

enum : int { kRms = 0, kLnMod = 1, kL2 = 2 };

template <int G>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// a: RMS weight [H] | LN scale [B, H] | unused.   b: LN shift [B, H].   s0: rstd | mean | 1/norm.   s1: LN rstd.
template <int G, int NV, int MODE>
__global__ void __launch_bounds__(kBlock) rownorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ a,
                                                            const bf16* __restrict__ b, bf16* __restrict__ y,
                                                            float* __restrict__ s0, float* __restrict__ s1,
                                                            long long rows, int S, int H, float eps) {
    constexpr int kRowsPerBlock = kBlock / G;
    const int nvec = H >> 3;
    const int gl = threadIdx.x % G;                     // lane inside the group
    const long long first = (long long)blockIdx.x * kRowsPerBlock + threadIdx.x / G;
    const long long step = (long long)gridDim.x * kRowsPerBlock;
    // every lane of a warp runs the same number of iterations (the shuffles need all 32 lanes): rows past the end are
    // computed on nothing and write nothing
    const long long iters = (rows + step - 1) / step;
    long long row = first;
    for (long long it = 0; it < iters; ++it, row += step) {
        const bool live = row < rows;
        const Vec8* xr = reinterpret_cast<const Vec8*>(x + (size_t)(live ? row : 0) * H);
        Vec8 cache[NV];
        float s = 0.f, ss = 0.f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int i = gl + j * G;
            if (live && i < nvec) {
                cache[j] = xr[i];
                float f[8];
                unpack8(cache[j], f);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    if (MODE == kLnMod) s += f[k];
                    ss += f[k] * f[k];
                }
            }
        }
        ss = group_sum<G>(ss);
        float mean = 0.f, r;
        if (MODE == kLnMod) {
            s = group_sum<G>(s);
            mean = s / (float)H;
            r = rsqrtf(fmaxf(ss / (float)H - mean * mean, 0.f) + eps);
        } else if (MODE == kRms) {
            r = rsqrtf(ss / (float)H + eps);
        } else {
            r = rsqrtf(ss + eps);
        }
        if (!live) continue;
        if (gl == 0) {
            if (MODE == kLnMod) {
                s0[row] = mean;
                s1[row] = r;
            } else if (s0) {
                s0[row] = r;
            }
        }
        const size_t wrow = MODE == kLnMod ? (size_t)(row / S) * H : 0;
        const Vec8* ar = reinterpret_cast<const Vec8*>(a + wrow);
        const Vec8* br = reinterpret_cast<const Vec8*>(b + wrow);
        Vec8* yr = reinterpret_cast<Vec8*>(y + (size_t)row * H);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int i = gl + j * G;
            if (i < nvec) {
                float f[8], o[8];
                unpack8(cache[j], f);
                if (MODE == kRms) {
                    float w[8];
                    unpack8(ar[i], w);
#pragma unroll
                    for (int k = 0; k < 8; ++k) o[k] = f[k] * r * w[k];
                } else if (MODE == kLnMod) {
                    float sc[8], sh[8];
                    unpack8(ar[i], sc);
                    unpack8(br[i], sh);
#pragma unroll
                    for (int k = 0; k < 8; ++k) o[k] = (f[k] - mean) * r * (1.f + sc[k]) + sh[k];
                } else {
#pragma unroll
                    for (int k = 0; k < 8; ++k) o[k] = f[k] * r;
                }
                yr[i] = pack8(o);
            }
        }
    }
}

template <int G, int NV, int MODE>
int launch_one(const void* x, const void* a, const void* b, void* y, float* s0, float* s1, long long rows, int S, int H,
               float eps, cudaStream_t st) {
    static int per_sm = 0;                              // resident blocks per SM of this instantiation
    if (per_sm == 0) {
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, rownorm_fwd_kernel<G, NV, MODE>, kBlock, 0);
        if (per_sm < 1) per_sm = 1;
    }
    constexpr int kRowsPerBlock = kBlock / G;
    long long need = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
    long long cap = 148LL * per_sm;
    const int grid = (int)(need < cap ? need : cap);
    if (grid == 0) return 0;
    rownorm_fwd_kernel<G, NV, MODE><<<grid, kBlock, 0, st>>>((const bf16*)x, (const bf16*)a, (const bf16*)b, (bf16*)y, s0, s1,
                                                             rows, S, H, eps);
    return (int)cudaGetLastError();
}

template <int MODE>
int launch(const void* x, const void* a, const void* b, void* y, float* s0, float* s1, long long rows, int S, int H,
           float eps, cudaStream_t st) {
    if (H % 8 || H < 8 || H > 256) return -1;
    const int nvec = H / 8;
#define MM_RN(G, NV) return launch_one<G, NV, MODE>(x, a, b, y, s0, s1, rows, S, H, eps, st)
    if (nvec <= 4) MM_RN(4, 1);
    if (nvec <= 8) MM_RN(8, 1);
    if (nvec <= 16) MM_RN(16, 1);
    MM_RN(32, 1);
#undef MM_RN
}

// ------------------------------------------------------------------------------------------ gated RMSNorm
// y = x * rsqrt(mean(x^2) + eps) * w * silu(z): the output norm of a gated-delta-net head (rows of 8 .. 256 elements).
// x is the delta rule's output, fp32 or bf16 (XF32); z, w, y, dy, dz are bf16; dx has x's type.  Same lane-group scheme
// as above.  Backward: with n = x * rstd, s = silu(z), u = n * w:  dz = dy * u * s',  du = dy * s,
// dx = rstd * (du * w - n * mean(du * w * n)),  dw += du * n summed over rows (per-lane partials, folded through shared
// memory into one fp32 atomic per column and block).
template <bool XF32>
__device__ __forceinline__ void load8(const void* base, size_t vec, float* f) {
    if (XF32) {
        const float4* p = reinterpret_cast<const float4*>(base) + 2 * vec;
        const float4 a = p[0], b = p[1];
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
        unpack8(reinterpret_cast<const Vec8*>(base)[vec], f);
    }
}
template <bool XF32>
__device__ __forceinline__ void store8(void* base, size_t vec, const float* f) {
    if (XF32) {
        float4* p = reinterpret_cast<float4*>(base) + 2 * vec;
        p[0] = make_float4(f[0], f[1], f[2], f[3]);
        p[1] = make_float4(f[4], f[5], f[6], f[7]);
    } else {
        reinterpret_cast<Vec8*>(base)[vec] = pack8(f);
    }
}

template <int G, bool XF32>
__global__ void __launch_bounds__(kBlock) gated_rms_fwd_kernel(const void* __restrict__ x, const bf16* __restrict__ z,
                                                              const bf16* __restrict__ w, bf16* __restrict__ y,
                                                              float* __restrict__ rstd_out, long long rows, int H, float eps) {
    constexpr int kRowsPerBlock = kBlock / G;
    const int nvec = H >> 3;
    const int gl = threadIdx.x % G;
    const long long step = (long long)gridDim.x * kRowsPerBlock;
    const long long iters = (rows + step - 1) / step;
    long long row = (long long)blockIdx.x * kRowsPerBlock + threadIdx.x / G;
    float wv[8];
    if (gl < nvec) unpack8(reinterpret_cast<const Vec8*>(w)[gl], wv);
    for (long long it = 0; it < iters; ++it, row += step) {
        const bool live = row < rows && gl < nvec;
        float f[8];
        float ss = 0.f;
        if (live) {
            load8<XF32>(x, (size_t)row * nvec + gl, f);
#pragma unroll
            for (int k = 0; k < 8; ++k) ss += f[k] * f[k];
        }
        ss = group_sum<G>(ss);
        if (!live) continue;
        const float r = rsqrtf(ss / (float)H + eps);
        if (gl == 0 && rstd_out) rstd_out[row] = r;
        float zz[8], o[8];
        unpack8(reinterpret_cast<const Vec8*>(z + (size_t)row * H)[gl], zz);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = f[k] * r * wv[k] * zz[k] / (1.f + __expf(-zz[k]));
        reinterpret_cast<Vec8*>(y + (size_t)row * H)[gl] = pack8(o);
    }
}

template <int G, bool XF32>
__global__ void __launch_bounds__(kBlock) gated_rms_bwd_kernel(const void* __restrict__ x, const bf16* __restrict__ z,
                                                              const bf16* __restrict__ w, const bf16* __restrict__ dy,
                                                              const float* __restrict__ rstd_in, void* __restrict__ dx,
                                                              bf16* __restrict__ dz, float* __restrict__ dw, long long rows,
                                                              int H) {
    constexpr int kRowsPerBlock = kBlock / G;
    __shared__ float sdw[256];
    const int nvec = H >> 3;
    const int gl = threadIdx.x % G;
    const long long step = (long long)gridDim.x * kRowsPerBlock;
    const long long iters = (rows + step - 1) / step;
    long long row = (long long)blockIdx.x * kRowsPerBlock + threadIdx.x / G;
    for (int i = threadIdx.x; i < 256; i += kBlock) sdw[i] = 0.f;
    __syncthreads();
    float wv[8], dwacc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) dwacc[k] = 0.f;
    if (gl < nvec) unpack8(reinterpret_cast<const Vec8*>(w)[gl], wv);
    for (long long it = 0; it < iters; ++it, row += step) {
        const bool live = row < rows && gl < nvec;
        float n[8], dn[8], g[8], zz[8];
        float dot = 0.f, r = 0.f;
        if (live) {
            r = rstd_in[row];
            load8<XF32>(x, (size_t)row * nvec + gl, n);
            unpack8(reinterpret_cast<const Vec8*>(dy + (size_t)row * H)[gl], g);
            unpack8(reinterpret_cast<const Vec8*>(z + (size_t)row * H)[gl], zz);
            float dzv[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                n[k] *= r;
                const float sg = 1.f / (1.f + __expf(-zz[k]));
                const float s = zz[k] * sg;
                dzv[k] = g[k] * n[k] * wv[k] * sg * (1.f + zz[k] * (1.f - sg));
                const float du = g[k] * s;
                dwacc[k] += du * n[k];
                dn[k] = du * wv[k];
                dot += dn[k] * n[k];
            }
            reinterpret_cast<Vec8*>(dz + (size_t)row * H)[gl] = pack8(dzv);
        }
        dot = group_sum<G>(dot) / (float)H;
        if (!live) continue;
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = r * (dn[k] - n[k] * dot);
        store8<XF32>(dx, (size_t)row * nvec + gl, o);
    }
    if (gl < nvec)
#pragma unroll
        for (int k = 0; k < 8; ++k) atomicAdd(&sdw[gl * 8 + k], dwacc[k]);
    __syncthreads();
    for (int i = threadIdx.x; i < H; i += kBlock) atomicAdd(&dw[i], sdw[i]);
}

template <bool XF32>
int gated_launch(bool bwd, const void* x, const void* z, const void* w, void* y_or_dy, float* rstd, void* dx, void* dz,
                 float* dw, long long rows, int H, float eps, cudaStream_t st) {
    if (H % 8 || H < 8 || H > 256) return -1;
    const int nvec = H / 8;
#define MM_GR(G)                                                                                                           \
    {                                                                                                                      \
        const long long need = (rows + kBlock / G - 1) / (kBlock / G);                                                     \
        const int grid = (int)(need < 148 * 8 ? need : 148 * 8);                                                           \
        if (grid == 0) return 0;                                                                                           \
        if (!bwd)                                                                                                          \
            gated_rms_fwd_kernel<G, XF32><<<grid, kBlock, 0, st>>>(x, (const bf16*)z, (const bf16*)w, (bf16*)y_or_dy, rstd, \
                                                                  rows, H, eps);                                           \
        else                                                                                                               \
            gated_rms_bwd_kernel<G, XF32><<<grid, kBlock, 0, st>>>(x, (const bf16*)z, (const bf16*)w,                       \
                                                                  (const bf16*)y_or_dy, rstd, dx, (bf16*)dz, dw, rows, H); \
        return (int)cudaGetLastError();                                                                                    \
    }
    if (nvec <= 4) MM_GR(4)
    if (nvec <= 8) MM_GR(8)
    if (nvec <= 16) MM_GR(16)
    MM_GR(32)
#undef MM_GR
}

}  // namespace

// y = rmsnorm(x) * w * silu(z).  x fp32 (x_f32 = 1) or bf16; rstd [rows] fp32 (optional in the forward).
MM_API int mm_gated_rms_fwd(const void* x, int x_f32, const void* z, const void* w, void* y, float* rstd, long long rows,
                            int H, float eps, cudaStream_t st) {
    return x_f32 ? gated_launch<true>(false, x, z, w, y, rstd, nullptr, nullptr, nullptr, rows, H, eps, st)
                 : gated_launch<false>(false, x, z, w, y, rstd, nullptr, nullptr, nullptr, rows, H, eps, st);
}

// dx (x's type), dz (bf16), dw (fp32 [H], zeroed by the caller; accumulated with atomics).
MM_API int mm_gated_rms_bwd(const void* x, int x_f32, const void* z, const void* w, const void* dy, const float* rstd,
                            void* dx, void* dz, float* dw, long long rows, int H, cudaStream_t st) {
    return x_f32 ? gated_launch<true>(true, x, z, w, const_cast<void*>(dy), const_cast<float*>(rstd), dx, dz, dw, rows, H, 0.f, st)
                 : gated_launch<false>(true, x, z, w, const_cast<void*>(dy), const_cast<float*>(rstd), dx, dz, dw, rows, H, 0.f, st);
}

// y = x * rsqrt(mean(x^2) + eps) * w;  rstd (optional) [rows] keeps the factor for the backward.
MM_API int mm_rownorm_rms_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int H, float eps,
                              cudaStream_t st) {
    return launch<kRms>(x, w, nullptr, y, rstd, nullptr, rows, 1, H, eps, st);
}

// y = LN(x) * (1 + scale[row / S]) + shift[row / S];  mean, rstd [rows].
MM_API int mm_rownorm_ln_mod_fwd(const void* x, const void* scale, const void* shift, void* y, float* mean, float* rstd,
                                 long long rows, int S, int H, float eps, cudaStream_t st) {
    return launch<kLnMod>(x, scale, shift, y, mean, rstd, rows, S, H, eps, st);
}

// y = x * rsqrt(sum(x^2) + eps);  rnorm (optional) [rows].
MM_API int mm_rownorm_l2_fwd(const void* x, void* y, float* rnorm, long long rows, int H, float eps, cudaStream_t st) {
    return launch<kL2>(x, nullptr, nullptr, y, rnorm, nullptr, rows, 1, H, eps, st);
}
