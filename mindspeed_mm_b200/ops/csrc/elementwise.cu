// Memory-bound fused ops: RMSNorm (fwd/bwd), SwiGLU (fwd/bwd), RoPE (half-rotation and interleaved,
// fwd/bwd), adaLN LayerNorm-modulate (fwd/bwd), gated residual, sharded AdamW.
//
// All kernels move 16-byte vectors (8 bf16), keep a row in registers between the reduction and the
// write so that every byte crosses HBM once, and size the grid as a multiple of the 148 SMs.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxVec = 4;  // cached 16-byte vectors per thread -> rows up to 256*4*8 = 8192 stay in registers

// ------------------------------------------------------------------------------------------ RMSNorm
// One 128-thread CTA per row at a time (several CTAs per SM keep enough rows in flight to cover HBM
// latency); NV = 16-byte vectors cached per thread, so a row of up to 128*NV*8 elements is read once.
constexpr int kRowThreads = 128;

template <int NV>
__global__ void __launch_bounds__(kRowThreads) rmsnorm_fwd_kernel(const bf16* __restrict__ x,
                                                                   const bf16* __restrict__ w, bf16* __restrict__ y,
                                                                   float* __restrict__ rstd_out, int T, int H,
                                                                   float eps) {
    __shared__ float red[72];
    const int nvec = H >> 3;
    // a thread owns the same columns in every row: its slice of the weight is read once, not once per row (re-reading it
    // made the L1 / load-store path, not HBM, the limit: 92 % L1 throughput at 0.67 of the copy bandwidth)
    Vec8 wc[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        int i = threadIdx.x + j * kRowThreads;
        if (i < nvec) wc[j] = reinterpret_cast<const Vec8*>(w)[i];
    }
    // the next row's loads are issued before this row's reduction, so they are in flight across the block barrier
    Vec8 cache[NV];
    if (blockIdx.x < T) {
        const Vec8* xr = reinterpret_cast<const Vec8*>(x + (size_t)blockIdx.x * H);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            int i = threadIdx.x + j * kRowThreads;
            if (i < nvec) cache[j] = xr[i];
        }
    }
    for (int row = blockIdx.x; row < T; row += gridDim.x) {
        Vec8 nxt[NV];
        const int nrow = row + gridDim.x;
        if (nrow < T) {
            const Vec8* xn = reinterpret_cast<const Vec8*>(x + (size_t)nrow * H);
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                int i = threadIdx.x + j * kRowThreads;
                if (i < nvec) nxt[j] = xn[i];
            }
        }
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            int i = threadIdx.x + j * kRowThreads;
            if (i < nvec) {
                float f[8];
                unpack8(cache[j], f);
#pragma unroll
                for (int k = 0; k < 8; ++k) ss += f[k] * f[k];
            }
        }
        ss = block_sum(ss, red);
        const float rstd = rsqrtf(ss / (float)H + eps);
        if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
        Vec8* yr = reinterpret_cast<Vec8*>(y + (size_t)row * H);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            int i = threadIdx.x + j * kRowThreads;
            if (i < nvec) {
                float f[8], g[8];
                unpack8(cache[j], f);
                unpack8(wc[j], g);
#pragma unroll
                for (int k = 0; k < 8; ++k) f[k] = f[k] * rstd * g[k];
                yr[i] = pack8(f);
            }
        }
#pragma unroll
        for (int j = 0; j < NV; ++j) cache[j] = nxt[j];
    }
}

// The same forward with 32-byte accesses: NV vectors of 16 elements per thread (rows of up to 128 * NV * 16 elements, a
// multiple of 16, 32-byte aligned).  The 16-byte form ran at 87 % L1 / TEX throughput with every access coalesced: the
// load-store path, not DRAM, was its limit; this form issues half as many memory instructions for the same bytes.
template <int NV>
__global__ void __launch_bounds__(kRowThreads) rmsnorm_fwd_v16_kernel(const bf16* __restrict__ x,
                                                                       const bf16* __restrict__ w, bf16* __restrict__ y,
                                                                       float* __restrict__ rstd_out, int T, int H,
                                                                       float eps) {
    __shared__ float red[72];
    const int nvec = H >> 4;
    Vec16 wc[NV], cache[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        int i = threadIdx.x + j * kRowThreads;
        if (i < nvec) wc[j] = ld_v16(w + (size_t)i * 16);
    }
    if (blockIdx.x < T) {
        const bf16* xr = x + (size_t)blockIdx.x * H;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            int i = threadIdx.x + j * kRowThreads;
            if (i < nvec) cache[j] = ld_v16(xr + (size_t)i * 16);
        }
    }
    for (int row = blockIdx.x; row < T; row += gridDim.x) {
        Vec16 nxt[NV];
        const int nrow = row + gridDim.x;
        if (nrow < T) {
            const bf16* xn = x + (size_t)nrow * H;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                int i = threadIdx.x + j * kRowThreads;
                if (i < nvec) nxt[j] = ld_v16(xn + (size_t)i * 16);
            }
        }
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            int i = threadIdx.x + j * kRowThreads;
            if (i < nvec) {
                float f[16];
                unpack16(cache[j], f);
#pragma unroll
                for (int k = 0; k < 16; ++k) ss += f[k] * f[k];
            }
        }
        ss = block_sum(ss, red);
        const float rstd = rsqrtf(ss / (float)H + eps);
        if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
        bf16* yr = y + (size_t)row * H;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            int i = threadIdx.x + j * kRowThreads;
            if (i < nvec) {
                float f[16], g[16];
                unpack16(cache[j], f);
                unpack16(wc[j], g);
#pragma unroll
                for (int k = 0; k < 16; ++k) f[k] = f[k] * rstd * g[k];
                st_v16(yr + (size_t)i * 16, pack16(f));
            }
        }
#pragma unroll
        for (int j = 0; j < NV; ++j) cache[j] = nxt[j];
    }
}

// dx = rstd * (g - xhat * mean(g * xhat)),  g = dy * w,  xhat = x * rstd;   dw += dy * xhat.
// Each CTA walks rows with stride gridDim.x and keeps its dw partial in registers; partials go to
// scratch [gridDim.x, H] fp32 and a second kernel folds them.  Requires H <= THREADS*NV*8.
template <int NV, int THREADS>
__global__ void __launch_bounds__(THREADS) rmsnorm_bwd_kernel(const bf16* __restrict__ x,
                                                                   const bf16* __restrict__ w,
                                                                   const bf16* __restrict__ dy,
                                                                   const float* __restrict__ rstd_in,
                                                                   bf16* __restrict__ dx,
                                                                   float* __restrict__ dw_partial, int T, int H) {
    __shared__ float red[72];
    const int nvec = H >> 3;
    float dwacc[NV][8];
    Vec8 wc[NV];            // this thread's slice of the weight, read once for all its rows
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        int i = threadIdx.x + j * THREADS;
        if (i < nvec) wc[j] = reinterpret_cast<const Vec8*>(w)[i];
#pragma unroll
        for (int k = 0; k < 8; ++k) dwacc[j][k] = 0.f;
    }
    // with 2 vectors per thread the next row's x and dy are loaded before this row's reduction (in flight across the
    // block barrier and the stores); wider rows take more threads, not more vectors: with 4 vectors and the second
    // copy the kernel needs 198 registers, two blocks fit an SM and it ran at 0.47 of the copy bandwidth against 0.59
    constexpr bool kPrefetch = NV <= 2;
    Vec8 xc[NV], gc[NV];
    auto load_row = [&](int r, Vec8* xd, Vec8* gd) {
        const Vec8* xr = reinterpret_cast<const Vec8*>(x + (size_t)r * H);
        const Vec8* gr = reinterpret_cast<const Vec8*>(dy + (size_t)r * H);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            int i = threadIdx.x + j * THREADS;
            if (i < nvec) {
                xd[j] = xr[i];
                gd[j] = gr[i];
            }
        }
    };
    float rstd_next = 0.f;          // the row's scalar is prefetched too: loaded at the top of its own iteration, its
                                    // latency would sit on every row's critical path
    if (kPrefetch && blockIdx.x < T) {
        load_row(blockIdx.x, xc, gc);
        rstd_next = rstd_in[blockIdx.x];
    }
    for (int row = blockIdx.x; row < T; row += gridDim.x) {
        Vec8 xn[kPrefetch ? NV : 1], gn[kPrefetch ? NV : 1];
        const int nrow = row + gridDim.x;
        float rstd;
        if constexpr (kPrefetch) {
            rstd = rstd_next;
            if (nrow < T) {
                load_row(nrow, xn, gn);
                rstd_next = rstd_in[nrow];
            }
        } else {
            rstd = rstd_in[row];
            load_row(row, xc, gc);
        }
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            int i = threadIdx.x + j * THREADS;
            if (i < nvec) {
                float a[8], b[8], ww[8];
                unpack8(xc[j], a);
                unpack8(gc[j], b);
                unpack8(wc[j], ww);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float xh = a[k] * rstd;
                    dwacc[j][k] += b[k] * xh;
                    dot += b[k] * ww[k] * xh;
                }
            }
        }
        dot = block_sum(dot, red) / (float)H;
        Vec8* dxr = reinterpret_cast<Vec8*>(dx + (size_t)row * H);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            int i = threadIdx.x + j * THREADS;
            if (i < nvec) {
                float a[8], b[8], ww[8], o[8];
                unpack8(xc[j], a);
                unpack8(gc[j], b);
                unpack8(wc[j], ww);
#pragma unroll
                for (int k = 0; k < 8; ++k) o[k] = rstd * (b[k] * ww[k] - a[k] * rstd * dot);
                dxr[i] = pack8(o);
            }
        }
        if constexpr (kPrefetch) {
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                xc[j] = xn[j];
                gc[j] = gn[j];
            }
        }
    }
    float* out = dw_partial + (size_t)blockIdx.x * H;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        int i = threadIdx.x + j * THREADS;
        if (i < nvec) {
            float4* o4 = reinterpret_cast<float4*>(out + i * 8);
            o4[0] = make_float4(dwacc[j][0], dwacc[j][1], dwacc[j][2], dwacc[j][3]);
            o4[1] = make_float4(dwacc[j][4], dwacc[j][5], dwacc[j][6], dwacc[j][7]);
        }
    }
}

// Folds [P, H] fp32 partials into bf16 [H]: one warp per 32 columns, lanes stride over P, then a
// transposed shuffle-free reduction through shared memory.
__global__ void fold_partials_kernel(const float* __restrict__ partial, bf16* __restrict__ out, int P, int H) {
    __shared__ float tile[8][33];
    const int c = blockIdx.x * 32 + threadIdx.x;  // blockDim = (32, 8)
    float s = 0.f;
    if (c < H)
        for (int p = threadIdx.y; p < P; p += 8) s += partial[(size_t)p * H + c];
    tile[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && c < H) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) t += tile[k][threadIdx.x];
        out[c] = __float2bfloat16(t);
    }
}

// ------------------------------------------------------------------------------------------ SwiGLU
// in: [T, 2F] = [gate | up];  out: [T, F] = silu(gate) * up
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, long long T, int F) {
    const int fv = F >> 3;
    const long long total = T * fv;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        long long r = idx / fv;
        int c = (int)(idx - r * fv);
        const Vec8* row = reinterpret_cast<const Vec8*>(in + r * 2 * F);
        float a[8], b[8];
        unpack8(row[c], a);
        unpack8(row[fv + c], b);
#pragma unroll
        for (int k = 0; k < 8; ++k) a[k] = a[k] / (1.f + __expf(-a[k])) * b[k];
        reinterpret_cast<Vec8*>(out + r * F)[c] = pack8(a);
    }
}

__global__ void swiglu_bwd_kernel(const bf16* __restrict__ in, const bf16* __restrict__ dout, bf16* __restrict__ din,
                                  long long T, int F) {
    const int fv = F >> 3;
    const long long total = T * fv;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        long long r = idx / fv;
        int c = (int)(idx - r * fv);
        const Vec8* row = reinterpret_cast<const Vec8*>(in + r * 2 * F);
        float a[8], b[8], g[8], da[8], db[8];
        unpack8(row[c], a);
        unpack8(row[fv + c], b);
        unpack8(reinterpret_cast<const Vec8*>(dout + r * F)[c], g);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            float s = 1.f / (1.f + __expf(-a[k]));
            float silu = a[k] * s;
            da[k] = g[k] * b[k] * (s + silu * (1.f - s));
            db[k] = g[k] * silu;
        }
        Vec8* orow = reinterpret_cast<Vec8*>(din + r * 2 * F);
        orow[c] = pack8(da);
        orow[fv + c] = pack8(db);
    }
}

// ------------------------------------------------------------------------------------------ GELU
// tanh form: 0.5 x (1 + tanh(c (x + 0.044715 x^3))), c = sqrt(2/pi); exact form: 0.5 x (1 + erf(x / sqrt 2)).
// The backward recomputes the activation's derivative from the saved input (one read of x and dy, one write).
template <bool TANH>
__device__ __forceinline__ float gelu_f(float x) {
    if (TANH) {
        const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
        return 0.5f * x * (1.f + tanhf(u));
    }
    return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
}
template <bool TANH>
__device__ __forceinline__ float gelu_df(float x) {
    if (TANH) {
        const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
        const float t = tanhf(u);
        return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * 0.7978845608028654f * (1.f + 3.f * 0.044715f * x * x);
    }
    return 0.5f * (1.f + erff(x * 0.7071067811865476f)) + x * 0.3989422804014327f * __expf(-0.5f * x * x);
}

template <bool TANH>
__global__ void gelu_fwd_kernel(const Vec8* __restrict__ in, Vec8* __restrict__ out, long long nvec) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
        float a[8];
        unpack8(in[i], a);
#pragma unroll
        for (int k = 0; k < 8; ++k) a[k] = gelu_f<TANH>(a[k]);
        out[i] = pack8(a);
    }
}

template <bool TANH>
__global__ void gelu_bwd_kernel(const Vec8* __restrict__ in, const Vec8* __restrict__ dout, Vec8* __restrict__ din,
                                long long nvec) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
        float a[8], g[8];
        unpack8(in[i], a);
        unpack8(dout[i], g);
#pragma unroll
        for (int k = 0; k < 8; ++k) a[k] = g[k] * gelu_df<TANH>(a[k]);
        din[i] = pack8(a);
    }
}

// ------------------------------------------------------------------------------------------ RoPE
// x: [T, N, D] with row stride `xs` elements between tokens (heads contiguous); out contiguous.
// half-rotation: cos/sin [T, D] (bf16): o1 = x1*c1 - x2*s1 ; o2 = x2*c2 + x1*s2  (sign flips for bwd)
__global__ void rope_half_kernel(const bf16* __restrict__ x, long long xs, const bf16* __restrict__ cosb,
                                 const bf16* __restrict__ sinb, bf16* __restrict__ out, int T, int N, int D,
                                 float sign) {
    const int hv = D >> 4;  // vectors per half
    const long long total = (long long)T * N * hv;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        int c = (int)(idx % hv);
        long long tn = idx / hv;
        int n = (int)(tn % N);
        long long t = tn / N;
        const bf16* xp = x + t * xs + (long long)n * D;
        float x1[8], x2[8], c1[8], c2[8], s1[8], s2[8], o1[8], o2[8];
        unpack8(reinterpret_cast<const Vec8*>(xp)[c], x1);
        unpack8(reinterpret_cast<const Vec8*>(xp + D / 2)[c], x2);
        const bf16* cp = cosb + t * D;
        const bf16* sp = sinb + t * D;
        unpack8(reinterpret_cast<const Vec8*>(cp)[c], c1);
        unpack8(reinterpret_cast<const Vec8*>(cp + D / 2)[c], c2);
        unpack8(reinterpret_cast<const Vec8*>(sp)[c], s1);
        unpack8(reinterpret_cast<const Vec8*>(sp + D / 2)[c], s2);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (sign > 0.f) {
                o1[k] = x1[k] * c1[k] - x2[k] * s1[k];
                o2[k] = x2[k] * c2[k] + x1[k] * s2[k];
            } else {  // transpose of the rotation
                o1[k] = x1[k] * c1[k] + x2[k] * s2[k];
                o2[k] = x2[k] * c2[k] - x1[k] * s1[k];
            }
        }
        bf16* op = out + (t * N + n) * (long long)D;
        reinterpret_cast<Vec8*>(op)[c] = pack8(o1);
        reinterpret_cast<Vec8*>(op + D / 2)[c] = pack8(o2);
    }
}

// the same rotation with 4-element (8-byte) accesses, for head dims whose half is a multiple of 4 but not of 8 (72, 88 ...)
__device__ __forceinline__ void unpack4(const uint2& v, float* f) {
    const bf162* p = reinterpret_cast<const bf162*>(&v);
    const float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ uint2 pack4(const float* f) {
    uint2 v;
    bf162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    v.x = *reinterpret_cast<uint32_t*>(&a);
    v.y = *reinterpret_cast<uint32_t*>(&b);
    return v;
}
__global__ void rope_half4_kernel(const bf16* __restrict__ x, long long xs, const bf16* __restrict__ cosb,
                                  const bf16* __restrict__ sinb, bf16* __restrict__ out, int T, int N, int D,
                                  float sign) {
    const int hv = D >> 3;  // 4-element vectors per half
    const long long total = (long long)T * N * hv;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        int c = (int)(idx % hv);
        long long tn = idx / hv;
        int n = (int)(tn % N);
        long long t = tn / N;
        const bf16* xp = x + t * xs + (long long)n * D;
        float x1[4], x2[4], c1[4], c2[4], s1[4], s2[4], o1[4], o2[4];
        unpack4(reinterpret_cast<const uint2*>(xp)[c], x1);
        unpack4(reinterpret_cast<const uint2*>(xp + D / 2)[c], x2);
        const bf16* cp = cosb + t * D;
        const bf16* sp = sinb + t * D;
        unpack4(reinterpret_cast<const uint2*>(cp)[c], c1);
        unpack4(reinterpret_cast<const uint2*>(cp + D / 2)[c], c2);
        unpack4(reinterpret_cast<const uint2*>(sp)[c], s1);
        unpack4(reinterpret_cast<const uint2*>(sp + D / 2)[c], s2);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (sign > 0.f) {
                o1[k] = x1[k] * c1[k] - x2[k] * s1[k];
                o2[k] = x2[k] * c2[k] + x1[k] * s2[k];
            } else {
                o1[k] = x1[k] * c1[k] + x2[k] * s2[k];
                o2[k] = x2[k] * c2[k] - x1[k] * s1[k];
            }
        }
        bf16* op = out + (t * N + n) * (long long)D;
        reinterpret_cast<uint2*>(op)[c] = pack4(o1);
        reinterpret_cast<uint2*>(op + D / 2)[c] = pack4(o2);
    }
}

// interleaved pairs: cos/sin [T, D/2] fp32
__global__ void rope_inter_kernel(const bf16* __restrict__ x, long long xs, const float* __restrict__ cosf_,
                                  const float* __restrict__ sinf_, bf16* __restrict__ out, int T, int N, int D,
                                  float sign) {
    const int dv = D >> 3;
    const long long total = (long long)T * N * dv;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        int c = (int)(idx % dv);
        long long tn = idx / dv;
        int n = (int)(tn % N);
        long long t = tn / N;
        float f[8], o[8];
        unpack8(reinterpret_cast<const Vec8*>(x + t * xs + (long long)n * D)[c], f);
        const float4 cs = reinterpret_cast<const float4*>(cosf_ + t * (D / 2))[c];
        const float4 sn = reinterpret_cast<const float4*>(sinf_ + t * (D / 2))[c];
        const float cc[4] = {cs.x, cs.y, cs.z, cs.w};
        const float ss[4] = {sn.x * sign, sn.y * sign, sn.z * sign, sn.w * sign};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            o[2 * k] = f[2 * k] * cc[k] - f[2 * k + 1] * ss[k];
            o[2 * k + 1] = f[2 * k] * ss[k] + f[2 * k + 1] * cc[k];
        }
        reinterpret_cast<Vec8*>(out + (t * N + n) * (long long)D)[c] = pack8(o);
    }
}

// ------------------------------------------------------------------------------------------ adaLN
// y = LN(x) * (1 + scale[b]) + shift[b];  x: [B*S, H], scale/shift: [B, H] (bf16); saves mean / rstd.
template <int NV>
__global__ void __launch_bounds__(kThreads) ln_mod_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ scale,
                                                              const bf16* __restrict__ shift, bf16* __restrict__ y,
                                                              float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                              int T, int S, int H, float eps) {
    __shared__ float red[72];
    const int nvec = H >> 3;
    // scale / shift of the batch entry the current row belongs to, kept (packed) in registers and re-read only when the
    // entry changes (never for an affine LayerNorm, B = 1): reading them per row tripled the traffic through L1.  NV is
    // the number of 16-byte vectors a thread owns, so a 3584-wide row costs 2 x 3 vectors of registers, not 4 x 3.
    Vec8 xc[NV], scv[NV], shv[NV];
    int cached_b = -1;
    auto load_row = [&](int r, Vec8* dst) {
        const Vec8* xr = reinterpret_cast<const Vec8*>(x + (size_t)r * H);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            int i = threadIdx.x + j * kThreads;
            if (i < nvec) dst[j] = xr[i];
        }
    };
    if (blockIdx.x < T) load_row(blockIdx.x, xc);
    for (int row = blockIdx.x; row < T; row += gridDim.x) {
        Vec8 xn[NV];                  // next row: in flight across this row's reduction and stores
        if (row + gridDim.x < T) load_row(row + gridDim.x, xn);
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            int i = threadIdx.x + j * kThreads;
            if (i < nvec) {
                float f[8];
                unpack8(xc[j], f);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    s1 += f[k];
                    s2 += f[k] * f[k];
                }
            }
        }
        block_sum2(s1, s2, red);
        const float mean = s1 / (float)H;
        const float rstd = rsqrtf(fmaxf(s2 / (float)H - mean * mean, 0.f) + eps);
        if (threadIdx.x == 0) {
            mean_out[row] = mean;
            rstd_out[row] = rstd;
        }
        const int b = row / S;
        if (b != cached_b) {
            cached_b = b;
            const Vec8* sc = reinterpret_cast<const Vec8*>(scale + (size_t)b * H);
            const Vec8* sh = reinterpret_cast<const Vec8*>(shift + (size_t)b * H);
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                int i = threadIdx.x + j * kThreads;
                if (i < nvec) {
                    scv[j] = sc[i];
                    shv[j] = sh[i];
                }
            }
        }
        Vec8* yr = reinterpret_cast<Vec8*>(y + (size_t)row * H);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            int i = threadIdx.x + j * kThreads;
            if (i < nvec) {
                float f[8], a[8], c[8], o[8];
                unpack8(xc[j], f);
                unpack8(scv[j], a);
                unpack8(shv[j], c);
#pragma unroll
                for (int k = 0; k < 8; ++k) o[k] = (f[k] - mean) * rstd * (1.f + a[k]) + c[k];
                yr[i] = pack8(o);
            }
        }
#pragma unroll
        for (int j = 0; j < NV; ++j) xc[j] = xn[j];
    }
}

// The same forward with 32-byte accesses (rows a multiple of 16 elements, 32-byte aligned pointers): NV vectors of 16 per
// thread.  As for RMSNorm, the 16-byte form was limited by the number of load / store instructions, not by DRAM.
template <int NV>
__global__ void __launch_bounds__(kThreads) ln_mod_fwd_v16_kernel(const bf16* __restrict__ x, const bf16* __restrict__ scale,
                                                                  const bf16* __restrict__ shift, bf16* __restrict__ y,
                                                                  float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                                  int T, int S, int H, float eps) {
    __shared__ float red[72];
    const int nvec = H >> 4;
    Vec16 xc[NV], scv[NV], shv[NV];
    int cached_b = -1;
    auto load_row = [&](int r, Vec16* dst) {
        const bf16* xr = x + (size_t)r * H;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            int i = threadIdx.x + j * kThreads;
            if (i < nvec) dst[j] = ld_v16(xr + (size_t)i * 16);
        }
    };
    if (blockIdx.x < T) load_row(blockIdx.x, xc);
    for (int row = blockIdx.x; row < T; row += gridDim.x) {
        Vec16 xn[NV];
        if (row + gridDim.x < T) load_row(row + gridDim.x, xn);
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            int i = threadIdx.x + j * kThreads;
            if (i < nvec) {
                float f[16];
                unpack16(xc[j], f);
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    s1 += f[k];
                    s2 += f[k] * f[k];
                }
            }
        }
        block_sum2(s1, s2, red);
        const float mean = s1 / (float)H;
        const float rstd = rsqrtf(fmaxf(s2 / (float)H - mean * mean, 0.f) + eps);
        if (threadIdx.x == 0) {
            mean_out[row] = mean;
            rstd_out[row] = rstd;
        }
        const int b = row / S;
        if (b != cached_b) {
            cached_b = b;
            const bf16* sc = scale + (size_t)b * H;
            const bf16* sh = shift + (size_t)b * H;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                int i = threadIdx.x + j * kThreads;
                if (i < nvec) {
                    scv[j] = ld_v16(sc + (size_t)i * 16);
                    shv[j] = ld_v16(sh + (size_t)i * 16);
                }
            }
        }
        bf16* yr = y + (size_t)row * H;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            int i = threadIdx.x + j * kThreads;
            if (i < nvec) {
                float f[16], a[16], c[16];
                unpack16(xc[j], f);
                unpack16(scv[j], a);
                unpack16(shv[j], c);
#pragma unroll
                for (int k = 0; k < 16; ++k) f[k] = (f[k] - mean) * rstd * (1.f + a[k]) + c[k];
                st_v16(yr + (size_t)i * 16, pack16(f));
            }
        }
#pragma unroll
        for (int j = 0; j < NV; ++j) xc[j] = xn[j];
    }
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)), g = dy * (1 + scale);
// dscale[b] += dy * xhat, dshift[b] += dy  -> per-CTA partials (CTA c handles rows of ONE batch entry).
__global__ void __launch_bounds__(kThreads) ln_mod_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ scale,
                                                              const bf16* __restrict__ dy,
                                                              const float* __restrict__ mean_in,
                                                              const float* __restrict__ rstd_in, bf16* __restrict__ dx,
                                                              float* __restrict__ dscale_partial,
                                                              float* __restrict__ dshift_partial, int S, int H,
                                                              int ctas_per_batch) {
    __shared__ float red[72];
    const int nvec = H >> 3;
    const int b = blockIdx.x / ctas_per_batch, lane_cta = blockIdx.x % ctas_per_batch;
    float sc[kMaxVec][8], dsc[kMaxVec][8], dsh[kMaxVec][8];
    const Vec8* scp = reinterpret_cast<const Vec8*>(scale + (size_t)b * H);
#pragma unroll
    for (int j = 0; j < kMaxVec; ++j) {
        int i = threadIdx.x + j * kThreads;
#pragma unroll
        for (int k = 0; k < 8; ++k) dsc[j][k] = dsh[j][k] = 0.f;
        if (i < nvec) unpack8(scp[i], sc[j]);
    }
    for (int s = lane_cta; s < S; s += ctas_per_batch) {
        const size_t row = (size_t)b * S + s;
        const Vec8* xr = reinterpret_cast<const Vec8*>(x + row * H);
        const Vec8* gr = reinterpret_cast<const Vec8*>(dy + row * H);
        const float mean = mean_in[row], rstd = rstd_in[row];
        float xh[kMaxVec][8], g[kMaxVec][8];
        float m1 = 0.f, m2 = 0.f;
#pragma unroll
        for (int j = 0; j < kMaxVec; ++j) {
            int i = threadIdx.x + j * kThreads;
            if (i < nvec) {
                float a[8], d[8];
                unpack8(xr[i], a);
                unpack8(gr[i], d);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    xh[j][k] = (a[k] - mean) * rstd;
                    dsc[j][k] += d[k] * xh[j][k];
                    dsh[j][k] += d[k];
                    g[j][k] = d[k] * (1.f + sc[j][k]);
                    m1 += g[j][k];
                    m2 += g[j][k] * xh[j][k];
                }
            }
        }
        block_sum2(m1, m2, red);
        m1 /= (float)H;
        m2 /= (float)H;
        Vec8* dxr = reinterpret_cast<Vec8*>(dx + row * H);
#pragma unroll
        for (int j = 0; j < kMaxVec; ++j) {
            int i = threadIdx.x + j * kThreads;
            if (i < nvec) {
                float o[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) o[k] = rstd * (g[j][k] - m1 - xh[j][k] * m2);
                dxr[i] = pack8(o);
            }
        }
    }
    float* o1 = dscale_partial + (size_t)blockIdx.x * H;
    float* o2 = dshift_partial + (size_t)blockIdx.x * H;
#pragma unroll
    for (int j = 0; j < kMaxVec; ++j) {
        int i = threadIdx.x + j * kThreads;
        if (i < nvec) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                o1[i * 8 + k] = dsc[j][k];
                o2[i * 8 + k] = dsh[j][k];
            }
        }
    }
}

// out[b, c] = sum_p partial[b*P + p, c]
__global__ void fold_partials_batched_kernel(const float* __restrict__ partial, bf16* __restrict__ out, int P, int H) {
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    int b = blockIdx.y;
    if (c >= H) return;
    float s = 0.f;
    for (int p = 0; p < P; ++p) s += partial[((size_t)b * P + p) * H + c];
    out[(size_t)b * H + c] = __float2bfloat16(s);
}

// out = x + gate[b] * y   (x,y: [B*S, H]; gate: [B, H])
__global__ void gated_residual_kernel(const bf16* __restrict__ x, const bf16* __restrict__ y,
                                      const bf16* __restrict__ gate, bf16* __restrict__ out, long long T, int S,
                                      int H) {
    const int hv = H >> 3;
    const long long total = T * hv;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        long long r = idx / hv;
        int c = (int)(idx - r * hv);
        int b = (int)(r / S);
        float a[8], d[8], g[8];
        unpack8(reinterpret_cast<const Vec8*>(x + r * H)[c], a);
        unpack8(reinterpret_cast<const Vec8*>(y + r * H)[c], d);
        unpack8(reinterpret_cast<const Vec8*>(gate + (size_t)b * H)[c], g);
#pragma unroll
        for (int k = 0; k < 8; ++k) a[k] += g[k] * d[k];
        reinterpret_cast<Vec8*>(out + r * H)[c] = pack8(a);
    }
}

// ------------------------------------------------------------------------------------------ AdamW
// One pass over this rank's shard: fp32 master/moments in place, bf16 copy out.  Elements below
// `split` get weight decay.  `scale_ptr` (optional, device) multiplies the gradient (clip coefficient).
template <typename G>
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                             const G* __restrict__ g, bf16* __restrict__ p16, long long n, long long split, float lr,
                             float b1, float b2, float eps, float wd, float bc1, float bc2, float gscale,
                             const float* __restrict__ scale_ptr) {
    const float gs = scale_ptr ? gscale * (*scale_ptr) : gscale;
    const long long nv = n >> 2;
    const uint64_t pol = l2_evict_first_policy();      // 28 bytes per parameter, each touched once
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
         i += (long long)gridDim.x * blockDim.x) {
        float4 pp = ld_stream_f4(reinterpret_cast<const float4*>(p) + i, pol);
        float4 mm = ld_stream_f4(reinterpret_cast<const float4*>(m) + i, pol);
        float4 vv = ld_stream_f4(reinterpret_cast<const float4*>(v) + i, pol);
        float gg[4];
        if constexpr (sizeof(G) == 2) {
            const uint2 raw = ld_stream_u2(reinterpret_cast<const uint2*>(g) + i, pol);
            const bf162* gp = reinterpret_cast<const bf162*>(&raw);
            float2 a = __bfloat1622float2(gp[0]), b = __bfloat1622float2(gp[1]);
            gg[0] = a.x; gg[1] = a.y; gg[2] = b.x; gg[3] = b.y;
        } else {
            float4 a = ld_stream_f4(reinterpret_cast<const float4*>(g) + i, pol);
            gg[0] = a.x; gg[1] = a.y; gg[2] = a.z; gg[3] = a.w;
        }
        float* P = &pp.x; float* M = &mm.x; float* V = &vv.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float gk = gg[k] * gs;
            const float decay = (i * 4 + k) < split ? wd : 0.f;
            M[k] = b1 * M[k] + (1.f - b1) * gk;
            V[k] = b2 * V[k] + (1.f - b2) * gk * gk;
            const float denom = sqrtf(V[k] / bc2) + eps;
            P[k] = P[k] * (1.f - lr * decay) - lr * (M[k] / bc1) / denom;
        }
        st_stream_f4(reinterpret_cast<float4*>(p) + i, pp, pol);
        st_stream_f4(reinterpret_cast<float4*>(m) + i, mm, pol);
        st_stream_f4(reinterpret_cast<float4*>(v) + i, vv, pol);
        bf162* o = reinterpret_cast<bf162*>(p16) + 2 * i;
        o[0] = __floats2bfloat162_rn(pp.x, pp.y);
        o[1] = __floats2bfloat162_rn(pp.z, pp.w);
    }
}

inline int grid_for(long long work_items, int threads, int per_sm = 8) {
    long long blocks = (work_items + threads - 1) / threads;
    long long cap = 148LL * per_sm;
    return (int)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

}  // namespace

// ------------------------------------------------------------------------------------------ C ABI
// Squared L2 norm of an fp32 buffer, for the global gradient norm over many flat shards: block b of the launch for
// buffer `slot` writes its partial to partials[slot * kSqNormBlocks + b] (fixed summation order: the result does not
// depend on scheduling).  The caller zero-fills `partials` once and sums it with one reduction.
constexpr int kSqNormBlocks = 128;

__global__ void __launch_bounds__(256) sq_norm_kernel(const float* __restrict__ x, long long n, float* __restrict__ partials) {
    __shared__ float red[40];
    float acc = 0.f;
    const long long n4 = n >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n4; i += 256ll * gridDim.x) {
        const float4 v = x4[i];
        acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
        const float v = x[(n4 << 2) + threadIdx.x];
        acc += v * v;
    }
    acc = block_sum(acc, red);
    if (threadIdx.x == 0) partials[blockIdx.x] = acc;
}

// Grid of a row-walking kernel: one wave of resident blocks (a second, partial wave would leave SMs idle at the end).
template <typename K>
static int resident_grid(K kernel, int threads, int rows, int& cache) {
    if (cache == 0) {
        int per_sm = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0);
        cache = 148 * (per_sm < 1 ? 1 : per_sm);
    }
    return rows < cache ? rows : cache;
}

static int g_rms_fwd_v16 = 1;
// 1 (default): rows that allow it use the 32-byte-access forward kernel; 0: always the 16-byte form (for A / B timing).
MM_API int mm_rmsnorm_set_v16(int on) {
    g_rms_fwd_v16 = on ? 1 : 0;
    return 0;
}

MM_API int mm_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int T, int H, float eps,
                          cudaStream_t st) {
    if (H % 8 || H > kRowThreads * 8 * 8) return -1;
    // measured at 3584 (two vectors of 16 per thread): 0.86 -> 0.91 of the copy bandwidth; wider rows keep the 16-byte form
    if (H % 16 == 0 && H <= kRowThreads * 2 * 16 && ((((uintptr_t)x | (uintptr_t)y | (uintptr_t)w)) & 31) == 0 && g_rms_fwd_v16) {
        const int nv16 = (H / 16 + kRowThreads - 1) / kRowThreads;
        static int h1 = 0, h2 = 0, h4 = 0;
#define MM_RMS_FWD16(NV)                                                                                        \
    rmsnorm_fwd_v16_kernel<NV><<<resident_grid(rmsnorm_fwd_v16_kernel<NV>, kRowThreads, T, h##NV), kRowThreads, 0, st>>>( \
        (const bf16*)x, (const bf16*)w, (bf16*)y, rstd, T, H, eps)
        if (nv16 <= 1) MM_RMS_FWD16(1);
        else if (nv16 <= 2) MM_RMS_FWD16(2);
        else MM_RMS_FWD16(4);
#undef MM_RMS_FWD16
        return (int)cudaGetLastError();
    }
    const int nv = (H / 8 + kRowThreads - 1) / kRowThreads;
    static int g2 = 0, g4 = 0, g8 = 0;
#define MM_RMS_FWD(NV)                                                                                  \
    rmsnorm_fwd_kernel<NV><<<resident_grid(rmsnorm_fwd_kernel<NV>, kRowThreads, T, g##NV), kRowThreads, 0, st>>>( \
        (const bf16*)x, (const bf16*)w, (bf16*)y, rstd, T, H, eps)
    if (nv <= 2) MM_RMS_FWD(2);
    else if (nv <= 4) MM_RMS_FWD(4);
    else MM_RMS_FWD(8);
#undef MM_RMS_FWD
    return (int)cudaGetLastError();
}

MM_API int mm_rmsnorm_bwd_grid(int T) { return T < 148 * 6 ? T : 148 * 6; }

// dw_partial: scratch of mm_rmsnorm_bwd_grid(T) * H floats.
MM_API int mm_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, void* dx, void* dw,
                          float* dw_partial, int T, int H, cudaStream_t st) {
    if (H % 8 || H > kRowThreads * 8 * 8) return -1;
    static int g128 = 0, g256 = 0, g512 = 0;
    int grid = mm_rmsnorm_bwd_grid(T);      // the scratch holds that many partial rows; one resident wave may be fewer
#define MM_RMS_BWD(TH)                                                                                              \
    grid = min(grid, resident_grid(rmsnorm_bwd_kernel<2, TH>, TH, T, g##TH));                                       \
    rmsnorm_bwd_kernel<2, TH><<<grid, TH, 0, st>>>((const bf16*)x, (const bf16*)w, (const bf16*)dy, rstd,          \
                                                   (bf16*)dx, dw_partial, T, H)
    if (H <= 128 * 16) { MM_RMS_BWD(128); }
    else if (H <= 256 * 16) { MM_RMS_BWD(256); }
    else { MM_RMS_BWD(512); }
#undef MM_RMS_BWD
    fold_partials_kernel<<<(H + 31) / 32, dim3(32, 8), 0, st>>>(dw_partial, (bf16*)dw, grid, H);
    return (int)cudaGetLastError();
}

MM_API int mm_swiglu_fwd(const void* in, void* out, long long T, int F, cudaStream_t st) {
    if (F % 8) return -1;
    swiglu_fwd_kernel<<<grid_for(T * (F / 8), 256), 256, 0, st>>>((const bf16*)in, (bf16*)out, T, F);
    return (int)cudaGetLastError();
}

MM_API int mm_swiglu_bwd(const void* in, const void* dout, void* din, long long T, int F, cudaStream_t st) {
    if (F % 8) return -1;
    swiglu_bwd_kernel<<<grid_for(T * (F / 8), 256), 256, 0, st>>>((const bf16*)in, (const bf16*)dout, (bf16*)din, T, F);
    return (int)cudaGetLastError();
}

// in / out / dout / din: contiguous bf16, n elements (multiple of 8, 16-byte aligned); tanh_form selects the approximation.
MM_API int mm_gelu_fwd(const void* in, void* out, long long n, int tanh_form, cudaStream_t st) {
    if (n % 8 || (((uintptr_t)in | (uintptr_t)out) & 15)) return -1;
    if (n == 0) return 0;
    if (tanh_form) gelu_fwd_kernel<true><<<grid_for(n / 8, 256), 256, 0, st>>>((const Vec8*)in, (Vec8*)out, n / 8);
    else gelu_fwd_kernel<false><<<grid_for(n / 8, 256), 256, 0, st>>>((const Vec8*)in, (Vec8*)out, n / 8);
    return (int)cudaGetLastError();
}

MM_API int mm_gelu_bwd(const void* in, const void* dout, void* din, long long n, int tanh_form, cudaStream_t st) {
    if (n % 8 || (((uintptr_t)in | (uintptr_t)dout | (uintptr_t)din) & 15)) return -1;
    if (n == 0) return 0;
    if (tanh_form)
        gelu_bwd_kernel<true><<<grid_for(n / 8, 256), 256, 0, st>>>((const Vec8*)in, (const Vec8*)dout, (Vec8*)din, n / 8);
    else
        gelu_bwd_kernel<false><<<grid_for(n / 8, 256), 256, 0, st>>>((const Vec8*)in, (const Vec8*)dout, (Vec8*)din, n / 8);
    return (int)cudaGetLastError();
}

MM_API int mm_rope_half(const void* x, long long xs, const void* cosb, const void* sinb, void* out, int T, int N,
                        int D, int backward, cudaStream_t st) {
    if (D % 8 || xs % 8) return -1;
    if (D % 16) {
        rope_half4_kernel<<<grid_for((long long)T * N * (D / 8), 256), 256, 0, st>>>(
            (const bf16*)x, xs, (const bf16*)cosb, (const bf16*)sinb, (bf16*)out, T, N, D, backward ? -1.f : 1.f);
        return (int)cudaGetLastError();
    }
    rope_half_kernel<<<grid_for((long long)T * N * (D / 16), 256), 256, 0, st>>>(
        (const bf16*)x, xs, (const bf16*)cosb, (const bf16*)sinb, (bf16*)out, T, N, D, backward ? -1.f : 1.f);
    return (int)cudaGetLastError();
}

MM_API int mm_rope_interleaved(const void* x, long long xs, const float* cosf_, const float* sinf_, void* out, int T,
                               int N, int D, int backward, cudaStream_t st) {
    if (D % 8 || xs % 8) return -1;
    rope_inter_kernel<<<grid_for((long long)T * N * (D / 8), 256), 256, 0, st>>>(
        (const bf16*)x, xs, cosf_, sinf_, (bf16*)out, T, N, D, backward ? -1.f : 1.f);
    return (int)cudaGetLastError();
}

MM_API int mm_ln_mod_fwd(const void* x, const void* scale, const void* shift, void* y, float* mean, float* rstd,
                         int T, int S, int H, float eps, cudaStream_t st) {
    if (H % 8 || H > kThreads * kMaxVec * 8) return -1;
    // 32-byte accesses where they measured faster: one vector of 16 per thread (rows up to 4096: 0.69 -> 0.76 of the copy
    // bandwidth at 4096); with two vectors per thread (5120) the 16-byte form stayed ahead (0.59 against 0.50)
    if (H % 16 == 0 && H <= kThreads * 16 && g_rms_fwd_v16 &&
        ((((uintptr_t)x | (uintptr_t)y | (uintptr_t)scale | (uintptr_t)shift)) & 31) == 0) {
        static int h1 = 0;
        ln_mod_fwd_v16_kernel<1><<<resident_grid(ln_mod_fwd_v16_kernel<1>, kThreads, T, h1), kThreads, 0, st>>>(
            (const bf16*)x, (const bf16*)scale, (const bf16*)shift, (bf16*)y, mean, rstd, T, S, H, eps);
        return (int)cudaGetLastError();
    }
    const int nv = (H / 8 + kThreads - 1) / kThreads;
    static int g1 = 0, g2 = 0, g4 = 0;
#define MM_LN_FWD(NV)                                                                                                \
    ln_mod_fwd_kernel<NV><<<resident_grid(ln_mod_fwd_kernel<NV>, kThreads, T, g##NV), kThreads, 0, st>>>(            \
        (const bf16*)x, (const bf16*)scale, (const bf16*)shift, (bf16*)y, mean, rstd, T, S, H, eps)
    if (nv <= 1) MM_LN_FWD(1);
    else if (nv <= 2) MM_LN_FWD(2);
    else MM_LN_FWD(4);
#undef MM_LN_FWD
    return (int)cudaGetLastError();
}

MM_API int mm_ln_mod_bwd_ctas(int B, int S) {
    int per = (148 * 4) / (B < 1 ? 1 : B);
    if (per < 1) per = 1;
    return per < S ? per : S;
}

// partials: 2 * B * mm_ln_mod_bwd_ctas(B,S) * H floats of scratch.
MM_API int mm_ln_mod_bwd(const void* x, const void* scale, const void* dy, const float* mean, const float* rstd,
                         void* dx, void* dscale, void* dshift, float* partials, int B, int S, int H,
                         cudaStream_t st) {
    if (H % 8 || H > kThreads * kMaxVec * 8) return -1;
    int per = mm_ln_mod_bwd_ctas(B, S);
    float* p1 = partials;
    float* p2 = partials + (size_t)B * per * H;
    ln_mod_bwd_kernel<<<B * per, kThreads, 0, st>>>((const bf16*)x, (const bf16*)scale, (const bf16*)dy, mean, rstd,
                                                    (bf16*)dx, p1, p2, S, H, per);
    dim3 g((H + 255) / 256, B);
    fold_partials_batched_kernel<<<g, 256, 0, st>>>(p1, (bf16*)dscale, per, H);
    fold_partials_batched_kernel<<<g, 256, 0, st>>>(p2, (bf16*)dshift, per, H);
    return (int)cudaGetLastError();
}

MM_API int mm_gated_residual(const void* x, const void* y, const void* gate, void* out, long long T, int S, int H,
                             cudaStream_t st) {
    if (H % 8) return -1;
    gated_residual_kernel<<<grid_for(T * (H / 8), 256), 256, 0, st>>>((const bf16*)x, (const bf16*)y, (const bf16*)gate,
                                                                      (bf16*)out, T, S, H);
    return (int)cudaGetLastError();
}

MM_API int mm_adamw(float* p, float* m, float* v, const void* g, int g_is_bf16, void* p16, long long n,
                    long long split, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                    float gscale, const float* scale_ptr, cudaStream_t st) {
    if (n % 4) return -1;
    int grid = grid_for(n / 4, 256, 16);
    if (g_is_bf16)
        adamw_kernel<bf16><<<grid, 256, 0, st>>>(p, m, v, (const bf16*)g, (bf16*)p16, n, split, lr, b1, b2, eps, wd, bc1,
                                                 bc2, gscale, scale_ptr);
    else
        adamw_kernel<float><<<grid, 256, 0, st>>>(p, m, v, (const float*)g, (bf16*)p16, n, split, lr, b1, b2, eps, wd,
                                                  bc1, bc2, gscale, scale_ptr);
    return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------ no-alloc variant
// RMSNorm backward with its dw partials in a fixed device array instead of caller memory; see mm_noalloc.h
// for who needs this and for the rules (size limits, first call outside capture, calls share the array).
#include <mutex>
#include "mm_noalloc.h"

static __device__ __align__(256) float g_noalloc_rms_partials[MM_NOALLOC_MAX_CTAS * MM_NOALLOC_MAX_H];

namespace {
constexpr int kNoAllocMaxDevices = 64;
float* g_noalloc_ptr[kNoAllocMaxDevices] = {};
std::mutex g_noalloc_mu;

// In host code the array's name is only a handle; the kernel needs the address the current device gave it.
int noalloc_workspace(float** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) return MM_NOALLOC_E_SYMBOL;
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (!g_noalloc_ptr[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_noalloc_rms_partials) != cudaSuccess || !p) {
            (void)cudaGetLastError();
            return MM_NOALLOC_E_SYMBOL;
        }
        g_noalloc_ptr[dev] = static_cast<float*>(p);
    }
    *out = g_noalloc_ptr[dev];
    return 0;
}
}  // namespace

MM_API const char* mm_noalloc_strerror(int code) {
    switch (code) {
        case 0: return "ok";
        case MM_NOALLOC_E_SIZE:
            return "mm_rmsnorm_bwd_noalloc: need T >= 1 and H a multiple of 8 with H <= 4096 (fixed workspace)";
        case MM_NOALLOC_E_SYMBOL:
            return "mm_rmsnorm_bwd_noalloc: could not resolve the device address of the built-in workspace";
        default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown error";
    }
}

MM_API int mm_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy, const float* rstd, void* dx, void* dw,
                                  int T, int H, cudaStream_t st) {
    if (T < 1 || H < 8 || H % 8 || H > MM_NOALLOC_MAX_H) return MM_NOALLOC_E_SIZE;
    float* partial = nullptr;
    if (int rc = noalloc_workspace(&partial)) return rc;
    const int grid = T < MM_NOALLOC_MAX_CTAS ? T : MM_NOALLOC_MAX_CTAS;
    if (H <= 128 * 16)
        rmsnorm_bwd_kernel<2, 128><<<grid, 128, 0, st>>>((const bf16*)x, (const bf16*)w, (const bf16*)dy, rstd,
                                                         (bf16*)dx, partial, T, H);
    else
        rmsnorm_bwd_kernel<2, 256><<<grid, 256, 0, st>>>((const bf16*)x, (const bf16*)w, (const bf16*)dy, rstd,
                                                         (bf16*)dx, partial, T, H);
    fold_partials_kernel<<<(H + 31) / 32, dim3(32, 8), 0, st>>>(partial, (bf16*)dw, grid, H);
    return (int)cudaGetLastError();
}

MM_API int mm_sq_norm_blocks() { return kSqNormBlocks; }

// x: fp32, 16-byte aligned, n elements; partials: this buffer's row of mm_sq_norm_blocks() floats (zero-filled by the
// caller: a short buffer uses fewer blocks and leaves the rest of its row untouched).
MM_API int mm_sq_norm(const float* x, long long n, float* partials, cudaStream_t st) {
    if (n <= 0) return 0;
    if ((uintptr_t)x & 15) return -1;
    long long want = (n / 4 + 255) / 256;
    const int grid = (int)(want < 1 ? 1 : (want > kSqNormBlocks ? kSqNormBlocks : want));
    sq_norm_kernel<<<grid, 256, 0, st>>>(x, n, partials);
    return (int)cudaGetLastError();
}
