// Auxiliary kernels of the gated-delta-net layer on packed sequences:
//   causal_conv1d (depthwise, kernel <= 8, optional SiLU, restarts at every sequence boundary) forward and backward,
//   l2norm over the head dim (forward and backward; the gated RMSNorm of the layer's output lives in rownorm.cu).
// x is [T, D] bf16 with the channel dim contiguous: a thread owns 8 channels (16 bytes) and walks a strip of
// tokens keeping the last K-1 inputs in registers, so every input is read once.
#include "common.cuh"

namespace {

constexpr int kMaxK = 8;
constexpr int kStrip = 32;   // tokens per thread strip

// seq_start[t] = first token index of the sequence token t belongs to (int32, precomputed from cu_seqlens).
// K is a template parameter so that the tap weights and the K-1 tokens of history stay in registers; the strip is
// walked in chunks of kChunk tokens whose loads are issued together.
constexpr int kChunk = 8;

template <int K, bool SILU>
__global__ void __launch_bounds__(128) conv1d_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                         const int* __restrict__ seq_start, bf16* __restrict__ y, int T,
                                                         int D) {
    const int dv = D >> 3;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= dv) return;
    const int t0 = blockIdx.y * kStrip, t1 = min(T, t0 + kStrip);
    float wk[K][8];
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
        for (int j = 0; j < 8; ++j) wk[k][j] = __bfloat162float(w[(size_t)(c * 8 + j) * K + k]);
    float hist[K][8];     // hist[i] = x[t - (K-1) + i]; hist[K-1] is the current token
    const int s0 = seq_start[t0];
#pragma unroll
    for (int i = 0; i < K - 1; ++i) {
        const int t = t0 - (K - 1) + i;
        if (t >= 0 && t >= s0) unpack8(reinterpret_cast<const Vec8*>(x + (size_t)t * D)[c], hist[i]);
        else
#pragma unroll
            for (int j = 0; j < 8; ++j) hist[i][j] = 0.f;
    }
    for (int tc = t0; tc < t1; tc += kChunk) {
        Vec8 in[kChunk];
        int st[kChunk];
#pragma unroll
        for (int u = 0; u < kChunk; ++u)
            if (tc + u < t1) {
                in[u] = reinterpret_cast<const Vec8*>(x + (size_t)(tc + u) * D)[c];
                st[u] = seq_start[tc + u];
            }
#pragma unroll
        for (int u = 0; u < kChunk; ++u) {
            const int t = tc + u;
            if (t >= t1) break;
            if (st[u] == t)      // a new sequence starts here: forget the history
#pragma unroll
                for (int i = 0; i < K - 1; ++i)
#pragma unroll
                    for (int j = 0; j < 8; ++j) hist[i][j] = 0.f;
            unpack8(in[u], hist[K - 1]);
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
            for (int k = 0; k < K; ++k)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] += wk[k][j] * hist[k][j];
            if (SILU)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = acc[j] / (1.f + __expf(-acc[j]));
            reinterpret_cast<Vec8*>(y + (size_t)t * D)[c] = pack8(acc);
#pragma unroll
            for (int i = 0; i < K - 1; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) hist[i][j] = hist[i + 1][j];
        }
    }
}

// dx[t] = sum_k w[k] * dpre[t + (K-1-k)] over outputs of the same sequence; dw[k] += dpre[u] * x[u - (K-1) + k].
// One pass over u = t0 .. t1 + K - 2 (the strip plus the K-1 outputs after it that still used its inputs): x[u] and dy[u]
// are read once, the pre-activation comes from the sliding history as in the forward, the last K values of dpre sit in a
// ring, and dx of token u - (K-1) is complete when u has been visited.  Weight gradients count outputs of the own strip
// only, so strips do not double count; they leave through fp32 atomics.
template <int K, bool SILU>
__global__ void __launch_bounds__(128) conv1d_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                         const int* __restrict__ seq_start, const int* __restrict__ seq_end,
                                                         const bf16* __restrict__ dy, bf16* __restrict__ dx,
                                                         float* __restrict__ dw, int T, int D) {
    const int dv = D >> 3;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= dv) return;
    const int t0 = blockIdx.y * kStrip, t1 = min(T, t0 + kStrip);
    float wk[K][8], dwacc[K][8];
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            wk[k][j] = __bfloat162float(w[(size_t)(c * 8 + j) * K + k]);
            dwacc[k][j] = 0.f;
        }
    float hist[K][8];     // inputs u-(K-1) .. u (zero before the start of u's sequence)
    float ring[K][8];     // ring[i] = dpre[u - (K-1) + i]
    int ring_t[K];        // the output token each ring slot holds (-1: none)
    const int s0 = seq_start[t0];
#pragma unroll
    for (int i = 0; i < K - 1; ++i) {
        const int t = t0 - (K - 1) + i;
        if (t >= 0 && t >= s0) unpack8(reinterpret_cast<const Vec8*>(x + (size_t)t * D)[c], hist[i]);
        else
#pragma unroll
            for (int j = 0; j < 8; ++j) hist[i][j] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < K; ++i) {
        ring_t[i] = -1;
#pragma unroll
        for (int j = 0; j < 8; ++j) ring[i][j] = 0.f;
    }
    const int u_end = min(T, t1 + K - 1);
    for (int u = t0; u < u_end + K - 1; ++u) {
        // shift the ring; slot K-1 receives dpre[u] (or nothing once u is past the last output that matters)
#pragma unroll
        for (int i = 0; i < K - 1; ++i) {
            ring_t[i] = ring_t[i + 1];
#pragma unroll
            for (int j = 0; j < 8; ++j) ring[i][j] = ring[i + 1][j];
        }
        ring_t[K - 1] = -1;
        if (u < u_end) {
            if (seq_start[u] == u)
#pragma unroll
                for (int i = 0; i < K - 1; ++i)
#pragma unroll
                    for (int j = 0; j < 8; ++j) hist[i][j] = 0.f;
            unpack8(reinterpret_cast<const Vec8*>(x + (size_t)u * D)[c], hist[K - 1]);
            float g[8];
            unpack8(reinterpret_cast<const Vec8*>(dy + (size_t)u * D)[c], g);
            if (SILU) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float pre = 0.f;
#pragma unroll
                    for (int k = 0; k < K; ++k) pre += wk[k][j] * hist[k][j];
                    const float sg = 1.f / (1.f + __expf(-pre));
                    g[j] = g[j] * sg * (1.f + pre * (1.f - sg));
                }
            }
            ring_t[K - 1] = u;
#pragma unroll
            for (int j = 0; j < 8; ++j) ring[K - 1][j] = g[j];
            if (u < t1)           // weight gradient of the own strip's outputs
#pragma unroll
                for (int k = 0; k < K; ++k)
#pragma unroll
                    for (int j = 0; j < 8; ++j) dwacc[k][j] += g[j] * hist[k][j];
#pragma unroll
            for (int i = 0; i < K - 1; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) hist[i][j] = hist[i + 1][j];
        }
        // input token t = u - (K-1) has now seen all its outputs t .. t + K - 1 (ring slots 0 .. K-1)
        const int t = u - (K - 1);
        if (t >= t0 && t < t1) {
            const int e = seq_end[t];
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
            for (int i = 0; i < K; ++i) {          // slot i holds output t + i, which used x[t] with tap K-1-i
                if (ring_t[i] == t + i && t + i < e)
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] += wk[K - 1 - i][j] * ring[i][j];
            }
            reinterpret_cast<Vec8*>(dx + (size_t)t * D)[c] = pack8(acc);
        }
    }
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
        for (int j = 0; j < 8; ++j) atomicAdd(&dw[(size_t)(c * 8 + j) * K + k], dwacc[k][j]);
}

// ---- l2norm over the last dim (D <= 256, one warp per row)
__global__ void l2norm_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, float* __restrict__ rnorm, long long rows,
                                  int D, float eps) {
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    float v[8];
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) {
        v[i >> 5] = __bfloat162float(x[row * D + i]);
        ss += v[i >> 5] * v[i >> 5];
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss + eps);
    if (lane == 0 && rnorm) rnorm[row] = r;
    for (int i = lane; i < D; i += 32) y[row * D + i] = __float2bfloat16(v[i >> 5] * r);
}

__global__ void l2norm_bwd_kernel(const bf16* __restrict__ y, const bf16* __restrict__ dy, const float* __restrict__ rnorm,
                                  bf16* __restrict__ dx, long long rows, int D) {
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    float yv[8], gv[8];
    float dot = 0.f;
    for (int i = lane; i < D; i += 32) {
        yv[i >> 5] = __bfloat162float(y[row * D + i]);
        gv[i >> 5] = __bfloat162float(dy[row * D + i]);
        dot += yv[i >> 5] * gv[i >> 5];
    }
    dot = warp_sum(dot);
    const float r = rnorm[row];
    for (int i = lane; i < D; i += 32) dx[row * D + i] = __float2bfloat16(r * (gv[i >> 5] - yv[i >> 5] * dot));
}

}  // namespace

#define MM_CONV_K(MACRO)                  \
    switch (K) {                          \
        case 1: MACRO(1); break;          \
        case 2: MACRO(2); break;          \
        case 3: MACRO(3); break;          \
        case 4: MACRO(4); break;          \
        case 5: MACRO(5); break;          \
        case 6: MACRO(6); break;          \
        case 7: MACRO(7); break;          \
        default: MACRO(8); break;         \
    }

MM_API int mm_conv1d_fwd(const void* x, const void* w, const int* seq_start, void* y, int T, int D, int K, int silu, cudaStream_t st) {
    if (D % 8 || K > kMaxK || K < 1) return -1;
    dim3 grid((D / 8 + 127) / 128, (T + kStrip - 1) / kStrip);
#define MM_CONV_FWD(KK)                                                                                                   \
    if (silu) conv1d_fwd_kernel<KK, true><<<grid, 128, 0, st>>>((const bf16*)x, (const bf16*)w, seq_start, (bf16*)y, T, D); \
    else conv1d_fwd_kernel<KK, false><<<grid, 128, 0, st>>>((const bf16*)x, (const bf16*)w, seq_start, (bf16*)y, T, D)
    MM_CONV_K(MM_CONV_FWD)
#undef MM_CONV_FWD
    return (int)cudaGetLastError();
}

// dw: fp32 [D, K], zeroed by the caller (accumulated with atomics).
MM_API int mm_conv1d_bwd(const void* x, const void* w, const int* seq_start, const int* seq_end, const void* dy, void* dx,
                         float* dw, int T, int D, int K, int silu, cudaStream_t st) {
    if (D % 8 || K > kMaxK || K < 1) return -1;
    dim3 grid((D / 8 + 127) / 128, (T + kStrip - 1) / kStrip);
#define MM_CONV_BWD(KK)                                                                                                  \
    if (silu)                                                                                                            \
        conv1d_bwd_kernel<KK, true><<<grid, 128, 0, st>>>((const bf16*)x, (const bf16*)w, seq_start, seq_end,           \
                                                          (const bf16*)dy, (bf16*)dx, dw, T, D);                         \
    else                                                                                                                 \
        conv1d_bwd_kernel<KK, false><<<grid, 128, 0, st>>>((const bf16*)x, (const bf16*)w, seq_start, seq_end,          \
                                                           (const bf16*)dy, (bf16*)dx, dw, T, D)
    MM_CONV_K(MM_CONV_BWD)
#undef MM_CONV_BWD
    return (int)cudaGetLastError();
}

MM_API int mm_l2norm_fwd(const void* x, void* y, float* rnorm, long long rows, int D, float eps, cudaStream_t st) {
    if (D > 256) return -1;
    l2norm_fwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const bf16*)x, (bf16*)y, rnorm, rows, D, eps);
    return (int)cudaGetLastError();
}

MM_API int mm_l2norm_bwd(const void* y, const void* dy, const float* rnorm, void* dx, long long rows, int D, cudaStream_t st) {
    if (D > 256) return -1;
    l2norm_bwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const bf16*)y, (const bf16*)dy, rnorm, (bf16*)dx, rows, D);
    return (int)cudaGetLastError();
}

