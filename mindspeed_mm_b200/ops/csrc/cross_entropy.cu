// Row-wise softmax cross entropy that turns bf16 logits into their gradient in place.
//
//   loss[t]   = logsumexp(z[t, :]) - z[t, label[t]]           (0 for ignored rows)
//   z[t, :]  <- (softmax(z[t, :]) - onehot(label[t]))          (0 for ignored rows)
//
// One CTA per row, two passes: pass 1 keeps a running (max, sum) per thread (online softmax) and merges
// them across the block; pass 2 re-reads the row (304 KB for V = 152064: still L2-resident) and writes
// the gradient.  fp32 math on bf16 storage; V must be a multiple of 8 and rows 16-byte aligned.
#include "common.cuh"

namespace {

constexpr int kCEThreads = 512;

__global__ void __launch_bounds__(kCEThreads) ce_fwd_bwd_kernel(bf16* __restrict__ z, long long ld,
                                                                const long long* __restrict__ labels,
                                                                float* __restrict__ loss, int V, int ignore_index) {
    __shared__ float red[72];
    const long long row = blockIdx.x;
    Vec8* zr = reinterpret_cast<Vec8*>(z + row * ld);
    const int nvec = V >> 3;
    const long long label = labels[row];
    if (label == ignore_index) {
        Vec8 zero;
#pragma unroll
        for (int i = 0; i < 4; ++i) zero.v[i] = __floats2bfloat162_rn(0.f, 0.f);
        for (int i = threadIdx.x; i < nvec; i += kCEThreads) zr[i] = zero;
        if (threadIdx.x == 0) loss[row] = 0.f;
        return;
    }
    float m = -INFINITY, s = 0.f;
    for (int i = threadIdx.x; i < nvec; i += kCEThreads) {
        float f[8];
        unpack8(zr[i], f);
        float lm = f[0];
#pragma unroll
        for (int k = 1; k < 8; ++k) lm = fmaxf(lm, f[k]);
        const float nm = fmaxf(m, lm);
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) acc += __expf(f[k] - nm);
        s = s * __expf(m - nm) + acc;
        m = nm;
    }
    // block max
    float wm = warp_max(m);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) red[wid] = wm;
    __syncthreads();
    float M = red[lane < (kCEThreads >> 5) ? lane : 0];
    M = warp_max(M);
    __syncthreads();
    const float S = block_sum(s * __expf(m - M), red);
    const float lse = M + __logf(S);
    if (threadIdx.x == 0) loss[row] = lse - __bfloat162float(z[row * ld + label]);
    __syncthreads();  // the label logit has been read before anyone overwrites it
    const int lvec = (int)(label >> 3), lpos = (int)(label & 7);
    for (int i = threadIdx.x; i < nvec; i += kCEThreads) {
        float f[8];
        unpack8(zr[i], f);
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = __expf(f[k] - lse);
        if (i == lvec) f[lpos] -= 1.f;
        zr[i] = pack8(f);
    }
}

}  // namespace

MM_API int mm_ce_fwd_bwd(void* logits, long long ld, const long long* labels, float* loss, int T, int V,
                         int ignore_index, cudaStream_t st) {
    if (V % 8 || ld % 8) return -1;
    ce_fwd_bwd_kernel<<<T, kCEThreads, 0, st>>>((bf16*)logits, ld, labels, loss, V, ignore_index);
    return (int)cudaGetLastError();
}
