// Chunk-local prologue of the gated delta rule (WY form), one CTA per (chunk of 64 tokens, head), K = V = 128:
//
//   gc = cumsum(g)                                 decay[i][j] = exp(gc_i - gc_j)  (j <= i)
//   A  = tril(beta_i * (k_i . k_j) * decay, -1)    T = (I + A)^-1   (unit lower triangular, forward substitution)
//   U  = T (v * beta)          W  = T (k * beta * exp(gc))
//   Qg = q * scale * exp(gc)   Kd = k * exp(gc_last - gc)          At = (q_i . k_j) * decay * scale  (j <= i)
//   gamma = exp(gc_last)
//
// Inputs are the packed [T, H, *] tensors of the layer (q, k already L2-normalised); a chunk never straddles a sequence,
// rows past the end of a sequence's last chunk are zero (beta = g = 0), so they leave T, U, W and the state untouched.
// Outputs are bf16 [H, NC, 64, *] (what the tcgen05 state-pass kernel reads) and gamma fp32 [H, NC].
// All arithmetic is fp32 on the CUDA cores: the op is 2 MFLOP per CTA and bound by the 64-step substitution, not by the
// products; the products use 4 x 4 / 4 x 8 register tiles over shared memory with an odd row stride (no bank conflicts).
#include "common.cuh"

namespace {

constexpr int C = 64, D = 128, LD = D + 1, LT = C + 1;
constexpr int kThreads = 256;
constexpr int kSmemFloats = 3 * C * LD + 2 * C * LT + 3 * C;      // sK, sQ, sX, sA/T, sAt(unused slot kept for T copy), gc/beta/eg
constexpr int kSmemBytes = kSmemFloats * 4;

__device__ __forceinline__ void load_rows(const bf16* __restrict__ src, long long tok0, int len, int H, int head, float* dst) {
    // [len, D] rows of one head from a packed [T, H, D] tensor -> fp32 [C][LD]; rows >= len are zero
    for (int i = threadIdx.x; i < C * (D / 8); i += kThreads) {
        const int r = i / (D / 8), c8 = i % (D / 8);
        float f[8];
        if (r < len) unpack8(reinterpret_cast<const Vec8*>(src + ((tok0 + r) * H + head) * (long long)D)[c8], f);
        else
#pragma unroll
            for (int k = 0; k < 8; ++k) f[k] = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) dst[r * LD + c8 * 8 + k] = f[k];
    }
}

__device__ __forceinline__ void store_rows(const float* src, int ld, bf16* __restrict__ dst, int cols) {
    // fp32 [C][ld] (first `cols` columns) -> bf16 [C][cols] contiguous
    for (int i = threadIdx.x; i < C * (cols / 8); i += kThreads) {
        const int r = i / (cols / 8), c8 = i % (cols / 8);
        float f[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = src[r * ld + c8 * 8 + k];
        reinterpret_cast<Vec8*>(dst + (size_t)r * cols)[c8] = pack8(f);
    }
}

__global__ void __launch_bounds__(kThreads) gdn_prologue_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v, const float* __restrict__ g,
    const float* __restrict__ beta, const int* __restrict__ chunk_tok0, const int* __restrict__ chunk_len,
    bf16* __restrict__ W, bf16* __restrict__ Qg, bf16* __restrict__ Kd, bf16* __restrict__ At, bf16* __restrict__ U,
    float* __restrict__ gamma, int H, int NC, float scale) {
    extern __shared__ float sm[];
    float* sK = sm;                     // [C][LD]
    float* sQ = sK + C * LD;            // [C][LD]   q, later v * beta
    float* sX = sQ + C * LD;            // [C][LD]   k * beta * exp(gc)
    float* sT = sX + C * LD;            // [C][LT]   A, then T = (I + A)^-1
    float* sS = sT + C * LT;            // [C][LT]   At staging
    float* gc = sS + C * LT;            // [C] cumulative log gate
    float* bt = gc + C;                 // [C] beta
    float* eg = bt + C;                 // [C] exp(gc)
    const int c = blockIdx.x, head = blockIdx.y;
    const long long tok0 = chunk_tok0[c];
    const int len = chunk_len[c];
    const size_t slab = ((size_t)head * NC + c) * C;          // row offset of this (head, chunk) in the [H, NC, 64, *] outputs

    if (threadIdx.x < C) {
        const int r = threadIdx.x;
        gc[r] = r < len ? g[(tok0 + r) * H + head] : 0.f;
        bt[r] = r < len ? beta[(tok0 + r) * H + head] : 0.f;
    }
    load_rows(k, tok0, len, H, head, sK);
    load_rows(q, tok0, len, H, head, sQ);
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.f;
        for (int r = 0; r < C; ++r) {
            s += gc[r];
            gc[r] = s;
        }
        gamma[(size_t)head * NC + c] = __expf(s);
    }
    __syncthreads();
    if (threadIdx.x < C) eg[threadIdx.x] = __expf(gc[threadIdx.x]);

    // ---- KK^T and QK^T: thread owns a 4 x 4 block of both
    {
        const int r0 = (threadIdx.x / 16) * 4, c0 = (threadIdx.x % 16) * 4;
        float kk[4][4], qk[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) kk[i][j] = qk[i][j] = 0.f;
        if (c0 <= r0 + 3) {               // blocks strictly above the diagonal are never used
            for (int d = 0; d < D; ++d) {
                float a[4], b[4], e[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    a[i] = sK[(r0 + i) * LD + d];
                    e[i] = sQ[(r0 + i) * LD + d];
                    b[i] = sK[(c0 + i) * LD + d];
                }
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        kk[i][j] += a[i] * b[j];
                        qk[i][j] += e[i] * b[j];
                    }
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int r = r0 + i, cc = c0 + j;
                const float dec = cc <= r ? __expf(gc[r] - gc[cc]) : 0.f;
                sT[r * LT + cc] = cc < r ? bt[r] * kk[i][j] * dec : 0.f;
                sS[r * LT + cc] = qk[i][j] * dec * scale;
            }
    }
    __syncthreads();
    store_rows(sS, LT, At + slab * C, C);
    __syncthreads();                    // sS is reused for T below

    // ---- warps 0-1: T = (I + A)^-1, one column per thread (a column only depends on itself);
    //      warps 2-7 meanwhile: Qg, Kd out, then X = k * beta * exp(gc)
    if (threadIdx.x < C) {
        const int col = threadIdx.x;
        // rows above the diagonal of column `col` are zero, the diagonal is one: start below it
        for (int i = 0; i < C; ++i) {
            float t = (i == col) ? 1.f : 0.f;
            if (i > col) {
                for (int j = col; j < i; ++j) t -= sT[i * LT + j] * sS[j * LT + col];
            }
            sS[i * LT + col] = t;         // sS now holds T (At was stored above); A stays in sT
        }
    } else {
        const int t = threadIdx.x - C, nth = kThreads - C;
        const float last = gc[C - 1];
        for (int i = t; i < C * (D / 8); i += nth) {
            const int r = i / (D / 8), c8 = i % (D / 8);
            float fq[8], fk[8], fx[8];
            const float sq = scale * eg[r], sk = __expf(last - gc[r]), sx = bt[r] * eg[r];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float kv = sK[r * LD + c8 * 8 + e];
                fq[e] = sQ[r * LD + c8 * 8 + e] * sq;
                fk[e] = kv * sk;
                fx[e] = kv * sx;
            }
            reinterpret_cast<Vec8*>(Qg + (slab + r) * D)[c8] = pack8(fq);
            reinterpret_cast<Vec8*>(Kd + (slab + r) * D)[c8] = pack8(fk);
#pragma unroll
            for (int e = 0; e < 8; ++e) sX[r * LD + c8 * 8 + e] = fx[e];
        }
    }
    __syncthreads();
    // sQ <- v * beta (q is no longer needed)
    for (int i = threadIdx.x; i < C * (D / 8); i += kThreads) {
        const int r = i / (D / 8), c8 = i % (D / 8);
        float f[8];
        if (r < len) unpack8(reinterpret_cast<const Vec8*>(v + ((tok0 + r) * H + head) * (long long)D)[c8], f);
        else
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) sQ[r * LD + c8 * 8 + e] = f[e] * bt[r];
    }
    __syncthreads();

    // ---- U = T (v beta), W = T X: thread owns 4 rows x 8 columns of both; T is lower triangular
    {
        const int r0 = (threadIdx.x / 16) * 4, c0 = (threadIdx.x % 16) * 8;
        float u[4][8], w[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) u[i][j] = w[i][j] = 0.f;
        for (int j = 0; j <= r0 + 3; ++j) {
            float tv[4], xv[8], vv[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) tv[i] = sS[(r0 + i) * LT + j];       // zero above the diagonal
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                vv[e] = sQ[j * LD + c0 + e];
                xv[e] = sX[j * LD + c0 + e];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    u[i][e] += tv[i] * vv[e];
                    w[i][e] += tv[i] * xv[e];
                }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            reinterpret_cast<Vec8*>(U + (slab + r0 + i) * D)[c0 / 8] = pack8(u[i]);
            reinterpret_cast<Vec8*>(W + (slab + r0 + i) * D)[c0 / 8] = pack8(w[i]);
        }
    }
}

}  // namespace

// q, k, v: packed [T, H, 128] bf16 (heads dense); g, beta: [T, H] fp32; chunk_tok0 / chunk_len: int32 [NC].
// W, Qg, Kd, U: bf16 [H, NC, 64, 128]; At: bf16 [H, NC, 64, 64]; gamma: fp32 [H, NC].
MM_API int mm_gdn_prologue(const void* q, const void* k, const void* v, const float* g, const float* beta,
                           const int* chunk_tok0, const int* chunk_len, void* W, void* Qg, void* Kd, void* At, void* U,
                           float* gamma, int H, int NC, float scale, cudaStream_t st) {
    if (NC == 0 || H == 0) return 0;
    static bool done = false;
    if (!done) {
        if (cudaFuncSetAttribute(gdn_prologue_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
            return -3;
        done = true;
    }
    gdn_prologue_kernel<<<dim3(NC, H), kThreads, kSmemBytes, st>>>(
        (const bf16*)q, (const bf16*)k, (const bf16*)v, g, beta, chunk_tok0, chunk_len, (bf16*)W, (bf16*)Qg, (bf16*)Kd,
        (bf16*)At, (bf16*)U, gamma, H, NC, scale);
    return (int)cudaGetLastError();
}
