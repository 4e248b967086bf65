// RMSNorm over the WHOLE hidden vector followed by interleaved-pair RoPE, applied on the head owner after a Ulysses
// head scatter (Wan: q and k are normalised over all 5120 channels before the heads are split,
// mindspeed_mm/models/predictor/dits/wan_dit.py:993-1007,1084-1086).
//
// After the scatter a rank holds, for ALL tokens, only the `blk` channels of its own heads, so the row statistics come
// from outside: ss[t, slot] = sum over all H channels of raw^2 (side output of the projection GEMM, exchanged between
// the ranks), rstd = rsqrt(ss / H + eps).
//
//   forward   y = rope(raw * rstd * w)                                    for slot q and slot k
//   backward  dyn = rope^T(dy);   DOT[t] = sum over ALL channels of dyn * w * raw   (partial per rank, summed over ranks)
//             draw = rstd * w * dyn - rstd^3 / H * raw * DOT[t];   dw[c] = sum_t dyn * raw * rstd
//
// raw: [T, pitch] bf16 with slot s at columns [s*blk, (s+1)*blk) (heads of D channels); cos / sin: [T, D/2] fp32;
// w: [2, blk] fp32-convertible bf16 (this rank's slices of the q and k norm weights).
#include "common.cuh"

namespace {

__device__ __forceinline__ void rope8(const float* f, const float4& cs, const float4& sn, float sign, float* o) {
    const float cc[4] = {cs.x, cs.y, cs.z, cs.w};
    const float ss[4] = {sn.x * sign, sn.y * sign, sn.z * sign, sn.w * sign};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        o[2 * k] = f[2 * k] * cc[k] - f[2 * k + 1] * ss[k];
        o[2 * k + 1] = f[2 * k] * ss[k] + f[2 * k + 1] * cc[k];
    }
}

struct QKP {
    const bf16* raw;
    long long pitch;
    const float* ss;        // [T, n_stats]
    int n_stats;
    const bf16* w;          // [2, blk]
    const float* cosf_;
    const float* sinf_;
    int T, blk, D, H;
    float eps;
};

__device__ __forceinline__ float rstd_of(const QKP& p, long long t, int slot) {
    return rsqrtf(p.ss[t * p.n_stats + slot] / (float)p.H + p.eps);
}

// out: [2, T, blk] bf16 (q then k), dense
__global__ void qk_norm_rope_fwd_kernel(QKP p, bf16* __restrict__ out) {
    const int bv = p.blk >> 3, dv = p.D >> 3;
    const long long total = 2LL * p.T * bv;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(idx % bv);
        const long long ts = idx / bv;
        const int slot = (int)(ts / p.T);
        const long long t = ts - (long long)slot * p.T;
        float f[8], wv[8], o[8];
        unpack8(reinterpret_cast<const Vec8*>(p.raw + t * p.pitch + (long long)slot * p.blk)[c], f);
        unpack8(reinterpret_cast<const Vec8*>(p.w + (long long)slot * p.blk)[c], wv);
        const float r = rstd_of(p, t, slot);
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = f[k] * r * wv[k];
        const int d = c % dv;
        const float4 cs = reinterpret_cast<const float4*>(p.cosf_ + t * (p.D / 2))[d];
        const float4 sn = reinterpret_cast<const float4*>(p.sinf_ + t * (p.D / 2))[d];
        rope8(f, cs, sn, 1.f, o);
        reinterpret_cast<Vec8*>(out + ((long long)slot * p.T + t) * p.blk)[c] = pack8(o);
    }
}

// dots[t, slot] = sum over this rank's channels of rope^T(dy) * w * raw; one warp per (slot, t).  dy: [2, T, blk].
__global__ void qk_norm_rope_dots_kernel(QKP p, const bf16* __restrict__ dy, float* __restrict__ dots) {
    const int bv = p.blk >> 3, dv = p.D >> 3;
    const int lane = threadIdx.x & 31;
    const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long ts = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); ts < 2LL * p.T; ts += warps) {
        const int slot = (int)(ts / p.T);
        const long long t = ts - (long long)slot * p.T;
        float acc = 0.f;
        for (int c = lane; c < bv; c += 32) {
            float g[8], f[8], wv[8], dyn[8];
            unpack8(reinterpret_cast<const Vec8*>(dy + ((long long)slot * p.T + t) * p.blk)[c], g);
            unpack8(reinterpret_cast<const Vec8*>(p.raw + t * p.pitch + (long long)slot * p.blk)[c], f);
            unpack8(reinterpret_cast<const Vec8*>(p.w + (long long)slot * p.blk)[c], wv);
            const int d = c % dv;
            const float4 cs = reinterpret_cast<const float4*>(p.cosf_ + t * (p.D / 2))[d];
            const float4 sn = reinterpret_cast<const float4*>(p.sinf_ + t * (p.D / 2))[d];
            rope8(g, cs, sn, -1.f, dyn);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc += dyn[k] * wv[k] * f[k];
        }
        acc = warp_sum(acc);
        if (lane == 0) dots[t * 2 + slot] = acc;
    }
}

// dw[slot, c] += sum over a chunk of rows of rope^T(dy) * raw * rstd; thread = one 8-channel vector, CTA row chunk = blockIdx.y
__global__ void qk_norm_rope_dw_kernel(QKP p, const bf16* __restrict__ dy, float* __restrict__ dw, int rows_per_cta) {
    const int bv = p.blk >> 3, dv = p.D >> 3;
    const int v = blockIdx.x * blockDim.x + threadIdx.x;      // over 2 * bv
    if (v >= 2 * bv) return;
    const int slot = v / bv, c = v - slot * bv, d = c % dv;
    const long long t0 = (long long)blockIdx.y * rows_per_cta;
    const long long t1 = min((long long)p.T, t0 + rows_per_cta);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (long long t = t0; t < t1; ++t) {
        float g[8], f[8], dyn[8];
        unpack8(reinterpret_cast<const Vec8*>(dy + ((long long)slot * p.T + t) * p.blk)[c], g);
        unpack8(reinterpret_cast<const Vec8*>(p.raw + t * p.pitch + (long long)slot * p.blk)[c], f);
        const float4 cs = reinterpret_cast<const float4*>(p.cosf_ + t * (p.D / 2))[d];
        const float4 sn = reinterpret_cast<const float4*>(p.sinf_ + t * (p.D / 2))[d];
        rope8(g, cs, sn, -1.f, dyn);
        const float r = rstd_of(p, t, slot);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] += dyn[k] * f[k] * r;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) atomicAdd(&dw[(long long)slot * p.blk + c * 8 + k], acc[k]);
}

// draw[t, slot*blk + c] = rstd * w * dyn - rstd^3 / H * raw * DOT, DOT = sum over `world` partial tables [world, T, 2]
__global__ void qk_norm_rope_bwd_kernel(QKP p, const bf16* __restrict__ dy, const float* __restrict__ dot_slots, int world,
                                        bf16* __restrict__ draw, long long dpitch) {
    const int bv = p.blk >> 3, dv = p.D >> 3;
    const long long total = 2LL * p.T * bv;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(idx % bv);
        const long long ts = idx / bv;
        const int slot = (int)(ts / p.T);
        const long long t = ts - (long long)slot * p.T;
        float g[8], f[8], wv[8], dyn[8], o[8];
        unpack8(reinterpret_cast<const Vec8*>(dy + ((long long)slot * p.T + t) * p.blk)[c], g);
        unpack8(reinterpret_cast<const Vec8*>(p.raw + t * p.pitch + (long long)slot * p.blk)[c], f);
        unpack8(reinterpret_cast<const Vec8*>(p.w + (long long)slot * p.blk)[c], wv);
        const int d = c % dv;
        const float4 cs = reinterpret_cast<const float4*>(p.cosf_ + t * (p.D / 2))[d];
        const float4 sn = reinterpret_cast<const float4*>(p.sinf_ + t * (p.D / 2))[d];
        rope8(g, cs, sn, -1.f, dyn);
        float dot = 0.f;
        for (int r = 0; r < world; ++r) dot += dot_slots[((long long)r * p.T + t) * 2 + slot];
        const float rs = rstd_of(p, t, slot);
        const float k2 = rs * rs * rs / (float)p.H * dot;
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = rs * wv[k] * dyn[k] - k2 * f[k];
        reinterpret_cast<Vec8*>(draw + t * dpitch + (long long)slot * p.blk)[c] = pack8(o);
    }
}

inline int flat_grid(long long work) {
    long long b = (work + 255) / 256;
    const long long cap = 148LL * 8;
    return (int)(b < 1 ? 1 : (b < cap ? b : cap));
}

inline bool bad(const QKP& p) { return p.blk % 8 || p.D % 8 || p.blk % p.D || p.pitch % 8 || p.T <= 0; }

}  // namespace

MM_API int mm_qk_norm_rope_fwd(const void* raw, long long pitch, const float* ss, int n_stats, const void* w, const float* cosf_,
                               const float* sinf_, void* out, int T, int blk, int D, int H, float eps, cudaStream_t st) {
    QKP p{(const bf16*)raw, pitch, ss, n_stats, (const bf16*)w, cosf_, sinf_, T, blk, D, H, eps};
    if (bad(p)) return -1;
    qk_norm_rope_fwd_kernel<<<flat_grid(2LL * T * (blk / 8)), 256, 0, st>>>(p, (bf16*)out);
    return (int)cudaGetLastError();
}

// dots: [T, 2] fp32 (this rank's partial); dw: [2, blk] fp32, zeroed by the caller
MM_API int mm_qk_norm_rope_bwd_partials(const void* raw, long long pitch, const float* ss, int n_stats, const void* w,
                                        const float* cosf_, const float* sinf_, const void* dy, float* dots, float* dw, int T,
                                        int blk, int D, int H, float eps, cudaStream_t st) {
    QKP p{(const bf16*)raw, pitch, ss, n_stats, (const bf16*)w, cosf_, sinf_, T, blk, D, H, eps};
    if (bad(p)) return -1;
    const long long warps_needed = 2LL * T;
    long long blocks = (warps_needed + 7) / 8;
    if (blocks > 148 * 8) blocks = 148 * 8;
    qk_norm_rope_dots_kernel<<<(int)blocks, 256, 0, st>>>(p, (const bf16*)dy, dots);
    const int vecs = 2 * (blk / 8);
    int chunks = (148 * 4 * 128) / (vecs < 128 ? 128 : vecs);
    if (chunks < 1) chunks = 1;
    if (chunks > T) chunks = T;
    const int rows_per = (T + chunks - 1) / chunks;
    dim3 grid((vecs + 127) / 128, (T + rows_per - 1) / rows_per);
    qk_norm_rope_dw_kernel<<<grid, 128, 0, st>>>(p, (const bf16*)dy, dw, rows_per);
    return (int)cudaGetLastError();
}

// dot_slots: [world, T, 2] fp32 partial tables of all ranks (local memory); draw: [T, dpitch] bf16, slots q and k written
MM_API int mm_qk_norm_rope_bwd(const void* raw, long long pitch, const float* ss, int n_stats, const void* w, const float* cosf_,
                               const float* sinf_, const void* dy, const float* dot_slots, int world, void* draw,
                               long long dpitch, int T, int blk, int D, int H, float eps, cudaStream_t st) {
    QKP p{(const bf16*)raw, pitch, ss, n_stats, (const bf16*)w, cosf_, sinf_, T, blk, D, H, eps};
    if (bad(p) || dpitch % 8) return -1;
    qk_norm_rope_bwd_kernel<<<flat_grid(2LL * T * (blk / 8)), 256, 0, st>>>(p, (const bf16*)dy, dot_slots, world, (bf16*)draw,
                                                                            dpitch);
    return (int)cudaGetLastError();
}
