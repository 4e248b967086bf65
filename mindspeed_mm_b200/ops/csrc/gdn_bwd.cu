// Backward chunk walk of the gated delta rule / Kimi delta attention on tcgen05, the mirror of gdn.cu.
//
// The forward walk is   Vn = U - W S,   O = Qg S + At Vn,   S' = gamma S + Kd^T Vn     (S: [K, V] state before the chunk).
// Given dO, the only sequential part of the backward is the gradient G = dL/dS' carried from the LAST chunk to the first:
//
//     dVn = At^T dO + Kd G                               [C, V]
//     G  <- gamma G + Qg^T dO - W^T dVn                  [K, V]     (gradient w.r.t. the state before the chunk)
//
// Everything else (dU = dVn, dW = -dVn S^T, dQg = dO S^T, dAt = dO Vn^T, dKd = Vn G^T, dgamma = <G, S>) is a batched product
// of saved per-chunk tensors and is left to the caller.  One CTA owns one (sequence, head) pair and keeps G^T [V = 128,
// K = 128] as fp32 in tensor memory for the whole walk; per chunk (transposed, one thread per row v):
//
//     E  = G^T Kd^T + dO^T At          [V, C]   A = bf16 copy of G^T (smem) / dO^T (smem), B = Kd K-major / At MN-major
//     dVn^T = E                                 epilogue threads: to global, and -dVn^T as bf16 into shared memory
//     G^T *= gamma                              TMEM read-modify-write (one factor, or one per key channel)
//     G^T += dO^T Qg + (-dVn^T) W      [V, K]   B = Qg, W MN-major
//
// G^T at the entry of a chunk (the gradient w.r.t. the state AFTER that chunk) is written out as bf16 for dKd / dgamma.
// Warp roles, the two-stage TMA ring (W, Qg, Kd, At of a chunk = 56 KB) and the bounded waits are those of gdn.cu.
#include "common.cuh"
#include "tc05.cuh"

namespace {
using namespace tc05;

constexpr int C = 64, DK = 128, DV = 128;
constexpr int kWBytes = C * DK * 2;          // 16 KB: two [64 x 64] swizzle atoms
constexpr int kAtomW = C * 128;              // 8 KB
constexpr int kAtBytes = C * C * 2;          // 8 KB
constexpr int kStageBytes = 3 * kWBytes + kAtBytes;   // 56 KB
constexpr int kSbBytes = DV * DK * 2;        // 32 KB: two [128 x 64] atoms
constexpr int kAtomSb = DV * 128;            // 16 KB
constexpr int kVnBytes = DV * C * 2;         // 16 KB
constexpr int kSmem = 2 * kStageBytes + kSbBytes + 2 * kVnBytes + 512 + 1024;

struct GdnBwdParams {
    const bf16* dO;           // [H, NC*C, DV]
    const float* gamma;       // [H, NC] or [H, NC, DK]
    const int* seq_chunks;    // [nseq + 1]
    bf16* dVn;                // [H, NC*C, DV]
    bf16* Gnext;              // [H, NC, DV, DK]: G^T at the entry of each chunk = gradient w.r.t. the state after it
    int* status;
    int NC, H;
    int gamma_per_channel;
};

__device__ __forceinline__ void store_row_bf16(uint8_t* dst, int v, const float* x) {
    // 64 values of row v -> [128 x 64] bf16 tile, 128-byte rows, 16-byte groups XOR-swizzled by the row
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        uint4 w;
        bf162 t0 = __floats2bfloat162_rn(x[8 * g + 0], x[8 * g + 1]);
        bf162 t1 = __floats2bfloat162_rn(x[8 * g + 2], x[8 * g + 3]);
        bf162 t2 = __floats2bfloat162_rn(x[8 * g + 4], x[8 * g + 5]);
        bf162 t3 = __floats2bfloat162_rn(x[8 * g + 6], x[8 * g + 7]);
        w.x = *reinterpret_cast<uint32_t*>(&t0);
        w.y = *reinterpret_cast<uint32_t*>(&t1);
        w.z = *reinterpret_cast<uint32_t*>(&t2);
        w.w = *reinterpret_cast<uint32_t*>(&t3);
        *reinterpret_cast<uint4*>(dst + v * 128 + ((g ^ (v & 7)) << 4)) = w;
    }
}

__global__ void __launch_bounds__(192, 1)
gdn_bwd_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmQ,
               const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmA, const GdnBwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sStage = smem;                          // [2][W | Qg | Kd | At]
    uint8_t* sGb = sStage + 2 * kStageBytes;         // bf16 copy of G^T
    uint8_t* sVn = sGb + kSbBytes;                   // -dVn^T
    uint8_t* sDo = sVn + kVnBytes;                   // dO^T
    uint64_t* bars = reinterpret_cast<uint64_t*>(sDo + kVnBytes);
    uint64_t* full = bars + 0;        // [2]
    uint64_t* empty = bars + 2;       // [2]
    uint64_t* bar_mma1 = bars + 4;
    uint64_t* bar_vn = bars + 5;
    uint64_t* bar_mma2 = bars + 6;
    uint64_t* bar_gb = bars + 7;      // bf16 copy of G^T and dO^T of the chunk are in shared memory
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.x, seq = blockIdx.y;
    const int c_begin = p.seq_chunks[seq], n_chunks = p.seq_chunks[seq + 1] - c_begin;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        mbar_init(bar_mma1, 1);
        mbar_init(bar_vn, 128);
        mbar_init(bar_mma2, 1);
        mbar_init(bar_gb, 128);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmW);
        prefetch_tmap(&tmQ);
        prefetch_tmap(&tmK);
        prefetch_tmap(&tmA);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 256);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tG = tmem_base, tE = tmem_base + 128;

    if (warp == 0) {
        // -------------------------------------------------------------------------------- TMA producer (last chunk first)
        if (lane == 0) {
            for (int i = 0; i < n_chunks; ++i) {
                const int st = i & 1;
                const uint32_t ph = (i >> 1) & 1;
                if (!mbar_wait(&empty[st], ph ^ 1, abort_flag)) { atomicExch(p.status, MM_TIMEOUT_TMA); break; }
                uint8_t* base = sStage + st * kStageBytes;
                const int row = (head * p.NC + c_begin + (n_chunks - 1 - i)) * C;
                mbar_expect_tx(&full[st], kStageBytes);
                tma_load_2d(base, &tmW, &full[st], 0, row);
                tma_load_2d(base + kAtomW, &tmW, &full[st], 64, row);
                tma_load_2d(base + kWBytes, &tmQ, &full[st], 0, row);
                tma_load_2d(base + kWBytes + kAtomW, &tmQ, &full[st], 64, row);
                tma_load_2d(base + 2 * kWBytes, &tmK, &full[st], 0, row);
                tma_load_2d(base + 2 * kWBytes + kAtomW, &tmK, &full[st], 64, row);
                tma_load_2d(base + 3 * kWBytes, &tmA, &full[st], 0, row);
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_kmaj_n64 = idesc_bf16(128, C, 0, 0);     // B = [64 x K] K-major (Kd as rows of keys)
            constexpr uint32_t idesc_mn_n64 = idesc_bf16(128, C, 0, 1);       // B = At [j, i], contraction over its rows
            constexpr uint32_t idesc_mn_n128 = idesc_bf16(128, DK, 0, 1);     // B = Qg / W [t, k], contraction over rows
            bool ok = true;
            const uint32_t gb = smem_u32(sGb), vn = smem_u32(sVn), dO = smem_u32(sDo);
            for (int i = 0; i < n_chunks; ++i) {
                const int st = i & 1;
                const uint32_t ph = (i >> 1) & 1, par = i & 1;
                const uint32_t base = smem_u32(sStage + st * kStageBytes);
                if (!mbar_wait(&full[st], ph, abort_flag) || !mbar_wait(bar_gb, par, abort_flag)) { ok = false; break; }
                fence_after_sync();
                // E = G^T Kd^T (contraction over the 128 key channels) + dO^T At (contraction over the 64 query rows)
#pragma unroll
                for (int k = 0; k < DK / 16; ++k) {
                    const uint64_t da = smem_desc_sw128(gb + (k >> 2) * kAtomSb + (k & 3) * 32, 16, 1024);
                    const uint32_t boff = (k >> 2) * kAtomW + (k & 3) * 32;
                    mma_ss(tE, da, smem_desc_sw128(base + 2 * kWBytes + boff, 16, 1024), idesc_kmaj_n64, k ? 1u : 0u);
                }
#pragma unroll
                for (int k = 0; k < C / 16; ++k) {
                    const uint64_t da = smem_desc_sw128(dO + k * 32, 16, 1024);
                    mma_ss(tE, da, smem_desc_sw128(base + 3 * kWBytes + k * 2048, kAtBytes, 1024), idesc_mn_n64, 1u);
                }
                mma_commit(bar_mma1);
                if (!mbar_wait(bar_vn, par, abort_flag)) { ok = false; break; }
                fence_after_sync();
                // G^T += dO^T Qg + (-dVn^T) W
#pragma unroll
                for (int k = 0; k < C / 16; ++k) {
                    const uint64_t d1 = smem_desc_sw128(dO + k * 32, 16, 1024);
                    const uint64_t d2 = smem_desc_sw128(vn + k * 32, 16, 1024);
                    mma_ss(tG, d1, smem_desc_sw128(base + kWBytes + k * 2048, kAtomW, 1024), idesc_mn_n128, 1u);
                    mma_ss(tG, d2, smem_desc_sw128(base + k * 2048, kAtomW, 1024), idesc_mn_n128, 1u);
                }
                mma_commit(bar_mma2);
                mma_commit(&empty[st]);
            }
            if (!ok) atomicExch(p.status, MM_TIMEOUT_MMA);
        }
    } else {
        // -------------------------------------------------------------------------------- state rows (warps 2..5)
        const int qd = warp & 3;
        const int v = qd * 32 + lane;
        const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0u;
#pragma unroll
        for (int j = 0; j < 4; ++j) tmem_st_32x32(tG + lane_off + j * 32, r);
        tmem_wait_st();
#pragma unroll
        for (int g = 0; g < 16; ++g)
            *reinterpret_cast<uint4*>(sGb + (g >> 3) * kAtomSb + v * 128 + (((g & 7) ^ (v & 7)) << 4)) = make_uint4(0, 0, 0, 0);

        bool ok = true;
        for (int i = 0; i < n_chunks; ++i) {
            const uint32_t par = i & 1;
            const int chunk = c_begin + (n_chunks - 1 - i);
            const size_t tok0 = ((size_t)head * p.NC + chunk) * C;
            // dO^T row of this thread into shared memory; G^T (bf16) at the chunk's entry out to global memory
            float u[C];
            const bf16* dp = p.dO + tok0 * DV + v;
#pragma unroll
            for (int t = 0; t < C; ++t) u[t] = __bfloat162float(dp[(size_t)t * DV]);
            store_row_bf16(sDo, v, u);
            if (p.Gnext) {
                bf16* dst = p.Gnext + (((size_t)head * p.NC + chunk) * DV + v) * DK;
#pragma unroll
                for (int g = 0; g < 16; ++g)
                    reinterpret_cast<uint4*>(dst)[g] =
                        *reinterpret_cast<const uint4*>(sGb + (g >> 3) * kAtomSb + v * 128 + (((g & 7) ^ (v & 7)) << 4));
            }
            fence_proxy_async();
            fence_before_sync();
            mbar_arrive(bar_gb);

            const float gamma = p.gamma_per_channel ? 1.f : p.gamma[(size_t)head * p.NC + chunk];
            const float4* gvec = reinterpret_cast<const float4*>(p.gamma + ((size_t)head * p.NC + chunk) * DK);
            if (!mbar_wait(bar_mma1, par, abort_flag)) { ok = false; break; }
            fence_after_sync();
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                tmem_ld_32x32(tE + lane_off + j * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int t = 0; t < 32; ++t) u[j * 32 + t] = __uint_as_float(r[t]);
            }
            bf16* vp = p.dVn + tok0 * DV + v;
#pragma unroll
            for (int t = 0; t < C; ++t) {
                vp[(size_t)t * DV] = __float2bfloat16(u[t]);
                u[t] = -u[t];
            }
            store_row_bf16(sVn, v, u);
            // decay the fp32 gradient state in place
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                tmem_ld_32x32(tG + lane_off + j * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int t = 0; t < 32; ++t) r[t] = __float_as_uint(__uint_as_float(r[t]) * gamma);
                if (p.gamma_per_channel) {
#pragma unroll
                    for (int t = 0; t < 8; ++t) {
                        const float4 gv = __ldg(gvec + j * 8 + t);
                        r[4 * t + 0] = __float_as_uint(__uint_as_float(r[4 * t + 0]) * gv.x);
                        r[4 * t + 1] = __float_as_uint(__uint_as_float(r[4 * t + 1]) * gv.y);
                        r[4 * t + 2] = __float_as_uint(__uint_as_float(r[4 * t + 2]) * gv.z);
                        r[4 * t + 3] = __float_as_uint(__uint_as_float(r[4 * t + 3]) * gv.w);
                    }
                }
                tmem_st_32x32(tG + lane_off + j * 32, r);
            }
            tmem_wait_st();
            fence_proxy_async();
            fence_before_sync();
            mbar_arrive(bar_vn);

            if (!mbar_wait(bar_mma2, par, abort_flag)) { ok = false; break; }
            fence_after_sync();
            // refresh the bf16 operand copy of G^T
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                tmem_ld_32x32(tG + lane_off + j * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    uint4 w;
                    bf162 t0 = __floats2bfloat162_rn(__uint_as_float(r[8 * g + 0]), __uint_as_float(r[8 * g + 1]));
                    bf162 t1 = __floats2bfloat162_rn(__uint_as_float(r[8 * g + 2]), __uint_as_float(r[8 * g + 3]));
                    bf162 t2 = __floats2bfloat162_rn(__uint_as_float(r[8 * g + 4]), __uint_as_float(r[8 * g + 5]));
                    bf162 t3 = __floats2bfloat162_rn(__uint_as_float(r[8 * g + 6]), __uint_as_float(r[8 * g + 7]));
                    w.x = *reinterpret_cast<uint32_t*>(&t0);
                    w.y = *reinterpret_cast<uint32_t*>(&t1);
                    w.z = *reinterpret_cast<uint32_t*>(&t2);
                    w.w = *reinterpret_cast<uint32_t*>(&t3);
                    const int gg = j * 4 + g;
                    *reinterpret_cast<uint4*>(sGb + (gg >> 3) * kAtomSb + v * 128 + (((gg & 7) ^ (v & 7)) << 4)) = w;
                }
            }
        }
        if (!ok && lane == 0) atomicExch(p.status, MM_TIMEOUT_EPI);
    }

    if (*abort_flag)
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        fence_after_sync();
        tmem_dealloc(tmem_base, 256);
    }
}

}  // namespace

// W, Qg, Kd: [H, NC*64, 128] bf16; At: [H, NC*64, 64] bf16; dO, dVn: [H, NC*64, 128] bf16; gamma as in mm_gdn_fwd;
// Gnext: [H, NC, 128, 128] bf16 (transposed: [v, k]) or null; seq_chunks: [nseq + 1] int32 (device).
MM_API int mm_gdn_bwd(const void* W, const void* Qg, const void* Kd, const void* At, const void* dO, const float* gamma,
                      const int* seq_chunks, void* dVn, void* Gnext, int H, int NC, int nseq, int gamma_per_channel,
                      int* status, cudaStream_t st) {
    if (H <= 0 || NC <= 0 || nseq <= 0) return -1;
    if (gamma_per_channel && ((uintptr_t)gamma & 15)) return -1;
    CUtensorMap tmW, tmQ, tmK, tmA;
    const uint64_t rows = (uint64_t)H * NC * C;
    int rc = make_tmap_2d(&tmW, W, rows, DK, DK, C, 64);
    rc |= make_tmap_2d(&tmQ, Qg, rows, DK, DK, C, 64);
    rc |= make_tmap_2d(&tmK, Kd, rows, DK, DK, C, 64);
    rc |= make_tmap_2d(&tmA, At, rows, C, C, C, 64);
    if (rc) return -2;
    if (cudaFuncSetAttribute(gdn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) return -3;
    GdnBwdParams p{(const bf16*)dO, gamma, seq_chunks, (bf16*)dVn, (bf16*)Gnext, status, NC, H, gamma_per_channel};
    gdn_bwd_kernel<<<dim3(H, nseq), 192, kSmem, st>>>(tmW, tmQ, tmK, tmA, p);
    return (int)cudaGetLastError();
}
