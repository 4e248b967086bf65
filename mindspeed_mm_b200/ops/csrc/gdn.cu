// Gated-delta-rule chunk recurrence on tcgen05 tensor cores with the running state resident in tensor memory.
//
// The chunk-local work of the WY form (cumulative gates, the triangular solve, u / w / decayed q and k, the masked
// intra-chunk attention) is batched over all chunks by the caller.  What cannot be batched is the walk over the
// chunks of one sequence, because every chunk needs the state its predecessor left.  One CTA owns one
// (sequence, head) pair and keeps the transposed state S^T [V=128, K=128] as fp32 in TMEM for the whole walk:
//
//   per chunk c (C = 64 tokens), with S the state before the chunk:
//     D1 = S^T W^T            [V, C]   (tcgen05, A = bf16 copy of S^T in shared memory, B = W  K-major)
//     D2 = S^T Qg^T           [V, C]
//     Vn^T = U^T - D1                  (epilogue threads; one thread per state row v)
//     S^T *= gamma_c                   (TMEM read-modify-write by the same threads)
//     D2 += Vn^T At^T         -> O^T   (A = Vn^T bf16 in shared memory, B = At K-major)
//     S^T += Vn^T Kd                   (B = Kd MN-major)
//
// Warp roles: warp 0 feeds a two-stage TMA ring (W, Qg, Kd, At of a chunk = 56 KB), warp 1 issues the MMAs,
// warps 2..5 are the 128 state-row threads.  Every wait is bounded; a wait that runs out sets the status word,
// raises the CTA's abort flag and the CTA falls through to the common TMEM release.
//
// Same operator as fla's chunk_gated_delta_rule used by the reference's Qwen3.5 GDN layer
// (fsdp/models/qwen3_5/modeling_qwen3_5.py, gated delta net block); the decomposition into kernels is this file's own.
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
constexpr int kSmem = 2 * kStageBytes + kSbBytes + kVnBytes + 512 + 1024;

struct GdnParams {
    const bf16* U;            // [H, NC*C, DV]
    const float* gamma;       // [H, NC] exp(sum of the chunk's log-gates), or [H, NC, DK] with one decay per key channel
    const int* seq_chunks;    // [nseq + 1] chunk ranges of the sequences
    bf16* O;                  // [H, NC*C, DV]
    bf16* Vn;                 // [H, NC*C, DV] or null
    bf16* Sprev;              // [H, NC, DV, DK] state before each chunk (transposed) or null
    float* Sfinal;            // [nseq, H, DV, DK] or null
    int* status;
    int NC, H;
    int gamma_per_channel;    // 0: one decay per (head, chunk) (gated delta rule); 1: one per key channel (KDA)
};

__global__ void __launch_bounds__(192, 1)
gdn_fwd_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmQ,
               const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmA, const GdnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sStage = smem;                          // [2][W | Qg | Kd | At]
    uint8_t* sSb = sStage + 2 * kStageBytes;
    uint8_t* sVn = sSb + kSbBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sVn + kVnBytes);
    uint64_t* full = bars + 0;        // [2]
    uint64_t* empty = bars + 2;       // [2]
    uint64_t* bar_mma1 = bars + 4;
    uint64_t* bar_vn = bars + 5;
    uint64_t* bar_mma2 = bars + 6;
    uint64_t* bar_sb = bars + 7;
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
        mbar_init(bar_sb, 128);
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
    const uint32_t tS = tmem_base, tD1 = tmem_base + 128, tD2 = tmem_base + 192;

    if (warp == 0) {
        // -------------------------------------------------------------------------------- TMA producer
        if (lane == 0) {
            for (int i = 0; i < n_chunks; ++i) {
                const int st = i & 1;
                const uint32_t ph = (i >> 1) & 1;
                if (!mbar_wait(&empty[st], ph ^ 1, abort_flag)) { atomicExch(p.status, MM_TIMEOUT_TMA); break; }
                uint8_t* base = sStage + st * kStageBytes;
                const int row = (head * p.NC + c_begin + i) * C;
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
            constexpr uint32_t idesc_n64 = idesc_bf16(128, C, 0, 0);
            constexpr uint32_t idesc_kd = idesc_bf16(128, DK, 0, 1);
            bool ok = true;
            const uint32_t sb = smem_u32(sSb), vn = smem_u32(sVn);
            for (int i = 0; i < n_chunks; ++i) {
                const int st = i & 1;
                const uint32_t ph = (i >> 1) & 1, par = i & 1;
                const uint32_t base = smem_u32(sStage + st * kStageBytes);
                if (!mbar_wait(&full[st], ph, abort_flag) || !mbar_wait(bar_sb, par, abort_flag)) { ok = false; break; }
                fence_after_sync();
#pragma unroll
                for (int k = 0; k < DK / 16; ++k) {
                    const uint64_t da = smem_desc_sw128(sb + (k >> 2) * kAtomSb + (k & 3) * 32, 16, 1024);
                    const uint32_t boff = (k >> 2) * kAtomW + (k & 3) * 32;
                    mma_ss(tD1, da, smem_desc_sw128(base + boff, 16, 1024), idesc_n64, k ? 1u : 0u);
                    mma_ss(tD2, da, smem_desc_sw128(base + kWBytes + boff, 16, 1024), idesc_n64, k ? 1u : 0u);
                }
                mma_commit(bar_mma1);
                if (!mbar_wait(bar_vn, par, abort_flag)) { ok = false; break; }
                fence_after_sync();
#pragma unroll
                for (int k = 0; k < C / 16; ++k) {
                    const uint64_t da = smem_desc_sw128(vn + k * 32, 16, 1024);
                    mma_ss(tD2, da, smem_desc_sw128(base + 3 * kWBytes + k * 32, 16, 1024), idesc_n64, 1u);
                    mma_ss(tS, da, smem_desc_sw128(base + 2 * kWBytes + k * 2048, kAtomW, 1024), idesc_kd, 1u);
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
        // zero state: fp32 in TMEM and its bf16 operand copy
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0u;
#pragma unroll
        for (int j = 0; j < 4; ++j) tmem_st_32x32(tS + lane_off + j * 32, r);
        tmem_wait_st();
#pragma unroll
        for (int g = 0; g < 16; ++g)
            *reinterpret_cast<uint4*>(sSb + (g >> 3) * kAtomSb + v * 128 + (((g & 7) ^ (v & 7)) << 4)) = make_uint4(0, 0, 0, 0);
        fence_proxy_async();
        fence_before_sync();
        mbar_arrive(bar_sb);

        bool ok = true;
        for (int i = 0; i < n_chunks; ++i) {
            const uint32_t par = i & 1;
            const int chunk = c_begin + i;
            const size_t tok0 = ((size_t)head * p.NC + chunk) * C;
            const bf16* up = p.U + tok0 * DV + v;
            float u[C];
#pragma unroll
            for (int t = 0; t < C; ++t) u[t] = __bfloat162float(up[(size_t)t * DV]);
            const float gamma = p.gamma_per_channel ? 1.f : p.gamma[(size_t)head * p.NC + chunk];
            const float4* gvec = reinterpret_cast<const float4*>(p.gamma + ((size_t)head * p.NC + chunk) * DK);
            if (p.Sprev) {   // bf16 state before this chunk: this thread's row of the operand copy
                bf16* dst = p.Sprev + (((size_t)head * p.NC + chunk) * DV + v) * DK;
#pragma unroll
                for (int g = 0; g < 16; ++g)
                    reinterpret_cast<uint4*>(dst)[g] =
                        *reinterpret_cast<const uint4*>(sSb + (g >> 3) * kAtomSb + v * 128 + (((g & 7) ^ (v & 7)) << 4));
            }
            if (!mbar_wait(bar_mma1, par, abort_flag)) { ok = false; break; }
            fence_after_sync();
            // Vn^T row = U^T row - D1 row
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                tmem_ld_32x32(tD1 + lane_off + j * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int t = 0; t < 32; ++t) u[j * 32 + t] -= __uint_as_float(r[t]);
            }
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                uint4 w;
                bf162 t0 = __floats2bfloat162_rn(u[8 * g + 0], u[8 * g + 1]);
                bf162 t1 = __floats2bfloat162_rn(u[8 * g + 2], u[8 * g + 3]);
                bf162 t2 = __floats2bfloat162_rn(u[8 * g + 4], u[8 * g + 5]);
                bf162 t3 = __floats2bfloat162_rn(u[8 * g + 6], u[8 * g + 7]);
                w.x = *reinterpret_cast<uint32_t*>(&t0);
                w.y = *reinterpret_cast<uint32_t*>(&t1);
                w.z = *reinterpret_cast<uint32_t*>(&t2);
                w.w = *reinterpret_cast<uint32_t*>(&t3);
                *reinterpret_cast<uint4*>(sVn + v * 128 + ((g ^ (v & 7)) << 4)) = w;
            }
            if (p.Vn) {
                bf16* vp = p.Vn + tok0 * DV + v;
#pragma unroll
                for (int t = 0; t < C; ++t) vp[(size_t)t * DV] = __float2bfloat16(u[t]);
            }
            // decay the fp32 state in place
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                tmem_ld_32x32(tS + lane_off + j * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int t = 0; t < 32; ++t) r[t] = __float_as_uint(__uint_as_float(r[t]) * gamma);
                if (p.gamma_per_channel) {   // column k of this thread's state row decays by gamma[k]: the same address
                                             // in every thread, a broadcast load
#pragma unroll
                    for (int t = 0; t < 8; ++t) {
                        const float4 gv = __ldg(gvec + j * 8 + t);
                        r[4 * t + 0] = __float_as_uint(__uint_as_float(r[4 * t + 0]) * gv.x);
                        r[4 * t + 1] = __float_as_uint(__uint_as_float(r[4 * t + 1]) * gv.y);
                        r[4 * t + 2] = __float_as_uint(__uint_as_float(r[4 * t + 2]) * gv.z);
                        r[4 * t + 3] = __float_as_uint(__uint_as_float(r[4 * t + 3]) * gv.w);
                    }
                }
                tmem_st_32x32(tS + lane_off + j * 32, r);
            }
            tmem_wait_st();
            fence_proxy_async();
            fence_before_sync();
            mbar_arrive(bar_vn);

            if (!mbar_wait(bar_mma2, par, abort_flag)) { ok = false; break; }
            fence_after_sync();
            bf16* op = p.O + tok0 * DV + v;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                tmem_ld_32x32(tD2 + lane_off + j * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int t = 0; t < 32; ++t) op[(size_t)(j * 32 + t) * DV] = __float2bfloat16(__uint_as_float(r[t]));
            }
            // refresh the bf16 operand copy of the state
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                tmem_ld_32x32(tS + lane_off + j * 32, r);
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
                    const int gg = j * 4 + g;   // 16-byte group of 8 k values: atom gg / 8, chunk gg % 8
                    *reinterpret_cast<uint4*>(sSb + (gg >> 3) * kAtomSb + v * 128 + (((gg & 7) ^ (v & 7)) << 4)) = w;
                }
            }
            fence_proxy_async();
            fence_before_sync();
            mbar_arrive(bar_sb);
        }
        if (ok && p.Sfinal) {
            float* dst = p.Sfinal + (((size_t)seq * p.H + head) * DV + v) * DK;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                tmem_ld_32x32(tS + lane_off + j * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int t = 0; t < 32; t += 4)
                    *reinterpret_cast<float4*>(dst + j * 32 + t) =
                        make_float4(__uint_as_float(r[t]), __uint_as_float(r[t + 1]), __uint_as_float(r[t + 2]),
                                    __uint_as_float(r[t + 3]));
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

// W, Qg, Kd: [H, NC*64, 128] bf16; At: [H, NC*64, 64] bf16; U, O, Vn: [H, NC*64, 128] bf16; gamma: [H, NC] fp32, or
// [H, NC, 128] with gamma_per_channel (Kimi delta attention: a decay per key channel);
// seq_chunks: [nseq + 1] int32 (device).  Vn, Sprev, Sfinal may be null.
MM_API int mm_gdn_fwd(const void* W, const void* Qg, const void* Kd, const void* At, const void* U, const float* gamma,
                      const int* seq_chunks, void* O, void* Vn, void* Sprev, float* Sfinal, int H, int NC, int nseq,
                      int gamma_per_channel, int* status, cudaStream_t st) {
    if (H <= 0 || NC <= 0 || nseq <= 0) return -1;
    if (gamma_per_channel && ((uintptr_t)gamma & 15)) return -1;
    CUtensorMap tmW, tmQ, tmK, tmA;
    const uint64_t rows = (uint64_t)H * NC * C;
    int rc = make_tmap_2d(&tmW, W, rows, DK, DK, C, 64);
    rc |= make_tmap_2d(&tmQ, Qg, rows, DK, DK, C, 64);
    rc |= make_tmap_2d(&tmK, Kd, rows, DK, DK, C, 64);
    rc |= make_tmap_2d(&tmA, At, rows, C, C, C, 64);
    if (rc) return -2;
    if (cudaFuncSetAttribute(gdn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) return -3;
    GdnParams p{(const bf16*)U, gamma, seq_chunks, (bf16*)O, (bf16*)Vn, (bf16*)Sprev, Sfinal, status, NC, H, gamma_per_channel};
    gdn_fwd_kernel<<<dim3(H, nseq), 192, kSmem, st>>>(tmW, tmQ, tmK, tmA, p);
    return (int)cudaGetLastError();
}
