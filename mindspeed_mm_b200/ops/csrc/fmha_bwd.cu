// Flash attention backward on tcgen05 / TMEM / TMA (head dim 128, packed sequences, GQA, optional causal mask).
//
// Two kernels, neither of which needs atomics or a reduction pass:
//
//   fmha_bwd_dq_kernel   one CTA = one 128-row query tile of one head; walks the key tiles like the forward:
//                           S = Q K_j^T, dP = dO V_j^T                       (tcgen05, accumulators in TMEM)
//                           P = exp2(S c - lse), dS = P (dP - delta)          (one thread per query row)
//                           dQ += dS K_j                                      (dS through swizzled smem)
//   fmha_bwd_dkv_kernel  one CTA = one 128-row key tile of one KV head; walks the query tiles (64 rows each) of
//                        every query head that shares the KV head, computing the transposed products so that
//                        the key index sits on the TMEM lanes:
//                           S^T = K Q_i^T, dP^T = V dO_i^T
//                           P^T, dS^T -> swizzled smem (A operands)
//                           dV += P^T dO_i,  dK += dS^T Q_i
//   delta = rowsum(dO * O) comes from a small pre-pass.
//
// The recomputation of S and dP in both kernels costs 7 tile products instead of 5, in exchange for fully
// deterministic accumulation in tensor memory.  Warp roles, barriers and bounded waits follow the forward kernel.
#include "common.cuh"
#include "tc05.cuh"

namespace {
using namespace tc05;

constexpr int HD = 128;
constexpr int kTile = 128 * HD * 2;        // 32 KiB: a 128-row tile of Q / K / V / dO, or a 128 x 128 dS tile
constexpr int kAtom = 128 * 128;           // one 64-element-wide swizzle atom of 128 rows
constexpr float kLog2e = 1.4426950408889634f;

struct BwdParams {
    const int* cu_q;
    const int* cu_k;
    const int* tile_seq;
    const int* tile_r0;
    const int* tile_nseq;   // sequences covered by each tile (> 1: packed short sequences, block-diagonal mask)
    const int* n_tiles;
    const float* lse;       // [Nq, T]  natural log
    const float* delta;     // [Nq, T]
    bf16* dq;               // [T, Nq, 128]
    bf16* dk;               // [Tk, Nkv, 128]
    bf16* dv;
    int T, Tk, Nq, Nkv, causal;
    int D;                  // head dim of the tensors in global memory (<= HD); shared-memory tiles stay HD wide
    float scale, scale_log2;
    int* status;
    int split;              // dK/dV kernel: 1 = one CTA per QUERY head writing partial dk / dv [Tk, Nq, 128]
};

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]; one warp per (t, h)
__global__ void fmha_delta_kernel(const bf16* __restrict__ o, const bf16* __restrict__ dO, float* __restrict__ delta, int T,
                                  int Nq, int D) {
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= (long long)T * Nq) return;
    const int lane = threadIdx.x & 31;
    uint2 a = make_uint2(0, 0), b = make_uint2(0, 0);
    if (lane * 4 < D) {                     // D is a multiple of 8: a lane's four elements are all inside or all outside
        a = reinterpret_cast<const uint2*>(o + row * D)[lane];
        b = reinterpret_cast<const uint2*>(dO + row * D)[lane];
    }
    const bf162* pa = reinterpret_cast<const bf162*>(&a);
    const bf162* pb = reinterpret_cast<const bf162*>(&b);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pb[i]);
        s += x.x * y.x + x.y * y.y;
    }
    s = warp_sum(s);
    if (lane == 0) delta[(size_t)(row % Nq) * T + row / Nq] = s;
}

__global__ void fmha_bwd_plan_kernel(const int* cu, int n_seqs, int* tile_seq, int* tile_r0, int* n_tiles, int* tile_nseq,
                                     int max_tiles, int rows, int descending, int pack) {
    if (threadIdx.x || blockIdx.x) return;
    if (pack) {          // non-causal self-attention: short sequences share tiles
        int n = 0;
        for (int b = 0; b < n_seqs && n < max_tiles;) b = plan_packed(cu, n_seqs, b, rows, tile_seq, tile_r0, tile_nseq, n, max_tiles);
        *n_tiles = n;
        return;
    }
    int n = 0, longest = 0;
    for (int b = 0; b < n_seqs; ++b) longest = max(longest, cu[b + 1] - cu[b]);
    const int nt = (longest + rows - 1) / rows;
    for (int k = 0; k < nt; ++k) {
        const int t = descending ? nt - 1 - k : k;     // heavy tiles first
        for (int b = 0; b < n_seqs && n < max_tiles; ++b)
            if (t * rows < cu[b + 1] - cu[b]) {
                tile_nseq[n] = 1;
                tile_seq[n] = b;
                tile_r0[n] = t * rows;
                ++n;
            }
    }
    *n_tiles = n;
}

__device__ __forceinline__ uint32_t pack2(float a, float b) {
    bf162 t = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&t);
}

// ============================================================================================== dQ
constexpr int kRingK = 3;                 // K ring depth of the dQ kernel (V stays 2 deep: it is released right after dP)
constexpr int kSmemDq = (2 + kRingK + 2) * kTile + 1024 + 1024;

__global__ void __launch_bounds__(320, 1)
fmha_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, const BwdParams p) {
    if ((int)blockIdx.x >= *p.n_tiles) return;     // whole CTA leaves before any barrier or TMEM allocation
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sdO = sQ + kTile;
    uint8_t* sK = sdO + kTile;              // [kRingK]
    uint8_t* sV = sK + kRingK * kTile;      // [2]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * kTile);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;              // [kRingK]
    uint64_t* k_empty = k_full + kRingK;      // [kRingK]
    uint64_t* v_full = k_empty + kRingK;      // [2]
    uint64_t* v_empty = v_full + 2;           // [2]
    uint64_t* s_full = v_full + 4;            // [2]
    uint64_t* s_empty = v_full + 6;           // [2]
    uint64_t* dp_full = v_full + 8;
    uint64_t* dp_empty = v_full + 9;
    uint64_t* ds_full = v_full + 10;
    uint64_t* dq_full = v_full + 11;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(v_full + 12);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = p.tile_seq[blockIdx.x];
    const int q0 = p.tile_r0[blockIdx.x];
    const int nseq = p.tile_nseq[blockIdx.x];
    constexpr bool live = true;
    const int head = blockIdx.y;
    const int kv_head = head / (p.Nq / p.Nkv);
    const int q_begin = p.cu_q[seq], q_len = p.cu_q[seq + nseq] - q_begin;
    const int k_begin = p.cu_k[seq], k_len = p.cu_k[seq + nseq] - k_begin;
    const int diag = k_len - q_len;
    int kv_end = k_len;
    if (p.causal) kv_end = min(k_len, q0 + 128 + diag);
    const int n_kv = live ? max(0, (kv_end + 127) / 128) : 0;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < kRingK; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&s_empty[i], 256);
        }
        mbar_init(dp_full, 1);
        mbar_init(dp_empty, 256);
        mbar_init(ds_full, 256);
        mbar_init(dq_full, 1);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmQ);
        prefetch_tmap(&tmK);
        prefetch_tmap(&tmV);
        prefetch_tmap(&tmdO);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tS = tmem_base, tdP = tmem_base + 256, tdQ = tmem_base + 384;

    if (warp == 0) {
        if (lane == 0 && n_kv > 0) {
            mbar_expect_tx(q_full, 2 * kTile);
            tma_load_3d(sQ, &tmQ, q_full, 0, head, q_begin + q0);
            tma_load_3d(sQ + kAtom, &tmQ, q_full, 64, head, q_begin + q0);
            tma_load_3d(sdO, &tmdO, q_full, 0, head, q_begin + q0);
            tma_load_3d(sdO + kAtom, &tmdO, q_full, 64, head, q_begin + q0);
            for (int j = 0; j < n_kv; ++j) {
                const int st = j & 1, ks = j % kRingK;
                const uint32_t ph = (j >> 1) & 1, kph = (j / kRingK) & 1;
                const int row = k_begin + j * 128;
                if (!mbar_wait(&k_empty[ks], kph ^ 1, abort_flag)) { atomicExch(p.status, MM_TIMEOUT_TMA); break; }
                mbar_expect_tx(&k_full[ks], kTile);
                tma_load_3d(sK + ks * kTile, &tmK, &k_full[ks], 0, kv_head, row);
                tma_load_3d(sK + ks * kTile + kAtom, &tmK, &k_full[ks], 64, kv_head, row);
                if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag)) { atomicExch(p.status, MM_TIMEOUT_TMA); break; }
                mbar_expect_tx(&v_full[st], kTile);
                tma_load_3d(sV + st * kTile, &tmV, &v_full[st], 0, kv_head, row);
                tma_load_3d(sV + st * kTile + kAtom, &tmV, &v_full[st], 64, kv_head, row);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && n_kv > 0) {
            constexpr uint32_t idesc_kk = idesc_bf16(128, 128, 0, 0);     // both operands K-major
            constexpr uint32_t idesc_kn = idesc_bf16(128, 128, 0, 1);     // B = K_j as [N = d, K = kv]: MN-major
            bool ok = mbar_wait(q_full, 0, abort_flag);
            const uint32_t qa = smem_u32(sQ), doa = smem_u32(sdO);
            auto issue_s = [&](int j) -> bool {
                const int st = j & 1, ks = j % kRingK;
                const uint32_t ph = (j >> 1) & 1, kph = (j / kRingK) & 1;
                if (!mbar_wait(&s_empty[st], ph ^ 1, abort_flag) || !mbar_wait(&k_full[ks], kph, abort_flag)) return false;
                fence_after_sync();
                const uint32_t ka = smem_u32(sK + ks * kTile);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (k >> 2) * kAtom + (k & 3) * 32;
                    mma_ss(tS + st * 128, smem_desc_sw128(qa + off, 16, 1024), smem_desc_sw128(ka + off, 16, 1024), idesc_kk,
                           k ? 1u : 0u);
                }
                mma_commit(&s_full[st]);
                return true;
            };
            auto issue_dp = [&](int j) -> bool {
                const int st = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                if (!mbar_wait(dp_empty, (j & 1) ^ 1, abort_flag) || !mbar_wait(&v_full[st], ph, abort_flag)) return false;
                fence_after_sync();
                const uint32_t va = smem_u32(sV + st * kTile);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (k >> 2) * kAtom + (k & 3) * 32;
                    mma_ss(tdP, smem_desc_sw128(doa + off, 16, 1024), smem_desc_sw128(va + off, 16, 1024), idesc_kk, k ? 1u : 0u);
                }
                mma_commit(dp_full);
                mma_commit(&v_empty[st]);
                return true;
            };
            if (ok) ok = issue_s(0);
            if (ok) ok = issue_dp(0);
            for (int j = 0; j < n_kv && ok; ++j) {
                const int st = j & 1;
                // S and dP of the next tile run on the tensor pipe while the threads work on tile j; dP's single
                // buffer is free as soon as the threads have pulled dP(j) into registers
                if (j + 1 < n_kv && !(ok = issue_s(j + 1) && issue_dp(j + 1))) break;
                // dQ += dS_j K_j
                if (!mbar_wait(ds_full, j & 1, abort_flag)) { ok = false; break; }
                fence_after_sync();
                const int ks = j % kRingK;
                const uint32_t ka = smem_u32(sK + ks * kTile);
                {
                    // dS(j) sits in the columns of S[st] that the row threads emptied into registers: keys 0..63 in
                    // columns 0..31, keys 64..127 in columns 64..95 (bf16 pairs); TS-form product
#pragma unroll
                    for (int k = 0; k < 128 / 16; ++k) {
                        const uint64_t db = smem_desc_sw128(ka + k * 2048, kAtom, 1024);
                        mma_ts(tdQ, tS + st * 128 + (k >> 2) * 64 + (k & 3) * 8, db, idesc_kn, (j | k) ? 1u : 0u);
                    }
                }
                mma_commit(&k_empty[ks]);
            }
            if (ok) mma_commit(dq_full);
            if (!ok) atomicExch(p.status, MM_TIMEOUT_MMA);
        }
    } else {
        // two warpgroups of 128 threads: both own all 128 query rows, each takes 64 of the 128 key columns of a tile
        const int half = (warp - 2) >> 2;
        const int qd = warp & 3;
        const int row = qd * 32 + lane;
        const int qi = q0 + row;
        const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
        const bool row_ok = qi < q_len;
        int vis_lo = 0, vis_hi = k_len;                  // keys this row may see (packed tiles: its own sequence)
        if (nseq > 1) packed_row_range(p.cu_q, seq, nseq, q_begin + qi, q_begin, vis_lo, vis_hi);
        const size_t stat = (size_t)head * p.T + q_begin + min(qi, max(q_len - 1, 0));
        const float lse2 = n_kv > 0 ? p.lse[stat] * kLog2e : 0.f;
        const float dlt = n_kv > 0 ? p.delta[stat] : 0.f;
        bool ok = true;
        for (int j = 0; j < n_kv; ++j) {
            const int st = j & 1;
            const uint32_t ph = (j >> 1) & 1;
            if (!mbar_wait(&s_full[st], ph, abort_flag) || !mbar_wait(dp_full, j & 1, abort_flag)) { ok = false; break; }
            fence_after_sync();
            uint32_t r[64], d[64];
            const uint32_t t_row = tS + st * 128 + half * 64 + lane_off;
            tmem_ld_32x32(t_row, r);
            tmem_ld_32x32(t_row + 32, r + 32);
            tmem_ld_32x32(tdP + half * 64 + lane_off, d);
            tmem_ld_32x32(tdP + half * 64 + lane_off + 32, d + 32);
            tmem_wait_ld();
            fence_before_sync();
            mbar_arrive(&s_empty[st]);
            mbar_arrive(dp_empty);
            const int kbase = j * 128 + half * 64;
            const int limit = !row_ok ? -1 : (p.causal ? min(k_len - 1, qi + diag) : vis_hi - 1);
            // packed fp32 math (two columns per instruction): dS = exp2(S * scale - lse) * (dP - delta)
            const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nl2 = make_float2(-lse2, -lse2), nd2 = make_float2(-dlt, -dlt);
            const bool tile_masked = kbase + 63 > limit || nseq > 1;   // some column of this row is hidden (or the row is padding)
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float2 x = __ffma2_rn(make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])), sc2, nl2);
                const float2 g = __fadd2_rn(make_float2(__uint_as_float(d[2 * i]), __uint_as_float(d[2 * i + 1])), nd2);
                float2 ds = __fmul2_rn(make_float2(exp2f(x.x), exp2f(x.y)), g);
                if (tile_masked) {
                    if (kbase + 2 * i > limit || kbase + 2 * i < vis_lo) ds.x = 0.f;
                    if (kbase + 2 * i + 1 > limit || kbase + 2 * i + 1 < vis_lo) ds.y = 0.f;
                }
                d[i] = pack2(ds.x, ds.y);
            }
            tmem_st_32x32(t_row, d);             // over the first 32 of the 64 fp32 columns this thread just read
            tmem_wait_st();
            fence_before_sync();
            mbar_arrive(ds_full);
        }
        bf16* dst = p.dq + ((size_t)(q_begin + qi) * p.Nq + head) * p.D + half * 64;
        if (ok && n_kv > 0 && mbar_wait(dq_full, 0, abort_flag)) {
            fence_after_sync();
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t d[32];
                tmem_ld_32x32(tdQ + half * 64 + lane_off + c * 32, d);
                tmem_wait_ld();
                if (row_ok) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint4 w;
                        w.x = pack2(__uint_as_float(d[g * 8 + 0]) * p.scale, __uint_as_float(d[g * 8 + 1]) * p.scale);
                        w.y = pack2(__uint_as_float(d[g * 8 + 2]) * p.scale, __uint_as_float(d[g * 8 + 3]) * p.scale);
                        w.z = pack2(__uint_as_float(d[g * 8 + 4]) * p.scale, __uint_as_float(d[g * 8 + 5]) * p.scale);
                        w.w = pack2(__uint_as_float(d[g * 8 + 6]) * p.scale, __uint_as_float(d[g * 8 + 7]) * p.scale);
                        if (half * 64 + c * 32 + g * 8 < p.D) reinterpret_cast<uint4*>(dst)[c * 4 + g] = w;
                    }
                }
            }
        } else if (n_kv == 0 && row_ok) {
            for (int g = 0; g < 8; ++g)
                if (half * 64 + g * 8 < p.D) reinterpret_cast<uint4*>(dst)[g] = make_uint4(0, 0, 0, 0);
        }
        if (!ok && lane == 0) atomicExch(p.status, MM_TIMEOUT_EPI);
    }

    if (*abort_flag)
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

// ============================================================================================== dK, dV
constexpr int BQ2 = 64;
constexpr int kQTile = BQ2 * HD * 2;       // 16 KiB: a 64-row tile of Q / dO
constexpr int kQAtom = BQ2 * 128;          // 8 KiB
constexpr int kPTile = 128 * BQ2 * 2;      // 16 KiB: P^T / dS^T, one swizzle atom of 128 rows
constexpr int kRing = 4;                   // Q_i / dO_i ring depth (the TMEM buffers of S^T / dP^T stay double)
constexpr int kSmemDkv = 2 * kTile + 2 * kRing * kQTile + 2048 + 1024;

__global__ void __launch_bounds__(320, 1)
fmha_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, const BwdParams p) {
    if ((int)blockIdx.x >= *p.n_tiles) return;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sK = smem;
    uint8_t* sV = sK + kTile;
    uint8_t* sQ = sV + kTile;            // [kRing]
    uint8_t* sdO = sQ + kRing * kQTile;  // [kRing]
    float* s_lse = reinterpret_cast<float*>(sdO + kRing * kQTile);    // [2][64]
    float* s_dlt = s_lse + 2 * BQ2;                            // [2][64]
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_dlt + 2 * BQ2);
    uint64_t* kv_full = bars + 0;
    uint64_t* full = bars + 1;        // [kRing]  Q_i / dO_i landed
    uint64_t* empty = bars + 1 + kRing;   // [kRing]
    uint64_t* st_full = bars + 1 + 2 * kRing;     // [2]  S^T / dP^T ready
    uint64_t* st_empty = st_full + 2;             // [2]
    uint64_t* pds_full = st_full + 4;
    uint64_t* acc_full = st_full + 5;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(st_full + 6);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = p.tile_seq[blockIdx.x];
    const int kv0 = p.tile_r0[blockIdx.x];
    const int Gfull = p.Nq / p.Nkv;
    const int kv_head = p.split ? blockIdx.y / Gfull : blockIdx.y;
    const int head0 = p.split ? blockIdx.y : kv_head * Gfull;     // first query head this CTA walks
    const int G = p.split ? 1 : Gfull;                              // ... and how many
    const int out_heads = p.split ? p.Nq : p.Nkv, out_head = blockIdx.y;
    const int q_begin = p.cu_q[seq], q_len = p.cu_q[seq + 1] - q_begin;
    const int k_begin = p.cu_k[seq], k_len = p.cu_k[seq + 1] - k_begin;
    const int diag = k_len - q_len;
    const int nq = (q_len + BQ2 - 1) / BQ2;
    const int i_min = p.causal ? min(nq, max(0, kv0 - diag) / BQ2) : 0;
    const int per_head = nq - i_min;
    const int n_it = per_head * G;

    if (threadIdx.x == 0) {
        mbar_init(kv_full, 1);
        for (int i = 0; i < kRing; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&st_full[i], 1);
            mbar_init(&st_empty[i], 256);
        }
        mbar_init(pds_full, 256);
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmQ);
        prefetch_tmap(&tmK);
        prefetch_tmap(&tmV);
        prefetch_tmap(&tmdO);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tST = tmem_base, tdPT = tmem_base + 128, tdV = tmem_base + 256, tdK = tmem_base + 384;

    if (warp == 0) {
        if (lane == 0 && n_it > 0) {
            mbar_expect_tx(kv_full, 2 * kTile);
            tma_load_3d(sK, &tmK, kv_full, 0, kv_head, k_begin + kv0);
            tma_load_3d(sK + kAtom, &tmK, kv_full, 64, kv_head, k_begin + kv0);
            tma_load_3d(sV, &tmV, kv_full, 0, kv_head, k_begin + kv0);
            tma_load_3d(sV + kAtom, &tmV, kv_full, 64, kv_head, k_begin + kv0);
            for (int it = 0; it < n_it; ++it) {
                const int st = it % kRing;
                const uint32_t ph = (it / kRing) & 1;
                const int head = head0 + it / per_head;
                const int row = q_begin + (i_min + it % per_head) * BQ2;
                if (!mbar_wait(&empty[st], ph ^ 1, abort_flag)) { atomicExch(p.status, MM_TIMEOUT_TMA); break; }
                mbar_expect_tx(&full[st], 2 * kQTile);
                tma_load_3d(sQ + st * kQTile, &tmQ, &full[st], 0, head, row);
                tma_load_3d(sQ + st * kQTile + kQAtom, &tmQ, &full[st], 64, head, row);
                tma_load_3d(sdO + st * kQTile, &tmdO, &full[st], 0, head, row);
                tma_load_3d(sdO + st * kQTile + kQAtom, &tmdO, &full[st], 64, head, row);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && n_it > 0) {
            constexpr uint32_t idesc_t = idesc_bf16(128, BQ2, 0, 0);       // S^T, dP^T: N = 64 query rows
            constexpr uint32_t idesc_acc = idesc_bf16(128, 128, 0, 1);     // dV, dK: B = dO_i / Q_i as [N = d, K = q]
            bool ok = mbar_wait(kv_full, 0, abort_flag);
            const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
            auto issue_t = [&](int it) -> bool {
                const int st = it & 1, rs = it % kRing;
                const uint32_t ph = (it >> 1) & 1, rph = (it / kRing) & 1;
                if (!mbar_wait(&st_empty[st], ph ^ 1, abort_flag) || !mbar_wait(&full[rs], rph, abort_flag)) return false;
                fence_after_sync();
                const uint32_t qa = smem_u32(sQ + rs * kQTile), doa = smem_u32(sdO + rs * kQTile);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t aoff = (k >> 2) * kAtom + (k & 3) * 32;
                    const uint32_t boff = (k >> 2) * kQAtom + (k & 3) * 32;
                    mma_ss(tST + st * BQ2, smem_desc_sw128(ka + aoff, 16, 1024), smem_desc_sw128(qa + boff, 16, 1024), idesc_t,
                           k ? 1u : 0u);
                    mma_ss(tdPT + st * BQ2, smem_desc_sw128(va + aoff, 16, 1024), smem_desc_sw128(doa + boff, 16, 1024), idesc_t,
                           k ? 1u : 0u);
                }
                mma_commit(&st_full[st]);
                return true;
            };
            if (ok) ok = issue_t(0);
            for (int it = 0; it < n_it && ok; ++it) {
                const int rs = it % kRing;
                if (it + 1 < n_it && !(ok = issue_t(it + 1))) break;
                if (!mbar_wait(pds_full, it & 1, abort_flag)) { ok = false; break; }
                fence_after_sync();
                const uint32_t qa = smem_u32(sQ + rs * kQTile), doa = smem_u32(sdO + rs * kQTile);
                // P^T / dS^T sit in the S^T / dP^T columns the row threads emptied (queries 0..31 in columns 0..15,
                // queries 32..63 in columns 32..47, bf16 pairs): TS-form products, no shared-memory round trip
                const int sb = it & 1;
#pragma unroll
                for (int k = 0; k < BQ2 / 16; ++k) {
                    const uint32_t acol = sb * BQ2 + (k >> 1) * 32 + (k & 1) * 8;
                    mma_ts(tdV, tST + acol, smem_desc_sw128(doa + k * 2048, kQAtom, 1024), idesc_acc, (it | k) ? 1u : 0u);
                    mma_ts(tdK, tdPT + acol, smem_desc_sw128(qa + k * 2048, kQAtom, 1024), idesc_acc, (it | k) ? 1u : 0u);
                }
                mma_commit(&empty[rs]);
            }
            if (ok) mma_commit(acc_full);
            if (!ok) atomicExch(p.status, MM_TIMEOUT_MMA);
        }
    } else {
        // two warpgroups of 128 threads: both own all 128 key rows, each takes 32 of the 64 query columns of a tile
        const int half = (warp - 2) >> 2;
        const int qd = warp & 3;
        const int row = qd * 32 + lane;                  // key row inside the tile
        const int tid2 = (warp - 2) * 32 + lane;         // 0..255
        const int kj = kv0 + row;                        // key index inside its sequence
        const bool row_ok = kj < k_len;
        const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
        // per-column statistics (lse for threads 0..63, delta for 64..127) are fetched one tile ahead
        auto load_stat = [&](int it) -> float {
            if (tid2 >= 128) return 0.f;
            const int head = head0 + it / per_head;
            const int qi = min((i_min + it % per_head) * BQ2 + (tid2 & 63), q_len - 1);
            const size_t idx = (size_t)head * p.T + q_begin + qi;
            return tid2 < 64 ? p.lse[idx] * kLog2e : p.delta[idx];
        };
        float pre = n_it > 0 ? load_stat(0) : 0.f;
        bool ok = true;
        for (int it = 0; it < n_it; ++it) {
            const int st = it & 1;
            const uint32_t ph = (it >> 1) & 1;
            const int qbase = (i_min + it % per_head) * BQ2;
            if (tid2 < 64) s_lse[st * BQ2 + tid2] = pre;
            else if (tid2 < 128) s_dlt[st * BQ2 + tid2 - 64] = pre;
            if (it + 1 < n_it) pre = load_stat(it + 1);
            asm volatile("bar.sync 1, 256;" ::: "memory");
            // a thread whose wait gave up keeps walking the loop for the named barrier above, so nobody waits for it
            if (ok && !mbar_wait(&st_full[st], ph, abort_flag)) ok = false;
            if (!ok) continue;
            fence_after_sync();
            uint32_t s[32], d[32];
            tmem_ld_32x32(tST + st * BQ2 + half * 32 + lane_off, s);
            tmem_ld_32x32(tdPT + st * BQ2 + half * 32 + lane_off, d);
            tmem_wait_ld();
            fence_before_sync();
            mbar_arrive(&st_empty[st]);
            // visible query columns for this key: qi < q_len and (not causal or kj <= qi + diag)
            const int c_lo = !row_ok ? BQ2 : (p.causal ? max(0, kj - diag - qbase) : 0);
            const int c_hi = min(BQ2, q_len - qbase);
            const float* ls = s_lse + st * BQ2 + half * 32;
            const float* dl = s_dlt + st * BQ2 + half * 32;
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                const int cc = half * 32 + c;
                const float pr = exp2f(__uint_as_float(s[c]) * p.scale_log2 - ls[c]);
                const float pv = (cc >= c_lo && cc < c_hi) ? pr : 0.f;
                s[c] = __float_as_uint(pv);
                d[c] = __float_as_uint(pv * (__uint_as_float(d[c]) - dl[c]));
            }
            uint32_t pw[16], dw[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                pw[i] = pack2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1]));
                dw[i] = pack2(__uint_as_float(d[2 * i]), __uint_as_float(d[2 * i + 1]));
            }
            // over the first 16 of the 32 fp32 columns this thread has just read from each accumulator
            tmem_st_32x16(tST + st * BQ2 + half * 32 + lane_off, pw);
            tmem_st_32x16(tdPT + st * BQ2 + half * 32 + lane_off, dw);
            tmem_wait_st();
            fence_before_sync();
            mbar_arrive(pds_full);
        }
        bf16* dvp = p.dv + ((size_t)(k_begin + kj) * out_heads + out_head) * p.D + half * 64;
        bf16* dkp = p.dk + ((size_t)(k_begin + kj) * out_heads + out_head) * p.D + half * 64;
        if (ok && n_it > 0 && mbar_wait(acc_full, 0, abort_flag)) {
            fence_after_sync();
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t a[32], b[32];
                tmem_ld_32x32(tdV + half * 64 + lane_off + c * 32, a);
                tmem_ld_32x32(tdK + half * 64 + lane_off + c * 32, b);
                tmem_wait_ld();
                if (row_ok) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint4 w, x;
                        w.x = pack2(__uint_as_float(a[g * 8 + 0]), __uint_as_float(a[g * 8 + 1]));
                        w.y = pack2(__uint_as_float(a[g * 8 + 2]), __uint_as_float(a[g * 8 + 3]));
                        w.z = pack2(__uint_as_float(a[g * 8 + 4]), __uint_as_float(a[g * 8 + 5]));
                        w.w = pack2(__uint_as_float(a[g * 8 + 6]), __uint_as_float(a[g * 8 + 7]));
                        x.x = pack2(__uint_as_float(b[g * 8 + 0]) * p.scale, __uint_as_float(b[g * 8 + 1]) * p.scale);
                        x.y = pack2(__uint_as_float(b[g * 8 + 2]) * p.scale, __uint_as_float(b[g * 8 + 3]) * p.scale);
                        x.z = pack2(__uint_as_float(b[g * 8 + 4]) * p.scale, __uint_as_float(b[g * 8 + 5]) * p.scale);
                        x.w = pack2(__uint_as_float(b[g * 8 + 6]) * p.scale, __uint_as_float(b[g * 8 + 7]) * p.scale);
                        if (half * 64 + c * 32 + g * 8 < p.D) {
                            reinterpret_cast<uint4*>(dvp)[c * 4 + g] = w;
                            reinterpret_cast<uint4*>(dkp)[c * 4 + g] = x;
                        }
                    }
                }
            }
        } else if (n_it == 0 && row_ok) {
            for (int g = 0; g < 8; ++g)
                if (half * 64 + g * 8 < p.D) {
                    reinterpret_cast<uint4*>(dvp)[g] = make_uint4(0, 0, 0, 0);
                    reinterpret_cast<uint4*>(dkp)[g] = make_uint4(0, 0, 0, 0);
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
        tmem_dealloc(tmem_base, 512);
    }
}

#include "fmha_bwd_dkv128.cuh"

}  // namespace

// Scratch: plan = 2 * (2 * max_tiles + 1) ints with max_tiles = mm_fmha_bwd_max_tiles; delta = Nq * T floats.
MM_API int mm_fmha_bwd_max_tiles(int T, int n_seqs) { return T / 128 + n_seqs + 1; }

// q, dO, o: [T, Nq, D]; k, v: [Tk, Nkv, D] (token strides q_ts / k_ts / v_ts elements, heads dense; dO and o dense); D <= 128,
// a multiple of 8 (narrower heads read zeros beyond D through the tensor maps' out-of-range fill);
// lse: [Nq, T] fp32 from the forward; outputs dq [T, Nq, D], dk / dv [Tk, Nkv, D] dense bf16
// (split_heads = 1: dk / dv are per-query-head partials [Tk, Nq, D] that the caller sums over each GQA group).
// variant 0: dK/dV kernel over 64-row query steps (fallback); anything else: 128-row query steps (default).
MM_API int mm_fmha_bwd(const void* q, const void* k, const void* v, const void* o, const void* dO, const float* lse,
                       float* delta, void* dq, void* dk, void* dv, const int* cu_q, const int* cu_k, int* plan, int T, int Tk,
                       int n_seqs, int Nq, int Nkv, int D, long long q_ts, long long k_ts, long long v_ts, int causal,
                       float scale, int split_heads, int variant, int* status, cudaStream_t st) {
    if (D > HD || D < 8 || D % 8 || Nq % Nkv || (q_ts | k_ts | v_ts) % 8) return -1;
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o | (uintptr_t)dO | (uintptr_t)dq | (uintptr_t)dk |
         (uintptr_t)dv) & 15)
        return -2;
    const int mq = mm_fmha_bwd_max_tiles(T, n_seqs), mk = mm_fmha_bwd_max_tiles(Tk, n_seqs);
    int* q_seq = plan;
    int* q_r0 = plan + mq;
    int* q_n = plan + 2 * mq;
    int* k_seq = plan + 2 * mq + 1;
    int* k_r0 = k_seq + mk;
    int* k_n = k_seq + 2 * mk;
    int* q_nseq = k_n + 1;
    int* k_nseq = q_nseq + mq;
    // short sequences share a tile when the mask allows it: non-causal, keys and queries the same packed sequences
    const int pack = !causal && cu_q == cu_k && T == Tk && variant != 0;
    fmha_delta_kernel<<<(unsigned)(((long long)T * Nq + 7) / 8), 256, 0, st>>>((const bf16*)o, (const bf16*)dO, delta, T, Nq, D);
    fmha_bwd_plan_kernel<<<1, 32, 0, st>>>(cu_q, n_seqs, q_seq, q_r0, q_n, q_nseq, mq, 128, 1, pack);
    // early key tiles see the most query tiles under a causal mask: emit them first
    fmha_bwd_plan_kernel<<<1, 32, 0, st>>>(cu_k, n_seqs, k_seq, k_r0, k_n, k_nseq, mk, 128, 0, pack);
    CUtensorMap tQ, tK, tV, tdO, tQ64, tdO64;
    int r;
    if ((r = make_tmap_3d(&tQ, q, D, Nq, T, D, q_ts, 64, 1, 128))) return 1000 + r;
    if ((r = make_tmap_3d(&tK, k, D, Nkv, Tk, D, k_ts, 64, 1, 128))) return 2000 + r;
    if ((r = make_tmap_3d(&tV, v, D, Nkv, Tk, D, v_ts, 64, 1, 128))) return 3000 + r;
    if ((r = make_tmap_3d(&tdO, dO, D, Nq, T, D, (long long)Nq * D, 64, 1, 128))) return 4000 + r;
    if ((r = make_tmap_3d(&tQ64, q, D, Nq, T, D, q_ts, 64, 1, BQ2))) return 5000 + r;
    if ((r = make_tmap_3d(&tdO64, dO, D, Nq, T, D, (long long)Nq * D, 64, 1, BQ2))) return 6000 + r;
    if (cudaFuncSetAttribute(fmha_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemDq) != cudaSuccess) return -3;
    if (cudaFuncSetAttribute(fmha_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemDkv) != cudaSuccess) return -3;
    BwdParams p{cu_q, cu_k, q_seq, q_r0, q_nseq, q_n, lse, delta, (bf16*)dq, (bf16*)dk, (bf16*)dv, T, Tk, Nq, Nkv, causal, D, scale,
                scale * kLog2e, status, split_heads};
    BwdParams pk = p;
    pk.tile_seq = k_seq;
    pk.tile_r0 = k_r0;
    pk.tile_nseq = k_nseq;
    pk.n_tiles = k_n;
    fmha_bwd_dq_kernel<<<dim3(mq, Nq), 320, kSmemDq, st>>>(tQ, tK, tV, tdO, p);
    if (variant != 0) {      // dK/dV over 128-row query steps: all four products at N = 128
        if (cudaFuncSetAttribute(fmha_bwd_dkv128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemDkv128) != cudaSuccess)
            return -3;
        fmha_bwd_dkv128_kernel<<<dim3(mk, split_heads ? Nq : Nkv), 320, kSmemDkv128, st>>>(tQ, tK, tV, tdO, pk);
        return (int)cudaGetLastError();
    }
    fmha_bwd_dkv_kernel<<<dim3(mk, split_heads ? Nq : Nkv), 320, kSmemDkv, st>>>(tQ64, tK, tV, tdO64, pk);
    return (int)cudaGetLastError();
}
