// Flash attention forward on tcgen05 / TMEM / TMA: packed (varlen) sequences, GQA, optional causal mask,
// head dim <= 128 (multiple of 8), bf16 in / bf16 out + fp32 log-sum-exp (for ring merging and for the backward pass).
// Tiles are always 128 wide in shared memory: the tensor maps carry the true head dim, so for a narrower head (the
// vision tower's 80) the TMA boxes read zeros beyond it (out-of-range fill) and the stores skip those columns; nothing
// is padded in global memory.
//
// One CTA = one 128-row query tile of one head.  It walks the 128-key tiles of its sequence:
//   warp 0      TMA producer: Q once, then K_j / V_j into 3-stage rings (128B-swizzled boxes of 64 x 128)
//   warp 1      MMA issuer:   S_j = Q K_j^T  -> TMEM S[j&1]      (issued one tile ahead of the softmax)
//                             O_j = P_j V_j  -> TMEM O[j&1]      (fresh accumulator per tile; P_j is the A operand
//                                                                 read from tensor memory)
//   warps 2-5   softmax:      thread = query row; pulls its 128-column row of S into registers in one go, writes
//                             P_j (bf16 pairs) back over the first 64 columns of S[j&1], keeps m / l
//   warps 6-9   accumulate:   O_acc = O_acc * 2^(m_old - m_new) + O_j in registers (reads O_j from TMEM),
//                             final normalise, bf16 store
// TMEM: S double buffer (2 x 128 cols) + O double buffer (2 x 128 cols) = 512 columns.
// Rescaling lives in registers, so TMEM is never read-modify-written and the tensor core runs QK of tile j+1
// while the softmax of tile j is in flight.  All mbarrier waits are bounded (tc05::mbar_wait).
#include "tc05.cuh"

namespace {

using namespace tc05;

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int kThreads = 320;
constexpr int kTileBytes = BQ * HD * 2;   // 32 KiB: Q, K, V and P tiles all have this size
constexpr int kAtomBytes = 128 * 128;     // one 64-element-wide swizzle atom of 128 rows
constexpr int kRing = 3;                  // K and V ring depth
constexpr int kSmem = (1 + 2 * kRing) * kTileBytes + 2048 + 1024;   // Q + 3K + 3V + (barriers, alpha ring, l) + align = 227 KB

struct FmhaParams {
    const int* cu_q;
    const int* cu_k;
    const int* tile_seq;
    const int* tile_q0;
    const int* n_tiles;
    const int* tile_nseq;   // sequences covered by each tile (> 1: packed short sequences, block-diagonal mask)
    bf16* o;
    float* lse;         // [Nq, T]
    int T, Nq, Nkv, causal;
    int D;              // head dim of the tensors in global memory (<= HD)
    float scale_log2;   // softmax scale * log2(e)
    int* status;
};

__global__ void fmha_plan_kernel(const int* cu_q, int n_seqs, int* tile_seq, int* tile_q0, int* n_tiles, int* tile_nseq,
                                 int max_tiles, int pack) {
    if (threadIdx.x || blockIdx.x) return;
    if (pack) {          // non-causal self-attention: short sequences share tiles (all tiles cost about the same)
        int n = 0;
        for (int b = 0; b < n_seqs && n < max_tiles;) b = plan_packed(cu_q, n_seqs, b, BQ, tile_seq, tile_q0, tile_nseq, n, max_tiles);
        *n_tiles = n;
        return;
    }
    // Later query tiles of a causal sequence have more key tiles: emit them first so the tail of the grid is
    // made of short work items.
    int n = 0, longest = 0;
    for (int b = 0; b < n_seqs; ++b) longest = max(longest, cu_q[b + 1] - cu_q[b]);
    for (int t = (longest + BQ - 1) / BQ - 1; t >= 0; --t)
        for (int b = 0; b < n_seqs && n < max_tiles; ++b)
            if (t * BQ < cu_q[b + 1] - cu_q[b]) {
                tile_seq[n] = b;
                tile_q0[n] = t * BQ;
                tile_nseq[n] = 1;
                ++n;
            }
    *n_tiles = n;
}

__global__ void __launch_bounds__(kThreads, 1)
fmha_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, FmhaParams p) {
    if ((int)blockIdx.x >= *p.n_tiles) return;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + kTileBytes;
    uint8_t* sV = sK + kRing * kTileBytes;
    uint8_t* aux = sV + kRing * kTileBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(aux);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;    // [kRing]
    uint64_t* k_empty = bars + 4;   // [kRing]
    uint64_t* v_full = bars + 7;    // [kRing]
    uint64_t* v_empty = bars + 10;  // [kRing]
    uint64_t* s_full = bars + 13;   // [2]
    uint64_t* p_full = bars + 15;   // [2]
    uint64_t* o_full = bars + 17;   // [2]
    uint64_t* o_empty = bars + 19;  // [2]
    uint64_t* fin = bars + 21;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 22);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* alpha_ring = reinterpret_cast<float*>(aux + 256);   // [2][128]
    float* l_final = alpha_ring + 2 * 128;                      // [128]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = p.tile_seq[blockIdx.x];
    const int q0 = p.tile_q0[blockIdx.x];
    const int head = blockIdx.y;
    const int kv_head = head / (p.Nq / p.Nkv);
    const int q_begin = p.cu_q[seq], q_len = p.cu_q[seq + 1] - q_begin;
    const int k_begin = p.cu_k[seq], k_len = p.cu_k[seq + 1] - k_begin;
    const int diag = k_len - q_len;   // causal: key j visible to query i iff j <= i + diag
    int kv_end = k_len;
    if (p.causal) kv_end = min(k_len, q0 + BQ + diag);
    const int n_kv = (kv_end + BKV - 1) / BKV;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < kRing; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 128);
            mbar_init(&o_full[i], 1);
            mbar_init(&o_empty[i], 128);
        }
        mbar_init(fin, 128);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmQ);
        prefetch_tmap(&tmK);
        prefetch_tmap(&tmV);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tS = tmem_base, tO = tmem_base + 256;

    if (warp == 0) {
        // ------------------------------------------------------------------------------ TMA producer
        if (lane == 0 && n_kv > 0) {
            mbar_expect_tx(q_full, kTileBytes);
            tma_load_3d(sQ, &tmQ, q_full, 0, head, q_begin + q0);
            tma_load_3d(sQ + kAtomBytes, &tmQ, q_full, 64, head, q_begin + q0);
            for (int j = 0; j < n_kv; ++j) {
                const int st = j % kRing;
                const uint32_t ph = (j / kRing) & 1;
                const int row = k_begin + j * BKV;
                if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag)) { atomicExch(p.status, MM_TIMEOUT_TMA); break; }
                mbar_expect_tx(&k_full[st], kTileBytes);
                tma_load_3d(sK + st * kTileBytes, &tmK, &k_full[st], 0, kv_head, row);
                tma_load_3d(sK + st * kTileBytes + kAtomBytes, &tmK, &k_full[st], 64, kv_head, row);
                if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag)) { atomicExch(p.status, MM_TIMEOUT_TMA); break; }
                mbar_expect_tx(&v_full[st], kTileBytes);
                tma_load_3d(sV + st * kTileBytes, &tmV, &v_full[st], 0, kv_head, row);
                tma_load_3d(sV + st * kTileBytes + kAtomBytes, &tmV, &v_full[st], 64, kv_head, row);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------------------ MMA issuer
        if (lane == 0 && n_kv > 0) {
            constexpr uint32_t idesc_qk = idesc_bf16(BQ, BKV, 0, 0);
            constexpr uint32_t idesc_pv = idesc_bf16(BQ, HD, 0, 1);
            bool ok = mbar_wait(q_full, 0, abort_flag);
            auto issue_qk = [&](int j) -> bool {
                // S[j & 1] was last read by the PV product of tile j - 2 (as P), which this thread issued earlier:
                // the tensor pipe runs its instructions in order, so no barrier guards the overwrite.
                const int st = j & 1, rs = j % kRing;
                if (!mbar_wait(&k_full[rs], (j / kRing) & 1, abort_flag)) return false;
                fence_after_sync();
                const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + rs * kTileBytes);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (k >> 2) * kAtomBytes + (k & 3) * 32;
                    mma_ss(tS + st * 128, smem_desc_sw128(qa + off, 16, 1024), smem_desc_sw128(ka + off, 16, 1024),
                           idesc_qk, k ? 1u : 0u);
                }
                mma_commit(&s_full[st]);
                mma_commit(&k_empty[rs]);
                return true;
            };
            if (ok) ok = issue_qk(0);
            for (int j = 0; j < n_kv && ok; ++j) {
                if (j + 1 < n_kv) ok = issue_qk(j + 1);
                if (!ok) break;
                const int st = j & 1, rs = j % kRing;
                const uint32_t ph = (j >> 1) & 1;
                if (!mbar_wait(&o_empty[st], ph ^ 1, abort_flag) || !mbar_wait(&v_full[rs], (j / kRing) & 1, abort_flag) ||
                    !mbar_wait(&p_full[st], ph, abort_flag)) { ok = false; break; }
                fence_after_sync();
                // P comes from tensor memory: bf16 pairs in the first 64 columns of S[st], 8 columns per K = 16 step
                const uint32_t va = smem_u32(sV + rs * kTileBytes);
#pragma unroll
                for (int k = 0; k < BKV / 16; ++k) {
                    const uint64_t db = smem_desc_sw128(va + k * 2048, kAtomBytes, 1024);
                    mma_ts(tO + st * 128, tS + st * 128 + k * 8, db, idesc_pv, k ? 1u : 0u);
                }
                mma_commit(&o_full[st]);
                mma_commit(&v_empty[rs]);
            }
            if (!ok) atomicExch(p.status, MM_TIMEOUT_MMA);
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------------------------ softmax (warps 2..5)
        const int qd = warp & 3;
        const int row = qd * 32 + lane;
        const int qi = q0 + row;                         // query index inside its sequence
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_kv; ++j) {
            const int st = j & 1;
            const uint32_t ph = (j >> 1) & 1;
            if (!mbar_wait(&s_full[st], ph, abort_flag)) { ok = false; break; }
            fence_after_sync();
            const uint32_t t_row = tS + st * 128 + ((uint32_t)(qd * 32) << 16);
            const int kbase = j * BKV;
            const bool need_mask = (kbase + BKV > k_len) || (p.causal && kbase + BKV - 1 > q0 + diag);
            const int limit = p.causal ? min(k_len - 1, qi + diag) : k_len - 1;   // last visible key index
            // one TMEM round trip: the whole 128-column row of S lands in registers, then S[st] is released
            uint32_t r[128];
            tmem_ld_32x32(t_row, r);
            tmem_ld_32x32(t_row + 32, r + 32);
            tmem_ld_32x32(t_row + 64, r + 64);
            tmem_ld_32x32(t_row + 96, r + 96);
            tmem_wait_ld();
            float mx = -INFINITY;
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < 128; ++i) {
                    float s = __uint_as_float(r[i]) * p.scale_log2;
                    if (kbase + i > limit) s = -INFINITY;
                    r[i] = __float_as_uint(s);
                    mx = fmaxf(mx, s);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 128; ++i) {
                    const float s = __uint_as_float(r[i]) * p.scale_log2;
                    r[i] = __float_as_uint(s);
                    mx = fmaxf(mx, s);
                }
            }
            const float m_new = fmaxf(m, mx);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float alpha = exp2f(m - m_use);        // m = -inf on the first tile -> 0
            // The accumulate warps must be done with tile j - 2 before its alpha slot is reused and before
            // p_full[st], which they wait on too, can complete again.
            if (j >= 2 && !mbar_wait(&o_empty[st], ((j - 2) >> 1) & 1, abort_flag)) { ok = false; break; }
            alpha_ring[st * 128 + row] = alpha;
            m = m_new;
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < 128; ++i) {
                const float e = exp2f(__uint_as_float(r[i]) - m_use);
                sum += e;
                r[i] = __float_as_uint(e);
            }
            l = l * alpha + sum;
            // P goes back into tensor memory as bf16 pairs over the first 64 columns of the S buffer just read; the
            // PV product takes it from there as its A operand.
#pragma unroll
            for (int i = 0; i < 64; ++i) {
                bf162 t = __floats2bfloat162_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                r[i] = *reinterpret_cast<uint32_t*>(&t);
            }
            tmem_st_32x32(t_row, r);
            tmem_st_32x32(t_row + 32, r + 32);
            tmem_wait_st();
            fence_before_sync();
            mbar_arrive(&p_full[st]);
        }
        l_final[row] = l;
        if (ok && qi < q_len && n_kv > 0)
            p.lse[(size_t)head * p.T + q_begin + qi] = (m == -INFINITY) ? -INFINITY : m * 0.6931471805599453f + logf(l);
        mbar_arrive(fin);
        if (!ok && lane == 0) atomicExch(p.status, MM_TIMEOUT_EPI);
    } else {
        // ------------------------------------------------------------------------------ accumulate (warps 6..9)
        const int qd = warp & 3;
        const int row = qd * 32 + lane;
        const int qi = q0 + row;
        float acc[HD];
#pragma unroll
        for (int i = 0; i < HD; ++i) acc[i] = 0.f;
        bool ok = true;
        for (int j = 0; j < n_kv; ++j) {
            const int st = j & 1;
            const uint32_t ph = (j >> 1) & 1;
            if (!mbar_wait(&p_full[st], ph, abort_flag) || !mbar_wait(&o_full[st], ph, abort_flag)) { ok = false; break; }
            fence_after_sync();
            const float alpha = alpha_ring[st * 128 + row];
            const uint32_t t_row = tO + st * 128 + ((uint32_t)(qd * 32) << 16);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t r[64];
                tmem_ld_32x32(t_row + c * 64, r);
                tmem_ld_32x32(t_row + c * 64 + 32, r + 32);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 64; ++i) acc[c * 64 + i] = acc[c * 64 + i] * alpha + __uint_as_float(r[i]);
            }
            fence_before_sync();
            mbar_arrive(&o_empty[st]);
        }
        if (ok && mbar_wait(fin, 0, abort_flag) && qi < q_len && n_kv > 0) {
            const float lsum = l_final[row];
            const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
            bf16* dst = p.o + ((size_t)(q_begin + qi) * p.Nq + head) * p.D;
#pragma unroll
            for (int g = 0; g < HD / 8; ++g) {
                if (g * 8 >= p.D) break;
                float f[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = acc[g * 8 + i] * inv;
                reinterpret_cast<Vec8*>(dst)[g] = pack8(f);
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

#include "fmha_fwd_split.cuh"

int g_fwd_variant = 0;   // 0: one softmax warpgroup; 1 / 2: split-softmax kernel with 2 / 4 compute warpgroups (fmha_fwd_split.cuh)

}  // namespace

// Selects the forward kernel for later calls (0 = default, 1 = split softmax).  Returns the previous value.
MM_API int mm_fmha_set_fwd_variant(int v) {
    const int prev = g_fwd_variant;
    g_fwd_variant = v;
    return prev;
}

// Scratch needed by the planner: 3 * max_tiles + 1 ints, max_tiles = T / 128 + n_seqs + 1.
MM_API int mm_fmha_max_tiles(int T, int n_seqs) { return T / BQ + n_seqs + 1; }

// q: [T, Nq, D] with q_ts elements between tokens (heads dense); k, v: [T, Nkv, D] likewise; o: [T, Nq, D]
// dense; lse: [Nq, T] fp32; cu_q / cu_k: int32 [n_seqs + 1] on the device; plan: int32 scratch (see above).
MM_API int mm_fmha_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu_q, const int* cu_k,
                       int* plan, int T, int Tk, int n_seqs, int Nq, int Nkv, int D, long long q_ts, long long k_ts,
                       long long v_ts, int causal, float scale, int* status, cudaStream_t st) {
    if (D > HD || D < 8 || D % 8 || Nq % Nkv || (q_ts | k_ts | v_ts) % 8) return -1;
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o) & 15) return -2;
    const int max_tiles = mm_fmha_max_tiles(T, n_seqs);
    int* tile_seq = plan;
    int* tile_q0 = plan + max_tiles;
    int* n_tiles = plan + 2 * max_tiles;
    int* tile_nseq = plan + 2 * max_tiles + 1;
    // short sequences share a tile when the mask allows it: non-causal, keys and queries the same packed sequences
    const int pack = !causal && cu_q == cu_k && T == Tk && g_fwd_variant != 0;
    fmha_plan_kernel<<<1, 32, 0, st>>>(cu_q, n_seqs, tile_seq, tile_q0, n_tiles, tile_nseq, max_tiles, pack);
    CUtensorMap tQ, tK, tV;
    int r;
    if ((r = make_tmap_3d(&tQ, q, D, Nq, T, D, q_ts, 64, 1, BQ))) return 1000 + r;
    if ((r = make_tmap_3d(&tK, k, D, Nkv, Tk, D, k_ts, 64, 1, BKV))) return 2000 + r;
    if ((r = make_tmap_3d(&tV, v, D, Nkv, Tk, D, v_ts, 64, 1, BKV))) return 3000 + r;
    static bool done = false;
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(fmha_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(fmha_fwd_split_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);

        if (e != cudaSuccess) return (int)e;
        done = true;
    }
    FmhaParams p{cu_q, cu_k, tile_seq, tile_q0, n_tiles, tile_nseq, (bf16*)o, lse, T, Nq, Nkv, causal, D,
                 scale * 1.4426950408889634f, status};
    dim3 grid(max_tiles, Nq);
    if (g_fwd_variant == 0)      // fallback: one softmax warpgroup, O folded in registers
        fmha_fwd_kernel<<<grid, kThreads, kSmem, st>>>(tQ, tK, tV, p);
    else                         // default: split softmax, O accumulated in tensor memory with lazy rescaling
        fmha_fwd_split_kernel<2, true><<<grid, 64 + 256, kSmem, st>>>(tQ, tK, tV, p);
    return (int)cudaGetLastError();
}
