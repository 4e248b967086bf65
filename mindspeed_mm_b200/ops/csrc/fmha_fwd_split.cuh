// Forward flash-attention kernel, "split" variant: included by fmha_fwd.cu inside its namespace (shares FmhaParams, the
// tile constants and the planner with the default kernel).
//
// Same producer / MMA-issuer warps and TMEM layout as the default kernel, but both compute warpgroups run the softmax:
//   warps 2-9   thread = (query row, half): warpgroup h owns key columns [64h, 64h+64) of S and head-dim columns
//               [64h, 64h+64) of O.  Per tile: pull its 64 columns of S, exchange the row maximum with the other half
//               through a shared-memory atomic max + one named barrier, exp2, write P_j (bf16 pairs) back over the
//               first 64 columns of S[j&1]; then fold O_{j-1} into its register accumulator.
// Two warps per scheduler hide each other's TMEM / special-function latency, and the exp2 work of a tile (16384 per
// 128 x 128) is spread over 256 threads.  A thread whose bounded wait gave up keeps taking part in the named barriers,
// so nobody is left waiting for it.

constexpr int kOrdNegInf = (int)0x807fffff;   // float_to_ordered(-inf)

// Order-preserving map float -> int (so that an integer atomic max is a float max) and back.
__device__ __forceinline__ int float_to_ordered(float f) {
    const int i = __float_as_int(f);
    return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float ordered_to_float(int i) { return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff); }

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ void named_barrier_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// PARTS compute warpgroups (2 or 4): each owns 128 / PARTS key columns of S and as many head-dim columns of O.
// LAZY: O is accumulated across key tiles by the tensor core itself (one TMEM accumulator, no per-tile fold in
// registers).  The reference maximum of a row is only moved when the running maximum has grown by more than 2^8
// since it was set; only then the row threads rescale their O columns in tensor memory (rare after the first tiles).
// P = exp2(S * scale - m_ref) is therefore at most 2^8, well inside bf16 / fp32 range, and the result is exact because
// l, the LSE and O all refer to the same m_ref.
template <int PARTS, bool LAZY = false>
__global__ void __launch_bounds__(64 + 128 * PARTS, 1)
fmha_fwd_split_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
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
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* maxbuf = reinterpret_cast<int*>(aux + 256);            // [3][128] row maxima as ordered ints, rotating
    float* l_sum = reinterpret_cast<float*>(aux + 256);         // [128], reuses maxbuf after the key loop
    constexpr int C = 128 / PARTS;                               // columns per compute thread
    constexpr int kCompute = 128 * PARTS;                        // compute threads
    constexpr int kAll = 64 + kCompute;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = p.tile_seq[blockIdx.x];
    const int q0 = p.tile_q0[blockIdx.x];
    const int head = blockIdx.y;
    const int kv_head = head / (p.Nq / p.Nkv);
    const int nseq = p.tile_nseq[blockIdx.x];          // > 1: consecutive short sequences packed into this tile
    const int q_begin = p.cu_q[seq], q_len = p.cu_q[seq + nseq] - q_begin;
    const int k_begin = p.cu_k[seq], k_len = p.cu_k[seq + nseq] - k_begin;
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
            mbar_init(&p_full[i], kCompute);
            mbar_init(&o_full[i], 1);
            mbar_init(&o_empty[i], kCompute);
        }
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
    for (int i = threadIdx.x; i < 3 * 128; i += kAll) maxbuf[i] = kOrdNegInf;
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
                if ((!LAZY && !mbar_wait(&o_empty[st], ph ^ 1, abort_flag)) || !mbar_wait(&v_full[rs], (j / kRing) & 1, abort_flag) ||
                    !mbar_wait(&p_full[st], ph, abort_flag)) { ok = false; break; }
                fence_after_sync();
                // P comes from tensor memory: bf16 pairs in the first 64 columns of S[st], 8 columns per K = 16 step
                const uint32_t va = smem_u32(sV + rs * kTileBytes);
#pragma unroll
                for (int k = 0; k < BKV / 16; ++k) {
                    const uint64_t db = smem_desc_sw128(va + k * 2048, kAtomBytes, 1024);
                    if constexpr (LAZY) mma_ts(tO, tS + st * 128 + k * 8, db, idesc_pv, (j | k) ? 1u : 0u);
                    else mma_ts(tO + st * 128, tS + st * 128 + k * 8, db, idesc_pv, k ? 1u : 0u);
                }
                mma_commit(&o_full[st]);
                mma_commit(&v_empty[rs]);
            }
            if (!ok) atomicExch(p.status, MM_TIMEOUT_MMA);
        }
    } else {
        // ------------------------------------------------------------------------------ compute (warps 2..9)
        const int half = (warp - 2) >> 2;                // which C key columns of S / C head-dim columns of O
        const int qd = warp & 3;                         // TMEM lane quarter this warp may touch
        const int row = qd * 32 + lane;
        const int qi = q0 + row;                         // query index inside its sequence
        const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
        int vis_lo = 0, vis_hi = k_len;                  // keys this row may see (packed tiles: its own sequence)
        if (nseq > 1) packed_row_range(p.cu_q, seq, nseq, q_begin + qi, q_begin, vis_lo, vis_hi);
        float m = -INFINITY, l = 0.f, alpha_pending = 0.f;
        float acc[C];
#pragma unroll
        for (int i = 0; i < C; ++i) acc[i] = 0.f;
        bool ok = true;
        auto fold = [&](int jj) {                        // O_acc = O_acc * alpha_jj + O_jj for this thread's 64 columns
            const int sb = jj & 1;
            if (ok && !mbar_wait(&o_full[sb], (jj >> 1) & 1, abort_flag)) ok = false;
            if (!ok) return;
            fence_after_sync();
            uint32_t o[C];
            const uint32_t t_o = tO + sb * 128 + half * C + lane_off;
            tmem_ld_32x32(t_o, o);
            if constexpr (C == 64) tmem_ld_32x32(t_o + 32, o + 32);
            tmem_wait_ld();
            fence_before_sync();
            mbar_arrive(&o_empty[sb]);
            const float2 a2 = make_float2(alpha_pending, alpha_pending);
#pragma unroll
            for (int i = 0; i < C / 2; ++i) {             // packed fp32: one instruction per two columns
                const float2 v = __ffma2_rn(make_float2(acc[2 * i], acc[2 * i + 1]), a2,
                                            make_float2(__uint_as_float(o[2 * i]), __uint_as_float(o[2 * i + 1])));
                acc[2 * i] = v.x;
                acc[2 * i + 1] = v.y;
            }
        };
        for (int j = 0; j < n_kv; ++j) {
            const int st = j & 1;
            const uint32_t ph = (j >> 1) & 1;
            if (ok && !mbar_wait(&s_full[st], ph, abort_flag)) ok = false;
            uint32_t r[C];
            const uint32_t t_s = tS + st * 128 + lane_off;
            const int kbase = j * BKV + half * C;
            if (ok) {
                fence_after_sync();
                tmem_ld_32x32(t_s + half * C, r);
                if constexpr (C == 64) tmem_ld_32x32(t_s + half * C + 32, r + 32);
                tmem_wait_ld();
                const bool need_mask = (kbase + C > k_len) || (p.causal && kbase + C - 1 > q0 + diag) || nseq > 1;
                const int limit = p.causal ? min(k_len - 1, qi + diag) : vis_hi - 1;  // last visible key index
                // the maximum is taken over the raw scores (the softmax scale is positive); scale and shift are folded
                // into one fused multiply-add in front of the exponential
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < C; ++i)
                        if (kbase + i > limit || kbase + i < vis_lo) r[i] = 0xff800000u;       // -inf
                }
                float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
                for (int i = 0; i < C; i += 8) {          // four independent chains of three-input maxima
                    mx0 = max3(mx0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                    mx1 = max3(mx1, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
                    mx2 = max3(mx2, __uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
                    mx3 = max3(mx3, __uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
                }
                const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
                atomicMax(&maxbuf[(j % 3) * 128 + row], float_to_ordered(mx));
            }
            // Both halves of every row have read their S columns and published their maximum.  After this barrier
            // the P columns may overwrite S, and the slot of tile j - 1 (next used by tile j + 2) may be reset.
            named_barrier_sync(1, kCompute);
            if (half == 0) maxbuf[((j + 2) % 3) * 128 + row] = kOrdNegInf;
            if (ok) {
                const float mx_all = ordered_to_float(maxbuf[(j % 3) * 128 + row]);
                float m_new = fmaxf(m, mx_all);
                if constexpr (LAZY) {
                    const bool grow = m_new > m + 8.f;           // also true for the first finite maximum (m = -inf)
                    if (!grow) m_new = m;
                    if (__any_sync(__activemask(), grow) && j > 0) {
                        // rescale this thread's O columns in tensor memory; PV_{j-1} must have landed, PV_j is not issued
                        // before every thread has arrived on p_full
                        const int sb = (j - 1) & 1;
                        if (!mbar_wait(&o_full[sb], ((j - 1) >> 1) & 1, abort_flag)) ok = false;
                        if (ok) {
                            fence_after_sync();
                            const float a = grow ? exp2f(m - (m_new == -INFINITY ? 0.f : m_new)) : 1.f;
                            const float2 a2 = make_float2(a, a);
                            uint32_t o[C];
                            const uint32_t t_o = tO + half * C + lane_off;
                            tmem_ld_32x32(t_o, o);
                            if constexpr (C == 64) tmem_ld_32x32(t_o + 32, o + 32);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < C / 2; ++i) {
                                const float2 v = __fmul2_rn(make_float2(__uint_as_float(o[2 * i]), __uint_as_float(o[2 * i + 1])), a2);
                                o[2 * i] = __float_as_uint(v.x);
                                o[2 * i + 1] = __float_as_uint(v.y);
                            }
                            tmem_st_32x32(t_o, o);
                            if constexpr (C == 64) tmem_st_32x32(t_o + 32, o + 32);
                            tmem_wait_st();
                        }
                    }
                }
                const float m_use = m_new == -INFINITY ? 0.f : m_new;
                const float alpha = exp2f(m - m_use);        // m = -inf on the first tile -> 0; 1 when the reference stays
                m = m_new;
                const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), ng2 = make_float2(-m_use, -m_use);
                float2 sum_a = make_float2(0.f, 0.f), sum_b = make_float2(0.f, 0.f);
#pragma unroll
                for (int i = 0; i < C / 2; i += 2) {      // two packed chains: exp2(s * scale - m), running sums, bf16 pairs
                    const float2 x0 = __ffma2_rn(make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])), sc2, ng2);
                    const float2 x1 = __ffma2_rn(make_float2(__uint_as_float(r[2 * i + 2]), __uint_as_float(r[2 * i + 3])), sc2, ng2);
                    const float2 e0 = make_float2(exp2f(x0.x), exp2f(x0.y));
                    const float2 e1 = make_float2(exp2f(x1.x), exp2f(x1.y));
                    sum_a = __fadd2_rn(sum_a, e0);
                    sum_b = __fadd2_rn(sum_b, e1);
                    bf162 t0 = __floats2bfloat162_rn(e0.x, e0.y), t1 = __floats2bfloat162_rn(e1.x, e1.y);
                    r[i] = *reinterpret_cast<uint32_t*>(&t0);
                    r[i + 1] = *reinterpret_cast<uint32_t*>(&t1);
                }
                l = l * alpha + ((sum_a.x + sum_a.y) + (sum_b.x + sum_b.y));
                // P: bf16 pairs over the first 64 columns of S[st]; this part's C keys are columns [C / 2 * part, + C / 2)
                if constexpr (C == 64) tmem_st_32x32(t_s + half * 32, r);
                else tmem_st_32x16(t_s + half * 16, r);
                tmem_wait_st();
                fence_before_sync();
                mbar_arrive(&p_full[st]);
                if constexpr (!LAZY) {
                    if (j > 0) fold(j - 1);                  // uses alpha of tile j - 1
                    alpha_pending = alpha;
                }
            }
        }
        if constexpr (LAZY) {
            // the accumulator of all tiles sits in tensor memory: take it once
            if (n_kv > 0) {
                const int sb = (n_kv - 1) & 1;
                if (ok && !mbar_wait(&o_full[sb], ((n_kv - 1) >> 1) & 1, abort_flag)) ok = false;
                if (ok) {
                    fence_after_sync();
                    uint32_t o[C];
                    const uint32_t t_o = tO + half * C + lane_off;
                    tmem_ld_32x32(t_o, o);
                    if constexpr (C == 64) tmem_ld_32x32(t_o + 32, o + 32);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < C; ++i) acc[i] = __uint_as_float(o[i]);
                }
            }
        } else {
            if (n_kv > 0) fold(n_kv - 1);
        }
        named_barrier_sync(1, kCompute);                     // maxbuf is free: reuse it for the row sums
        if (half == 0) l_sum[row] = 0.f;
        named_barrier_sync(1, kCompute);
        atomicAdd(&l_sum[row], l);
        named_barrier_sync(1, kCompute);
        if (ok && qi < q_len && n_kv > 0) {
            const float lsum = l_sum[row];
            const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
            if (half == 0)
                p.lse[(size_t)head * p.T + q_begin + qi] = (m == -INFINITY) ? -INFINITY : m * 0.6931471805599453f + logf(lsum);
            bf16* dst = p.o + ((size_t)(q_begin + qi) * p.Nq + head) * p.D + half * C;
#pragma unroll
            for (int g = 0; g < C / 8; ++g) {
                if (half * C + g * 8 >= p.D) break;
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

