// dK / dV backward kernel with 128-row query steps (variant 5 of mm_fmha_bwd); included by fmha_bwd.cu inside its
// namespace (shares BwdParams, the tile constants and pack2 with the default kernels).
//
// One CTA = one 128-row key tile of one KV head (or of one query head when p.split).  Per 128-row query tile i:
//     S^T_i  = K Q_i^T          128 x 128 x 128   SS   -> TMEM columns [0, 128)
//     dP^T_i = V dO_i^T         128 x 128 x 128   SS   -> TMEM columns [128, 256)
//     dV    += P^T_i  dO_i      128 x 128 x 128   TS   (P^T_i  written by the row threads over their own S^T columns)
//     dK    += dS^T_i Q_i       128 x 128 x 128   TS   (dS^T_i written over their own dP^T columns)
// All four products have N = 128, so every tcgen05.mma runs at the full 64 clocks (the 64-row steps of the default
// kernel pay 48 clocks for N = 64 products, i.e. 1.5x for S^T and dP^T) and the operand traffic from shared memory
// drops from 256 KB to 192 KB per 128 query rows.  S^T and dP^T are single-buffered; the tensor pipe is kept busy by the
// issue order   S_0 dP_0 | dV_i S_{i+1} dK_i dP_{i+1} | ...   in which the product that follows a wait never depends on
// the row threads' other phase: while they turn S_{i+1} into P_{i+1}, the pipe runs dK_i and dP_{i+1}; while they turn
// dP_{i+1} into dS_{i+1}, it runs dV_{i+1} and S_{i+2}.
//
//   warp 0      TMA: K, V once; Q_i into a 3-deep and dO_i into a 2-deep ring (Q is released by dK_i, dO by dV_i)
//   warp 1      MMA issuer
//   warps 2-9   row threads: thread = (key row, half): 64 of the 128 query columns.  Phase 1: P = exp2(S * scale -
//               lse), masked, kept in registers and written as bf16 pairs over the first 32 of its own 64 S^T columns.
//               Phase 2: dS = P * (dP - delta), written the same way over dP^T.
// TMEM: S^T 128 | dP^T 128 | dV 128 | dK 128 = 512 columns.  Every mbarrier wait is bounded; a thread whose wait gave
// up keeps taking part in the named barrier of the statistics exchange, so nobody is left waiting for it.

constexpr int kRingQ128 = 3;    // Q_i is needed first (S^T_i) and released last (dK_i): it gets the deeper ring
constexpr int kRingDO128 = 2;
constexpr int kSmemDkv128 = (2 + kRingQ128 + kRingDO128) * kTile + 2 * 128 * 4 + 256 + 1024;    // K, V, Q ring, dO ring, stats, barriers, align

__global__ void __launch_bounds__(320, 1)
fmha_bwd_dkv128_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, const BwdParams p) {
    if ((int)blockIdx.x >= *p.n_tiles) return;
    constexpr int BQ = 128;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sK = smem;
    uint8_t* sV = sK + kTile;
    uint8_t* sQ = sV + kTile;                     // [kRingQ128]
    uint8_t* sdO = sQ + kRingQ128 * kTile;        // [kRingDO128]
    float* s_lse = reinterpret_cast<float*>(sdO + kRingDO128 * kTile);     // [128]
    float* s_dlt = s_lse + BQ;                                              // [128]
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_dlt + BQ);
    uint64_t* kv_full = bars + 0;
    uint64_t* q_full = bars + 1;                  // [kRingQ128]
    uint64_t* q_empty = q_full + kRingQ128;       // [kRingQ128]
    uint64_t* do_full = q_empty + kRingQ128;      // [kRingDO128]
    uint64_t* do_empty = do_full + kRingDO128;    // [kRingDO128]
    uint64_t* s_full = do_empty + kRingDO128;
    uint64_t* dp_full = s_full + 1;
    uint64_t* p_full = s_full + 2;
    uint64_t* ds_full = s_full + 3;
    uint64_t* acc_full = s_full + 4;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 5);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = p.tile_seq[blockIdx.x];
    const int kv0 = p.tile_r0[blockIdx.x];
    const int Gfull = p.Nq / p.Nkv;
    const int kv_head = p.split ? blockIdx.y / Gfull : blockIdx.y;
    const int head0 = p.split ? blockIdx.y : kv_head * Gfull;
    const int G = p.split ? 1 : Gfull;
    const int out_heads = p.split ? p.Nq : p.Nkv, out_head = blockIdx.y;
    const int nseq = p.tile_nseq[blockIdx.x];          // > 1: consecutive short sequences packed into this tile
    const int q_begin = p.cu_q[seq], q_len = p.cu_q[seq + nseq] - q_begin;
    const int k_begin = p.cu_k[seq], k_len = p.cu_k[seq + nseq] - k_begin;
    const int diag = k_len - q_len;
    const int nq = (q_len + BQ - 1) / BQ;
    const int i_min = p.causal ? min(nq, max(0, kv0 - diag) / BQ) : 0;    // first query tile that can see this key tile
    const int per_head = nq - i_min;
    const int n_it = per_head * G;

    if (threadIdx.x == 0) {
        mbar_init(kv_full, 1);
        for (int i = 0; i < kRingQ128; ++i) {
            mbar_init(&q_full[i], 1);
            mbar_init(&q_empty[i], 1);
        }
        for (int i = 0; i < kRingDO128; ++i) {
            mbar_init(&do_full[i], 1);
            mbar_init(&do_empty[i], 1);
        }
        mbar_init(s_full, 1);
        mbar_init(dp_full, 1);
        mbar_init(p_full, 256);
        mbar_init(ds_full, 256);
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
        // ------------------------------------------------------------------------------ TMA producer
        if (lane == 0 && n_it > 0) {
            mbar_expect_tx(kv_full, 2 * kTile);
            tma_load_3d(sK, &tmK, kv_full, 0, kv_head, k_begin + kv0);
            tma_load_3d(sK + kAtom, &tmK, kv_full, 64, kv_head, k_begin + kv0);
            tma_load_3d(sV, &tmV, kv_full, 0, kv_head, k_begin + kv0);
            tma_load_3d(sV + kAtom, &tmV, kv_full, 64, kv_head, k_begin + kv0);
            for (int it = 0; it < n_it; ++it) {
                const int qs = it % kRingQ128, ds = it % kRingDO128;
                const uint32_t qph = (it / kRingQ128) & 1, dph = (it / kRingDO128) & 1;
                const int head = head0 + it / per_head;
                const int row = q_begin + (i_min + it % per_head) * BQ;
                if (!mbar_wait(&q_empty[qs], qph ^ 1, abort_flag)) { atomicExch(p.status, MM_TIMEOUT_TMA); break; }
                mbar_expect_tx(&q_full[qs], kTile);
                tma_load_3d(sQ + qs * kTile, &tmQ, &q_full[qs], 0, head, row);
                tma_load_3d(sQ + qs * kTile + kAtom, &tmQ, &q_full[qs], 64, head, row);
                if (!mbar_wait(&do_empty[ds], dph ^ 1, abort_flag)) { atomicExch(p.status, MM_TIMEOUT_TMA); break; }
                mbar_expect_tx(&do_full[ds], kTile);
                tma_load_3d(sdO + ds * kTile, &tmdO, &do_full[ds], 0, head, row);
                tma_load_3d(sdO + ds * kTile + kAtom, &tmdO, &do_full[ds], 64, head, row);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------------------ MMA issuer
        if (lane == 0 && n_it > 0) {
            constexpr uint32_t idesc_t = idesc_bf16(128, 128, 0, 0);       // S^T, dP^T
            constexpr uint32_t idesc_acc = idesc_bf16(128, 128, 0, 1);     // dV, dK: B = dO_i / Q_i read as [N = d, K = q]
            bool ok = mbar_wait(kv_full, 0, abort_flag);
            const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
            auto issue_t = [&](int it, uint32_t a_base, const uint8_t* b_tiles, uint64_t* landed, int ring, uint32_t tdst,
                               uint64_t* done) -> bool {
                const int rs = it % ring;
                if (!mbar_wait(&landed[rs], (it / ring) & 1, abort_flag)) return false;
                fence_after_sync();
                const uint32_t ba = smem_u32(b_tiles + rs * kTile);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (k >> 2) * kAtom + (k & 3) * 32;
                    mma_ss(tdst, smem_desc_sw128(a_base + off, 16, 1024), smem_desc_sw128(ba + off, 16, 1024), idesc_t, k ? 1u : 0u);
                }
                mma_commit(done);
                return true;
            };
            // bf16 pairs of query columns [64 h, 64 h + 64) live in the first 32 columns of half h's 64-column region
            auto a_col = [](int k) -> uint32_t { return (uint32_t)((k >> 2) * 64 + (k & 3) * 8); };
            if (ok) ok = issue_t(0, ka, sQ, q_full, kRingQ128, tST, s_full);
            if (ok) ok = issue_t(0, va, sdO, do_full, kRingDO128, tdPT, dp_full);
            for (int it = 0; it < n_it && ok; ++it) {
                const int qs = it % kRingQ128, ds = it % kRingDO128;
                const uint32_t par = it & 1;
                if (!mbar_wait(p_full, par, abort_flag)) { ok = false; break; }
                fence_after_sync();
                const uint32_t doa = smem_u32(sdO + ds * kTile), qa = smem_u32(sQ + qs * kTile);
#pragma unroll
                for (int k = 0; k < BQ / 16; ++k)
                    mma_ts(tdV, tST + a_col(k), smem_desc_sw128(doa + k * 2048, kAtom, 1024), idesc_acc, (it | k) ? 1u : 0u);
                mma_commit(&do_empty[ds]);
                if (it + 1 < n_it && !(ok = issue_t(it + 1, ka, sQ, q_full, kRingQ128, tST, s_full))) break;
                if (!mbar_wait(ds_full, par, abort_flag)) { ok = false; break; }
                fence_after_sync();
#pragma unroll
                for (int k = 0; k < BQ / 16; ++k)
                    mma_ts(tdK, tdPT + a_col(k), smem_desc_sw128(qa + k * 2048, kAtom, 1024), idesc_acc, (it | k) ? 1u : 0u);
                mma_commit(&q_empty[qs]);
                if (it + 1 < n_it && !(ok = issue_t(it + 1, va, sdO, do_full, kRingDO128, tdPT, dp_full))) break;
            }
            if (ok) mma_commit(acc_full);
            if (!ok) atomicExch(p.status, MM_TIMEOUT_MMA);
        }
    } else {
        // ------------------------------------------------------------------------------ row threads (warps 2..9)
        const int half = (warp - 2) >> 2;
        const int qd = warp & 3;
        const int row = qd * 32 + lane;                  // key row inside the tile
        const int tid2 = (warp - 2) * 32 + lane;         // 0..255
        const int kj = kv0 + row;                        // key index inside its sequence
        const bool row_ok = kj < k_len;
        int vis_lo = 0, vis_hi = q_len;                  // queries that see this key (packed tiles: its own sequence)
        if (nseq > 1) packed_row_range(p.cu_k, seq, nseq, k_begin + kj, k_begin, vis_lo, vis_hi);
        const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
        // per-column statistics (lse from threads 0..127, delta from 128..255) are fetched one tile ahead
        auto load_stat = [&](int it) -> float {
            const int head = head0 + it / per_head;
            const int qi = min((i_min + it % per_head) * BQ + (tid2 & 127), q_len - 1);
            const size_t idx = (size_t)head * p.T + q_begin + qi;
            return tid2 < 128 ? p.lse[idx] * kLog2e : p.delta[idx];
        };
        float pre = n_it > 0 ? load_stat(0) : 0.f;
        bool ok = true;
        for (int it = 0; it < n_it; ++it) {
            const uint32_t par = it & 1;
            const int qbase = (i_min + it % per_head) * BQ;
            // the statistics buffer is single: everybody must be done with tile it - 1 before it is overwritten
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (tid2 < 128) s_lse[tid2] = pre;
            else s_dlt[tid2 - 128] = pre;
            if (it + 1 < n_it) pre = load_stat(it + 1);
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (ok && !mbar_wait(s_full, par, abort_flag)) ok = false;
            if (!ok) continue;
            fence_after_sync();
            uint32_t s[64];
            const uint32_t t_s = tST + half * 64 + lane_off, t_d = tdPT + half * 64 + lane_off;
            tmem_ld_32x32(t_s, s);
            tmem_ld_32x32(t_s + 32, s + 32);
            tmem_wait_ld();
            // visible query columns for this key: qi < q_len and (not causal or kj <= qi + diag)
            const int c_lo = !row_ok ? BQ : (p.causal ? max(0, kj - diag - qbase) : max(0, vis_lo - qbase));
            const int c_hi = min(BQ, vis_hi - qbase);
            const float* ls = s_lse + half * 64;
            const float* dl = s_dlt + half * 64;
            // packed fp32 math (two query columns per instruction): P = exp2(S^T * scale - lse)
            const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
            const bool col_masked = c_lo > half * 64 || c_hi < half * 64 + 64;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float2 x = __ffma2_rn(make_float2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1])), sc2,
                                            make_float2(-ls[2 * i], -ls[2 * i + 1]));
                float2 pr = make_float2(exp2f(x.x), exp2f(x.y));
                if (col_masked) {
                    const int cc = half * 64 + 2 * i;
                    if (cc < c_lo || cc >= c_hi) pr.x = 0.f;
                    if (cc + 1 < c_lo || cc + 1 >= c_hi) pr.y = 0.f;
                }
                s[2 * i] = __float_as_uint(pr.x);
                s[2 * i + 1] = __float_as_uint(pr.y);
            }
            {
                uint32_t pw[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) pw[i] = pack2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1]));
                tmem_st_32x32(t_s, pw);                  // over the first 32 of the 64 fp32 columns this thread has just read
                tmem_wait_st();
                fence_before_sync();
                mbar_arrive(p_full);
            }
            if (!mbar_wait(dp_full, par, abort_flag)) { ok = false; continue; }
            fence_after_sync();
            {
                uint32_t d[64];
                tmem_ld_32x32(t_d, d);
                tmem_ld_32x32(t_d + 32, d + 32);
                tmem_wait_ld();
                uint32_t dw[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {               // dS = P * (dP - delta)
                    const float2 g = __fadd2_rn(make_float2(__uint_as_float(d[2 * i]), __uint_as_float(d[2 * i + 1])),
                                                make_float2(-dl[2 * i], -dl[2 * i + 1]));
                    const float2 ds = __fmul2_rn(make_float2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1])), g);
                    dw[i] = pack2(ds.x, ds.y);
                }
                tmem_st_32x32(t_d, dw);
                tmem_wait_st();
                fence_before_sync();
                mbar_arrive(ds_full);
            }
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
