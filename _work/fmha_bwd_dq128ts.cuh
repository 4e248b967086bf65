// dQ backward kernel with Q and dO resident in tensor memory (variant 6 of mm_fmha_bwd); included by fmha_bwd.cu
// inside its namespace (shares BwdParams, the tile constants and pack2 with the default kernels).
//
// One CTA = one 128-row query tile of one head, walking the 128-row key tiles j of its sequence:
//     S_j   = Q K_j^T      128 x 128 x 128   TS  (A = Q from tensor memory)          -> TMEM columns [128, 256)
//     dP_j  = dO V_j^T     128 x 128 x 128   TS  (A = dO from tensor memory)         -> TMEM columns [256, 384)
//     dQ   += dS_j K_j     128 x 128 x 128   TS  (A = dS_j, written over dP's columns) -> TMEM columns [384, 512)
// Q and dO are copied once from their TMA staging tiles into TMEM columns [0, 64) and [64, 128) as bf16 pairs.  That
// (1) halves the shared-memory operand traffic of the S and dP products, which otherwise need the SM's full 128 B per
// clock and collide with the TMA writes of the next tiles, and (2) frees 64 KB of shared memory, so that K runs in a
// 4-deep and V in a 3-deep ring (K_j lives until dQ_j, V_j until dP_j) and the tile stream's latency stays hidden.
// S and dP are single-buffered; the issue order   dP_j  S_{j+1}  dQ_j  dP_{j+1} ...   lets S_{j+1} run while the row
// threads turn dP_j into dS_j, and their exp2 work on S_{j+1} overlaps dQ_j and dP_{j+1}.
//
//   warp 0      TMA: Q, dO into the first K / V ring slots; after the copy to TMEM, the K_j / V_j stream
//   warp 1      MMA issuer
//   warps 2-9   row threads: thread = (query row, half): 64 of the 128 key columns.  P = exp2(S * scale - lse) kept in
//               registers as soon as S_j is there (S is released for S_{j+1}); dS = P * (dP - delta) written as bf16 pairs
//               over the first 32 of its own 64 dP columns.
// Every mbarrier wait is bounded (tc05::mbar_wait).

constexpr int kRingK6 = 4, kRingV6 = 3;
constexpr int kSmemDq6 = (kRingK6 + kRingV6) * kTile + 512 + 1024;

__global__ void __launch_bounds__(320, 1)
fmha_bwd_dq128ts_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                        const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, const BwdParams p) {
    if ((int)blockIdx.x >= *p.n_tiles) return;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sK = smem;                               // [kRingK6]
    uint8_t* sV = sK + kRingK6 * kTile;               // [kRingV6]
    uint8_t* sQstage = sK;                            // Q / dO pass through the first ring slots
    uint8_t* sdOstage = sV;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + kRingV6 * kTile);
    uint64_t* q_full = bars + 0;
    uint64_t* q_done = bars + 1;
    uint64_t* k_full = bars + 2;                      // [kRingK6]
    uint64_t* k_empty = k_full + kRingK6;
    uint64_t* v_full = k_empty + kRingK6;             // [kRingV6]
    uint64_t* v_empty = v_full + kRingV6;
    uint64_t* s_full = v_empty + kRingV6;
    uint64_t* s_empty = s_full + 1;
    uint64_t* dp_full = s_full + 2;
    uint64_t* ds_full = s_full + 3;
    uint64_t* dq_full = s_full + 4;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 5);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = p.tile_seq[blockIdx.x];
    const int q0 = p.tile_r0[blockIdx.x];
    const int head = blockIdx.y;
    const int kv_head = head / (p.Nq / p.Nkv);
    const int q_begin = p.cu_q[seq], q_len = p.cu_q[seq + 1] - q_begin;
    const int k_begin = p.cu_k[seq], k_len = p.cu_k[seq + 1] - k_begin;
    const int diag = k_len - q_len;
    int kv_end = k_len;
    if (p.causal) kv_end = min(k_len, q0 + 128 + diag);
    const int n_kv = max(0, (kv_end + 127) / 128);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(q_done, 256);
        for (int i = 0; i < kRingK6; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
        }
        for (int i = 0; i < kRingV6; ++i) {
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
        }
        mbar_init(s_full, 1);
        mbar_init(s_empty, 256);
        mbar_init(dp_full, 1);
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
    const uint32_t tQ = tmem_base, tdO = tmem_base + 64, tS = tmem_base + 128, tdP = tmem_base + 256, tdQ = tmem_base + 384;

    if (warp == 0) {
        // ------------------------------------------------------------------------------ TMA producer
        if (lane == 0 && n_kv > 0) {
            mbar_expect_tx(q_full, 2 * kTile);
            tma_load_3d(sQstage, &tmQ, q_full, 0, head, q_begin + q0);
            tma_load_3d(sQstage + kAtom, &tmQ, q_full, 64, head, q_begin + q0);
            tma_load_3d(sdOstage, &tmdO, q_full, 0, head, q_begin + q0);
            tma_load_3d(sdOstage + kAtom, &tmdO, q_full, 64, head, q_begin + q0);
            bool ok = mbar_wait(q_done, 0, abort_flag);         // the staging slots are free again
            for (int j = 0; j < n_kv && ok; ++j) {
                const int ks = j % kRingK6, vs = j % kRingV6;
                const uint32_t kph = (j / kRingK6) & 1, vph = (j / kRingV6) & 1;
                const int row = k_begin + j * 128;
                if (!mbar_wait(&k_empty[ks], kph ^ 1, abort_flag)) { ok = false; break; }
                mbar_expect_tx(&k_full[ks], kTile);
                tma_load_3d(sK + ks * kTile, &tmK, &k_full[ks], 0, kv_head, row);
                tma_load_3d(sK + ks * kTile + kAtom, &tmK, &k_full[ks], 64, kv_head, row);
                if (!mbar_wait(&v_empty[vs], vph ^ 1, abort_flag)) { ok = false; break; }
                mbar_expect_tx(&v_full[vs], kTile);
                tma_load_3d(sV + vs * kTile, &tmV, &v_full[vs], 0, kv_head, row);
                tma_load_3d(sV + vs * kTile + kAtom, &tmV, &v_full[vs], 64, kv_head, row);
            }
            if (!ok) atomicExch(p.status, MM_TIMEOUT_TMA);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------------------ MMA issuer
        if (lane == 0 && n_kv > 0) {
            constexpr uint32_t idesc_s = idesc_bf16(128, 128, 0, 0);
            constexpr uint32_t idesc_dq = idesc_bf16(128, HD, 0, 1);      // B = K_j read as [N = d, K = key]
            bool ok = mbar_wait(q_done, 0, abort_flag);
            auto issue_s = [&](int j) -> bool {
                const int ks = j % kRingK6;
                if (!mbar_wait(s_empty, (j & 1) ^ 1, abort_flag) || !mbar_wait(&k_full[ks], (j / kRingK6) & 1, abort_flag)) return false;
                fence_after_sync();
                const uint32_t ka = smem_u32(sK + ks * kTile);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    mma_ts(tS, tQ + k * 8, smem_desc_sw128(ka + (k >> 2) * kAtom + (k & 3) * 32, 16, 1024), idesc_s, k ? 1u : 0u);
                mma_commit(s_full);
                return true;
            };
            auto issue_dp = [&](int j) -> bool {
                const int vs = j % kRingV6;
                if (!mbar_wait(&v_full[vs], (j / kRingV6) & 1, abort_flag)) return false;
                fence_after_sync();
                const uint32_t va = smem_u32(sV + vs * kTile);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    mma_ts(tdP, tdO + k * 8, smem_desc_sw128(va + (k >> 2) * kAtom + (k & 3) * 32, 16, 1024), idesc_s, k ? 1u : 0u);
                mma_commit(dp_full);
                mma_commit(&v_empty[vs]);
                return true;
            };
            if (ok) ok = issue_s(0);
            if (ok) ok = issue_dp(0);
            for (int j = 0; j < n_kv && ok; ++j) {
                const int ks = j % kRingK6;
                // S_{j+1} may overwrite S as soon as the row threads hold S_j in registers
                if (j + 1 < n_kv && !(ok = issue_s(j + 1))) break;
                if (!mbar_wait(ds_full, j & 1, abort_flag)) { ok = false; break; }
                fence_after_sync();
                const uint32_t ka = smem_u32(sK + ks * kTile);
                // dS_j: keys 0..63 as bf16 pairs in dP columns 0..31, keys 64..127 in columns 64..95
#pragma unroll
                for (int k = 0; k < 128 / 16; ++k)
                    mma_ts(tdQ, tdP + (k >> 2) * 64 + (k & 3) * 8, smem_desc_sw128(ka + k * 2048, kAtom, 1024), idesc_dq,
                           (j | k) ? 1u : 0u);
                mma_commit(&k_empty[ks]);
                // dP_{j+1} lands on the columns dQ_j reads dS_j from: it follows dQ_j in the (in-order) tensor pipe
                if (j + 1 < n_kv && !(ok = issue_dp(j + 1))) break;
            }
            if (ok) mma_commit(dq_full);
            if (!ok) atomicExch(p.status, MM_TIMEOUT_MMA);
        }
    } else {
        // ------------------------------------------------------------------------------ row threads (warps 2..9)
        const int half = (warp - 2) >> 2;
        const int qd = warp & 3;
        const int row = qd * 32 + lane;
        const int qi = q0 + row;
        const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
        const bool row_ok = qi < q_len;
        bool ok = true;
        if (n_kv > 0) {
            // warpgroup 0 copies Q, warpgroup 1 copies dO: swizzled staging tile -> bf16 pairs in tensor memory
            ok = mbar_wait(q_full, 0, abort_flag);
            if (ok) {
                const uint8_t* src = half == 0 ? sQstage : sdOstage;
                const uint32_t dst = (half == 0 ? tQ : tdO) + lane_off;
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2) {
                    uint32_t w[32];
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const uint4 v4 = *reinterpret_cast<const uint4*>(src + h2 * kAtom + row * 128 + ((c ^ (row & 7)) << 4));
                        w[4 * c + 0] = v4.x;
                        w[4 * c + 1] = v4.y;
                        w[4 * c + 2] = v4.z;
                        w[4 * c + 3] = v4.w;
                    }
                    tmem_st_32x32(dst + h2 * 32, w);
                }
                tmem_wait_st();
                fence_before_sync();
                mbar_arrive(q_done);
            }
        }
        const size_t stat = (size_t)head * p.T + q_begin + min(qi, max(q_len - 1, 0));
        const float lse2 = n_kv > 0 ? p.lse[stat] * kLog2e : 0.f;
        const float dlt = n_kv > 0 ? p.delta[stat] : 0.f;
        const int limit = !row_ok ? -1 : (p.causal ? min(k_len - 1, qi + diag) : k_len - 1);
        const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nl2 = make_float2(-lse2, -lse2), nd2 = make_float2(-dlt, -dlt);
        for (int j = 0; j < n_kv && ok; ++j) {
            const uint32_t par = j & 1;
            if (!mbar_wait(s_full, par, abort_flag)) { ok = false; break; }
            fence_after_sync();
            uint32_t r[64];
            tmem_ld_32x32(tS + half * 64 + lane_off, r);
            tmem_ld_32x32(tS + half * 64 + 32 + lane_off, r + 32);
            tmem_wait_ld();
            fence_before_sync();
            mbar_arrive(s_empty);
            const int kbase = j * 128 + half * 64;
            const bool tile_masked = kbase + 63 > limit;
#pragma unroll
            for (int i = 0; i < 32; ++i) {           // P = exp2(S * scale - lse), two columns per instruction
                const float2 x = __ffma2_rn(make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])), sc2, nl2);
                float2 pr = make_float2(exp2f(x.x), exp2f(x.y));
                if (tile_masked) {
                    if (kbase + 2 * i > limit) pr.x = 0.f;
                    if (kbase + 2 * i + 1 > limit) pr.y = 0.f;
                }
                r[2 * i] = __float_as_uint(pr.x);
                r[2 * i + 1] = __float_as_uint(pr.y);
            }
            if (!mbar_wait(dp_full, par, abort_flag)) { ok = false; break; }
            fence_after_sync();
            uint32_t d[64];
            const uint32_t t_d = tdP + half * 64 + lane_off;
            tmem_ld_32x32(t_d, d);
            tmem_ld_32x32(t_d + 32, d + 32);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) {           // dS = P * (dP - delta)
                const float2 g = __fadd2_rn(make_float2(__uint_as_float(d[2 * i]), __uint_as_float(d[2 * i + 1])), nd2);
                const float2 ds = __fmul2_rn(make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])), g);
                d[i] = pack2(ds.x, ds.y);
            }
            tmem_st_32x32(t_d, d);                   // over the first 32 of the 64 fp32 columns this thread has just read
            tmem_wait_st();
            fence_before_sync();
            mbar_arrive(ds_full);
        }
        bf16* dst = p.dq + ((size_t)(q_begin + qi) * p.Nq + head) * HD + half * 64;
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
                        reinterpret_cast<uint4*>(dst)[c * 4 + g] = w;
                    }
                }
            }
        } else if (n_kv == 0 && row_ok) {
            for (int g = 0; g < 8; ++g) reinterpret_cast<uint4*>(dst)[g] = make_uint4(0, 0, 0, 0);
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
