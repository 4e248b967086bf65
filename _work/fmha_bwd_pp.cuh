// Flash attention backward, "ping-pong" variants of the two kernels in fmha_bwd.cu.
//
// Same math and the same tile products; what changes is the schedule inside a CTA.  In fmha_bwd.cu both compute
// warpgroups work on the same tile in lock step, so every tile pays the full chain
//     MMA -> commit -> TMEM load -> exp / multiply -> shared store -> arrive -> MMA
// end to end, and the operand rings are only two deep.  Here
//   * key tiles are 64 wide, so S / dP / dS are double-buffered within the same TMEM and shared-memory budget and
//     the K / V (or Q / dO) rings are 4 (3) deep: loads are issued several tiles ahead;
//   * warpgroup 0 owns the even tiles and warpgroup 1 the odd tiles: while one warpgroup is in its exp phase the
//     tensor core runs the other tile's products, and the accumulating product of tile j overlaps the softmax
//     work of tile j + 1.
// Measured on B200 (75600 tokens x 5 heads): 81.9 ms against 72.1 ms for the lock-step kernels, i.e. the halved N
// of the S / dP products (operands streamed from shared memory at 192 B per clock and SM instead of 128) costs
// more than the extra overlap gains.  Kept as `variant = 1` of mm_fmha_bwd for comparison; the default is 0.
// Included by fmha_bwd.cu inside its anonymous namespace (shares BwdParams, pack2 and the tile constants).
constexpr int BK = 64;                     // key rows per step (dQ kernel) / query rows per step (dK/dV kernel)
constexpr int kKTile = BK * HD * 2;        // 16 KiB
constexpr int kKAtom = BK * 128;           // 8 KiB
constexpr int kDsTile = 128 * BK * 2;      // 16 KiB: dS / P^T / dS^T tile (one atom of 128 rows)

// ============================================================================================== dQ
constexpr int kStagesDq = 4;
constexpr int kSmemDqPP = 2 * kTile + 2 * kStagesDq * kKTile + 2 * kDsTile + 1024 + 1024;

// kTS: dS is handed to the dQ product through tensor memory (written over the tile's dP columns with tcgen05.st and
// consumed as the A operand of a TS-form MMA) instead of through swizzled shared memory.
template <bool kTS>
__global__ void __launch_bounds__(320, 1)
fmha_bwd_dq_pp_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, const BwdParams p) {
    if ((int)blockIdx.x >= *p.n_tiles) return;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sdO = sQ + kTile;
    uint8_t* sK = sdO + kTile;                    // [4]
    uint8_t* sV = sK + kStagesDq * kKTile;        // [4]
    uint8_t* sdS = sV + kStagesDq * kKTile;       // [2]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + 2 * kDsTile);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;      // [4]
    uint64_t* k_empty = bars + 5;     // [4]
    uint64_t* v_full = bars + 9;      // [4]
    uint64_t* v_empty = bars + 13;    // [4]
    uint64_t* s_full = bars + 17;     // [2]   S and dP of a tile are committed together
    uint64_t* s_empty = bars + 19;    // [2]
    uint64_t* ds_full = bars + 21;    // [2]
    uint64_t* ds_empty = bars + 23;   // [2]
    uint64_t* dq_full = bars + 25;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 26);
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
    const int n_kv = max(0, (kv_end + BK - 1) / BK);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < kStagesDq; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&s_empty[i], 128);
            mbar_init(&ds_full[i], 128);
            mbar_init(&ds_empty[i], 1);
        }
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
    // S[2] : 0..127 (64 columns each), dP[2] : 128..255, dQ : 256..383
    const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdQ = tmem_base + 256;

    if (warp == 0) {
        if (lane == 0 && n_kv > 0) {
            mbar_expect_tx(q_full, 2 * kTile);
            tma_load_3d(sQ, &tmQ, q_full, 0, head, q_begin + q0);
            tma_load_3d(sQ + kAtom, &tmQ, q_full, 64, head, q_begin + q0);
            tma_load_3d(sdO, &tmdO, q_full, 0, head, q_begin + q0);
            tma_load_3d(sdO + kAtom, &tmdO, q_full, 64, head, q_begin + q0);
            for (int j = 0; j < n_kv; ++j) {
                const int st = j % kStagesDq;
                const uint32_t ph = (j / kStagesDq) & 1;
                const int row = k_begin + j * BK;
                if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag)) { atomicExch(p.status, MM_TIMEOUT_TMA); break; }
                mbar_expect_tx(&k_full[st], kKTile);
                tma_load_3d(sK + st * kKTile, &tmK, &k_full[st], 0, kv_head, row);
                tma_load_3d(sK + st * kKTile + kKAtom, &tmK, &k_full[st], 64, kv_head, row);
                if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag)) { atomicExch(p.status, MM_TIMEOUT_TMA); break; }
                mbar_expect_tx(&v_full[st], kKTile);
                tma_load_3d(sV + st * kKTile, &tmV, &v_full[st], 0, kv_head, row);
                tma_load_3d(sV + st * kKTile + kKAtom, &tmV, &v_full[st], 64, kv_head, row);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && n_kv > 0) {
            constexpr uint32_t idesc_s = idesc_bf16(128, BK, 0, 0);        // S, dP: N = 64 keys
            constexpr uint32_t idesc_dq = idesc_bf16(128, HD, 0, 1);       // dQ: B = K_j as [N = d, K = 64 keys]
            bool ok = mbar_wait(q_full, 0, abort_flag);
            const uint32_t qa = smem_u32(sQ), doa = smem_u32(sdO);
            auto issue_s_dp = [&](int j) -> bool {
                const int st = j % kStagesDq, b = j & 1;
                const uint32_t ph = (j / kStagesDq) & 1, bph = (j >> 1) & 1;
                if (!mbar_wait(&s_empty[b], bph ^ 1, abort_flag) || !mbar_wait(&k_full[st], ph, abort_flag) ||
                    !mbar_wait(&v_full[st], ph, abort_flag))
                    return false;
                fence_after_sync();
                const uint32_t ka = smem_u32(sK + st * kKTile), va = smem_u32(sV + st * kKTile);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t aoff = (k >> 2) * kAtom + (k & 3) * 32;
                    const uint32_t boff = (k >> 2) * kKAtom + (k & 3) * 32;
                    mma_ss(tS + b * BK, smem_desc_sw128(qa + aoff, 16, 1024), smem_desc_sw128(ka + boff, 16, 1024), idesc_s,
                           k ? 1u : 0u);
                    mma_ss(tdP + b * BK, smem_desc_sw128(doa + aoff, 16, 1024), smem_desc_sw128(va + boff, 16, 1024), idesc_s,
                           k ? 1u : 0u);
                }
                mma_commit(&s_full[b]);
                mma_commit(&v_empty[st]);
                return true;
            };
            if (ok) ok = issue_s_dp(0);
            if (ok && n_kv > 1) ok = issue_s_dp(1);
            for (int j = 0; j < n_kv && ok; ++j) {
                const int st = j % kStagesDq, b = j & 1;
                const uint32_t bph = (j >> 1) & 1;
                // S / dP of tile j + 2 go into the buffers tile j's warpgroup has just emptied into registers
                if (!kTS && j + 2 < n_kv && !(ok = issue_s_dp(j + 2))) break;
                if (!mbar_wait(&ds_full[b], bph, abort_flag)) { ok = false; break; }
                fence_after_sync();
                const uint32_t ka = smem_u32(sK + st * kKTile), dsa = smem_u32(sdS + b * kDsTile);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    const uint64_t db = smem_desc_sw128(ka + k * 2048, kKAtom, 1024);
                    if (kTS) mma_ts(tdQ, tdP + b * BK + k * 8, db, idesc_dq, (j | k) ? 1u : 0u);
                    else mma_ss(tdQ, smem_desc_sw128(dsa + k * 32, 16, 1024), db, idesc_dq, (j | k) ? 1u : 0u);
                }
                mma_commit(&ds_empty[b]);
                mma_commit(&k_empty[st]);
                // TS: dS(j) sits in dP[b]'s columns; the in-order tensor pipe runs dP(j + 2) after dQ(j)
                if (kTS && j + 2 < n_kv && !(ok = issue_s_dp(j + 2))) break;
            }
            if (ok) mma_commit(dq_full);
            if (!ok) atomicExch(p.status, MM_TIMEOUT_MMA);
        }
    } else {
        // warpgroup w owns the tiles j = w, w + 2, ...; thread = query row, 64 key columns per tile
        const int wg = (warp - 2) >> 2;
        const int qd = warp & 3;
        const int row = qd * 32 + lane;
        const int qi = q0 + row;
        const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
        const bool row_ok = qi < q_len;
        const size_t stat = (size_t)head * p.T + q_begin + min(qi, max(q_len - 1, 0));
        const float lse2 = n_kv > 0 ? p.lse[stat] * kLog2e : 0.f;
        const float dlt = n_kv > 0 ? p.delta[stat] : 0.f;
        const int limit = !row_ok ? -1 : (p.causal ? min(k_len - 1, qi + diag) : k_len - 1);
        uint8_t* my_ds = sdS + wg * kDsTile;
        bool ok = true;
        for (int j = wg; j < n_kv; j += 2) {
            const uint32_t bph = (j >> 1) & 1;
            if (!mbar_wait(&s_full[wg], bph, abort_flag)) { ok = false; break; }
            fence_after_sync();
            uint32_t r[64], d[64];
            tmem_ld_32x32(tS + wg * BK + lane_off, r);
            tmem_ld_32x32(tS + wg * BK + lane_off + 32, r + 32);
            tmem_ld_32x32(tdP + wg * BK + lane_off, d);
            tmem_ld_32x32(tdP + wg * BK + lane_off + 32, d + 32);
            tmem_wait_ld();
            fence_before_sync();
            mbar_arrive(&s_empty[wg]);
            const int kbase = j * BK;
#pragma unroll
            for (int i = 0; i < 64; ++i) {
                const float pr = exp2f(__uint_as_float(r[i]) * p.scale_log2 - lse2);
                const float pv = kbase + i > limit ? 0.f : pr;
                r[i] = __float_as_uint(pv * (__uint_as_float(d[i]) - dlt));
            }
            if (kTS) {
                // 64 keys -> 32 columns of bf16 pairs over the first half of this tile's dP columns
#pragma unroll
                for (int i = 0; i < 32; ++i) d[i] = pack2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                tmem_st_32x32(tdP + wg * BK + lane_off, d);
                tmem_wait_st();
                fence_before_sync();
                mbar_arrive(&ds_full[wg]);
                continue;
            }
            if (j >= 2 && !mbar_wait(&ds_empty[wg], ((j >> 1) - 1) & 1, abort_flag)) { ok = false; break; }
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                uint4 w;
                w.x = pack2(__uint_as_float(r[8 * g + 0]), __uint_as_float(r[8 * g + 1]));
                w.y = pack2(__uint_as_float(r[8 * g + 2]), __uint_as_float(r[8 * g + 3]));
                w.z = pack2(__uint_as_float(r[8 * g + 4]), __uint_as_float(r[8 * g + 5]));
                w.w = pack2(__uint_as_float(r[8 * g + 6]), __uint_as_float(r[8 * g + 7]));
                *reinterpret_cast<uint4*>(my_ds + row * 128 + ((g ^ (row & 7)) << 4)) = w;
            }
            fence_proxy_async();
            mbar_arrive(&ds_full[wg]);
        }
        // epilogue: each warpgroup stores one half of the head dim
        bf16* dst = p.dq + ((size_t)(q_begin + qi) * p.Nq + head) * HD + wg * 64;
        if (ok && n_kv > 0 && mbar_wait(dq_full, 0, abort_flag)) {
            fence_after_sync();
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t d[32];
                tmem_ld_32x32(tdQ + wg * 64 + lane_off + c * 32, d);
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

// ============================================================================================== dK, dV
constexpr int kStagesKv = 3;
constexpr int kSmemDkvPP = 2 * kTile + 2 * kStagesKv * kKTile + 4 * kDsTile + 1024 + 1024;

__global__ void __launch_bounds__(320, 1)
fmha_bwd_dkv_pp_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, const BwdParams p) {
    if ((int)blockIdx.x >= *p.n_tiles) return;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sK = smem;
    uint8_t* sV = sK + kTile;
    uint8_t* sQ = sV + kTile;                       // [3]
    uint8_t* sdO = sQ + kStagesKv * kKTile;         // [3]
    uint8_t* sP = sdO + kStagesKv * kKTile;         // [2]  one per warpgroup
    uint8_t* sdS = sP + 2 * kDsTile;                // [2]
    float* s_lse = reinterpret_cast<float*>(sdS + 2 * kDsTile);    // [2][64]
    float* s_dlt = s_lse + 2 * BK;                                   // [2][64]
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_dlt + 2 * BK);
    uint64_t* kv_full = bars + 0;
    uint64_t* full = bars + 1;         // [3]
    uint64_t* empty = bars + 4;        // [3]
    uint64_t* st_full = bars + 7;      // [2]
    uint64_t* st_empty = bars + 9;     // [2]
    uint64_t* pds_full = bars + 11;    // [2]
    uint64_t* pds_empty = bars + 13;   // [2]
    uint64_t* acc_full = bars + 15;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = p.tile_seq[blockIdx.x];
    const int kv0 = p.tile_r0[blockIdx.x];
    const int Gfull = p.Nq / p.Nkv;
    const int kv_head = p.split ? blockIdx.y / Gfull : blockIdx.y;
    const int head0 = p.split ? blockIdx.y : kv_head * Gfull;
    const int G = p.split ? 1 : Gfull;
    const int out_heads = p.split ? p.Nq : p.Nkv, out_head = blockIdx.y;
    const int q_begin = p.cu_q[seq], q_len = p.cu_q[seq + 1] - q_begin;
    const int k_begin = p.cu_k[seq], k_len = p.cu_k[seq + 1] - k_begin;
    const int diag = k_len - q_len;
    const int nq = (q_len + BK - 1) / BK;
    const int i_min = p.causal ? min(nq, max(0, kv0 - diag) / BK) : 0;
    const int per_head = nq - i_min;
    const int n_it = per_head * G;

    if (threadIdx.x == 0) {
        mbar_init(kv_full, 1);
        for (int i = 0; i < kStagesKv; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&st_full[i], 1);
            mbar_init(&st_empty[i], 128);
            mbar_init(&pds_full[i], 128);
            mbar_init(&pds_empty[i], 1);
        }
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
                const int st = it % kStagesKv;
                const uint32_t ph = (it / kStagesKv) & 1;
                const int head = head0 + it / per_head;
                const int row = q_begin + (i_min + it % per_head) * BK;
                if (!mbar_wait(&empty[st], ph ^ 1, abort_flag)) { atomicExch(p.status, MM_TIMEOUT_TMA); break; }
                mbar_expect_tx(&full[st], 2 * kKTile);
                tma_load_3d(sQ + st * kKTile, &tmQ, &full[st], 0, head, row);
                tma_load_3d(sQ + st * kKTile + kKAtom, &tmQ, &full[st], 64, head, row);
                tma_load_3d(sdO + st * kKTile, &tmdO, &full[st], 0, head, row);
                tma_load_3d(sdO + st * kKTile + kKAtom, &tmdO, &full[st], 64, head, row);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && n_it > 0) {
            constexpr uint32_t idesc_t = idesc_bf16(128, BK, 0, 0);
            constexpr uint32_t idesc_acc = idesc_bf16(128, 128, 0, 1);
            bool ok = mbar_wait(kv_full, 0, abort_flag);
            const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
            auto issue_t = [&](int it) -> bool {
                const int st = it % kStagesKv, b = it & 1;
                const uint32_t ph = (it / kStagesKv) & 1, bph = (it >> 1) & 1;
                if (!mbar_wait(&st_empty[b], bph ^ 1, abort_flag) || !mbar_wait(&full[st], ph, abort_flag)) return false;
                fence_after_sync();
                const uint32_t qa = smem_u32(sQ + st * kKTile), doa = smem_u32(sdO + st * kKTile);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t aoff = (k >> 2) * kAtom + (k & 3) * 32;
                    const uint32_t boff = (k >> 2) * kKAtom + (k & 3) * 32;
                    mma_ss(tST + b * BK, smem_desc_sw128(ka + aoff, 16, 1024), smem_desc_sw128(qa + boff, 16, 1024), idesc_t,
                           k ? 1u : 0u);
                    mma_ss(tdPT + b * BK, smem_desc_sw128(va + aoff, 16, 1024), smem_desc_sw128(doa + boff, 16, 1024), idesc_t,
                           k ? 1u : 0u);
                }
                mma_commit(&st_full[b]);
                return true;
            };
            if (ok) ok = issue_t(0);
            if (ok && n_it > 1) ok = issue_t(1);
            for (int it = 0; it < n_it && ok; ++it) {
                const int st = it % kStagesKv, b = it & 1;
                const uint32_t bph = (it >> 1) & 1;
                if (it + 2 < n_it && !(ok = issue_t(it + 2))) break;
                if (!mbar_wait(&pds_full[b], bph, abort_flag)) { ok = false; break; }
                fence_after_sync();
                const uint32_t qa = smem_u32(sQ + st * kKTile), doa = smem_u32(sdO + st * kKTile);
                const uint32_t pa = smem_u32(sP + b * kDsTile), dsa = smem_u32(sdS + b * kDsTile);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    mma_ss(tdV, smem_desc_sw128(pa + k * 32, 16, 1024), smem_desc_sw128(doa + k * 2048, kKAtom, 1024), idesc_acc,
                           (it | k) ? 1u : 0u);
                    mma_ss(tdK, smem_desc_sw128(dsa + k * 32, 16, 1024), smem_desc_sw128(qa + k * 2048, kKAtom, 1024), idesc_acc,
                           (it | k) ? 1u : 0u);
                }
                mma_commit(&pds_empty[b]);
                mma_commit(&empty[st]);
            }
            if (ok) mma_commit(acc_full);
            if (!ok) atomicExch(p.status, MM_TIMEOUT_MMA);
        }
    } else {
        // warpgroup w owns the query tiles it = w, w + 2, ...; thread = key row, all 64 query columns of the tile
        const int wg = (warp - 2) >> 2;
        const int qd = warp & 3;
        const int row = qd * 32 + lane;
        const int kj = kv0 + row;
        const bool row_ok = kj < k_len;
        const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
        float* my_lse = s_lse + wg * BK;
        float* my_dlt = s_dlt + wg * BK;
        uint8_t* my_p = sP + wg * kDsTile;
        uint8_t* my_ds = sdS + wg * kDsTile;
        auto load_stat = [&](int it) -> float {
            const int head = head0 + it / per_head;
            const int qi = min((i_min + it % per_head) * BK + (row & 63), q_len - 1);
            const size_t idx = (size_t)head * p.T + q_begin + qi;
            return row < 64 ? p.lse[idx] * kLog2e : p.delta[idx];
        };
        float pre = wg < n_it ? load_stat(wg) : 0.f;
        bool ok = true;
        for (int it = wg; it < n_it; it += 2) {
            const uint32_t bph = (it >> 1) & 1;
            const int qbase = (i_min + it % per_head) * BK;
            // the previous tile's readers of my_lse / my_dlt are past their loop: same warpgroup, program order + barrier
            if (wg == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
            else asm volatile("bar.sync 2, 128;" ::: "memory");
            if (row < 64) my_lse[row] = pre;
            else my_dlt[row - 64] = pre;
            if (it + 2 < n_it) pre = load_stat(it + 2);
            if (wg == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
            else asm volatile("bar.sync 2, 128;" ::: "memory");
            if (!mbar_wait(&st_full[wg], bph, abort_flag)) { ok = false; break; }
            fence_after_sync();
            const int c_lo = !row_ok ? BK : (p.causal ? max(0, kj - diag - qbase) : 0);
            const int c_hi = min(BK, q_len - qbase);
            if (it >= 2 && !mbar_wait(&pds_empty[wg], ((it >> 1) - 1) & 1, abort_flag)) { ok = false; break; }
            // two passes of 32 query columns keep the live registers low
#pragma unroll
            for (int hcol = 0; hcol < 2; ++hcol) {
                uint32_t s[32], d[32];
                tmem_ld_32x32(tST + wg * BK + lane_off + hcol * 32, s);
                tmem_ld_32x32(tdPT + wg * BK + lane_off + hcol * 32, d);
                tmem_wait_ld();
                if (hcol == 1) {
                    fence_before_sync();
                    mbar_arrive(&st_empty[wg]);
                }
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const int cc = hcol * 32 + c;
                    const float pr = exp2f(__uint_as_float(s[c]) * p.scale_log2 - my_lse[cc]);
                    const float pv = (cc >= c_lo && cc < c_hi) ? pr : 0.f;
                    s[c] = __float_as_uint(pv);
                    d[c] = __float_as_uint(pv * (__uint_as_float(d[c]) - my_dlt[cc]));
                }
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    uint4 w, x;
                    w.x = pack2(__uint_as_float(s[8 * g + 0]), __uint_as_float(s[8 * g + 1]));
                    w.y = pack2(__uint_as_float(s[8 * g + 2]), __uint_as_float(s[8 * g + 3]));
                    w.z = pack2(__uint_as_float(s[8 * g + 4]), __uint_as_float(s[8 * g + 5]));
                    w.w = pack2(__uint_as_float(s[8 * g + 6]), __uint_as_float(s[8 * g + 7]));
                    x.x = pack2(__uint_as_float(d[8 * g + 0]), __uint_as_float(d[8 * g + 1]));
                    x.y = pack2(__uint_as_float(d[8 * g + 2]), __uint_as_float(d[8 * g + 3]));
                    x.z = pack2(__uint_as_float(d[8 * g + 4]), __uint_as_float(d[8 * g + 5]));
                    x.w = pack2(__uint_as_float(d[8 * g + 6]), __uint_as_float(d[8 * g + 7]));
                    const int off = row * 128 + (((hcol * 4 + g) ^ (row & 7)) << 4);
                    *reinterpret_cast<uint4*>(my_p + off) = w;
                    *reinterpret_cast<uint4*>(my_ds + off) = x;
                }
            }
            fence_proxy_async();
            mbar_arrive(&pds_full[wg]);
        }
        bf16* dvp = p.dv + ((size_t)(k_begin + kj) * out_heads + out_head) * HD + wg * 64;
        bf16* dkp = p.dk + ((size_t)(k_begin + kj) * out_heads + out_head) * HD + wg * 64;
        if (ok && n_it > 0 && mbar_wait(acc_full, 0, abort_flag)) {
            fence_after_sync();
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t a[32], b[32];
                tmem_ld_32x32(tdV + wg * 64 + lane_off + c * 32, a);
                tmem_ld_32x32(tdK + wg * 64 + lane_off + c * 32, b);
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
                        reinterpret_cast<uint4*>(dvp)[c * 4 + g] = w;
                        reinterpret_cast<uint4*>(dkp)[c * 4 + g] = x;
                    }
                }
            }
        } else if (n_it == 0 && row_ok) {
            for (int g = 0; g < 8; ++g) {
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

// ============================================================================================== dK, dV with TS-form MMAs
// Measured on the SS-form kernels: a 128 x 128 x 16 product whose two operands come from shared memory needs the
// SM's full 128 B / clock of shared-memory bandwidth, so the TMA fills and the P^T / dS^T stores stretch every
// tile.  Here every A operand lives in tensor memory:
//   K and V of the CTA's key tile are copied once from shared memory into TMEM (64 columns each),
//   P^T and dS^T are written by the row threads over the S^T / dP^T columns they have just read (tcgen05.st),
// so the tensor pipe reads only the streamed Q_i / dO_i tiles from shared memory, and the shared memory that held
// K and V becomes a deeper Q_i / dO_i ring.
constexpr int kRingTs = 6;
constexpr int kSmemDkvTs = 2 * kRingTs * kKTile + 2048 + 1024;     // 6 x 32 KiB ring; K / V are staged through slots 0 and 1

__global__ void __launch_bounds__(320, 1)
fmha_bwd_dkv_ts_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, const BwdParams p) {
    if ((int)blockIdx.x >= *p.n_tiles) return;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;                              // [kRingTs] 16 KiB each
    uint8_t* sdO = sQ + kRingTs * kKTile;            // [kRingTs]
    // K and V (32 KiB each) are staged through the first two slots of each ring before the walk starts
    uint8_t* sKstage = sQ;
    uint8_t* sVstage = sdO;
    float* s_lse = reinterpret_cast<float*>(sdO + kRingTs * kKTile);    // [2][64]
    float* s_dlt = s_lse + 2 * BK;                                        // [2][64]
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_dlt + 2 * BK);
    uint64_t* kv_full = bars + 0;
    uint64_t* kv_done = bars + 1;                    // K / V copied into TMEM: the ring may start
    uint64_t* full = bars + 2;                       // [kRingTs]
    uint64_t* empty = full + kRingTs;                // [kRingTs]
    uint64_t* st_full = empty + kRingTs;
    uint64_t* pds_full = st_full + 1;
    uint64_t* acc_full = st_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(st_full + 3);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = p.tile_seq[blockIdx.x];
    const int kv0 = p.tile_r0[blockIdx.x];
    const int Gfull = p.Nq / p.Nkv;
    const int kv_head = p.split ? blockIdx.y / Gfull : blockIdx.y;
    const int head0 = p.split ? blockIdx.y : kv_head * Gfull;
    const int G = p.split ? 1 : Gfull;
    const int out_heads = p.split ? p.Nq : p.Nkv, out_head = blockIdx.y;
    const int q_begin = p.cu_q[seq], q_len = p.cu_q[seq + 1] - q_begin;
    const int k_begin = p.cu_k[seq], k_len = p.cu_k[seq + 1] - k_begin;
    const int diag = k_len - q_len;
    const int nq = (q_len + BK - 1) / BK;
    const int i_min = p.causal ? min(nq, max(0, kv0 - diag) / BK) : 0;
    const int per_head = nq - i_min;
    const int n_it = per_head * G;

    if (threadIdx.x == 0) {
        mbar_init(kv_full, 1);
        mbar_init(kv_done, 256);
        for (int i = 0; i < kRingTs; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        mbar_init(st_full, 1);
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
    // K : 0..63, V : 64..127 (bf16 pairs), S^T : 128..191, dP^T : 192..255, dV : 256..383, dK : 384..511
    const uint32_t tK = tmem_base, tV = tmem_base + 64, tST = tmem_base + 128, tdPT = tmem_base + 192, tdV = tmem_base + 256,
                   tdK = tmem_base + 384;

    if (warp == 0) {
        if (lane == 0 && n_it > 0) {
            mbar_expect_tx(kv_full, 2 * kTile);
            tma_load_3d(sKstage, &tmK, kv_full, 0, kv_head, k_begin + kv0);
            tma_load_3d(sKstage + kAtom, &tmK, kv_full, 64, kv_head, k_begin + kv0);
            tma_load_3d(sVstage, &tmV, kv_full, 0, kv_head, k_begin + kv0);
            tma_load_3d(sVstage + kAtom, &tmV, kv_full, 64, kv_head, k_begin + kv0);
            bool ok = mbar_wait(kv_done, 0, abort_flag);          // staging area is free again
            for (int it = 0; it < n_it && ok; ++it) {
                const int st = it % kRingTs;
                const uint32_t ph = (it / kRingTs) & 1;
                const int head = head0 + it / per_head;
                const int row = q_begin + (i_min + it % per_head) * BK;
                if (!mbar_wait(&empty[st], ph ^ 1, abort_flag)) { ok = false; break; }
                mbar_expect_tx(&full[st], 2 * kKTile);
                tma_load_3d(sQ + st * kKTile, &tmQ, &full[st], 0, head, row);
                tma_load_3d(sQ + st * kKTile + kKAtom, &tmQ, &full[st], 64, head, row);
                tma_load_3d(sdO + st * kKTile, &tmdO, &full[st], 0, head, row);
                tma_load_3d(sdO + st * kKTile + kKAtom, &tmdO, &full[st], 64, head, row);
            }
            if (!ok) atomicExch(p.status, MM_TIMEOUT_TMA);
        }
    } else if (warp == 1) {
        if (lane == 0 && n_it > 0) {
            constexpr uint32_t idesc_t = idesc_bf16(128, BK, 0, 0);
            constexpr uint32_t idesc_acc = idesc_bf16(128, 128, 0, 1);
            bool ok = mbar_wait(kv_done, 0, abort_flag);
            for (int it = 0; it < n_it && ok; ++it) {
                const int st = it % kRingTs;
                const uint32_t ph = (it / kRingTs) & 1;
                if (!mbar_wait(&full[st], ph, abort_flag)) { ok = false; break; }
                fence_after_sync();
                const uint32_t qa = smem_u32(sQ + st * kKTile), doa = smem_u32(sdO + st * kKTile);
                // S^T = K Q_i^T, dP^T = V dO_i^T   (A from tensor memory: 8 columns per 16-wide k step)
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t boff = (k >> 2) * kKAtom + (k & 3) * 32;
                    mma_ts(tST, tK + k * 8, smem_desc_sw128(qa + boff, 16, 1024), idesc_t, k ? 1u : 0u);
                    mma_ts(tdPT, tV + k * 8, smem_desc_sw128(doa + boff, 16, 1024), idesc_t, k ? 1u : 0u);
                }
                mma_commit(st_full);
                if (!mbar_wait(pds_full, it & 1, abort_flag)) { ok = false; break; }
                fence_after_sync();
                // dV += P^T dO_i, dK += dS^T Q_i; P^T / dS^T sit in the S^T / dP^T columns: queries 0..31 in columns
                // 0..15, queries 32..63 in columns 32..47
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    const uint32_t acol = (k >> 1) * 32 + (k & 1) * 8;
                    mma_ts(tdV, tST + acol, smem_desc_sw128(doa + k * 2048, kKAtom, 1024), idesc_acc, (it | k) ? 1u : 0u);
                    mma_ts(tdK, tdPT + acol, smem_desc_sw128(qa + k * 2048, kKAtom, 1024), idesc_acc, (it | k) ? 1u : 0u);
                }
                mma_commit(&empty[st]);
            }
            if (ok) mma_commit(acc_full);
            if (!ok) atomicExch(p.status, MM_TIMEOUT_MMA);
        }
    } else {
        const int half = (warp - 2) >> 2;
        const int qd = warp & 3;
        const int row = qd * 32 + lane;
        const int tid2 = (warp - 2) * 32 + lane;
        const int kj = kv0 + row;
        const bool row_ok = kj < k_len;
        const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
        bool ok = true;
        if (n_it > 0) {
            // warpgroup 0 copies K, warpgroup 1 copies V: this thread's row of 128 values, un-swizzled, into TMEM
            ok = mbar_wait(kv_full, 0, abort_flag);
            const uint8_t* src = half == 0 ? sKstage : sVstage;
            const uint32_t dst = (half == 0 ? tK : tV) + lane_off;
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
            mbar_arrive(kv_done);
        }
        auto load_stat = [&](int it) -> float {
            if (tid2 >= 128) return 0.f;
            const int head = head0 + it / per_head;
            const int qi = min((i_min + it % per_head) * BK + (tid2 & 63), q_len - 1);
            const size_t idx = (size_t)head * p.T + q_begin + qi;
            return tid2 < 64 ? p.lse[idx] * kLog2e : p.delta[idx];
        };
        float pre = n_it > 0 ? load_stat(0) : 0.f;
        for (int it = 0; it < n_it && ok; ++it) {
            const int sb = it & 1;
            const int qbase = (i_min + it % per_head) * BK;
            if (tid2 < 64) s_lse[sb * BK + tid2] = pre;
            else if (tid2 < 128) s_dlt[sb * BK + tid2 - 64] = pre;
            if (it + 1 < n_it) pre = load_stat(it + 1);
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (!mbar_wait(st_full, it & 1, abort_flag)) { ok = false; break; }
            fence_after_sync();
            uint32_t s[32], d[32];
            tmem_ld_32x32(tST + half * 32 + lane_off, s);
            tmem_ld_32x32(tdPT + half * 32 + lane_off, d);
            tmem_wait_ld();
            const int c_lo = !row_ok ? BK : (p.causal ? max(0, kj - diag - qbase) : 0);
            const int c_hi = min(BK, q_len - qbase);
            const float* ls = s_lse + sb * BK + half * 32;
            const float* dl = s_dlt + sb * BK + half * 32;
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
            // over the fp32 columns this thread has just read: 16 columns of bf16 pairs at the start of its half
            tmem_st_32x16(tST + half * 32 + lane_off, pw);
            tmem_st_32x16(tdPT + half * 32 + lane_off, dw);
            tmem_wait_st();
            fence_before_sync();
            mbar_arrive(pds_full);
        }
        bf16* dvp = p.dv + ((size_t)(k_begin + kj) * out_heads + out_head) * HD + half * 64;
        bf16* dkp = p.dk + ((size_t)(k_begin + kj) * out_heads + out_head) * HD + half * 64;
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
                        reinterpret_cast<uint4*>(dvp)[c * 4 + g] = w;
                        reinterpret_cast<uint4*>(dkp)[c * 4 + g] = x;
                    }
                }
            }
        } else if (n_it == 0 && row_ok) {
            for (int g = 0; g < 8; ++g) {
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

// ============================================================================================== dQ with TS-form MMAs
// Q and dO of the CTA's query tile are copied once into tensor memory; per 64-key step S = Q K_j^T and dP = dO V_j^T
// read only K_j / V_j from shared memory, dS goes back into dP's columns (tcgen05.st) and feeds dQ += dS K_j as a
// TMEM operand.  S is double-buffered so that the next step's scores are ready when the row threads come back;
// dP(j + 1) follows dQ(j) on the in-order tensor pipe because both use the same columns.
constexpr int kRingDqTs = 6;
constexpr int kSmemDqTs = 2 * kRingDqTs * kKTile + 1024 + 1024;

__global__ void __launch_bounds__(320, 1)
fmha_bwd_dq_ts_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, const BwdParams p) {
    if ((int)blockIdx.x >= *p.n_tiles) return;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sK = smem;                               // [kRingDqTs] 16 KiB each
    uint8_t* sV = sK + kRingDqTs * kKTile;            // [kRingDqTs]
    uint8_t* sQstage = sK;                            // Q / dO (32 KiB each) pass through the rings' first slots
    uint8_t* sdOstage = sV;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + kRingDqTs * kKTile);
    uint64_t* q_full = bars + 0;
    uint64_t* q_done = bars + 1;
    uint64_t* k_full = bars + 2;                      // [R]
    uint64_t* k_empty = k_full + kRingDqTs;
    uint64_t* v_full = k_empty + kRingDqTs;
    uint64_t* v_empty = v_full + kRingDqTs;
    uint64_t* s_full = v_empty + kRingDqTs;           // [2]
    uint64_t* s_empty = s_full + 2;                   // [2]
    uint64_t* dp_full = s_full + 4;
    uint64_t* ds_full = s_full + 5;
    uint64_t* dq_full = s_full + 6;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 7);
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
    const int n_kv = max(0, (kv_end + BK - 1) / BK);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(q_done, 256);
        for (int i = 0; i < kRingDqTs; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&s_empty[i], 256);
        }
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
    // Q : 0..63, dO : 64..127 (bf16 pairs), S[2] : 128..255, dP (then dS) : 256..319, dQ : 320..447
    const uint32_t tQ = tmem_base, tdO = tmem_base + 64, tS = tmem_base + 128, tdP = tmem_base + 256, tdQ = tmem_base + 320;

    if (warp == 0) {
        if (lane == 0 && n_kv > 0) {
            mbar_expect_tx(q_full, 2 * kTile);
            tma_load_3d(sQstage, &tmQ, q_full, 0, head, q_begin + q0);
            tma_load_3d(sQstage + kAtom, &tmQ, q_full, 64, head, q_begin + q0);
            tma_load_3d(sdOstage, &tmdO, q_full, 0, head, q_begin + q0);
            tma_load_3d(sdOstage + kAtom, &tmdO, q_full, 64, head, q_begin + q0);
            bool ok = mbar_wait(q_done, 0, abort_flag);
            for (int j = 0; j < n_kv && ok; ++j) {
                const int st = j % kRingDqTs;
                const uint32_t ph = (j / kRingDqTs) & 1;
                const int row = k_begin + j * BK;
                if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag)) { ok = false; break; }
                mbar_expect_tx(&k_full[st], kKTile);
                tma_load_3d(sK + st * kKTile, &tmK, &k_full[st], 0, kv_head, row);
                tma_load_3d(sK + st * kKTile + kKAtom, &tmK, &k_full[st], 64, kv_head, row);
                if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag)) { ok = false; break; }
                mbar_expect_tx(&v_full[st], kKTile);
                tma_load_3d(sV + st * kKTile, &tmV, &v_full[st], 0, kv_head, row);
                tma_load_3d(sV + st * kKTile + kKAtom, &tmV, &v_full[st], 64, kv_head, row);
            }
            if (!ok) atomicExch(p.status, MM_TIMEOUT_TMA);
        }
    } else if (warp == 1) {
        if (lane == 0 && n_kv > 0) {
            constexpr uint32_t idesc_s = idesc_bf16(128, BK, 0, 0);
            constexpr uint32_t idesc_dq = idesc_bf16(128, HD, 0, 1);
            bool ok = mbar_wait(q_done, 0, abort_flag);
            auto issue_s = [&](int j) -> bool {
                const int st = j % kRingDqTs, b = j & 1;
                const uint32_t ph = (j / kRingDqTs) & 1, bph = (j >> 1) & 1;
                if (!mbar_wait(&s_empty[b], bph ^ 1, abort_flag) || !mbar_wait(&k_full[st], ph, abort_flag)) return false;
                fence_after_sync();
                const uint32_t ka = smem_u32(sK + st * kKTile);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    mma_ts(tS + b * BK, tQ + k * 8, smem_desc_sw128(ka + (k >> 2) * kKAtom + (k & 3) * 32, 16, 1024), idesc_s,
                           k ? 1u : 0u);
                mma_commit(&s_full[b]);
                return true;
            };
            auto issue_dp = [&](int j) -> bool {
                const int st = j % kRingDqTs;
                const uint32_t ph = (j / kRingDqTs) & 1;
                if (!mbar_wait(&v_full[st], ph, abort_flag)) return false;
                fence_after_sync();
                const uint32_t va = smem_u32(sV + st * kKTile);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    mma_ts(tdP, tdO + k * 8, smem_desc_sw128(va + (k >> 2) * kKAtom + (k & 3) * 32, 16, 1024), idesc_s,
                           k ? 1u : 0u);
                mma_commit(dp_full);
                mma_commit(&v_empty[st]);
                return true;
            };
            if (ok) ok = issue_s(0);
            if (ok) ok = issue_dp(0);
            if (ok && n_kv > 1) ok = issue_s(1);
            for (int j = 0; j < n_kv && ok; ++j) {
                const int st = j % kRingDqTs;
                if (!mbar_wait(ds_full, j & 1, abort_flag)) { ok = false; break; }
                fence_after_sync();
                const uint32_t ka = smem_u32(sK + st * kKTile);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)
                    mma_ts(tdQ, tdP + (k >> 1) * 32 + (k & 1) * 8, smem_desc_sw128(ka + k * 2048, kKAtom, 1024), idesc_dq,
                           (j | k) ? 1u : 0u);
                mma_commit(&k_empty[st]);
                if (j + 1 < n_kv && !(ok = issue_dp(j + 1))) break;        // same columns as dS(j): after dQ(j) in the pipe
                if (j + 2 < n_kv && !(ok = issue_s(j + 2))) break;
            }
            if (ok) mma_commit(dq_full);
            if (!ok) atomicExch(p.status, MM_TIMEOUT_MMA);
        }
    } else {
        const int half = (warp - 2) >> 2;
        const int qd = warp & 3;
        const int row = qd * 32 + lane;
        const int qi = q0 + row;
        const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
        const bool row_ok = qi < q_len;
        bool ok = true;
        if (n_kv > 0) {
            ok = mbar_wait(q_full, 0, abort_flag);
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
        const size_t stat = (size_t)head * p.T + q_begin + min(qi, max(q_len - 1, 0));
        const float lse2 = n_kv > 0 ? p.lse[stat] * kLog2e : 0.f;
        const float dlt = n_kv > 0 ? p.delta[stat] : 0.f;
        const int limit = !row_ok ? -1 : (p.causal ? min(k_len - 1, qi + diag) : k_len - 1);
        for (int j = 0; j < n_kv && ok; ++j) {
            const int b = j & 1;
            if (!mbar_wait(&s_full[b], (j >> 1) & 1, abort_flag)) { ok = false; break; }
            fence_after_sync();
            uint32_t r[32], d[32];
            tmem_ld_32x32(tS + b * BK + half * 32 + lane_off, r);
            tmem_wait_ld();
            fence_before_sync();
            mbar_arrive(&s_empty[b]);
            const int kbase = j * BK + half * 32;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float pr = exp2f(__uint_as_float(r[i]) * p.scale_log2 - lse2);
                r[i] = __float_as_uint(kbase + i > limit ? 0.f : pr);
            }
            if (!mbar_wait(dp_full, j & 1, abort_flag)) { ok = false; break; }
            fence_after_sync();
            tmem_ld_32x32(tdP + half * 32 + lane_off, d);
            tmem_wait_ld();
            uint32_t w[16];
#pragma unroll
            for (int i = 0; i < 16; ++i)
                w[i] = pack2(__uint_as_float(r[2 * i]) * (__uint_as_float(d[2 * i]) - dlt),
                             __uint_as_float(r[2 * i + 1]) * (__uint_as_float(d[2 * i + 1]) - dlt));
            tmem_st_32x16(tdP + half * 32 + lane_off, w);
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
