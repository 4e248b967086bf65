// Persistent, warp-specialised bf16 GEMM on the 5th-gen tensor cores.
//
//   C[M,N] (bf16) = op(A) * op(B) (+ bias[N])        fp32 accumulation in TMEM
//
// Operand layouts (both row-major in memory):
//   A_MN = 0: A is [M, K] (K contiguous)      A_MN = 1: A is stored as [K, M] (M contiguous)
//   B_MN = 0: B is [N, K] (K contiguous)      B_MN = 1: B is stored as [K, N] (N contiguous)
// so forward  y = x W^T      is (A_MN=0, B_MN=0) on (x [T,K], W [N,K]),
//    dgrad    dx = dy W      is (A_MN=0, B_MN=1) on (dy [T,N], W [N,K] read as [K'=N, N'=K]),
//    wgrad    dW = dy^T x    is (A_MN=1, B_MN=1) on (dy [T,N] read as [K'=T, M'=N], x [T,K] read as [K'=T, N'=K]).
//
// One CTA per SM walks output tiles of 128 x BN.  Roles:
//   warp 0     : TMA producer  (cp.async.bulk.tensor into a multi-stage 128B-swizzled smem ring)
//   warp 1     : MMA issuer    (one elected thread issues tcgen05.mma; tcgen05.commit frees ring slots)
//   warps 2..5 : epilogue      (tcgen05.ld TMEM -> registers -> bf16 -> swizzled smem -> TMA store)
// The accumulator is double-buffered in TMEM (2 x BN columns) so the epilogue of tile i overlaps the main
// loop of tile i+1.  Tiles are visited in groups of 8 M-blocks per N sweep to keep A/B tiles L2-resident.
// All mbarrier waits are bounded (tc05::mbar_wait); a timeout is reported through `status` and the CTA
// unwinds: it lets in-flight copies land, frees its TMEM and returns.
#include "tc05.cuh"

namespace {

using namespace tc05;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kThreads = 192;
constexpr int kEpiThreads = 128;
constexpr int kSmemBudget = 227 * 1024;

template <int BN>
struct Cfg {
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kBBytes = BN * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kCBytes = 2 * BM * 64 * 2;  // two 128x64 bf16 staging slabs
    static constexpr int kAux = 1024;                // barriers etc.
    static constexpr int kStages = (kSmemBudget - kCBytes - kAux - 1024) / kStageBytes;
    static constexpr int kSmem = kStages * kStageBytes + kCBytes + kAux + 1024;
    static constexpr int kTmemCols = 2 * BN;
};

struct Params {
    int M, N, K;
    const bf16* bias;
    int* status;
    int group_m;
    // output routing (fused all-to-all / reduce-scatter push): where a 128 x 64 output slab goes
    //   mode 0: C[m, n] of this GPU
    //   mode 1: column blocks of width `blk` are dealt round-robin to `world` destinations (Ulysses head scatter):
    //           dst = (n / blk) % world, column (n / (blk * world)) * blk + n % blk, row row_off + m
    //   mode 2: row blocks of `blk` rows go to destination m / blk, stored at row rank * blk + m % blk
    //           (every source has its own slot on the destination, which then sums the slots)
    int mode, blk, world, rank, row_off;
    // optional side output: stats[m * n_slots + n / per_slot] += sum over the tile's columns of (bf16-rounded output)^2,
    // i.e. the sum of squares of every output row per column group, taken from the accumulators (a normalisation over
    // the whole row can then be applied after the columns have been scattered to other GPUs)
    float* stats = nullptr;
    int n_slots = 1, per_slot = 0;
};

constexpr int kMaxDst = 8;
struct TMapSet {
    CUtensorMap m[kMaxDst];
};

__device__ __forceinline__ void tile_coords(int tile, int m_blocks, int n_blocks, int group_m, int& mb, int& nb) {
    const int per_group = group_m * n_blocks;
    const int g = tile / per_group;
    const int first_m = g * group_m;
    const int gm = min(group_m, m_blocks - first_m);
    const int r = tile - g * per_group;
    mb = first_m + r % gm;
    nb = r / gm;
}

// SWIGLU (BN = 256, K-major operands, no bias): B is the fused [2F, K] gate/up weight, p.N = F.  A tile's accumulator holds
// 128 gate columns (weight rows nb*128 ..) next to the 128 up columns of the same features (rows F + nb*128 ..); the
// epilogue writes silu(gate) * up, so the [M, 2F] pre-activation never reaches memory.
template <int BN, bool A_MN, bool B_MN, bool SWIGLU = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ TMapSet tmC, Params p) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + C::kStages * C::kABytes;
    uint8_t* sC = sB + C::kStages * C::kBBytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(sC + C::kCBytes);
    uint64_t* empty = full + C::kStages;
    uint64_t* tfull = empty + C::kStages;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* epi_stop = abort_flag + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int m_blocks = (p.M + BM - 1) / BM;
    const int n_blocks = SWIGLU ? p.N / 128 : (p.N + BN - 1) / BN;
    const int n_tiles = m_blocks * n_blocks;
    const int k_blocks = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&tfull[a], 1);
            mbar_init(&tempty[a], kEpiThreads);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
        for (int d = 0; d < (p.mode ? p.world : 1); ++d) prefetch_tmap(&tmC.m[d]);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::kTmemCols);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                int mb, nb;
                tile_coords(tile, m_blocks, n_blocks, p.group_m, mb, nb);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
                        atomicExch(p.status, MM_TIMEOUT_TMA);
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&full[stage], C::kStageBytes);
                    uint8_t* a = sA + stage * C::kABytes;
                    uint8_t* b = sB + stage * C::kBBytes;
                    if constexpr (!A_MN) {
                        tma_load_2d(a, &tmA, &full[stage], kb * BK, mb * BM);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j)
                            tma_load_2d(a + j * (BK * 128), &tmA, &full[stage], mb * BM + j * 64, kb * BK);
                    }
                    if constexpr (SWIGLU) {
                        tma_load_2d(b, &tmB, &full[stage], kb * BK, nb * 128);
                        tma_load_2d(b + 128 * 128, &tmB, &full[stage], kb * BK, p.N + nb * 128);
                    } else if constexpr (!B_MN) {
                        tma_load_2d(b, &tmB, &full[stage], kb * BK, nb * BN);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            tma_load_2d(b + j * (BK * 128), &tmB, &full[stage], nb * BN + j * 64, kb * BK);
                    }
                    if (++stage == C::kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
                const int acc = it & 1;
                if (!mbar_wait(&tempty[acc], ((it >> 1) & 1) ^ 1, abort_flag)) {
                    atomicExch(p.status, MM_TIMEOUT_MMA);
                    break;
                }
                fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&full[stage], phase, abort_flag)) {
                        atomicExch(p.status, MM_TIMEOUT_MMA);
                        ok = false;
                        break;
                    }
                    fence_after_sync();
                    const uint32_t a0 = smem_u32(sA + stage * C::kABytes);
                    const uint32_t b0 = smem_u32(sB + stage * C::kBBytes);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        // K-major: 16 elements of K = 32 bytes inside the swizzle atom.
                        // MN-major: 16 rows of K = two 8-row groups = 2048 bytes.
                        const uint64_t da = A_MN ? smem_desc_sw128(a0 + k * 2048, BK * 128, 1024)
                                                 : smem_desc_sw128(a0 + k * 32, 16, 1024);
                        const uint64_t db = B_MN ? smem_desc_sw128(b0 + k * 2048, BK * 128, 1024)
                                                 : smem_desc_sw128(b0 + k * 32, 16, 1024);
                        mma_ss(d_tmem, da, db, idesc, (kb | k) ? 1u : 0u);
                    }
                    mma_commit(&empty[stage]);  // slot reusable once these MMAs have read it
                    if (++stage == C::kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (ok) mma_commit(&tfull[acc]);
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int q = warp & 3;            // TMEM lane quarter this warp may read
        const int row = q * 32 + lane;     // row inside the 128-row tile
        const bool issuer = threadIdx.x == 64;
        int it = 0;
        int slab_count = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
            int mb, nb;
            tile_coords(tile, m_blocks, n_blocks, p.group_m, mb, nb);
            const int acc = it & 1;
            if (!mbar_wait(&tfull[acc], (it >> 1) & 1, abort_flag) && lane == 0) atomicExch(p.status, MM_TIMEOUT_EPI);
            // make the go / no-go decision identical for all 128 epilogue threads before any bar.sync below
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (issuer) *epi_stop = *abort_flag;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*epi_stop) break;
            fence_after_sync();
            const uint32_t t_row = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
            constexpr int kSlabs = SWIGLU ? 2 : BN / 64;
#pragma unroll 1
            for (int slab = 0; slab < kSlabs; ++slab, ++slab_count) {
                uint8_t* buf = sC + (slab_count & 1) * (BM * 128);
                if (issuer) tma_wait_read<1>();  // the store that last read this buffer has drained
                asm volatile("bar.sync 1, 128;" ::: "memory");
                uint32_t r[64];
                if constexpr (SWIGLU) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        uint32_t u[32];
                        tmem_ld_32x32(t_row + slab * 64 + h * 32, r + h * 32);
                        tmem_ld_32x32(t_row + 128 + slab * 64 + h * 32, u);
                        tmem_wait_ld();
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            const float g = __uint_as_float(r[h * 32 + c]);
                            r[h * 32 + c] = __float_as_uint(__fdividef(g, 1.f + __expf(-g)) * __uint_as_float(u[c]));
                        }
                    }
                } else {
                    tmem_ld_32x32(t_row + slab * 64, r);
                    tmem_ld_32x32(t_row + slab * 64 + 32, r + 32);
                    tmem_wait_ld();
                }
                const int n0 = (SWIGLU ? nb * 128 : nb * BN) + slab * 64;
                if (!SWIGLU && p.bias != nullptr) {
#pragma unroll
                    for (int c = 0; c < 64; ++c) {
                        const int n = n0 + c;
                        const float bv = n < p.N ? __bfloat162float(p.bias[n]) : 0.f;
                        r[c] = __float_as_uint(__uint_as_float(r[c]) + bv);
                    }
                }
                if (!SWIGLU && p.stats != nullptr) {
                    float ss = 0.f;
#pragma unroll
                    for (int c = 0; c < 64; ++c) {
                        const float v = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[c])));
                        ss += (n0 + c < p.N) ? v * v : 0.f;
                    }
                    const int m = mb * BM + row;
                    if (m < p.M && n0 < p.N) atomicAdd(&p.stats[(size_t)m * p.n_slots + n0 / p.per_slot], ss);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    uint4 v;
                    bf162 t0 = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
                    bf162 t1 = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
                    bf162 t2 = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
                    bf162 t3 = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
                    v.x = *reinterpret_cast<uint32_t*>(&t0);
                    v.y = *reinterpret_cast<uint32_t*>(&t1);
                    v.z = *reinterpret_cast<uint32_t*>(&t2);
                    v.w = *reinterpret_cast<uint32_t*>(&t3);
                    *reinterpret_cast<uint4*>(buf + row * 128 + ((j ^ (row & 7)) << 4)) = v;
                }
                fence_proxy_async();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (issuer) {
                    if (p.mode == 0) {
                        tma_store_2d(&tmC.m[0], buf, n0, mb * BM);
                    } else if (p.mode == 1) {
                        const int b = n0 / p.blk;
                        tma_store_2d(&tmC.m[b % p.world], buf, (b / p.world) * p.blk + n0 % p.blk, p.row_off + mb * BM);
                    } else {
                        const int m0 = mb * BM;
                        tma_store_2d(&tmC.m[m0 / p.blk], buf, n0, p.rank * p.blk + m0 % p.blk);
                    }
                    tma_commit();
                }
            }
            fence_before_sync();
            mbar_arrive(&tempty[acc]);
        }
        if (issuer) tma_wait_all<0>();
    }

    // ---------------------------------------------------------------------- teardown
    if (*abort_flag) {
        // give copies that may still be in flight time to land before the CTA's smem is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        fence_after_sync();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

struct Route {
    int mode = 0, blk = 0, world = 1, rank = 0, row_off = 0;
    void* const* dst = nullptr;     // mode != 0: `world` destination base pointers (peer-mapped)
    long long dst_rows = 0, dst_cols = 0;
    float* stats = nullptr;         // see Params::stats
    int n_slots = 1;
};

template <int BN, bool A_MN, bool B_MN, bool SWIGLU = false>
int launch(const void* A, const void* B, void* Cc, const void* bias, int M, int N, int K, long long lda, long long ldb,
           long long ldc, int* status, cudaStream_t st, const Route& rt = Route()) {
    using C = Cfg<BN>;
    CUtensorMap tA, tB;
    TMapSet tC;
    int r;
    // A_MN: memory is [K, M] -> rows=K, cols=M, box = 64 k-rows x 64 m ;  else rows=M, cols=K, box = 128 x 64
    r = A_MN ? make_tmap_2d(&tA, A, K, M, lda, BK, 64) : make_tmap_2d(&tA, A, M, K, lda, BM, BK);
    if (r) return 1000 + r;
    if (SWIGLU)
        r = make_tmap_2d(&tB, B, 2LL * N, K, ldb, 128, BK);      // gate and up halves are fetched as two 128-row boxes
    else
        r = B_MN ? make_tmap_2d(&tB, B, K, N, ldb, BK, 64) : make_tmap_2d(&tB, B, N, K, ldb, BN, BK);
    if (r) return 2000 + r;
    if (rt.mode == 0) {
        r = make_tmap_2d(&tC.m[0], Cc, M, N, ldc, BM, 64);
        if (r) return 3000 + r;
    } else {
        if (rt.world > kMaxDst) return -5;
        for (int d = 0; d < rt.world; ++d) {
            if (rt.mode == 1) {
                // this launch owns rows [row_off, row_off + M) of every destination: the map covers exactly those, so the
                // last (partial) row tile is clipped instead of spilling into the next source's rows
                if (rt.row_off + (long long)M > rt.dst_rows) return -6;
                r = make_tmap_2d(&tC.m[d], (const char*)rt.dst[d] + (size_t)rt.row_off * ldc * 2, M, rt.dst_cols, ldc, BM, 64);
            } else {
                r = make_tmap_2d(&tC.m[d], rt.dst[d], rt.dst_rows, rt.dst_cols, ldc, BM, 64);
            }
            if (r) return 3000 + r;
        }
    }
    auto kern = gemm_kernel<BN, A_MN, B_MN, SWIGLU>;
    static bool done = false;
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
        if (e != cudaSuccess) return (int)e;
        done = true;
    }
    const int m_blocks = (M + BM - 1) / BM, n_blocks = SWIGLU ? N / 128 : (N + BN - 1) / BN;
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    const int tiles = m_blocks * n_blocks;
    Params p{M, N, K, (const bf16*)bias, status, 8, rt.mode, rt.blk, rt.world, rt.rank, rt.mode == 1 ? 0 : rt.row_off,
             rt.stats, rt.n_slots, rt.n_slots > 0 ? N / rt.n_slots : N};
    const int grid = tiles < sms ? tiles : sms;
    kern<<<grid, kThreads, C::kSmem, st>>>(tA, tB, tC, p);
    return (int)cudaGetLastError();
}

}  // namespace

// lda/ldb/ldc: elements between consecutive rows of the tensors as laid out in memory.
// Requirements: base pointers 16-byte aligned; ld* multiples of 8; `status` is a device int (0 = ok).
MM_API int mm_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                        long long ldb, long long ldc, int a_mn, int b_mn, int bn, int* status, cudaStream_t st) {
    if ((lda | ldb | ldc) % 8) return -1;
    if (((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) & 15) return -2;
    if (M <= 0 || N <= 0 || K <= 0) return -3;
#define MM_DISPATCH(BN_)                                                                                          \
    if (!a_mn && !b_mn) return launch<BN_, false, false>(A, B, C, bias, M, N, K, lda, ldb, ldc, status, st);      \
    if (!a_mn && b_mn) return launch<BN_, false, true>(A, B, C, bias, M, N, K, lda, ldb, ldc, status, st);        \
    if (a_mn && !b_mn) return launch<BN_, true, false>(A, B, C, bias, M, N, K, lda, ldb, ldc, status, st);        \
    return launch<BN_, true, true>(A, B, C, bias, M, N, K, lda, ldb, ldc, status, st);
    if (bn == 128) {
        MM_DISPATCH(128)
    }
    MM_DISPATCH(256)
#undef MM_DISPATCH
}


// C[M, F] = silu(A W_gate^T) * (A W_up^T) with W = [W_gate; W_up] stored as one [2F, K] matrix.  F % 128 == 0.
MM_API int mm_gemm_swiglu_bf16(const void* A, const void* W, void* C, int M, int F, int K, long long lda, long long ldw,
                               long long ldc, int* status, cudaStream_t st) {
    if ((lda | ldw | ldc) % 8) return -1;
    if (((uintptr_t)A | (uintptr_t)W | (uintptr_t)C) & 15) return -2;
    if (M <= 0 || F <= 0 || K <= 0 || F % 128) return -3;
    return launch<256, false, false, true>(A, W, C, nullptr, M, F, K, lda, ldw, ldc, status, st);
}


// Routed output (the collective is the epilogue: slabs are written straight into the destinations' buffers over
// NVLink).  K-major operands (y = x W^T + bias).  mode 1: all-to-all of column blocks (Ulysses head scatter),
// requires blk % 64 == 0; mode 2: push of row blocks into per-source slots (first half of a reduce-scatter),
// requires blk % 128 == 0.  dst[d]: base of destination d's [dst_rows, dst_cols] bf16 buffer with row pitch ldc.
// b_mn = 1: B is stored [K, N] row-major (the NN product of a data-gradient GEMM) instead of [N, K].
MM_API int mm_gemm_bf16_routed_ex(const void* A, const void* B, const void* bias, int M, int N, int K, long long lda,
                                  long long ldb, void* const* dst, long long dst_rows, long long dst_cols, long long ldc,
                                  int mode, int blk, int world, int rank, int row_off, int b_mn, int* status,
                                  cudaStream_t st) {
    if ((lda | ldb | ldc) % 8) return -1;
    if (((uintptr_t)A | (uintptr_t)B) & 15) return -2;
    if (mode == 1 && (blk % 64 || N % (blk * world))) return -3;
    if (mode == 2 && (blk % 128 || M != blk * world)) return -3;
    if (mode != 1 && mode != 2) return -4;
    Route rt;
    rt.mode = mode; rt.blk = blk; rt.world = world; rt.rank = rank; rt.row_off = row_off;
    rt.dst = dst; rt.dst_rows = dst_rows; rt.dst_cols = dst_cols;
    const bool wide = (mode == 1 && blk % 256 == 0) || (mode == 2 && N >= 256);
    if (b_mn) {
        if (wide) return launch<256, false, true>(A, B, nullptr, bias, M, N, K, lda, ldb, ldc, status, st, rt);
        return launch<128, false, true>(A, B, nullptr, bias, M, N, K, lda, ldb, ldc, status, st, rt);
    }
    if (wide) return launch<256, false, false>(A, B, nullptr, bias, M, N, K, lda, ldb, ldc, status, st, rt);
    return launch<128, false, false>(A, B, nullptr, bias, M, N, K, lda, ldb, ldc, status, st, rt);
}

// Mode 1 (K-major operands) with the row statistics side output: stats [M, n_slots] fp32, zeroed by the caller, receives
// the sum of squares of each output row over each of the n_slots equal column groups (q | k | v).
MM_API int mm_gemm_bf16_routed_stats(const void* A, const void* B, const void* bias, int M, int N, int K, long long lda,
                                     long long ldb, void* const* dst, long long dst_rows, long long dst_cols, long long ldc,
                                     int blk, int world, int rank, int row_off, float* stats, int n_slots, int* status,
                                     cudaStream_t st) {
    if ((lda | ldb | ldc) % 8) return -1;
    if (((uintptr_t)A | (uintptr_t)B) & 15) return -2;
    if (blk % 64 || N % (blk * world) || n_slots < 1 || N % n_slots || (N / n_slots) % 64) return -3;
    Route rt;
    rt.mode = 1; rt.blk = blk; rt.world = world; rt.rank = rank; rt.row_off = row_off;
    rt.dst = dst; rt.dst_rows = dst_rows; rt.dst_cols = dst_cols;
    rt.stats = stats; rt.n_slots = n_slots;
    if (blk % 256 == 0) return launch<256, false, false>(A, B, nullptr, bias, M, N, K, lda, ldb, ldc, status, st, rt);
    return launch<128, false, false>(A, B, nullptr, bias, M, N, K, lda, ldb, ldc, status, st, rt);
}

MM_API int mm_gemm_bf16_routed(const void* A, const void* B, const void* bias, int M, int N, int K, long long lda,
                               long long ldb, void* const* dst, long long dst_rows, long long dst_cols, long long ldc,
                               int mode, int blk, int world, int rank, int row_off, int* status, cudaStream_t st) {
    return mm_gemm_bf16_routed_ex(A, B, bias, M, N, K, lda, ldb, dst, dst_rows, dst_cols, ldc, mode, blk, world, rank,
                                  row_off, 0, status, st);
}

// out[r, :] = sum_s slots[s * rows + r, :]   (second half of the reduce-scatter: fold the per-source slots)
namespace {
__global__ void fold_slots_kernel(const bf16* __restrict__ slots, bf16* __restrict__ out, long long rows, int cols,
                                  long long pitch, int world) {
    const int cv = cols >> 3;
    const long long total = rows * cv;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cv;
        const int c = (int)(i - r * cv);
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int s = 0; s < world; ++s) {
            float f[8];
            unpack8(reinterpret_cast<const Vec8*>(slots + (s * rows + r) * pitch)[c], f);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] += f[k];
        }
        reinterpret_cast<Vec8*>(out + r * cols)[c] = pack8(acc);
    }
}
}  // namespace

MM_API int mm_fold_slots(const void* slots, void* out, long long rows, int cols, long long pitch, int world, cudaStream_t st) {
    if (cols % 8 || pitch % 8) return -1;
    long long work = rows * (cols / 8);
    int grid = (int)((work + 255) / 256 < 148 * 8 ? (work + 255) / 256 : 148 * 8);
    fold_slots_kernel<<<grid < 1 ? 1 : grid, 256, 0, st>>>((const bf16*)slots, (bf16*)out, rows, cols, pitch, world);
    return (int)cudaGetLastError();
}
