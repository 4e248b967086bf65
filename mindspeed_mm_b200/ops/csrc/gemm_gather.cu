// All-gather fused into the consuming GEMM:  C = gather(A) * B^T (+bias), where slabs of A live in peers' memory.
//
// Same persistent tcgen05 pipeline as gemm.cu (TMA producer, MMA issuer, 4 epilogue warps, TMEM double buffer)
// plus ONE extra warp per CTA that is the collective: its elected thread walks 128 x 64 boxes of the remote
// slabs, TMA-loads each box from the peer's memory into a small shared-memory ring (plain, non-multicast TMA
// loads on a peer-mapped tensor map) and TMA-stores it into this GPU's own copy of A.  When a CTA has stored
// all of its boxes of slab s it bumps flags[s]; the producer warp only issues loads of A tiles from a slab whose
// counter shows that all CTAs have delivered (bounded wait).  Tiles that only need the local slab are scheduled
// first, so the tensor cores start at once and the NVLink transfer hides under the math, tile by tile.
//
//   axis 0 (rows)   : slab s = rows [s*extent, (s+1)*extent) of A      (sequence-parallel all-gather -> column-parallel GEMM)
//   axis 2 (columns): slab s = K columns [s*extent, (s+1)*extent) of A (Ulysses output projection: heads come back from peers)
// Every remote tile crosses NVLink exactly once and is read by the GEMM from local memory.  flags[] are monotonic
// counters (target = epoch * gridDim.x), so nothing has to be cleared between launches.
#include "tc05.cuh"

namespace {

using namespace tc05;

constexpr int BM = 128, BK = 64;
constexpr int kThreads = 224;          // 7 warps: TMA, MMA, 4 x epilogue, gather
constexpr int kEpiThreads = 128;
constexpr int kMaxPeers = 8;
constexpr int kRingSlots = 2;
constexpr int kBoxBytes = BM * BK * 2;  // 16 KiB

template <int BN>
struct Cfg {
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kBBytes = BN * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kCBytes = 2 * BM * 64 * 2;
    static constexpr int kRingBytes = kRingSlots * kBoxBytes;
    static constexpr int kStages = (227 * 1024 - kCBytes - kRingBytes - 2048) / kStageBytes;
    static constexpr int kSmem = kStages * kStageBytes + kCBytes + kRingBytes + 2048;
    static constexpr int kTmemCols = 2 * BN;
};

struct TMapSet {
    CUtensorMap m[kMaxPeers];
};

struct GParams {
    int M, N, K;
    const bf16* bias;
    int* status;
    int axis, extent, world, rank;
    int src_rows, src_cols;      // shape of one remote slab
    uint32_t* flags;             // [world] monotonic arrival counters (device memory of this GPU)
    uint32_t target;             // epoch * gridDim.x
};

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

__device__ bool wait_slab(const uint32_t* flag, uint32_t target, volatile int* abort_flag) {
    if ((int32_t)(ld_acquire_gpu(flag) - target) >= 0) return true;
    const long long t0 = clock64();
    while ((int32_t)(ld_acquire_gpu(flag) - target) < 0) {
        if (*abort_flag) return false;
        if (clock64() - t0 > (1LL << 32)) {
            *abort_flag = 1;
            return false;
        }
        __nanosleep(100);
    }
    return true;
}

// B_MN = false: B is [N, K] (K contiguous, y = gather(A) B^T); B_MN = true: B is stored [K, N] (N contiguous: the
// data-gradient product dx = gather(g) W with W [N', K'] read as [K = N', N = K']).
template <int BN, bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_gather_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmC, const __grid_constant__ TMapSet tmSrc, GParams p) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = sA + C::kStages * C::kABytes;
    uint8_t* sC = sB + C::kStages * C::kBBytes;
    uint8_t* sR = sC + C::kCBytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(sR + C::kRingBytes);
    uint64_t* empty = full + C::kStages;
    uint64_t* tfull = empty + C::kStages;
    uint64_t* tempty = tfull + 2;
    uint64_t* rbar = tempty + 2;                      // [kRingSlots]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(rbar + kRingSlots);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* epi_stop = abort_flag + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_blocks = (p.M + BM - 1) / BM, n_blocks = (p.N + BN - 1) / BN;
    const int n_tiles = m_blocks * n_blocks;
    const int k_blocks = (p.K + BK - 1) / BK;
    // local-slab-first visiting order
    const int rot_m = p.axis == 0 ? (p.rank * p.extent) / BM : 0;
    const int rot_k = p.axis == 2 ? (p.rank * p.extent) / BK : 0;
    auto coords = [&](int tile, int& mb, int& nb) {
        // M-major inside an N sweep of 8 row blocks: neighbouring CTAs share B tiles; rows rotated to start local
        const int gm = 8;
        const int per_group = gm * n_blocks;
        const int g = tile / per_group;
        const int first = g * gm;
        const int cnt = min(gm, m_blocks - first);
        const int r = tile - g * per_group;
        mb = (first + r % cnt + rot_m) % m_blocks;
        nb = r / cnt;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&tfull[a], 1);
            mbar_init(&tempty[a], kEpiThreads);
        }
        for (int r = 0; r < kRingSlots; ++r) mbar_init(&rbar[r], 1);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
        prefetch_tmap(&tmC);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::kTmemCols);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 6) {
        // ------------------------------------------------------------------ gather: peer -> smem ring -> local A
        if (lane == 0) {
            const int bx = (p.src_cols + BK - 1) / BK, by = (p.src_rows + BM - 1) / BM;
            const int boxes = bx * by;
            uint32_t issued = 0;
            bool ok = true;
            for (int hop = 1; hop < p.world && ok; ++hop) {
                const int s = (p.rank + hop) % p.world;           // staggered: every rank reads a different peer
                const int dx = p.axis == 2 ? s * p.extent : 0, dy = p.axis == 0 ? s * p.extent : 0;
                for (int b = blockIdx.x; b < boxes; b += gridDim.x, ++issued) {
                    const int slot = issued % kRingSlots;
                    const uint32_t ph = (issued / kRingSlots) & 1;
                    const int x = (b % bx) * BK, y = (b / bx) * BM;
                    if (issued >= kRingSlots) tma_wait_read<kRingSlots - 1>();   // the store that used this slot has read it
                    mbar_expect_tx(&rbar[slot], kBoxBytes);
                    tma_load_2d(sR + slot * kBoxBytes, &tmSrc.m[s], &rbar[slot], x, y);
                    if (!mbar_wait(&rbar[slot], ph, abort_flag)) {
                        atomicExch(p.status, MM_TIMEOUT_PEER);
                        ok = false;
                        break;
                    }
                    tma_store_2d(&tmA, sR + slot * kBoxBytes, x + dx, y + dy);
                    tma_commit();
                }
                if (!ok) break;
                tma_wait_all<0>();                 // this CTA's part of slab s is in local memory
                fence_proxy_async_all();
                __threadfence();
                atomicAdd(&p.flags[s], 1u);
            }
        }
    } else if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int ready_mask = 1 << p.rank;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                int mb, nb;
                coords(tile, mb, nb);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    const int kbe = (kb + rot_k) % k_blocks;
                    const int slab = p.axis == 0 ? min((mb * BM) / p.extent, p.world - 1) : min((kbe * BK) / p.extent, p.world - 1);
                    if (!(ready_mask >> slab & 1)) {
                        if (!wait_slab(&p.flags[slab], p.target, abort_flag)) {
                            atomicExch(p.status, MM_TIMEOUT_PEER);
                            ok = false;
                            break;
                        }
                        fence_proxy_async_all();
                        ready_mask |= 1 << slab;
                    }
                    if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
                        atomicExch(p.status, MM_TIMEOUT_TMA);
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&full[stage], C::kStageBytes);
                    tma_load_2d(sA + stage * C::kABytes, &tmA, &full[stage], kbe * BK, mb * BM);
                    if constexpr (!B_MN) {
                        tma_load_2d(sB + stage * C::kBBytes, &tmB, &full[stage], kbe * BK, nb * BN);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            tma_load_2d(sB + stage * C::kBBytes + j * (BK * 128), &tmB, &full[stage], nb * BN + j * 64, kbe * BK);
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
            constexpr uint32_t idesc = idesc_bf16(BM, BN, 0, B_MN ? 1 : 0);
            int stage = 0, it = 0;
            uint32_t phase = 0;
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
                    const uint32_t a0 = smem_u32(sA + stage * C::kABytes), b0 = smem_u32(sB + stage * C::kBBytes);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t db = B_MN ? smem_desc_sw128(b0 + k * 2048, BK * 128, 1024)
                                                 : smem_desc_sw128(b0 + k * 32, 16, 1024);
                        mma_ss(d_tmem, smem_desc_sw128(a0 + k * 32, 16, 1024), db, idesc, (kb | k) ? 1u : 0u);
                    }
                    mma_commit(&empty[stage]);
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
        const int q = warp & 3, row = q * 32 + lane;
        const bool issuer = threadIdx.x == 64;
        int it = 0, slab_count = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
            int mb, nb;
            coords(tile, mb, nb);
            const int acc = it & 1;
            if (!mbar_wait(&tfull[acc], (it >> 1) & 1, abort_flag) && lane == 0) atomicExch(p.status, MM_TIMEOUT_EPI);
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (issuer) *epi_stop = *abort_flag;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*epi_stop) break;
            fence_after_sync();
            const uint32_t t_row = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int slab = 0; slab < BN / 64; ++slab, ++slab_count) {
                uint8_t* buf = sC + (slab_count & 1) * (BM * 128);
                if (issuer) tma_wait_read<1>();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                uint32_t r[64];
                tmem_ld_32x32(t_row + slab * 64, r);
                tmem_ld_32x32(t_row + slab * 64 + 32, r + 32);
                tmem_wait_ld();
                const int n0 = nb * BN + slab * 64;
                if (p.bias != nullptr) {
#pragma unroll
                    for (int c = 0; c < 64; ++c) {
                        const float bv = n0 + c < p.N ? __bfloat162float(p.bias[n0 + c]) : 0.f;
                        r[c] = __float_as_uint(__uint_as_float(r[c]) + bv);
                    }
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
                    tma_store_2d(&tmC, buf, n0, mb * BM);
                    tma_commit();
                }
            }
            fence_before_sync();
            mbar_arrive(&tempty[acc]);
        }
        if (issuer) tma_wait_all<0>();
    }

    if (*abort_flag)
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        fence_after_sync();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

template <int BN, bool B_MN>
int launch(const void* A, const void* B, void* Cc, const void* bias, int M, int N, int K, long long lda, long long ldb,
           long long ldc, void* const* src, long long src_pitch, int src_rows, int src_cols, int axis, int extent, int world,
           int rank, uint32_t* flags, uint32_t epoch, int* status, cudaStream_t st) {
    using C = Cfg<BN>;
    CUtensorMap tA, tB, tC;
    TMapSet tS;
    int r;
    if ((r = make_tmap_2d(&tA, A, M, K, lda, BM, BK))) return 1000 + r;
    if ((r = B_MN ? make_tmap_2d(&tB, B, K, N, ldb, BK, 64) : make_tmap_2d(&tB, B, N, K, ldb, BN, BK))) return 2000 + r;
    if ((r = make_tmap_2d(&tC, Cc, M, N, ldc, BM, 64))) return 3000 + r;
    for (int s = 0; s < world; ++s) {
        if (s == rank) {
            tS.m[s] = tA;
            continue;
        }
        if ((r = make_tmap_2d(&tS.m[s], src[s], src_rows, src_cols, src_pitch, BM, BK))) return 4000 + r;
    }
    for (int s = world; s < kMaxPeers; ++s) tS.m[s] = tA;
    auto kern = gemm_gather_kernel<BN, B_MN>;
    static bool done = false;
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
        if (e != cudaSuccess) return (int)e;
        done = true;
    }
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int grid = tiles < sms ? tiles : sms;
    GParams p{M, N, K, (const bf16*)bias, status, axis, extent, world, rank, src_rows, src_cols, flags, epoch * (uint32_t)grid};
    kern<<<grid, kThreads, C::kSmem, st>>>(tA, tB, tC, tS, p);
    return (int)cudaGetLastError();
}

}  // namespace

// A: this GPU's full-size [M, K] operand; its own slab must already be in place, the others are filled by the
// kernel from src[s] (peer-mapped base of rank s's [src_rows, src_cols] slab, row pitch src_pitch elements).
// axis 0: extent = rows per slab (multiple of 128); axis 2: extent = K columns per slab (multiple of 64).
// flags: `world` uint32 counters in this GPU's memory, zero before the first launch; epoch = 1, 2, 3 ... per launch
// with the same grid.  The caller brackets the launch with a cross-rank barrier (sources stable / consumed).
MM_API int mm_gemm_gather_bf16_ex(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                                  long long ldb, long long ldc, void* const* src, long long src_pitch, int src_rows,
                                  int src_cols, int axis, int extent, int world, int rank, unsigned* flags, unsigned epoch,
                                  int b_mn, int* status, cudaStream_t st) {
    if ((lda | ldb | ldc | src_pitch) % 8) return -1;
    if (world > kMaxPeers || (axis != 0 && axis != 2)) return -2;
    if ((axis == 0 && extent % BM) || (axis == 2 && extent % BK)) return -3;
#define MM_GG(BN_, MN_)                                                                                                     \
    return launch<BN_, MN_>(A, B, C, bias, M, N, K, lda, ldb, ldc, src, src_pitch, src_rows, src_cols, axis, extent, world, \
                            rank, flags, epoch, status, st)
    if (N >= 256) {
        if (b_mn) MM_GG(256, true);
        MM_GG(256, false);
    }
    if (b_mn) MM_GG(128, true);
    MM_GG(128, false);
#undef MM_GG
}

// b_mn = 0 form (y = gather(A) B^T with B [N, K]).
MM_API int mm_gemm_gather_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                               long long ldb, long long ldc, void* const* src, long long src_pitch, int src_rows,
                               int src_cols, int axis, int extent, int world, int rank, unsigned* flags, unsigned epoch,
                               int* status, cudaStream_t st) {
    return mm_gemm_gather_bf16_ex(A, B, C, bias, M, N, K, lda, ldb, ldc, src, src_pitch, src_rows, src_cols, axis, extent,
                                  world, rank, flags, epoch, 0, status, st);
}
