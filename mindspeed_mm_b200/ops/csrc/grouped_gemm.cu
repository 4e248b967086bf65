// Grouped (per-expert) bf16 GEMMs for MoE on tcgen05, all three passes, on an ALIGNED token layout:
// the rows of expert e are [off[e], off[e+1]) with every off a multiple of 128 (pad rows are zero), so no tile
// ever straddles two experts and TMA stores need no clipping.
//
//   mode 0 (fwd)   y[r, :]  = x[r, :]  @ W[e]        x [R, K]  W [E, K, N]  y [R, N]
//   mode 1 (dgrad) dx[r, :] = dy[r, :] @ W[e]^T      dy [R, N]              dx [R, K]
//   mode 2 (wgrad) dW[e]    = x_e^T @ dy_e           contraction over the expert's rows; dW [E, K, N]
//
// A one-thread planner turns the device-side offsets into a tile list (expert, row block, column block); the
// persistent CTAs (TMA producer / MMA issuer / 4 epilogue warps, TMEM double buffer: same pipeline as gemm.cu; output
// tiles 128 x 256, or 128 x 128 when the tiled dimension is not a multiple of 256)
// walk that list, so routing skew costs nothing but the tiles it produces.  Experts without tokens produce no
// tiles (wgrad output is pre-zeroed by the caller).  Reference op: torch_npu.npu_grouped_matmul with group_list
// (mindspeed_mm/fsdp/ops/moe_ops/gemm.py:16-92).
#include "tc05.cuh"

namespace {

using namespace tc05;

constexpr int BM = 128, BK = 64;
constexpr int kThreads = 192, kEpiThreads = 128;
constexpr int kABytes = BM * BK * 2;
constexpr int kCBytes = 2 * BM * 64 * 2;

// Output tiles are 128 x 256 when the tiled output dimension allows it (the tensor pipe reads the A tile once per 256
// columns instead of once per 128: the 128 x 128 tile is bound by shared-memory operand reads), else 128 x 128.
template <int BN>
struct Cfg {
    static constexpr int kBBytes = BN * BK * 2, kStageBytes = kABytes + kBBytes;
    static constexpr int kStages = BN == 256 ? 4 : 6;
    static constexpr int kSmem = kStages * kStageBytes + kCBytes + 2048;
    static constexpr int kTmemCols = 2 * BN;
};

struct GGParams {
    const int* off;          // [E + 1] aligned row offsets (device)
    const int* tile_e;       // planner output
    const int* tile_m;
    const int* tile_n;
    const int* n_tiles;
    int K, N;                // weight shape [E, K, N]
    int* status;
};

// modes 0/1: one tile per (expert row block, output column block); mode 2: per (expert, K block, N block)
__global__ void gg_plan_kernel(const int* off, int E, int mode, int K, int N, int BN, int* tile_e, int* tile_m, int* tile_n,
                               int* n_tiles, int max_tiles) {
    if (threadIdx.x || blockIdx.x) return;
    int n = 0;
    if (mode == 2) {
        for (int e = 0; e < E; ++e) {
            if (off[e + 1] == off[e]) continue;
            for (int nb = 0; nb < N / BN; ++nb)
                for (int mb = 0; mb < K / BM && n < max_tiles; ++mb) {
                    tile_e[n] = e; tile_m[n] = mb; tile_n[n] = nb; ++n;
                }
        }
    } else {
        const int cols = (mode == 0 ? N : K) / BN;
        for (int e = 0; e < E; ++e)
            for (int nb = 0; nb < cols; ++nb)
                for (int r = off[e]; r < off[e + 1] && n < max_tiles; r += BM) {
                    tile_e[n] = e; tile_m[n] = r / BM; tile_n[n] = nb; ++n;
                }
    }
    *n_tiles = n;
}

template <int MODE, int BN>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, GGParams p) {
    constexpr int kBBytes = Cfg<BN>::kBBytes, kStageBytes = Cfg<BN>::kStageBytes, kStages = Cfg<BN>::kStages;
    constexpr int kTmemCols = Cfg<BN>::kTmemCols;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = sA + kStages * kABytes;
    uint8_t* sC = sB + kStages * kBBytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(sC + kCBytes);
    uint64_t* empty = full + kStages;
    uint64_t* tfull = empty + kStages;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* epi_stop = abort_flag + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = *p.n_tiles;
    auto kblocks = [&](int e) { return MODE == 2 ? (p.off[e + 1] - p.off[e]) / BK : (MODE == 0 ? p.K : p.N) / BK; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
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
        prefetch_tmap(&tmC);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                const int e = p.tile_e[t], mb = p.tile_m[t], nb = p.tile_n[t];
                const int kbs = kblocks(e);
                for (int kb = 0; kb < kbs; ++kb) {
                    if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
                        atomicExch(p.status, MM_TIMEOUT_TMA);
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&full[stage], kStageBytes);
                    uint8_t* a = sA + stage * kABytes;
                    uint8_t* b = sB + stage * kBBytes;
                    if constexpr (MODE == 0) {
                        tma_load_2d(a, &tmA, &full[stage], kb * BK, mb * BM);
#pragma unroll
                        for (int a64 = 0; a64 < BN / 64; ++a64)                                   // W[e][k, n], N-contiguous: one
                            tma_load_3d(b + a64 * BK * 128, &tmB, &full[stage], nb * BN + 64 * a64, kb * BK, e);   // atom per 64 n
                    } else if constexpr (MODE == 1) {
                        tma_load_2d(a, &tmA, &full[stage], kb * BK, mb * BM);
                        tma_load_3d(b, &tmB, &full[stage], kb * BK, nb * BN, e);                 // rows = K (output), contraction = N
                    } else {
                        const int r0 = p.off[e] + kb * BK;
                        tma_load_2d(a, &tmA, &full[stage], mb * BM, r0);                         // x[r, k]: M = k index
                        tma_load_2d(a + BK * 128, &tmA, &full[stage], mb * BM + 64, r0);
#pragma unroll
                        for (int a64 = 0; a64 < BN / 64; ++a64)                                   // dy[r, n]
                            tma_load_2d(b + a64 * BK * 128, &tmB, &full[stage], nb * BN + 64 * a64, r0);
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr bool A_MN = MODE == 2, B_MN = MODE != 1;
            constexpr uint32_t idesc = idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
            int stage = 0, it = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++it) {
                const int kbs = kblocks(p.tile_e[t]);
                const int acc = it & 1;
                if (!mbar_wait(&tempty[acc], ((it >> 1) & 1) ^ 1, abort_flag)) {
                    atomicExch(p.status, MM_TIMEOUT_MMA);
                    break;
                }
                fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < kbs; ++kb) {
                    if (!mbar_wait(&full[stage], phase, abort_flag)) {
                        atomicExch(p.status, MM_TIMEOUT_MMA);
                        ok = false;
                        break;
                    }
                    fence_after_sync();
                    const uint32_t a0 = smem_u32(sA + stage * kABytes), b0 = smem_u32(sB + stage * kBBytes);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t da = A_MN ? smem_desc_sw128(a0 + k * 2048, BK * 128, 1024) : smem_desc_sw128(a0 + k * 32, 16, 1024);
                        const uint64_t db = B_MN ? smem_desc_sw128(b0 + k * 2048, BK * 128, 1024) : smem_desc_sw128(b0 + k * 32, 16, 1024);
                        mma_ss(d_tmem, da, db, idesc, (kb | k) ? 1u : 0u);
                    }
                    mma_commit(&empty[stage]);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (ok) mma_commit(&tfull[acc]);
            }
        }
    } else {
        const int q = warp & 3, row = q * 32 + lane;
        const bool issuer = threadIdx.x == 64;
        int it = 0, slab_count = 0;
        for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++it) {
            const int e = p.tile_e[t], mb = p.tile_m[t], nb = p.tile_n[t];
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
                    if constexpr (MODE == 2) tma_store_3d(&tmC, buf, nb * BN + slab * 64, mb * BM, e);
                    else tma_store_2d(&tmC, buf, nb * BN + slab * 64, mb * BM);
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
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

template <int MODE, int BN>
int launch(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tC, const GGParams& p, int grid, cudaStream_t st) {
    auto kern = grouped_gemm_kernel<MODE, BN>;
    static bool done = false;
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::kSmem);
        if (e != cudaSuccess) return (int)e;
        done = true;
    }
    kern<<<grid, kThreads, Cfg<BN>::kSmem, st>>>(tA, tB, tC, p);
    return (int)cudaGetLastError();
}

}  // namespace

// Upper bound of the tile count (128-wide column blocks; the 256-wide plan has at most as many).
MM_API int mm_grouped_gemm_max_tiles(int R, int E, int K, int N, int mode) {
    if (mode == 2) return E * (K / BM) * (N / 128) + 1;
    return (R / BM + E) * ((mode == 0 ? N : K) / 128) + 1;
}

// a, b, c by mode:  0: a = x [R,K], b = W [E,K,N], c = y [R,N]      1: a = dy [R,N], b = W, c = dx [R,K]
//                   2: a = x [R,K], b = dy [R,N], c = dW [E,K,N] (zero it first)
// off: int32 [E+1] on the device, multiples of 128, off[E] <= R.  plan: int32 scratch of 3 * max_tiles + 1.
// K and N must be multiples of 128.
MM_API int mm_grouped_gemm_bf16(const void* a, const void* b, void* c, const int* off, int* plan, int R, int E, int K, int N,
                                int mode, int* status, cudaStream_t st) {
    if (K % 128 || N % 128 || R % 128 || mode < 0 || mode > 2) return -1;
    const int max_tiles = mm_grouped_gemm_max_tiles(R, E, K, N, mode);
    int* tile_e = plan;
    int* tile_m = plan + max_tiles;
    int* tile_n = plan + 2 * max_tiles;
    int* n_tiles = plan + 3 * max_tiles;
    const int BN = ((mode == 1 ? K : N) % 256 == 0) ? 256 : 128;      // the dimension the column blocks tile
    gg_plan_kernel<<<1, 32, 0, st>>>(off, E, mode, K, N, BN, tile_e, tile_m, tile_n, n_tiles, max_tiles);
    CUtensorMap tA, tB, tC;
    int r;
    if (mode == 0) {
        if ((r = make_tmap_2d(&tA, a, R, K, K, BM, BK))) return 1000 + r;
        if ((r = make_tmap_3d(&tB, b, N, K, E, N, (uint64_t)K * N, 64, BK, 1))) return 2000 + r;
        if ((r = make_tmap_2d(&tC, c, R, N, N, BM, 64))) return 3000 + r;
    } else if (mode == 1) {
        if ((r = make_tmap_2d(&tA, a, R, N, N, BM, BK))) return 1000 + r;
        if ((r = make_tmap_3d(&tB, b, N, K, E, N, (uint64_t)K * N, BK, BN, 1))) return 2000 + r;
        if ((r = make_tmap_2d(&tC, c, R, K, K, BM, 64))) return 3000 + r;
    } else {
        if ((r = make_tmap_2d(&tA, a, R, K, K, BK, 64))) return 1000 + r;      // boxes of 64 rows (contraction) x 64 k
        if ((r = make_tmap_2d(&tB, b, R, N, N, BK, 64))) return 2000 + r;
        if ((r = make_tmap_3d(&tC, c, N, K, E, N, (uint64_t)K * N, 64, BM, 1))) return 3000 + r;
    }
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    GGParams p{off, tile_e, tile_m, tile_n, n_tiles, K, N, status};
    const int grid = max_tiles - 1 < sms ? (max_tiles - 1 < 1 ? 1 : max_tiles - 1) : sms;
    if (BN == 256) {
        if (mode == 0) return launch<0, 256>(tA, tB, tC, p, grid, st);
        if (mode == 1) return launch<1, 256>(tA, tB, tC, p, grid, st);
        return launch<2, 256>(tA, tB, tC, p, grid, st);
    }
    if (mode == 0) return launch<0, 128>(tA, tB, tC, p, grid, st);
    if (mode == 1) return launch<1, 128>(tA, tB, tC, p, grid, st);
    return launch<2, 128>(tA, tB, tC, p, grid, st);
}

// ------------------------------------------------------------------------------------------ permute / unpermute
namespace {
// dst_row[i] for every (token, slot) pair i = t * k + s, in the aligned expert-major layout; pad rows get -1 source.
__global__ void moe_permute_kernel(const bf16* __restrict__ x, const int* __restrict__ src_of_row, bf16* __restrict__ out,
                                   int R, int H) {
    const int hv = H >> 3;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)R * hv;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / hv), c = (int)(i % hv);
        const int s = src_of_row[r];
        Vec8 v;
        if (s >= 0) v = reinterpret_cast<const Vec8*>(x + (size_t)s * H)[c];
        else {
#pragma unroll
            for (int k = 0; k < 4; ++k) v.v[k] = __floats2bfloat162_rn(0.f, 0.f);
        }
        reinterpret_cast<Vec8*>(out + (size_t)r * H)[c] = v;
    }
}
// out[t, :] = sum_s probs[t, s] * y[row_of_pair[t * k + s], :]
__global__ void moe_unpermute_kernel(const bf16* __restrict__ y, const int* __restrict__ row_of_pair,
                                     const bf16* __restrict__ probs, bf16* __restrict__ out, int T, int k, int H) {
    const int hv = H >> 3;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)T * hv;
         i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / hv), c = (int)(i % hv);
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int s = 0; s < k; ++s) {
            const float w = __bfloat162float(probs[t * k + s]);
            float f[8];
            unpack8(reinterpret_cast<const Vec8*>(y + (size_t)row_of_pair[t * k + s] * H)[c], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += w * f[j];
        }
        reinterpret_cast<Vec8*>(out + (size_t)t * H)[c] = pack8(acc);
    }
}
}  // namespace

MM_API int mm_moe_permute(const void* x, const int* src_of_row, void* out, int R, int H, cudaStream_t st) {
    if (H % 8) return -1;
    long long work = (long long)R * (H / 8);
    int grid = (int)((work + 255) / 256 < 148 * 16 ? (work + 255) / 256 : 148 * 16);
    moe_permute_kernel<<<grid < 1 ? 1 : grid, 256, 0, st>>>((const bf16*)x, src_of_row, (bf16*)out, R, H);
    return (int)cudaGetLastError();
}

MM_API int mm_moe_unpermute(const void* y, const int* row_of_pair, const void* probs, void* out, int T, int k, int H,
                            cudaStream_t st) {
    if (H % 8) return -1;
    long long work = (long long)T * (H / 8);
    int grid = (int)((work + 255) / 256 < 148 * 16 ? (work + 255) / 256 : 148 * 16);
    moe_unpermute_kernel<<<grid < 1 ? 1 : grid, 256, 0, st>>>((const bf16*)y, row_of_pair, (const bf16*)probs, (bf16*)out, T, k, H);
    return (int)cudaGetLastError();
}
