// Collectives issued from kernels over NVLink peer memory (no NCCL on this path).
//
// Every rank owns a symmetric arena (same layout on every GPU, peer base pointers exchanged once).  The
// kernels below take a table of peer pointers and use plain loads/stores on them: NVSwitch gives every
// pair full bandwidth, so each collective is one hop and "pull" based - the consumer reads what it needs
// from the producers' memory:
//
//   mm_p2p_allgather      full[p*S + i] = shard_p[i]                      (ZeRO-3 parameter gather)
//   mm_p2p_rs_adamw       g = sum_p grad_p[r*S + i] / div  (bf16 on the wire, fp32 accumulate)
//                         -> AdamW on this rank's fp32 master/moments -> bf16 shard    (one pass)
//   mm_p2p_rs             same reduction, written (or accumulated) as fp32 for a deferred update
//
// They use no shared memory and few registers, so they co-reside on SMs that a persistent tcgen05 GEMM
// (1 CTA/SM, all shared memory) is using, and overlap with it from a side stream.
//
// Cross-rank ordering uses sequence-numbered flags in the arena (st.release.sys / ld.acquire.sys):
//   ready[slot]        written by the owner once its gradients for publication `seq` are in `slot`
//   done[slot][peer]   written by each reader into the OWNER's arena once it has finished reading
// Waits are bounded (~8 s); on timeout the kernel records MM_TIMEOUT_PEER in `status`, skips its work and
// returns, leaving the context usable.
#include "common.cuh"

namespace {

constexpr int kMaxPeers = 16;
struct Peers {
    void* p[kMaxPeers];
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Limit of every peer-flag wait in cycles (default 2^34, about 9 s); mm_p2p_set_wait_limit changes it, e.g. so that a
// test of the time-out path finishes in a fraction of a second.
__device__ long long g_wait_limit = 1LL << 34;

// true when *flag >= want (sequence numbers only grow); false once the limit has passed.
__device__ bool wait_flag_geq(const uint32_t* flag, uint32_t want) {
    const long long t0 = clock64();
    const long long limit = g_wait_limit;
    while ((int32_t)(ld_acquire_sys(flag) - want) < 0) {
        if (clock64() - t0 > limit) return false;
        __nanosleep(200);
    }
    return true;
}

struct uint4x {
    uint4 v;
};

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// ------------------------------------------------------------------------------------------ all-gather
// Peers are visited in a rank-staggered round-robin of 64 KiB chunks so that at any moment every link
// carries traffic and no owner is read by all ranks at once.
__global__ void __launch_bounds__(256) p2p_allgather_kernel(Peers shards, uint4* __restrict__ full, long long shard_vec,
                                                            int world, int rank) {
    constexpr long long kChunk = 4096;  // uint4 per chunk = 64 KiB
    const long long chunks_per_peer = (shard_vec + kChunk - 1) / kChunk;
    const long long total_chunks = chunks_per_peer * world;
    for (long long c = blockIdx.x; c < total_chunks; c += gridDim.x) {
        const int hop = (int)(c % world);
        const int peer = (rank + 1 + hop) % world;  // own shard comes last in each round
        const long long chunk = c / world;
        const long long base = chunk * kChunk;
        const long long n = min(kChunk, shard_vec - base);
        const uint4* src = reinterpret_cast<const uint4*>(shards.p[peer]) + base;
        uint4* dst = full + peer * shard_vec + base;
        for (long long i = threadIdx.x; i < n; i += 4 * 256) {
            uint4 r[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (i + u * 256 < n) r[u] = ld_stream(src + i + u * 256);
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (i + u * 256 < n) dst[i + u * 256] = r[u];
        }
    }
}

// ------------------------------------------------------------------------------------------ reduce-scatter (+AdamW)
struct RSParams {
    Peers grads;          // each rank's flat bf16 gradient buffer for this slot (full length)
    Peers flags;          // each rank's flag block
    long long shard_elems;
    int world, rank, slot;
    uint32_t seq;
    float inv_div;
    int* status;
    uint32_t* counter;    // local, zero between launches
};
// flag block layout (uint32): ready[2] | done[2][kMaxPeers]
__device__ __forceinline__ uint32_t* flag_ready(void* base, int slot) { return reinterpret_cast<uint32_t*>(base) + slot; }
__device__ __forceinline__ uint32_t* flag_done(void* base, int slot, int peer) {
    return reinterpret_cast<uint32_t*>(base) + 2 + slot * kMaxPeers + peer;
}

__device__ bool rs_prologue(const RSParams& P) {
    __shared__ int ok_s;
    if (threadIdx.x == 0) ok_s = 1;
    __syncthreads();
    // every CTA checks every peer itself: no CTA depends on another CTA of this launch
    if (threadIdx.x < P.world && threadIdx.x != P.rank) {
        if (!wait_flag_geq(flag_ready(P.flags.p[threadIdx.x], P.slot), P.seq)) {
            atomicExch(P.status, MM_TIMEOUT_PEER);
            ok_s = 0;
        }
    }
    __syncthreads();
    return ok_s != 0;
}

__device__ void rs_epilogue(const RSParams& P) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t prev = atomicAdd(P.counter, 1u);
        if (prev == gridDim.x - 1) {
            *P.counter = 0;
            __threadfence_system();
            for (int p = 0; p < P.world; ++p)
                if (p != P.rank) st_release_sys(flag_done(P.flags.p[p], P.slot, P.rank), P.seq);
        }
    }
}

__device__ __forceinline__ void reduce8(const RSParams& P, long long vec_idx, float* acc, uint64_t pol) {
    const long long off = (long long)P.rank * (P.shard_elems >> 3) + vec_idx;
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    uint4 r[kMaxPeers];
#pragma unroll
    for (int p = 0; p < kMaxPeers; ++p)
        if (p < P.world) r[p] = ld_stream_u4(reinterpret_cast<const uint4*>(P.grads.p[p]) + off, pol);
#pragma unroll
    for (int p = 0; p < kMaxPeers; ++p)
        if (p < P.world) {
            float f[8];
            unpack8(*reinterpret_cast<const Vec8*>(&r[p]), f);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] += f[k];
        }
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] *= P.inv_div;
}

struct AdamParams {
    float* p;
    float* m;
    float* v;
    bf16* p16;
    long long split;
    float lr, b1, b2, eps, wd, bc1, bc2;
};

__global__ void __launch_bounds__(256) p2p_rs_adamw_kernel(RSParams P, AdamParams A) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        __threadfence_system();
        st_release_sys(flag_ready(P.flags.p[P.rank], P.slot), P.seq);  // publish: my gradients are in place
    }
    const uint64_t pol = l2_evict_first_policy();
    // A CTA whose wait ran out skips the reduction (the peer's gradients are not there) but still takes part in the
    // epilogue: the arrival counter returns to zero and the slot is handed back, so the next launch on this slot works.
    const long long nvec = rs_prologue(P) ? (P.shard_elems >> 3) : 0;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
        float g[8];
        reduce8(P, i, g, pol);
        const float4* Pp = reinterpret_cast<const float4*>(A.p) + 2 * i;
        const float4* Mp = reinterpret_cast<const float4*>(A.m) + 2 * i;
        const float4* Vp = reinterpret_cast<const float4*>(A.v) + 2 * i;
        float4 p0 = ld_stream_f4(Pp, pol), p1 = ld_stream_f4(Pp + 1, pol);
        float4 m0 = ld_stream_f4(Mp, pol), m1 = ld_stream_f4(Mp + 1, pol);
        float4 v0 = ld_stream_f4(Vp, pol), v1 = ld_stream_f4(Vp + 1, pol);
        float pp[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
        float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
        float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float decay = (i * 8 + k) < A.split ? A.wd : 0.f;
            mm[k] = A.b1 * mm[k] + (1.f - A.b1) * g[k];
            vv[k] = A.b2 * vv[k] + (1.f - A.b2) * g[k] * g[k];
            pp[k] = pp[k] * (1.f - A.lr * decay) - A.lr * (mm[k] / A.bc1) / (sqrtf(vv[k] / A.bc2) + A.eps);
        }
        st_stream_f4(reinterpret_cast<float4*>(A.p) + 2 * i, make_float4(pp[0], pp[1], pp[2], pp[3]), pol);
        st_stream_f4(reinterpret_cast<float4*>(A.p) + 2 * i + 1, make_float4(pp[4], pp[5], pp[6], pp[7]), pol);
        st_stream_f4(reinterpret_cast<float4*>(A.m) + 2 * i, make_float4(mm[0], mm[1], mm[2], mm[3]), pol);
        st_stream_f4(reinterpret_cast<float4*>(A.m) + 2 * i + 1, make_float4(mm[4], mm[5], mm[6], mm[7]), pol);
        st_stream_f4(reinterpret_cast<float4*>(A.v) + 2 * i, make_float4(vv[0], vv[1], vv[2], vv[3]), pol);
        st_stream_f4(reinterpret_cast<float4*>(A.v) + 2 * i + 1, make_float4(vv[4], vv[5], vv[6], vv[7]), pol);
        reinterpret_cast<Vec8*>(A.p16)[i] = pack8(pp);
    }
    rs_epilogue(P);
}

__global__ void __launch_bounds__(256) p2p_rs_kernel(RSParams P, float* __restrict__ out, int accumulate) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        __threadfence_system();
        st_release_sys(flag_ready(P.flags.p[P.rank], P.slot), P.seq);
    }
    const uint64_t pol = l2_evict_first_policy();
    const long long nvec = rs_prologue(P) ? (P.shard_elems >> 3) : 0;   // see p2p_rs_adamw_kernel
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
        float g[8];
        reduce8(P, i, g, pol);
        float4* o = reinterpret_cast<float4*>(out) + 2 * i;
        if (accumulate) {
            float4 a = o[0], b = o[1];
            g[0] += a.x; g[1] += a.y; g[2] += a.z; g[3] += a.w;
            g[4] += b.x; g[5] += b.y; g[6] += b.z; g[7] += b.w;
        }
        o[0] = make_float4(g[0], g[1], g[2], g[3]);
        o[1] = make_float4(g[4], g[5], g[6], g[7]);
    }
    rs_epilogue(P);
}

// Owner-side wait before a gradient slot is overwritten: all readers of publication `seq` are done.
__global__ void p2p_wait_done_kernel(void* my_flags, int slot, uint32_t seq, int world, int rank, int* status) {
    if (threadIdx.x < world && threadIdx.x != rank) {
        if (!wait_flag_geq(flag_done(my_flags, slot, threadIdx.x), seq)) atomicExch(status, MM_TIMEOUT_PEER);
    }
}

// ------------------------------------------------------------------------------------------ arena barrier
// bar[p] in MY block = the last barrier number that rank p has reached.  Arrival: write my number into my entry of
// every rank's block (release, system scope: everything this stream wrote before the barrier is visible to a peer that
// acquires the flag); then wait until every entry of my own block has reached the number.  The wait is bounded like
// every other peer wait: on expiry MM_TIMEOUT_PEER goes to the status word and the kernel returns.
__global__ void p2p_barrier_kernel(Peers bars, int world, int rank, uint32_t seq, int* status) {
    const int p = threadIdx.x;
    if (p >= world) return;
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(bars.p[p]) + rank, seq);
    if (!wait_flag_geq(reinterpret_cast<const uint32_t*>(bars.p[rank]) + p, seq)) atomicExch(status, MM_TIMEOUT_PEER);
}

// ------------------------------------------------------------------------------------------ MoE row exchange
// Expert-parallel dispatch / combine as direct peer memory traffic: a token row goes straight from the sender's
// activation tensor into its slot of the destination rank's expert slab (and back), so the all-to-all and the
// permute are one pass over the data.  Row maps are computed on the host side of the op from the exchanged
// per-expert histograms.  One warp moves one row with 16-byte accesses.
//   scatter: peer[dst_rank[i]][dst_row[i]] = src[src_row[i]]            (push)
//   gather : out[i] = peer[dst_rank[i]][dst_row[i]]                      (pull)
__global__ void __launch_bounds__(256) p2p_scatter_rows_kernel(const uint4* __restrict__ src, const int* __restrict__ src_row,
                                                               const int* __restrict__ dst_rank,
                                                               const int* __restrict__ dst_row, Peers bufs, int n, int row_vec) {
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (i >= n) return;
    const int lane = threadIdx.x & 31;
    const uint4* s = src + (size_t)src_row[i] * row_vec;
    uint4* d = reinterpret_cast<uint4*>(bufs.p[dst_rank[i]]) + (size_t)dst_row[i] * row_vec;
    for (int v = lane; v < row_vec; v += 32) d[v] = s[v];
}

__global__ void __launch_bounds__(256) p2p_gather_rows_kernel(uint4* __restrict__ out, const int* __restrict__ dst_rank,
                                                              const int* __restrict__ dst_row, Peers bufs, int n, int row_vec) {
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (i >= n) return;
    const int lane = threadIdx.x & 31;
    const uint4* s = reinterpret_cast<const uint4*>(bufs.p[dst_rank[i]]) + (size_t)dst_row[i] * row_vec;
    uint4* d = out + (size_t)i * row_vec;
    for (int v = lane; v < row_vec; v += 32) d[v] = ld_stream(s + v);
}

// ------------------------------------------------------------------------------------------ plain peer copy
// dst <- src for `n_vec` 16-byte vectors; either side may be a peer-mapped address (pull or push).  Used by ring
// attention to bring the next K/V block into local memory while the current block is being computed.
__global__ void __launch_bounds__(256) p2p_copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, long long n_vec) {
    const long long stride = (long long)gridDim.x * blockDim.x * 4;
    for (long long i = (long long)blockIdx.x * blockDim.x * 4 + threadIdx.x; i < n_vec; i += stride) {
        uint4 r[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i + u * 256 < n_vec) r[u] = ld_stream(src + i + u * 256);
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i + u * 256 < n_vec) dst[i + u * 256] = r[u];
    }
}

Peers make_peers(void* const* ptrs, int world) {
    Peers P;
    for (int i = 0; i < kMaxPeers; ++i) P.p[i] = i < world ? ptrs[i] : nullptr;
    return P;
}

}  // namespace

MM_API int mm_p2p_flag_bytes() { return (2 + 2 * kMaxPeers + 2) * 4; }

// shard_ptrs[p]: address of rank p's shard (peer-mapped); full: local destination of world*shard_elems bf16.
MM_API int mm_p2p_allgather(void* const* shard_ptrs, void* full, long long shard_elems, int world, int rank, int ctas,
                            cudaStream_t st) {
    if (world > kMaxPeers || shard_elems % 8) return -1;
    p2p_allgather_kernel<<<ctas, 256, 0, st>>>(make_peers(shard_ptrs, world), (uint4*)full, shard_elems / 8, world, rank);
    return (int)cudaGetLastError();
}

// The same gather on the copy engines: one cudaMemcpyAsync per peer shard (peer-mapped source, local destination), in
// the same rank-staggered order, own shard last.  No SM is used, so a GEMM that owns every SM keeps them; the copies
// are ordered on `st` like a kernel would be.
MM_API int mm_p2p_allgather_ce(void* const* shard_ptrs, void* full, long long shard_bytes, int world, int rank,
                               cudaStream_t st) {
    if (world > kMaxPeers) return -1;
    for (int hop = 0; hop < world; ++hop) {
        const int peer = (rank + 1 + hop) % world;
        cudaError_t e = cudaMemcpyAsync(reinterpret_cast<char*>(full) + (size_t)peer * shard_bytes, shard_ptrs[peer],
                                        (size_t)shard_bytes, cudaMemcpyDeviceToDevice, st);
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

MM_API int mm_p2p_rs_adamw(void* const* grad_ptrs, void* const* flag_ptrs, long long shard_elems, int world, int rank,
                           int slot, unsigned seq, float inv_div, float* p, float* m, float* v, void* p16,
                           long long split, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                           int* status, int ctas, cudaStream_t st) {
    if (world > kMaxPeers || shard_elems % 8) return -1;
    RSParams P{make_peers(grad_ptrs, world), make_peers(flag_ptrs, world), shard_elems, world, rank, slot, seq, inv_div,
               status, reinterpret_cast<uint32_t*>(flag_ptrs[rank]) + 2 + 2 * kMaxPeers};
    AdamParams A{p, m, v, (bf16*)p16, split, lr, b1, b2, eps, wd, bc1, bc2};
    p2p_rs_adamw_kernel<<<ctas, 256, 0, st>>>(P, A);
    return (int)cudaGetLastError();
}

MM_API int mm_p2p_rs(void* const* grad_ptrs, void* const* flag_ptrs, long long shard_elems, int world, int rank, int slot,
                     unsigned seq, float inv_div, float* out, int accumulate, int* status, int ctas, cudaStream_t st) {
    if (world > kMaxPeers || shard_elems % 8) return -1;
    RSParams P{make_peers(grad_ptrs, world), make_peers(flag_ptrs, world), shard_elems, world, rank, slot, seq, inv_div,
               status, reinterpret_cast<uint32_t*>(flag_ptrs[rank]) + 2 + 2 * kMaxPeers};
    p2p_rs_kernel<<<ctas, 256, 0, st>>>(P, out, accumulate);
    return (int)cudaGetLastError();
}

MM_API int mm_p2p_barrier_bytes() { return kMaxPeers * 4; }

// bar_ptrs[p]: address of rank p's barrier block (kMaxPeers uint32, zero at start); seq: 1, 2, 3, ... per arena.
MM_API int mm_p2p_barrier(void* const* bar_ptrs, int world, int rank, unsigned seq, int* status, cudaStream_t st) {
    if (world > kMaxPeers) return -1;
    p2p_barrier_kernel<<<1, 32, 0, st>>>(make_peers(bar_ptrs, world), world, rank, seq, status);
    return (int)cudaGetLastError();
}

MM_API int mm_p2p_wait_done(void* my_flags, int slot, unsigned seq, int world, int rank, int* status, cudaStream_t st) {
    p2p_wait_done_kernel<<<1, 32, 0, st>>>(my_flags, slot, seq, world, rank, status);
    return (int)cudaGetLastError();
}

// src: [*, H] bf16 local; src_row / dst_rank / dst_row: int32 [n] on the device; buf_ptrs[p]: rank p's slab (peer-mapped).
MM_API int mm_p2p_scatter_rows(const void* src, const int* src_row, const int* dst_rank, const int* dst_row,
                               void* const* buf_ptrs, int n, int H, int world, cudaStream_t st) {
    if (world > kMaxPeers || H % 8) return -1;
    if (n == 0) return 0;
    p2p_scatter_rows_kernel<<<(n + 7) / 8, 256, 0, st>>>((const uint4*)src, src_row, dst_rank, dst_row, make_peers(buf_ptrs, world),
                                                         n, H / 8);
    return (int)cudaGetLastError();
}

MM_API int mm_p2p_gather_rows(void* out, const int* dst_rank, const int* dst_row, void* const* buf_ptrs, int n, int H,
                              int world, cudaStream_t st) {
    if (world > kMaxPeers || H % 8) return -1;
    if (n == 0) return 0;
    p2p_gather_rows_kernel<<<(n + 7) / 8, 256, 0, st>>>((uint4*)out, dst_rank, dst_row, make_peers(buf_ptrs, world), n, H / 8);
    return (int)cudaGetLastError();
}

MM_API int mm_p2p_copy(void* dst, const void* src, long long nbytes, int ctas, cudaStream_t st) {
    if (nbytes % 16 || ((uintptr_t)dst | (uintptr_t)src) & 15) return -1;
    if (nbytes == 0) return 0;
    p2p_copy_kernel<<<ctas, 256, 0, st>>>((uint4*)dst, (const uint4*)src, nbytes / 16);
    return (int)cudaGetLastError();
}

// cycles <= 0 restores the default.  Applies to kernels launched afterwards on the current device.
MM_API int mm_p2p_set_wait_limit(long long cycles) {
    const long long v = cycles > 0 ? cycles : (1LL << 34);
    return (int)cudaMemcpyToSymbol(g_wait_limit, &v, sizeof(v));
}
