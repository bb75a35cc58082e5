// LayerNorm / RMSNorm (+ fused activation) forward and backward, bulk-async
// variant for sm_100a: one persistent CTA of 16 warps per SM.  Tiles of whole
// rows stream from HBM into a shared-memory ring with cp.async.bulk (TMA, this
// CTA only, no multicast) completing on mbarriers; the warps read the tiles from
// shared memory, reduce the row statistics with warp shuffles and write the
// outputs with 16-byte coalesced stores.  The bytes in flight per SM are the
// ring, independent of register use, so HBM stays busy while rows are reduced.
//
// There is no dedicated producer warp: 16 warps is 4 per scheduler, which leaves
// each thread 128 registers (a 17th warp would cut that to 96 and spill the
// backward accumulators).  Thread 0 refills a stage as soon as every warp has
// released it, one tile behind the tile it is about to consume.
//
// Work split inside a tile: a group of TPR threads owns a row, each thread VPT
// 16-byte vectors of it (the same mapping as the register-row kernels).
//
// Every wait is bounded: a barrier that does not complete within the limit
// makes the CTA record a code in the device status word and leave.
#pragma once
#include "norm_kernels.cuh"

namespace nb2 {

// `status` kernel argument: a device word, 0 = ok, else (code << 16 | blockIdx) of the
// first CTA that gave up waiting.
constexpr unsigned int kStatusFullTimeout = 1;    // tile never arrived
constexpr unsigned int kStatusEmptyTimeout = 2;   // stage never released
constexpr long long kWaitCycleLimit = 4000000000LL;   // ~2 s at 1.9 GHz

constexpr int kTmaWarps = 16;
constexpr int kTmaThreads = kTmaWarps * 32;
constexpr int kTmaHeaderBytes = 1024;             // barriers + reduction scratch, ahead of the ring
constexpr int kTmaMaxStages = 8;
constexpr uint32_t kBulkChunk = 32768;            // bytes per cp.async.bulk

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and records `code`) when the phase did not
// complete in time or another thread of the CTA already gave up.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                  unsigned int code, unsigned int* status) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (unsigned int it = 0; it < 0x40000000u; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if ((it & 63u) == 63u && clock64() - t0 > kWaitCycleLimit) break;
    }
    *abort_flag = 1;
    atomicCAS(status, 0u, (code << 16) | (blockIdx.x & 0xffffu));
    return false;
}
// After giving up: wait (bounded by time only) for a copy already issued into a
// stage, so no bulk write is still in flight into this CTA's shared memory at exit.
__device__ __forceinline__ void mbar_wait_drain(uint64_t* bar, uint32_t parity) {
    const long long t0 = clock64();
    for (unsigned int it = 0; it < 0x40000000u; ++it) {
        if (mbar_try_wait(bar, parity)) return;
        if ((it & 63u) == 63u && clock64() - t0 > kWaitCycleLimit) return;
    }
}
// global -> shared bulk copy (TMA, this CTA only), completion on `bar`; evict-first in L2
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy) : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// all threads of a row group (TPR of them) agree on `ok`
template <int TPR>
__device__ __forceinline__ bool group_all(bool ok, int barrier_id) {
    if constexpr (TPR <= 32) {
        return __all_sync(0xffffffffu, ok);
    } else {
        uint32_t r;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.u32 q, %1, 0;\n\t"
            "bar.red.and.pred p, %2, %3, q;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(r) : "r"((uint32_t)ok), "r"(barrier_id), "r"(TPR) : "memory");
        return r != 0;
    }
}

// The ring of one CTA: one source tensor forward (x), two backward (x, dy); a
// stage holds the same row range of each source.  The feeder lives in shared
// memory (only thread 0 issues copies; keeping its state out of registers
// leaves them to the row maths).
struct TileFeeder {
    const uint8_t* src0;
    const uint8_t* src1;          // nullptr when there is one source
    unsigned int* status;
    int64_t rows;
    int64_t ntiles;
    uint64_t policy;
    int row_bytes, tile_rows, stages;
    uint32_t tile_bytes, stage_bytes;
    int next_issue;               // my next tile (per-CTA sequence number) to copy
    int abort_flag;
};

// Shared memory: header (kTmaHeaderBytes: full[8] | empty[8] | red_a[64] | red_b[64] | TileFeeder),
// then gamma and beta (the reads of a row's parameters are shared-memory reads: a
// per-row global load sits on the critical path of every row even when it hits L1),
// then the ring.
__host__ __device__ inline int tma_param_bytes(int D, int elt) { return (D * elt + 1023) & ~1023; }

struct TmaSmem {
    uint64_t* full;
    uint64_t* empty;
    float* red_a;
    float* red_b;
    TileFeeder* f;
    uint8_t* ring;
    const uint4* gamma;           // the affine parameters, copied once per CTA
    const uint4* beta;
    // param_bytes: bytes of ONE parameter vector, rounded up to 16 (see tma_param_bytes)
    __device__ __forceinline__ TmaSmem(uint8_t* smem, int param_bytes)
        : full(reinterpret_cast<uint64_t*>(smem)), empty(reinterpret_cast<uint64_t*>(smem) + kTmaMaxStages),
          red_a(reinterpret_cast<float*>(smem + 128)), red_b(reinterpret_cast<float*>(smem + 384)),
          f(reinterpret_cast<TileFeeder*>(smem + 640)), ring(smem + kTmaHeaderBytes + 2 * param_bytes),
          gamma(reinterpret_cast<const uint4*>(smem + kTmaHeaderBytes)),
          beta(reinterpret_cast<const uint4*>(smem + kTmaHeaderBytes + param_bytes)) {}
    __device__ __forceinline__ volatile int* abort_flag() const { return &f->abort_flag; }

    __device__ __forceinline__ bool tile_exists(int k) const {
        return (int64_t)blockIdx.x + (int64_t)k * gridDim.x < f->ntiles;
    }
    // thread 0: copy my k-th tile (tile index blockIdx.x + k * gridDim.x) into stage k % stages
    __device__ __forceinline__ void issue(int k) const {
        const TileFeeder& t = *f;
        const int64_t tile = (int64_t)blockIdx.x + (int64_t)k * gridDim.x;
        const int s = k % t.stages;
        const int64_t r0 = tile * t.tile_rows;
        const int64_t nr = (t.rows - r0 < t.tile_rows) ? t.rows - r0 : t.tile_rows;
        const uint32_t bytes = (uint32_t)nr * t.row_bytes;
        mbar_arrive_expect_tx(&full[s], t.src1 != nullptr ? 2 * bytes : bytes);
        uint8_t* dst = ring + (size_t)s * t.stage_bytes;
        const uint8_t* a = t.src0 + r0 * (int64_t)t.row_bytes;
        for (uint32_t off = 0; off < bytes; off += kBulkChunk) {
            const uint32_t n = bytes - off < kBulkChunk ? bytes - off : kBulkChunk;
            bulk_g2s(dst + off, a + off, n, &full[s], t.policy);
        }
        if (t.src1 != nullptr) {
            const uint8_t* b = t.src1 + r0 * (int64_t)t.row_bytes;
            for (uint32_t off = 0; off < bytes; off += kBulkChunk) {
                const uint32_t n = bytes - off < kBulkChunk ? bytes - off : kBulkChunk;
                bulk_g2s(dst + t.tile_bytes + off, b + off, n, &full[s], t.policy);
            }
        }
    }
    // thread 0, opportunistically: refill every stage that all warps have released
    __device__ __forceinline__ void poll() const {
        while (tile_exists(f->next_issue)) {
            const int kp = f->next_issue - f->stages;             // the tile whose stage is recycled
            if (!mbar_try_wait(&empty[kp % f->stages], (uint32_t)((kp / f->stages) & 1))) break;
            issue(f->next_issue);
            f->next_issue = f->next_issue + 1;
        }
    }
    // thread 0, before the CTA consumes its k-th tile: make sure that tile has been requested
    __device__ __forceinline__ void ensure(int k) const {
        while (f->next_issue <= k && tile_exists(f->next_issue)) {
            const int kp = f->next_issue - f->stages;
            if (!mbar_wait_bounded(&empty[kp % f->stages], (uint32_t)((kp / f->stages) & 1), abort_flag(),
                                   kStatusEmptyTimeout, f->status)) {
                // gave up: let the copies already in flight land before leaving
                for (int kb = kp + 1; kb < f->next_issue; ++kb)
                    mbar_wait_drain(&full[kb % f->stages], (uint32_t)((kb / f->stages) & 1));
                return;
            }
            issue(f->next_issue);
            f->next_issue = f->next_issue + 1;
        }
    }
};

__device__ __forceinline__ void tma_setup(const TmaSmem& sm, const void* src0, const void* src1, int64_t rows,
                                          int row_bytes, int tile_rows, int stages, unsigned int* status,
                                          const void* gamma, const void* beta) {
    for (int i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) {
        if (gamma != nullptr) const_cast<uint4*>(sm.gamma)[i] = ld_param(reinterpret_cast<const uint4*>(gamma) + i);
        if (beta != nullptr) const_cast<uint4*>(sm.beta)[i] = ld_param(reinterpret_cast<const uint4*>(beta) + i);
    }
    if (threadIdx.x == 0) {
        TileFeeder& t = *sm.f;
        t.src0 = reinterpret_cast<const uint8_t*>(src0);
        t.src1 = reinterpret_cast<const uint8_t*>(src1);
        t.status = status;
        t.rows = rows;
        t.ntiles = (rows + tile_rows - 1) / tile_rows;
        t.policy = policy_evict_first();
        t.row_bytes = row_bytes;
        t.tile_rows = tile_rows;
        t.stages = stages;
        t.tile_bytes = (uint32_t)tile_rows * row_bytes;
        t.stage_bytes = (src1 != nullptr ? 2u : 1u) * t.tile_bytes;
        t.next_issue = 0;
        t.abort_flag = 0;
        for (int s = 0; s < stages; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], kTmaWarps); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int k = 0; k < stages && sm.tile_exists(k); ++k) sm.issue(k);      // prologue: fill the ring
        sm.f->next_issue = stages;
    }
}

// ------------------------------------------------------------------ forward
// FAST: D == TPR * VPT * EPV exactly and the affine parameters are present, so the
// inner loops carry no predicates.
template <typename T, int TPR, int VPT, int ACT, bool RMS, bool FAST>
__global__ void __launch_bounds__(kTmaThreads, 1)
norm_fwd_tma_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                    T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                    int64_t rows, int D, float eps, int tile_rows, int stages,
                    unsigned int* __restrict__ status) {
    constexpr int EPV = VecTraits<T>::EPV;
    constexpr int RPC = kTmaThreads / TPR;        // row slots
    constexpr int WPR = (TPR + 31) / 32;
    static_assert(kTmaThreads % TPR == 0, "row groups must tile the CTA");
    static_assert(TPR <= 32 || RPC <= 14, "one named barrier per multi-warp row slot");

    extern __shared__ __align__(1024) uint8_t smem[];
    const TmaSmem sm(smem, tma_param_bytes(D, (int)sizeof(T)));
    const int row_bytes = D * (int)sizeof(T);
    const uint32_t stage_bytes = (uint32_t)tile_rows * row_bytes;
    const int64_t ntiles = (rows + tile_rows - 1) / tile_rows;
    tma_setup(sm, x, nullptr, rows, row_bytes, tile_rows, stages, status, gamma, RMS ? nullptr : beta);

    const int nvec = D / EPV;
    const int slot = threadIdx.x / TPR;
    const int tr = threadIdx.x % TPR;
    const float inv_d = 1.0f / (float)D;
    const bool has_g = FAST || gamma != nullptr;
    const bool has_b = !RMS && (FAST || beta != nullptr);

    int k = 0;
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++k) {
        const int s = k % stages;
        if (threadIdx.x == 0) { sm.poll(); sm.ensure(k); }
        bool ok = mbar_wait_bounded(&sm.full[s], (uint32_t)((k / stages) & 1), sm.abort_flag(), kStatusFullTimeout, status);
        ok = group_all<TPR>(ok, slot + 1);
        if (!ok) break;
        const int64_t r0 = tile * tile_rows;
        const int nr = (int)((rows - r0 < tile_rows) ? rows - r0 : tile_rows);
        const uint8_t* stage = sm.ring + (size_t)s * stage_bytes;

        for (int r = slot; r < nr; r += RPC) {
            const uint4* srow = reinterpret_cast<const uint4*>(stage + (size_t)r * row_bytes);
            float v[VPT][EPV];
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                if (FAST || (tr + j * TPR) < nvec) {
                    unpack<T>(srow[tr + j * TPR], v[j]);
#pragma unroll
                    for (int e = 0; e < EPV; ++e) sum += RMS ? v[j][e] * v[j][e] : v[j][e];
                }
            }
            float mu = 0.f, rs;
            if constexpr (RMS) {
                rs = rsqrtf(row_sum<TPR>(sum, sm.red_a + slot * WPR, slot + 1) * inv_d + eps);
            } else {
                mu = row_sum<TPR>(sum, sm.red_a + slot * WPR, slot + 1) * inv_d;
                float q = 0.f;
#pragma unroll
                for (int j = 0; j < VPT; ++j) {
                    if (FAST || (tr + j * TPR) < nvec) {
#pragma unroll
                        for (int e = 0; e < EPV; ++e) { v[j][e] -= mu; q = fmaf(v[j][e], v[j][e], q); }
                    }
                }
                rs = rsqrtf(row_sum<TPR>(q, sm.red_b + slot * WPR, slot + 1) * inv_d + eps);
            }
            const int64_t row = r0 + r;
            if (tr == 0) {
                if (!RMS && mean_out != nullptr) mean_out[row] = mu;
                if (rstd_out != nullptr) rstd_out[row] = rs;
            }
            T* yr = y + row * (int64_t)D;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                if (FAST || (tr + j * TPR) < nvec) {
                    float g[EPV], b[EPV], o[EPV];
                    if (has_g) unpack<T>(sm.gamma[tr + j * TPR], g);
                    if (has_b) unpack<T>(sm.beta[tr + j * TPR], b);
#pragma unroll
                    for (int e = 0; e < EPV; ++e) {
                        float z = v[j][e] * rs;                 // v already holds x - mean for LayerNorm
                        if (has_g) z = has_b ? fmaf(z, g[e], b[e]) : z * g[e];
                        else if (has_b) z += b[e];
                        o[e] = act_fwd<ACT>(z);
                    }
                    st_stream(yr + (size_t)(tr + j * TPR) * EPV, pack<T>(o));
                }
            }
            if constexpr (TPR > 32 && RMS) named_barrier(slot + 1, TPR);   // red_a reuse
        }
        __syncwarp();
        if ((threadIdx.x & 31) == 0) mbar_arrive(&sm.empty[s]);             // this warp is done with the stage
        if (threadIdx.x == 0) sm.poll();
    }
}

// ----------------------------------------------------------------- backward
template <typename T, int TPR, int VPT, int ACT, bool RMS, bool FAST>
__global__ void __launch_bounds__(kTmaThreads, 1)
norm_bwd_tma_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                    const T* __restrict__ gamma, const T* __restrict__ beta,
                    const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                    T* __restrict__ dx, float* __restrict__ partials,
                    int64_t rows, int D, int tile_rows, int stages,
                    unsigned int* __restrict__ status) {
    constexpr int EPV = VecTraits<T>::EPV;
    constexpr int RPC = kTmaThreads / TPR;
    constexpr int WPR = (TPR + 31) / 32;
    constexpr int NP = NormPartials<RMS>::N;
    constexpr int COLS = TPR * VPT * EPV;
    static_assert(kTmaThreads % TPR == 0, "row groups must tile the CTA");
    static_assert(TPR <= 32 || RPC <= 14, "one named barrier per multi-warp row slot");

    extern __shared__ __align__(1024) uint8_t smem[];
    const TmaSmem sm(smem, tma_param_bytes(D, (int)sizeof(T)));
    const int row_bytes = D * (int)sizeof(T);
    const uint32_t tile_bytes = (uint32_t)tile_rows * row_bytes;      // one tensor's share of a stage
    const uint32_t stage_bytes = 2 * tile_bytes;                     // x tile then dy tile
    const int64_t ntiles = (rows + tile_rows - 1) / tile_rows;
    tma_setup(sm, x, dy, rows, row_bytes, tile_rows, stages, status, gamma, RMS ? nullptr : beta);

    const int nvec = D / EPV;
    const int slot = threadIdx.x / TPR;
    const int tr = threadIdx.x % TPR;
    const float inv_d = 1.0f / (float)D;
    const bool has_g = FAST || gamma != nullptr;
    const bool has_b = !RMS && (FAST || beta != nullptr);

    float acc_g[VPT][EPV], acc_b[RMS ? 1 : VPT][EPV];
#pragma unroll
    for (int j = 0; j < VPT; ++j)
#pragma unroll
        for (int e = 0; e < EPV; ++e) { acc_g[j][e] = 0.f; if (!RMS) acc_b[j][e] = 0.f; }

    // The saved statistics of the slot's first row in a tile are fetched one tile
    // ahead, so their global-memory latency never sits in front of a row's maths.
    float mu_next = 0.f, rs_next = 0.f;
    {
        const int64_t row = (int64_t)blockIdx.x * tile_rows + slot;
        if (row < rows) { if (!RMS) mu_next = __ldg(mean_in + row); rs_next = __ldg(rstd_in + row); }
    }
    int k = 0;
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++k) {
        const int s = k % stages;
        if (threadIdx.x == 0) { sm.poll(); sm.ensure(k); }
        float mu = mu_next, rs = rs_next;
        {
            const int64_t row = (tile + gridDim.x) * tile_rows + slot;
            if (row < rows) { if (!RMS) mu_next = __ldg(mean_in + row); rs_next = __ldg(rstd_in + row); }
        }
        bool ok = mbar_wait_bounded(&sm.full[s], (uint32_t)((k / stages) & 1), sm.abort_flag(), kStatusFullTimeout, status);
        ok = group_all<TPR>(ok, slot + 1);
        if (!ok) break;
        const int64_t r0 = tile * tile_rows;
        const int nr = (int)((rows - r0 < tile_rows) ? rows - r0 : tile_rows);
        const uint8_t* stage = sm.ring + (size_t)s * stage_bytes;

        for (int r = slot; r < nr; r += RPC) {
            const uint4* sx = reinterpret_cast<const uint4*>(stage + (size_t)r * row_bytes);
            const uint4* sd = reinterpret_cast<const uint4*>(stage + tile_bytes + (size_t)r * row_bytes);
            const int64_t row = r0 + r;
            if (r != slot) { mu = RMS ? 0.f : __ldg(mean_in + row); rs = __ldg(rstd_in + row); }
            float xh[VPT][EPV], gg[VPT][EPV];
            float s1 = 0.f, s2 = 0.f;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                if (FAST || (tr + j * TPR) < nvec) {
                    float xv[EPV], dv[EPV], g[EPV], b[EPV];
                    unpack<T>(sx[tr + j * TPR], xv);
                    unpack<T>(sd[tr + j * TPR], dv);
                    if (has_g) unpack<T>(sm.gamma[tr + j * TPR], g);
                    if (has_b && ACT != NB2_ACT_NONE) unpack<T>(sm.beta[tr + j * TPR], b);
#pragma unroll
                    for (int e = 0; e < EPV; ++e) {
                        const float h = (xv[e] - mu) * rs;
                        float dz = dv[e];
                        if constexpr (ACT != NB2_ACT_NONE) {
                            float z = h;
                            if (has_g) z = has_b ? fmaf(z, g[e], b[e]) : z * g[e];
                            else if (has_b) z += b[e];
                            dz *= act_grad<ACT>(z);
                        }
                        acc_g[j][e] = fmaf(dz, h, acc_g[j][e]);
                        if constexpr (!RMS) acc_b[j][e] += dz;
                        const float gv = has_g ? __fmul_rn(dz, g[e]) : dz;   // rounded once: g - mean(g) cancels exactly
                        s1 += gv;
                        s2 = fmaf(gv, h, s2);
                        xh[j][e] = h;
                        gg[j][e] = gv;
                    }
                }
            }
            float m1 = 0.f;
            if constexpr (!RMS) m1 = row_sum<TPR>(s1, sm.red_a + slot * WPR, slot + 1) * inv_d;
            const float m2 = row_sum<TPR>(s2, sm.red_b + slot * WPR, slot + 1) * inv_d;
            T* xo = dx + row * (int64_t)D;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                if (FAST || (tr + j * TPR) < nvec) {
                    float o[EPV];
#pragma unroll
                    for (int e = 0; e < EPV; ++e) o[e] = rs * (gg[j][e] - m1 - xh[j][e] * m2);
                    st_stream(xo + (size_t)(tr + j * TPR) * EPV, pack<T>(o));
                }
            }
            if constexpr (TPR > 32 && RMS) named_barrier(slot + 1, TPR);   // red_b reuse
        }
        __syncwarp();
        if ((threadIdx.x & 31) == 0) mbar_arrive(&sm.empty[s]);
        if (threadIdx.x == 0) sm.poll();
    }

    if (partials == nullptr) return;
    // Combine the row slots in a fixed order through shared memory.  The ring is
    // free for that: after the barrier every warp is past its last tile, and no
    // copy is in flight (each issued tile was waited for).
    float* comb = reinterpret_cast<float*>(sm.ring);
    float* out = partials + (size_t)blockIdx.x * NP * D;
    __syncthreads();
    for (int sl = 0; sl < RPC; ++sl) {
        if (slot == sl) {
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                if (FAST || (tr + j * TPR) < nvec) {
                    const int c0 = (tr + j * TPR) * EPV;
#pragma unroll
                    for (int e = 0; e < EPV; ++e) {
                        if (sl == 0) {
                            comb[c0 + e] = acc_g[j][e];
                            if constexpr (!RMS) comb[COLS + c0 + e] = acc_b[j][e];
                        } else {
                            comb[c0 + e] += acc_g[j][e];
                            if constexpr (!RMS) comb[COLS + c0 + e] += acc_b[j][e];
                        }
                    }
                }
            }
        }
        __syncthreads();
    }
    for (int c = threadIdx.x; c < D; c += kTmaThreads) {
        out[c] = comb[c];
        if constexpr (!RMS) out[D + c] = comb[COLS + c];
    }
}

}  // namespace nb2
