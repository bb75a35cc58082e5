// LayerNorm / RMSNorm (+ fused activation) forward and backward, bulk-async
// variant for sm_100a: one persistent CTA of 16 warps per SM.  Whole rows stream
// from HBM into shared-memory rings with cp.async.bulk (TMA, this CTA only, no
// multicast) completing on mbarriers; the warps move a row from shared memory
// into registers, reduce its statistics with warp shuffles and write the output
// with 16-byte coalesced stores.  The bytes in flight per SM are the rings,
// independent of register use, so HBM stays busy while rows are being reduced.
//
// Work split: a group of TPR threads owns a row, each thread VPT 16-byte vectors
// of it (the mapping of the register-row kernels).  16 warps is 4 per scheduler,
// which leaves each thread 128 registers; a 17th (producer) warp would cut that
// to 96 and spill the backward accumulators, so each group's first thread issues
// the group's copies itself.
//
// Every wait is bounded: a barrier that does not complete within the limit
// makes the CTA record a code in the device status word and leave.
#pragma once
#include "norm_kernels.cuh"

namespace nb2 {

// `status` kernel argument: a device word, 0 = ok, else (code << 16 | blockIdx) of the
// first CTA that gave up waiting.
constexpr unsigned int kStatusFullTimeout = 1;    // a requested row never arrived
constexpr unsigned int kStatusSelfTest = 3;       // the self-test's wait ran out, as it must
constexpr long long kWaitCycleLimit = 4000000000LL;   // ~2 s at 1.9 GHz

constexpr int kTmaWarps = 16;
constexpr int kTmaThreads = kTmaWarps * 32;
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
                                                  unsigned int code, unsigned int* status,
                                                  long long cycle_limit = kWaitCycleLimit) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (unsigned int it = 0; it < 0x40000000u; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if ((it & 63u) == 63u && clock64() - t0 > cycle_limit) break;
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
// Has any thread of this row group given up waiting?  The flag is per group and only raised
// inside a wait, i.e. before the row reduction's barrier, so right after that reduction every
// thread of the group reads the same value (one warp: made uniform with a vote).
template <int TPR>
__device__ __forceinline__ bool group_gave_up(volatile int* abort_flag) {
    const bool gave_up = *abort_flag != 0;
    if constexpr (TPR <= 32) return __any_sync(0xffffffffu, gave_up);
    else return gave_up;
}

// Two row sums in one round: the shuffles of both interleave and a multi-warp group meets at one
// barrier instead of two.  `red` holds WPR pairs and must not be the buffer the previous row used
// (callers alternate two buffers by row parity, which is what makes a single barrier per row enough).
template <int TPR>
__device__ __forceinline__ float2 row_sum2(float2 v, float2* red, int barrier_id) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v.x += __shfl_xor_sync(0xffffffffu, v.x, o);
        v.y += __shfl_xor_sync(0xffffffffu, v.y, o);
    }
    if constexpr (TPR > 32) {
        constexpr int WPR = TPR / 32;
        const int w = (threadIdx.x % TPR) >> 5;
        if ((threadIdx.x & 31) == 0) red[w] = v;
        named_barrier(barrier_id, TPR);
        float2 t = make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < WPR; ++i) { const float2 r = red[i]; t.x += r.x; t.y += r.y; }
        v = t;
    }
    return v;
}

// Every row group owns a private ring of `stages` row slots.  Its leader thread
// requests rows ahead; a slot is re-requested as soon as the group has moved the
// row into registers, i.e. before the row's arithmetic, so the copies of the next
// rows overlap all of it.  Groups never wait for one another.
//
// Shared memory: header (full barriers [24 groups][8 stages], reduction scratch,
// abort flag), then gamma and beta (a per-row global load of the parameters would
// sit on the critical path of every row even when it hits L1), then the rings.
// The parameters are kept as fp32 whatever the activation type: a bf16 kernel would otherwise
// spend two integer instructions per column and row turning them into fp32 again.
constexpr int kTmaMaxGroups = 24;
// Packed fp32 pair instructions where the kernel is bound by issue rather than by memory: the
// bf16 kernels (measured on B200: forward +7-17%, backward +15-21% together with the single
// reduction round); the fp32 kernels measured 2-5% faster on the scalar forms.
template <typename T> constexpr bool kPackedFwd = sizeof(T) == 2;
template <typename T> constexpr bool kPackedBwd = sizeof(T) == 2;
constexpr int kTmaHeaderBytes = 3072;
__host__ __device__ inline int tma_param_bytes(int D, int /*elt*/) { return (D * 4 + 1023) & ~1023; }

struct TmaSmem {
    uint64_t* full;               // [kTmaMaxGroups][kTmaMaxStages]
    float* red_a;                 // [64]
    float* red_b;                 // [64]
    volatile int* abort_flag;     // [kTmaMaxGroups]: one per row group, raised only by that group's threads
    const uint4* gamma;
    const uint4* beta;
    uint8_t* ring;
    __device__ __forceinline__ TmaSmem(uint8_t* smem, int param_bytes)
        : full(reinterpret_cast<uint64_t*>(smem)),
          red_a(reinterpret_cast<float*>(smem + 1536)), red_b(reinterpret_cast<float*>(smem + 1792)),
          abort_flag(reinterpret_cast<volatile int*>(smem + 2048)),
          gamma(reinterpret_cast<const uint4*>(smem + kTmaHeaderBytes)),
          beta(reinterpret_cast<const uint4*>(smem + kTmaHeaderBytes + param_bytes)),
          ring(smem + kTmaHeaderBytes + 2 * param_bytes) {}
};

// One parameter array in shared memory, as fp32.  For fp32 activations entry v is the v-th 16-byte
// vector.  For bf16 the 8 columns of activation vector v are split into entry v (columns 0-3) and
// entry nvec + v (columns 4-7), so that a warp reading consecutive v touches consecutive 16 bytes.
template <typename T> __device__ __forceinline__ void store_param(uint4* dst, int v, int nvec, const uint4& raw);
template <> __device__ __forceinline__ void store_param<float>(uint4* dst, int v, int, const uint4& raw) { dst[v] = raw; }
template <> __device__ __forceinline__ void store_param<__nv_bfloat16>(uint4* dst, int v, int nvec, const uint4& raw) {
    dst[v] = make_uint4(raw.x << 16, raw.x & 0xffff0000u, raw.y << 16, raw.y & 0xffff0000u);
    dst[nvec + v] = make_uint4(raw.z << 16, raw.z & 0xffff0000u, raw.w << 16, raw.w & 0xffff0000u);
}
template <typename T> __device__ __forceinline__ void load_param2(const uint4* src, int v, int nvec, float2* f);
template <> __device__ __forceinline__ void load_param2<float>(const uint4* src, int v, int, float2* f) {
    unpack2<float>(src[v], f);
}
template <> __device__ __forceinline__ void load_param2<__nv_bfloat16>(const uint4* src, int v, int nvec, float2* f) {
    unpack2<float>(src[v], f);
    unpack2<float>(src[nvec + v], f + 2);
}

// parameters into shared memory, barriers initialised; ends with a CTA barrier
template <typename T>
__device__ __forceinline__ void tma_setup(const TmaSmem& sm, int groups, int stages, int row_bytes,
                                          const void* gamma, const void* beta) {
    const int nvec = row_bytes / 16;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        if (gamma != nullptr) store_param<T>(const_cast<uint4*>(sm.gamma), i, nvec, ld_param(reinterpret_cast<const uint4*>(gamma) + i));
        if (beta != nullptr) store_param<T>(const_cast<uint4*>(sm.beta), i, nvec, ld_param(reinterpret_cast<const uint4*>(beta) + i));
    }
    if (threadIdx.x == 0) {
        for (int g = 0; g < groups; ++g)
            for (int s = 0; s < stages; ++s) mbar_init(&sm.full[g * kTmaMaxStages + s], 1);
        for (int g = 0; g < kTmaMaxGroups; ++g) sm.abort_flag[g] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
}

// group leader: request one row of each source (up to three) into a slot, one after the other;
// each source has its own row index (the same row for plain tensors, a looked-up row for a gather)
__device__ __forceinline__ void request_rows(uint64_t* bar, uint8_t* slot, const uint8_t* src0, int64_t r0,
                                             const uint8_t* src1, int64_t r1, const uint8_t* src2, int64_t r2,
                                             uint32_t row_bytes, uint64_t policy) {
    const uint32_t nsrc = 1u + (src1 != nullptr) + (src2 != nullptr);
    mbar_arrive_expect_tx(bar, nsrc * row_bytes);
    for (uint32_t off = 0; off < row_bytes; off += kBulkChunk) {
        const uint32_t n = row_bytes - off < kBulkChunk ? row_bytes - off : kBulkChunk;
        bulk_g2s(slot + off, src0 + r0 * (int64_t)row_bytes + off, n, bar, policy);
        if (src1 != nullptr) bulk_g2s(slot + row_bytes + off, src1 + r1 * (int64_t)row_bytes + off, n, bar, policy);
        if (src2 != nullptr) bulk_g2s(slot + 2 * row_bytes + off, src2 + r2 * (int64_t)row_bytes + off, n, bar, policy);
    }
}
__device__ __forceinline__ void request_row(uint64_t* bar, uint8_t* slot, const uint8_t* src0, const uint8_t* src1,
                                            const uint8_t* src2, int64_t row, uint32_t row_bytes, uint64_t policy) {
    request_rows(bar, slot, src0, row, src1, row, src2, row, row_bytes, policy);
}

// Optional row lookup of the residual forward kernel (BERT's embedding front end,
// src/block/details/transformers/bert.hpp:162-189): x rows are table rows picked by token id,
// res rows repeat with the sequence length, and one more constant row is added.
struct RowGather {
    const void* ids;       // NULL: x is a plain [rows, D] tensor
    int64_t vocab;         // rows of the x table
    int64_t res_period;    // 0: res row == row; else res row == row % res_period
    const void* extra;     // NULL or one [D] row added to every sum
    int64_t* status;       // NULL or int64[2]: {1, first bad position} when an id is outside the table
    int ids_are_i32;
};
__device__ __forceinline__ int64_t gather_id(const RowGather& g, int64_t row) {
    return g.ids_are_i32 ? (int64_t)reinterpret_cast<const int32_t*>(g.ids)[row] : reinterpret_cast<const int64_t*>(g.ids)[row];
}

// ------------------------------------------------------------------ forward
// D == TPR * VPT * EPV exactly and the affine parameters are present (the host
// checks both), so the inner loops carry no predicates.
// RES: the normalised row is x + res (the residual add in front of a norm,
// src/block/details/transformers/classic.hpp:442-445, mamba.hpp:409-415); the sum, rounded
// to T as the reference's own `residual + attention` tensor would be, is also written out
// because it is the next residual.
template <typename T, int TPR, int VPT, int ACT, bool RMS, bool RES, int NT>
__global__ void __launch_bounds__(NT, 1)
norm_fwd_tma_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ gamma,
                    const T* __restrict__ beta, T* __restrict__ sum_out,
                    T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                    int64_t rows, int D, float eps, int stages, unsigned int* __restrict__ status,
                    const RowGather gather) {
    constexpr int EPV = VecTraits<T>::EPV;
    constexpr bool PK = kPackedFwd<T>;
    constexpr int RPC = NT / TPR;                 // row groups
    constexpr int WPR = (TPR + 31) / 32;
    static_assert(NT % TPR == 0 && RPC <= kTmaMaxGroups, "row groups must tile the CTA");
    static_assert(TPR <= 32 || RPC <= 14, "one named barrier per multi-warp row group");

    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t row_bytes = (uint32_t)D * sizeof(T);
    const TmaSmem sm(smem, tma_param_bytes(D, (int)sizeof(T)));
    pdl_release();
    pdl_wait();
    tma_setup<T>(sm, RPC, stages, (int)row_bytes, gamma, RMS ? nullptr : beta);

    const int grp = threadIdx.x / TPR;
    const int tr = threadIdx.x % TPR;
    const float inv_d = 1.0f / (float)D;
    uint64_t* full = sm.full + grp * kTmaMaxStages;
    volatile int* gave_up = sm.abort_flag + grp;
    const uint32_t slot_bytes = RES ? 2 * row_bytes : row_bytes;     // a row of x, then the same row of res
    uint8_t* ring = sm.ring + (size_t)grp * stages * slot_bytes;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(x);
    const uint8_t* src_res = RES ? reinterpret_cast<const uint8_t*>(res) : nullptr;
    const int64_t first = (int64_t)blockIdx.x * RPC + grp;
    const int64_t stride = (int64_t)gridDim.x * RPC;
    uint64_t policy = 0;
    // leader: which source rows a logical row maps to (identity unless a gather is configured)
    // `id` is the looked-up row of x when a gather is configured (ignored otherwise)
    auto request = [&](int s, int64_t row, int64_t id) {
        int64_t xr = row, rr = row;
        if constexpr (RES) {
            if (gather.ids != nullptr) {
                xr = id;
                if (xr < 0 || xr >= gather.vocab) xr = 0;           // the consumers zero this row's x part
            }
            if (gather.res_period > 0) rr = row % gather.res_period;
        }
        request_rows(&full[s], ring + (size_t)s * slot_bytes, src, xr, src_res, rr, nullptr, 0, row_bytes, policy);
    };
    const bool looked_up = RES && gather.ids != nullptr;
    // With a gather every request needs its row's id first.  Ids are fetched one step before they are used -- by the
    // leader for the row it will request next, by every thread for the row it will check next -- so that no id load
    // sits between a freed slot and its next request.
    int64_t lead_id = 0, seen_id = 0;
    if (tr == 0) {
        policy = policy_evict_first();
        for (int s = 0; s < stages; ++s) {
            const int64_t row = first + s * stride;
            if (row < rows) request(s, row, looked_up ? gather_id(gather, row) : 0);
        }
        const int64_t next = first + (int64_t)stages * stride;
        if (looked_up && next < rows) lead_id = gather_id(gather, next);
    }
    if (looked_up && first < rows) seen_id = gather_id(gather, first);
    uint4 epk[RES ? VPT : 1];                                  // the constant extra row of a gather, if any
    bool has_extra = false;
    if constexpr (RES) {
        has_extra = gather.extra != nullptr;
        if (has_extra) {
#pragma unroll
            for (int j = 0; j < VPT; ++j) epk[j] = ld_param(reinterpret_cast<const T*>(gather.extra) + (size_t)(tr + j * TPR) * EPV);
        }
    }

    // 16-warp CTAs have the registers to keep this thread's gamma/beta columns for the whole
    // kernel; 24-warp CTAs read them from shared memory per row.
    // (fp32 only: a bf16 thread has twice the columns, and its parameters are fp32 in shared memory)
    constexpr bool PREG = NT <= 512 && EPV == 4;
    const int nvec = D / EPV;
    uint4 gpk[PREG ? VPT : 1], bpk[PREG ? VPT : 1];
    if constexpr (PREG) {
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            gpk[j] = sm.gamma[tr + j * TPR];
            if constexpr (!RMS) bpk[j] = sm.beta[tr + j * TPR];
        }
    }

    int i = 0, s = 0;
    uint32_t phase = 0;                                  // s = i % stages, phase = (i / stages) & 1
    for (int64_t row = first; row < rows; row += stride, ++i) {
        // A wait that gives up raises the group's abort flag.  Leaving here would strand the rest of
        // the group at the next barrier, so the thread carries on with whatever the slot holds and
        // the whole group leaves together after the reduction below.
        mbar_wait_bounded(&full[s], phase, gave_up, kStatusFullTimeout, status);
        const uint4* srow = reinterpret_cast<const uint4*>(ring + (size_t)s * slot_bytes);
        float2 v[VPT][EPV / 2];                                  // pairs of adjacent columns
        float2 sum2 = make_float2(0.f, 0.f);
        bool x_ok = true;
        if constexpr (RES) {
            if (looked_up) {
                const int64_t id = seen_id;
                if (row + stride < rows) seen_id = gather_id(gather, row + stride);
                x_ok = id >= 0 && id < gather.vocab;
                if (!x_ok && tr == 0 && gather.status != nullptr) { gather.status[0] = 1; gather.status[1] = row; }
            }
        }
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            unpack2<T>(srow[tr + j * TPR], v[j]);
            if constexpr (RES) {
                if (!x_ok) {
#pragma unroll
                    for (int e = 0; e < EPV / 2; ++e) v[j][e] = make_float2(0.f, 0.f);
                }
                float2 r[EPV / 2];
                unpack2<T>(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(srow) + row_bytes)[tr + j * TPR], r);
#pragma unroll
                for (int e = 0; e < EPV / 2; ++e) v[j][e] = add2<PK>(v[j][e], r[e]);
                if (has_extra) {
                    unpack2<T>(epk[j], r);
#pragma unroll
                    for (int e = 0; e < EPV / 2; ++e) v[j][e] = add2<PK>(v[j][e], r[e]);
                }
                const uint4 packed = pack2<T>(v[j]);
                if (sum_out != nullptr) st_stream(sum_out + row * (int64_t)D + (size_t)(tr + j * TPR) * EPV, packed);
                unpack2<T>(packed, v[j]);                       // normalise what was stored (matters for bf16)
            }
#pragma unroll
            for (int e = 0; e < EPV / 2; ++e) sum2 = RMS ? fma2<PK>(v[j][e], v[j][e], sum2) : add2<PK>(sum2, v[j][e]);
        }
        // The first reduction doubles as the point where every thread of the group has its
        // part of the row in registers: the slot is free, request the row `stages` ahead.
        float mu = 0.f, rs;
        // RMSNorm has this one reduction per row: alternating the buffer by row parity orders its reuse
        float* red0_buf = (RMS && (i & 1)) ? sm.red_b : sm.red_a;
        const float red0 = row_sum<TPR>(sum2.x + sum2.y, red0_buf + grp * WPR, grp + 1) * inv_d;
        if (group_gave_up<TPR>(gave_up)) break;
        if (tr == 0) {
            const int64_t ahead = row + (int64_t)stages * stride;
            if (ahead < rows) {
                request(s, ahead, lead_id);
                if (looked_up && ahead + stride < rows) lead_id = gather_id(gather, ahead + stride);
            }
        }
        if (++s == stages) { s = 0; phase ^= 1u; }
        if constexpr (RMS) {
            rs = rsqrtf(red0 + eps);
        } else {
            mu = red0;
            const float2 nmu = splat2(-mu);
            float2 q2 = make_float2(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < VPT; ++j)
#pragma unroll
                for (int e = 0; e < EPV / 2; ++e) { v[j][e] = add2<PK>(v[j][e], nmu); q2 = fma2<PK>(v[j][e], v[j][e], q2); }
            rs = rsqrtf(row_sum<TPR>(q2.x + q2.y, sm.red_b + grp * WPR, grp + 1) * inv_d + eps);
        }
        if (tr == 0) {
            if (!RMS && mean_out != nullptr) mean_out[row] = mu;
            if (rstd_out != nullptr) rstd_out[row] = rs;
        }
        T* yr = y + row * (int64_t)D;
        const float2 rs2 = splat2(rs);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            float2 g[EPV / 2], b[EPV / 2], o[EPV / 2];
            if constexpr (PREG) {
                unpack2<T>(gpk[j], g);
                if constexpr (!RMS) unpack2<T>(bpk[j], b);
            } else {
                load_param2<T>(sm.gamma, tr + j * TPR, nvec, g);
                if constexpr (!RMS) load_param2<T>(sm.beta, tr + j * TPR, nvec, b);
            }
#pragma unroll
            for (int e = 0; e < EPV / 2; ++e) {
                const float2 h = mul2<PK>(v[j][e], rs2);                     // v holds x - mean for LayerNorm
                const float2 z = RMS ? mul2<PK>(h, g[e]) : fma2<PK>(h, g[e], b[e]);
                o[e] = act_fwd2<ACT, PK>(z);
            }
            st_stream(yr + (size_t)(tr + j * TPR) * EPV, pack2<T>(o));
        }
    }
    if (tr == 0 && *gave_up) {
        // gave up: let the copies this group still has in flight land before the CTA leaves
        for (int b = 0; b < stages; ++b) {
            const int ib = i + b;
            if (first + (int64_t)ib * stride < rows) mbar_wait_drain(&full[ib % stages], (uint32_t)((ib / stages) & 1));
        }
    }
}

// ----------------------------------------------------------------- backward
// RES: dx = (norm backward of dy) + dres, the gradient that reaches the normalised tensor
// through the residual branch as well; one pass instead of a backward plus an add.
template <typename T, int TPR, int VPT, int ACT, bool RMS, bool RES, int NT = kTmaThreads>
__global__ void __launch_bounds__(NT, 1)
norm_bwd_tma_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ dres,
                    const T* __restrict__ gamma, const T* __restrict__ beta,
                    const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                    T* __restrict__ dx, float* __restrict__ partials,
                    int64_t rows, int D, int stages, unsigned int* __restrict__ status) {
    constexpr int EPV = VecTraits<T>::EPV;
    constexpr bool PK = kPackedBwd<T>;
    constexpr int RPC = NT / TPR;
    constexpr int WPR = (TPR + 31) / 32;
    constexpr int NP = NormPartials<RMS>::N;
    constexpr int COLS = TPR * VPT * EPV;
    static_assert(NT % TPR == 0 && RPC <= kTmaMaxGroups, "row groups must tile the CTA");
    static_assert(TPR <= 32 || RPC <= 14, "one named barrier per multi-warp row group");

    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t row_bytes = (uint32_t)D * sizeof(T);
    const uint32_t slot_bytes = (RES ? 3 : 2) * row_bytes;          // a row of x, of dy (and of dres)
    const TmaSmem sm(smem, tma_param_bytes(D, (int)sizeof(T)));
    pdl_release();
    pdl_wait();
    tma_setup<T>(sm, RPC, stages, (int)row_bytes, gamma, RMS ? nullptr : beta);

    const int grp = threadIdx.x / TPR;
    const int tr = threadIdx.x % TPR;
    const int nvec = D / EPV;
    const float inv_d = 1.0f / (float)D;
    uint64_t* full = sm.full + grp * kTmaMaxStages;
    volatile int* gave_up = sm.abort_flag + grp;
    uint8_t* ring = sm.ring + (size_t)grp * stages * slot_bytes;
    const uint8_t* src0 = reinterpret_cast<const uint8_t*>(x);
    const uint8_t* src1 = reinterpret_cast<const uint8_t*>(dy);
    const uint8_t* src2 = RES ? reinterpret_cast<const uint8_t*>(dres) : nullptr;
    const int64_t first = (int64_t)blockIdx.x * RPC + grp;
    const int64_t stride = (int64_t)gridDim.x * RPC;
    uint64_t policy = 0;
    if (tr == 0) {
        policy = policy_evict_first();
        for (int s = 0; s < stages; ++s) {
            const int64_t row = first + s * stride;
            if (row < rows) request_row(&full[s], ring + (size_t)s * slot_bytes, src0, src1, src2, row, row_bytes, policy);
        }
    }

    float2 acc_g[VPT][EPV / 2], acc_b[RMS ? 1 : VPT][EPV / 2];
#pragma unroll
    for (int j = 0; j < VPT; ++j)
#pragma unroll
        for (int e = 0; e < EPV / 2; ++e) { acc_g[j][e] = make_float2(0.f, 0.f); if (!RMS) acc_b[j][e] = make_float2(0.f, 0.f); }

    // the saved statistics are fetched one row ahead, off the critical path
    float mu_next = 0.f, rs_next = 0.f;
    if (first < rows) { if (!RMS) mu_next = __ldg(mean_in + first); rs_next = __ldg(rstd_in + first); }

    int i = 0, s = 0;
    uint32_t phase = 0;                                  // s = i % stages, phase = (i / stages) & 1
    for (int64_t row = first; row < rows; row += stride, ++i) {
        const float mu = mu_next, rs = rs_next;
        if (row + stride < rows) { if (!RMS) mu_next = __ldg(mean_in + row + stride); rs_next = __ldg(rstd_in + row + stride); }
        // see the forward kernel: a thread whose wait gave up stays with its group until the reduction
        mbar_wait_bounded(&full[s], phase, gave_up, kStatusFullTimeout, status);
        const uint4* sx = reinterpret_cast<const uint4*>(ring + (size_t)s * slot_bytes);
        const uint4* sd = reinterpret_cast<const uint4*>(ring + (size_t)s * slot_bytes + row_bytes);
        float2 xh[VPT][EPV / 2], gg[VPT][EPV / 2];               // pairs of adjacent columns
        float2 s1 = make_float2(0.f, 0.f), s2 = make_float2(0.f, 0.f);
        const float2 nmu = splat2(-mu), rs2 = splat2(rs);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            float2 xv[EPV / 2], dv[EPV / 2], g[EPV / 2], b[EPV / 2];
            unpack2<T>(sx[tr + j * TPR], xv);
            unpack2<T>(sd[tr + j * TPR], dv);
            load_param2<T>(sm.gamma, tr + j * TPR, nvec, g);
            if constexpr (!RMS && ACT != NB2_ACT_NONE) load_param2<T>(sm.beta, tr + j * TPR, nvec, b);
#pragma unroll
            for (int e = 0; e < EPV / 2; ++e) {
                const float2 h = mul2<PK>(add2<PK>(xv[e], nmu), rs2);
                float2 dz = dv[e];
                if constexpr (ACT != NB2_ACT_NONE) {
                    const float2 z = RMS ? mul2<PK>(h, g[e]) : fma2<PK>(h, g[e], b[e]);
                    dz = mul2<PK>(dz, act_grad2<ACT, PK>(z));
                }
                acc_g[j][e] = fma2<PK>(dz, h, acc_g[j][e]);
                if constexpr (!RMS) acc_b[j][e] = add2<PK>(acc_b[j][e], dz);
                const float2 gv = mul2<PK>(dz, g[e]);       // rounded once: g - mean(g) cancels exactly
                s1 = add2<PK>(s1, gv);
                s2 = fma2<PK>(gv, h, s2);
                xh[j][e] = h;
                gg[j][e] = gv;
            }
        }
        // One reduction round per row (both sums together); the buffer alternates with the row's
        // parity, so no second barrier is needed before it is written again.  After it every thread
        // of the group is done with the slot.
        float m1 = 0.f, m2;
        float* red = (i & 1) ? sm.red_b : sm.red_a;
        if constexpr (!RMS) {
            const float2 m = row_sum2<TPR>(make_float2(s1.x + s1.y, s2.x + s2.y), reinterpret_cast<float2*>(red) + grp * WPR, grp + 1);
            m1 = m.x * inv_d;
            m2 = m.y * inv_d;
        } else {
            m2 = row_sum<TPR>(s2.x + s2.y, red + grp * WPR, grp + 1) * inv_d;
        }
        if (group_gave_up<TPR>(gave_up)) break;
        if (!RES && tr == 0) {
            const int64_t ahead = row + (int64_t)stages * stride;
            if (ahead < rows) request_row(&full[s], ring + (size_t)s * slot_bytes, src0, src1, src2, ahead, row_bytes, policy);
        }
        T* xo = dx + row * (int64_t)D;
        const float2 nm1 = splat2(-m1), nm2 = splat2(-m2);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            float2 o[EPV / 2];
#pragma unroll
            for (int e = 0; e < EPV / 2; ++e) o[e] = mul2<PK>(rs2, fma2<PK>(xh[j][e], nm2, add2<PK>(gg[j][e], nm1)));
            if constexpr (RES) {
                float2 r[EPV / 2];
                unpack2<T>(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(sx) + 2 * row_bytes)[tr + j * TPR], r);
#pragma unroll
                for (int e = 0; e < EPV / 2; ++e) o[e] = add2<PK>(o[e], r[e]);
            }
            st_stream(xo + (size_t)(tr + j * TPR) * EPV, pack2<T>(o));
        }
        if constexpr (RES) {
            // dres is read from the slot at the very end, so the slot is recycled here, not after
            // the first reduction: the whole group must be past its reads first.
            if constexpr (TPR > 32) named_barrier(grp + 1, TPR); else __syncwarp();
            if (tr == 0) {
                const int64_t ahead = row + (int64_t)stages * stride;
                if (ahead < rows) request_row(&full[s], ring + (size_t)s * slot_bytes, src0, src1, src2, ahead, row_bytes, policy);
            }
        }
        if (++s == stages) { s = 0; phase ^= 1u; }
    }
    if (tr == 0 && *gave_up) {
        for (int b = 0; b < stages; ++b) {
            const int ib = i + b;
            if (first + (int64_t)ib * stride < rows) mbar_wait_drain(&full[ib % stages], (uint32_t)((ib / stages) & 1));
        }
    }

    if (partials == nullptr) return;
    // Combine the row groups in a fixed order through shared memory.  The rings are
    // free for that: past the barrier every group has consumed every row it requested.
    float* comb = reinterpret_cast<float*>(sm.ring);
    float* out = partials + (size_t)blockIdx.x * NP * D;
    __syncthreads();
    for (int sl = 0; sl < RPC; ++sl) {
        if (grp == sl) {
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int c0 = (tr + j * TPR) * EPV;
#pragma unroll
                for (int e = 0; e < EPV; ++e) {
                    const float ag = (e & 1) ? acc_g[j][e / 2].y : acc_g[j][e / 2].x;
                    float ab = 0.f;
                    if constexpr (!RMS) ab = (e & 1) ? acc_b[j][e / 2].y : acc_b[j][e / 2].x;
                    if (sl == 0) {
                        comb[c0 + e] = ag;
                        if constexpr (!RMS) comb[COLS + c0 + e] = ab;
                    } else {
                        comb[c0 + e] += ag;
                        if constexpr (!RMS) comb[COLS + c0 + e] += ab;
                    }
                }
            }
        }
        __syncthreads();
    }
    for (int c = threadIdx.x; c < D; c += NT) {
        out[c] = comb[c];
        if constexpr (!RMS) out[D + c] = comb[COLS + c];
    }
}

}  // namespace nb2
