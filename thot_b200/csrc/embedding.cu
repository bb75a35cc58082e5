// Token-embedding gather (forward) and its deterministic scatter-add (backward).
//
// Reference semantics: torch::nn::Embedding::forward as Nott calls it
// (src/block/details/transformers/bert.hpp:162-163,176-187; ebt.hpp:124-126;
// classic.hpp:366-370): out[t,:] = table[ids[t],:], and through autograd
// dtable[v,:] = sum_{t: ids[t]==v} dout[t,:].
#include <cub/device/device_radix_sort.cuh>
#include "launchers.h"
#include "norm_tma_kernels.cuh"     // mbarrier / cp.async.bulk helpers

namespace nb2 {

template <typename I> __device__ __forceinline__ int64_t load_id(const void* ids, int64_t t) {
    return (int64_t)reinterpret_cast<const I*>(ids)[t];
}

// ------------------------------------------------------------------- forward
// A CTA copies EMB_TOK table rows per iteration, so each thread keeps EMB_TOK
// independent 16-byte loads in flight; a bad id yields a zero row and a status
// word instead of a fault.
constexpr int EMB_TOK = 4;

template <typename I, bool VEC, int ELT>
__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const uint8_t* __restrict__ table, const void* __restrict__ ids,
                     uint8_t* __restrict__ out, int64_t tokens, int64_t vocab, int64_t row_bytes,
                     int64_t* __restrict__ status) {
    for (int64_t t0 = (int64_t)blockIdx.x * EMB_TOK; t0 < tokens; t0 += (int64_t)gridDim.x * EMB_TOK) {
        int64_t id[EMB_TOK];
        bool ok[EMB_TOK];
#pragma unroll
        for (int k = 0; k < EMB_TOK; ++k) {
            id[k] = (t0 + k < tokens) ? load_id<I>(ids, t0 + k) : 0;
            ok[k] = id[k] >= 0 && id[k] < vocab;
            if (!ok[k] && t0 + k < tokens && threadIdx.x == 0 && status != nullptr) {
                status[0] = 1;
                status[1] = t0 + k;
            }
        }
        if constexpr (VEC) {
            const int64_t nv = row_bytes >> 4;
            for (int64_t v = threadIdx.x; v < nv; v += blockDim.x) {
                uint4 r[EMB_TOK];
#pragma unroll
                for (int k = 0; k < EMB_TOK; ++k) {
                    r[k] = make_uint4(0u, 0u, 0u, 0u);
                    if (t0 + k < tokens && ok[k])
                        r[k] = __ldg(reinterpret_cast<const uint4*>(table + id[k] * row_bytes) + v);
                }
#pragma unroll
                for (int k = 0; k < EMB_TOK; ++k)
                    if (t0 + k < tokens) st_stream(out + (t0 + k) * row_bytes + (v << 4), r[k]);
            }
        } else {
            // element-wise copy for rows that are not 16-byte multiples / aligned
            const int64_t ne = row_bytes / ELT;
            for (int k = 0; k < EMB_TOK; ++k) {
                if (t0 + k >= tokens) break;
                for (int64_t e = threadIdx.x; e < ne; e += blockDim.x) {
                    if constexpr (ELT == 4) {
                        reinterpret_cast<uint32_t*>(out + (t0 + k) * row_bytes)[e] =
                            ok[k] ? reinterpret_cast<const uint32_t*>(table + id[k] * row_bytes)[e] : 0u;
                    } else {
                        reinterpret_cast<uint16_t*>(out + (t0 + k) * row_bytes)[e] =
                            ok[k] ? reinterpret_cast<const uint16_t*>(table + id[k] * row_bytes)[e] : (uint16_t)0;
                    }
                }
            }
        }
    }
}

// Copy-engine gather: one warp per CTA, whose first lane drives a private ring of row slots.
// A table row travels HBM -> shared memory -> HBM as two bulk copies (cp.async.bulk, this CTA only)
// and never touches a register; the other lanes only help with the rare zero row of a bad id.
// Slot reuse waits for the outgoing copy to have read the slot (bulk-group wait), the incoming
// copy completes on the slot's mbarrier; both waits are bounded like every wait in this library.
constexpr int EMB_RING = 4;
__device__ __forceinline__ void bulk_s2g(void* dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

template <typename I>
__global__ void __launch_bounds__(32)
embedding_fwd_bulk_kernel(const uint8_t* __restrict__ table, const void* __restrict__ ids, uint8_t* __restrict__ out,
                          int64_t tokens, int64_t vocab, uint32_t row_bytes, int64_t* __restrict__ status,
                          unsigned int* __restrict__ dev_status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    volatile int* gave_up = reinterpret_cast<volatile int*>(smem + 64);
    uint8_t* ring = smem + 128;
    const int lane = threadIdx.x;
    pdl_release();
    pdl_wait();
    if (lane == 0) {
        for (int s = 0; s < EMB_RING; ++s) mbar_init(&full[s], 1);
        *gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    const int64_t first = blockIdx.x, stride = gridDim.x;
    const uint64_t policy = policy_evict_first();
    // a token whose id is outside the table is not requested; its output row is zero-filled
    auto request = [&](int k) {
        const int64_t t = first + (int64_t)k * stride;
        if (t >= tokens) return;
        const int64_t id = load_id<I>(ids, t);
        if (id < 0 || id >= vocab) return;
        const int s = k % EMB_RING;
        mbar_arrive_expect_tx(&full[s], row_bytes);
        for (uint32_t off = 0; off < row_bytes; off += kBulkChunk) {
            const uint32_t n = row_bytes - off < kBulkChunk ? row_bytes - off : kBulkChunk;
            bulk_g2s(ring + (size_t)s * row_bytes + off, table + id * (int64_t)row_bytes + off, n, &full[s], policy);
        }
    };
    if (lane == 0)
        for (int k = 0; k < EMB_RING; ++k) request(k);
    int k = 0;
    uint32_t parity = 0;                               // bit s: parity of slot s's next completed load
    for (int64_t t = first; t < tokens; t += stride, ++k) {
        const int s = k % EMB_RING;
        const int64_t id = load_id<I>(ids, t);
        const bool ok = id >= 0 && id < vocab;          // uniform over the warp
        if (ok) {
            if (lane == 0) {
                if (mbar_wait_bounded(&full[s], (parity >> s) & 1u, gave_up, kStatusFullTimeout, dev_status)) {
                    bulk_s2g(out + t * (int64_t)row_bytes, ring + (size_t)s * row_bytes, row_bytes);
                    bulk_commit();
                    bulk_wait_read_all();                // the slot may be overwritten once the copy out has read it
                    parity ^= 1u << s;                   // only a completed phase flips: the drain below waits on a timed-out slot's own phase
                }
            }
        } else {
            if (lane == 0 && status != nullptr) { status[0] = 1; status[1] = t; }
            for (uint32_t off = lane * 16; off < row_bytes; off += 32 * 16)
                *reinterpret_cast<uint4*>(out + t * (int64_t)row_bytes + off) = make_uint4(0u, 0u, 0u, 0u);
        }
        if (__shfl_sync(0xffffffffu, *gave_up, 0)) break;
        if (lane == 0) request(k + EMB_RING);
    }
    if (lane == 0) {
        bulk_wait_all();                                 // outgoing copies done before the CTA's shared memory goes away
        if (*gave_up) {
            // copies still inbound into the ring must land before the CTA leaves
            for (int b = 0; b < EMB_RING; ++b) {
                const int kb = k + b;
                const int64_t t = first + (int64_t)kb * stride;
                if (t < tokens) {
                    const int64_t id = load_id<I>(ids, t);
                    if (id >= 0 && id < vocab) mbar_wait_drain(&full[kb % EMB_RING], (parity >> (kb % EMB_RING)) & 1u);
                }
            }
        }
    }
}

template <typename I>
static int launch_emb_fwd_i(const void* table, const void* ids, void* out, int64_t tokens, int64_t vocab,
                            int64_t D, int dtype, int64_t* status, cudaStream_t st) {
    if (tokens == 0 || D == 0) return 0;
    const int elt = dtype == NB2_F32 ? 4 : 2;
    const int64_t row_bytes = D * elt;
    const bool vec_ok = (row_bytes % 16 == 0) && aligned16(table) && aligned16(out);
    if (vec_ok && row_bytes >= 1024 && row_bytes <= 48 * 1024) {
        // rows of 1-48 KiB: the copy engine moves them; smaller rows are cheaper through registers
        auto kern = embedding_fwd_bulk_kernel<I>;
        const size_t smem = 128 + (size_t)EMB_RING * row_bytes;
        static thread_local size_t configured_all[kMaxDevices] = {};
        size_t& configured = configured_all[current_device_slot()];
        if (smem > configured) {
            int rc = cuda_status(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                                 "embedding_fwd_bulk_kernel shared memory");
            if (rc != 0) return rc;
            configured = smem;
        }
        int per_sm = (int)((200 * 1024) / (smem + 1024));
        if (per_sm > 16) per_sm = 16;
        if (per_sm < 1) per_sm = 1;
        int64_t g = (int64_t)sm_count() * per_sm;
        if (g > tokens) g = tokens;
        const cudaError_t e = launch_pdl(kern, dim3((unsigned)g), dim3(32), smem, st, (const uint8_t*)table, ids, (uint8_t*)out, tokens,
                                         vocab, (uint32_t)row_bytes, status, device_status_ptr());
        return cuda_status(e, "embedding fwd (bulk) launch");
    }
    int64_t grid = (tokens + EMB_TOK - 1) / EMB_TOK;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (grid > cap) grid = cap;
    const uint8_t* tb = (const uint8_t*)table;
    uint8_t* ob = (uint8_t*)out;
    if (vec_ok)
        embedding_fwd_kernel<I, true, 4><<<(unsigned)grid, 256, 0, st>>>(tb, ids, ob, tokens, vocab, row_bytes, status);
    else if (elt == 4)
        embedding_fwd_kernel<I, false, 4><<<(unsigned)grid, 256, 0, st>>>(tb, ids, ob, tokens, vocab, row_bytes, status);
    else
        embedding_fwd_kernel<I, false, 2><<<(unsigned)grid, 256, 0, st>>>(tb, ids, ob, tokens, vocab, row_bytes, status);
    return cuda_status(cudaGetLastError(), "embedding fwd launch");
}

int launch_embedding_fwd(const void* table, const void* ids, void* out, int64_t tokens, int64_t vocab,
                         int64_t D, int dtype, int index_type, int64_t* status, cudaStream_t st) {
    return index_type == NB2_I32 ? launch_emb_fwd_i<int32_t>(table, ids, out, tokens, vocab, D, dtype, status, st)
                                 : launch_emb_fwd_i<int64_t>(table, ids, out, tokens, vocab, D, dtype, status, st);
}

// ------------------------------------------------------------------ backward
// keys = (id << 32 | t) radix-sorted by id, so equal ids are contiguous and ordered by t;
// one CTA per table row sums that row's run in fp32 in that order.  No atomics: the
// result is bit-reproducible.  Ids outside [0, vocab) get the key id = vocab and
// belong to no row.
template <typename I>
__global__ void __launch_bounds__(256)
embedding_keys_kernel(const void* __restrict__ ids, uint64_t* __restrict__ keys, int64_t tokens, int64_t vocab) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= tokens) return;
    int64_t id = load_id<I>(ids, t);
    if (id < 0 || id >= vocab) id = vocab;
    keys[t] = ((uint64_t)id << 32) | (uint64_t)(uint32_t)t;
}

constexpr int64_t kLongRun = 1024;      // tokens of one id beyond which the row goes to the long-run kernel

// row_range[v] = {first, one past last} sorted position whose id is v; both stay -1 (the preset)
// for a table row no token used
__global__ void __launch_bounds__(256)
embedding_row_range_kernel(const uint64_t* __restrict__ keys, int2* __restrict__ row_range, int64_t tokens, int64_t vocab) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= tokens) return;
    const int64_t id = (int64_t)(keys[i] >> 32);
    const int64_t prev = i == 0 ? -1 : (int64_t)(keys[i - 1] >> 32);
    if (id != prev) {
        if (id < vocab) row_range[id].x = (int32_t)i;
        if (prev >= 0 && prev < vocab) row_range[prev].y = (int32_t)i;
    }
    if (i == tokens - 1 && id < vocab) row_range[id].y = (int32_t)tokens;
}

// TR threads per table row v (CTA = 128 threads = 128 / TR table rows at a time): sum the dout rows
// of v's run of sorted keys in fp32 in ascending t, or write zeros when no token used the row.
// Every row of dtable is written exactly once, so no separate clearing pass is needed.  The run's
// bounds are known up front, so U tokens' keys and then U x VU row vectors are all in flight before
// the first addition; the additions keep the ascending order.
template <typename T, int TR, int VU, int U>
__global__ void __launch_bounds__(128)
embedding_bwd_kernel(const T* __restrict__ dout, const uint64_t* __restrict__ keys,
                     const int2* __restrict__ row_range, T* __restrict__ dtable,
                     int64_t tokens, int64_t vocab, int64_t D, unsigned int* __restrict__ long_rows) {
    constexpr int EPV = VecTraits<T>::EPV;
    constexpr int RPC = 128 / TR;
    const int tr = threadIdx.x % TR;
    const int64_t nvec = D / EPV;
    for (int64_t v = (int64_t)blockIdx.x * RPC + threadIdx.x / TR; v < vocab; v += (int64_t)gridDim.x * RPC) {
        const int2 range = __ldg(row_range + v);
        const int64_t lo = range.x < 0 ? 0 : range.x, hi = range.x < 0 ? 0 : range.y;
        if (hi - lo > kLongRun) {
            // one id used by very many tokens (padding, say): left to embedding_bwd_long_kernel, which
            // spreads the row's columns over many warps.  The counter starts at -1 (the 0xff preset).
            if (tr == 0) long_rows[2 + atomicAdd(long_rows, 1u)] = (unsigned int)v;
            continue;
        }
        T* dst = dtable + v * D;
        for (int64_t c0 = tr; c0 < nvec; c0 += (int64_t)VU * TR) {
            float acc[VU][EPV];
#pragma unroll
            for (int u = 0; u < VU; ++u)
#pragma unroll
                for (int e = 0; e < EPV; ++e) acc[u][e] = 0.f;
            for (int64_t j = lo; j < hi; j += U) {
                const T* src[U];
#pragma unroll
                for (int k = 0; k < U; ++k) {
                    const int64_t jj = j + k < hi ? j + k : hi - 1;             // clamp: the extra loads are discarded
                    src[k] = dout + (int64_t)(__ldg(keys + jj) & 0xffffffffu) * D;
                }
                uint4 r[U][VU];
#pragma unroll
                for (int k = 0; k < U; ++k)
#pragma unroll
                    for (int u = 0; u < VU; ++u) {
                        const int64_t c = c0 + (int64_t)u * TR;
                        if (c < nvec && j + k < hi) r[k][u] = ld_stream(src[k] + c * EPV);
                    }
#pragma unroll
                for (int k = 0; k < U; ++k) {
                    if (j + k < hi) {
#pragma unroll
                        for (int u = 0; u < VU; ++u) {
                            const int64_t c = c0 + (int64_t)u * TR;
                            if (c < nvec) {
                                float f[EPV];
                                unpack<T>(r[k][u], f);
#pragma unroll
                                for (int e = 0; e < EPV; ++e) acc[u][e] += f[e];
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < VU; ++u) {
                const int64_t c = c0 + (int64_t)u * TR;
                if (c < nvec) st_stream(dst + c * EPV, pack<T>(acc[u]));
            }
        }
    }
}

// Table rows with a run of more than kLongRun tokens.  One warp per (row, 32 consecutive 16-byte
// columns): it walks the whole run with U tokens in flight, so the additions of every column keep
// the ascending-t order of the short-run kernel (same bits), while the row is spread over
// D * elt / 512 warps instead of one.  long_rows[0] + 1 = number of rows listed from long_rows[1].
template <typename T>
__global__ void __launch_bounds__(128)
embedding_bwd_long_kernel(const T* __restrict__ dout, const uint64_t* __restrict__ keys,
                          const int2* __restrict__ row_range, T* __restrict__ dtable, int64_t D,
                          const unsigned int* __restrict__ long_rows) {
    constexpr int EPV = VecTraits<T>::EPV;
    constexpr int U = 8;
    const unsigned int count = long_rows[0] + 1u;
    const int64_t nvec = D / EPV;
    const int64_t c = ((int64_t)blockIdx.x * 4 + (threadIdx.x >> 5)) * 32 + (threadIdx.x & 31);
    if (c >= nvec) return;
    for (unsigned int r = blockIdx.y; r < count; r += gridDim.y) {
        const int64_t v = long_rows[1 + r];
        const int2 range = __ldg(row_range + v);
        float acc[EPV];
#pragma unroll
        for (int e = 0; e < EPV; ++e) acc[e] = 0.f;
        for (int64_t j = range.x; j < range.y; j += U) {
            uint4 rv[U];
#pragma unroll
            for (int k = 0; k < U; ++k)
                if (j + k < range.y) rv[k] = ld_stream(dout + (int64_t)(__ldg(keys + j + k) & 0xffffffffu) * D + c * EPV);
#pragma unroll
            for (int k = 0; k < U; ++k) {
                if (j + k < range.y) {
                    float f[EPV];
                    unpack<T>(rv[k], f);
#pragma unroll
                    for (int e = 0; e < EPV; ++e) acc[e] += f[e];
                }
            }
        }
        st_stream(dtable + v * D + c * EPV, pack<T>(acc));
    }
}

// any width / alignment: one CTA per table row, scalar columns
template <typename T>
__global__ void __launch_bounds__(128)
embedding_bwd_generic_kernel(const T* __restrict__ dout, const uint64_t* __restrict__ keys,
                             const int2* __restrict__ row_range, T* __restrict__ dtable,
                             int64_t tokens, int64_t vocab, int64_t D) {
    for (int64_t v = blockIdx.x; v < vocab; v += gridDim.x) {
        const int2 range = __ldg(row_range + v);
        const int64_t lo = range.x < 0 ? 0 : range.x, hi = range.x < 0 ? 0 : range.y;
        for (int64_t c = threadIdx.x; c < D; c += blockDim.x) {
            float acc = 0.f;
            for (int64_t j = lo; j < hi; ++j) acc += to_f32(dout[(int64_t)(keys[j] & 0xffffffffu) * D + c]);
            dtable[v * D + c] = from_f32<T>(acc);
        }
    }
}

// The radix sort only has to order the id half of the keys: it is stable and the keys are built in
// ascending t, so equal ids keep ascending t.  Bits [32, 32 + bits(vocab)) -> two 8-bit passes for
// a 32k vocabulary instead of six over the whole key.
static int key_bits(int64_t vocab) {
    int b = 1;
    while (((int64_t)1 << b) <= vocab && b < 31) ++b;   // ids 0..vocab inclusive (sentinel)
    return 32 + b;
}
constexpr int kKeyBeginBit = 32;

static size_t cub_temp_bytes(int64_t tokens, int64_t vocab) {
    size_t bytes = 0;
    cub::DeviceRadixSort::SortKeys(nullptr, bytes, (const uint64_t*)nullptr, (uint64_t*)nullptr,
                                   (int)tokens, kKeyBeginBit, key_bits(vocab));
    return bytes;
}

static size_t round256(size_t v) { return (v + 255) & ~(size_t)255; }
// list of long-run table rows: a counter and at most tokens / kLongRun entries
static size_t max_long_rows(int64_t tokens) { return (size_t)(tokens / kLongRun) + 1; }
static size_t long_list_bytes(int64_t tokens) { return (max_long_rows(tokens) + 2) * 4; }

size_t embedding_bwd_workspace(int64_t tokens, int64_t vocab) {
    if (tokens <= 0) return 256;
    return 2 * round256((size_t)tokens * 8) + round256(cub_temp_bytes(tokens, vocab)) + round256((size_t)vocab * 8) +
           round256(long_list_bytes(tokens)) + 256;
}

// Workspace carve-up shared by the two phases below.
struct EmbBwdWs { uint64_t* keys_in; uint64_t* keys_out; void* temp; size_t temp_bytes; int2* row_range; unsigned int* long_rows; };
static EmbBwdWs carve_bwd_ws(void* ws, int64_t tokens, int64_t vocab) {
    uint8_t* base = (uint8_t*)(((uintptr_t)ws + 255) & ~(uintptr_t)255);
    EmbBwdWs w;
    w.keys_in = (uint64_t*)base;
    w.keys_out = (uint64_t*)(base + round256((size_t)tokens * 8));
    w.temp = base + 2 * round256((size_t)tokens * 8);
    w.temp_bytes = cub_temp_bytes(tokens, vocab);
    w.row_range = (int2*)((uint8_t*)w.temp + round256(w.temp_bytes));
    w.long_rows = (unsigned int*)((uint8_t*)w.row_range + round256((size_t)vocab * 8));
    return w;
}

// Phase 1 (needs only the ids): sorted (id, t) keys and each table row's run of them.
int launch_embedding_bwd_index(const void* ids, int64_t tokens, int64_t vocab, int index_type, void* ws,
                               size_t ws_bytes, cudaStream_t st) {
    if (tokens == 0) return 0;
    NB2_REQUIRE(tokens < ((int64_t)1 << 31), NB2_ERR_SHAPE, "embedding bwd: %lld tokens exceed 2^31-1", (long long)tokens);
    NB2_REQUIRE(ws != nullptr, NB2_ERR_NULL, "embedding bwd: workspace is NULL");
    NB2_REQUIRE(ws_bytes >= embedding_bwd_workspace(tokens, vocab), NB2_ERR_WORKSPACE,
                "embedding bwd: workspace %zu < required %zu", ws_bytes, embedding_bwd_workspace(tokens, vocab));
    const EmbBwdWs w = carve_bwd_ws(ws, tokens, vocab);
    const unsigned kgrid = (unsigned)((tokens + 255) / 256);
    if (index_type == NB2_I32) embedding_keys_kernel<int32_t><<<kgrid, 256, 0, st>>>(ids, w.keys_in, tokens, vocab);
    else                       embedding_keys_kernel<int64_t><<<kgrid, 256, 0, st>>>(ids, w.keys_in, tokens, vocab);
    int rc = cuda_status(cudaGetLastError(), "embedding keys launch");
    if (rc != 0) return rc;
    size_t temp_bytes = w.temp_bytes;
    rc = cuda_status(cub::DeviceRadixSort::SortKeys(w.temp, temp_bytes, w.keys_in, w.keys_out, (int)tokens,
                                                    kKeyBeginBit, key_bits(vocab), st), "embedding key sort");
    if (rc != 0) return rc;
    rc = cuda_status(cudaMemsetAsync(w.row_range, 0xff, (size_t)vocab * 8, st), "embedding row-range preset");
    if (rc != 0) return rc;
    embedding_row_range_kernel<<<kgrid, 256, 0, st>>>(w.keys_out, w.row_range, tokens, vocab);
    return cuda_status(cudaGetLastError(), "embedding row-range launch");
}

// Phase 2: the row sums, from the index phase 1 left in the same workspace.
int launch_embedding_bwd_sum(const void* dout, void* dtable, int64_t tokens, int64_t vocab, int64_t D, int dtype,
                             void* ws, cudaStream_t st) {
    const int elt = dtype == NB2_F32 ? 4 : 2;
    if (tokens == 0 || D == 0)       // nothing to sum: the gradient is all zeros
        return cuda_status(cudaMemsetAsync(dtable, 0, (size_t)vocab * D * elt, st), "embedding bwd memset");
    const EmbBwdWs w = carve_bwd_ws(ws, tokens, vocab);
    const uint64_t* keys_out = w.keys_out;
    const int2* row_range = w.row_range;
    unsigned int* long_rows = w.long_rows;
    // the list of long runs belongs to this call (an index may serve several): its counter restarts at -1
    int rc0 = cuda_status(cudaMemsetAsync(long_rows, 0xff, 4, st), "embedding long-run list preset");
    if (rc0 != 0) return rc0;
    const bool vec = (D * elt) % 16 == 0 && aligned16(dout) && aligned16(dtable);
    const int64_t cap = (int64_t)sm_count() * 64;
    const int64_t nvec = D * elt / 16;
    auto grid_for = [&](int rows_per_cta) {
        const int64_t need = (vocab + rows_per_cta - 1) / rows_per_cta;
        return (unsigned)(need < cap ? need : cap);
    };
#define NB2_EMB_BWD(T_)                                                                                                   \
    do {                                                                                                                   \
        if (!vec)                                                                                                          \
            embedding_bwd_generic_kernel<T_><<<grid_for(1), 128, 0, st>>>((const T_*)dout, keys_out, row_range, (T_*)dtable, tokens, vocab, D); \
        else if (nvec <= 128)   /* rows up to 2 KiB: a warp per table row, four tokens in flight */                         \
            embedding_bwd_kernel<T_, 32, 4, 4><<<grid_for(4), 128, 0, st>>>((const T_*)dout, keys_out, row_range, (T_*)dtable, tokens, vocab, D, long_rows); \
        else                    /* wider rows: the CTA per table row, two tokens in flight */                               \
            embedding_bwd_kernel<T_, 128, 4, 2><<<grid_for(1), 128, 0, st>>>((const T_*)dout, keys_out, row_range, (T_*)dtable, tokens, vocab, D, long_rows); \
        if (vec && tokens > kLongRun)                                                                                       \
            embedding_bwd_long_kernel<T_><<<dim3((unsigned)((nvec + 127) / 128), (unsigned)(max_long_rows(tokens) < 1024 ? max_long_rows(tokens) : 1024)), 128, 0, st>>>(        \
                (const T_*)dout, keys_out, row_range, (T_*)dtable, D, long_rows);                                           \
    } while (0)
    if (dtype == NB2_F32) NB2_EMB_BWD(float);
    else                  NB2_EMB_BWD(__nv_bfloat16);
#undef NB2_EMB_BWD
    return cuda_status(cudaGetLastError(), "embedding bwd launch");
}

int launch_embedding_bwd(const void* dout, const void* ids, void* dtable, int64_t tokens, int64_t vocab,
                         int64_t D, int dtype, int index_type, void* ws, size_t ws_bytes, cudaStream_t st) {
    if (tokens > 0 && D > 0) {
        const int rc = launch_embedding_bwd_index(ids, tokens, vocab, index_type, ws, ws_bytes, st);
        if (rc != 0) return rc;
    }
    return launch_embedding_bwd_sum(dout, dtable, tokens, vocab, D, dtype, ws, st);
}

}  // namespace nb2
