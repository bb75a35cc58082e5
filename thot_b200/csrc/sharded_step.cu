// Row-sharded norm step across the GPUs of one box, one process per GPU.
//
// Rows are independent, so the forward and dX need no communication; the only exchange is the sum
// over ranks of the [2, D] (LayerNorm) or [D] (RMSNorm) fp32 parameter gradients that the partial
// reduce produces.  Two exchange forms are built, both stream-ordered and both started by the same
// call that does the partial reduce:
//
//   NB2_EXCHANGE_NCCL  the partial reduce writes the rank's sums, then ncclAllReduce (in place, fp32
//                      sum) runs on a side stream owned by the communicator; the caller's stream
//                      waits for it only where the gradients are needed.
//   NB2_EXCHANGE_PEER  the partial-reduce kernel itself stores the rank's sums into a slot of every
//                      peer's receive buffer (plain 8-byte stores over NVLink to memory mapped with
//                      CUDA IPC; every stored word carries the exchange number beside its value, so
//                      no flag and no fence are needed).  The same kernel, one step later, first
//                      picks up what the peers stored for the previous step -- long since arrived --
//                      and adds the ranks' slots in rank order, so every rank gets the same bits.
//                      One launch per step, the same count as the single-GPU partial reduce.  No
//                      multicast object, no TMA on peer memory, no collective library on the step
//                      path.
//
// NCCL is reached through dlopen (the library has no link-time dependency on it); the functions used
// are ncclGetUniqueId, ncclCommInitRank, ncclAllReduce, ncclAllGather, ncclCommGetAsyncError,
// ncclCommAbort, ncclCommDestroy and ncclGetErrorString.
//
// Failure handling is on the host: nb2_comm_wait polls the exchange's completion event and the
// communicator's asynchronous error state under a deadline; on an error or on expiry it aborts the
// communicator (ncclCommAbort) and returns NB2_ERR_COMM / NB2_ERR_COMM_TIMEOUT.  The device-side
// wait of the peer form is bounded like every other wait in this library and reports through the
// device status word.
//
// The reference is single-device (src/core.hpp:1706-1708 pins cuda:0) and consumes parameter
// gradients only in the optimizer step after loss.backward() (src/core.hpp:3811-3820), which is why
// the exchange of step k may overlap the forward of step k+1.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <new>
#include <thread>

#include "launchers.h"

namespace nb2 {

constexpr int kMaxRanks = 16;
constexpr unsigned int kStatusPeerTimeout = 4;      // a peer's gradient slot never arrived
constexpr int XC_COLS = 32;                         // columns per CTA of the exchange kernels
constexpr int XC_THREADS = 256;

// ------------------------------------------------------------------ NCCL through dlopen
struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    char why[256] = "";
};

static NcclApi load_nccl() {
    NcclApi api;
    const char* env = getenv("NB2_NCCL_LIB");
    void* h = nullptr;
    if (env != nullptr && *env) h = dlopen(env, RTLD_NOW | RTLD_LOCAL);
    // a copy the process has already loaded (libtorch's, for one) is preferred to a second one
    if (h == nullptr) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL | RTLD_NOLOAD);
    if (h == nullptr) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (h == nullptr) h = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    if (h == nullptr) {
        snprintf(api.why, sizeof(api.why), "libnccl.so.2 not found (%s); set NB2_NCCL_LIB to its path", dlerror());
        return api;
    }
    bool ok = true;
    auto sym = [&](const char* name) {
        void* p = dlsym(h, name);
        if (p == nullptr) { ok = false; snprintf(api.why, sizeof(api.why), "NCCL symbol %s missing", name); }
        return p;
    };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(sym("ncclCommAbort"));
    api.CommGetAsyncError = reinterpret_cast<decltype(api.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    if (ok) api.handle = h;
    return api;
}

// loaded once per process, by whichever thread asks first (a function-local static is initialised under a lock)
static const NcclApi& nccl_state() {
    static const NcclApi api = load_nccl();
    return api;
}
static const NcclApi* nccl_api() {
    const NcclApi& api = nccl_state();
    return api.handle != nullptr ? &api : nullptr;
}

static int nccl_status(const NcclApi* api, ncclResult_t r, const char* what) {
    if (r == ncclSuccess) return 0;
    set_error("%s: NCCL error %d (%s)", what, (int)r, api && api->GetErrorString ? api->GetErrorString(r) : "?");
    return NB2_ERR_COMM;
}

// ------------------------------------------------------------------ host watchdog
// Waits until done() says the exchange finished.  failed() reports an asynchronous error of the
// communicator (0 = none); abort() tears the communicator down so that a collective kernel still
// waiting for a rank that will not come leaves the GPU.  The three are callbacks so that the policy
// can be exercised without a GPU or a second rank (nb2_selftest_comm_watchdog).
struct Watch {
    bool (*done)(void*);
    int (*failed)(void*);
    void (*abort)(void*);
    void* ctx;
};
static int watch_exchange(const Watch& w, double timeout_s) {
    using clock = std::chrono::steady_clock;
    const auto deadline = clock::now() + std::chrono::duration_cast<clock::duration>(std::chrono::duration<double>(timeout_s));
    unsigned spins = 0;
    for (;;) {
        if (w.done(w.ctx)) return 0;
        const int err = w.failed(w.ctx);
        if (err != 0) {
            w.abort(w.ctx);
            set_error("gradient exchange failed: the communicator reported asynchronous error %d; it was aborted", err);
            return NB2_ERR_COMM;
        }
        if (clock::now() >= deadline) {
            w.abort(w.ctx);
            set_error("gradient exchange did not finish within %.3f s (a rank that never joined?); the communicator was aborted", timeout_s);
            return NB2_ERR_COMM_TIMEOUT;
        }
        if (++spins > 64) std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

}  // namespace nb2

using namespace nb2;

// ------------------------------------------------------------------ the communicator
struct nb2_comm {
    int rank = 0, world = 1, mode = NB2_EXCHANGE_NCCL, device = 0;
    ncclComm_t nccl = nullptr;
    bool aborted = false;
    cudaStream_t side = nullptr;                 // NCCL form: the allreduce runs here
    cudaEvent_t ready = nullptr, done = nullptr; // fork to / join from the side stream; `done` is what nb2_comm_wait polls
    bool outstanding = false;                    // begin() issued, end() not yet
    float* out_pending = nullptr;
    int64_t ncols_pending = 0;
    // peer form
    int64_t max_cols = 0;
    uint32_t step = 0;                           // exchange counter; every stored word carries it
    uint2* slots = nullptr;                      // [2][world][max_cols] of {value bits, exchange number}: this rank's receive buffer
    uint2* peer_slots[kMaxRanks] = {};           // the same buffer of every rank as mapped here (own entry = slots)
    void* ipc_base[kMaxRanks] = {};              // what cudaIpcOpenMemHandle returned, to close again
};

namespace nb2 {

struct PeerPtrs {
    uint2* slots[kMaxRanks];
};

// One 8-byte word {value bits, exchange number}: stored and loaded as a unit, so a reader that sees the
// number it waits for also sees the value that was stored with it.
__device__ __forceinline__ void st_word(uint2* p, float v, uint32_t step) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(step) : "memory");
}
__device__ __forceinline__ uint2 ld_word(const uint2* p) {
    uint2 w;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(w.x), "=r"(w.y) : "l"(p) : "memory");
    return w;
}

// The exchange kernel, 32 columns per CTA, two phases:
//  collect (prev_out != NULL): the previous exchange.  Thread (rank r, column c) waits (bounded) until word
//           [parity of prev_step][r][c] of this rank's buffer carries prev_step, then the ranks' values are added in
//           rank order (fp64, rounded once): every rank adds the same numbers in the same order, so all ranks
//           hold identical gradients.  A wait that runs out records kStatusPeerTimeout in the device status word
//           and the CTA writes nothing.
//  post    (partials != NULL): this exchange.  The per-CTA partials are summed as in the stand-alone partial
//           reduce (fp64, fixed order) and the CTA's first warp stores its 32 sums, each with the exchange number,
//           into slot [parity of step][rank] of every rank's buffer (its own included).
// A slot parity is rewritten two exchanges later; by then its owner has collected it, because a peer can only
// store exchange k+2 after it collected k+1, which needed this rank's store of k+1, which this rank issues after
// its own collect of k (the barrier between the two phases).
template <bool VEC>
__global__ void __launch_bounds__(XC_THREADS)
exchange_kernel(const float* __restrict__ partials, int n_partials, int64_t ncols, PeerPtrs peers, int rank, int world,
                int64_t max_cols, uint32_t step, float* __restrict__ prev_out, int64_t prev_ncols, uint32_t prev_step,
                unsigned int* __restrict__ status, long long cycle_limit) {
    __shared__ double red[32][XC_COLS + 1];
    __shared__ int gave_up;
    const int64_t cbase = (int64_t)blockIdx.x * XC_COLS;
    pdl_release();
    pdl_wait();
    if (prev_out != nullptr) {
        if (threadIdx.x == 0) gave_up = 0;
        __syncthreads();
        const int r = threadIdx.x >> 5, cl = threadIdx.x & 31;          // 8 ranks per pass x 32 columns
        const int64_t c = cbase + cl;
        for (int r0 = 0; r0 < world; r0 += XC_THREADS / 32) {
            float v = 0.f;
            if (r0 + r < world && c < prev_ncols) {
                const uint2* src = peers.slots[rank] + ((size_t)(prev_step & 1u) * world + (r0 + r)) * (size_t)max_cols + (size_t)c;
                uint2 w = ld_word(src);
                if (w.y != prev_step) {
                    const long long t0 = clock64();
                    for (unsigned int it = 0; it < 0x40000000u && w.y != prev_step; ++it) {
                        w = ld_word(src);
                        if (w.y != prev_step && (it & 15u) == 15u && clock64() - t0 > cycle_limit) break;
                    }
                }
                if (w.y != prev_step) {
                    gave_up = 1;
                    atomicCAS(status, 0u, (kStatusPeerTimeout << 16) | (blockIdx.x & 0xffffu));
                }
                v = __uint_as_float(w.x);
            }
            if (r0 + r < kMaxRanks) red[r0 + r][cl] = (double)v;
        }
        __syncthreads();
        if (threadIdx.x < 32 && !gave_up && c < prev_ncols) {
            double t = 0.0;
            for (int q = 0; q < world; ++q) t += red[q][threadIdx.x];
            prev_out[c] = (float)t;
        }
        __syncthreads();                 // the collected words are consumed before this CTA stores the next exchange
    }
    if (ncols == 0) return;              // collect only
    if constexpr (VEC) {
        const int cl = threadIdx.x % 8, pl = threadIdx.x / 8;          // 8 column lanes x 4 columns, 32 partial lanes
        const int64_t c0 = cbase + cl * 4;
        double acc[4] = {0.0, 0.0, 0.0, 0.0};
        if (c0 < ncols) {
#pragma unroll 4
            for (int p = pl; p < n_partials; p += 32) {
                const float4 v = *reinterpret_cast<const float4*>(partials + (size_t)p * ncols + c0);
                acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) red[pl][cl * 4 + e] = acc[e];
    } else {
        const int cl = threadIdx.x & 31, pl = threadIdx.x >> 5;        // 32 column lanes, 8 partial lanes
        const int64_t c = cbase + cl;
        double acc = 0.0;
        if (c < ncols)
            for (int p = pl; p < n_partials; p += 8) acc += partials[(size_t)p * ncols + c];
        red[pl][cl] = acc;
#pragma unroll
        for (int p = 8 + pl; p < 32; p += 8) red[p][cl] = 0.0;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int64_t c = cbase + threadIdx.x;
        if (c < ncols) {
            double t = 0.0;
#pragma unroll
            for (int p = 0; p < 32; ++p) t += red[p][threadIdx.x];
            const float v = (float)t;
            const size_t at = ((size_t)(step & 1u) * world + rank) * (size_t)max_cols + (size_t)c;
            for (int r = 0; r < world; ++r) st_word(peers.slots[r] + at, v, step);
        }
    }
}

static bool ev_done(void* p) { return cudaEventQuery(static_cast<nb2_comm*>(p)->done) != cudaErrorNotReady; }
static int nccl_failed(void* p) {
    nb2_comm* c = static_cast<nb2_comm*>(p);
    const NcclApi* api = nccl_api();
    if (c->nccl == nullptr || api == nullptr || c->aborted) return 0;
    ncclResult_t st = ncclSuccess;
    if (api->CommGetAsyncError(c->nccl, &st) != ncclSuccess) return (int)ncclInternalError;
    return (st == ncclSuccess || st == ncclInProgress) ? 0 : (int)st;
}
static void nccl_abort(void* p) {
    nb2_comm* c = static_cast<nb2_comm*>(p);
    const NcclApi* api = nccl_api();
    if (c->nccl != nullptr && api != nullptr && !c->aborted) {
        api->CommAbort(c->nccl);
        c->aborted = true;
        c->nccl = nullptr;
    }
}

static void comm_free(nb2_comm* c) {
    if (c == nullptr) return;
    for (int i = 0; i < kMaxRanks; ++i)
        if (c->ipc_base[i] != nullptr) cudaIpcCloseMemHandle(c->ipc_base[i]);
    cudaFree(c->slots);
    if (c->ready) cudaEventDestroy(c->ready);
    if (c->done) cudaEventDestroy(c->done);
    if (c->side) cudaStreamDestroy(c->side);
    const NcclApi* api = nccl_api();
    if (c->nccl != nullptr && api != nullptr) api->CommDestroy(c->nccl);
    delete c;
}

}  // namespace nb2

#define CM_CUDA(call)                                                 \
    do {                                                              \
        int rc_ = cuda_status((call), #call);                         \
        if (rc_ != 0) { comm_free(c); return rc_; }                   \
    } while (0)
#define CM_NCCL(call)                                                 \
    do {                                                              \
        int rc_ = nccl_status(api, (call), #call);                    \
        if (rc_ != 0) { comm_free(c); return rc_; }                   \
    } while (0)

extern "C" {

int nb2_comm_unique_id(void* id_host) {
    NB2_REQUIRE(id_host != nullptr, NB2_ERR_NULL, "comm id: NULL output");
    const NcclApi* api = nccl_api();
    NB2_REQUIRE(api != nullptr, NB2_ERR_COMM, "NCCL is not available: %s", nccl_state().why);
    static_assert(NB2_COMM_ID_BYTES == NCCL_UNIQUE_ID_BYTES, "the id is NCCL's");
    ncclUniqueId id;
    int rc = nccl_status(api, api->GetUniqueId(&id), "ncclGetUniqueId");
    if (rc != 0) return rc;
    memcpy(id_host, &id, sizeof(id));
    return 0;
}

int nb2_comm_create(nb2_comm** comm, const void* id_host, int rank, int world, int mode, int64_t max_cols) {
    NB2_REQUIRE(comm != nullptr, NB2_ERR_NULL, "comm create: NULL out pointer");
    *comm = nullptr;
    NB2_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, NB2_ERR_SHAPE,
                "comm create: rank %d of %d (at most %d ranks, one per GPU of a box)", rank, world, kMaxRanks);
    NB2_REQUIRE(mode == NB2_EXCHANGE_NCCL || mode == NB2_EXCHANGE_PEER, NB2_ERR_DTYPE, "comm create: unknown exchange form %d", mode);
    NB2_REQUIRE(max_cols > 0 && max_cols <= ((int64_t)1 << 24), NB2_ERR_SHAPE, "comm create: max_cols=%lld", (long long)max_cols);
    NB2_REQUIRE(world == 1 || id_host != nullptr, NB2_ERR_NULL, "comm create: NULL id");
    nb2_comm* c = new (std::nothrow) nb2_comm();
    NB2_REQUIRE(c != nullptr, NB2_ERR_NULL, "comm create: out of host memory");
    c->rank = rank; c->world = world; c->mode = mode;
    c->max_cols = (max_cols + XC_COLS - 1) / XC_COLS * XC_COLS;
    CM_CUDA(cudaGetDevice(&c->device));
    CM_CUDA(cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking));
    CM_CUDA(cudaEventCreateWithFlags(&c->ready, cudaEventDisableTiming));
    CM_CUDA(cudaEventCreateWithFlags(&c->done, cudaEventDisableTiming));
    const NcclApi* api = nullptr;
    if (world > 1) {
        api = nccl_api();
        if (api == nullptr) { comm_free(c); set_error("comm create: NCCL is not available: %s", nccl_state().why); return NB2_ERR_COMM; }
        ncclUniqueId id;
        memcpy(&id, id_host, sizeof(id));
        CM_NCCL(api->CommInitRank(&c->nccl, world, id, rank));
    }
    if (mode == NB2_EXCHANGE_PEER) {
        const size_t slot_bytes = (size_t)2 * world * c->max_cols * sizeof(uint2);
        CM_CUDA(cudaMalloc((void**)&c->slots, slot_bytes));
        CM_CUDA(cudaMemset(c->slots, 0, slot_bytes));      // exchange numbers start at 1, so a cleared word never matches
        c->peer_slots[rank] = c->slots;
        if (world > 1) {
            // every rank's IPC handle, gathered with the communicator that was just made
            cudaIpcMemHandle_t mine;
            CM_CUDA(cudaIpcGetMemHandle(&mine, c->slots));
            uint8_t *dsend = nullptr, *drecv = nullptr;
            const size_t hb = sizeof(mine);
            CM_CUDA(cudaMalloc((void**)&dsend, hb));
            if (cudaMalloc((void**)&drecv, hb * world) != cudaSuccess) { cudaFree(dsend); comm_free(c); set_error("comm create: out of device memory"); return (int)cudaErrorMemoryAllocation; }
            cudaIpcMemHandle_t all[kMaxRanks];
            int rc = cuda_status(cudaMemcpy(dsend, &mine, hb, cudaMemcpyHostToDevice), "comm create: staging the handle");
            if (rc == 0) rc = nccl_status(api, api->AllGather(dsend, drecv, hb, ncclUint8, c->nccl, c->side), "ncclAllGather of the IPC handles");
            if (rc == 0) rc = cuda_status(cudaStreamSynchronize(c->side), "comm create: handle exchange");
            if (rc == 0) rc = cuda_status(cudaMemcpy(all, drecv, hb * world, cudaMemcpyDeviceToHost), "comm create: reading the handles");
            cudaFree(dsend);
            cudaFree(drecv);
            if (rc != 0) { comm_free(c); return rc; }
            for (int r = 0; r < world; ++r) {
                if (r == rank) continue;
                void* ps = nullptr;
                CM_CUDA(cudaIpcOpenMemHandle(&ps, all[r], cudaIpcMemLazyEnablePeerAccess));
                c->ipc_base[r] = ps;
                c->peer_slots[r] = static_cast<uint2*>(ps);
            }
            // nobody may store into a buffer that its owner has not cleared yet
            float* token = nullptr;
            CM_CUDA(cudaMalloc((void**)&token, sizeof(float)));
            rc = cuda_status(cudaMemset(token, 0, sizeof(float)), "comm create: barrier token");
            if (rc == 0) rc = nccl_status(api, api->AllReduce(token, token, 1, ncclFloat, ncclSum, c->nccl, c->side), "comm create: barrier");
            if (rc == 0) rc = cuda_status(cudaStreamSynchronize(c->side), "comm create: barrier");
            cudaFree(token);
            if (rc != 0) { comm_free(c); return rc; }
        }
    }
    *comm = c;
    return 0;
}

int nb2_comm_destroy(nb2_comm* comm) {
    if (comm != nullptr) {
        cudaSetDevice(comm->device);
        cudaDeviceSynchronize();
        comm_free(comm);
    }
    return 0;
}

int nb2_comm_info(const nb2_comm* comm, int* rank, int* world, int* mode) {
    NB2_REQUIRE(comm != nullptr, NB2_ERR_NULL, "comm info: NULL communicator");
    if (rank) *rank = comm->rank;
    if (world) *world = comm->world;
    if (mode) *mode = comm->mode;
    return 0;
}

// launches the peer form's kernel: collect of the outstanding exchange (if any) and/or post of a new one
static int launch_exchange(nb2_comm* c, const float* partials, int64_t n_partials, int64_t ncols, uint32_t step,
                           float* prev_out, int64_t prev_ncols, uint32_t prev_step, cudaStream_t st, long long cycle_limit) {
    PeerPtrs pp;
    for (int r = 0; r < kMaxRanks; ++r) pp.slots[r] = c->peer_slots[r];
    const int64_t cols = ncols > prev_ncols ? ncols : prev_ncols;
    const int grid = (int)((cols + XC_COLS - 1) / XC_COLS);
    if (grid == 0) return 0;
    const bool vec = ncols % 4 == 0 && aligned16(partials);
    const cudaError_t e = vec ? launch_pdl(exchange_kernel<true>, dim3(grid), dim3(XC_THREADS), 0, st, partials, (int)n_partials, ncols, pp,
                                           c->rank, c->world, c->max_cols, step, prev_out, prev_ncols, prev_step,
                                           device_status_ptr(), cycle_limit)
                              : launch_pdl(exchange_kernel<false>, dim3(grid), dim3(XC_THREADS), 0, st, partials, (int)n_partials, ncols, pp,
                                           c->rank, c->world, c->max_cols, step, prev_out, prev_ncols, prev_step,
                                           device_status_ptr(), cycle_limit);
    return cuda_status(e, "exchange_kernel launch");
}

int nb2_grad_exchange_begin(nb2_comm* c, const float* partials, int64_t n_partials, int64_t ncols, float* grads,
                            void* stream) {
    NB2_REQUIRE(n_partials >= 0 && n_partials < ((int64_t)1 << 31) && ncols >= 0, NB2_ERR_SHAPE,
                "gradient exchange: n_partials=%lld ncols=%lld", (long long)n_partials, (long long)ncols);
    if (c == nullptr || (c->world == 1 && c->mode == NB2_EXCHANGE_NCCL))
        return nb2_colreduce_partials(partials, n_partials, ncols, grads, stream);
    NB2_REQUIRE(!c->aborted, NB2_ERR_COMM, "gradient exchange: the communicator was aborted");
    NB2_REQUIRE(ncols <= c->max_cols, NB2_ERR_SHAPE, "gradient exchange: ncols=%lld exceeds the communicator's max_cols=%lld",
                (long long)ncols, (long long)c->max_cols);
    NB2_REQUIRE(ncols == 0 || (grads != nullptr && (partials != nullptr || n_partials == 0)), NB2_ERR_NULL, "gradient exchange: NULL pointer");
    NB2_REQUIRE(!(c->outstanding && c->out_pending == grads && ncols > 0), NB2_ERR_COMM,
                "gradient exchange: the previous exchange into this buffer is still outstanding (end it, or alternate two buffers)");
    cudaStream_t st = (cudaStream_t)stream;
    if (c->mode == NB2_EXCHANGE_NCCL) {
        int rc = nb2_grad_exchange_end(c, stream);           // one allreduce in flight on the side stream
        if (rc != 0 || ncols == 0) return rc;
        const NcclApi* api = nccl_api();
        rc = nb2_colreduce_partials(partials, n_partials, ncols, grads, stream);
        if (rc != 0) return rc;
        rc = cuda_status(cudaEventRecord(c->ready, st), "gradient exchange: fork");
        if (rc == 0) rc = cuda_status(cudaStreamWaitEvent(c->side, c->ready, 0), "gradient exchange: fork");
        if (rc == 0) rc = nccl_status(api, api->AllReduce(grads, grads, (size_t)ncols, ncclFloat, ncclSum, c->nccl, c->side), "ncclAllReduce");
        if (rc == 0) rc = cuda_status(cudaEventRecord(c->done, c->side), "gradient exchange: join");
        if (rc != 0) return rc;
    } else {
        if (ncols == 0) return nb2_grad_exchange_end(c, stream);
        // the outstanding exchange, if any, is collected by the same launch that posts this one
        const uint32_t prev_step = c->step;
        c->step += 1;
        if (c->step == 0) c->step = 1;
        const int rc = launch_exchange(c, partials, n_partials, ncols, c->step, c->outstanding ? c->out_pending : nullptr,
                                       c->outstanding ? c->ncols_pending : 0, prev_step, st, (long long)kWaitCycleLimit);
        if (rc != 0) return rc;
    }
    c->outstanding = true;
    c->out_pending = grads;
    c->ncols_pending = ncols;
    return 0;
}

int nb2_grad_exchange_end(nb2_comm* c, void* stream) {
    if (c == nullptr || !c->outstanding) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    c->outstanding = false;
    if (c->mode == NB2_EXCHANGE_NCCL) return cuda_status(cudaStreamWaitEvent(st, c->done, 0), "gradient exchange: join");
    const int rc = launch_exchange(c, nullptr, 0, 0, 0, c->out_pending, c->ncols_pending, c->step, st, (long long)kWaitCycleLimit);
    if (rc != 0) return rc;
    return cuda_status(cudaEventRecord(c->done, st), "gradient exchange: completion event");
}

int nb2_comm_wait(nb2_comm* c, double timeout_s) {
    NB2_REQUIRE(c != nullptr, NB2_ERR_NULL, "comm wait: NULL communicator");
    NB2_REQUIRE(timeout_s > 0.0, NB2_ERR_SHAPE, "comm wait: timeout %g s", timeout_s);
    NB2_REQUIRE(!c->aborted, NB2_ERR_COMM, "comm wait: the communicator was aborted");
    const Watch w{ev_done, nccl_failed, nccl_abort, c};
    const int rc = watch_exchange(w, timeout_s);
    if (rc != 0) return rc;
    const cudaError_t e = cudaEventQuery(c->done);
    return e == cudaSuccess ? 0 : cuda_status(e, "gradient exchange");
}

// The peer form's device-side wait against a flag that no rank will publish, with a limit of
// `cycle_limit` SM cycles: the kernel must return by itself and leave kStatusPeerTimeout in the
// device status word.  Nothing is written to any gradient buffer.
int nb2_selftest_peer_wait(nb2_comm* c, int64_t cycle_limit, void* stream) {
    NB2_REQUIRE(c != nullptr && c->mode == NB2_EXCHANGE_PEER, NB2_ERR_NULL, "peer-wait self-test: needs a communicator in the peer form");
    NB2_REQUIRE(cycle_limit > 0 && cycle_limit <= 2000000000LL, NB2_ERR_SHAPE, "peer-wait self-test: cycle_limit=%lld must be in (0, 2e9]", (long long)cycle_limit);
    NB2_REQUIRE(!c->outstanding, NB2_ERR_COMM, "peer-wait self-test: an exchange is outstanding");
    // collect 32 columns of an exchange number nobody has stored; the sums (never formed) would go to the slot buffer itself
    return launch_exchange(c, nullptr, 0, 0, 0, reinterpret_cast<float*>(c->slots), XC_COLS, c->step + 0x40000001u,
                           (cudaStream_t)stream, (long long)cycle_limit);
}

// `world` communicators of the peer form in ONE process, all on the current device, linked to one another as if
// they were the ranks of a box (every "peer" buffer is local memory).  It lets a single GPU run the peer exchange with
// 2-16 ranks' worth of data: the caller issues every rank's begin for step k before any rank's begin for step k+1, so
// the collect phase of each launch finds all it waits for already stored (no launch ever waits for a later one).
int nb2_selftest_comm_group(nb2_comm** comms, int world, int64_t max_cols) {
    NB2_REQUIRE(comms != nullptr, NB2_ERR_NULL, "comm group: NULL output");
    NB2_REQUIRE(world >= 1 && world <= kMaxRanks && max_cols > 0 && max_cols <= ((int64_t)1 << 24), NB2_ERR_SHAPE,
                "comm group: world=%d max_cols=%lld", world, (long long)max_cols);
    for (int r = 0; r < world; ++r) comms[r] = nullptr;
    int rc = 0;
    for (int r = 0; r < world && rc == 0; ++r) rc = nb2_comm_create(&comms[r], nullptr, 0, 1, NB2_EXCHANGE_PEER, max_cols);
    if (rc != 0) {
        for (int r = 0; r < world; ++r) { nb2_comm_destroy(comms[r]); comms[r] = nullptr; }
        return rc;
    }
    // each was made as a one-rank communicator with room for one slot; give every rank a buffer for `world` slots
    for (int r = 0; r < world && rc == 0; ++r) {
        nb2_comm* c = comms[r];
        cudaFree(c->slots);
        c->slots = nullptr;
        const size_t bytes = (size_t)2 * world * c->max_cols * sizeof(uint2);
        rc = cuda_status(cudaMalloc((void**)&c->slots, bytes), "comm group: receive buffer");
        if (rc == 0) rc = cuda_status(cudaMemset(c->slots, 0, bytes), "comm group: clearing the receive buffer");
        c->rank = r;
        c->world = world;
    }
    for (int r = 0; r < world && rc == 0; ++r)
        for (int q = 0; q < world; ++q) comms[r]->peer_slots[q] = comms[q]->slots;
    if (rc != 0) {
        for (int r = 0; r < world; ++r) { nb2_comm_destroy(comms[r]); comms[r] = nullptr; }
    }
    return rc;
}

int nb2_comm_abort(nb2_comm* c) {
    NB2_REQUIRE(c != nullptr, NB2_ERR_NULL, "comm abort: NULL communicator");
    nccl_abort(c);
    c->aborted = true;
    return 0;
}

// ---- the watchdog policy against scripted callbacks (no GPU, no second rank)
namespace {
struct FakeExchange { int polls_until_done, polls_until_error, error_code, polls, aborts; };
bool fake_done(void* p) { auto* f = static_cast<FakeExchange*>(p); ++f->polls; return f->polls_until_done >= 0 && f->polls > f->polls_until_done; }
int fake_failed(void* p) { auto* f = static_cast<FakeExchange*>(p); return f->polls_until_error >= 0 && f->polls > f->polls_until_error ? f->error_code : 0; }
void fake_abort(void* p) { ++static_cast<FakeExchange*>(p)->aborts; }
}  // namespace

int nb2_selftest_comm_watchdog(int polls_until_done, int polls_until_error, int error_code, double timeout_s, int* aborts_host) {
    FakeExchange f{polls_until_done, polls_until_error, error_code, 0, 0};
    const Watch w{fake_done, fake_failed, fake_abort, &f};
    const int rc = watch_exchange(w, timeout_s);
    if (aborts_host) *aborts_host = f.aborts;
    return rc;
}

}  // extern "C"

// ------------------------------------------------------------------ the step
struct nb2_step {
    nb2_comm* comm = nullptr;
    int norm = 0, dtype = 0, act = 0, device = 0;
    int64_t rows = 0, D = 0;
    double eps = 0;
    float *mean = nullptr, *rstd = nullptr, *partials = nullptr;
};

static void step_free(nb2_step* s) {
    if (s == nullptr) return;
    cudaFree(s->mean); cudaFree(s->rstd); cudaFree(s->partials);
    delete s;
}

extern "C" {

int nb2_step_create(nb2_step** step, nb2_comm* comm, int norm, int64_t rows, int64_t D, int dtype, int act, double eps) {
    NB2_REQUIRE(step != nullptr, NB2_ERR_NULL, "step create: NULL out pointer");
    *step = nullptr;
    NB2_REQUIRE(norm == NB2_NORM_LAYER || norm == NB2_NORM_RMS, NB2_ERR_DTYPE, "step create: unknown norm %d", norm);
    NB2_REQUIRE(dtype == NB2_F32 || dtype == NB2_BF16, NB2_ERR_DTYPE, "step create: dtype=%d", dtype);
    NB2_REQUIRE(act == NB2_ACT_NONE || act == NB2_ACT_GELU || act == NB2_ACT_SILU, NB2_ERR_DTYPE, "step create: act=%d", act);
    NB2_REQUIRE(rows >= 0 && D > 0 && D < ((int64_t)1 << 31), NB2_ERR_SHAPE, "step create: rows=%lld D=%lld", (long long)rows, (long long)D);
    const int64_t ncols = (norm == NB2_NORM_LAYER ? 2 : 1) * D;
    NB2_REQUIRE(comm == nullptr || ncols <= comm->max_cols, NB2_ERR_SHAPE,
                "step create: %lld gradient columns exceed the communicator's max_cols=%lld", (long long)ncols, (long long)comm->max_cols);
    nb2_step* s = new (std::nothrow) nb2_step();
    NB2_REQUIRE(s != nullptr, NB2_ERR_NULL, "step create: out of host memory");
    s->comm = comm; s->norm = norm; s->rows = rows; s->D = D; s->dtype = dtype; s->act = act; s->eps = eps;
    int rc = cuda_status(cudaGetDevice(&s->device), "cudaGetDevice");
    const size_t nstat = (size_t)(rows > 0 ? rows : 1) * sizeof(float);
    if (rc == 0) rc = cuda_status(cudaMalloc((void**)&s->mean, nstat), "step create: mean");
    if (rc == 0) rc = cuda_status(cudaMalloc((void**)&s->rstd, nstat), "step create: rstd");
    if (rc == 0) rc = cuda_status(cudaMalloc((void**)&s->partials, nb2_workspace_bytes(NB2_WS_NORM_BWD, rows, D, dtype)), "step create: partials");
    if (rc != 0) { step_free(s); return rc; }
    *step = s;
    return 0;
}

int nb2_step_destroy(nb2_step* step) {
    if (step != nullptr) {
        cudaSetDevice(step->device);
        cudaDeviceSynchronize();
        step_free(step);
    }
    return 0;
}

int nb2_step_run(nb2_step* s, const void* x, const void* dy, const void* gamma, const void* beta, void* y, void* dx,
                 float* grads, void* stream) {
    NB2_REQUIRE(s != nullptr, NB2_ERR_NULL, "step: NULL step");
    NB2_REQUIRE(gamma != nullptr && grads != nullptr, NB2_ERR_NULL, "step: gamma and grads must be non-NULL");
    const bool rms = s->norm == NB2_NORM_RMS;
    int rc = rms ? nb2_rmsnorm_fwd(x, gamma, y, s->rstd, s->rows, s->D, s->eps, s->dtype, s->act, stream)
                 : nb2_layernorm_fwd(x, gamma, beta, y, s->mean, s->rstd, s->rows, s->D, s->eps, s->dtype, s->act, stream);
    if (rc != 0) return rc;
    // The previous step's exchange had this step's forward to finish in.  NCCL form: the stream joins the side
    // stream here.  Peer form: nothing to do, the launch that posts this step's sums collects the previous ones.
    if (s->comm != nullptr && s->comm->mode == NB2_EXCHANGE_NCCL) {
        rc = nb2_grad_exchange_end(s->comm, stream);
        if (rc != 0) return rc;
    }
    int64_t parts = 0;
    rc = rms ? nb2_rmsnorm_bwd(x, dy, gamma, s->rstd, dx, s->partials, &parts, s->rows, s->D, s->dtype, s->act, stream)
             : nb2_layernorm_bwd(x, dy, gamma, beta, s->mean, s->rstd, dx, s->partials, &parts, s->rows, s->D, s->dtype, s->act, stream);
    if (rc != 0) return rc;
    return nb2_grad_exchange_begin(s->comm, s->partials, parts, (rms ? 1 : 2) * s->D, grads, stream);
}

int nb2_step_finish(nb2_step* s, void* stream) {
    NB2_REQUIRE(s != nullptr, NB2_ERR_NULL, "step: NULL step");
    return nb2_grad_exchange_end(s->comm, stream);
}

}  // extern "C"
