// Host-side selection of a norm kernel configuration.  Included by the eight
// norm_{fwd,bwd}_{ln,rms}_{f32,bf16}.cu translation units, each of which
// instantiates one element type, one norm kind and one direction so that they
// compile in parallel.
#pragma once
#include <stdlib.h>
#include <string.h>
#include "norm_tma_kernels.cuh"

namespace nb2 {

struct NormArgs {
    const void* x; const void* dy; const void* gamma; const void* beta;
    const float* mean; const float* rstd;       // backward inputs
    float* mean_out; float* rstd_out;           // forward outputs
    void* y; void* dx; float* partials;
    int64_t rows; int64_t D; float eps; int act; bool rms;
    cudaStream_t stream;
};

unsigned int* device_status_ptr();              // api.cu: the device status word of the current device
constexpr int kMaxDevices = 64;
int current_device_slot();                      // api.cu: cudaGetDevice() folded into [0, kMaxDevices)
constexpr size_t kTmaMaxSmem = 227 * 1024;

// Which kernel family to use: 0 = by shape (default), 1 = register-row only,
// 2 = bulk-async ring wherever the shape fits it.  NB2_NORM_PATH=reg|tma
// overrides the default for measurements.
static inline int norm_path_override() {
    static int cached = -1;
    if (cached < 0) {
        const char* e = getenv("NB2_NORM_PATH");
        cached = (e == nullptr) ? 0 : (strcmp(e, "reg") == 0 ? 1 : (strcmp(e, "tma") == 0 ? 2 : 0));
    }
    return cached;
}

// ---- register-row kernels: threads per row for `nvec` 16-byte vectors at VPT per thread
static inline int pick_tpr(int64_t nvec, int vpt) {
    for (int tpr = 32; tpr <= 512; tpr *= 2)
        if (nvec <= (int64_t)tpr * vpt) return tpr;
    return 0;
}
// vectors per thread: forward keeps 4 for both types; backward keeps 16
// elements per thread (its dgamma/dbeta accumulators live in registers).
template <typename T> constexpr int fwd_vpt() { return 4; }
template <typename T> constexpr int bwd_vpt() { return 16 / VecTraits<T>::EPV; }

static inline int ctas_per_sm(int tpr) { return tpr > 256 ? 1 : 2; }

// Grid of the persistent register-row backward kernel == number of partials it writes.
static inline int64_t norm_bwd_grid(int64_t rows, int tpr, int sms) {
    const int threads = tpr > 256 ? tpr : 256;
    const int rpc = threads / tpr;
    int64_t need = (rows + rpc - 1) / rpc;
    int64_t cap = (int64_t)sms * ctas_per_sm(tpr);
    if (need < 1) need = 1;
    return need < cap ? need : cap;
}
// any-width path: row blocks of the column-sum kernel
static inline int64_t norm_bwd_generic_parts(int64_t rows) {
    int64_t p = (rows + 255) / 256;
    if (p < 1) p = 1;
    return p > 256 ? 256 : p;
}

// ---- bulk-async ring kernels: exact-fit shapes only (D == TPR * VPT * EPV), parameters present.
struct TmaShape { int tpr, vpt; };
static inline TmaShape tma_bwd_shape_fwddecl(int64_t D, int epv);
// forward holds 32 elements per thread and row (24 for the 768-wide rows)
static inline TmaShape tma_fwd_shape(int64_t D, int epv) {
    if (const char* e = getenv("NB2_FWD_EPT")) { if (atoi(e) == 16) return tma_bwd_shape_fwddecl(D, epv); }
    if (D == 768) return {32, 24 / epv};
    for (int tpr = 32; tpr <= 512; tpr *= 2)
        if (D == (int64_t)tpr * 32) return {tpr, 32 / epv};
    return {0, 0};
}
// backward holds 16 (its accumulators take the registers)
static inline TmaShape tma_bwd_shape(int64_t D, int epv);
static inline TmaShape tma_bwd_shape_fwddecl(int64_t D, int epv) { return tma_bwd_shape(D, epv); }
static inline TmaShape tma_bwd_shape(int64_t D, int epv) {
    if (D == 768) return epv == 4 ? TmaShape{64, 3} : TmaShape{32, 3};
    for (int tpr = 32; tpr <= 512; tpr *= 2)
        if (D == (int64_t)tpr * 16) return {tpr, 16 / epv};
    return {0, 0};
}
// ring depth: every row group gets `stages` row slots; one "layer" (a slot of every
// group) is 32-64 KiB, and the rings may take what 200 KiB leave after the parameters
struct TmaTiling { int stages; size_t smem; };
static inline TmaTiling tma_tiling(int64_t D, int elt, int tpr, int nsrc) {
    const int rpc = kTmaThreads / tpr;
    const size_t layer = (size_t)rpc * D * elt * nsrc;
    const size_t fixed = kTmaHeaderBytes + 2 * (size_t)tma_param_bytes((int)D, elt);
    TmaTiling t;
    t.stages = 2;
    int max_stages = 4;
    if (const char* e = getenv("NB2_TMA_STAGES")) max_stages = atoi(e);
    while (t.stages < max_stages && fixed + (size_t)(t.stages + 1) * layer <= 216 * 1024) ++t.stages;
    t.smem = fixed + t.stages * layer;
    return t;
}
static inline int64_t tma_grid(int64_t rows, int tpr, int sms) {
    const int rpc = kTmaThreads / tpr;
    const int64_t need = (rows + rpc - 1) / rpc;
    return need < sms ? (need < 1 ? 1 : need) : sms;
}

// Should this (norm, direction, dtype, D) use the ring kernels?  Measured on B200 over
// D in {768 .. 8192}, 2^17 rows: LayerNorm (two statistics passes, erf epilogue) gains
// from the ring in backward at every width and in forward except for fp32 rows above
// 8 KiB; RMSNorm is lean enough that plain register-row loads already run at 92-96% of
// the copy rate, and only its fp32 forward at D >= 2048 gains.
static inline bool tma_preferred(bool rms, int64_t D, int elt, bool bwd) {
    const int ov = norm_path_override();
    if (ov == 1) return false;
    if (ov == 2) return true;
    if (!rms) return bwd ? true : (elt == 2 || D * elt <= 8192);
    return !bwd && elt == 4 && D >= 2048;
}
// does the ring of this shape fit the SM's shared memory at all
static inline bool tma_fits(int64_t D, int elt, int tpr, int nsrc) {
    return tma_tiling(D, elt, tpr, nsrc).smem <= kTmaMaxSmem;
}

template <typename T, bool RMS> int launch_norm_fwd(const NormArgs& a);
template <typename T, bool RMS> int launch_norm_bwd(const NormArgs& a, int64_t* n_partials);

template <typename T>
static inline bool norm_fast_path_ok(const NormArgs& a, int vpt) {
    constexpr int EPV = VecTraits<T>::EPV;
    if (a.D % EPV != 0) return false;
    if (pick_tpr(a.D / EPV, vpt) == 0) return false;
    if (!aligned16(a.x) || (a.y && !aligned16(a.y)) || (a.dy && !aligned16(a.dy)) ||
        (a.dx && !aligned16(a.dx)) || (a.gamma && !aligned16(a.gamma)) ||
        (a.beta && !aligned16(a.beta)) || (a.partials && !aligned16(a.partials)))
        return false;
    return true;
}

}  // namespace nb2
