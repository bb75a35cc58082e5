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
    const void* res = nullptr; void* sum_out = nullptr;   // forward: normalise x + res, also write the sum
    const void* dres = nullptr;                           // backward: dx += dres
    RowGather gather = {nullptr, 0, 0, nullptr, nullptr, 0};   // forward with res: optional row lookup (BERT front end)
    int64_t rows; int64_t D; float eps; int act; bool rms;
    cudaStream_t stream;
};

unsigned int* device_status_ptr();              // api.cu: the device status word of the current device
constexpr int kMaxDevices = 64;
int current_device_slot();                      // api.cu: cudaGetDevice() folded into [0, kMaxDevices)
constexpr size_t kTmaMaxSmem = 227 * 1024;
// launcher result: the shape has no fused residual kernel; the caller composes add + norm instead
constexpr int kNotFused = -1000;

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
// Both directions hold 4 (fp32) or 2..4 (bf16) 16-byte vectors per thread and row.
// Forward: 4 vectors for either type (16 fp32 / 32 bf16 elements), measured best on B200.
// Widths of the form 3 * 2^k (384 ... 6144 fp32, 768 ... 6144 bf16) take three vectors per thread.
static inline TmaShape tma_fwd_shape(int64_t D, int epv) {
    for (int tpr = 32; tpr <= 512; tpr *= 2) {
        if (D == (int64_t)tpr * 4 * epv) return {tpr, 4};
        if (D == (int64_t)tpr * 3 * epv && (epv == 4 || tpr <= 256)) return {tpr, 3};
        if (D == (int64_t)tpr * 5 * epv && tpr <= 256) return {tpr, 5};                  // 5 * 2^k: 1280, 2560, 5120 (and 10240 bf16)
    }
    // 7 * 2^k (1792, 3584, 7168; 14336 in bf16): row groups of 7 or 14 warps in CTAs of 448 threads
    for (int tpr = 224; tpr <= 448; tpr *= 2)
        for (int vpt = 4; vpt >= 2; vpt -= 2)
            if (D == (int64_t)tpr * vpt * epv) return {tpr, vpt};
    return {0, 0};
}
// Backward: 16 elements per thread (its dgamma/dbeta accumulators take the registers).
static inline TmaShape tma_bwd_shape(int64_t D, int epv) {
    for (int tpr = 32; tpr <= 512; tpr *= 2) {
        if (D == (int64_t)tpr * 16) return {tpr, 16 / epv};
        if (D == (int64_t)tpr * 3 * epv && (epv == 4 || tpr <= 256)) return {tpr, 3};     // 12 fp32 / 24 bf16 columns per thread
        if (epv == 4 && D == (int64_t)tpr * 20 && tpr <= 256) return {tpr, 5};               // 5 * 2^k in fp32: 20 columns per thread
    }
    // 5 * 2^k in bf16: 40 columns per thread do not fit the registers, so the row group itself takes a 5 * 2^k size
    // (five or ten warps; CTAs of 480 and 320 threads): 16 columns per thread at 2560 and 5120, 8 at 1280
    if (epv == 8 && D == 2560) return {160, 2};
    if (epv == 8 && D == 5120) return {320, 2};
    if (epv == 8 && D == 1280) return {160, 1};
    // 7 * 2^k: groups of 224 or 448 threads, 16 columns per thread (8 at D = 1792)
    for (int tpr = 224; tpr <= 448; tpr *= 2) {
        if (D == (int64_t)tpr * 16) return {tpr, 16 / epv};
        if (D == (int64_t)tpr * 8) return {tpr, 8 / epv};
    }
    return {0, 0};
}
// ring depth: every row group gets `stages` row slots; one "layer" (a slot of every
// group) is 16-64 KiB
struct TmaTiling { int stages; size_t smem; };
static inline TmaTiling tma_tiling(int64_t D, int elt, int tpr, int nsrc, int threads = kTmaThreads) {
    const int rpc = threads / tpr;
    const size_t layer = (size_t)rpc * D * elt * nsrc;
    const size_t fixed = kTmaHeaderBytes + 2 * (size_t)tma_param_bytes((int)D, elt);
    TmaTiling t;
    t.stages = 2;
    // two slots per group already cover the latency (deeper rings measured the same); a third
    // is taken only while the whole allocation stays small
    if (fixed + 3 * layer <= 100 * 1024) t.stages = 3;
    t.smem = fixed + t.stages * layer;
    return t;
}
static inline int64_t tma_grid(int64_t rows, int tpr, int sms, int threads = kTmaThreads) {
    const int rpc = threads / tpr;
    const int64_t need = (rows + rpc - 1) / rpc;
    return need < sms ? (need < 1 ? 1 : need) : sms;
}

// Should this (norm, direction, dtype, D) use the ring kernels?  Measured on B200 over
// D in {768 .. 8192}, 2^17 rows, both families on the same inputs:
//   LayerNorm backward: ring at every width (fp32 6.2-6.6 TB/s vs 3.9-4.5 register-row).
//   LayerNorm forward : ring for bf16 and for fp32 rows up to 16 KiB; wider fp32 rows are
//                       better served by 512 threads loading straight into registers.
//   RMSNorm is lean enough that register-row loads already run at 92-96% of the copy
//   rate; the ring only wins for rows of 16 KiB and more, and for the bf16 backward.
//   That last rule holds with GELU fused (0.86 against 0.84 at 32 KiB rows); without an activation, or
//   with SiLU, the LayerNorm forward ring wins there too (0.99 against 0.89, 0.92 against 0.88).
//   D = 768 is the one width with a three-vector ring form (768 = 64 x 3 x 4 = 32 x 3 x 8), while the register-row
//   kernels cover it with four vectors per thread and a quarter of the lanes idle: there the ring also takes the
//   RMSNorm fp32 backward (0.94 against 0.87 with SiLU fused) and, with an activation fused, the bf16 forward (0.87
//   against 0.82); the fp32 forward stays (0.87 against 0.86).
static inline bool tma_preferred(bool rms, int64_t D, int elt, bool bwd, int act = NB2_ACT_GELU) {
    const int ov = norm_path_override();
    if (ov == 1) return false;
    if (ov == 2) return true;
    const int64_t row_bytes = D * elt;
    if (!rms) return bwd ? true : (elt == 2 || row_bytes <= 16384 || act != NB2_ACT_GELU || D % 3 == 0 || D % 5 == 0 || D % 7 == 0);
    if (D == 768) return bwd ? true : (elt == 2 && act != NB2_ACT_NONE);
    // the wider 3 * 2^k widths (1536, 3072, 6144): ring in both directions and types (fp32 backward 0.93-1.02 against 0.80-0.89,
    // bf16 forward 0.85-0.93 against 0.76-0.82, fp32 forward level to +5%)
    if (D % 3 == 0 && D > 768) return true;
    if (D % 5 == 0 || D % 7 == 0) return true;          // 5 * 2^k, 7 * 2^k: the register-row kernels would leave up to 37% of the lanes idle
    return bwd ? (elt == 2 || row_bytes >= 16384) : (elt == 4 && row_bytes >= 16384);
}
// does the ring of this shape fit the SM's shared memory at all
// Forward CTAs: 16 warps (parameters in registers for fp32), or 24 (parameters read from shared memory per row).
// Measured on B200 with the activation of the sweep fused, same box, both forms on the same inputs:
//   LayerNorm bf16 with GELU fused, every width: 24 warps (0.85-0.87 of the copy rate against 0.74-0.75 at D = 1024, 0.82
//                                                against 0.73 at 2048, 0.82 against 0.74 at 4096, 0.76 against 0.63 at 8192)
//   LayerNorm fp32 with GELU, rows >= 16 KiB   : 24 warps (1.00 against 0.91 at D = 4096)
//   LayerNorm fp32 with GELU, 8 KiB rows       : 16 warps (0.95 / 0.93 / 0.90 against 0.87 / 0.88 / 0.88 at 2^17 / 2^19 / 2^20 rows)
//   LayerNorm fp32 with GELU, narrower rows    : 16 warps (24 measured -10% at D = 1024)
//   RMSNorm                                    : 16 warps (0.98 against 0.90 at fp32 D = 4096; level at 8192)
// and with no activation fused 16 warps win at every width (LayerNorm fp32 D = 4096: 0.95 against 0.89; bf16 D = 4096: 0.93
// against 0.83; bf16 D = 8192: 0.90 against 0.87): the extra warps only pay for GELU's arithmetic.
static inline int fwd_warps_override() {        // NB2_FWD_WARPS=16|24 forces one form where both exist (measurements)
    static const int v = [] { const char* e = getenv("NB2_FWD_WARPS"); return e == nullptr ? 0 : atoi(e); }();
    return v;
}
static inline int fwd_threads(int tpr, int64_t row_bytes, int elt, bool rms, bool fused_gelu) {
    const bool narrow = tpr == 32 || tpr == 64;            // these have a 24-warp form for bf16 LayerNorm + GELU only
    if (!narrow && tpr != 128 && tpr != 256) return 512;
    if (narrow && !(elt == 2 && !rms && fused_gelu)) return 512;
    const int ov = fwd_warps_override();
    if (ov == 16) return 512;
    if (ov == 24) return 768;
    if (rms || !fused_gelu) return 512;
    return (elt == 2 || row_bytes >= 16384) ? 768 : 512;
}
static inline bool tma_fits(int64_t D, int elt, int tpr, int nsrc, int threads = kTmaThreads) {
    return tma_tiling(D, elt, tpr, nsrc, threads).smem <= kTmaMaxSmem;
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
    // the fused residual kernels copy these with 16-byte bulk copies and vector accesses as well
    if ((a.res && !aligned16(a.res)) || (a.sum_out && !aligned16(a.sum_out)) || (a.dres && !aligned16(a.dres)) ||
        (a.gather.extra && !aligned16(a.gather.extra)))
        return false;
    return true;
}

}  // namespace nb2
