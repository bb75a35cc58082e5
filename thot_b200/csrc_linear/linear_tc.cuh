// Fully connected layer with its bias and activation as the GEMM's epilogue, on the 5th-generation tensor
// cores:  y[M, N] = act( x[M, K] . W[N, K]^T + bias[N] )   (bf16 in and out, fp32 accumulation in TMEM).
//
// Reference: Nott's FC layer is torch::nn::Linear bound into a RegisteredLayer with the activation that follows
// it (src/layer/details/fc.hpp:31-49), run as `layer.forward` then `apply(layer.activation, .)` by the feed
// forward loop of the transformer blocks (src/block/details/transformers/classic.hpp:446-452) -- a GEMM, a bias
// pass and an activation pass over [M, N] in libtorch.  Here the bias and the activation ride in the epilogue:
// the accumulator tile leaves TMEM once, gets the bias row and the activation in registers and is stored.
//
// The mainloop and the epilogue pipeline are CUTLASS's sm_100 collectives (tcgen05.mma issued by one thread,
// operands staged by TMA from this GPU's memory, every tile with a single consumer so that no multicast load is
// generated, accumulators in TMEM, tcgen05.ld for the epilogue); the activation functors are this library's own
// (the same fitted erfc GELU and SiLU as the row kernels), plugged into the epilogue visitor tree.
#pragma once

#include "cutlass/cutlass.h"
#include "cute/tensor.hpp"
#include "cutlass/numeric_types.h"
#include "cutlass/gemm/device/gemm_universal_adapter.h"
#include "cutlass/gemm/kernel/gemm_universal.hpp"
#include "cutlass/gemm/collective/collective_builder.hpp"
#include "cutlass/epilogue/collective/collective_builder.hpp"
#include "cutlass/epilogue/fusion/operations.hpp"
#include "cutlass/util/packed_stride.hpp"

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../csrc/nb2_common.cuh"

// This translation unit is built into a library of its own (libnott_b200_linear.so) that the core library loads on
// first use: it is the only part of the tree that instantiates CUTLASS collectives.  It reports errors through a
// caller-provided buffer and uses nothing of the core library but the inline device functions of nb2_common.cuh.
namespace nb2 {

struct LinErr {
    char* buf;
    size_t len;
    void set(const char* fmt, ...) const {
        if (buf == nullptr || len == 0) return;
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, len, fmt, ap);
        va_end(ap);
    }
};

// activation functors for the epilogue visitor tree: scalar and fragment (Array) forms
template <int ACT, class T>
struct EpilogueAct {
    static const bool kIsHeavy = ACT != NB2_ACT_NONE;
    CUTLASS_HOST_DEVICE T operator()(T const& v) const {
#if defined(__CUDA_ARCH__)
        return T(act_fwd<ACT>(float(v)));
#else
        return v;
#endif
    }
};
template <int ACT, class T, int N>
struct EpilogueAct<ACT, cutlass::Array<T, N>> {
    static const bool kIsHeavy = ACT != NB2_ACT_NONE;
    // Fragments are processed as pairs on the packed fp32 pipe (fma.rn.f32x2: one issue slot for two columns; each
    // half rounds as the scalar instruction would, so the values are those of the scalar form).  The epilogue runs on
    // four warps per CTA beside the MMA, and with K <= 1024 it, not the mainloop, sets the tile time.
    CUTLASS_HOST_DEVICE cutlass::Array<T, N> operator()(cutlass::Array<T, N> const& v) const {
        cutlass::Array<T, N> y;
#if defined(__CUDA_ARCH__)
        CUTLASS_PRAGMA_UNROLL
        for (int i = 0; i + 1 < N; i += 2) {
            const float2 r = act_fwd2<ACT, true>(make_float2(float(v[i]), float(v[i + 1])));
            y[i] = T(r.x);
            y[i + 1] = T(r.y);
        }
        if constexpr (N % 2 != 0) y[N - 1] = EpilogueAct<ACT, T>()(v[N - 1]);
#else
        y = v;
#endif
        return y;
    }
};
template <class T> using EpilogueNone = EpilogueAct<NB2_ACT_NONE, T>;
template <class T> using EpilogueGelu = EpilogueAct<NB2_ACT_GELU, T>;
template <class T> using EpilogueSilu = EpilogueAct<NB2_ACT_SILU, T>;

using LinElem = cutlass::bfloat16_t;
// Two tilings.  PAIR = false: one SM per 128 x 128 tile, cluster 1x1x1.  PAIR = true: two SMs of a 2x1 cluster
// share one 256 x 128 tile (tcgen05.mma.cta_group::2, each CTA stages its own half of the operands; with a
// cluster of 2 along M and 1 along N no operand tile has a second consumer, so the loads stay plain, non-multicast
// TMA copies).  The pair form is the default for M >= 256.
template <bool PAIR> struct LinShape {
    using Tile = cute::Shape<cute::_128, cute::_128, cute::_64>;
    using Cluster = cute::Shape<cute::_1, cute::_1, cute::_1>;
};
template <> struct LinShape<true> {
    using Tile = cute::Shape<cute::_256, cute::_128, cute::_64>;
    using Cluster = cute::Shape<cute::_2, cute::_1, cute::_1>;
};

// The epilogue works through a CTA's 128 x 128 accumulator half in 128 x 64 steps: with the activation in it the four
// epilogue warps are the longer side of the tile pipeline when K <= 1024, and fewer, larger steps (two TMEM loads, two
// shared-memory stages and two TMA stores per tile instead of four) measured 7-8 % faster there than the builder's 128 x 32
// (GELU, K = 1024: 125.5 us against 135.6; K = 768: 165.5 against 179.3), level at K = 4096; 128 x 128 was 10-17 % slower.
template <class FusionOp, bool PAIR>
struct LinearGemm {
    using LinTile = typename LinShape<PAIR>::Tile;
    using LinCluster = typename LinShape<PAIR>::Cluster;
    using CollectiveEpilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
        cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, LinTile, LinCluster,
        cute::Shape<cute::_128, cute::_64>, float, float,      // epilogue sub-tile per step (the builder's automatic choice is 128 x 32)
        void, cutlass::layout::RowMajor, 8,
        LinElem, cutlass::layout::RowMajor, 8,
        std::conditional_t<PAIR, cutlass::epilogue::TmaWarpSpecialized2Sm, cutlass::epilogue::TmaWarpSpecialized1Sm>, FusionOp>::CollectiveOp;
    using CollectiveMainloop = typename cutlass::gemm::collective::CollectiveBuilder<
        cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp,
        LinElem, cutlass::layout::RowMajor, 8,          // x [M, K], K contiguous
        LinElem, cutlass::layout::ColumnMajor, 8,       // W [N, K] row-major == B [K, N] column-major
        float, LinTile, LinCluster,
        cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename CollectiveEpilogue::SharedStorage))>,
        std::conditional_t<PAIR, cutlass::gemm::KernelTmaWarpSpecialized2SmSm100, cutlass::gemm::KernelTmaWarpSpecialized1SmSm100>>::CollectiveOp;
    using Kernel = cutlass::gemm::kernel::GemmUniversal<cute::Shape<int, int, int, int>, CollectiveMainloop, CollectiveEpilogue, void>;
    using Gemm = cutlass::gemm::device::GemmUniversalAdapter<Kernel>;
};

// One launch.  z_out == nullptr: D = act(acc + bias).  z_out given (AUX): also stores acc + bias, the backward's input.
template <template <class> class Act, bool AUX, bool PAIR>
int run_linear(const void* x, const void* w, const void* bias, void* z_out, void* y, int64_t M, int64_t N, int64_t K,
               void* workspace, size_t workspace_bytes, cudaStream_t st, const LinErr& err) {
    using FusionPlain = cutlass::epilogue::fusion::LinCombPerColBiasEltAct<Act, LinElem, float, LinElem>;
    using FusionAux = cutlass::epilogue::fusion::LinCombPerColBiasEltActAux<cutlass::layout::RowMajor, Act, LinElem, float, LinElem, LinElem>;
    using Fusion = std::conditional_t<AUX, FusionAux, FusionPlain>;
    using G = LinearGemm<Fusion, PAIR>;
    using Gemm = typename G::Gemm;
    using StrideA = typename Gemm::GemmKernel::StrideA;
    using StrideB = typename Gemm::GemmKernel::StrideB;
    using StrideD = typename Gemm::GemmKernel::StrideD;
    const int m = (int)M, n = (int)N, k = (int)K;
    typename Gemm::Arguments args{};
    args.mode = cutlass::gemm::GemmUniversalMode::kGemm;
    args.problem_shape = {m, n, k, 1};
    args.mainloop.ptr_A = static_cast<const LinElem*>(x);
    args.mainloop.dA = cutlass::make_cute_packed_stride(StrideA{}, cute::make_shape(m, k, 1));
    args.mainloop.ptr_B = static_cast<const LinElem*>(w);
    args.mainloop.dB = cutlass::make_cute_packed_stride(StrideB{}, cute::make_shape(n, k, 1));
    args.epilogue.ptr_C = nullptr;
    args.epilogue.ptr_D = static_cast<LinElem*>(y);
    args.epilogue.dD = cutlass::make_cute_packed_stride(StrideD{}, cute::make_shape(m, n, 1));
    args.epilogue.thread.alpha = 1.0f;
    args.epilogue.thread.beta = 0.0f;
    args.epilogue.thread.bias_ptr = static_cast<const LinElem*>(bias);      // NULL: no bias (the visitor broadcasts 0)
    if constexpr (AUX) {
        args.epilogue.thread.aux_ptr = static_cast<LinElem*>(z_out);
        args.epilogue.thread.dAux = cutlass::make_cute_packed_stride(StrideD{}, cute::make_shape(m, n, 1));
    }
    Gemm gemm;
    if (gemm.can_implement(args) != cutlass::Status::kSuccess) {
        err.set("linear: shape M=%lld N=%lld K=%lld is not supported by the tensor-core kernel (N and K must be multiples of 8)",
                (long long)M, (long long)N, (long long)K);
        return NB2_ERR_SHAPE;
    }
    const size_t need = Gemm::get_workspace_size(args);
    if (need > workspace_bytes || (need > 0 && workspace == nullptr)) {
        err.set("linear: workspace %zu < required %zu", workspace_bytes, need);
        return NB2_ERR_WORKSPACE;
    }
    cutlass::Status s = gemm.initialize(args, workspace, st);
    if (s != cutlass::Status::kSuccess) {
        err.set("linear: kernel initialisation failed (%s)", cutlassGetStatusString(s));
        return NB2_ERR_SHAPE;
    }
    s = gemm.run(st);
    if (s != cutlass::Status::kSuccess) {
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) {
            err.set("linear (tcgen05 GEMM) launch: %s (%s)", cudaGetErrorString(e), cudaGetErrorName(e));
            return (int)e;
        }
        err.set("linear: launch failed (%s)", cutlassGetStatusString(s));
        return NB2_ERR_SHAPE;
    }
    return 0;
}

// NB2_LINEAR_TILE=single|pair overrides the choice of tiling, for measurements
static inline int linear_tile_override() {
    static int cached = -1;
    if (cached < 0) {
        const char* e = getenv("NB2_LINEAR_TILE");
        cached = (e == nullptr) ? 0 : (strcmp(e, "single") == 0 ? 1 : (strcmp(e, "pair") == 0 ? 2 : 0));
    }
    return cached;
}

template <bool AUX, bool PAIR>
int run_linear_tile(const void* x, const void* w, const void* bias, void* z_out, void* y, int64_t M, int64_t N, int64_t K, int act,
                    void* workspace, size_t workspace_bytes, cudaStream_t st, const LinErr& err) {
    switch (act) {
        case NB2_ACT_NONE: return run_linear<EpilogueNone, AUX, PAIR>(x, w, bias, z_out, y, M, N, K, workspace, workspace_bytes, st, err);
        case NB2_ACT_GELU: return run_linear<EpilogueGelu, AUX, PAIR>(x, w, bias, z_out, y, M, N, K, workspace, workspace_bytes, st, err);
        case NB2_ACT_SILU: return run_linear<EpilogueSilu, AUX, PAIR>(x, w, bias, z_out, y, M, N, K, workspace, workspace_bytes, st, err);
        default: err.set("linear: unknown activation %d", act); return NB2_ERR_DTYPE;
    }
}

template <bool AUX>
int run_linear_act(const void* x, const void* w, const void* bias, void* z_out, void* y, int64_t M, int64_t N, int64_t K, int act,
                   void* workspace, size_t workspace_bytes, cudaStream_t st, const LinErr& err) {
    const int ov = linear_tile_override();
    const bool pair = ov == 2 || (ov == 0 && M >= 256);
    if (pair) return run_linear_tile<AUX, true>(x, w, bias, z_out, y, M, N, K, act, workspace, workspace_bytes, st, err);
    return run_linear_tile<AUX, false>(x, w, bias, z_out, y, M, N, K, act, workspace, workspace_bytes, st, err);
}

}  // namespace nb2
