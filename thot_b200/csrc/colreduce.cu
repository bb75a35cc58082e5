// Second pass of the norm backward: sum the per-CTA [ncols] fp32 partials into
// one [ncols] vector.  fp64 accumulation in a fixed order, so the result does
// not depend on how CTAs were scheduled.
#include "launchers.h"

namespace nb2 {

constexpr int CR_PL = 32;   // partial lanes per CTA
constexpr int CR_CL = 8;    // column lanes per CTA (x4 columns each)

__global__ void __launch_bounds__(CR_PL * CR_CL)
colreduce_vec_kernel(const float* __restrict__ partials, int n_partials, int64_t ncols, float* __restrict__ out) {
    __shared__ double red[CR_PL][CR_CL * 4 + 1];
    const int cl = threadIdx.x % CR_CL, pl = threadIdx.x / CR_CL;
    const int64_t c0 = ((int64_t)blockIdx.x * CR_CL + cl) * 4;
    pdl_release();
    pdl_wait();
    double acc[4] = {0.0, 0.0, 0.0, 0.0};
    if (c0 < ncols) {
#pragma unroll 4
        for (int p = pl; p < n_partials; p += CR_PL) {
            const float4 v = *reinterpret_cast<const float4*>(partials + (size_t)p * ncols + c0);
            acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
        }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) red[pl][cl * 4 + e] = acc[e];
    __syncthreads();
    if (threadIdx.x < CR_CL * 4) {
        const int64_t c = (int64_t)blockIdx.x * CR_CL * 4 + threadIdx.x;
        if (c < ncols) {
            double t = 0.0;
#pragma unroll
            for (int p = 0; p < CR_PL; ++p) t += red[p][threadIdx.x];
            out[c] = (float)t;
        }
    }
}

__global__ void __launch_bounds__(256)
colreduce_scalar_kernel(const float* __restrict__ partials, int n_partials, int64_t ncols, float* __restrict__ out) {
    __shared__ double red[8][33];
    const int cl = threadIdx.x & 31, pl = threadIdx.x >> 5;
    const int64_t c = (int64_t)blockIdx.x * 32 + cl;
    double acc = 0.0;
    if (c < ncols)
        for (int p = pl; p < n_partials; p += 8) acc += partials[(size_t)p * ncols + c];
    red[pl][cl] = acc;
    __syncthreads();
    if (pl == 0 && c < ncols) {
        double t = 0.0;
#pragma unroll
        for (int p = 0; p < 8; ++p) t += red[p][cl];
        out[c] = (float)t;
    }
}

int launch_colreduce(const float* partials, int64_t n_partials, int64_t ncols, float* out, cudaStream_t st) {
    if (ncols == 0) return 0;
    if (ncols % 4 == 0 && aligned16(partials)) {
        const int64_t grid = (ncols / 4 + CR_CL - 1) / CR_CL;
        cudaError_t e = launch_pdl(colreduce_vec_kernel, dim3((unsigned)grid), dim3(CR_PL * CR_CL), 0, st, partials, (int)n_partials, ncols, out);
        if (e != cudaSuccess) return cuda_status(e, "colreduce launch");
    } else {
        const int64_t grid = (ncols + 31) / 32;
        colreduce_scalar_kernel<<<(unsigned)grid, 256, 0, st>>>(partials, (int)n_partials, ncols, out);
    }
    return cuda_status(cudaGetLastError(), "colreduce launch");
}

}  // namespace nb2
