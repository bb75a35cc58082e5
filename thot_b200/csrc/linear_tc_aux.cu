// nb2_linear_bias_act_fwd with the pre-activation z = x.W^T + bias stored beside y (training: the backward's input)
#include "linear_tc.cuh"
namespace nb2 {
int launch_linear_aux(const void* x, const void* w, const void* bias, void* z_out, void* y, int64_t M, int64_t N, int64_t K, int act,
                      void* workspace, size_t workspace_bytes, cudaStream_t st) {
    return run_linear_act<true>(x, w, bias, z_out, y, M, N, K, act, workspace, workspace_bytes, st);
}
}  // namespace nb2
