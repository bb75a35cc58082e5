// nb2_linear_bias_act_fwd without the pre-activation output (inference, or an identity activation)
#include "linear_tc.cuh"
namespace nb2 {
int launch_linear_plain(const void* x, const void* w, const void* bias, void* y, int64_t M, int64_t N, int64_t K, int act,
                        void* workspace, size_t workspace_bytes, cudaStream_t st) {
    return run_linear_act<false>(x, w, bias, nullptr, y, M, N, K, act, workspace, workspace_bytes, st);
}
}  // namespace nb2
