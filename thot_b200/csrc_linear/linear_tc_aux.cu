// The linear layer with the pre-activation z = x.W^T + bias stored beside y (training: the backward's input).
#include "linear_tc.cuh"

#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif
extern "C" int nb2lin_aux(const void* x, const void* w, const void* bias, void* z_out, void* y, int64_t M, int64_t N, int64_t K,
                          int act, void* workspace, size_t workspace_bytes, void* stream, char* err, size_t err_len) {
    return nb2::run_linear_act<true>(x, w, bias, z_out, y, M, N, K, act, workspace, workspace_bytes, (cudaStream_t)stream,
                                     nb2::LinErr{err, err_len});
}
#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
