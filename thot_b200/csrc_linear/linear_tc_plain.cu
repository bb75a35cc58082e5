// The linear layer without the pre-activation output (inference, or an identity activation).
#include "linear_tc.cuh"

#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif
extern "C" int nb2lin_plain(const void* x, const void* w, const void* bias, void* y, int64_t M, int64_t N, int64_t K, int act,
                            void* workspace, size_t workspace_bytes, void* stream, char* err, size_t err_len) {
    return nb2::run_linear_act<false>(x, w, bias, nullptr, y, M, N, K, act, workspace, workspace_bytes, (cudaStream_t)stream,
                                      nb2::LinErr{err, err_len});
}
#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
