#include "norm_bwd_impl.cuh"
template int nb2::launch_norm_bwd<__nv_bfloat16, true>(const nb2::NormArgs&, int64_t*);
