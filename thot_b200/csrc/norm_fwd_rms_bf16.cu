#include "norm_fwd_impl.cuh"
template int nb2::launch_norm_fwd<__nv_bfloat16, true>(const nb2::NormArgs&);
