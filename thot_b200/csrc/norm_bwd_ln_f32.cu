#include "norm_bwd_impl.cuh"
template int nb2::launch_norm_bwd<float, false>(const nb2::NormArgs&, int64_t*);
