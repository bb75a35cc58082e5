#include "norm_fwd_impl.cuh"
template int nb2::launch_norm_fwd<float, true>(const nb2::NormArgs&);
