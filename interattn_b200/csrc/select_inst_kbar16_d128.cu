// Instantiations of the selection kernels (select_kernel.cuh): kbar16, d128.
#include "select_kernel.cuh"

namespace ia {
int launch_select_kbar16_d128(const SelectParams& p, const AttendRequest& ar, int n_pairs, int group, cudaStream_t stream) {
  return launch_group<__nv_bfloat16, 128, __nv_bfloat16>(p, ar, n_pairs, group, stream);
}
}  // namespace ia
