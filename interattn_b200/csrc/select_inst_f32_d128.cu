// Instantiations of the selection kernels (select_kernel.cuh): f32, d128.
#include "select_kernel.cuh"

namespace ia {
int launch_select_f32_d128(const SelectParams& p, const AttendRequest& ar, int n_pairs, int group, cudaStream_t stream) {
  return launch_group<float, 128>(p, ar, n_pairs, group, stream);
}
}  // namespace ia
