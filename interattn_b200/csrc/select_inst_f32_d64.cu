// Instantiations of the selection kernels (select_kernel.cuh): f32, d64.
#include "select_kernel.cuh"

namespace ia {
int launch_select_f32_d64(const SelectParams& p, const AttendRequest& ar, int n_pairs, int group, cudaStream_t stream) {
  return launch_group<float, 64>(p, ar, n_pairs, group, stream);
}
}  // namespace ia
