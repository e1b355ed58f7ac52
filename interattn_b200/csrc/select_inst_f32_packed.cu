// Instantiations of the selection kernels (select_kernel.cuh): f32 pools, packed range.
#include "select_kernel.cuh"

namespace ia {
int launch_select_f32_packed(const SelectParams& p, const AttendRequest& ar, int n_pairs, int group, int head_dim,
                             cudaStream_t stream) {
  return head_dim == 128 ? launch_group_packed<float, 128>(p, ar, n_pairs, group, stream)
                         : launch_group_packed<float, 64>(p, ar, n_pairs, group, stream);
}
}  // namespace ia
