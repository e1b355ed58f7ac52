// Instantiations of the selection kernels (select_kernel.cuh): bf16, d64, packed range.
#include "select_kernel.cuh"

namespace ia {
int launch_select_bf16_d64_packed(const SelectParams& p, const AttendRequest& ar, int n_pairs, int group,
                                  cudaStream_t stream) {
  return launch_group_packed<__nv_bfloat16, 64>(p, ar, n_pairs, group, stream);
}
}  // namespace ia
