// Instantiations of the selection kernels (select_kernel.cuh): bf16, d128, diag.
#include "select_kernel.cuh"

namespace ia {
int launch_select_bf16_d128_diag(const SelectParams& p, const AttendRequest& ar, int n_pairs, int group, cudaStream_t stream) {
  return launch_group_bound<__nv_bfloat16, 128, float, true>(p, ar, n_pairs, group, stream);
}
}  // namespace ia
