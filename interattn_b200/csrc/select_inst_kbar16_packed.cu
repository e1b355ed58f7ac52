// Instantiations of the selection kernels (select_kernel.cuh): bf16 pools with bf16 k_bar, packed range.
#include "select_kernel.cuh"

namespace ia {
int launch_select_kbar16_packed(const SelectParams& p, const AttendRequest& ar, int n_pairs, int group, int head_dim,
                                cudaStream_t stream) {
  return head_dim == 128 ? launch_group_packed<__nv_bfloat16, 128, __nv_bfloat16>(p, ar, n_pairs, group, stream)
                         : launch_group_packed<__nv_bfloat16, 64, __nv_bfloat16>(p, ar, n_pairs, group, stream);
}
}  // namespace ia
