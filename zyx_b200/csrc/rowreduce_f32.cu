// f32 instantiations of the row kernels (+ the cross-entropy family, whose logits are f32).
#include "rowreduce_impl.cuh"
namespace zyxb {
void launch_row_f32(int fam, const RowParams& p, cudaStream_t s) {
  if (fam == FAM_CE) launch_row_family<float, FAM_CE>(p, s);
  else launch_row_dtype<float>(fam, p, s);
}
}  // namespace zyxb
