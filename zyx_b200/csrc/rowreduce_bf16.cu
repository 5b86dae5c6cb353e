// bf16 instantiations of the row kernels.
#include "rowreduce_impl.cuh"
namespace zyxb {
void launch_row_bf16(int fam, const RowParams& p, cudaStream_t s) { launch_row_dtype<bf16_t>(fam, p, s); }
}  // namespace zyxb
