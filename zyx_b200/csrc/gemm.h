// Matmul launch parameters shared by the SIMT and tensor-core paths.
#pragma once
#include <type_traits>

#include "internal.h"

namespace zyxb {

struct GemmParams {
  const void* a; const void* b; const void* bias;
  const void* z;   // MUL_*_GRAD epilogues: [m, n] (per batch, C's stride)
  void* c; void* preact;
  uint64_t m, n, k, batch;
  int64_t stride_a, stride_b, stride_c;   // elements between consecutive (outer) batches
  uint64_t lda, ldb, ldc;                 // row pitch of the stored operands, elements
  uint64_t batch_inner;                   // >= 1; matrix z: (z / batch_inner) * stride + (z % batch_inner) * stride_inner
  int64_t stride_a_inner, stride_b_inner, stride_c_inner;
  int trans_a, trans_b;                   // A stored [k,m] / B stored [n,k]
  int epilogue;
  int tri;                                // ZYXB_TRI_*
  float alpha;
  int rn;
  bool vec_a, vec_b;
  int splits;        // SIMT path: > 1 = the k range is divided over this many CTAs per tile, partial sums go to `partial`
  void* partial;     // [batch][splits][m][n] accumulators (f32 / i32) in the context's scratch
};

int launch_gemm_simt(GemmParams p, int dtype, const LaunchCtx& lc, std::string& err);
// Tensor-core path (tcgen05 + TMEM + TMA).  Returns true when the shape is one it takes.
bool gemm_tc_supported(const GemmParams& p, int dtype, const LaunchCtx& lc);
int launch_gemm_tc(const GemmParams& p, int dtype, const LaunchCtx& lc, std::string& err);
// f32 on the tensor cores at f32 accuracy (three TF32 products per k-step on operands split into hi + lo)
bool gemm_tf32x3_supported(const GemmParams& p, int dtype, const LaunchCtx& lc);
int launch_gemm_tf32x3(const GemmParams& p, const LaunchCtx& lc, std::string& err);

}  // namespace zyxb
