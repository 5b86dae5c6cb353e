// Matmul programs: validation and the choice between the tensor-core and the SIMT path.
// Tensor::dot (zyx/src/tensor/mod.rs:1469-1490); the descriptor is what a match of the
// reduce-of-product pattern yields (zyx/src/vendor/matmul.rs:43-71).
#include <stdlib.h>

#include "gemm.h"

namespace zyxb {

int validate_gemm(const zyxb_gemm_desc& d, std::string& err) {
  if (d.dtype != ZYXB_F32 && d.dtype != ZYXB_BF16 && d.dtype != ZYXB_F16 && d.dtype != ZYXB_I32) {
    err = "gemm: dtype must be f32, bf16, f16 or i32"; return ZYXB_ERR_KERNEL_COMPILATION;
  }
  if (d.m == 0 || d.n == 0 || d.k == 0 || d.batch == 0) { err = "gemm: m, n, k and batch must be positive"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.m > 0x7fffffffull || d.n > 0x7fffffffull || d.k > 0x7fffffffull) { err = "gemm: dimension too large"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.epilogue < ZYXB_EPI_NONE || d.epilogue > ZYXB_EPI_MUL_GELU_GRAD) { err = "gemm: unknown epilogue"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.dtype == ZYXB_I32 && (d.epilogue != ZYXB_EPI_NONE || d.store_preact || (d.alpha != 0.0f && d.alpha != 1.0f))) {
    err = "gemm: integer matmul takes no epilogue"; return ZYXB_ERR_KERNEL_COMPILATION;
  }
  if (d.stride_a < 0 || d.stride_b < 0 || d.stride_c < 0) { err = "gemm: negative batch stride"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.batch > 1 && (uint64_t)d.stride_c < d.m * d.n) { err = "gemm: batch stride of C smaller than one matrix"; return ZYXB_ERR_KERNEL_COMPILATION; }
  return ZYXB_OK;
}

int launch_gemm(const zyxb_gemm_desc& d, void* const* args, const uint64_t* arg_bytes, int n_args, const LaunchCtx& lc,
                std::string& err) {
  const bool has_bias = d.epilogue >= ZYXB_EPI_BIAS && d.epilogue <= ZYXB_EPI_BIAS_GELU;
  const bool has_z = d.epilogue == ZYXB_EPI_MUL_RELU_GRAD || d.epilogue == ZYXB_EPI_MUL_GELU_GRAD;
  const int want = 2 + (has_bias || has_z ? 1 : 0) + 1 + (d.store_preact ? 1 : 0);
  ZYXB_CHECK_ARG(n_args == want, "gemm: expected args a, b [,bias | ,z] -> c [,preact]");
  const uint64_t es = dtype_size(d.dtype);
  const uint64_t need_a = ((d.batch - 1) * (uint64_t)d.stride_a + d.m * d.k) * es;
  const uint64_t need_b = ((d.batch - 1) * (uint64_t)d.stride_b + d.k * d.n) * es;
  const uint64_t need_c = ((d.batch - 1) * (uint64_t)d.stride_c + d.m * d.n) * es;
  int i = 0;
  GemmParams p{};
  ZYXB_CHECK_ARG(arg_bytes[i] >= need_a, "gemm: A too small"); p.a = args[i++];
  ZYXB_CHECK_ARG(arg_bytes[i] >= need_b, "gemm: B too small"); p.b = args[i++];
  if (has_bias) { ZYXB_CHECK_ARG(arg_bytes[i] >= d.n * es, "gemm: bias too small"); p.bias = args[i++]; }
  if (has_z) { ZYXB_CHECK_ARG(arg_bytes[i] >= need_c, "gemm: z too small"); p.z = args[i++]; }
  ZYXB_CHECK_ARG(arg_bytes[i] >= need_c, "gemm: C too small"); p.c = args[i++];
  if (d.store_preact) { ZYXB_CHECK_ARG(arg_bytes[i] >= need_c, "gemm: preact too small"); p.preact = args[i++]; }
  p.m = d.m; p.n = d.n; p.k = d.k; p.batch = d.batch;
  p.stride_a = d.stride_a; p.stride_b = d.stride_b; p.stride_c = d.batch > 1 ? d.stride_c : (int64_t)(d.m * d.n);
  p.trans_a = d.trans_a ? 1 : 0; p.trans_b = d.trans_b ? 1 : 0; p.epilogue = d.epilogue;
  p.alpha = d.alpha == 0.0f ? 1.0f : d.alpha; p.rn = lc.round_nearest ? 1 : 0;
  static const bool force_simt = getenv("ZYXB_FORCE_SIMT_GEMM") != nullptr;
  if (!force_simt && gemm_tc_supported(p, d.dtype, lc)) return launch_gemm_tc(p, d.dtype, lc, err);
  return launch_gemm_simt(p, d.dtype, lc, err);
}

}  // namespace zyxb
