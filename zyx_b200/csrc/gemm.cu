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
  if (d.epilogue < ZYXB_EPI_NONE || d.epilogue > ZYXB_EPI_ADD) { err = "gemm: unknown epilogue"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.dtype == ZYXB_I32 && (d.epilogue != ZYXB_EPI_NONE || d.store_preact || (d.alpha != 0.0f && d.alpha != 1.0f))) {
    err = "gemm: integer matmul takes no epilogue"; return ZYXB_ERR_KERNEL_COMPILATION;
  }
  if (d.stride_a < 0 || d.stride_b < 0 || d.stride_c < 0 || d.stride_a_inner < 0 || d.stride_b_inner < 0 || d.stride_c_inner < 0) {
    err = "gemm: negative batch stride"; return ZYXB_ERR_KERNEL_COMPILATION;
  }
  if (d.tri < ZYXB_TRI_NONE || d.tri > ZYXB_TRI_AT_LOWER) { err = "gemm: unknown triangular mode"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.tri == ZYXB_TRI_OUT_LOWER && d.m != d.n) { err = "gemm: a lower-triangular result needs m == n"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if ((d.tri == ZYXB_TRI_A_LOWER || d.tri == ZYXB_TRI_AT_LOWER) && d.m != d.k) { err = "gemm: a lower-triangular A needs m == k"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if ((d.tri == ZYXB_TRI_A_LOWER && d.trans_a) || (d.tri == ZYXB_TRI_AT_LOWER && !d.trans_a)) {
    err = "gemm: A_LOWER takes A stored [m,k], AT_LOWER takes A stored [k,m]"; return ZYXB_ERR_KERNEL_COMPILATION;
  }
  if (d.batch > 1 && d.stride_c == 0) { err = "gemm: batches of C must not overlap (stride_c is 0)"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.batch_inner > 1 && d.stride_c_inner == 0) { err = "gemm: inner batches of C must not overlap"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.batch * (d.batch_inner ? d.batch_inner : 1) > 65535) { err = "gemm: more than 65535 matrices in one launch"; return ZYXB_ERR_KERNEL_COMPILATION; }
  return ZYXB_OK;
}

// Elements a strided operand spans: the last matrix's offset plus its last row.
// Computed in 128 bits and saturated, so that huge caller-supplied strides or pitches cannot wrap around into a small value
// that passes the buffer-size checks below.
static uint64_t span(uint64_t batch, int64_t stride, uint64_t inner, int64_t stride_inner, uint64_t rows, uint64_t ld, uint64_t cols) {
  if (stride < 0 || stride_inner < 0) return UINT64_MAX;
  const unsigned __int128 v = (unsigned __int128)(batch - 1) * (uint64_t)stride + (unsigned __int128)(inner - 1) * (uint64_t)stride_inner +
                              (unsigned __int128)(rows - 1) * ld + cols;
  return v > ((unsigned __int128)1 << 60) ? UINT64_MAX : (uint64_t)v;
}

int launch_gemm(const zyxb_gemm_desc& d, void* const* args, const uint64_t* arg_bytes, int n_args, const LaunchCtx& lc,
                std::string& err) {
  const bool has_bias = d.epilogue >= ZYXB_EPI_BIAS && d.epilogue <= ZYXB_EPI_BIAS_GELU;
  const bool has_z = d.epilogue == ZYXB_EPI_MUL_RELU_GRAD || d.epilogue == ZYXB_EPI_MUL_GELU_GRAD || d.epilogue == ZYXB_EPI_ADD;
  const int want = 2 + (has_bias || has_z ? 1 : 0) + 1 + (d.store_preact ? 1 : 0);
  ZYXB_CHECK_ARG(n_args == want, "gemm: expected args a, b [,bias | ,z] -> c [,preact]");
  const uint64_t es = dtype_size(d.dtype);
  GemmParams p{};
  p.m = d.m; p.n = d.n; p.k = d.k; p.batch = d.batch;
  p.batch_inner = d.batch_inner ? d.batch_inner : 1;
  p.trans_a = d.trans_a ? 1 : 0; p.trans_b = d.trans_b ? 1 : 0; p.epilogue = d.epilogue; p.tri = d.tri;
  const uint64_t a_rows = p.trans_a ? d.k : d.m, a_cols = p.trans_a ? d.m : d.k;
  const uint64_t b_rows = p.trans_b ? d.n : d.k, b_cols = p.trans_b ? d.k : d.n;
  p.lda = d.lda ? d.lda : a_cols; p.ldb = d.ldb ? d.ldb : b_cols; p.ldc = d.ldc ? d.ldc : d.n;
  ZYXB_CHECK_ARG(p.lda >= a_cols && p.ldb >= b_cols && p.ldc >= d.n, "gemm: row pitch smaller than the row");
  p.stride_a = d.stride_a; p.stride_b = d.stride_b;
  p.stride_c = (d.batch > 1 || d.stride_c) ? d.stride_c : (int64_t)(d.m * p.ldc);
  p.stride_a_inner = d.stride_a_inner; p.stride_b_inner = d.stride_b_inner; p.stride_c_inner = d.stride_c_inner;
  auto bytes_of = [es](uint64_t elems) { return elems == UINT64_MAX ? UINT64_MAX : elems * es; };     // elems <= 2^60, es <= 8
  const uint64_t need_a = bytes_of(span(d.batch, p.stride_a, p.batch_inner, p.stride_a_inner, a_rows, p.lda, a_cols));
  const uint64_t need_b = bytes_of(span(d.batch, p.stride_b, p.batch_inner, p.stride_b_inner, b_rows, p.ldb, b_cols));
  const uint64_t need_c = bytes_of(span(d.batch, p.stride_c, p.batch_inner, p.stride_c_inner, d.m, p.ldc, d.n));
  int i = 0;
  ZYXB_CHECK_ARG(arg_bytes[i] >= need_a, "gemm: A too small"); p.a = args[i++];
  ZYXB_CHECK_ARG(arg_bytes[i] >= need_b, "gemm: B too small"); p.b = args[i++];
  if (has_bias) { ZYXB_CHECK_ARG(arg_bytes[i] >= d.n * es, "gemm: bias too small"); p.bias = args[i++]; }
  if (has_z) { ZYXB_CHECK_ARG(arg_bytes[i] >= need_c, "gemm: z too small"); p.z = args[i++]; }
  ZYXB_CHECK_ARG(arg_bytes[i] >= need_c, "gemm: C too small"); p.c = args[i++];
  if (d.store_preact) { ZYXB_CHECK_ARG(arg_bytes[i] >= need_c, "gemm: preact too small"); p.preact = args[i++]; }
  p.alpha = d.alpha == 0.0f ? 1.0f : d.alpha; p.rn = lc.round_nearest ? 1 : 0;
  static const bool force_simt = getenv("ZYXB_FORCE_SIMT_GEMM") != nullptr;
  if (!force_simt && gemm_tc_supported(p, d.dtype, lc)) return launch_gemm_tc(p, d.dtype, lc, err);
  if (!force_simt && gemm_tf32x3_supported(p, d.dtype, lc)) return launch_gemm_tf32x3(p, lc, err);
  return launch_gemm_simt(p, d.dtype, lc, err);
}

}  // namespace zyxb
