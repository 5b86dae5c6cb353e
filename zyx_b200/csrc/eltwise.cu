// Elementwise kernels: 128-bit vectorised, grid-stride, one read of every input and one
// write of the output.  Formulas follow zyx/src/tensor/elementwise.rs literally:
//   relu = (x > 0) * x                                  (289-293)
//   tanh = (exp(x+x) - 1) / (exp(x+x) + 1)              (585-588)
//   gelu = x * 0.5 * (tanh((x + x*x*x*0.044715) * sqrt(2/pi)) + 1)   (168-170)
//   sigmoid = exp(x) / (exp(x) + 1)                     (457-460)
// with scalar constants cast to the tensor dtype first (zyx/src/tensor/mod.rs:3033-3113).
#include <algorithm>

#include "common.cuh"
#include "eltwise_math.cuh"
#include "internal.h"

namespace zyxb {

struct EwParams {
  const void* a; const void* b; void* y;
  uint64_t n_vec;   // number of VEC-wide packs
  uint64_t cols;    // BIAS_ADD
  float p0;
  int rn;
};

template <typename T, typename TO, int VEC, int OP>
__global__ void __launch_bounds__(256) eltwise_kernel(EwParams p) {
  using S = typename Elem<T>::store_t;
  using SO = typename Elem<TO>::store_t;
  const S* a = reinterpret_cast<const S*>(p.a);
  const S* b = reinterpret_cast<const S*>(p.b);
  SO* y = reinterpret_cast<SO*>(p.y);
  const GeluConsts gc = gelu_consts<T>();
  const float cp = const_cast_dtype<T>(p.p0);
  const bool rn = p.rn != 0;
  constexpr bool BINARY = (OP == ZYXB_EW_ADD || OP == ZYXB_EW_SUB || OP == ZYXB_EW_MUL || OP == ZYXB_EW_RELU_BWD ||
                           OP == ZYXB_EW_GELU_BWD || OP == ZYXB_EW_MSE_BWD);
  for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < p.n_vec; i += (uint64_t)gridDim.x * 256) {
    RawVec<T, VEC> pa, pb;
    pa.load_stream(a + i * VEC);
    if constexpr (BINARY) pb.load_stream(b + i * VEC);
    if constexpr (OP == ZYXB_EW_BIAS_ADD) {
      if constexpr (VEC > 1) pb.load(b + (i * VEC) % p.cols);   // cols % VEC == 0 checked by the host
      else pb.load(b + i % p.cols);
    }
    typename Elem<T>::acc_t xa[VEC], za[VEC];
    pa.decode(xa);
    if constexpr (BINARY || OP == ZYXB_EW_BIAS_ADD) pb.decode(za);
    typename Elem<TO>::acc_t ro[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      const float x = (float)xa[k];
      float z = 0.0f, r;
      if constexpr (BINARY || OP == ZYXB_EW_BIAS_ADD) z = (float)za[k];
      if constexpr (OP == ZYXB_EW_RELU) r = relu_ref(x);
      else if constexpr (OP == ZYXB_EW_GELU) r = gelu_ref<T>(x, gc);
      else if constexpr (OP == ZYXB_EW_ADD || OP == ZYXB_EW_BIAS_ADD) r = x + z;
      else if constexpr (OP == ZYXB_EW_SUB) r = x - z;
      else if constexpr (OP == ZYXB_EW_MUL) r = x * z;
      else if constexpr (OP == ZYXB_EW_SCALE) r = x * cp;
      else if constexpr (OP == ZYXB_EW_RELU_BWD) r = x * (z > 0.0f ? 1.0f : 0.0f);
      else if constexpr (OP == ZYXB_EW_GELU_BWD) r = x * gelu_grad_ref<T>(z, gc);
      else if constexpr (OP == ZYXB_EW_MSE_BWD) r = (x - z) * 2.0f * p.p0;
      else if constexpr (OP == ZYXB_EW_TANH) r = tanh_ref<T>(x);
      else if constexpr (OP == ZYXB_EW_SIGMOID) { const float e = exp_for<T>(x); r = e / (e + 1.0f); }
      else if constexpr (OP == ZYXB_EW_EXP) r = exp_for<T>(x);
      else r = x;  // CAST
      ro[k] = (typename Elem<TO>::acc_t)r;
    }
    RawVec<TO, VEC> out;
    out.encode(ro, rn);
    out.store_stream(y + i * VEC);
  }
}

template <typename T, typename TO, int OP>
static void launch_ew(const zyxb_eltwise_desc& d, void* const* args, int n_in, const LaunchCtx& lc) {
  using S = typename Elem<T>::store_t;
  using SO = typename Elem<TO>::store_t;
  constexpr int V = 16 / (sizeof(S) > sizeof(SO) ? sizeof(S) : sizeof(SO));
  EwParams p{};
  p.a = args[0]; p.b = n_in > 1 ? args[1] : nullptr; p.y = args[n_in]; p.cols = d.cols ? d.cols : 1; p.p0 = d.p0;
  p.rn = lc.round_nearest ? 1 : 0;
  bool vec_ok = d.numel % V == 0 && (uintptr_t)p.a % 16 == 0 && (uintptr_t)p.y % 16 == 0 && (p.b == nullptr || (uintptr_t)p.b % 16 == 0);
  if (OP == ZYXB_EW_BIAS_ADD) vec_ok = vec_ok && (p.cols % V == 0);
  p.n_vec = vec_ok ? d.numel / V : d.numel;
  const unsigned grid = (unsigned)std::max<uint64_t>(1, std::min<uint64_t>((p.n_vec + 255) / 256, 16ull * lc.sm_count));
  if (vec_ok) eltwise_kernel<T, TO, V, OP><<<grid, 256, 0, lc.stream>>>(p);
  else eltwise_kernel<T, TO, 1, OP><<<grid, 256, 0, lc.stream>>>(p);
}

template <typename T>
static void launch_ew_dtype(const zyxb_eltwise_desc& d, void* const* args, int n_in, const LaunchCtx& lc) {
  switch (d.op) {
#define ZYXB_EW_CASE(OP) case OP: launch_ew<T, T, OP>(d, args, n_in, lc); break;
    ZYXB_EW_CASE(ZYXB_EW_RELU) ZYXB_EW_CASE(ZYXB_EW_GELU) ZYXB_EW_CASE(ZYXB_EW_ADD) ZYXB_EW_CASE(ZYXB_EW_SUB)
    ZYXB_EW_CASE(ZYXB_EW_MUL) ZYXB_EW_CASE(ZYXB_EW_SCALE) ZYXB_EW_CASE(ZYXB_EW_RELU_BWD) ZYXB_EW_CASE(ZYXB_EW_GELU_BWD)
    ZYXB_EW_CASE(ZYXB_EW_MSE_BWD) ZYXB_EW_CASE(ZYXB_EW_TANH) ZYXB_EW_CASE(ZYXB_EW_SIGMOID) ZYXB_EW_CASE(ZYXB_EW_EXP)
    ZYXB_EW_CASE(ZYXB_EW_BIAS_ADD)
#undef ZYXB_EW_CASE
    default: break;
  }
}

static int ew_inputs(int op) {
  switch (op) {
    case ZYXB_EW_ADD: case ZYXB_EW_SUB: case ZYXB_EW_MUL: case ZYXB_EW_RELU_BWD: case ZYXB_EW_GELU_BWD: case ZYXB_EW_MSE_BWD:
    case ZYXB_EW_BIAS_ADD: return 2;
    default: return 1;
  }
}
static bool ew_float(int d) { return d == ZYXB_F32 || d == ZYXB_BF16 || d == ZYXB_F16; }

int validate_eltwise(const zyxb_eltwise_desc& d, std::string& err) {
  if (d.op < ZYXB_EW_RELU || d.op > ZYXB_EW_BIAS_ADD) { err = "eltwise: unknown op"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.numel == 0) { err = "eltwise: numel must be positive"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (!ew_float(d.dtype)) { err = "eltwise: dtype must be f32, bf16 or f16"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.op == ZYXB_EW_CAST && !ew_float(d.dtype_out)) { err = "cast: dtype_out must be f32, bf16 or f16"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.op == ZYXB_EW_BIAS_ADD && (d.cols == 0 || d.numel % d.cols != 0)) { err = "bias_add: numel must be a multiple of cols"; return ZYXB_ERR_KERNEL_COMPILATION; }
  return ZYXB_OK;
}

template <typename T>
static void launch_cast_from(const zyxb_eltwise_desc& d, void* const* args, const LaunchCtx& lc) {
  switch (d.dtype_out) {
    case ZYXB_F32: launch_ew<T, float, ZYXB_EW_CAST>(d, args, 1, lc); break;
    case ZYXB_BF16: launch_ew<T, bf16_t, ZYXB_EW_CAST>(d, args, 1, lc); break;
    default: launch_ew<T, f16_t, ZYXB_EW_CAST>(d, args, 1, lc); break;
  }
}

int launch_eltwise(const zyxb_eltwise_desc& d, void* const* args, const uint64_t* arg_bytes, int n_args, const LaunchCtx& lc,
                   std::string& err) {
  const int n_in = ew_inputs(d.op);
  ZYXB_CHECK_ARG(n_args == n_in + 1, "eltwise: wrong number of arguments");
  const uint64_t es = dtype_size(d.dtype), eo = dtype_size(d.op == ZYXB_EW_CAST ? d.dtype_out : d.dtype);
  ZYXB_CHECK_ARG(arg_bytes[0] >= d.numel * es, "eltwise: first input too small");
  if (n_in == 2) ZYXB_CHECK_ARG(arg_bytes[1] >= (d.op == ZYXB_EW_BIAS_ADD ? d.cols : d.numel) * es, "eltwise: second input too small");
  ZYXB_CHECK_ARG(arg_bytes[n_in] >= d.numel * eo, "eltwise: output too small");
  if (d.op == ZYXB_EW_CAST) {
    switch (d.dtype) {
      case ZYXB_F32: launch_cast_from<float>(d, args, lc); break;
      case ZYXB_BF16: launch_cast_from<bf16_t>(d, args, lc); break;
      default: launch_cast_from<f16_t>(d, args, lc); break;
    }
  } else {
    switch (d.dtype) {
      case ZYXB_F32: launch_ew_dtype<float>(d, args, n_in, lc); break;
      case ZYXB_BF16: launch_ew_dtype<bf16_t>(d, args, n_in, lc); break;
      default: launch_ew_dtype<f16_t>(d, args, n_in, lc); break;
    }
  }
  return check_launch(lc, err, "eltwise");
}

}  // namespace zyxb
