// Scalar formulas shared by the elementwise kernels and the GEMM epilogues; they restate
// zyx/src/tensor/elementwise.rs so that fused and unfused paths agree with the reference.
#pragma once
#include "common.cuh"

namespace zyxb {

// exp(x) = 2^(x*log2(e)) on the SFU: relative error about 2^-21 for the moderate |x| a softmax
// sees after the row maximum has been subtracted — two instructions instead of ~20, which
// keeps a one-pass softmax memory-bound instead of issue-bound.
__device__ __forceinline__ float fast_exp(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x * 1.4426950408889634f));
  return r;
}
// f32 tensors get the accurate expf (the tanh-by-exp formulas cancel near zero, so the last
// ulp of exp matters at the 1e-5 level); 16-bit tensors get the SFU form.
template <typename T> __device__ __forceinline__ float exp_for(float x) { return fast_exp(x); }
template <> __device__ __forceinline__ float exp_for<float>(float x) { return expf(x); }

struct GeluConsts { float half, a, s; };
// 0.5, 0.044715 and sqrt(2/pi) as rank-0 scalars cast to the tensor dtype
template <typename T> __device__ __forceinline__ GeluConsts gelu_consts() {
  return GeluConsts{const_cast_dtype<T>(0.5f), const_cast_dtype<T>(0.044715f), const_cast_dtype<T>(0.7978845608028654f)};
}
__device__ __forceinline__ float relu_ref(float x) { return (x > 0.0f ? 1.0f : 0.0f) * x; }
template <typename T> __device__ __forceinline__ float tanh_ref(float x) {
  const float e = exp_for<T>(x + x);
  return (e - 1.0f) / (e + 1.0f);
}
template <typename T> __device__ __forceinline__ float gelu_ref(float x, const GeluConsts& c) {
  return x * c.half * (tanh_ref<T>((x + x * x * x * c.a) * c.s) + 1.0f);
}
// derivative of gelu_ref by the product and chain rules
template <typename T> __device__ __forceinline__ float gelu_grad_ref(float x, const GeluConsts& c) {
  const float u = (x + x * x * x * c.a) * c.s;
  const float t = tanh_ref<T>(u);
  const float du = (1.0f + 3.0f * c.a * x * x) * c.s;
  return c.half * (t + 1.0f) + x * c.half * (1.0f - t * t) * du;
}

}  // namespace zyxb
