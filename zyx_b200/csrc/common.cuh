// Device-side helpers shared by every kernel file: storage <-> f32 conversions that follow
// the reference C backend (zyx/src/codegen/c.rs:452-497), vector I/O, warp/block reductions.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

namespace zyxb {

struct bf16_t { uint16_t bits; };
struct f16_t { uint16_t bits; };

// ---- conversions -----------------------------------------------------------------------
// Loads widen exactly.  Stores truncate by default, as f32tobf16 / f32tof16 in the reference
// C backend do (bits >> 16; f16: mantissa cut, subnormals flushed to signed zero), or round
// to nearest even when the context was created with round_nearest.
__device__ __forceinline__ float bf16_to_f32(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }
__device__ __forceinline__ uint16_t f32_to_bf16(float v, bool rn) {
  uint32_t b = __float_as_uint(v);
  if (rn) {
    if ((b & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((b >> 16) | 0x40);  // quiet NaN
    b += 0x7fffu + ((b >> 16) & 1u);
  }
  return (uint16_t)(b >> 16);
}
__device__ __forceinline__ float f16_to_f32(uint16_t h) { return __half2float(__ushort_as_half(h)); }   // exact, IEEE subnormals
__device__ __forceinline__ uint16_t f32_to_f16(float v, bool rn) {
  uint32_t f = __float_as_uint(v);
  uint32_t sign = (f >> 16) & 0x8000u, exp = (f >> 23) & 0xff, man = f & 0x7fffffu;
  if (exp == 0) return (uint16_t)sign;
  if (exp == 255) return (uint16_t)(sign | 0x7c00u | (man >> 13));
  int ne = (int)exp - 127 + 15;
  if (ne >= 31) return (uint16_t)(sign | 0x7c00u);
  if (ne <= 0) return (uint16_t)sign;
  uint32_t h = sign | ((uint32_t)ne << 10) | (man >> 13);
  if (rn) {
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h += 1;  // may carry into the exponent: still correct
  }
  return (uint16_t)h;
}

template <typename T> struct Elem;
template <> struct Elem<float> {
  using store_t = float; using acc_t = float;
  static __device__ __forceinline__ float load(float v) { return v; }
  static __device__ __forceinline__ float store(float v, bool) { return v; }
};
template <> struct Elem<bf16_t> {
  using store_t = uint16_t; using acc_t = float;
  static __device__ __forceinline__ float load(uint16_t v) { return bf16_to_f32(v); }
  static __device__ __forceinline__ uint16_t store(float v, bool rn) { return f32_to_bf16(v, rn); }
};
template <> struct Elem<f16_t> {
  using store_t = uint16_t; using acc_t = float;
  static __device__ __forceinline__ float load(uint16_t v) { return f16_to_f32(v); }
  static __device__ __forceinline__ uint16_t store(float v, bool rn) { return f32_to_f16(v, rn); }
};
template <> struct Elem<int32_t> {
  using store_t = int32_t; using acc_t = int32_t;
  static __device__ __forceinline__ int32_t load(int32_t v) { return v; }
  static __device__ __forceinline__ int32_t store(int32_t v, bool) { return v; }
};

// a rank-0 scalar operand is cast to the tensor dtype before use (zyx/src/tensor/mod.rs:3033-3113)
template <typename T> __device__ __forceinline__ float const_cast_dtype(float v) {
  return Elem<T>::load(Elem<T>::store(v, false));
}
template <> __device__ __forceinline__ float const_cast_dtype<float>(float v) { return v; }

// ---- 128-bit vector I/O ------------------------------------------------------------------
// VEC elements of storage type S moved as one aligned access when VEC * sizeof(S) == 16.
template <typename S, int VEC> struct alignas(sizeof(S) * VEC) Pack { S v[VEC]; };

template <typename S, int VEC>
__device__ __forceinline__ Pack<S, VEC> load_pack(const S* p) {
  return *reinterpret_cast<const Pack<S, VEC>*>(p);
}
// streaming variants: data touched once, keep it from displacing L2-resident operands
template <typename S, int VEC>
__device__ __forceinline__ Pack<S, VEC> load_pack_stream(const S* p) {
  Pack<S, VEC> r;
  if constexpr (sizeof(S) * VEC == 16) {
    uint4 u = __ldcs(reinterpret_cast<const uint4*>(p));
    r = *reinterpret_cast<Pack<S, VEC>*>(&u);
  } else {
    r = *reinterpret_cast<const Pack<S, VEC>*>(p);
  }
  return r;
}
template <typename S, int VEC>
__device__ __forceinline__ void store_pack(S* p, const Pack<S, VEC>& v) {
  *reinterpret_cast<Pack<S, VEC>*>(p) = v;
}
template <typename S, int VEC>
__device__ __forceinline__ void store_pack_stream(S* p, const Pack<S, VEC>& v) {
  if constexpr (sizeof(S) * VEC == 16) {
    __stcs(reinterpret_cast<uint4*>(p), *reinterpret_cast<const uint4*>(&v));
  } else {
    *reinterpret_cast<Pack<S, VEC>*>(p) = v;
  }
}

// The register image of VEC storage elements, held as 32-bit words whenever the byte count allows, so that a 128-bit
// load of eight 16-bit values stays four registers until a pass widens it (two ALU operations per bf16 pair) and a store
// packs a truncated bf16 pair with one byte permute (the high halves of two f32 words).
template <typename T, int VEC> struct RawVec {
  using S = typename Elem<T>::store_t;
  using A = typename Elem<T>::acc_t;
  static constexpr int BYTES = VEC * (int)sizeof(S);
  static constexpr bool WORDS = BYTES % 4 == 0;
  static constexpr int NW = WORDS ? BYTES / 4 : 1;
  uint32_t w[NW];

  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < NW; ++i) w[i] = 0u;
  }
  __device__ __forceinline__ void load_stream(const S* p) {
    if constexpr (BYTES == 16) {
      const uint4 u = __ldcs(reinterpret_cast<const uint4*>(p));
      w[0] = u.x; w[1] = u.y; w[2] = u.z; w[3] = u.w;
    } else if constexpr (BYTES == 8) {
      const uint2 u = __ldcs(reinterpret_cast<const uint2*>(p));
      w[0] = u.x; w[1] = u.y;
    } else if constexpr (WORDS) {
#pragma unroll
      for (int i = 0; i < NW; ++i) w[i] = reinterpret_cast<const uint32_t*>(p)[i];
    } else {
      w[0] = (uint32_t)*reinterpret_cast<const uint16_t*>(p);
    }
  }
  __device__ __forceinline__ void load(const S* p) {
    if constexpr (BYTES == 16) {
      const uint4 u = *reinterpret_cast<const uint4*>(p);
      w[0] = u.x; w[1] = u.y; w[2] = u.z; w[3] = u.w;
    } else {
      load_stream(p);
    }
  }
  __device__ __forceinline__ void store(S* p) const {
    if constexpr (BYTES == 16) *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    else store_stream(p);
  }
  __device__ __forceinline__ void store_stream(S* p) const {
    if constexpr (BYTES == 16) {
      __stcs(reinterpret_cast<uint4*>(p), make_uint4(w[0], w[1], w[2], w[3]));
    } else if constexpr (BYTES == 8) {
      __stcs(reinterpret_cast<uint2*>(p), make_uint2(w[0], w[1]));
    } else if constexpr (WORDS) {
#pragma unroll
      for (int i = 0; i < NW; ++i) reinterpret_cast<uint32_t*>(p)[i] = w[i];
    } else {
      *reinterpret_cast<uint16_t*>(p) = (uint16_t)w[0];
    }
  }
  __device__ __forceinline__ void decode(A (&out)[VEC]) const {
    if constexpr (sizeof(S) == 4) {
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        if constexpr (std::is_same_v<A, float>) out[k] = __uint_as_float(w[k]); else out[k] = (A)w[k];
      }
    } else if constexpr (WORDS) {
#pragma unroll
      for (int j = 0; j < NW; ++j) {
        if constexpr (std::is_same_v<T, bf16_t>) {
          out[2 * j] = __uint_as_float(w[j] << 16);
          out[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        } else {
          out[2 * j] = Elem<T>::load((uint16_t)(w[j] & 0xffffu));
          out[2 * j + 1] = Elem<T>::load((uint16_t)(w[j] >> 16));
        }
      }
    } else {
      out[0] = Elem<T>::load((uint16_t)w[0]);
    }
  }
  __device__ __forceinline__ void encode(const A (&val)[VEC], bool rn) {
    if constexpr (sizeof(S) == 4) {
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        if constexpr (std::is_same_v<A, float>) w[k] = __float_as_uint(val[k]); else w[k] = (uint32_t)val[k];
      }
    } else if constexpr (WORDS) {
      if constexpr (std::is_same_v<T, bf16_t>) {
        if (!rn) {
#pragma unroll
          for (int j = 0; j < NW; ++j) w[j] = __byte_perm(__float_as_uint(val[2 * j]), __float_as_uint(val[2 * j + 1]), 0x7632);
          return;
        }
      }
#pragma unroll
      for (int j = 0; j < NW; ++j)
        w[j] = (uint32_t)Elem<T>::store(val[2 * j], rn) | ((uint32_t)Elem<T>::store(val[2 * j + 1], rn) << 16);
    } else {
      w[0] = (uint32_t)Elem<T>::store(val[0], rn);
    }
  }
};

// ---- reductions ----------------------------------------------------------------------------
struct OpSum { template <typename A> __device__ __forceinline__ A operator()(A a, A b) const { return a + b; } };
struct OpMax { template <typename A> __device__ __forceinline__ A operator()(A a, A b) const { return a > b ? a : b; } };
struct OpMin { template <typename A> __device__ __forceinline__ A operator()(A a, A b) const { return a < b ? a : b; } };
struct OpMaxF { __device__ __forceinline__ float operator()(float a, float b) const { return fmaxf(a, b); } };

template <typename A, typename Op>
__device__ __forceinline__ A warp_reduce(A v, Op op) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = op(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Reduce across a group of GROUP threads (GROUP == 32: a warp; otherwise the whole CTA, whose
// size must be GROUP).  `scratch` needs GROUP/32 elements of shared memory; every thread of the
// group gets the result.  Two barriers per call make back-to-back calls on one scratch safe.
template <int GROUP, typename A, typename Op>
__device__ __forceinline__ A group_reduce(A v, Op op, A* scratch, A identity) {
  v = warp_reduce(v, op);
  if constexpr (GROUP > 32) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    A w = (lane < GROUP / 32) ? scratch[lane] : identity;
    v = warp_reduce(w, op);
    __syncthreads();
  }
  return v;
}

}  // namespace zyxb

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device setting of a kernel: a context that drives several GPUs must raise
// it on each of them.  `mask` (one static word per kernel instantiation) remembers the CUDA devices already configured.
template <class Kernel>
inline cudaError_t ensure_dynamic_smem(Kernel kern, int bytes, uint64_t* mask) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const uint64_t bit = 1ull << (dev & 63);
  if (*mask & bit) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) *mask |= bit;
  return e;
}
