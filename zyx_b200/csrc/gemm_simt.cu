// SIMT matmul on the FP32 / INT32 pipes: the exact path.
//   - f32: the tuned f32 matmul (tensor cores would need TF32, which cannot hold 1e-5);
//   - i32: bit-exact integer matmul (wrapping i32 accumulator, zyx/src/tensor/reduce_ops.rs:52-60);
//   - bf16 / f16: shapes the tensor-core kernel does not take (tiny or unaligned); products
//     are exact in f32 and the accumulator is f32, as in the reference C backend.
// C[b] = epi(alpha * op(A[b]) . op(B[b]) + bias)      Tensor::dot, zyx/src/tensor/mod.rs:1469-1490
//
// 128x128 output tile per CTA, BK = 16, 256 threads, 8x8 accumulators per thread, operands
// staged through shared memory as [k][m] / [k][n] so that the inner product reads two
// conflict-free float4 per operand per k; the next k-tile is fetched into registers while
// the current one is multiplied (one barrier per k-tile).
#include <algorithm>

#include "common.cuh"
#include "eltwise_math.cuh"
#include "gemm.h"

namespace zyxb {

constexpr int SBM = 128, SBN = 128, SBK = 16, STHREADS = 256;
constexpr int SPAD = 4;   // row padding of the staged tiles (keeps the transposing stores to 2-way conflicts)

// Fetch 4 consecutive elements along the contiguous axis of an operand, zero outside the
// matrix.  `vec` says the 4 elements may be read with one aligned access.
template <typename T, typename ACC>
__device__ __forceinline__ void fetch4(const typename Elem<T>::store_t* base, int64_t ld, int64_t outer, int64_t inner,
                                       int64_t outer_lim, int64_t inner_lim, bool vec, ACC (&out)[4]) {
  using S = typename Elem<T>::store_t;
#pragma unroll
  for (int c = 0; c < 4; ++c) out[c] = (ACC)0;
  if (outer >= outer_lim || inner >= inner_lim) return;
  const S* p = base + outer * ld + inner;
  if (vec && inner + 4 <= inner_lim) {
    Pack<S, 4> pk = load_pack<S, 4>(p);
#pragma unroll
    for (int c = 0; c < 4; ++c) out[c] = (ACC)Elem<T>::load(pk.v[c]);
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c)
      if (inner + c < inner_lim) out[c] = (ACC)Elem<T>::load(p[c]);
  }
}

template <typename T, typename ACC, bool TA, bool TB>
__global__ void __launch_bounds__(STHREADS) gemm_simt_kernel(GemmParams p) {
  using S = typename Elem<T>::store_t;
  __shared__ __align__(16) ACC As[2][SBK][SBM + SPAD];
  __shared__ __align__(16) ACC Bs[2][SBK][SBN + SPAD];
  const int tid = threadIdx.x;
  const int64_t m = p.m, n = p.n, k = p.k;
  const int64_t m0 = (int64_t)blockIdx.y * SBM, n0 = (int64_t)blockIdx.x * SBN;
  const int64_t bz = blockIdx.z / p.splits, split = blockIdx.z % p.splits;
  const int64_t zo = bz / p.batch_inner, zi = bz % p.batch_inner;
  const S* A = reinterpret_cast<const S*>(p.a) + zo * p.stride_a + zi * p.stride_a_inner;
  const S* B = reinterpret_cast<const S*>(p.b) + zo * p.stride_b + zi * p.stride_b_inner;
  const int64_t lda = (int64_t)p.lda, ldb = (int64_t)p.ldb, ldc = (int64_t)p.ldc;
  const int64_t c_off = zo * p.stride_c + zi * p.stride_c_inner;
  const bool va = p.vec_a, vb = p.vec_b;

  // per-thread fetch coordinates: two 4-element groups of A and of B per k-tile
  ACC ra[2][4], rb[2][4];
  auto fetch_tile = [&](int64_t k0) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int g = tid + j * STHREADS;   // 0..511
      if constexpr (TA) {   // A stored [k, m]: contiguous along m
        const int kk = g / (SBM / 4), mi = (g % (SBM / 4)) * 4;
        fetch4<T, ACC>(A, lda, k0 + kk, m0 + mi, k, m, va, ra[j]);
      } else {              // A stored [m, k]: contiguous along k
        const int mi = g / (SBK / 4), kk = (g % (SBK / 4)) * 4;
        fetch4<T, ACC>(A, lda, m0 + mi, k0 + kk, m, k, va, ra[j]);
      }
      if constexpr (TB) {   // B stored [n, k]: contiguous along k
        const int ni = g / (SBK / 4), kk = (g % (SBK / 4)) * 4;
        fetch4<T, ACC>(B, ldb, n0 + ni, k0 + kk, n, k, vb, rb[j]);
      } else {              // B stored [k, n]: contiguous along n
        const int kk = g / (SBN / 4), ni = (g % (SBN / 4)) * 4;
        fetch4<T, ACC>(B, ldb, k0 + kk, n0 + ni, k, n, vb, rb[j]);
      }
    }
  };
  auto stage_tile = [&](int buf) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int g = tid + j * STHREADS;
      if constexpr (TA) {
        const int kk = g / (SBM / 4), mi = (g % (SBM / 4)) * 4;
#pragma unroll
        for (int c = 0; c < 4; ++c) As[buf][kk][mi + c] = ra[j][c];
      } else {
        const int mi = g / (SBK / 4), kk = (g % (SBK / 4)) * 4;
#pragma unroll
        for (int c = 0; c < 4; ++c) As[buf][kk + c][mi] = ra[j][c];
      }
      if constexpr (TB) {
        const int ni = g / (SBK / 4), kk = (g % (SBK / 4)) * 4;
#pragma unroll
        for (int c = 0; c < 4; ++c) Bs[buf][kk + c][ni] = rb[j][c];
      } else {
        const int kk = g / (SBN / 4), ni = (g % (SBN / 4)) * 4;
#pragma unroll
        for (int c = 0; c < 4; ++c) Bs[buf][kk][ni + c] = rb[j][c];
      }
    }
  };

  const int ty = tid / 16, tx = tid % 16;   // 16 x 16 threads, each 2x2 blocks of 4x4
  ACC acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = (ACC)0;

  const int64_t all_tiles = (k + SBK - 1) / SBK;
  const int64_t per_split = (all_tiles + p.splits - 1) / p.splits;
  const int64_t t_first = split * per_split, n_tiles = min(all_tiles, t_first + per_split);   // this CTA's k-tiles: [t_first, n_tiles)
  if (t_first < n_tiles) {
    fetch_tile(t_first * SBK);
    stage_tile((int)(t_first & 1));
  }
  __syncthreads();
  for (int64_t t = t_first; t < n_tiles; ++t) {
    const int buf = (int)(t & 1);
    if (t + 1 < n_tiles) fetch_tile((t + 1) * SBK);
#pragma unroll
    for (int kk = 0; kk < SBK; ++kk) {
      ACC a[8], b[8];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          a[h * 4 + c] = As[buf][kk][h * 64 + ty * 4 + c];
          b[h * 4 + c] = Bs[buf][kk][h * 64 + tx * 4 + c];
        }
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if constexpr (std::is_same_v<ACC, float>) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          else acc[i][j] = (ACC)((uint32_t)acc[i][j] + (uint32_t)a[i] * (uint32_t)b[j]);
        }
    }
    if (t + 1 < n_tiles) {
      stage_tile(buf ^ 1);
      __syncthreads();
    }
  }

  if (p.splits > 1) {   // partial sums of this k range; gemm_splitk_finish_kernel adds them in order and applies the epilogue
    ACC* part = reinterpret_cast<ACC*>(p.partial) + ((bz * p.splits + split) * m) * n;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int64_t r = m0 + (i / 4) * 64 + ty * 4 + (i % 4);
      if (r >= m) continue;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int64_t c = n0 + (j / 4) * 64 + tx * 4 + (j % 4);
        if (c < n) part[r * n + c] = acc[i][j];
      }
    }
    return;
  }
  // epilogue: alpha, bias, activation; optional second output with the pre-activation
  S* C = reinterpret_cast<S*>(p.c) + c_off;
  S* Z = p.preact ? reinterpret_cast<S*>(p.preact) + c_off : nullptr;
  const S* bias = reinterpret_cast<const S*>(p.bias);
  const S* zin = p.z ? reinterpret_cast<const S*>(p.z) + c_off : nullptr;
  const bool rn = p.rn != 0;
  if constexpr (std::is_same_v<ACC, float>) {
    const GeluConsts gc = gelu_consts<T>();
    const float calpha = const_cast_dtype<T>(p.alpha);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int64_t r = m0 + (i / 4) * 64 + ty * 4 + (i % 4);
      if (r >= m) continue;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int64_t c = n0 + (j / 4) * 64 + tx * 4 + (j % 4);
        if (c >= n) continue;
        float v = acc[i][j];
        if (p.alpha != 1.0f) v *= calpha;
        if (p.epilogue >= ZYXB_EPI_BIAS && p.epilogue <= ZYXB_EPI_BIAS_GELU) v += (float)Elem<T>::load(bias[c]);
        if (Z) Z[r * ldc + c] = Elem<T>::store(v, rn);
        if (p.epilogue == ZYXB_EPI_BIAS_RELU) v = relu_ref(v);
        else if (p.epilogue == ZYXB_EPI_BIAS_GELU) v = gelu_ref<T>(v, gc);
        else if (p.epilogue == ZYXB_EPI_MUL_RELU_GRAD) v *= ((float)Elem<T>::load(zin[r * ldc + c]) > 0.0f ? 1.0f : 0.0f);
        else if (p.epilogue == ZYXB_EPI_MUL_GELU_GRAD) v *= gelu_grad_ref<T>((float)Elem<T>::load(zin[r * ldc + c]), gc);
        else if (p.epilogue == ZYXB_EPI_ADD) v += (float)Elem<T>::load(zin[r * ldc + c]);
        C[r * ldc + c] = Elem<T>::store(v, rn);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int64_t r = m0 + (i / 4) * 64 + ty * 4 + (i % 4);
      if (r >= m) continue;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int64_t c = n0 + (j / 4) * 64 + tx * 4 + (j % 4);
        if (c < n) C[r * ldc + c] = acc[i][j];
      }
    }
  }
}

// Second pass of a split-k matmul: the partial sums of each output element are added in split order (so the result does
// not depend on which CTA finished first) and the epilogue is applied.
template <typename T, typename ACC>
__global__ void __launch_bounds__(256) gemm_splitk_finish_kernel(GemmParams p) {
  using S = typename Elem<T>::store_t;
  const int64_t m = p.m, n = p.n, ldc = (int64_t)p.ldc;
  const int64_t per = m * n, total = per * (int64_t)(p.batch * p.batch_inner);
  const ACC* part = reinterpret_cast<const ACC*>(p.partial);
  const S* bias = reinterpret_cast<const S*>(p.bias);
  const bool rn = p.rn != 0;
  for (int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * 256) {
    const int64_t bz = idx / per, e = idx % per, r = e / n, c = e % n;
    const int64_t zo = bz / p.batch_inner, zi = bz % p.batch_inner;
    const int64_t off = zo * p.stride_c + zi * p.stride_c_inner + r * ldc + c;
    ACC sum = (ACC)0;
    for (int s = 0; s < p.splits; ++s) {
      const ACC v = part[(bz * p.splits + s) * per + e];
      if constexpr (std::is_same_v<ACC, float>) sum += v; else sum = (ACC)((uint32_t)sum + (uint32_t)v);
    }
    S* C = reinterpret_cast<S*>(p.c);
    if constexpr (std::is_same_v<ACC, float>) {
      const GeluConsts gc = gelu_consts<T>();
      const S* zin = reinterpret_cast<const S*>(p.z);
      float v = sum;
      if (p.alpha != 1.0f) v *= const_cast_dtype<T>(p.alpha);
      if (p.epilogue >= ZYXB_EPI_BIAS && p.epilogue <= ZYXB_EPI_BIAS_GELU) v += (float)Elem<T>::load(bias[c]);
      if (p.preact) reinterpret_cast<S*>(p.preact)[off] = Elem<T>::store(v, rn);
      if (p.epilogue == ZYXB_EPI_BIAS_RELU) v = relu_ref(v);
      else if (p.epilogue == ZYXB_EPI_BIAS_GELU) v = gelu_ref<T>(v, gc);
      else if (p.epilogue == ZYXB_EPI_MUL_RELU_GRAD) v *= ((float)Elem<T>::load(zin[off]) > 0.0f ? 1.0f : 0.0f);
      else if (p.epilogue == ZYXB_EPI_MUL_GELU_GRAD) v *= gelu_grad_ref<T>((float)Elem<T>::load(zin[off]), gc);
      else if (p.epilogue == ZYXB_EPI_ADD) v += (float)Elem<T>::load(zin[off]);
      C[off] = Elem<T>::store(v, rn);
    } else {
      C[off] = sum;
    }
  }
}

template <typename T, typename ACC>
static void launch_simt_t(const GemmParams& p, dim3 grid, cudaStream_t s) {
  if (p.trans_a) {
    if (p.trans_b) gemm_simt_kernel<T, ACC, true, true><<<grid, STHREADS, 0, s>>>(p);
    else gemm_simt_kernel<T, ACC, true, false><<<grid, STHREADS, 0, s>>>(p);
  } else {
    if (p.trans_b) gemm_simt_kernel<T, ACC, false, true><<<grid, STHREADS, 0, s>>>(p);
    else gemm_simt_kernel<T, ACC, false, false><<<grid, STHREADS, 0, s>>>(p);
  }
}

int launch_gemm_simt(GemmParams p, int dtype, const LaunchCtx& lc, std::string& err) {
  const uint64_t gx = (p.n + SBN - 1) / SBN, gy = (p.m + SBM - 1) / SBM;
  ZYXB_CHECK_ARG(gy <= 65535 && p.batch * p.batch_inner <= 65535, "gemm: m or batch too large for the SIMT path");
  // Few output tiles and a long k: divide k over several CTAs per tile (a [64, 784] x [784, 128] Linear is one tile and
  // would occupy one SM for 49 k-steps), partial sums in the context's scratch, a second launch adds them in order.
  const uint64_t n_mat = p.batch * p.batch_inner, tiles = gx * gy * n_mat, k_tiles = (p.k + SBK - 1) / SBK;
  p.splits = 1;
  p.partial = lc.scratch;
  if (tiles * 2 <= (uint64_t)lc.sm_count && k_tiles >= 16) {   // k >= 256: shorter sums are not worth a second launch
    uint64_t s = std::min<uint64_t>({k_tiles / 2, ((uint64_t)lc.sm_count + tiles - 1) / tiles, (uint64_t)32});
    while (s > 1 && n_mat * s * p.m * p.n * 4 > lc.scratch_bytes) --s;
    if (s > 1 && n_mat * s <= 65535) p.splits = (int)s;
  }
  dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)(n_mat * p.splits));
  // one aligned access per 4 elements needs the contiguous extent, the batch stride and the base aligned
  const uint64_t es = dtype_size(dtype);
  const uint64_t align_elems = 4;   // one access of 4 elements: 16 B for 4-byte, 8 B for 2-byte types
  p.vec_a = (p.lda % align_elems == 0) && ((uintptr_t)p.a % (4 * es) == 0) && ((uint64_t)p.stride_a % align_elems == 0) &&
            ((uint64_t)p.stride_a_inner % align_elems == 0);
  p.vec_b = (p.ldb % align_elems == 0) && ((uintptr_t)p.b % (4 * es) == 0) && ((uint64_t)p.stride_b % align_elems == 0) &&
            ((uint64_t)p.stride_b_inner % align_elems == 0);
  switch (dtype) {
    case ZYXB_F32: launch_simt_t<float, float>(p, grid, lc.stream); break;
    case ZYXB_BF16: launch_simt_t<bf16_t, float>(p, grid, lc.stream); break;
    case ZYXB_F16: launch_simt_t<f16_t, float>(p, grid, lc.stream); break;
    case ZYXB_I32: launch_simt_t<int32_t, int32_t>(p, grid, lc.stream); break;
    default: err = "gemm: dtype"; return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  }
  if (p.splits > 1) {
    const unsigned fgrid = (unsigned)std::min<uint64_t>((n_mat * p.m * p.n + 255) / 256, (uint64_t)lc.sm_count * 8);
    switch (dtype) {
      case ZYXB_F32: gemm_splitk_finish_kernel<float, float><<<fgrid, 256, 0, lc.stream>>>(p); break;
      case ZYXB_BF16: gemm_splitk_finish_kernel<bf16_t, float><<<fgrid, 256, 0, lc.stream>>>(p); break;
      case ZYXB_F16: gemm_splitk_finish_kernel<f16_t, float><<<fgrid, 256, 0, lc.stream>>>(p); break;
      default: gemm_splitk_finish_kernel<int32_t, int32_t><<<fgrid, 256, 0, lc.stream>>>(p); break;
    }
    return check_launch(lc, err, "gemm_simt (split k)", 2);
  }
  return check_launch(lc, err, "gemm_simt");
}

}  // namespace zyxb
