// Row kernels: an elementwise chain with a trailing reduce over the last axis, one pass over HBM.
//
// A row is owned by a GROUP of threads (a warp, or a whole CTA).  When the row fits in
// ITEMS 128-bit vectors per thread it is read from HBM exactly once into registers, reduced
// with warp shuffles (+ one shared-memory hop across warps) and written exactly once.
// ITEMS == 0 selects the streaming form for rows too long for registers: every pass re-reads
// the row (the second and third reads hit L2 for rows up to a few MB).
//
// Arithmetic follows the reference decompositions: softmax / ln_softmax
// (zyx/src/tensor/mod.rs:1427-1461), LayerNorm::forward with unbiased variance
// (zyx-nn/src/layer_norm.rs:95-135, zyx/src/tensor/reduce_ops.rs:113-125), reduce_impl
// (reduce_ops.rs:45-157), cross_entropy (tensor/mod.rs:1639-1655).
#pragma once
#include <stdlib.h>
#include <math_constants.h>

#include <algorithm>
#include <type_traits>

#include "common.cuh"
#include "eltwise_math.cuh"
#include "internal.h"

namespace zyxb {

enum RowFamily { FAM_REDUCE = 0, FAM_SOFTMAX = 1, FAM_LAYERNORM = 2, FAM_SOFTMAX_BWD = 3, FAM_LAYERNORM_BWD = 4, FAM_CE = 5 };

struct RowParams {
  const void* x;    // first input
  const void* x2;   // second input (dp / dy / labels)
  const void* w;    // layernorm weight
  const void* b;    // layernorm bias
  void* y;          // output
  uint64_t rows, cols;
  int op;           // ZYXB_RR_*
  int correction;
  float eps;
  float scale;      // softmax pre-scale (1 = none)
  int causal;
  uint64_t period;
  int rn;           // round-to-nearest stores
  int sm_count;     // host side only: size of the persistent grid of the staged kernel
  uint32_t* status; // device status word (bounded waits report here)
};

// A warp-per-row kernel with two cached inputs holds 2 x ITEMS 128-bit vectors per thread: ask for five CTAs of 128 threads
// per SM (about 100 registers) so the packed rows are decoded per pass instead of being kept as floats at a third of the occupancy.
constexpr int row_min_ctas(int group, int items, int fam) {
  return (group == 32 && items == 8 && (fam == FAM_SOFTMAX_BWD || fam == FAM_LAYERNORM_BWD)) ? 5 : 1;
}

template <typename T, int VEC, int ITEMS, int GROUP, int FAM>
__global__ void __launch_bounds__(GROUP == 32 ? 128 : GROUP, row_min_ctas(GROUP, ITEMS, FAM)) row_kernel(RowParams p) {
  using S = typename Elem<T>::store_t;
  using A = typename Elem<T>::acc_t;
  constexpr bool CACHED = ITEMS > 0;
  constexpr int NI = CACHED ? ITEMS : 1;
  constexpr bool TWO_IN = (FAM == FAM_SOFTMAX_BWD || FAM == FAM_LAYERNORM_BWD);
  __shared__ A red[32];

  const int gl = (GROUP == 32) ? (threadIdx.x & 31) : threadIdx.x;
  const uint64_t row = (GROUP == 32) ? (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5) : (uint64_t)blockIdx.x;
  if (row >= p.rows) return;  // GROUP == 32: whole warps leave, nobody waits on a CTA barrier
  const uint64_t cols = p.cols;
  const S* xr = reinterpret_cast<const S*>(p.x) + row * cols;
  const S* x2r = TWO_IN ? reinterpret_cast<const S*>(p.x2) + row * cols : nullptr;
  const bool rn = p.rn != 0;
  const uint64_t step = (uint64_t)GROUP * VEC;
  const int n_iter = CACHED ? ITEMS : (int)((cols + step - 1) / step);

  // causal softmax (and its backward): columns past the diagonal are masked, so they are never read
  uint64_t lim = cols;
  if constexpr (FAM == FAM_SOFTMAX || FAM == FAM_SOFTMAX_BWD) {
    if (p.causal) lim = min((uint64_t)(row % p.period) + 1, cols);
  }

  // the cached row stays in its storage form (16-bit rows: eight elements per four registers) and is widened per pass
  using Raw = RawVec<T, VEC>;
  Raw v[NI];
  Raw v2[TWO_IN ? NI : 1];
  (void)v2;

  auto fetch_raw = [&](const S* base, uint64_t c) -> Raw {
    Raw r;
    if (c < lim) r.load_stream(base + c); else r.zero();
    return r;
  };
  auto decode = [&](const Raw& r, A (&out)[VEC]) { r.decode(out); };
  if constexpr (CACHED) {
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      const uint64_t c = ((uint64_t)it * GROUP + gl) * VEC;
      if (c < cols) {
        v[it] = fetch_raw(xr, c);
        if constexpr (TWO_IN) v2[it] = fetch_raw(x2r, c);
      }
    }
  }
  // visit every vector of the row that this thread owns: f(column, values, values2)
  auto for_each = [&](auto&& f) {
    if constexpr (CACHED) {
#pragma unroll
      for (int it = 0; it < ITEMS; ++it) {
        const uint64_t c = ((uint64_t)it * GROUP + gl) * VEC;
        if (c < cols) {
          A a[VEC];
          decode(v[it], a);
          if constexpr (TWO_IN) { A a2[VEC]; decode(v2[it], a2); f(c, a, a2); } else f(c, a, a);
        }
      }
    } else {
      for (int it = 0; it < n_iter; ++it) {
        const uint64_t c = ((uint64_t)it * GROUP + gl) * VEC;
        if (c < cols) {
          A a[VEC], a2[VEC];
          decode(fetch_raw(xr, c), a);
          if constexpr (TWO_IN) { decode(fetch_raw(x2r, c), a2); f(c, a, a2); } else f(c, a, a);
        }
      }
    }
  };
  auto write = [&](S* base, uint64_t c, const A (&val)[VEC]) {
    Raw r;
    r.encode(val, rn);
    r.store_stream(base + c);
  };

  // ---------------------------------------------------------------------------------------
  if constexpr (FAM == FAM_REDUCE) {
    S* out = reinterpret_cast<S*>(p.y);
    if constexpr (std::is_same_v<A, int32_t>) {
      // integers: exact, wrapping i32 accumulator
      A acc = (p.op == ZYXB_RR_SUM) ? 0 : (p.op == ZYXB_RR_MAX ? INT32_MIN : INT32_MAX);
      for_each([&](uint64_t, const A (&a)[VEC], const A (&)[VEC]) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          if (p.op == ZYXB_RR_SUM) acc = (A)((uint32_t)acc + (uint32_t)a[k]);
          else if (p.op == ZYXB_RR_MAX) acc = a[k] > acc ? a[k] : acc;
          else acc = a[k] < acc ? a[k] : acc;
        }
      });
      if (p.op == ZYXB_RR_SUM) acc = group_reduce<GROUP>(acc, OpSum(), red, (A)0);
      else if (p.op == ZYXB_RR_MAX) acc = group_reduce<GROUP>(acc, OpMax(), red, (A)INT32_MIN);
      else acc = group_reduce<GROUP>(acc, OpMin(), red, (A)INT32_MAX);
      if (gl == 0) out[row] = acc;
    } else {
      float res;
      if (p.op == ZYXB_RR_MAX || p.op == ZYXB_RR_MIN) {
        const float sgn = p.op == ZYXB_RR_MAX ? 1.0f : -1.0f;   // min = -max(-x)
        float acc = -CUDART_INF_F;
        for_each([&](uint64_t, const A (&a)[VEC], const A (&)[VEC]) {
#pragma unroll
          for (int k = 0; k < VEC; ++k) acc = fmaxf(sgn * (float)a[k], acc);
        });
        res = sgn * group_reduce<GROUP>(acc, OpMaxF(), (float*)red, -CUDART_INF_F);
      } else {
        float acc = 0.0f;
        for_each([&](uint64_t, const A (&a)[VEC], const A (&)[VEC]) {
#pragma unroll
          for (int k = 0; k < VEC; ++k) acc += (float)a[k];
        });
        res = group_reduce<GROUP>(acc, OpSum(), (float*)red, 0.0f);
        if (p.op != ZYXB_RR_SUM) {
          const float mean = res / const_cast_dtype<T>((float)cols);
          res = mean;
          if (p.op == ZYXB_RR_VAR || p.op == ZYXB_RR_STD) {
            float sq = 0.0f;
            for_each([&](uint64_t, const A (&a)[VEC], const A (&)[VEC]) {
#pragma unroll
              for (int k = 0; k < VEC; ++k) { const float d = (float)a[k] - mean; sq = fmaf(d, d, sq); }
            });
            sq = group_reduce<GROUP>(sq, OpSum(), (float*)red, 0.0f);
            res = sq / const_cast_dtype<T>((float)((int64_t)cols - p.correction));
            if (p.op == ZYXB_RR_STD) res = sqrtf(res);
          }
        }
      }
      if (gl == 0) out[row] = Elem<T>::store((A)res, rn);
    }
  }
  // ---------------------------------------------------------------------------------------
  else if constexpr (FAM == FAM_SOFTMAX && CACHED && !std::is_same_v<A, int32_t>) {
    // Cached softmax / ln_softmax.  Work is decided per 128-bit vector: vectors wholly left of the causal limit take the
    // unmasked loops, the one vector that straddles it masks per element, vectors right of it cost nothing but the store of
    // zeros.  The exponentials are computed twice (sum pass, output pass) rather than kept: 64 more live registers per
    // thread cost more in occupancy than the second SFU operation does.
    constexpr float LOG2E = 1.4426950408889634f;
    constexpr bool HALF2 = sizeof(S) == 2 && VEC % 2 == 0;
    const uint32_t cols32 = (uint32_t)cols, lim32 = (uint32_t)lim;
    const float mul = const_cast_dtype<T>(p.scale);      // 1 when unscaled
    float mx = -CUDART_INF_F;
    if (mul > 0.0f) {
      // x -> fl(x * mul) is monotone for mul > 0, so max(x * mul) = max(x) * mul exactly; 16-bit rows take the maximum of
      // whole vectors on the packed pairs
      uint32_t pm = std::is_same_v<T, bf16_t> ? 0xff80ff80u : 0xfc00fc00u;   // (-inf, -inf)
      (void)pm;
#pragma unroll
      for (int it = 0; it < ITEMS; ++it) {
        const uint32_t c = ((uint32_t)it * GROUP + gl) * VEC;
        if (c < lim32) {
          if (c + VEC <= lim32) {
            if constexpr (HALF2) {
#pragma unroll
              for (int j = 0; j < Raw::NW; ++j) {
                if constexpr (std::is_same_v<T, bf16_t>) asm("max.bf16x2 %0, %0, %1;" : "+r"(pm) : "r"(v[it].w[j]));
                else asm("max.f16x2 %0, %0, %1;" : "+r"(pm) : "r"(v[it].w[j]));
              }
            } else {
              A a[VEC];
              decode(v[it], a);
#pragma unroll
              for (int k = 0; k < VEC; ++k) mx = fmaxf((float)a[k], mx);
            }
          } else {
            A a[VEC];
            decode(v[it], a);
#pragma unroll
            for (int k = 0; k < VEC; ++k) mx = (c + k < lim32) ? fmaxf((float)a[k], mx) : mx;
          }
        }
      }
      if constexpr (HALF2) {
        mx = fmaxf(mx, fmaxf((float)Elem<T>::load((uint16_t)(pm & 0xffffu)), (float)Elem<T>::load((uint16_t)(pm >> 16))));
      }
      mx *= mul;
    } else {
#pragma unroll
      for (int it = 0; it < ITEMS; ++it) {
        const uint32_t c = ((uint32_t)it * GROUP + gl) * VEC;
        if (c < lim32) {
          A a[VEC];
          decode(v[it], a);
#pragma unroll
          for (int k = 0; k < VEC; ++k) mx = (c + k < lim32) ? fmaxf((float)a[k] * mul, mx) : mx;
        }
      }
    }
    mx = group_reduce<GROUP>(mx, OpMaxF(), (float*)red, -CUDART_INF_F);
    const float nmx = -mx * LOG2E, m2 = mul * LOG2E;
    S* yr = reinterpret_cast<S*>(p.y) + row * cols;
    // sum pass and output pass.  UNIT: mul == 1, the product is skipped.  16-bit rows fold mul into the exponent's scale
    // (one FMA per element; the argument moves by an ulp, far inside their tolerance), f32 rows round x*mul first as the
    // reference does.
    auto finish = [&](auto log_tag, auto unit_tag) {
      constexpr bool LOGF = decltype(log_tag)::value, UNIT = decltype(unit_tag)::value;
      auto ex = [&](float a) -> float {                     // exp(a*mul - mx)
        float arg, r;
        if constexpr (sizeof(S) == 2) arg = fmaf(a, m2, nmx);
        else if constexpr (UNIT) arg = fmaf(a, LOG2E, nmx);
        else arg = fmaf(a * mul, LOG2E, nmx);
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(arg));
        return r;
      };
      float s = 0.0f;
#pragma unroll
      for (int it = 0; it < ITEMS; ++it) {
        const uint32_t c = ((uint32_t)it * GROUP + gl) * VEC;
        if (c < lim32) {
          A a[VEC];
          decode(v[it], a);
          if (c + VEC <= lim32) {
#pragma unroll
            for (int k = 0; k < VEC; ++k) s += ex((float)a[k]);
          } else {
#pragma unroll
            for (int k = 0; k < VEC; ++k) s += (c + k < lim32) ? ex((float)a[k]) : 0.0f;
          }
        }
      }
      s = group_reduce<GROUP>(s, OpSum(), (float*)red, 0.0f);
      const float inv = 1.0f / s, ls = LOGF ? logf(s) : 0.0f;
      const float MASKED = LOGF ? -CUDART_INF_F : 0.0f;
#pragma unroll
      for (int it = 0; it < ITEMS; ++it) {
        const uint32_t c = ((uint32_t)it * GROUP + gl) * VEC;
        if (c < cols32) {
          A o[VEC];
          if (c < lim32) {
            A a[VEC];
            decode(v[it], a);
            const bool whole = c + VEC <= lim32;
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
              float r;
              if constexpr (LOGF) r = ((UNIT ? (float)a[k] : (float)a[k] * mul) - mx) - ls;
              else r = ex((float)a[k]) * inv;
              if (!whole && !(c + k < lim32)) r = MASKED;
              o[k] = (A)r;
            }
          } else {
#pragma unroll
            for (int k = 0; k < VEC; ++k) o[k] = (A)MASKED;
          }
          write(yr, c, o);
        }
      }
    };
    const bool unit = mul == 1.0f && sizeof(S) == 4;       // 16-bit rows have one variant
    if (p.op == ZYXB_RR_SOFTMAX) { if (unit) finish(std::false_type(), std::true_type()); else finish(std::false_type(), std::false_type()); }
    else { if (unit) finish(std::true_type(), std::true_type()); else finish(std::true_type(), std::false_type()); }
  }
  // ---------------------------------------------------------------------------------------
  else if constexpr (FAM == FAM_SOFTMAX || FAM == FAM_CE) {
    // streamed softmax / ln_softmax and cross-entropy forward/backward all start from max and sum(exp(x-max))
    const bool scaled = p.scale != 1.0f;
    const float cscale = const_cast_dtype<T>(p.scale);
    auto val = [&](float a, uint64_t c) -> float {
      if (scaled) a *= cscale;
      return c < lim ? a : -CUDART_INF_F;
    };
    float mx = -CUDART_INF_F;
    for_each([&](uint64_t c, const A (&a)[VEC], const A (&)[VEC]) {
#pragma unroll
      for (int k = 0; k < VEC; ++k) mx = fmaxf(val((float)a[k], c + k), mx);
    });
    mx = group_reduce<GROUP>(mx, OpMaxF(), (float*)red, -CUDART_INF_F);
    float s = 0.0f;
    for_each([&](uint64_t c, const A (&a)[VEC], const A (&)[VEC]) {
#pragma unroll
      for (int k = 0; k < VEC; ++k) s += fast_exp(val((float)a[k], c + k) - mx);
    });
    s = group_reduce<GROUP>(s, OpSum(), (float*)red, 0.0f);
    if constexpr (FAM == FAM_SOFTMAX) {
      S* yr = reinterpret_cast<S*>(p.y) + row * cols;
      if (p.op == ZYXB_RR_SOFTMAX) {
        const float inv = 1.0f / s;
        for_each([&](uint64_t c, const A (&a)[VEC], const A (&)[VEC]) {
          A o[VEC];
#pragma unroll
          for (int k = 0; k < VEC; ++k) o[k] = (A)(fast_exp(val((float)a[k], c + k) - mx) * inv);
          write(yr, c, o);
        });
      } else {  // ln_softmax: (x - max) - ln(sum)
        const float ls = logf(s);
        for_each([&](uint64_t c, const A (&a)[VEC], const A (&)[VEC]) {
          A o[VEC];
#pragma unroll
          for (int k = 0; k < VEC; ++k) o[k] = (A)((val((float)a[k], c + k) - mx) - ls);
          write(yr, c, o);
        });
      }
    } else {
      const int32_t label = reinterpret_cast<const int32_t*>(p.x2)[row];
      if (p.op == ZYXB_RR_CROSS_ENTROPY) {
        // per_sample = sum_j -((x_j - max) - ln s) * onehot_j: only j == label contributes
        const float ls = logf(s);
        float acc = 0.0f;
        for_each([&](uint64_t c, const A (&a)[VEC], const A (&)[VEC]) {
#pragma unroll
          for (int k = 0; k < VEC; ++k)
            if ((int64_t)(c + k) == (int64_t)label) acc += -(((float)a[k] - mx) - ls);
        });
        acc = group_reduce<GROUP>(acc, OpSum(), (float*)red, 0.0f);
        if (gl == 0) reinterpret_cast<float*>(p.y)[row] = acc;
      } else {  // d mean-CE / d logits = (softmax - onehot) / rows
        S* yr = reinterpret_cast<S*>(p.y) + row * cols;
        const float inv = 1.0f / s, invr = 1.0f / (float)p.rows;
        for_each([&](uint64_t c, const A (&a)[VEC], const A (&)[VEC]) {
          A o[VEC];
#pragma unroll
          for (int k = 0; k < VEC; ++k) {
            const float sm = fast_exp((float)a[k] - mx) * inv;
            o[k] = (A)((sm - ((int64_t)(c + k) == (int64_t)label ? 1.0f : 0.0f)) * invr);
          }
          write(yr, c, o);
        });
      }
    }
  }
  // ---------------------------------------------------------------------------------------
  else if constexpr (FAM == FAM_LAYERNORM) {
    float acc = 0.0f;
    for_each([&](uint64_t, const A (&a)[VEC], const A (&)[VEC]) {
#pragma unroll
      for (int k = 0; k < VEC; ++k) acc += (float)a[k];
    });
    const float mean = group_reduce<GROUP>(acc, OpSum(), (float*)red, 0.0f) / const_cast_dtype<T>((float)cols);
    float sq = 0.0f;
    for_each([&](uint64_t, const A (&a)[VEC], const A (&)[VEC]) {
#pragma unroll
      for (int k = 0; k < VEC; ++k) { const float d = (float)a[k] - mean; sq = fmaf(d, d, sq); }
    });
    sq = group_reduce<GROUP>(sq, OpSum(), (float*)red, 0.0f);
    const float var = sq / const_cast_dtype<T>((float)((int64_t)cols - 1));   // unbiased
    const float rstd = 1.0f / sqrtf(var + const_cast_dtype<T>(p.eps));
    S* yr = reinterpret_cast<S*>(p.y) + row * cols;
    const S* wp = reinterpret_cast<const S*>(p.w);
    const S* bp = reinterpret_cast<const S*>(p.b);
    for_each([&](uint64_t c, const A (&a)[VEC], const A (&)[VEC]) {
      A o[VEC];
#pragma unroll
      for (int k = 0; k < VEC; ++k) o[k] = (A)(((float)a[k] - mean) * rstd);
      if (wp) {
        Raw pk; A wv[VEC];
        pk.load(wp + c); pk.decode(wv);
#pragma unroll
        for (int k = 0; k < VEC; ++k) o[k] = (A)((float)o[k] * (float)wv[k]);
      }
      if (bp) {
        Raw pk; A bv[VEC];
        pk.load(bp + c); pk.decode(bv);
#pragma unroll
        for (int k = 0; k < VEC; ++k) o[k] = (A)((float)o[k] + (float)bv[k]);
      }
      write(yr, c, o);
    });
  }
  // ---------------------------------------------------------------------------------------
  else if constexpr (FAM == FAM_SOFTMAX_BWD && CACHED) {
    // ds = p * (dp - sum(dp * p)), decided per vector like the forward: past a causal diagonal p counts as 0
    const uint32_t cols32 = (uint32_t)cols, lim32 = (uint32_t)lim;
    float acc = 0.0f;
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      const uint32_t c = ((uint32_t)it * GROUP + gl) * VEC;
      if (c < lim32) {
        A a[VEC], d[VEC];
        decode(v[it], a);
        decode(v2[it], d);
        if (c + VEC <= lim32) {
#pragma unroll
          for (int k = 0; k < VEC; ++k) acc = fmaf((float)a[k], (float)d[k], acc);
        } else {
#pragma unroll
          for (int k = 0; k < VEC; ++k) acc = (c + k < lim32) ? fmaf((float)a[k], (float)d[k], acc) : acc;
        }
      }
    }
    acc = group_reduce<GROUP>(acc, OpSum(), (float*)red, 0.0f);
    S* yr = reinterpret_cast<S*>(p.y) + row * cols;
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      const uint32_t c = ((uint32_t)it * GROUP + gl) * VEC;
      if (c < cols32) {
        A o[VEC];
        if (c < lim32) {
          A a[VEC], d[VEC];
          decode(v[it], a);
          decode(v2[it], d);
          const bool whole = c + VEC <= lim32;
#pragma unroll
          for (int k = 0; k < VEC; ++k) {
            const float r = (float)a[k] * ((float)d[k] - acc);
            o[k] = (A)((whole || c + k < lim32) ? r : 0.0f);
          }
        } else {
#pragma unroll
          for (int k = 0; k < VEC; ++k) o[k] = (A)0;
        }
        write(yr, c, o);
      }
    }
  }
  // ---------------------------------------------------------------------------------------
  else if constexpr (FAM == FAM_SOFTMAX_BWD) {
    // streamed form.  ds = p * (dp - sum(dp * p)); elements past a causal diagonal count as p = 0
    float acc = 0.0f;
    for_each([&](uint64_t c, const A (&a)[VEC], const A (&d)[VEC]) {
#pragma unroll
      for (int k = 0; k < VEC; ++k) acc = (c + k < lim) ? fmaf((float)a[k], (float)d[k], acc) : acc;
    });
    acc = group_reduce<GROUP>(acc, OpSum(), (float*)red, 0.0f);
    S* yr = reinterpret_cast<S*>(p.y) + row * cols;
    for_each([&](uint64_t c, const A (&a)[VEC], const A (&d)[VEC]) {
      A o[VEC];
#pragma unroll
      for (int k = 0; k < VEC; ++k) o[k] = (c + k < lim) ? (A)((float)a[k] * ((float)d[k] - acc)) : (A)0;
      write(yr, c, o);
    });
  }
  // ---------------------------------------------------------------------------------------
  else if constexpr (FAM == FAM_LAYERNORM_BWD) {
    // dx = (g - mean(g) - (x-mean) * sum(g*(x-mean)) / ((n-1) * (var+eps))) / sqrt(var+eps), g = dy*w
    const S* wp = reinterpret_cast<const S*>(p.w);
    const float n = (float)cols;
    float acc = 0.0f;
    for_each([&](uint64_t, const A (&a)[VEC], const A (&)[VEC]) {
#pragma unroll
      for (int k = 0; k < VEC; ++k) acc += (float)a[k];
    });
    const float mean = group_reduce<GROUP>(acc, OpSum(), (float*)red, 0.0f) / n;
    float sq = 0.0f, sg = 0.0f, sgd = 0.0f;
    for_each([&](uint64_t c, const A (&a)[VEC], const A (&d)[VEC]) {
      A wv[VEC];
      if (wp) {
        Raw pk;
        pk.load(wp + c); pk.decode(wv);
      }
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        const float dx = (float)a[k] - mean;
        const float g = wp ? (float)d[k] * wv[k] : (float)d[k];
        sq = fmaf(dx, dx, sq); sg += g; sgd = fmaf(g, dx, sgd);
      }
    });
    sq = group_reduce<GROUP>(sq, OpSum(), (float*)red, 0.0f);
    sg = group_reduce<GROUP>(sg, OpSum(), (float*)red, 0.0f);
    sgd = group_reduce<GROUP>(sgd, OpSum(), (float*)red, 0.0f);
    const float s2 = sq / (n - 1.0f) + const_cast_dtype<T>(p.eps);
    const float rs = 1.0f / sqrtf(s2);
    const float k1 = sg / n, k2 = sgd / ((n - 1.0f) * s2);
    S* yr = reinterpret_cast<S*>(p.y) + row * cols;
    for_each([&](uint64_t c, const A (&a)[VEC], const A (&d)[VEC]) {
      A wv[VEC];
      if (wp) {
        Raw pk;
        pk.load(wp + c); pk.decode(wv);
      }
      A o[VEC];
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        const float dx = (float)a[k] - mean;
        const float g = wp ? (float)d[k] * wv[k] : (float)d[k];
        if (p.op == ZYXB_RR_LAYERNORM_DYXHAT) o[k] = (A)((float)d[k] * (dx * rs));   // dy * xhat: summed over rows it is d(weight)
        else o[k] = (A)((g - k1 - dx * k2) * rs);
      }
      write(yr, c, o);
    });
  }
}

// ---- long rows staged through shared memory with bulk (TMA) copies -------------------------------------
// For rows of 16 KB .. 128 KB (softmax, ln_softmax, layernorm): a persistent CTA of 512 threads per SM walks its
// rows; while it reduces and stores row i from registers, one bulk copy (cp.async.bulk, completion on an mbarrier)
// is already bringing row i+1 into shared memory, so every SM keeps loads and stores in flight at the same time
// instead of alternating between them.  The row is read from HBM once and written once.
constexpr int STG_THREADS = 512;
constexpr uint64_t STG_WAIT_NS = 2000000000ull;

__device__ __forceinline__ uint32_t stg_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t stg_timer_ns() { uint64_t t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ uint32_t stg_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok;
}
// thread 0: arm the barrier with the row's byte count and start the bulk copy (in chunks of at most 32 KB)
__device__ __forceinline__ void stg_fetch_row(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy reads of the buffer are done; the async proxy may overwrite it
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
  for (uint32_t off = 0; off < bytes; off += 32768u) {
    const uint32_t n = min(32768u, bytes - off);
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst + off), "l"((const char*)src + off), "r"(n), "r"(bar) : "memory");
  }
}

template <typename T, int ITEMS, int FAM>
__global__ void __launch_bounds__(STG_THREADS, 1) row_staged_kernel(RowParams p, uint32_t* status) {
  using S = typename Elem<T>::store_t;
  constexpr int VEC = 16 / sizeof(S);
  extern __shared__ __align__(128) uint8_t stg_smem[];
  __shared__ float red[32];
  __shared__ __align__(8) uint64_t bar_storage;
  __shared__ int abort_flag;
  const uint32_t buf = stg_smem_u32(stg_smem), bar = stg_smem_u32(&bar_storage);
  const uint64_t cols = p.cols;
  const uint32_t row_bytes = (uint32_t)(cols * sizeof(S));
  const S* X = reinterpret_cast<const S*>(p.x);
  S* Y = reinterpret_cast<S*>(p.y);
  const bool rn = p.rn != 0;
  const int tid = threadIdx.x;
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(1) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    abort_flag = 0;
  }
  __syncthreads();
  uint64_t row = blockIdx.x;
  if (tid == 0 && row < p.rows) stg_fetch_row(buf, X + row * cols, row_bytes, bar);
  uint32_t parity = 0;
  const bool scaled = p.scale != 1.0f;
  const float cscale = const_cast_dtype<T>(p.scale);
  for (; row < p.rows; row += gridDim.x) {
    // wait (bounded) for this row to land in shared memory
    if (!stg_try_wait(bar, parity)) {
      const uint64_t t0 = stg_timer_ns();
      while (!stg_try_wait(bar, parity)) {
        if (stg_timer_ns() - t0 > STG_WAIT_NS) { abort_flag = 1; atomicOr(status, 8u); break; }
      }
    }
    __syncthreads();
    if (abort_flag) return;
    parity ^= 1;
    float v[ITEMS][VEC];
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      const uint64_t c = ((uint64_t)it * STG_THREADS + tid) * VEC;
      if (c < cols) {
        RawVec<T, VEC> pk;
        pk.load(reinterpret_cast<const S*>(stg_smem + c * sizeof(S)));
        pk.decode(v[it]);
      }
    }
    __syncthreads();                                   // every thread has its part of the row in registers
    const uint64_t next = row + gridDim.x;
    if (tid == 0 && next < p.rows) stg_fetch_row(buf, X + next * cols, row_bytes, bar);
    S* yr = Y + row * cols;
    auto for_each = [&](auto&& f) {
#pragma unroll
      for (int it = 0; it < ITEMS; ++it) {
        const uint64_t c = ((uint64_t)it * STG_THREADS + tid) * VEC;
        if (c < cols) f(c, v[it]);
      }
    };
    auto write = [&](uint64_t c, const float (&o)[VEC]) {
      RawVec<T, VEC> pk;
      pk.encode(o, rn);
      pk.store_stream(yr + c);
    };
    if constexpr (FAM == FAM_SOFTMAX) {
      // Scale and causal mask are applied once, in place (masked entries become -inf, whose exponential is 0); the three
      // passes that follow are free of compares.  Plain softmax then replaces each entry by its exponential (one SFU
      // operation per element); the log form keeps x.
      constexpr float LOG2E = 1.4426950408889634f;
      const uint32_t cols32 = (uint32_t)cols, lim32 = p.causal ? (uint32_t)min((uint64_t)(row % p.period) + 1, cols) : cols32;
      float mx = -CUDART_INF_F;
#pragma unroll
      for (int it = 0; it < ITEMS; ++it) {
        const uint32_t c = ((uint32_t)it * STG_THREADS + tid) * VEC;
        if (c < cols32) {
          if (scaled) {
#pragma unroll
            for (int k = 0; k < VEC; ++k) v[it][k] *= cscale;
          }
          if (c + VEC > lim32) {
#pragma unroll
            for (int k = 0; k < VEC; ++k) v[it][k] = c + k < lim32 ? v[it][k] : -CUDART_INF_F;
          }
#pragma unroll
          for (int k = 0; k < VEC; ++k) mx = fmaxf(v[it][k], mx);
        }
      }
      mx = group_reduce<STG_THREADS>(mx, OpMaxF(), red, -CUDART_INF_F);
      const float nmx = -mx * LOG2E;
      auto ex = [&](float a) -> float {                   // exp(a - mx)
        float r;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(fmaf(a, LOG2E, nmx)));
        return r;
      };
      float sum = 0.0f;
      if (p.op == ZYXB_RR_SOFTMAX) {
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
          const uint32_t c = ((uint32_t)it * STG_THREADS + tid) * VEC;
          if (c < cols32) {
#pragma unroll
            for (int k = 0; k < VEC; ++k) { v[it][k] = ex(v[it][k]); sum += v[it][k]; }
          }
        }
        sum = group_reduce<STG_THREADS>(sum, OpSum(), red, 0.0f);
        const float inv = 1.0f / sum;
        for_each([&](uint64_t c, const float (&e)[VEC]) {
          float o[VEC];
#pragma unroll
          for (int k = 0; k < VEC; ++k) o[k] = e[k] * inv;
          write(c, o);
        });
      } else {
        for_each([&](uint64_t, const float (&a)[VEC]) {
#pragma unroll
          for (int k = 0; k < VEC; ++k) sum += ex(a[k]);
        });
        sum = group_reduce<STG_THREADS>(sum, OpSum(), red, 0.0f);
        const float ls = logf(sum);
        for_each([&](uint64_t c, const float (&a)[VEC]) {
          float o[VEC];
#pragma unroll
          for (int k = 0; k < VEC; ++k) o[k] = (a[k] - mx) - ls;
          write(c, o);
        });
      }
    } else {   // layernorm, unbiased variance
      float acc = 0.0f;
      for_each([&](uint64_t, const float (&a)[VEC]) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc += a[k];
      });
      const float mean = group_reduce<STG_THREADS>(acc, OpSum(), red, 0.0f) / const_cast_dtype<T>((float)cols);
      float sq = 0.0f;
      for_each([&](uint64_t, const float (&a)[VEC]) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) { const float d = a[k] - mean; sq = fmaf(d, d, sq); }
      });
      sq = group_reduce<STG_THREADS>(sq, OpSum(), red, 0.0f);
      const float rstd = 1.0f / sqrtf(sq / const_cast_dtype<T>((float)((int64_t)cols - 1)) + const_cast_dtype<T>(p.eps));
      const S* wp = reinterpret_cast<const S*>(p.w);
      const S* bp = reinterpret_cast<const S*>(p.b);
      for_each([&](uint64_t c, const float (&a)[VEC]) {
        float o[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) o[k] = (a[k] - mean) * rstd;
        if (wp) {
          RawVec<T, VEC> pk; float wv[VEC];
          pk.load(wp + c); pk.decode(wv);
#pragma unroll
          for (int k = 0; k < VEC; ++k) o[k] *= wv[k];
        }
        if (bp) {
          RawVec<T, VEC> pk; float bv[VEC];
          pk.load(bp + c); pk.decode(bv);
#pragma unroll
          for (int k = 0; k < VEC; ++k) o[k] += bv[k];
        }
        write(c, o);
      });
    }
  }
}

// Takes the launch when the shape suits it; returns false otherwise.
template <typename T, int FAM>
static bool launch_row_staged(const RowParams& p, cudaStream_t s, int sm_count, uint32_t* status) {
  using S = typename Elem<T>::store_t;
  constexpr int V = 16 / sizeof(S);
  constexpr int ITEMS = 64 / V;                                   // 64 values per thread in registers
  const uint64_t row_bytes = p.cols * sizeof(S);
  if (row_bytes < 16384 || p.cols > (uint64_t)STG_THREADS * ITEMS * V || p.cols % V || p.rows < 2ull * sm_count) return false;
  if ((uintptr_t)p.x % 16 || (uintptr_t)p.y % 16 || (p.w && (uintptr_t)p.w % 16) || (p.b && (uintptr_t)p.b % 16)) return false;
  auto kern = row_staged_kernel<T, ITEMS, FAM>;
  static uint64_t configured = 0;
  if (ensure_dynamic_smem(kern, 128 * 1024, &configured) != cudaSuccess) { cudaGetLastError(); return false; }
  kern<<<(unsigned)std::min<uint64_t>(p.rows, (uint64_t)sm_count), STG_THREADS, (size_t)row_bytes, s>>>(p, status);
  return true;
}

// ---- long rows on thread-block cluster pairs: a cluster of two CTAs per row ---------------------------------
// (layernorm with or without weight and bias; rows of 16 .. 128 KB.)
// With weight and bias the staged kernel above would read 2 x row bytes of parameters from L2 for every row.  Here two
// CTAs (one thread-block cluster, two SMs) share each row: each keeps its half of weight and bias in shared memory for
// the whole launch (2 x 64 KB) next to a 64 KB stage for its half-rows, so parameters are read from L2 once per CTA.
// The halves combine their statistics through distributed shared memory once per row: each CTA computes the sum and
// the centred second moment of its half exactly (two passes over registers), writes the pair into its partner's
// shared memory (asynchronous stores that complete a barrier there), and both hold
//   mean = (s0 + s1) / n,    sum (x - mean)^2 = M0 + M1 + n/2 * ((mean0 - mean)^2 + (mean1 - mean)^2),
// which is algebraically the reference's two-pass variance (zyx-nn/src/layer_norm.rs:117-131).
// Softmax stays on the single-CTA staged kernel above: it has no parameters to keep resident and reaches the HBM peak there.
constexpr int LNC_ITEMS = 8;   // vectors per thread: 512 threads x 8 x 16 bytes = 64 KB per half-row

__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <typename T, int FAM>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(STG_THREADS, 1) row_cluster_kernel(RowParams p, uint32_t* status) {
  using S = typename Elem<T>::store_t;
  constexpr int VEC = 16 / sizeof(S);
  extern __shared__ __align__(128) uint8_t stg_smem[];          // [stage | weight half | bias half]
  __shared__ float red[32];
  __shared__ float xchg[2][2];                                  // [row parity][sum, second moment] written by the partner
  __shared__ __align__(8) uint64_t bar_storage[4];              // stage, parameters, exchange slot 0 / 1
  __shared__ int abort_flag;
  const int tid = threadIdx.x;
  const uint32_t half = cluster_ctarank();
  const uint64_t cols = p.cols, hc = cols / 2;                  // this CTA's columns: [half * hc, half * hc + hc)
  const uint32_t half_bytes = (uint32_t)(hc * sizeof(S));
  const uint32_t buf = stg_smem_u32(stg_smem), bar = stg_smem_u32(&bar_storage[0]), wbar = stg_smem_u32(&bar_storage[1]);
  const S* X = reinterpret_cast<const S*>(p.x) + half * hc;
  S* Y = reinterpret_cast<S*>(p.y) + half * hc;
  static_assert(FAM == FAM_LAYERNORM, "cluster pairs serve layernorm only");
  const bool affine = p.w != nullptr;                  // weight and bias come together (the launcher checks)
  const S* w_s = reinterpret_cast<const S*>(stg_smem + half_bytes);
  const S* b_s = reinterpret_cast<const S*>(stg_smem + 2 * (size_t)half_bytes);
  const bool rn = p.rn != 0;
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(1) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(wbar), "r"(1) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(stg_smem_u32(&bar_storage[2])), "r"(1) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(stg_smem_u32(&bar_storage[3])), "r"(1) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    abort_flag = 0;
  }
  __syncthreads();
  cluster_sync_all();                                  // the partner's barriers exist before anything is sent to them
  const uint64_t n_clusters = gridDim.x / 2;
  uint64_t row = blockIdx.x / 2;
  if (tid == 0 && affine) {
    // weight and bias halves: one expected byte count, two sets of copies
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(wbar), "r"(2 * half_bytes) : "memory");
    for (int which = 0; which < 2; ++which) {
      const char* src = reinterpret_cast<const char*>((which ? reinterpret_cast<const S*>(p.b) : reinterpret_cast<const S*>(p.w)) + half * hc);
      for (uint32_t off = 0; off < half_bytes; off += 32768u) {
        const uint32_t nb = min(32768u, half_bytes - off);
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(buf + (1 + which) * half_bytes + off), "l"(src + off), "r"(nb), "r"(wbar) : "memory");
      }
    }
  }
  if (tid == 0 && row < p.rows) stg_fetch_row(buf, X + row * cols, half_bytes, bar);
  // the partner's exchange slots and their barriers, as addresses in the cluster's shared window
  uint32_t peer_xchg, peer_xbar;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer_xchg) : "r"(stg_smem_u32(&xchg[0][0])), "r"(half ^ 1u));
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer_xbar) : "r"(stg_smem_u32(&bar_storage[2])), "r"(half ^ 1u));
  auto bounded_wait = [&](uint32_t b, uint32_t parity) {
    if (!stg_try_wait(b, parity)) {
      const uint64_t t0 = stg_timer_ns();
      while (!stg_try_wait(b, parity)) {
        if (stg_timer_ns() - t0 > STG_WAIT_NS) { abort_flag = 1; atomicOr(status, 8u); break; }
      }
    }
  };
  if (affine) bounded_wait(wbar, 0);                  // weight and bias arrive once
  uint32_t parity = 0, it_row = 0;
  const float n = const_cast_dtype<T>((float)cols), nm1 = const_cast_dtype<T>((float)((int64_t)cols - 1));
  const float n_half = (float)hc;
  // Both CTAs of a cluster walk the same rows; a CTA whose copy timed out keeps sending its (meaningless) pair with its
  // work skipped, so that its partner is never left waiting, and every wait is bounded anyway.
  for (; row < p.rows; row += n_clusters, ++it_row) {
    bounded_wait(bar, parity);
    __syncthreads();
    const bool dead = abort_flag != 0;
    parity ^= 1;
    float v[LNC_ITEMS][VEC];
#pragma unroll
    for (int it = 0; it < LNC_ITEMS; ++it) {
      const uint64_t c = ((uint64_t)it * STG_THREADS + tid) * VEC;
#pragma unroll
      for (int k = 0; k < VEC; ++k) v[it][k] = 0.0f;
      if (c < hc && !dead) {
        RawVec<T, VEC> pk;
        pk.load(reinterpret_cast<const S*>(stg_smem + c * sizeof(S)));
        pk.decode(v[it]);
      }
    }
    __syncthreads();                                   // the half-row is in registers: the stage may be refilled
    const uint64_t next = row + n_clusters;
    if (tid == 0 && next < p.rows && !dead) stg_fetch_row(buf, X + next * cols, half_bytes, bar);
    // this half's pair of statistics: (sum, centred second moment)
    float st0, st1;
    {
      float acc = 0.0f;
#pragma unroll
      for (int it = 0; it < LNC_ITEMS; ++it)
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc += v[it][k];   // columns past hc hold zeros
      st0 = group_reduce<STG_THREADS>(acc, OpSum(), red, 0.0f);
      const float mean_h = st0 / n_half;
      float sq = 0.0f;
#pragma unroll
      for (int it = 0; it < LNC_ITEMS; ++it) {
        const uint64_t c = ((uint64_t)it * STG_THREADS + tid) * VEC;
        if (c < hc) {
#pragma unroll
          for (int k = 0; k < VEC; ++k) { const float d = v[it][k] - mean_h; sq = fmaf(d, d, sq); }
        }
      }
      st1 = group_reduce<STG_THREADS>(sq, OpSum(), red, 0.0f);
    }
    // The pair travels as two asynchronous 4-byte stores that complete a barrier in the partner's shared memory: no
    // cluster-wide barrier or fence per row (a release fence here would wait for the previous row's output stores).
    // Slots alternate by row; a CTA can be at most one row ahead of its partner, because it needs the partner's pair
    // of row i to finish row i.
    const uint32_t slot = it_row & 1u, xbar = stg_smem_u32(&bar_storage[2 + slot]);
    if (tid == 0) {
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(xbar), "r"(8) : "memory");
      asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
                   ::"r"(peer_xchg + slot * 8u), "r"(__float_as_uint(st0)), "r"(peer_xbar + slot * 8u) : "memory");
      asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
                   ::"r"(peer_xchg + slot * 8u + 4u), "r"(__float_as_uint(st1)), "r"(peer_xbar + slot * 8u) : "memory");
    }
    bounded_wait(xbar, (it_row >> 1) & 1u);            // the partner's pair has landed in xchg[slot]
    const float o0 = reinterpret_cast<volatile float*>(&xchg[slot][0])[0], o1 = reinterpret_cast<volatile float*>(&xchg[slot][0])[1];
    // identical arithmetic in both CTAs: operands ordered by half, not by "mine / theirs"
    const float a0 = half == 0 ? st0 : o0, a1 = half == 0 ? o0 : st0;
    const float b0 = half == 0 ? st1 : o1, b1 = half == 0 ? o1 : st1;
    S* yr = Y + row * cols;
    {
      const float mean = (a0 + a1) / n;
      const float d0 = a0 / n_half - mean, d1 = a1 / n_half - mean;
      const float m2 = (b0 + b1) + n_half * (d0 * d0 + d1 * d1);
      const float rstd = 1.0f / sqrtf(m2 / nm1 + const_cast_dtype<T>(p.eps));
      if (!dead) {
#pragma unroll
        for (int it = 0; it < LNC_ITEMS; ++it) {
          const uint64_t c = ((uint64_t)it * STG_THREADS + tid) * VEC;
          if (c < hc) {
            RawVec<T, VEC> po;
            float o[VEC];
#pragma unroll
            for (int k = 0; k < VEC; ++k) o[k] = (v[it][k] - mean) * rstd;
            if (affine) {
              RawVec<T, VEC> pw, pb;
              float wv[VEC], bv[VEC];
              pw.load(w_s + c); pw.decode(wv);
              pb.load(b_s + c); pb.decode(bv);
#pragma unroll
              for (int k = 0; k < VEC; ++k) o[k] = o[k] * wv[k] + bv[k];
            }
            po.encode(o, rn);
            po.store_stream(yr + c);
          }
        }
      }
    }
  }
  cluster_sync_all();                                  // no CTA leaves while its partner might still address its shared memory
}

// Takes layernorm launches whose rows split into two halves of 8 .. 64 KB; returns false otherwise.
template <typename T, int FAM>
static bool launch_row_cluster(const RowParams& p, cudaStream_t s, int sm_count, uint32_t* status) {
  using S = typename Elem<T>::store_t;
  constexpr int V = 16 / sizeof(S);
  static const bool off = getenv("ZYXB_NO_ROW_CLUSTER") != nullptr;
  if (off || sm_count < 2 || (p.w == nullptr) != (p.b == nullptr)) return false;
  const uint64_t hc = p.cols / 2, half_bytes = hc * sizeof(S);
  if (p.cols % (2 * V) || half_bytes < 8192 || half_bytes > 65536 || hc > (uint64_t)STG_THREADS * LNC_ITEMS * V) return false;
  if (p.rows < (uint64_t)sm_count) return false;      // at least two rows per cluster
  if ((uintptr_t)p.x % 16 || (uintptr_t)p.y % 16 || (p.w && ((uintptr_t)p.w % 16 || (uintptr_t)p.b % 16))) return false;
  auto kern = row_cluster_kernel<T, FAM>;
  static uint64_t configured = 0;
  if (ensure_dynamic_smem(kern, 3 * 65536, &configured) != cudaSuccess) { cudaGetLastError(); return false; }
  const unsigned clusters = (unsigned)std::min<uint64_t>(p.rows, (uint64_t)(sm_count / 2));
  kern<<<2 * clusters, STG_THREADS, (size_t)((p.w ? 3 : 1) * half_bytes), s>>>(p, status);
  return true;
}

// ---- host-side geometry selection -----------------------------------------------------------
template <typename T, int VEC, int ITEMS, int GROUP, int FAM>
static void launch_row_geom(const RowParams& p, cudaStream_t s) {
  if constexpr (GROUP == 32) {
    const unsigned rows_per_cta = 4;
    row_kernel<T, VEC, ITEMS, GROUP, FAM><<<(unsigned)((p.rows + rows_per_cta - 1) / rows_per_cta), 128, 0, s>>>(p);
  } else {
    row_kernel<T, VEC, ITEMS, GROUP, FAM><<<(unsigned)p.rows, GROUP, 0, s>>>(p);
  }
}

// Pick the smallest geometry whose register budget holds the row; fall back to streaming.
template <typename T, int VEC, int FAM>
static void launch_row_vec(const RowParams& p, cudaStream_t s) {
  constexpr bool TWO_IN = (FAM == FAM_SOFTMAX_BWD || FAM == FAM_LAYERNORM_BWD);
  const uint64_t c = p.cols;
  // a warp per row up to 8 vectors per thread: measured on [262144, 2048] bf16 rows a CTA of 256 threads per row
  // (one vector per thread, two barriers per row) is 1.7x slower for softmax than a warp holding the whole row
  if (c <= 32ull * 2 * VEC) launch_row_geom<T, VEC, 2, 32, FAM>(p, s);
  else if (c <= 32ull * 8 * VEC) launch_row_geom<T, VEC, 8, 32, FAM>(p, s);
  else if (c <= 256ull * 4 * VEC) launch_row_geom<T, VEC, 4, 256, FAM>(p, s);
  else if (c <= 1024ull * 4 * VEC) launch_row_geom<T, VEC, 4, 1024, FAM>(p, s);
  else if (!TWO_IN && VEC > 1 && c <= 1024ull * 8 * VEC) launch_row_geom<T, VEC, (TWO_IN || VEC == 1) ? 4 : 8, 1024, FAM>(p, s);
  else launch_row_geom<T, VEC, 0, 1024, FAM>(p, s);
}

template <typename T, int FAM>
static void launch_row_family(const RowParams& p, cudaStream_t s) {
  using S = typename Elem<T>::store_t;
  constexpr int V = 16 / sizeof(S);
  // 128-bit accesses need every row to start on a 16-byte boundary
  const bool vec_ok = (p.cols % V == 0) && ((uintptr_t)p.x % 16 == 0) && ((uintptr_t)p.y % 16 == 0) &&
                      (p.x2 == nullptr || FAM == FAM_CE || (uintptr_t)p.x2 % 16 == 0) &&
                      (p.w == nullptr || (uintptr_t)p.w % 16 == 0) && (p.b == nullptr || (uintptr_t)p.b % 16 == 0);
  if constexpr ((FAM == FAM_SOFTMAX || FAM == FAM_LAYERNORM) && !std::is_same_v<T, int32_t>) {
    // layernorm with weight / bias stays on the register kernel: its per-element weight and bias loads (L2 latency,
    // 16 dependent iterations per thread at 512 threads) cost more than the staging gains (measured 0.70 vs 0.79 of peak)
    const bool affine = FAM == FAM_LAYERNORM && (p.w || p.b);
    // Measured at f32 [8192, 32768]: layernorm 0.99 of the HBM peak on cluster pairs (0.76-0.79 without them); softmax
    // 0.996 on the single-CTA stage below against 0.90 on pairs (twice the row iterations per CTA, nothing to keep resident).
    if constexpr (FAM == FAM_LAYERNORM) {
      if (vec_ok && p.sm_count > 0 && p.status && launch_row_cluster<T, FAM>(p, s, p.sm_count, p.status)) return;
    }
    if (vec_ok && !affine && p.sm_count > 0 && p.status && launch_row_staged<T, FAM>(p, s, p.sm_count, p.status)) return;
  }
  if (vec_ok) launch_row_vec<T, V, FAM>(p, s);
  else launch_row_vec<T, 1, FAM>(p, s);
}

// One translation unit per dtype instantiates this.
template <typename T>
static void launch_row_dtype(int fam, const RowParams& p, cudaStream_t s) {
  switch (fam) {
    case FAM_REDUCE: launch_row_family<T, FAM_REDUCE>(p, s); break;
    case FAM_SOFTMAX: launch_row_family<T, FAM_SOFTMAX>(p, s); break;
    case FAM_LAYERNORM: launch_row_family<T, FAM_LAYERNORM>(p, s); break;
    case FAM_SOFTMAX_BWD: launch_row_family<T, FAM_SOFTMAX_BWD>(p, s); break;
    case FAM_LAYERNORM_BWD: launch_row_family<T, FAM_LAYERNORM_BWD>(p, s); break;
    default: break;
  }
}

void launch_row_f32(int fam, const RowParams& p, cudaStream_t s);
void launch_row_bf16(int fam, const RowParams& p, cudaStream_t s);
void launch_row_f16(int fam, const RowParams& p, cudaStream_t s);
void launch_row_i32(const RowParams& p, cudaStream_t s);

}  // namespace zyxb
