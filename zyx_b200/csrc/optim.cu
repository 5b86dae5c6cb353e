// Fused optimizer update: one pass over every parameter tensor of a model per launch
// (p, g and the state are each read once and written once), instead of the 6-12 tensor
// expressions per parameter the reference builds.  The arithmetic is the reference's:
//   SGD::update    zyx-optim/src/sgd.rs:45-84
//   Adam::update   zyx-optim/src/adam.rs:51-98
//   AdamW::update  zyx-optim/src/adamw.rs:51-97   (p - mh / ((sqrt(vh) + eps) * lr), then p * (1 - lr*wd))
// Hyper-parameters enter as rank-0 scalars and are cast to the tensor dtype first
// (zyx/src/tensor/mod.rs:3033-3113); state tensors are stored in the tensor dtype and the
// stored (rounded) value is what the rest of the step uses.
#include <algorithm>
#include <cmath>
#include <type_traits>

#include "common.cuh"
#include "internal.h"

namespace zyxb {

constexpr int OPT_MAX_TENSORS = 32;   // tensors per launch; larger models take several launches
constexpr int OPT_THREADS = 256;
constexpr int OPT_UNROLL = 2;         // packs per thread per chunk

struct OptTable {
  void* p[OPT_MAX_TENSORS];
  const void* g[OPT_MAX_TENSORS];
  void* m[OPT_MAX_TENSORS];
  void* v[OPT_MAX_TENSORS];
  uint64_t numel[OPT_MAX_TENSORS];
  uint32_t chunk_start[OPT_MAX_TENSORS + 1];   // prefix sum of chunks per tensor
  int n;
};

struct OptHyper {
  float lr, wd, momentum, one_minus_damp, beta1, beta2, one_minus_b1, one_minus_b2, bc1, bc2, eps, decay, grad_scale;
  float rbc1, rbc2;   // 1 / bc1, 1 / bc2 of the dtype-cast bias corrections (filled in on the device)
  int nesterov, maximize, first, mode;   // mode: 0 Adam, 1 AdamW as the reference writes it, 2 textbook AdamW
  int rn;
};

// f32 tensors use IEEE division and square root (1e-5 parity); 16-bit tensors, whose results are
// cut to 8 or 11 significant bits anyway, use the SFU forms (a few ulp of f32) so that the kernel
// stays memory-bound.
template <typename T> __device__ __forceinline__ float opt_div(float a, float b) { return __fdividef(a, b); }
template <> __device__ __forceinline__ float opt_div<float>(float a, float b) { return a / b; }
__device__ __forceinline__ float opt_rcp(float a) { float r; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a)); return r; }
template <typename T> __device__ __forceinline__ float opt_sqrt(float a) { float r; asm("sqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(a)); return r; }
template <> __device__ __forceinline__ float opt_sqrt<float>(float a) { return sqrtf(a); }

template <typename T, int ALGO>
__device__ __forceinline__ void opt_update(float& pv, float gv, float& mv, float& vv, const OptHyper& h, bool rn) {
  auto round_state = [&](float x) { return (float)Elem<T>::load(Elem<T>::store(x, rn)); };
  if (h.grad_scale != 1.0f) gv *= h.grad_scale;
  if constexpr (ALGO == ZYXB_OPT_SGD) {
    if (h.wd != 0.0f) gv = gv + pv * h.wd;
    if (h.momentum != 0.0f) {
      float bv = h.first ? gv : mv * h.momentum + gv * h.one_minus_damp;
      bv = round_state(bv); mv = bv;
      gv = h.nesterov ? gv + bv * h.momentum : bv;
    }
    pv = h.maximize ? pv + gv * h.lr : pv - gv * h.lr;
  } else {
    if (h.mode == 0 && h.wd != 0.0f) gv = gv + pv * h.wd;
    float nm = h.first ? gv * h.one_minus_b1 : mv * h.beta1 + gv * h.one_minus_b1;
    float nv = h.first ? gv * gv * h.one_minus_b2 : vv * h.beta2 + gv * gv * h.one_minus_b2;
    nm = round_state(nm); nv = round_state(nv);
    mv = nm; vv = nv;
    float mh, vh, np;
    if constexpr (std::is_same_v<T, float>) {
      mh = nm / h.bc1; vh = nv / h.bc2;
      if (h.mode == 1) np = pv - mh / ((sqrtf(vh) + h.eps) * h.lr);
      else np = pv - h.lr * mh / (sqrtf(vh) + h.eps);
    } else {
      // 16-bit tensors: reciprocals of the bias corrections are formed once per thread, the remaining division is
      // one SFU reciprocal; a few ulp of f32, far inside the 8 / 11 significant bits the result keeps
      mh = nm * h.rbc1; vh = nv * h.rbc2;
      if (h.mode == 1) np = pv - mh * opt_rcp((opt_sqrt<T>(vh) + h.eps) * h.lr);
      else np = pv - h.lr * mh * opt_rcp(opt_sqrt<T>(vh) + h.eps);
    }
    if (h.mode != 0 && h.wd != 0.0f) np = np * h.decay;
    pv = np;
  }
}

template <typename T, int VEC, int ALGO>
__global__ void __launch_bounds__(OPT_THREADS) optim_kernel(OptTable tab, OptHyper hy) {
  using S = typename Elem<T>::store_t;
  // which tensor does this CTA's chunk belong to
  int t = 0;
  while (t + 1 < tab.n && blockIdx.x >= tab.chunk_start[t + 1]) ++t;
  const uint64_t chunk = blockIdx.x - tab.chunk_start[t];
  const uint64_t numel = tab.numel[t];
  S* p = reinterpret_cast<S*>(tab.p[t]);
  const S* g = reinterpret_cast<const S*>(tab.g[t]);
  S* m = reinterpret_cast<S*>(tab.m[t]);
  S* v = reinterpret_cast<S*>(tab.v[t]);
  const bool rn = hy.rn != 0;
  const bool use_m = (ALGO != ZYXB_OPT_SGD) || (hy.momentum != 0.0f);
  // hyper-parameters as scalars of the tensor dtype
  OptHyper h = hy;
  h.lr = const_cast_dtype<T>(hy.lr); h.wd = const_cast_dtype<T>(hy.wd); h.momentum = const_cast_dtype<T>(hy.momentum);
  h.one_minus_damp = const_cast_dtype<T>(hy.one_minus_damp); h.beta1 = const_cast_dtype<T>(hy.beta1);
  h.beta2 = const_cast_dtype<T>(hy.beta2); h.one_minus_b1 = const_cast_dtype<T>(hy.one_minus_b1);
  h.one_minus_b2 = const_cast_dtype<T>(hy.one_minus_b2); h.bc1 = const_cast_dtype<T>(hy.bc1); h.bc2 = const_cast_dtype<T>(hy.bc2);
  h.eps = const_cast_dtype<T>(hy.eps); h.decay = const_cast_dtype<T>(hy.decay);
  h.rbc1 = 1.0f / h.bc1; h.rbc2 = 1.0f / h.bc2;
  // keep the "is it zero" tests on the caller's values, as the reference tests its f32 fields
  if (hy.wd == 0.0f) h.wd = 0.0f;
  if (hy.momentum == 0.0f) h.momentum = 0.0f;

  const uint64_t base = chunk * (uint64_t)(OPT_THREADS * OPT_UNROLL * VEC);
  const bool read_state = use_m && !hy.first;
  // all loads of the chunk are issued before any store: p, m and v are read and written through
  // pointers the compiler must assume may alias, so a load placed after a store would wait for it
  RawVec<T, VEC> pp[OPT_UNROLL], pg[OPT_UNROLL], pm[OPT_UNROLL], pv[OPT_UNROLL];
  bool whole[OPT_UNROLL];
#pragma unroll
  for (int u = 0; u < OPT_UNROLL; ++u) {
    const uint64_t i = base + ((uint64_t)u * OPT_THREADS + threadIdx.x) * VEC;
    whole[u] = i + VEC <= numel;
    if (whole[u]) {
      pp[u].load(p + i);
      pg[u].load_stream(g + i);
      if (read_state) {
        pm[u].load(m + i);
        if constexpr (ALGO != ZYXB_OPT_SGD) pv[u].load(v + i);
      }
    }
  }
#pragma unroll
  for (int u = 0; u < OPT_UNROLL; ++u) {
    const uint64_t i = base + ((uint64_t)u * OPT_THREADS + threadIdx.x) * VEC;
    if (whole[u]) {
      float fp[VEC], fg[VEC], fm[VEC], fv[VEC];
      pp[u].decode(fp);
      pg[u].decode(fg);
#pragma unroll
      for (int k = 0; k < VEC; ++k) { fm[k] = 0.0f; fv[k] = 0.0f; }
      if (read_state) {
        pm[u].decode(fm);
        if constexpr (ALGO != ZYXB_OPT_SGD) pv[u].decode(fv);
      }
#pragma unroll
      for (int k = 0; k < VEC; ++k) opt_update<T, ALGO>(fp[k], fg[k], fm[k], fv[k], h, rn);
      pp[u].encode(fp, rn);
      pp[u].store(p + i);
      if (use_m) {
        pm[u].encode(fm, rn);
        pm[u].store(m + i);
        if constexpr (ALGO != ZYXB_OPT_SGD) { pv[u].encode(fv, rn); pv[u].store(v + i); }
      }
    } else {
      // ragged tail of a tensor whose length is not a multiple of VEC
      for (uint64_t j = i; j < numel && j < i + VEC; ++j) {
        float fp = (float)Elem<T>::load(p[j]), fg = (float)Elem<T>::load(g[j]);
        float fm = read_state ? (float)Elem<T>::load(m[j]) : 0.0f;
        float fv = (read_state && ALGO != ZYXB_OPT_SGD) ? (float)Elem<T>::load(v[j]) : 0.0f;
        opt_update<T, ALGO>(fp, fg, fm, fv, h, rn);
        p[j] = Elem<T>::store(fp, rn);
        if (use_m) { m[j] = Elem<T>::store(fm, rn); if constexpr (ALGO != ZYXB_OPT_SGD) v[j] = Elem<T>::store(fv, rn); }
      }
    }
  }
}

template <typename T, int ALGO>
static void launch_opt(const OptTable& tab, const OptHyper& h, bool vec_ok, unsigned grid, cudaStream_t s) {
  using S = typename Elem<T>::store_t;
  constexpr int V = 16 / sizeof(S);
  if (vec_ok) optim_kernel<T, V, ALGO><<<grid, OPT_THREADS, 0, s>>>(tab, h);
  else optim_kernel<T, 1, ALGO><<<grid, OPT_THREADS, 0, s>>>(tab, h);
}

int validate_optim(const zyxb_optim_desc& d, std::string& err) {
  if (d.algo < ZYXB_OPT_SGD || d.algo > ZYXB_OPT_ADAMW) { err = "optim: unknown algorithm"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.dtype != ZYXB_F32 && d.dtype != ZYXB_BF16 && d.dtype != ZYXB_F16) { err = "optim: dtype must be f32, bf16 or f16"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.n_tensors <= 0 || d.numel == nullptr) { err = "optim: needs at least one tensor and its numel array"; return ZYXB_ERR_KERNEL_COMPILATION; }
  for (int i = 0; i < d.n_tensors; ++i)
    if (d.numel[i] == 0) { err = "optim: empty tensor"; return ZYXB_ERR_KERNEL_COMPILATION; }
  return ZYXB_OK;
}

int launch_optim(const zyxb_optim_desc& d, const uint64_t* numel, uint64_t step, void* const* args, const uint64_t* arg_bytes,
                 int n_args, const LaunchCtx& lc, std::string& err) {
  const int n = d.n_tensors;
  const bool sgd = d.algo == ZYXB_OPT_SGD;
  const bool sgd_mom = sgd && d.momentum != 0.0f;
  const int groups = sgd ? (sgd_mom ? 3 : 2) : 4;
  ZYXB_CHECK_ARG(n_args == groups * n, "optim: expected args p[0..n), g[0..n) [, state...]");
  const uint64_t es = dtype_size(d.dtype);
  for (int gidx = 0; gidx < groups; ++gidx)
    for (int i = 0; i < n; ++i) ZYXB_CHECK_ARG(arg_bytes[gidx * n + i] >= numel[i] * es, "optim: buffer smaller than its tensor");

  OptHyper h{};
  h.lr = d.lr; h.wd = d.weight_decay; h.momentum = d.momentum; h.one_minus_damp = 1.0f - d.dampening;
  h.beta1 = d.beta1; h.beta2 = d.beta2; h.one_minus_b1 = 1.0f - d.beta1; h.one_minus_b2 = 1.0f - d.beta2;
  h.bc1 = 1.0f - powf(d.beta1, (float)step); h.bc2 = 1.0f - powf(d.beta2, (float)step);
  h.eps = d.eps; h.decay = 1.0f - d.lr * d.weight_decay; h.grad_scale = d.grad_scale == 0.0f ? 1.0f : d.grad_scale;
  h.nesterov = d.nesterov; h.maximize = d.maximize; h.first = step == 1 ? 1 : 0;
  h.mode = d.algo == ZYXB_OPT_ADAM ? 0 : (d.standard ? 2 : 1);
  h.rn = lc.round_nearest ? 1 : 0;

  const uint64_t vec = 16 / es;
  int launches = 0;
  for (int t0 = 0; t0 < n; t0 += OPT_MAX_TENSORS) {
    OptTable tab{};
    tab.n = std::min(OPT_MAX_TENSORS, n - t0);
    bool vec_ok = true;
    uint64_t chunks = 0;
    for (int i = 0; i < tab.n; ++i) {
      const int t = t0 + i;
      tab.p[i] = args[t]; tab.g[i] = args[n + t];
      tab.m[i] = groups > 2 ? args[2 * n + t] : nullptr;
      tab.v[i] = groups > 3 ? args[3 * n + t] : nullptr;
      tab.numel[i] = numel[t];
      for (const void* q : {(const void*)tab.p[i], tab.g[i], (const void*)tab.m[i], (const void*)tab.v[i]})
        if (q && (uintptr_t)q % 16 != 0) vec_ok = false;
    }
    const uint64_t per_chunk = (uint64_t)OPT_THREADS * OPT_UNROLL * (vec_ok ? vec : 1);
    for (int i = 0; i < tab.n; ++i) {
      tab.chunk_start[i] = (uint32_t)chunks;
      chunks += (tab.numel[i] + per_chunk - 1) / per_chunk;
      ZYXB_CHECK_ARG(chunks < 0x7fffffffull, "optim: too many elements for one launch");
    }
    tab.chunk_start[tab.n] = (uint32_t)chunks;
    const unsigned grid = (unsigned)chunks;
#define ZYXB_OPT_DISPATCH(T)                                                                  \
  switch (d.algo) {                                                                           \
    case ZYXB_OPT_SGD: launch_opt<T, ZYXB_OPT_SGD>(tab, h, vec_ok, grid, lc.stream); break;   \
    default: launch_opt<T, ZYXB_OPT_ADAM>(tab, h, vec_ok, grid, lc.stream); break;            \
  }
    switch (d.dtype) {
      case ZYXB_F32: ZYXB_OPT_DISPATCH(float) break;
      case ZYXB_BF16: ZYXB_OPT_DISPATCH(bf16_t) break;
      default: ZYXB_OPT_DISPATCH(f16_t) break;
    }
#undef ZYXB_OPT_DISPATCH
    ++launches;
  }
  return check_launch(lc, err, "optim", launches);
}

}  // namespace zyxb
