// Host-side dispatch of the row kernels, plus the reductions that cross rows:
// column sums (bias gradients), the mean of per-sample losses and the MSE loss.
#include <stdlib.h>

#include <algorithm>

#include "rowreduce_impl.cuh"

namespace zyxb {

void launch_row_i32(const RowParams& p, cudaStream_t s) { launch_row_family<int32_t, FAM_REDUCE>(p, s); }

// ---- mean over rows of the per-sample losses (cross_entropy ReduceOp::Mean,
//      zyx/src/tensor/mod.rs:1650) --------------------------------------------------------------
__global__ void __launch_bounds__(256) mean_of_rows_kernel(const float* per, float* out, uint64_t rows) {
  __shared__ float red[32];
  float acc = 0.0f;
  for (uint64_t r = threadIdx.x; r < rows; r += 256) acc += per[r];
  acc = group_reduce<256>(acc, OpSum(), red, 0.0f);
  if (threadIdx.x == 0) out[0] = acc / (float)rows;
}

// ---- column sums: y[j] = sum_r x[r, j] -----------------------------------------------------
// Stage 1: a CTA of 8 warps owns a strip of 32*VEC columns and one slice of the rows; each warp reads whole
// 32*VEC-column segments of its rows (one coalesced 512-byte access per row per warp, four rows in flight),
// the eight warps fold through shared memory.  Partials go to scratch as f32 [splits, cols].
// Stage 2 folds the (few) splits in order and stores in the tensor dtype.
constexpr int COLSUM_WARPS = 8;
template <typename T, int VEC>
__global__ void __launch_bounds__(32 * COLSUM_WARPS) colsum_partial_kernel(const typename Elem<T>::store_t* x, float* partial, uint64_t rows,
                                                                           uint64_t cols, uint64_t rows_per_split) {
  using S = typename Elem<T>::store_t;
  __shared__ float fold[COLSUM_WARPS][32 * VEC + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint64_t c = ((uint64_t)blockIdx.x * 32 + lane) * VEC;
  const bool live = c < cols;
  const uint64_t r0 = (uint64_t)blockIdx.y * rows_per_split;
  const uint64_t r1 = min(r0 + rows_per_split, rows);
  float acc[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) acc[k] = 0.0f;
  if (live) {
    uint64_t r = r0 + warp;
    for (; r + 3 * COLSUM_WARPS < r1; r += 4 * COLSUM_WARPS) {   // four independent loads in flight per thread
      RawVec<T, VEC> pk[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) pk[u].load_stream(x + (r + u * COLSUM_WARPS) * cols + c);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        typename Elem<T>::acc_t a[VEC];
        pk[u].decode(a);
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc[k] += (float)a[k];
      }
    }
    for (; r < r1; r += COLSUM_WARPS) {
      RawVec<T, VEC> pk;
      pk.load_stream(x + r * cols + c);
      typename Elem<T>::acc_t a[VEC];
      pk.decode(a);
#pragma unroll
      for (int k = 0; k < VEC; ++k) acc[k] += (float)a[k];
    }
  }
#pragma unroll
  for (int k = 0; k < VEC; ++k) fold[warp][lane * VEC + k] = acc[k];
  __syncthreads();
  for (int i = threadIdx.x; i < 32 * VEC; i += 32 * COLSUM_WARPS) {
    const uint64_t cc = (uint64_t)blockIdx.x * 32 * VEC + i;
    if (cc < cols) {
      float t = 0.0f;
#pragma unroll
      for (int w = 0; w < COLSUM_WARPS; ++w) t += fold[w][i];
      partial[(uint64_t)blockIdx.y * cols + cc] = t;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) colsum_final_kernel(const float* partial, typename Elem<T>::store_t* y, uint64_t cols,
                                                           uint32_t splits, int rn) {
  const uint64_t c = (uint64_t)blockIdx.x * 256 + threadIdx.x;
  if (c >= cols) return;
  float acc = 0.0f;
  for (uint32_t s = 0; s < splits; ++s) acc += partial[(uint64_t)s * cols + c];
  y[c] = Elem<T>::store(acc, rn != 0);
}

template <typename T>
static int launch_colsum(const void* x, void* y, uint64_t rows, uint64_t cols, const LaunchCtx& lc, std::string& err) {
  using S = typename Elem<T>::store_t;
  constexpr int V = 16 / sizeof(S);
  const bool vec_ok = cols % V == 0 && (uintptr_t)x % 16 == 0;
  const uint64_t per_cta = 32ull * (vec_ok ? V : 1);
  const uint64_t col_blocks = (cols + per_cta - 1) / per_cta;
  uint64_t splits = (4ull * lc.sm_count + col_blocks - 1) / col_blocks;
  splits = std::max<uint64_t>(1, std::min<uint64_t>({splits, (rows + 31) / 32, 64ull, lc.scratch_bytes / (cols * sizeof(float))}));
  ZYXB_CHECK_ARG(cols * sizeof(float) <= lc.scratch_bytes, "colsum: cols too large for the scratch buffer");
  ZYXB_CHECK_ARG(col_blocks <= 0x7fffffffull, "colsum: too many columns");
  const uint64_t rps = (rows + splits - 1) / splits;
  splits = (rows + rps - 1) / rps;
  dim3 grid((unsigned)col_blocks, (unsigned)splits);
  float* partial = reinterpret_cast<float*>(lc.scratch);
  if (vec_ok) colsum_partial_kernel<T, V><<<grid, 32 * COLSUM_WARPS, 0, lc.stream>>>((const S*)x, partial, rows, cols, rps);
  else colsum_partial_kernel<T, 1><<<grid, 32 * COLSUM_WARPS, 0, lc.stream>>>((const S*)x, partial, rows, cols, rps);
  colsum_final_kernel<T><<<(unsigned)((cols + 255) / 256), 256, 0, lc.stream>>>(partial, (S*)y, cols, (uint32_t)splits, lc.round_nearest);
  return check_launch(lc, err, "colsum", 2);
}

// ---- column sums without any allocation ------------------------------------------------------------
// Same two-stage kernels as launch_colsum, but the f32 partials live in a fixed array that is part of the
// loaded module, so the call path never reaches an allocator.  The array is shared by every call on the
// device and keeps whatever the previous call left in it; stage 1 overwrites every partial that stage 2
// reads, so nothing needs clearing, but two calls that overlap on the GPU (different streams or threads)
// would write the same partials and race.
constexpr uint64_t COLSUM_STATIC_FLOATS = 1ull << 20;      // 4 MiB of device memory per GPU, held until the process exits
static __device__ __align__(256) float g_colsum_static[COLSUM_STATIC_FLOATS];
constexpr int COLSUM_STATIC_MAX_DEVICES = 64;
static float* g_colsum_static_ptr[COLSUM_STATIC_MAX_DEVICES];   // device address of the array, per CUDA device

uint64_t colsum_static_capacity() { return COLSUM_STATIC_FLOATS; }
// whether the array's address on this CUDA device has been looked up already (the look-up cannot be part of a stream capture)
bool colsum_static_ready(int cuda_device) {
  return cuda_device >= 0 && cuda_device < COLSUM_STATIC_MAX_DEVICES && g_colsum_static_ptr[cuda_device] != nullptr;
}

// In host code the array's name is only a handle for the runtime, not a device address: the address is
// looked up once per device (with that device current) and cached.
static int colsum_static_address(int cuda_device, float** out, std::string& err) {
  if (cuda_device < 0 || cuda_device >= COLSUM_STATIC_MAX_DEVICES) { err = "colsum_static: device index out of range"; return ZYXB_ERR_KERNEL_LAUNCH; }
  if (!g_colsum_static_ptr[cuda_device]) {
    float* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_colsum_static);
    if (e != cudaSuccess || !ptr) {
      err = std::string("colsum_static: cudaGetSymbolAddress: ") + cudaGetErrorString(e);
      return ZYXB_ERR_KERNEL_LAUNCH;
    }
    g_colsum_static_ptr[cuda_device] = ptr;
  }
  *out = g_colsum_static_ptr[cuda_device];
  return ZYXB_OK;
}

template <typename T>
static int launch_colsum_static_t(const void* x, void* y, uint64_t rows, uint64_t cols, float* partial, const LaunchCtx& lc,
                                  std::string& err) {
  using S = typename Elem<T>::store_t;
  constexpr int V = 16 / sizeof(S);
  const bool vec_ok = cols % V == 0 && (uintptr_t)x % 16 == 0;
  const uint64_t per_cta = 32ull * (vec_ok ? V : 1);
  const uint64_t col_blocks = (cols + per_cta - 1) / per_cta;
  uint64_t splits = (4ull * lc.sm_count + col_blocks - 1) / col_blocks;
  splits = std::max<uint64_t>(1, std::min<uint64_t>({splits, (rows + 31) / 32, 64ull, COLSUM_STATIC_FLOATS / cols}));
  const uint64_t rps = (rows + splits - 1) / splits;
  splits = (rows + rps - 1) / rps;
  dim3 grid((unsigned)col_blocks, (unsigned)splits);
  if (vec_ok) colsum_partial_kernel<T, V><<<grid, 32 * COLSUM_WARPS, 0, lc.stream>>>((const S*)x, partial, rows, cols, rps);
  else colsum_partial_kernel<T, 1><<<grid, 32 * COLSUM_WARPS, 0, lc.stream>>>((const S*)x, partial, rows, cols, rps);
  colsum_final_kernel<T><<<(unsigned)((cols + 255) / 256), 256, 0, lc.stream>>>(partial, (S*)y, cols, (uint32_t)splits, lc.round_nearest);
  return check_launch(lc, err, "colsum_static", 2);
}

int launch_colsum_static(int dtype, const void* x, void* y, uint64_t rows, uint64_t cols, const LaunchCtx& lc, std::string& err) {
  if (rows == 0 || cols == 0) { err = "colsum_static: rows and cols must be positive"; return ZYXB_ERR_INCORRECT_KERNEL_ARG; }
  if (cols > COLSUM_STATIC_FLOATS) {
    err = "colsum_static: " + std::to_string(cols) + " columns exceed the fixed scratch of " + std::to_string(COLSUM_STATIC_FLOATS) +
          " floats; use a ZYXB_RR_COLSUM program instead";
    return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  }
  if ((cols + 31) / 32 > 0x7fffffffull) { err = "colsum_static: too many columns"; return ZYXB_ERR_INCORRECT_KERNEL_ARG; }
  float* partial = nullptr;
  int st = colsum_static_address(lc.device, &partial, err);
  if (st) return st;
  switch (dtype) {
    case ZYXB_F32: return launch_colsum_static_t<float>(x, y, rows, cols, partial, lc, err);
    case ZYXB_BF16: return launch_colsum_static_t<bf16_t>(x, y, rows, cols, partial, lc, err);
    case ZYXB_F16: return launch_colsum_static_t<f16_t>(x, y, rows, cols, partial, lc, err);
    default: err = "colsum_static: dtype must be f32, bf16 or f16"; return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  }
}

// ---- MSE loss: mean((y - t)^2) over every element, f32 result ---------------------------------
template <typename T, int VEC>
__global__ void __launch_bounds__(256) mse_partial_kernel(const typename Elem<T>::store_t* y, const typename Elem<T>::store_t* t,
                                                          float* partial, uint64_t n_vec) {
  using S = typename Elem<T>::store_t;
  __shared__ float red[32];
  float acc = 0.0f;
  for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < n_vec; i += (uint64_t)gridDim.x * 256) {
    RawVec<T, VEC> a, b;
    a.load_stream(y + i * VEC);
    b.load_stream(t + i * VEC);
    typename Elem<T>::acc_t fa[VEC], fb[VEC];
    a.decode(fa);
    b.decode(fb);
#pragma unroll
    for (int k = 0; k < VEC; ++k) { const float d = (float)fa[k] - (float)fb[k]; acc = fmaf(d, d, acc); }
  }
  acc = group_reduce<256>(acc, OpSum(), red, 0.0f);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}
__global__ void __launch_bounds__(256) mse_final_kernel(const float* partial, float* out, uint32_t n_partial, double inv_n) {
  __shared__ double red[32];
  double acc = 0.0;
  for (uint32_t i = threadIdx.x; i < n_partial; i += 256) acc += (double)partial[i];
  acc = group_reduce<256>(acc, OpSum(), red, 0.0);
  if (threadIdx.x == 0) out[0] = (float)(acc * inv_n);
}
template <typename T>
static int launch_mse(const void* y, const void* t, void* out, uint64_t n, const LaunchCtx& lc, std::string& err) {
  using S = typename Elem<T>::store_t;
  constexpr int V = 16 / sizeof(S);
  const bool vec_ok = n % V == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)t % 16 == 0;
  const uint64_t n_vec = vec_ok ? n / V : n;
  uint32_t grid = (uint32_t)std::min<uint64_t>((n_vec + 255) / 256, 8ull * lc.sm_count);
  grid = std::max(grid, 1u);
  ZYXB_CHECK_ARG(grid * sizeof(float) <= lc.scratch_bytes, "mse: scratch too small");
  float* partial = reinterpret_cast<float*>(lc.scratch);
  if (vec_ok) mse_partial_kernel<T, V><<<grid, 256, 0, lc.stream>>>((const S*)y, (const S*)t, partial, n_vec);
  else mse_partial_kernel<T, 1><<<grid, 256, 0, lc.stream>>>((const S*)y, (const S*)t, partial, n_vec);
  mse_final_kernel<<<1, 256, 0, lc.stream>>>(partial, (float*)out, grid, 1.0 / (double)n);
  return check_launch(lc, err, "mse", 2);
}

// ---- validation and dispatch ---------------------------------------------------------------------
static bool is_float_dtype(int d) { return d == ZYXB_F32 || d == ZYXB_BF16 || d == ZYXB_F16; }

int validate_rowreduce(const zyxb_rowreduce_desc& d, std::string& err) {
  if (d.op < ZYXB_RR_SUM || d.op > ZYXB_RR_LAYERNORM_DYXHAT) { err = "rowreduce: unknown op"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.rows == 0 || d.cols == 0) { err = "rowreduce: rows and cols must be positive"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.rows > 0x7fffffffull) { err = "rowreduce: more than 2^31-1 rows"; return ZYXB_ERR_KERNEL_COMPILATION; }
  const bool int_ok = d.dtype == ZYXB_I32 && (d.op == ZYXB_RR_SUM || d.op == ZYXB_RR_MAX || d.op == ZYXB_RR_MIN);
  if (!is_float_dtype(d.dtype) && !int_ok) { err = "rowreduce: dtype not supported for this op"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if ((d.op == ZYXB_RR_CROSS_ENTROPY || d.op == ZYXB_RR_CROSS_ENTROPY_BWD) && d.dtype != ZYXB_F32) {
    err = "cross_entropy: logits must be f32"; return ZYXB_ERR_KERNEL_COMPILATION;
  }
  if (d.causal && d.period == 0) { err = "softmax: causal mask needs period > 0"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if ((d.op == ZYXB_RR_VAR || d.op == ZYXB_RR_STD) && (int64_t)d.cols - d.correction <= 0) {
    err = "var: cols - correction must be positive"; return ZYXB_ERR_KERNEL_COMPILATION;
  }
  if ((d.op == ZYXB_RR_LAYERNORM || d.op == ZYXB_RR_LAYERNORM_BWD || d.op == ZYXB_RR_LAYERNORM_DYXHAT) && d.cols < 2) {
    err = "layernorm: unbiased variance needs at least 2 columns"; return ZYXB_ERR_KERNEL_COMPILATION;
  }
  return ZYXB_OK;
}

int launch_rowreduce(const zyxb_rowreduce_desc& d, void* const* args, const uint64_t* arg_bytes, int n_args, const LaunchCtx& lc,
                     std::string& err) {
  const uint64_t es = dtype_size(d.dtype);
  const uint64_t full = d.rows * d.cols * es;
  RowParams p{};
  p.rows = d.rows; p.cols = d.cols; p.op = d.op; p.correction = d.correction; p.eps = d.eps;
  p.scale = d.scale == 0.0f ? 1.0f : d.scale; p.causal = d.causal; p.period = d.period; p.rn = lc.round_nearest ? 1 : 0;
  static const bool no_staged = getenv("ZYXB_NO_STAGED_ROWS") != nullptr;
  p.sm_count = no_staged ? 0 : lc.sm_count; p.status = lc.status_word;
  int fam = -1;
  switch (d.op) {
    case ZYXB_RR_SUM: case ZYXB_RR_MAX: case ZYXB_RR_MIN: case ZYXB_RR_MEAN: case ZYXB_RR_VAR: case ZYXB_RR_STD:
      ZYXB_CHECK_ARG(n_args == 2, "reduce: expected args x -> y");
      ZYXB_CHECK_ARG(arg_bytes[0] >= full && arg_bytes[1] >= d.rows * es, "reduce: buffer too small");
      p.x = args[0]; p.y = args[1]; fam = FAM_REDUCE; break;
    case ZYXB_RR_SOFTMAX: case ZYXB_RR_LN_SOFTMAX:
      ZYXB_CHECK_ARG(n_args == 2, "softmax: expected args x -> y");
      ZYXB_CHECK_ARG(arg_bytes[0] >= full && arg_bytes[1] >= full, "softmax: buffer too small");
      p.x = args[0]; p.y = args[1]; fam = FAM_SOFTMAX; break;
    case ZYXB_RR_LAYERNORM: {
      const int want = 2 + (d.has_weight ? 1 : 0) + (d.has_bias ? 1 : 0);
      ZYXB_CHECK_ARG(n_args == want, "layernorm: expected args x [,weight][,bias] -> y");
      int i = 0; p.x = args[i++];
      ZYXB_CHECK_ARG(arg_bytes[0] >= full, "layernorm: x too small");
      if (d.has_weight) { ZYXB_CHECK_ARG(arg_bytes[i] >= d.cols * es, "layernorm: weight too small"); p.w = args[i++]; }
      if (d.has_bias) { ZYXB_CHECK_ARG(arg_bytes[i] >= d.cols * es, "layernorm: bias too small"); p.b = args[i++]; }
      ZYXB_CHECK_ARG(arg_bytes[i] >= full, "layernorm: y too small");
      p.y = args[i]; fam = FAM_LAYERNORM; break;
    }
    case ZYXB_RR_SOFTMAX_BWD:
      ZYXB_CHECK_ARG(n_args == 3, "softmax_bwd: expected args p, dp -> ds");
      ZYXB_CHECK_ARG(arg_bytes[0] >= full && arg_bytes[1] >= full && arg_bytes[2] >= full, "softmax_bwd: buffer too small");
      p.x = args[0]; p.x2 = args[1]; p.y = args[2]; fam = FAM_SOFTMAX_BWD; break;
    case ZYXB_RR_LAYERNORM_BWD: {
      const int want = 3 + (d.has_weight ? 1 : 0);
      ZYXB_CHECK_ARG(n_args == want, "layernorm_bwd: expected args x, dy [,weight] -> dx");
      ZYXB_CHECK_ARG(arg_bytes[0] >= full && arg_bytes[1] >= full && arg_bytes[want - 1] >= full, "layernorm_bwd: buffer too small");
      p.x = args[0]; p.x2 = args[1];
      if (d.has_weight) { ZYXB_CHECK_ARG(arg_bytes[2] >= d.cols * es, "layernorm_bwd: weight too small"); p.w = args[2]; }
      p.y = args[want - 1]; fam = FAM_LAYERNORM_BWD; break;
    }
    case ZYXB_RR_LAYERNORM_DYXHAT:
      ZYXB_CHECK_ARG(n_args == 3, "layernorm_dyxhat: expected args x, dy -> out");
      ZYXB_CHECK_ARG(arg_bytes[0] >= full && arg_bytes[1] >= full && arg_bytes[2] >= full, "layernorm_dyxhat: buffer too small");
      p.x = args[0]; p.x2 = args[1]; p.y = args[2]; fam = FAM_LAYERNORM_BWD; break;
    case ZYXB_RR_CROSS_ENTROPY: {
      ZYXB_CHECK_ARG(n_args == 4, "cross_entropy: expected args logits, labels -> per_sample, mean");
      ZYXB_CHECK_ARG(arg_bytes[0] >= full && arg_bytes[1] >= d.rows * 4 && arg_bytes[2] >= d.rows * 4 && arg_bytes[3] >= 4,
                     "cross_entropy: buffer too small");
      p.x = args[0]; p.x2 = args[1]; p.y = args[2];
      launch_row_f32(FAM_CE, p, lc.stream);
      mean_of_rows_kernel<<<1, 256, 0, lc.stream>>>((const float*)args[2], (float*)args[3], d.rows);
      return check_launch(lc, err, "cross_entropy", 2);
    }
    case ZYXB_RR_CROSS_ENTROPY_BWD:
      ZYXB_CHECK_ARG(n_args == 3, "cross_entropy_bwd: expected args logits, labels -> dlogits");
      ZYXB_CHECK_ARG(arg_bytes[0] >= full && arg_bytes[1] >= d.rows * 4 && arg_bytes[2] >= full, "cross_entropy_bwd: buffer too small");
      p.x = args[0]; p.x2 = args[1]; p.y = args[2];
      launch_row_f32(FAM_CE, p, lc.stream);
      return check_launch(lc, err, "cross_entropy_bwd");
    case ZYXB_RR_COLSUM:
      ZYXB_CHECK_ARG(n_args == 2, "colsum: expected args x -> y");
      ZYXB_CHECK_ARG(arg_bytes[0] >= full && arg_bytes[1] >= d.cols * es, "colsum: buffer too small");
      switch (d.dtype) {
        case ZYXB_F32: return launch_colsum<float>(args[0], args[1], d.rows, d.cols, lc, err);
        case ZYXB_BF16: return launch_colsum<bf16_t>(args[0], args[1], d.rows, d.cols, lc, err);
        default: return launch_colsum<f16_t>(args[0], args[1], d.rows, d.cols, lc, err);
      }
    case ZYXB_RR_MSE:
      ZYXB_CHECK_ARG(n_args == 3, "mse: expected args y, t -> loss");
      ZYXB_CHECK_ARG(arg_bytes[0] >= full && arg_bytes[1] >= full && arg_bytes[2] >= 4, "mse: buffer too small");
      switch (d.dtype) {
        case ZYXB_F32: return launch_mse<float>(args[0], args[1], args[2], d.rows * d.cols, lc, err);
        case ZYXB_BF16: return launch_mse<bf16_t>(args[0], args[1], args[2], d.rows * d.cols, lc, err);
        default: return launch_mse<f16_t>(args[0], args[1], args[2], d.rows * d.cols, lc, err);
      }
    default:
      err = "rowreduce: unknown op"; return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  }
  switch (d.dtype) {
    case ZYXB_F32: launch_row_f32(fam, p, lc.stream); break;
    case ZYXB_BF16: launch_row_bf16(fam, p, lc.stream); break;
    case ZYXB_F16: launch_row_f16(fam, p, lc.stream); break;
    case ZYXB_I32: launch_row_i32(p, lc.stream); break;
    default: err = "rowreduce: dtype"; return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  }
  return check_launch(lc, err, "rowreduce");
}

}  // namespace zyxb
