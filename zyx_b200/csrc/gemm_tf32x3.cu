// f32 matmul on the tensor cores at f32 accuracy: every operand x is split into hi = tf32(x) and lo = tf32(x - hi), both
// rounded to nearest, and
//   a.b ~= a_hi.b_hi + a_hi.b_lo + a_lo.b_hi          (three tensor-core products per k-step, f32 accumulation in TMEM).
// Products of tf32 values are exact in f32; what is dropped is a_lo.b_lo and x - hi - lo, each near 2^-22 of the product
// and, because both splits round to nearest, of either sign: the error behaves like f32 rounding noise.  (A kind::tf32
// tcgen05.mma truncates the f32 words it reads; with hi = truncation the dropped terms all carry the product's sign and add
// up to a bias of about 1e-6 of sum |a||b| - measured, ten times the 1e-5 bar at k = 4096.  So hi and lo are stored
// already rounded, and the hardware's truncation has nothing left to cut.)
// That meets the 1e-5 bar of the f32 path where plain TF32 (2^-11) cannot, at a third of the TF32 rate instead of the
// FP32 FMA rate.  Tensor::dot for f32, zyx/src/tensor/mod.rs:1469-1490; accumulation dtype reduce_ops.rs:52-60.
//
// Two launches: a preparation kernel per operand writes hi and lo (transposed, for an operand whose contraction axis is
// not the contiguous one) into the context's scratch, so that the matmul kernel reads four K-major f32 streams
// {A_hi, A_lo, B_hi, B_lo} by TMA; the matmul kernel is the persistent TMA / tcgen05 / TMEM pipeline of the 16-bit
// matmul with three MMAs per k-step.  Plain C = alpha * A.B (+ bias) problems only; everything else stays on the FFMA kernel.
#include <cuda.h>
#include <stdlib.h>

#include <algorithm>

#include "common.cuh"
#include "gemm.h"
#include "tc_ptx.cuh"

namespace zyxb {

constexpr int X3_BM = 128, X3_BN = 256, X3_BK = 32;          // 32 f32 = one 128-byte swizzle atom along K
constexpr int X3_UMMA_K = 8, X3_STAGES = 2;
constexpr int X3_CHUNK_BLOCKS = 2;                          // k-blocks (of 32) per accumulator: 64 k per chunk
constexpr int X3_THREADS = 320, X3_EPI_THREADS = 256;
constexpr int X3_A_BYTES = X3_BM * X3_BK * 4, X3_B_BYTES = X3_BN * X3_BK * 4;
constexpr int X3_STAGE_BYTES = 2 * (X3_A_BYTES + X3_B_BYTES);   // hi and lo of both operands: 96 KB
constexpr int X3_BAR_OFFSET = X3_STAGES * X3_STAGE_BYTES;
constexpr int X3_SMEM_TOTAL = X3_BAR_OFFSET + 256 + 1024;
enum { X3_ERR_PRODUCER = 2048u, X3_ERR_MMA = 4096u, X3_ERR_EPILOGUE = 8192u };

struct X3Params {
  const float* bias; float* c;
  uint32_t m, n, k, tiles_m, tiles_n, ldc;
  float alpha;
  int has_bias;
  uint32_t* status;
};

// nearest tf32 (10 explicit mantissa bits) of an f32, as an f32 whose low 13 bits are zero
__device__ __forceinline__ float tf32_rn(float x) {
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
  return __uint_as_float(u);
}
__device__ __forceinline__ void tf32_split(float x, float& hi, float& lo) {
  hi = tf32_rn(x);
  lo = tf32_rn(x - hi);
}

// hi and lo of x (rows of `cols` elements with pitch ld), written densely
__global__ void __launch_bounds__(256) x3_split_kernel(const float* __restrict__ x, float* __restrict__ hi, float* __restrict__ lo, uint64_t rows,
                                                       uint64_t cols, uint64_t ld) {
  const uint64_t n4 = cols / 4, total = rows * n4;
  for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (uint64_t)gridDim.x * 256) {
    const uint64_t r = i / n4, c = (i % n4) * 4;
    const float4 v = *reinterpret_cast<const float4*>(x + r * ld + c);
    float4 h, l;
    tf32_split(v.x, h.x, l.x); tf32_split(v.y, h.y, l.y); tf32_split(v.z, h.z, l.z); tf32_split(v.w, h.w, l.w);
    *reinterpret_cast<float4*>(hi + r * cols + c) = h;
    *reinterpret_cast<float4*>(lo + r * cols + c) = l;
  }
}
// x stored [rows, cols] with pitch ld -> hi and lo of x^T [cols, rows] (32 x 32 tiles through shared memory)
__global__ void __launch_bounds__(256) x3_transpose_split_kernel(const float* __restrict__ x, float* __restrict__ t_hi, float* __restrict__ t_lo,
                                                                 uint64_t rows, uint64_t cols, uint64_t ld) {
  __shared__ float tile[32][33];
  const uint64_t c0 = (uint64_t)blockIdx.x * 32, r0 = (uint64_t)blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
  for (int j = ty; j < 32; j += 8)
    tile[j][tx] = (r0 + j < rows && c0 + tx < cols) ? x[(r0 + j) * ld + c0 + tx] : 0.0f;
  __syncthreads();
  for (int j = ty; j < 32; j += 8) {
    const uint64_t orow = c0 + j, ocol = r0 + tx;
    if (orow < cols && ocol < rows) {
      float h, l;
      tf32_split(tile[tx][j], h, l);
      t_hi[orow * rows + ocol] = h;
      t_lo[orow * rows + ocol] = l;
    }
  }
}

__global__ void __launch_bounds__(X3_THREADS, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_al,
                   const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_bl, X3Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t bar_base = base + X3_BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (X3_STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * X3_STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * X3_STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + X3_BAR_OFFSET + 8 * (2 * X3_STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * X3_BN;
  if (threadIdx.x == 0) {
    for (int s = 0; s < X3_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), X3_EPI_THREADS / 32); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const uint32_t total_tiles = p.tiles_m * p.tiles_n;
  const uint32_t k_blocks = (p.k + X3_BK - 1) / X3_BK;
  constexpr uint32_t GROUP_M = 16;   // tiles that run together share A and B panels in L2
  auto tile_coords = [&](uint32_t t, uint32_t& tm, uint32_t& tn) {
    const uint32_t group_size = GROUP_M * p.tiles_n;
    const uint32_t g = t / group_size, first_m = g * GROUP_M;
    const uint32_t rows_in_group = min(GROUP_M, p.tiles_m - first_m);
    const uint32_t in_group = t % group_size;
    tm = first_m + in_group % rows_in_group;
    tn = in_group / rows_in_group;
  };

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, issued = 0;
      bool ok = true;
      for (uint32_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        uint32_t tm, tn;
        tile_coords(t, tm, tn);
        for (uint32_t kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, p.status, X3_ERR_PRODUCER)) { ok = false; break; }
          const uint32_t a_dst = base + stage * X3_STAGE_BYTES, al_dst = a_dst + X3_A_BYTES, b_dst = al_dst + X3_A_BYTES, bl_dst = b_dst + X3_B_BYTES;
          mbar_expect_tx(full_bar(stage), X3_STAGE_BYTES);
          const int k0 = (int)(kb * X3_BK);
          tma_load_4d(a_dst, &map_a, full_bar(stage), k0, (int)(tm * X3_BM), 0, 0);
          tma_load_4d(al_dst, &map_al, full_bar(stage), k0, (int)(tm * X3_BM), 0, 0);
          tma_load_4d(b_dst, &map_b, full_bar(stage), k0, (int)(tn * X3_BN), 0, 0);
          tma_load_4d(bl_dst, &map_bl, full_bar(stage), k0, (int)(tn * X3_BN), 0, 0);
          ++issued;
          if (++stage == X3_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        uint32_t s = stage, ph = phase;
        const uint32_t n_back = issued < (uint32_t)X3_STAGES ? issued : (uint32_t)X3_STAGES;
        for (uint32_t i = 0; i < n_back; ++i) {
          if (s == 0) { s = X3_STAGES - 1; ph ^= 1; } else --s;
          const uint64_t t0 = global_timer_ns();
          while (!mbar_try_wait(full_bar(s), ph) && global_timer_ns() - t0 < TC_WAIT_NS) {}
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // kind::tf32: f32 accumulate (bit 4), A and B format TF32 (2) at bits 7 and 10, both K-major, N >> 3 at 17, M >> 4 at 24
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(X3_BN >> 3) << 17) | ((uint32_t)(X3_BM >> 4) << 24);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (uint32_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        for (uint32_t kb = 0; kb < k_blocks && ok; ++kb) {
          const uint32_t in_chunk = kb % X3_CHUNK_BLOCKS;
          if (in_chunk == 0) {   // a new k-chunk starts in the other accumulator, from zero
            if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, abort_flag, p.status, X3_ERR_MMA)) { ok = false; break; }
            tc_fence_after();
          }
          const uint32_t d_tmem = tmem_base + acc * X3_BN;
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, X3_ERR_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = base + stage * X3_STAGE_BYTES, al_addr = a_addr + X3_A_BYTES, b_addr = al_addr + X3_A_BYTES, bl_addr = b_addr + X3_B_BYTES;
#pragma unroll
          for (int kk = 0; kk < X3_BK / X3_UMMA_K; ++kk) {   // 8 f32 = 32 bytes inside the swizzle atom
            const uint64_t ah = make_smem_desc(a_addr + kk * 32, 16, 1024), al = make_smem_desc(al_addr + kk * 32, 16, 1024);
            const uint64_t bh = make_smem_desc(b_addr + kk * 32, 16, 1024), bl = make_smem_desc(bl_addr + kk * 32, 16, 1024);
            // the small terms first, so that the large one is added to an accumulator that already holds them
            asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                         ::"r"(d_tmem), "l"(al), "l"(bh), "r"(idesc), "r"((in_chunk | (uint32_t)kk) != 0 ? 1u : 0u) : "memory");
            asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                         ::"r"(d_tmem), "l"(ah), "l"(bl), "r"(idesc), "r"(1u) : "memory");
            asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                         ::"r"(d_tmem), "l"(ah), "l"(bh), "r"(idesc), "r"(1u) : "memory");
          }
          umma_commit(empty_bar(stage));
          if (++stage == X3_STAGES) { stage = 0; phase ^= 1; }
          if (in_chunk == X3_CHUNK_BLOCKS - 1 || kb + 1 == k_blocks) {   // chunk complete: hand it to the epilogue warps
            umma_commit(tfull_bar(acc));
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
          }
        }
      }
    }
  } else {
    // epilogue (warps 2..9): two warps per TMEM lane quarter, each taking half of the columns
    const int col_half = (warp - 2) >> 2;
    const uint32_t quarter = (uint32_t)(warp & 3);
    const uint32_t row_in_tile = quarter * 32 + lane;
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    const uint32_t n_chunks = (k_blocks + X3_CHUNK_BLOCKS - 1) / X3_CHUNK_BLOCKS;
    for (uint32_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      uint32_t tm, tn;
      tile_coords(t, tm, tn);
      // The tensor core adds into its accumulator with truncation, which over thousands of k-steps grows into a bias of
      // 1e-4 of the result (measured).  So an accumulator only ever holds one k-chunk; the chunks are added here, in f32
      // with rounding to nearest, in this thread's registers: 128 columns of its row.
      float sum[X3_BN / 2];
#pragma unroll
      for (int i = 0; i < X3_BN / 2; ++i) sum[i] = 0.0f;
      for (uint32_t ck = 0; ck < n_chunks && ok; ++ck) {
        if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, X3_ERR_EPILOGUE)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int ch = 0; ch < X3_BN / 64; ++ch) {
          uint32_t r[32];
          tmem_ld32(tmem_base + ((quarter * 32u) << 16) + acc * X3_BN + (col_half * (X3_BN / 64) + ch) * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) sum[ch * 32 + i] += __uint_as_float(r[i]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok) break;
      const uint32_t row = tm * X3_BM + row_in_tile, col0 = tn * X3_BN + col_half * (X3_BN / 2);
      if (row < p.m) {
        float* crow = p.c + (int64_t)row * p.ldc;
#pragma unroll
        for (int q = 0; q < X3_BN / 8; ++q) {
          const uint32_t c = col0 + q * 4;
          if (c < p.n) {   // n is a multiple of 4
            float4 v = make_float4(sum[4 * q], sum[4 * q + 1], sum[4 * q + 2], sum[4 * q + 3]);
            if (p.alpha != 1.0f) { v.x *= p.alpha; v.y *= p.alpha; v.z *= p.alpha; v.w *= p.alpha; }
            if (p.has_bias) {
              const float4 bv = *reinterpret_cast<const float4*>(p.bias + c);
              v.x += bv.x; v.y += bv.y; v.z += bv.z; v.w += bv.w;
            }
            *reinterpret_cast<float4*>(crow + c) = v;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- host side ---------------------------------------------------------------------------------------
static bool encode_map_f32(void* fn, CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_outer) {
  cuuint64_t dims[4] = {inner, outer, 1, 1};
  cuuint64_t strides[3] = {ld * 4, ld * outer * 4, ld * outer * 4};
  cuuint32_t box[4] = {32, box_outer, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return reinterpret_cast<EncodeTiledFn>(fn)(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// scratch the prepared operands need: hi and lo of A as [m, k] and of B as [n, k]
static uint64_t x3_scratch_bytes(const GemmParams& p) { return 2 * (p.m * p.k + p.n * p.k) * 4; }

bool gemm_tf32x3_supported(const GemmParams& p, int dtype, const LaunchCtx& lc) {
  static const bool off = getenv("ZYXB_NO_TF32X3") != nullptr;
  if (off || dtype != ZYXB_F32 || !lc.tma_encode) return false;
  if (p.batch * p.batch_inner != 1) return false;
  if (p.epilogue != ZYXB_EPI_NONE && p.epilogue != ZYXB_EPI_BIAS) return false;
  if (p.preact || p.z) return false;
  if (p.m < 512 || p.n < 512 || p.k < 256) return false;            // small problems: the FFMA kernel (with split k) is faster
  if (p.m % 4 || p.n % 4 || p.k % 4 || p.lda % 4 || p.ldb % 4 || p.ldc % 4) return false;
  if ((uintptr_t)p.a % 16 || (uintptr_t)p.b % 16 || (uintptr_t)p.c % 16 || (p.bias && (uintptr_t)p.bias % 16)) return false;
  if (p.m > 0x7fffff00ull || p.n > 0x7fffff00ull || p.k > 0x7fffff00ull || p.ldc > 0xffffffffull) return false;
  return x3_scratch_bytes(p) <= lc.scratch_bytes;
}

int launch_gemm_tf32x3(const GemmParams& p, const LaunchCtx& lc, std::string& err) {
  float* a_hi = reinterpret_cast<float*>(lc.scratch);
  float* a_lo = a_hi + p.m * p.k;
  float* b_hi = a_lo + p.m * p.k;
  float* b_lo = b_hi + p.n * p.k;
  const float* A = reinterpret_cast<const float*>(p.a);
  const float* B = reinterpret_cast<const float*>(p.b);
  const unsigned split_grid = (unsigned)lc.sm_count * 8;
  if (p.trans_a)     // stored [k, m] -> [m, k]
    x3_transpose_split_kernel<<<dim3((unsigned)((p.m + 31) / 32), (unsigned)((p.k + 31) / 32)), 256, 0, lc.stream>>>(A, a_hi, a_lo, p.k, p.m, p.lda);
  else
    x3_split_kernel<<<split_grid, 256, 0, lc.stream>>>(A, a_hi, a_lo, p.m, p.k, p.lda);
  if (!p.trans_b)    // stored [k, n] -> [n, k]
    x3_transpose_split_kernel<<<dim3((unsigned)((p.n + 31) / 32), (unsigned)((p.k + 31) / 32)), 256, 0, lc.stream>>>(B, b_hi, b_lo, p.k, p.n, p.ldb);
  else
    x3_split_kernel<<<split_grid, 256, 0, lc.stream>>>(B, b_hi, b_lo, p.n, p.k, p.ldb);
  const int kernels = 3;
  CUtensorMap ma, mal, mb, mbl;
  const bool okm = encode_map_f32(lc.tma_encode, &ma, a_hi, p.k, p.m, p.k, X3_BM) && encode_map_f32(lc.tma_encode, &mal, a_lo, p.k, p.m, p.k, X3_BM) &&
                   encode_map_f32(lc.tma_encode, &mb, b_hi, p.k, p.n, p.k, X3_BN) && encode_map_f32(lc.tma_encode, &mbl, b_lo, p.k, p.n, p.k, X3_BN);
  if (!okm) { err = "gemm (tf32x3): cuTensorMapEncodeTiled rejected an operand"; return ZYXB_ERR_KERNEL_LAUNCH; }
  X3Params xp{};
  xp.bias = reinterpret_cast<const float*>(p.bias); xp.c = reinterpret_cast<float*>(p.c);
  xp.m = (uint32_t)p.m; xp.n = (uint32_t)p.n; xp.k = (uint32_t)p.k; xp.ldc = (uint32_t)p.ldc;
  xp.tiles_m = (uint32_t)((p.m + X3_BM - 1) / X3_BM); xp.tiles_n = (uint32_t)((p.n + X3_BN - 1) / X3_BN);
  xp.alpha = p.alpha; xp.has_bias = p.epilogue == ZYXB_EPI_BIAS ? 1 : 0; xp.status = lc.status_word;
  static uint64_t configured = 0;
  {
    cudaError_t e = ensure_dynamic_smem(gemm_tf32x3_kernel, X3_SMEM_TOTAL, &configured);
    if (e != cudaSuccess) { err = std::string("gemm (tf32x3): ") + cudaGetErrorString(e); return ZYXB_ERR_KERNEL_LAUNCH; }
  }
  const unsigned grid = (unsigned)std::min<uint64_t>((uint64_t)xp.tiles_m * xp.tiles_n, (uint64_t)lc.sm_count);
  gemm_tf32x3_kernel<<<grid, X3_THREADS, X3_SMEM_TOTAL, lc.stream>>>(ma, mal, mb, mbl, xp);
  return check_launch(lc, err, "gemm (tf32x3)", kernels);
}

}  // namespace zyxb
