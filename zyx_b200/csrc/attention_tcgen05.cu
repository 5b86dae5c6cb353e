// Fused self-attention forward on the 5th-generation tensor cores: per (batch, head, 128-query tile) one CTA computes
//   O = softmax(scale * Q.K^T [causal mask]) . V            MultiheadAttention::forward, zyx-nn/src/multi_head_attention.rs:197-226
// without ever writing the [T, T] score matrix: S = Q.K_j^T goes to TMEM, softmax warps turn it into P_j (bf16/f16, in
// shared memory) with the running-maximum recurrence, and P_j.V_j accumulates into an O tile that also lives in TMEM.
// q, k, v and o are [B, T, H*D] activations addressed in place as strided per-head views (row pitch ld, head stride D).
// The row-wise log-sum-exp is stored for a backward pass.
//
// Two CTAs of 192 threads per SM (112 KB of shared memory and 256 TMEM columns each), key tiles of 64:
//   warp 0      TMA producer (one lane): Q once, then K_j into a 2-stage ring and V_j into a single stage
//   warp 1      MMA issuer   (one lane): S_{j+1} = Q.K_{j+1}^T is issued before P_j.V_j, so the tensor core works on the
//               next scores while the softmax warps work on the current ones (S is double-buffered in TMEM)
//   warps 2..5  softmax      : thread = query row = TMEM lane; row maximum and sum stay in registers
// Numerics: scores and the running sum stay f32; P is rounded to the storage type (nearest) only as the tensor-core
// operand; the reference rounds the materialised scores and probabilities instead (truncation), which the 2e-2 tolerance
// of 16-bit results covers.  Every mbarrier wait is time-bounded and reports through the device status word.
#include <cuda.h>
#include <math_constants.h>

#include <algorithm>

#include "common.cuh"
#include "internal.h"
#include "tc_ptx.cuh"

namespace zyxb {

constexpr int AT_BM = 128, AT_BN = 64, AT_D = 128;
constexpr int AT_THREADS = 192;
constexpr int AT_SOFTMAX_WARPS = 4;        // barriers the softmax warps signal count warps: one lane arrives per warp
constexpr int AT_Q_BYTES = AT_BM * AT_D * 2;                 // 32 KB: two boxes of [128 rows x 64 d]
constexpr int AT_KV_BYTES = AT_BN * AT_D * 2;                // 16 KB: two boxes of [64 keys x 64 d]
constexpr int AT_P_BYTES = AT_BM * AT_BN * 2;                // 16 KB: [128 rows x 64 keys]
constexpr int AT_Q_OFF = 0, AT_K_OFF = AT_Q_BYTES, AT_V_OFF = AT_K_OFF + 2 * AT_KV_BYTES;
constexpr int AT_P_OFF = AT_V_OFF + AT_KV_BYTES;            // V is single-buffered (measured: a second stage changes nothing)
constexpr int AT_BAR_OFF = AT_P_OFF + 2 * AT_P_BYTES;        // P is double-buffered: the softmax of tile j+1 does not wait for P_j.V_j
// no alignment slack: the kernel requires the dynamic shared memory window to start on a 1024-byte boundary (it does
// when the kernel has no static shared memory) and reports through the status word otherwise
constexpr int AT_SMEM_TOTAL = AT_BAR_OFF + 256;
enum { AT_ERR_PRODUCER = 16u, AT_ERR_MMA = 32u, AT_ERR_SOFTMAX = 64u, AT_ERR_ALIGN = 1024u };

struct AttnParams {
  void* o; float* lse;
  uint32_t T, heads;
  uint32_t ldo;                 // row pitch of o, elements
  int64_t stride_o_batch;       // elements between batches of o (heads are D apart)
  float scale_log2;             // softmax scale * log2(e)
  int causal, rn, is_bf16;
  uint32_t* status;
};

__global__ void __launch_bounds__(AT_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, AttnParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {                                        // swizzle atoms repeat every 1024 B: refuse rather than compute garbage
    if (threadIdx.x == 0) atomicOr(p.status, AT_ERR_ALIGN);
    return;
  }
  uint8_t* base_ptr = smem_raw;
  const uint32_t bar = base + AT_BAR_OFF;
  const uint32_t q_full = bar;
  auto k_full = [&](int s) { return bar + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar + 8u * (3 + s); };
  auto v_full = [&](int s) { return bar + 8u * (5 + s); };
  auto v_empty = [&](int s) { return bar + 8u * (7 + s); };
  auto s_full = [&](int b) { return bar + 8u * (9 + b); };
  auto s_empty = [&](int b) { return bar + 8u * (11 + b); };
  const uint32_t p_full = bar + 8u * 13, pv_done = bar + 8u * 14;
  auto p_empty = [&](int b) { return bar + 8u * (15 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + AT_BAR_OFF + 8 * 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy query tiles (late rows of a causal mask) are scheduled first
  const uint32_t n_qt = p.T / AT_BM;
  const uint32_t qt = p.causal ? n_qt - 1 - blockIdx.x : blockIdx.x;
  const uint32_t bh = blockIdx.y, b = bh / p.heads, h = bh % p.heads;
  const uint32_t n_kv = p.causal ? (qt + 1) * (AT_BM / AT_BN) : p.T / AT_BN;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(k_full(s), 1); mbar_init(k_empty(s), 1); mbar_init(v_full(s), 1); mbar_init(v_empty(s), 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(s_full(i), 1); mbar_init(s_empty(i), AT_SOFTMAX_WARPS); }
    mbar_init(p_full, AT_SOFTMAX_WARPS);
    mbar_init(pv_done, 1);
    mbar_init(p_empty(0), 1); mbar_init(p_empty(1), 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  constexpr uint32_t TMEM_COLS = 256;                        // S0 (64) | S1 (64) | O (128)
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 2 * AT_BN;

  if (warp == 0) {
    // ---------------------------------- TMA producer ----------------------------------
    if (lane == 0) {
      mbar_expect_tx(q_full, AT_Q_BYTES);
      for (int c = 0; c < 2; ++c) tma_load_4d(base + AT_Q_OFF + c * (AT_Q_BYTES / 2), &map_q, q_full, c * 64, (int)(qt * AT_BM), (int)h, (int)b);
      uint32_t issued = 0, v_issued = 0;
      bool ok = true;
      for (uint32_t j = 0; j < n_kv && ok; ++j) {
        const int s = (int)(j & 1);
        if (!mbar_wait(k_empty(s), ((j >> 1) & 1) ^ 1, abort_flag, p.status, AT_ERR_PRODUCER)) { ok = false; break; }
        const uint32_t k_dst = base + AT_K_OFF + s * AT_KV_BYTES;
        mbar_expect_tx(k_full(s), AT_KV_BYTES);
        for (int c = 0; c < 2; ++c) tma_load_4d(k_dst + c * (AT_KV_BYTES / 2), &map_k, k_full(s), c * 64, (int)(j * AT_BN), (int)h, (int)b);
        if (!mbar_wait(v_empty(0), (j & 1) ^ 1, abort_flag, p.status, AT_ERR_PRODUCER)) { ok = false; ++issued; break; }
        mbar_expect_tx(v_full(0), AT_KV_BYTES);
        for (int c = 0; c < 2; ++c)
          tma_load_4d(base + AT_V_OFF + c * (AT_KV_BYTES / 2), &map_v, v_full(0), c * 64, (int)(j * AT_BN), (int)h, (int)b);
        ++issued; ++v_issued;
      }
      if (!ok) {   // drain: wait (bounded) for copies still in flight so none lands after the CTA has gone
        const uint64_t t0 = global_timer_ns();
        for (uint32_t i = 0; i < 2 && i < issued; ++i) {
          const uint32_t j = issued - 1 - i;
          while (!mbar_try_wait(k_full(j & 1), (j >> 1) & 1) && global_timer_ns() - t0 < TC_WAIT_NS) {}
        }
        if (v_issued) while (!mbar_try_wait(v_full(0), (v_issued - 1) & 1) && global_timer_ns() - t0 < TC_WAIT_NS) {}
        while (!mbar_try_wait(q_full, 0) && global_timer_ns() - t0 < TC_WAIT_NS) {}
      }
    }
  } else if (warp == 1) {
    // ---------------------------------- MMA issuer ----------------------------------
    if (lane == 0) {
      const bool bf16 = p.is_bf16 != 0;
      const uint32_t idesc_s = make_idesc(bf16, false, false, AT_BM, AT_BN);    // Q (K-major) x K (K-major)
      const uint32_t idesc_pv = make_idesc(bf16, false, true, AT_BM, AT_D);     // P (K-major) x V (N-major)
      auto issue_s = [&](uint32_t j) {
        const uint32_t k_addr = base + AT_K_OFF + (j & 1) * AT_KV_BYTES, d_tmem = tmem_base + (j & 1) * AT_BN;
#pragma unroll
        for (int c = 0; c < 2; ++c)          // 64-wide chunks of d
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(d_tmem, make_smem_desc(base + AT_Q_OFF + c * (AT_Q_BYTES / 2) + kk * 32, 16, 1024),
                     make_smem_desc(k_addr + c * (AT_KV_BYTES / 2) + kk * 32, 16, 1024), idesc_s, (c | kk) != 0 ? 1u : 0u);
        umma_commit(k_empty(j & 1));       // K_j may be overwritten once these have read it
        umma_commit(s_full(j & 1));
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, AT_ERR_MMA) && mbar_wait(k_full(0), 0, abort_flag, p.status, AT_ERR_MMA);
      if (ok) { tc_fence_after(); issue_s(0); }
      for (uint32_t j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          const uint32_t jn = j + 1;
          if (!mbar_wait(k_full(jn & 1), (jn >> 1) & 1, abort_flag, p.status, AT_ERR_MMA)) { ok = false; break; }
          if (!mbar_wait(s_empty(jn & 1), ((jn >> 1) & 1) ^ 1, abort_flag, p.status, AT_ERR_MMA)) { ok = false; break; }
          tc_fence_after();
          issue_s(jn);
        }
        if (!mbar_wait(p_full, j & 1, abort_flag, p.status, AT_ERR_MMA)) { ok = false; break; }
        if (!mbar_wait(v_full(0), j & 1, abort_flag, p.status, AT_ERR_MMA)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < AT_BN / 16; ++kk)   // 16 keys per instruction; V rows are 128 B of one 64-wide d chunk, chunks 8 KB apart
          umma_f16(tmem_o, make_smem_desc(base + AT_P_OFF + (j & 1) * AT_P_BYTES + kk * 32, 16, 1024),
                   make_smem_desc(base + AT_V_OFF + kk * (16 * 128), AT_KV_BYTES / 2, 1024), idesc_pv, (j != 0 || kk != 0) ? 1u : 0u);
        umma_commit(v_empty(0));           // V_j has been read
        umma_commit(pv_done);              // O holds tiles 0..j
        umma_commit(p_empty(j & 1));       // this P buffer may be overwritten (signalled after pv_done: a warp that has seen
                                           // P_{j}'s buffer free may rely on pv_done having reached phase j as well)
      }
    }
  } else {
    // ---------------------------------- softmax warps ----------------------------------
    const uint32_t quarter = (uint32_t)(warp & 3);           // TMEM lanes this warp may access
    const uint32_t row = quarter * 32 + lane;                // row of the query tile
    const uint32_t lane_addr = (quarter * 32u) << 16;
    const bool bf16 = p.is_bf16 != 0;
    float m = -CUDART_INF_F, l = 0.0f;
    bool ok = true;
    for (uint32_t j = 0; j < n_kv && ok; ++j) {
      const uint32_t sb = j & 1;
      if (!mbar_wait(s_full(sb), (j >> 1) & 1, abort_flag, p.status, AT_ERR_SOFTMAX)) { ok = false; break; }
      tc_fence_after();
      const bool diag = p.causal && (j + 1) * AT_BN > qt * AT_BM;   // some keys of the tile lie past some rows
      const int32_t shift = (int32_t)(j * AT_BN) - (int32_t)(qt * AT_BM);         // key c of the tile is masked for row r when c + shift > r
      // pass A: row maximum of this tile
      float mx = -CUDART_INF_F;
#pragma unroll 1
      for (int ch = 0; ch < AT_BN / 32; ++ch) {
        uint32_t r[32];
        tmem_ld32(tmem_base + lane_addr + sb * AT_BN + ch * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float s = __uint_as_float(r[i]);
          mx = (diag && ch * 32 + i + shift > (int32_t)row) ? mx : fmaxf(mx, s);
        }
      }
      const float m_new = fmaxf(m, mx * p.scale_log2);
      const bool same = m_new == m;
      const float alpha = same ? 1.0f : ex2f(m - m_new);     // first tile: exp2(-inf) = 0
      // this tile's P buffer was last read by P.V two tiles ago (this also bounds how far the softmax runs ahead:
      // P.V of tile j-2 is complete from here on)
      if (!mbar_wait(p_empty(sb), ((j >> 1) & 1) ^ 1, abort_flag, p.status, AT_ERR_SOFTMAX)) { ok = false; break; }
      // O is rescaled only when some row's maximum moved, and only then does the warp wait for the previous P.V
      if (j > 0 && !__all_sync(0xffffffffu, same)) {
        if (!mbar_wait(pv_done, (j - 1) & 1, abort_flag, p.status, AT_ERR_SOFTMAX)) { ok = false; break; }
        tc_fence_after();
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t r[32];
          tmem_ld32(tmem_o + lane_addr + ch * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st32(tmem_o + lane_addr + ch * 32, r);
        }
        tmem_st_wait();
      }
      // pass B: exponentials, running sum, P tile into shared memory in the swizzled K-major layout the MMA reads
      float sum = 0.0f;
      uint8_t* p_row = base_ptr + AT_P_OFF + sb * AT_P_BYTES + row * 128;
#pragma unroll 1
      for (int ch = 0; ch < AT_BN / 32; ++ch) {
        uint32_t r[32];
        tmem_ld32(tmem_base + lane_addr + sb * AT_BN + ch * 32, r);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float e0 = ex2f(fmaf(__uint_as_float(r[2 * i]), p.scale_log2, -m_new));
          float e1 = ex2f(fmaf(__uint_as_float(r[2 * i + 1]), p.scale_log2, -m_new));
          if (diag) {
            e0 = ch * 32 + 2 * i + shift > (int32_t)row ? 0.0f : e0;
            e1 = ch * 32 + 2 * i + 1 + shift > (int32_t)row ? 0.0f : e1;
          }
          sum += e0 + e1;
          pk[i] = pack2(e0, e1, bf16);
        }
        // columns ch*32 .. +31 = 64 bytes = four 16-byte chunks of the row, chunk index ch * 4 + q, XOR-swizzled by the row
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t chunk = (uint32_t)(ch * 4 + q) ^ (row & 7u);
          *reinterpret_cast<uint4*>(p_row + chunk * 16) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(s_empty(sb));          // this S buffer may be overwritten by S_{j+2}
        mbar_arrive(p_full);
      }
      l = l * alpha + sum;
      m = m_new;
    }
    if (ok && mbar_wait(pv_done, (n_kv - 1) & 1, abort_flag, p.status, AT_ERR_SOFTMAX)) {
      tc_fence_after();
      const float inv = 1.0f / l;
      const bool rn = p.rn != 0;
      const uint64_t grow = (uint64_t)qt * AT_BM + row;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.o) + (int64_t)b * p.stride_o_batch + (int64_t)grow * p.ldo + (int64_t)h * AT_D;
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t r[32];
        tmem_ld32(tmem_o + lane_addr + ch * 32, r);
        tmem_ld_wait();
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float a = __uint_as_float(r[2 * i]) * inv, c = __uint_as_float(r[2 * i + 1]) * inv;
          const uint16_t lo = bf16 ? f32_to_bf16(a, rn) : f32_to_f16(a, rn), hi = bf16 ? f32_to_bf16(c, rn) : f32_to_f16(c, rn);
          w[i] = (uint32_t)lo | ((uint32_t)hi << 16);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(orow + ch * 32 + q * 8) = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
      }
      if (p.lse) p.lse[(uint64_t)bh * p.T + grow] = (m + log2f(l)) * 0.6931471805599453f;   // natural log of sum(exp(scale * s))
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
int validate_attention(const zyxb_attention_desc& d, std::string& err) {
  if (d.dtype != ZYXB_BF16 && d.dtype != ZYXB_F16) { err = "attention: dtype must be bf16 or f16"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.head_dim != AT_D) { err = "attention: head_dim must be 128"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.batch == 0 || d.heads == 0 || d.seq == 0) { err = "attention: batch, heads and seq must be positive"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.seq % AT_BM) { err = "attention: seq must be a multiple of 128"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.batch * d.heads > 65535) { err = "attention: more than 65535 (batch, head) pairs"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.seq > 0x7fffff00ull) { err = "attention: seq too large"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (!(d.scale >= 0.0f)) { err = "attention: scale must be positive (0 = 1/sqrt(head_dim))"; return ZYXB_ERR_KERNEL_COMPILATION; }
  return ZYXB_OK;
}

int launch_attention(const zyxb_attention_desc& d, void* const* args, const uint64_t* arg_bytes, int n_args, const LaunchCtx& lc,
                     std::string& err) {
  ZYXB_CHECK_ARG(n_args == 5, "attention: expected args q, k, v -> o, lse");
  ZYXB_CHECK_ARG(lc.tma_encode != nullptr, "attention: no tensor-map encoder (driver entry point missing)");
  const uint64_t E = d.heads * d.head_dim, ld = d.ld ? d.ld : E;
  ZYXB_CHECK_ARG(ld >= E && ld % 8 == 0, "attention: row pitch must cover heads*head_dim and be a multiple of 8 elements");
  const uint64_t need = ((d.batch * d.seq - 1) * ld + E) * 2;
  for (int i = 0; i < 4; ++i) {
    ZYXB_CHECK_ARG(arg_bytes[i] >= need, "attention: q, k, v or o too small");
    ZYXB_CHECK_ARG((uintptr_t)args[i] % 16 == 0, "attention: operands must be 16-byte aligned");
  }
  ZYXB_CHECK_ARG(arg_bytes[4] >= d.batch * d.heads * d.seq * 4, "attention: lse too small");
  const bool bf16 = d.dtype == ZYXB_BF16;
  CUtensorMap mq, mk, mv;
  const bool okm = encode_map(lc.tma_encode, &mq, bf16, args[0], d.head_dim, d.seq, ld, d.heads, d.head_dim, d.batch, d.seq * ld, AT_BM) &&
                   encode_map(lc.tma_encode, &mk, bf16, args[1], d.head_dim, d.seq, ld, d.heads, d.head_dim, d.batch, d.seq * ld, AT_BN) &&
                   encode_map(lc.tma_encode, &mv, bf16, args[2], d.head_dim, d.seq, ld, d.heads, d.head_dim, d.batch, d.seq * ld, AT_BN);
  if (!okm) { err = "attention: cuTensorMapEncodeTiled rejected an operand"; return ZYXB_ERR_KERNEL_LAUNCH; }
  AttnParams p{};
  p.o = args[3]; p.lse = reinterpret_cast<float*>(args[4]);
  p.T = (uint32_t)d.seq; p.heads = (uint32_t)d.heads; p.ldo = (uint32_t)ld; p.stride_o_batch = (int64_t)(d.seq * ld);
  const float scale = d.scale > 0.0f ? d.scale : 1.0f / sqrtf((float)d.head_dim);
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = d.causal ? 1 : 0; p.rn = lc.round_nearest ? 1 : 0; p.is_bf16 = bf16 ? 1 : 0; p.status = lc.status_word;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM_TOTAL);
    if (e != cudaSuccess) { err = std::string("attention: ") + cudaGetErrorString(e); return ZYXB_ERR_KERNEL_LAUNCH; }
    configured = true;
  }
  const dim3 grid((unsigned)(d.seq / AT_BM), (unsigned)(d.batch * d.heads));
  attn_fwd_kernel<<<grid, AT_THREADS, AT_SMEM_TOTAL, lc.stream>>>(mq, mk, mv, p);
  return check_launch(lc, err, "attention");
}

}  // namespace zyxb
