// Fused self-attention forward on the 5th-generation tensor cores: per (batch, head, 128-query tile) one CTA computes
//   O = softmax(scale * Q.K^T [causal mask]) . V            MultiheadAttention::forward, zyx-nn/src/multi_head_attention.rs:197-226
// without ever writing the [T, T] score matrix: S = Q.K_j^T goes to TMEM, softmax warps turn it into P_j (bf16/f16, in
// shared memory) with the running-maximum recurrence, and P_j.V_j accumulates into an O tile that also lives in TMEM.
// q, k, v and o are [B, T, H*D] activations addressed in place as strided per-head views (row pitch ld, head stride D).
// The row-wise log-sum-exp is stored for a backward pass.
//
// One CTA of 352 threads per SM, 128 x 128 tiles (224 KB of shared memory, 384 TMEM columns):
//   warp 0      TMA producer (one lane): Q once, then K_j and V_j into 2-stage rings
//   warp 1      MMA issuer   (one lane): S_j = Q.K_j^T, up to two tiles ahead of the softmax (S is double-buffered in TMEM)
//   warp 10     MMA issuer   (one lane): O += P_j.V_j (P is double-buffered in shared memory)
//   warps 2..9  softmax      : two threads per query row (TMEM lane), 64 keys of the tile each; running maximum and sums
//               stay in registers
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

constexpr int AT_BM = 128, AT_BN = 128, AT_D = 128;
constexpr int AT_THREADS = 352;
constexpr int AT_SOFTMAX_WARPS = 8;        // barriers the softmax warps signal count warps: one lane arrives per warp
constexpr int AT_TILE = 128 * 128 * 2;     // one 128 x 128 16-bit tile, 32 KB
constexpr int AT_Q_OFF = 0, AT_K_OFF = AT_TILE, AT_V_OFF = AT_K_OFF + 2 * AT_TILE, AT_P_OFF = AT_V_OFF + 2 * AT_TILE;
constexpr int AT_XCHG_OFF = AT_P_OFF + 2 * AT_TILE;          // 2 KB: row maxima / sums exchanged between the two column halves
constexpr int AT_BAR_OFF = AT_XCHG_OFF + 2048;
// 224 KB of tiles + 2 KB + barriers: no room for alignment slack, so the kernel requires the dynamic shared memory window
// to start on a 1024-byte boundary (it does when the kernel has no static shared memory) and reports otherwise
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

__global__ void __launch_bounds__(AT_THREADS, 1)
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
  // every barrier that is reused across tiles exists once per buffer (index = tile & 1), so that a role running a tile
  // ahead can never complete two phases of a barrier before its waiter has seen the first
  const uint32_t q_full = bar;
  auto k_full = [&](int s) { return bar + 8u * (1 + s); };
  auto v_full = [&](int s) { return bar + 8u * (3 + s); };
  auto s_full = [&](int s) { return bar + 8u * (5 + s); };    // S_j complete: the softmax may read it, K stage j & 1 is free
  auto s_empty = [&](int s) { return bar + 8u * (7 + s); };   // the softmax holds S_j in registers
  auto p_full = [&](int s) { return bar + 8u * (9 + s); };    // P_j is in shared memory (and O rescaled if it had to be)
  auto pv_done = [&](int s) { return bar + 8u * (11 + s); };  // P_j.V_j complete: V stage and P buffer j & 1 are free
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + AT_BAR_OFF + 8 * 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy query tiles (late rows of a causal mask) are scheduled first
  const uint32_t n_qt = p.T / AT_BM;
  // x = (batch, head), y = query tile: every heavy CTA of the launch (late query rows under a causal mask) starts before any light one
  const uint32_t qt = p.causal ? n_qt - 1 - blockIdx.y : blockIdx.y;
  const uint32_t bh = blockIdx.x, b = bh / p.heads, h = bh % p.heads;
  const uint32_t n_kv = p.causal ? qt + 1 : p.T / AT_BN;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full(s), 1); mbar_init(v_full(s), 1); mbar_init(s_full(s), 1); mbar_init(pv_done(s), 1);
      mbar_init(s_empty(s), AT_SOFTMAX_WARPS); mbar_init(p_full(s), AT_SOFTMAX_WARPS);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  constexpr uint32_t TMEM_COLS = 512;                        // S0 | S1 | O (384 used; allocations are powers of two)
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 2 * AT_BN;

  if (warp == 0) {
    // ---------------------------------- TMA producer ----------------------------------
    if (lane == 0) {
      mbar_expect_tx(q_full, AT_TILE);
      for (int c = 0; c < 2; ++c) tma_load_4d(base + AT_Q_OFF + c * (AT_TILE / 2), &map_q, q_full, c * 64, (int)(qt * AT_BM), (int)h, (int)b);
      uint32_t k_issued = 0, v_issued = 0;
      bool ok = true;
      for (uint32_t j = 0; j < n_kv; ++j) {
        const int s = (int)(j & 1);
        const uint32_t free_parity = ((j >> 1) & 1) ^ 1;     // the phase two tiles back
        if (!mbar_wait(s_full(s), free_parity, abort_flag, p.status, AT_ERR_PRODUCER)) { ok = false; break; }
        mbar_expect_tx(k_full(s), AT_TILE);
        for (int c = 0; c < 2; ++c)
          tma_load_4d(base + AT_K_OFF + s * AT_TILE + c * (AT_TILE / 2), &map_k, k_full(s), c * 64, (int)(j * AT_BN), (int)h, (int)b);
        ++k_issued;
        if (!mbar_wait(pv_done(s), free_parity, abort_flag, p.status, AT_ERR_PRODUCER)) { ok = false; break; }
        mbar_expect_tx(v_full(s), AT_TILE);
        for (int kb = 0; kb < 2; ++kb)      // 64 keys per k-block, two 64-wide boxes of d each
          for (int c = 0; c < 2; ++c)
            tma_load_4d(base + AT_V_OFF + s * AT_TILE + kb * (AT_TILE / 2) + c * (AT_TILE / 4), &map_v, v_full(s), c * 64,
                        (int)(j * AT_BN) + kb * 64, (int)h, (int)b);
        ++v_issued;
      }
      if (!ok) {   // drain: wait (bounded) for copies still in flight so none lands after the CTA has gone
        const uint64_t t0 = global_timer_ns();
        for (uint32_t i = 0; i < 2; ++i) {
          if (i < k_issued) { const uint32_t j = k_issued - 1 - i; while (!mbar_try_wait(k_full(j & 1), (j >> 1) & 1) && global_timer_ns() - t0 < TC_WAIT_NS) {} }
          if (i < v_issued) { const uint32_t j = v_issued - 1 - i; while (!mbar_try_wait(v_full(j & 1), (j >> 1) & 1) && global_timer_ns() - t0 < TC_WAIT_NS) {} }
        }
        while (!mbar_try_wait(q_full, 0) && global_timer_ns() - t0 < TC_WAIT_NS) {}
      }
    }
  } else if (warp == 1) {
    // ---------------------------------- MMA issuer ----------------------------------
    // 128-wide tiles on purpose: an instruction of N = 64 occupies the tensor core as long as one of N = 128, and every
    // instruction and commit costs the issuing thread tens to hundreds of cycles, so fewer and larger is faster.
    if (lane == 0) {
      const bool bf16 = p.is_bf16 != 0;
      const uint32_t idesc_s = make_idesc(bf16, false, false, AT_BM, AT_BN);    // Q (K-major) x K (K-major)
      auto issue_s = [&](uint32_t j) {
        const uint32_t k_addr = base + AT_K_OFF + (j & 1) * AT_TILE, d_tmem = tmem_base + (j & 1) * AT_BN;
#pragma unroll
        for (int c = 0; c < 2; ++c)          // 64-wide chunks of d
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(d_tmem, make_smem_desc(base + AT_Q_OFF + c * (AT_TILE / 2) + kk * 32, 16, 1024),
                     make_smem_desc(k_addr + c * (AT_TILE / 2) + kk * 32, 16, 1024), idesc_s, (c | kk) != 0 ? 1u : 0u);
        umma_commit(s_full(j & 1));
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, AT_ERR_MMA);
      for (uint32_t j = 0; j < n_kv && ok; ++j) {
        if (!mbar_wait(k_full(j & 1), (j >> 1) & 1, abort_flag, p.status, AT_ERR_MMA)) { ok = false; break; }
        if (!mbar_wait(s_empty(j & 1), ((j >> 1) & 1) ^ 1, abort_flag, p.status, AT_ERR_MMA)) { ok = false; break; }
        tc_fence_after();
        issue_s(j);
      }
    }
  } else if (warp == 10) {
    // ---------------------------------- second MMA issuer: O += P_j . V_j ----------------------------------
    // Issuing an instruction costs its thread about as long as the tensor core needs to execute it, so the two products
    // of a tile are issued by two threads: the scores of tile j+1 and the output update of tile j proceed side by side.
    if (lane == 0) {
      const bool bf16 = p.is_bf16 != 0;
      const uint32_t idesc_pv = make_idesc(bf16, false, true, AT_BM, AT_D);     // P (K-major) x V (N-major)
      bool ok = true;
      for (uint32_t j = 0; j < n_kv && ok; ++j) {
        if (!mbar_wait(p_full(j & 1), (j >> 1) & 1, abort_flag, p.status, AT_ERR_MMA)) { ok = false; break; }
        if (!mbar_wait(v_full(j & 1), (j >> 1) & 1, abort_flag, p.status, AT_ERR_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t p_addr = base + AT_P_OFF + (j & 1) * AT_TILE, v_addr = base + AT_V_OFF + (j & 1) * AT_TILE;
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)       // 64 keys per k-block
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)     // V rows are 128 B of one 64-wide d chunk, the two chunks 8 KB apart
            umma_f16(tmem_o, make_smem_desc(p_addr + kb * (AT_TILE / 2) + kk * 32, 16, 1024),
                     make_smem_desc(v_addr + kb * (AT_TILE / 2) + kk * (16 * 128), AT_TILE / 4, 1024), idesc_pv,
                     (j != 0 || (kb | kk) != 0) ? 1u : 0u);
        umma_commit(pv_done(j & 1));
      }
    }
  } else {
    // ---------------------------------- softmax warps ----------------------------------
    // Two warps per TMEM lane quarter: warp 2+q takes keys 0..63 of the tile, warp 6+q keys 64..127, for the same 32 rows.
    // The two halves of a row exchange their maximum through shared memory (a 64-thread named barrier per quarter);
    // each keeps the running sum of its own keys, and the halves are added once at the end.
    const uint32_t quarter = (uint32_t)(warp & 3);           // TMEM lanes this warp may access
    const int half = (warp - 2) >> 2;
    const uint32_t row = quarter * 32 + lane;                // row of the query tile
    const uint32_t lane_addr = (quarter * 32u) << 16;
    const bool bf16 = p.is_bf16 != 0;
    float* xchg = reinterpret_cast<float*>(base_ptr + AT_XCHG_OFF);          // [2 parities][2 halves][128 rows]
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory"); };
    float m = -CUDART_INF_F, l = 0.0f;
    bool ok = true;
    for (uint32_t j = 0; j < n_kv && ok; ++j) {
      const uint32_t sb = j & 1;
      if (!mbar_wait(s_full(sb), (j >> 1) & 1, abort_flag, p.status, AT_ERR_SOFTMAX)) { ok = false; break; }
      tc_fence_after();
      uint32_t r[64];
      {
        uint32_t (&r0)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[0]);
        uint32_t (&r1)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[32]);
        tmem_ld32(tmem_base + lane_addr + sb * AT_BN + half * 64, r0);
        tmem_ld32(tmem_base + lane_addr + sb * AT_BN + half * 64 + 32, r1);
      }
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty(sb));               // the scores are in registers: S_{j+2} may overwrite the buffer
      // key c of this thread's 64 is masked for its row when c > lim; only the diagonal tile takes the masked loops
      const bool diag = p.causal && j == qt;
      const int32_t lim = (int32_t)row - half * 64;
      float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};   // independent chains
      if (!diag) {
#pragma unroll
        for (int i = 0; i < 64; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(r[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) mx4[i & 3] = i > lim ? mx4[i & 3] : fmaxf(mx4[i & 3], __uint_as_float(r[i]));
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      float* xm = xchg + (j & 1) * 256;
      xm[half * 128 + row] = mx;
      pair_sync();
      mx = fmaxf(mx, xm[(half ^ 1) * 128 + row]);
      // The reference point m of the exponentials follows the running maximum lazily: it moves only when the maximum has
      // grown by more than 2^8 beyond it, so exponentials stay below 256 (exact enough in the 16-bit operand, far from
      // overflow in the f32 sums) and the output tile is rescaled a few times per row instead of at almost every tile.
      // Normalising by the sum at the end makes the result independent of the reference point.
      const float m_seen = fmaxf(m, mx * p.scale_log2);      // a half that is wholly masked contributes -inf; the row is not
      const bool same = !(m_seen - m > 8.0f);                // first tile: m = -inf, the difference is +inf
      const float m_new = same ? m : m_seen;
      const float alpha = same ? 1.0f : ex2f(m - m_new);     // first tile: exp2(-inf) = 0
      // exponentials of this thread's 64 keys, rounded to the storage type as the tensor-core operand
      float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      uint32_t pk[32];
      if (!diag) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float e0 = ex2f(fmaf(__uint_as_float(r[2 * i]), p.scale_log2, -m_new));
          const float e1 = ex2f(fmaf(__uint_as_float(r[2 * i + 1]), p.scale_log2, -m_new));
          sum4[i & 3] += e0 + e1;
          pk[i] = pack2(e0, e1, bf16);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float e0 = ex2f(fmaf(__uint_as_float(r[2 * i]), p.scale_log2, -m_new));
          float e1 = ex2f(fmaf(__uint_as_float(r[2 * i + 1]), p.scale_log2, -m_new));
          e0 = 2 * i > lim ? 0.0f : e0;
          e1 = 2 * i + 1 > lim ? 0.0f : e1;
          sum4[i & 3] += e0 + e1;
          pk[i] = pack2(e0, e1, bf16);
        }
      }
      // this tile's P buffer was last read by P.V two tiles ago (this also bounds how far the softmax runs ahead)
      if (!mbar_wait(pv_done(sb), ((j >> 1) & 1) ^ 1, abort_flag, p.status, AT_ERR_SOFTMAX)) { ok = false; break; }
      // O is rescaled only when some row's maximum moved, and only then does the warp wait for the previous P.V
      if (j > 0 && !__all_sync(0xffffffffu, same)) {
        if (!mbar_wait(pv_done(sb ^ 1), ((j - 1) >> 1) & 1, abort_flag, p.status, AT_ERR_SOFTMAX)) { ok = false; break; }
        tc_fence_after();
#pragma unroll 1
        for (int ch = 0; ch < 2; ++ch) {                     // this thread's half of the 128 output columns
          uint32_t o[32];
          tmem_ld32(tmem_o + lane_addr + half * 64 + ch * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(tmem_o + lane_addr + half * 64 + ch * 32, o);
        }
        tmem_st_wait();
      }
      // 64 keys = the row's 128 bytes of k-block `half` of the P tile: eight 16-byte chunks, XOR-swizzled by the row
      uint8_t* p_row = base_ptr + AT_P_OFF + sb * AT_TILE + half * (AT_TILE / 2) + row * 128;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const uint32_t chunk = (uint32_t)q ^ (row & 7u);
        *reinterpret_cast<uint4*>(p_row + chunk * 16) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(sb));
      l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      m = m_new;
    }
    if (ok && mbar_wait(pv_done((n_kv - 1) & 1), ((n_kv - 1) >> 1) & 1, abort_flag, p.status, AT_ERR_SOFTMAX)) {
      tc_fence_after();
      float* xl = xchg + (n_kv & 1) * 256;                   // the parity the last tile did not use
      xl[half * 128 + row] = l;
      pair_sync();
      l += xl[(half ^ 1) * 128 + row];
      const float inv = 1.0f / l;
      const bool rn = p.rn != 0;
      const uint64_t grow = (uint64_t)qt * AT_BM + row;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.o) + (int64_t)b * p.stride_o_batch + (int64_t)grow * p.ldo + (int64_t)h * AT_D + half * 64;
#pragma unroll 1
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t o[32];
        tmem_ld32(tmem_o + lane_addr + half * 64 + ch * 32, o);
        tmem_ld_wait();
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float a = __uint_as_float(o[2 * i]) * inv, c = __uint_as_float(o[2 * i + 1]) * inv;
          const uint16_t lo = bf16 ? f32_to_bf16(a, rn) : f32_to_f16(a, rn), hi = bf16 ? f32_to_bf16(c, rn) : f32_to_f16(c, rn);
          w[i] = (uint32_t)lo | ((uint32_t)hi << 16);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(orow + ch * 32 + q * 8) = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
      }
      if (p.lse && half == 0) p.lse[(uint64_t)bh * p.T + grow] = (m + log2f(l)) * 0.6931471805599453f;   // ln sum exp(scale * s)
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
  // grid: x = (batch, head) pairs, y = 128-row tiles
  if (d.batch > 0x7fffffffull || d.heads > 0x7fffffffull || d.batch * d.heads > 0x7fffffffull) { err = "attention: too many (batch, head) pairs"; return ZYXB_ERR_KERNEL_COMPILATION; }
  if (d.seq / AT_BM > 65535) { err = "attention: seq too large (more than 65535 tiles of 128 rows)"; return ZYXB_ERR_KERNEL_COMPILATION; }
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
  if (attention_fwd2_supported(d)) return launch_attention_fwd2(d, args, lc, err);     // two query tiles per CTA
  const bool bf16 = d.dtype == ZYXB_BF16;
  CUtensorMap mq, mk, mv;
  const bool okm = encode_map(lc.tma_encode, &mq, bf16, args[0], d.head_dim, d.seq, ld, d.heads, d.head_dim, d.batch, d.seq * ld, AT_BM) &&
                   encode_map(lc.tma_encode, &mk, bf16, args[1], d.head_dim, d.seq, ld, d.heads, d.head_dim, d.batch, d.seq * ld, AT_BN) &&
                   encode_map(lc.tma_encode, &mv, bf16, args[2], d.head_dim, d.seq, ld, d.heads, d.head_dim, d.batch, d.seq * ld, 64);
  if (!okm) { err = "attention: cuTensorMapEncodeTiled rejected an operand"; return ZYXB_ERR_KERNEL_LAUNCH; }
  AttnParams p{};
  p.o = args[3]; p.lse = reinterpret_cast<float*>(args[4]);
  p.T = (uint32_t)d.seq; p.heads = (uint32_t)d.heads; p.ldo = (uint32_t)ld; p.stride_o_batch = (int64_t)(d.seq * ld);
  const float scale = d.scale > 0.0f ? d.scale : 1.0f / sqrtf((float)d.head_dim);
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = d.causal ? 1 : 0; p.rn = lc.round_nearest ? 1 : 0; p.is_bf16 = bf16 ? 1 : 0; p.status = lc.status_word;
  static uint64_t configured = 0;
  {
    cudaError_t e = ensure_dynamic_smem(attn_fwd_kernel, AT_SMEM_TOTAL, &configured);
    if (e != cudaSuccess) { err = std::string("attention: ") + cudaGetErrorString(e); return ZYXB_ERR_KERNEL_LAUNCH; }
  }
  const dim3 grid((unsigned)(d.batch * d.heads), (unsigned)(d.seq / AT_BM));
  attn_fwd_kernel<<<grid, AT_THREADS, AT_SMEM_TOTAL, lc.stream>>>(mq, mk, mv, p);
  return check_launch(lc, err, "attention");
}

}  // namespace zyxb
