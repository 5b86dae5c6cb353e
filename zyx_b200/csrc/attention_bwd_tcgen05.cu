// Fused self-attention backward on the 5th-generation tensor cores.  Given q, k, v, the forward's o and log-sum-exp, and
// the upstream gradient dO, it produces dq, dk, dv without materialising the [T, T] probabilities or their gradient:
//   P = exp(scale * Q.K^T - lse)   dV = P^T.dO   dP = dO.V^T   dS = P * (dP - delta) * scale   dQ = dS.K   dK = dS^T.Q
// with delta_i = sum_d dO_id * O_id.  It is the adjoint of the subgraph of MultiheadAttention::forward between the
// projections (zyx-nn/src/multi_head_attention.rs:197-226), which zyx's autograd (zyx/src/graph/autograd.rs:14-424) would
// emit as four matmuls and a softmax adjoint over the stored probabilities.
//
// Three launches:
//   attn_delta_kernel      delta [B*H, T] f32
//   attn_bwd_dq_kernel     work item = one 128-query tile: loops over key tiles of 64; S and dP in TMEM (lane = query),
//                          dS to shared memory as the A operand of dQ += dS.K_j
//   attn_bwd_dkdv_kernel   work item = one 128-key tile: loops over query tiles of 64; S^T = K.Q^T and dP^T = V.dO^T in TMEM
//                          (lane = key), P^T and dS^T to shared memory as the A operands of dV += P^T.dO_i, dK += dS^T.Q_i
// Both tensor-core kernels are persistent: one CTA per SM walks the work items (see the comments at their heads).
// Each kernel recomputes S and dP (7 tensor-core products per tile pair instead of 5) so that no accumulator is shared
// between CTAs: no atomics, no reduction pass, bit-reproducible results.
// One shared-memory image of a [rows, 128] tile (two 128-byte-swizzled boxes of 64 columns) serves both as a K-major
// operand (contraction over the 128 columns) and as an MN-major B operand (contraction over the rows): only the
// descriptor differs.  352 threads: warp 0 TMA producer, warps 1 and 10 MMA issuers (the recomputed scores / the gradient
// accumulations: issuing an instruction occupies its thread about as long as the tensor core executes it, so two threads
// issue side by side), warps 2..9 elementwise (two warps per TMEM lane quarter, each taking half of the columns).  Every mbarrier wait is time-bounded and reports through the status word.
#include <cuda.h>
#include <math_constants.h>

#include <algorithm>

#include "common.cuh"
#include "internal.h"
#include "tc_ptx.cuh"

namespace zyxb {

constexpr int AB_THREADS = 352, AB_EW_WARPS = 8;   // barriers the elementwise warps signal count warps: one lane arrives per warp
constexpr int AB_BIG = 128 * 128 * 2;        // [128 rows x 128 d] tile, 32 KB
constexpr int AB_SMALL = 64 * 128 * 2;       // [64 rows x 128 d] tile, 16 KB
constexpr int AB_PT = 128 * 64 * 2;          // [128 rows x 64] probability / dS tile, 16 KB
enum { AB_ERR_PRODUCER = 128u, AB_ERR_MMA = 256u, AB_ERR_EW = 512u };

struct AttnBwdParams {
  void* dq; void* dk; void* dv;
  const float* lse; const float* delta;
  uint32_t T, heads, ld;
  int64_t stride_batch;         // elements between batches of the [B, T, H*D] activations
  float scale, scale_log2;
  int causal, rn, is_bf16;
  uint32_t n_bh;                // batch * heads
  uint32_t* status;
};

// ---- delta = rowsum(dO * O) ------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) attn_delta_kernel(const uint16_t* __restrict__ o, const uint16_t* __restrict__ dO, float* delta,
                                                         uint32_t B, uint32_t T, uint32_t H, uint32_t ld, int is_bf16) {
  const uint64_t w = (uint64_t)blockIdx.x * 8 + (threadIdx.x >> 5);       // one warp per (b, t, h)
  const uint32_t lane = threadIdx.x & 31;
  if (w >= (uint64_t)B * T * H) return;
  const uint32_t h = (uint32_t)(w % H);
  const uint64_t bt = w / H;
  const uint32_t t = (uint32_t)(bt % T), b = (uint32_t)(bt / T);
  const uint64_t off = bt * ld + (uint64_t)h * 128 + lane * 4;
  const uint2 a = *reinterpret_cast<const uint2*>(o + off), g = *reinterpret_cast<const uint2*>(dO + off);
  auto lo = [&](uint32_t x) { return is_bf16 ? __uint_as_float(x << 16) : f16_to_f32((uint16_t)(x & 0xffffu)); };
  auto hi = [&](uint32_t x) { return is_bf16 ? __uint_as_float(x & 0xffff0000u) : f16_to_f32((uint16_t)(x >> 16)); };
  float acc = lo(a.x) * lo(g.x) + hi(a.x) * hi(g.x) + lo(a.y) * lo(g.y) + hi(a.y) * hi(g.y);
  acc = warp_reduce(acc, OpSum());
  if (lane == 0) delta[((uint64_t)b * H + h) * T + t] = acc;
}

// 32 f32 values of a row (one TMEM chunk) leave as 32 16-bit values = 64 bytes.  The lanes of a warp hold 32 consecutive rows: a plain store would touch 32 rows per instruction, so sixteen rows
// at a time go through a 1280-byte shared-memory stage (rows of 64 B, padded to 80) and leave as eight rows x 64 contiguous
// bytes per store instruction - a quarter of the memory transactions.  `out_row0`: the warp's first row at this chunk's column.
__device__ __forceinline__ void store_rows_staged(uint8_t* stage, uint16_t* out_row0, int64_t ld, const uint32_t (&r)[32], bool bf16, bool rn, int lane) {
  uint32_t w[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float a = __uint_as_float(r[2 * i]), c = __uint_as_float(r[2 * i + 1]);
    const uint16_t lo = bf16 ? f32_to_bf16(a, rn) : f32_to_f16(a, rn), hi = bf16 ? f32_to_bf16(c, rn) : f32_to_f16(c, rn);
    w[i] = (uint32_t)lo | ((uint32_t)hi << 16);
  }
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    if ((lane >> 4) == pass) {
#pragma unroll
      for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(stage + (lane & 15) * 80 + q * 16) = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r16 = (lane >> 2) + 8 * i, chunk = lane & 3;
      const uint4 val = *reinterpret_cast<const uint4*>(stage + r16 * 80 + chunk * 16);
      *reinterpret_cast<uint4*>(out_row0 + (int64_t)(pass * 16 + r16) * ld + chunk * 8) = val;
    }
    __syncwarp();
  }
}
// write 32 packed columns (16 words) of row `row` into a [128 x 64] K-major swizzled tile; `half` selects columns 0..31 / 32..63
__device__ __forceinline__ void write_tile_row(uint8_t* tile, uint32_t row, int half, const uint32_t (&pk)[16]) {
  uint8_t* p_row = tile + row * 128;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint32_t chunk = (uint32_t)(half * 4 + q) ^ (row & 7u);
    *reinterpret_cast<uint4*>(p_row + chunk * 16) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
  }
}

// ---- dQ ----------------------------------------------------------------------------------------------------
namespace dqk {
constexpr int NS = 4;                      // K_j / V_j stages: a tile is requested three iterations before its first use
constexpr int Q_OFF = 0, DO_OFF = AB_BIG, KV_OFF = 2 * AB_BIG, STAGE = 2 * AB_SMALL, DS_OFF = KV_OFF + NS * STAGE;
constexpr int BAR_OFF = DS_OFF + 2 * AB_PT, SMEM_TOTAL = BAR_OFF + 256 + 1024;   // dS is double-buffered
}  // namespace dqk

__global__ void __launch_bounds__(AB_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                   const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, AttnBwdParams p) {
  using namespace dqk;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t bar = base + BAR_OFF;
  const uint32_t qdo_full = bar;
  auto kv_full = [&](int s) { return bar + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bar + 8u * (1 + NS + s); };
  auto sdp_full = [&](int b) { return bar + 8u * (1 + 2 * NS + b); };
  auto sdp_empty = [&](int b) { return bar + 8u * (3 + 2 * NS + b); };
  // barriers of double-buffered tiles exist once per buffer: a role that runs a tile ahead can then never complete two
  // phases of one barrier before its waiter has seen the first
  auto ds_full = [&](int b) { return bar + 8u * (5 + 2 * NS + b); };
  auto ds_empty = [&](int b) { return bar + 8u * (7 + 2 * NS + b); };
  const uint32_t qdo_empty = bar + 8u * (9 + 2 * NS);                // every S / dP product of a work item has finished: Q and dO may be overwritten
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + BAR_OFF + 8 * (10 + 2 * NS));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Persistent: a work item is one (batch, head, 128-query tile); items are numbered heaviest first (late query rows visit the
  // most key tiles under a causal mask; all (batch, head) pairs of one query tile, then the next lighter tile) and dealt to
  // the CTAs - one per SM - in rounds walked forwards and backwards in turn.  Barriers, TMEM and tensor maps are set up once,
  // every ring and double-buffer phase is counted in key tiles across items, and the next item's Q, dO, first K / V tiles and
  // first S / dP products are under way while the elementwise warps write the finished item's dQ.
  const uint32_t n_qt = p.T / 128, n_items = n_qt * p.n_bh;
  auto nth_item = [&](uint32_t i) { return i * gridDim.x + ((i & 1) ? gridDim.x - 1 - blockIdx.x : blockIdx.x); };
  auto item_qt = [&](uint32_t item) { const uint32_t y = item / p.n_bh; return p.causal ? n_qt - 1 - y : y; };
  auto item_bh = [&](uint32_t item) { return item % p.n_bh; };
  auto kv_tiles = [&](uint32_t qt) { return p.causal ? (qt + 1) * 2 : p.T / 64; };

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    mbar_init(qdo_empty, 1);
    for (int s = 0; s < NS; ++s) { mbar_init(kv_full(s), 1); mbar_init(kv_empty(s), 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(sdp_full(s), 1); mbar_init(sdp_empty(s), AB_EW_WARPS); }
    for (int s = 0; s < 2; ++s) { mbar_init(ds_full(s), AB_EW_WARPS); mbar_init(ds_empty(s), 1); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  constexpr uint32_t TMEM_COLS = 512;      // S0 S1 (64 each) | dP0 dP1 (64 each) | dQ (128)
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_dq = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t t = 0, it = 0;                                 // K / V tiles and items issued so far by this CTA
      bool ok = true;
      for (uint32_t item = nth_item(0); item < n_items && ok; item = nth_item(++it)) {
        const uint32_t qt = item_qt(item), bh = item_bh(item), b = bh / p.heads, h = bh % p.heads;
        if (it > 0 && !mbar_wait(qdo_empty, (it - 1) & 1, abort_flag, p.status, AB_ERR_PRODUCER)) { ok = false; break; }
        mbar_expect_tx(qdo_full, 2 * AB_BIG);
        for (int c = 0; c < 2; ++c) {
          tma_load_4d(base + Q_OFF + c * (AB_BIG / 2), &map_q, qdo_full, c * 64, (int)(qt * 128), (int)h, (int)b);
          tma_load_4d(base + DO_OFF + c * (AB_BIG / 2), &map_do, qdo_full, c * 64, (int)(qt * 128), (int)h, (int)b);
        }
        const uint32_t n_kv = kv_tiles(qt);
        for (uint32_t j = 0; j < n_kv; ++j, ++t) {
          const int s = (int)(t % NS);
          if (!mbar_wait(kv_empty(s), ((t / NS) & 1) ^ 1, abort_flag, p.status, AB_ERR_PRODUCER)) { ok = false; break; }
          const uint32_t k_dst = base + KV_OFF + s * STAGE, v_dst = k_dst + AB_SMALL;
          mbar_expect_tx(kv_full(s), 2 * AB_SMALL);
          for (int c = 0; c < 2; ++c) {
            tma_load_4d(k_dst + c * (AB_SMALL / 2), &map_k, kv_full(s), c * 64, (int)(j * 64), (int)h, (int)b);
            tma_load_4d(v_dst + c * (AB_SMALL / 2), &map_v, kv_full(s), c * 64, (int)(j * 64), (int)h, (int)b);
          }
        }
      }
      if (!ok) {   // drain: wait (bounded) for the copies still in flight so none lands after the CTA has gone
        const uint64_t t_start = global_timer_ns();
        for (uint32_t i = 0; i < NS && i < t; ++i) {
          const uint32_t j = t - 1 - i;
          while (!mbar_try_wait(kv_full(j % NS), (j / NS) & 1) && global_timer_ns() - t_start < TC_WAIT_NS) {}
        }
        // Q / dO of the item being set up when a wait failed (item number `it`) may still be in flight
        while (!mbar_try_wait(qdo_full, it & 1) && global_timer_ns() - t_start < 100000000ull) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const bool bf16 = p.is_bf16 != 0;
      const uint32_t idesc_s = make_idesc(bf16, false, false, 128, 64);      // [128 q x d] x [64 keys x d]^T
      auto issue_sdp = [&](uint32_t j) {      // j: key tile counted across this CTA's items
        const uint32_t k_addr = base + KV_OFF + (j % NS) * STAGE, v_addr = k_addr + AB_SMALL;
        const uint32_t t_s = tmem_base + (j & 1) * 64, t_dp = tmem_base + 128 + (j & 1) * 64;
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(t_s, make_smem_desc(base + Q_OFF + c * (AB_BIG / 2) + kk * 32, 16, 1024),
                     make_smem_desc(k_addr + c * (AB_SMALL / 2) + kk * 32, 16, 1024), idesc_s, (c | kk) != 0 ? 1u : 0u);
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(t_dp, make_smem_desc(base + DO_OFF + c * (AB_BIG / 2) + kk * 32, 16, 1024),
                     make_smem_desc(v_addr + c * (AB_SMALL / 2) + kk * 32, 16, 1024), idesc_s, (c | kk) != 0 ? 1u : 0u);
        umma_commit(sdp_full(j & 1));
      };
      uint32_t t = 0, it = 0;
      bool ok = true;
      for (uint32_t item = nth_item(0); item < n_items && ok; item = nth_item(++it)) {
        const uint32_t n_kv = kv_tiles(item_qt(item));
        if (!mbar_wait(qdo_full, it & 1, abort_flag, p.status, AB_ERR_MMA)) { ok = false; break; }
        for (uint32_t j = 0; j < n_kv && ok; ++j, ++t) {
          if (!mbar_wait(kv_full(t % NS), (t / NS) & 1, abort_flag, p.status, AB_ERR_MMA)) { ok = false; break; }
          if (!mbar_wait(sdp_empty(t & 1), ((t >> 1) & 1) ^ 1, abort_flag, p.status, AB_ERR_MMA)) { ok = false; break; }
          tc_fence_after();
          issue_sdp(t);
        }
        if (ok) umma_commit(qdo_empty);
      }
    }
  } else if (warp == 10) {
    // second MMA issuer (issuing an instruction costs its thread about as long as the tensor core needs to execute it):
    // dQ += dS_j . K_j, while warp 1 issues the scores of the next tiles
    if (lane == 0) {
      const uint32_t idesc_dq = make_idesc(p.is_bf16 != 0, false, true, 128, 128);     // dS [128 q x 64 keys] x K_j [64 keys x d]
      uint32_t t = 0, it = 0;
      bool ok = true;
      for (uint32_t item = nth_item(0); item < n_items && ok; item = nth_item(++it)) {
        const uint32_t n_kv = kv_tiles(item_qt(item));
        // the item's first product overwrites dQ: the elementwise warps have read the previous item's dQ before they arrive on
        // ds_full for this item's first tile (program order in every one of them)
        for (uint32_t j = 0; j < n_kv && ok; ++j, ++t) {
          if (!mbar_wait(ds_full(t & 1), (t >> 1) & 1, abort_flag, p.status, AB_ERR_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t k_addr = base + KV_OFF + (t % NS) * STAGE;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)     // 16 keys per instruction; K_j read MN-major: rows of 128 B, the two d chunks 8 KB apart
            umma_f16(tmem_dq, make_smem_desc(base + DS_OFF + (t & 1) * AB_PT + kk * 32, 16, 1024),
                     make_smem_desc(k_addr + kk * (16 * 128), AB_SMALL / 2, 1024), idesc_dq, (j != 0 || kk != 0) ? 1u : 0u);
          umma_commit(kv_empty(t % NS));
          umma_commit(ds_empty(t & 1));
        }
      }
    }
  } else {
    const uint32_t quarter = (uint32_t)(warp & 3);
    const int half = (warp - 2) >> 2;
    const uint32_t row = quarter * 32 + lane;
    const uint32_t lane_addr = (quarter * 32u) << 16;
    const bool bf16 = p.is_bf16 != 0;
    uint32_t t0 = 0;
    bool ok = true;
    for (uint32_t it = 0, item = nth_item(0); item < n_items && ok; item = nth_item(++it)) {
      const uint32_t qt = item_qt(item), bh = item_bh(item), b = bh / p.heads, h = bh % p.heads, n_kv = kv_tiles(qt);
      const uint32_t grow = qt * 128 + row;
      const float lse2 = p.lse[(uint64_t)bh * p.T + grow] * 1.4426950408889634f;
      const float dl = p.delta[(uint64_t)bh * p.T + grow];
      for (uint32_t j = 0; j < n_kv && ok; ++j) {
        const uint32_t t = t0 + j, sb = t & 1;
        if (!mbar_wait(sdp_full(sb), (t >> 1) & 1, abort_flag, p.status, AB_ERR_EW)) { ok = false; break; }
        tc_fence_after();
        uint32_t s[32], d[32];
        tmem_ld32(tmem_base + lane_addr + sb * 64 + half * 32, s);
        tmem_ld32(tmem_base + lane_addr + 128 + sb * 64 + half * 32, d);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sdp_empty(sb));
        const int32_t key0 = (int32_t)(j * 64 + half * 32);
        const bool diag = p.causal && key0 + 31 > (int32_t)grow;
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = ex2f(fmaf(__uint_as_float(s[2 * i]), p.scale_log2, -lse2));
          float p1 = ex2f(fmaf(__uint_as_float(s[2 * i + 1]), p.scale_log2, -lse2));
          if (diag) {
            p0 = key0 + 2 * i > (int32_t)grow ? 0.0f : p0;
            p1 = key0 + 2 * i + 1 > (int32_t)grow ? 0.0f : p1;
          }
          const float g0 = p0 * (__uint_as_float(d[2 * i]) - dl) * p.scale, g1 = p1 * (__uint_as_float(d[2 * i + 1]) - dl) * p.scale;
          pk[i] = pack2(g0, g1, bf16);
        }
        if (!mbar_wait(ds_empty(sb), ((t >> 1) & 1) ^ 1, abort_flag, p.status, AB_ERR_EW)) { ok = false; break; }   // read two tiles ago
        write_tile_row(base_ptr + DS_OFF + sb * AB_PT, row, half, pk);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(ds_full(sb));
      }
      const uint32_t t_last = t0 + n_kv - 1;
      if (!ok || !mbar_wait(ds_empty(t_last & 1), (t_last >> 1) & 1, abort_flag, p.status, AB_ERR_EW)) { ok = false; break; }
      tc_fence_after();
      // every dS tile of the item has been written and consumed: that shared memory serves as the output stage
      uint16_t* out0 = reinterpret_cast<uint16_t*>(p.dq) + (int64_t)b * p.stride_batch + (int64_t)(qt * 128 + quarter * 32) * p.ld + (int64_t)h * 128 + half * 64;
      uint8_t* stage = base_ptr + DS_OFF + (warp - 2) * 1280;
#pragma unroll 1
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t r[32];
        tmem_ld32(tmem_dq + lane_addr + half * 64 + ch * 32, r);
        tmem_ld_wait();
        store_rows_staged(stage, out0 + ch * 32, (int64_t)p.ld, r, bf16, p.rn != 0, lane);
      }
      tc_fence_before();
      // no warp writes the next item's dS while another still stages its output rows in that memory
      asm volatile("bar.sync 1, %0;" ::"n"(AB_EW_WARPS * 32) : "memory");
      t0 += n_kv;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- dK, dV ------------------------------------------------------------------------------------------------
namespace dkv {
constexpr int NS = 3;                      // Q_i / dO_i stages
constexpr int K_OFF = 0, V_OFF = AB_BIG, QDO_OFF = 2 * AB_BIG, STAGE = 2 * AB_SMALL, PT_OFF = QDO_OFF + NS * STAGE, DST_OFF = PT_OFF + 2 * AB_PT;
constexpr int BAR_OFF = DST_OFF + 2 * AB_PT, SMEM_TOTAL = BAR_OFF + 256 + 1024;   // P^T and dS^T are double-buffered
}  // namespace dkv

__global__ void __launch_bounds__(AB_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                     const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, AttnBwdParams p) {
  using namespace dkv;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t bar = base + BAR_OFF;
  const uint32_t kv_full = bar;
  auto qdo_full = [&](int s) { return bar + 8u * (1 + s); };
  auto qdo_empty = [&](int s) { return bar + 8u * (1 + NS + s); };
  auto sdp_full = [&](int b) { return bar + 8u * (1 + 2 * NS + b); };
  auto sdp_empty = [&](int b) { return bar + 8u * (3 + 2 * NS + b); };
  auto pt_full = [&](int b) { return bar + 8u * (5 + 2 * NS + b); };
  auto dst_full = [&](int b) { return bar + 8u * (7 + 2 * NS + b); };
  auto pt_empty = [&](int b) { return bar + 8u * (9 + 2 * NS + b); };
  auto dst_empty = [&](int b) { return bar + 8u * (11 + 2 * NS + b); };
  const uint32_t kv_empty = bar + 8u * (13 + 2 * NS);                // every S^T / dP^T product of a work item has finished: K and V may be overwritten
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + BAR_OFF + 8 * (14 + 2 * NS));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Persistent like the dQ kernel: a work item is one (batch, head, 128-key tile), numbered head by head (item = head * tiles +
  // key tile), so that the CTAs running at one time work on a few heads and meet in L2 on their Q and dO; one CTA per SM takes
  // one item of every round of gridDim.x, the rounds walked forwards and backwards in turn, which also mixes heavy (early) and
  // light (late) key tiles evenly.  Ring and double-buffer phases are counted in query tiles across items.
  const uint32_t n_kt = p.T / 128, n_items = n_kt * p.n_bh;
  auto nth_item = [&](uint32_t i) { return i * gridDim.x + ((i & 1) ? gridDim.x - 1 - blockIdx.x : blockIdx.x); };
  auto item_kt = [&](uint32_t item) { return item % n_kt; };               // key tile; early tiles are the heavy ones under a causal mask
  auto item_bh = [&](uint32_t item) { return item / n_kt; };
  auto first_q = [&](uint32_t kt) { return p.causal ? kt * 2 : 0u; };     // first 64-query tile that sees these keys

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(kv_empty, 1);
    for (int s = 0; s < NS; ++s) { mbar_init(qdo_full(s), 1); mbar_init(qdo_empty(s), 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(sdp_full(s), 1); mbar_init(sdp_empty(s), AB_EW_WARPS); }
    for (int s = 0; s < 2; ++s) {
      mbar_init(pt_full(s), AB_EW_WARPS); mbar_init(dst_full(s), AB_EW_WARPS); mbar_init(pt_empty(s), 1); mbar_init(dst_empty(s), 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  constexpr uint32_t TMEM_COLS = 512;      // S^T0 S^T1 (64 each) | dP^T0 dP^T1 (64 each) | dV (128) | dK (128)
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_dv = tmem_base + 256, tmem_dk = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t t = 0, it = 0;                                 // Q / dO tiles and items issued so far by this CTA
      bool ok = true;
      for (uint32_t item = nth_item(0); item < n_items && ok; item = nth_item(++it)) {
        const uint32_t kt = item_kt(item), bh = item_bh(item), b = bh / p.heads, h = bh % p.heads;
        const uint32_t i_first = first_q(kt), n_q = p.T / 64 - i_first;
        if (it > 0 && !mbar_wait(kv_empty, (it - 1) & 1, abort_flag, p.status, AB_ERR_PRODUCER)) { ok = false; break; }
        mbar_expect_tx(kv_full, 2 * AB_BIG);
        for (int c = 0; c < 2; ++c) {
          tma_load_4d(base + K_OFF + c * (AB_BIG / 2), &map_k, kv_full, c * 64, (int)(kt * 128), (int)h, (int)b);
          tma_load_4d(base + V_OFF + c * (AB_BIG / 2), &map_v, kv_full, c * 64, (int)(kt * 128), (int)h, (int)b);
        }
        for (uint32_t i = 0; i < n_q; ++i, ++t) {
          const int s = (int)(t % NS);
          if (!mbar_wait(qdo_empty(s), ((t / NS) & 1) ^ 1, abort_flag, p.status, AB_ERR_PRODUCER)) { ok = false; break; }
          const uint32_t q_dst = base + QDO_OFF + s * STAGE, do_dst = q_dst + AB_SMALL;
          mbar_expect_tx(qdo_full(s), 2 * AB_SMALL);
          for (int c = 0; c < 2; ++c) {
            tma_load_4d(q_dst + c * (AB_SMALL / 2), &map_q, qdo_full(s), c * 64, (int)((i_first + i) * 64), (int)h, (int)b);
            tma_load_4d(do_dst + c * (AB_SMALL / 2), &map_do, qdo_full(s), c * 64, (int)((i_first + i) * 64), (int)h, (int)b);
          }
        }
      }
      if (!ok) {   // drain: wait (bounded) for the copies still in flight so none lands after the CTA has gone
        const uint64_t t_start = global_timer_ns();
        for (uint32_t k = 0; k < NS && k < t; ++k) {
          const uint32_t i = t - 1 - k;
          while (!mbar_try_wait(qdo_full(i % NS), (i / NS) & 1) && global_timer_ns() - t_start < TC_WAIT_NS) {}
        }
        // K / V of the item being set up when a wait failed (item number `it`) may still be in flight
        while (!mbar_try_wait(kv_full, it & 1) && global_timer_ns() - t_start < 100000000ull) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const bool bf16 = p.is_bf16 != 0;
      const uint32_t idesc_st = make_idesc(bf16, false, false, 128, 64);     // [128 keys x d] x [64 q x d]^T
      auto issue_sdp = [&](uint32_t i) {      // i: query tile counted across this CTA's items
        const uint32_t q_addr = base + QDO_OFF + (i % NS) * STAGE, do_addr = q_addr + AB_SMALL;
        const uint32_t t_s = tmem_base + (i & 1) * 64, t_dp = tmem_base + 128 + (i & 1) * 64;
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(t_s, make_smem_desc(base + K_OFF + c * (AB_BIG / 2) + kk * 32, 16, 1024),
                     make_smem_desc(q_addr + c * (AB_SMALL / 2) + kk * 32, 16, 1024), idesc_st, (c | kk) != 0 ? 1u : 0u);
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(t_dp, make_smem_desc(base + V_OFF + c * (AB_BIG / 2) + kk * 32, 16, 1024),
                     make_smem_desc(do_addr + c * (AB_SMALL / 2) + kk * 32, 16, 1024), idesc_st, (c | kk) != 0 ? 1u : 0u);
        umma_commit(sdp_full(i & 1));
      };
      uint32_t t = 0, it = 0;
      bool ok = true;
      for (uint32_t item = nth_item(0); item < n_items && ok; item = nth_item(++it)) {
        const uint32_t n_q = p.T / 64 - first_q(item_kt(item));
        if (!mbar_wait(kv_full, it & 1, abort_flag, p.status, AB_ERR_MMA)) { ok = false; break; }
        for (uint32_t i = 0; i < n_q && ok; ++i, ++t) {
          if (!mbar_wait(qdo_full(t % NS), (t / NS) & 1, abort_flag, p.status, AB_ERR_MMA)) { ok = false; break; }
          if (!mbar_wait(sdp_empty(t & 1), ((t >> 1) & 1) ^ 1, abort_flag, p.status, AB_ERR_MMA)) { ok = false; break; }
          tc_fence_after();
          issue_sdp(t);
        }
        if (ok) umma_commit(kv_empty);
      }
    }
  } else if (warp == 10) {
    // second MMA issuer: dV += P^T . dO_i and dK += dS^T . Q_i, while warp 1 issues the scores of the next tiles
    if (lane == 0) {
      const uint32_t idesc_acc = make_idesc(p.is_bf16 != 0, false, true, 128, 128);    // [128 keys x 64 q] x [64 q x d]
      uint32_t t = 0, it = 0;
      bool ok = true;
      for (uint32_t item = nth_item(0); item < n_items && ok; item = nth_item(++it)) {
        const uint32_t n_q = p.T / 64 - first_q(item_kt(item));
        // the item's first products overwrite dV and dK: the elementwise warps have read the previous item's before they arrive
        // on pt_full / dst_full for this item's first tile (program order in every one of them)
        for (uint32_t i = 0; i < n_q && ok; ++i, ++t) {
          const uint32_t q_addr = base + QDO_OFF + (t % NS) * STAGE, do_addr = q_addr + AB_SMALL;
          if (!mbar_wait(pt_full(t & 1), (t >> 1) & 1, abort_flag, p.status, AB_ERR_MMA)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)     // dV += P^T . dO_i, 16 queries per instruction, dO_i read MN-major
            umma_f16(tmem_dv, make_smem_desc(base + PT_OFF + (t & 1) * AB_PT + kk * 32, 16, 1024),
                     make_smem_desc(do_addr + kk * (16 * 128), AB_SMALL / 2, 1024), idesc_acc, (i != 0 || kk != 0) ? 1u : 0u);
          umma_commit(pt_empty(t & 1));
          if (!mbar_wait(dst_full(t & 1), (t >> 1) & 1, abort_flag, p.status, AB_ERR_MMA)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)     // dK += dS^T . Q_i
            umma_f16(tmem_dk, make_smem_desc(base + DST_OFF + (t & 1) * AB_PT + kk * 32, 16, 1024),
                     make_smem_desc(q_addr + kk * (16 * 128), AB_SMALL / 2, 1024), idesc_acc, (i != 0 || kk != 0) ? 1u : 0u);
          umma_commit(qdo_empty(t % NS));
          umma_commit(dst_empty(t & 1));
        }
      }
    }
  } else {
    const uint32_t quarter = (uint32_t)(warp & 3);
    const int half = (warp - 2) >> 2;
    const uint32_t row = quarter * 32 + lane;                               // key row of the tile
    const uint32_t lane_addr = (quarter * 32u) << 16;
    const bool bf16 = p.is_bf16 != 0;
    uint32_t t0 = 0;
    bool ok = true;
    for (uint32_t it = 0, item = nth_item(0); item < n_items && ok; item = nth_item(++it)) {
      const uint32_t kt = item_kt(item), bh = item_bh(item), b = bh / p.heads, h = bh % p.heads;
      const uint32_t i_first = first_q(kt), n_q = p.T / 64 - i_first;
      const int32_t gkey = (int32_t)(kt * 128 + row);
      const float* lse_bh = p.lse + (uint64_t)bh * p.T;
      const float* delta_bh = p.delta + (uint64_t)bh * p.T;
      for (uint32_t i = 0; i < n_q && ok; ++i) {
        const uint32_t t = t0 + i, sb = t & 1;
        if (!mbar_wait(sdp_full(sb), (t >> 1) & 1, abort_flag, p.status, AB_ERR_EW)) { ok = false; break; }
        tc_fence_after();
        uint32_t s[32], d[32];
        tmem_ld32(tmem_base + lane_addr + sb * 64 + half * 32, s);
        tmem_ld32(tmem_base + lane_addr + 128 + sb * 64 + half * 32, d);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sdp_empty(sb));
        const int32_t q0 = (int32_t)((i_first + i) * 64 + half * 32);         // first query of this thread's 32 columns
        const bool diag = p.causal && q0 < gkey;                              // some of them precede the key
        uint32_t pk[16];
        float pr[32];
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          const float4 l4 = __ldg(reinterpret_cast<const float4*>(lse_bh + q0) + c4);
          const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = c4 * 4 + e;
            float v = ex2f(fmaf(__uint_as_float(s[c]), p.scale_log2, -lv[e] * 1.4426950408889634f));
            if (diag) v = q0 + c < gkey ? 0.0f : v;
            pr[c] = v;
          }
        }
#pragma unroll
        for (int i2 = 0; i2 < 16; ++i2) pk[i2] = pack2(pr[2 * i2], pr[2 * i2 + 1], bf16);
        if (!mbar_wait(pt_empty(sb), ((t >> 1) & 1) ^ 1, abort_flag, p.status, AB_ERR_EW)) { ok = false; break; }   // read two tiles ago
        write_tile_row(base_ptr + PT_OFF + sb * AB_PT, row, half, pk);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(pt_full(sb));
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          const float4 d4 = __ldg(reinterpret_cast<const float4*>(delta_bh + q0) + c4);
          const float dv4[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = c4 * 4 + e;
            pr[c] = pr[c] * (__uint_as_float(d[c]) - dv4[e]) * p.scale;
          }
        }
#pragma unroll
        for (int i2 = 0; i2 < 16; ++i2) pk[i2] = pack2(pr[2 * i2], pr[2 * i2 + 1], bf16);
        if (!mbar_wait(dst_empty(sb), ((t >> 1) & 1) ^ 1, abort_flag, p.status, AB_ERR_EW)) { ok = false; break; }
        write_tile_row(base_ptr + DST_OFF + sb * AB_PT, row, half, pk);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(dst_full(sb));
      }
      const uint32_t t_last = t0 + n_q - 1;
      if (!ok || !mbar_wait(dst_empty(t_last & 1), (t_last >> 1) & 1, abort_flag, p.status, AB_ERR_EW)) { ok = false; break; }
      tc_fence_after();
      // every dS^T tile of the item has been written and consumed (and dV's last product was issued before dK's): that
      // shared memory serves as the output stage
      const int64_t off = (int64_t)b * p.stride_batch + (int64_t)(gkey - (int32_t)lane) * p.ld + (int64_t)h * 128 + half * 64;   // the warp's first row
      uint16_t* out_v = reinterpret_cast<uint16_t*>(p.dv) + off;
      uint16_t* out_k = reinterpret_cast<uint16_t*>(p.dk) + off;
      uint8_t* stage = base_ptr + DST_OFF + (warp - 2) * 1280;
#pragma unroll 1
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t r[32];
        tmem_ld32(tmem_dv + lane_addr + half * 64 + ch * 32, r);
        tmem_ld_wait();
        store_rows_staged(stage, out_v + ch * 32, (int64_t)p.ld, r, bf16, p.rn != 0, lane);
        tmem_ld32(tmem_dk + lane_addr + half * 64 + ch * 32, r);
        tmem_ld_wait();
        store_rows_staged(stage, out_k + ch * 32, (int64_t)p.ld, r, bf16, p.rn != 0, lane);
      }
      tc_fence_before();
      // no warp writes the next item's dS^T while another still stages its output rows in that memory
      asm volatile("bar.sync 1, %0;" ::"n"(AB_EW_WARPS * 32) : "memory");
      t0 += n_q;
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
int launch_attention_bwd(const zyxb_attention_desc& d, void* const* args, const uint64_t* arg_bytes, int n_args, const LaunchCtx& lc,
                         std::string& err) {
  ZYXB_CHECK_ARG(n_args == 9, "attention backward: expected args q, k, v, o, do, lse -> dq, dk, dv");
  ZYXB_CHECK_ARG(lc.tma_encode != nullptr, "attention backward: no tensor-map encoder (driver entry point missing)");
  const uint64_t E = d.heads * d.head_dim, ld = d.ld ? d.ld : E;
  ZYXB_CHECK_ARG(ld >= E && ld % 8 == 0, "attention backward: row pitch must cover heads*head_dim and be a multiple of 8 elements");
  const uint64_t need = ((d.batch * d.seq - 1) * ld + E) * 2, n_rows = d.batch * d.heads * d.seq;
  for (int i : {0, 1, 2, 3, 4, 6, 7, 8}) {
    ZYXB_CHECK_ARG(arg_bytes[i] >= need, "attention backward: an activation or gradient buffer is too small");
    ZYXB_CHECK_ARG((uintptr_t)args[i] % 16 == 0, "attention backward: operands must be 16-byte aligned");
  }
  ZYXB_CHECK_ARG(arg_bytes[5] >= n_rows * 4 && (uintptr_t)args[5] % 16 == 0, "attention backward: lse too small or misaligned");
  ZYXB_CHECK_ARG(lc.scratch_bytes >= n_rows * 4, "attention backward: batch*heads*seq exceeds the scratch buffer");
  const bool bf16 = d.dtype == ZYXB_BF16;
  float* delta = reinterpret_cast<float*>(lc.scratch);
  attn_delta_kernel<<<(unsigned)((n_rows + 7) / 8), 256, 0, lc.stream>>>(reinterpret_cast<const uint16_t*>(args[3]),
                                                                          reinterpret_cast<const uint16_t*>(args[4]), delta, (uint32_t)d.batch,
                                                                          (uint32_t)d.seq, (uint32_t)d.heads, (uint32_t)ld, bf16 ? 1 : 0);
  auto map = [&](CUtensorMap* m, const void* ptr, uint32_t rows) {
    return encode_map(lc.tma_encode, m, bf16, ptr, d.head_dim, d.seq, ld, d.heads, d.head_dim, d.batch, d.seq * ld, rows);
  };
  CUtensorMap q128, do128, k64, v64, q64, do64, k128, v128;
  const bool okm = map(&q128, args[0], 128) && map(&do128, args[4], 128) && map(&k64, args[1], 64) && map(&v64, args[2], 64) &&
                   map(&q64, args[0], 64) && map(&do64, args[4], 64) && map(&k128, args[1], 128) && map(&v128, args[2], 128);
  if (!okm) { err = "attention backward: cuTensorMapEncodeTiled rejected an operand"; return ZYXB_ERR_KERNEL_LAUNCH; }
  AttnBwdParams p{};
  p.dq = args[6]; p.dk = args[7]; p.dv = args[8];
  p.lse = reinterpret_cast<const float*>(args[5]); p.delta = delta;
  p.T = (uint32_t)d.seq; p.heads = (uint32_t)d.heads; p.ld = (uint32_t)ld; p.stride_batch = (int64_t)(d.seq * ld);
  p.scale = d.scale > 0.0f ? d.scale : 1.0f / sqrtf((float)d.head_dim);
  p.scale_log2 = p.scale * 1.4426950408889634f;
  p.causal = d.causal ? 1 : 0; p.rn = lc.round_nearest ? 1 : 0; p.is_bf16 = bf16 ? 1 : 0; p.status = lc.status_word;
  static uint64_t configured_dq = 0, configured_dkdv = 0;
  {
    cudaError_t e = ensure_dynamic_smem(attn_bwd_dq_kernel, dqk::SMEM_TOTAL, &configured_dq);
    if (e == cudaSuccess) e = ensure_dynamic_smem(attn_bwd_dkdv_kernel, dkv::SMEM_TOTAL, &configured_dkdv);
    if (e != cudaSuccess) { err = std::string("attention backward: ") + cudaGetErrorString(e); return ZYXB_ERR_KERNEL_LAUNCH; }
  }
  // Both kernels are persistent: one CTA per SM walks the (batch, head, tile) items (ZYXB_ATTENTION_CTA_PER_ITEM: one CTA per
  // item).  dQ numbers its items heaviest query tile first; dK/dV head by head, so that the CTAs running at one time meet in
  // L2 on the Q and dO of a few heads (with one CTA per key tile, heads in the slow grid dimension measured 0.800 ms per
  // backward against 0.847 with heads in the fast one).
  p.n_bh = (uint32_t)(d.batch * d.heads);
  const uint64_t n_items = (uint64_t)p.n_bh * (d.seq / 128);
  if (n_items > 0x7fffffffull) { err = "attention backward: too many work items"; return ZYXB_ERR_INCORRECT_KERNEL_ARG; }
  static const bool per_item = getenv("ZYXB_ATTENTION_CTA_PER_ITEM") != nullptr;
  const unsigned grid_dq = (unsigned)(per_item ? n_items : std::min<uint64_t>(n_items, (uint64_t)lc.sm_count));
  attn_bwd_dq_kernel<<<grid_dq, AB_THREADS, dqk::SMEM_TOTAL, lc.stream>>>(q128, do128, k64, v64, p);
  attn_bwd_dkdv_kernel<<<grid_dq, AB_THREADS, dkv::SMEM_TOTAL, lc.stream>>>(q64, do64, k128, v128, p);
  return check_launch(lc, err, "attention backward", 3);
}

}  // namespace zyxb
