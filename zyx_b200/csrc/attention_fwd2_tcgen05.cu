// Fused self-attention forward, persistent, two query tiles per CTA (used when seq is a multiple of 256; attention_tcgen05.cu otherwise).
//   O = softmax(scale * Q.K^T [causal mask]) . V            MultiheadAttention::forward, zyx-nn/src/multi_head_attention.rs:197-226
//
// What bounded the one-tile kernel was not arithmetic: with Q, two K, two V and two P tiles the shared memory was full, so the
// K/V rings were two deep against a load latency of thousands of clocks, every K/V tile was fetched from L2 once per 128 query
// rows, and P went through shared memory (a 32 KB write and a 32 KB operand read per tile on top of the products' own 128 KB).
// Here a work item is 256 query rows (tiles a and b) of one (batch, head), and one CTA per SM walks the items:
//   - every K_j / V_j tile is loaded once and used by both query tiles: half the L2 traffic and twice the work per ring slot;
//   - P never touches shared memory: the softmax writes it as packed 16-bit pairs over the first 64 columns of its own S tile
//     in TMEM, and P.V takes its A operand from TMEM (tcgen05.mma with a tensor-memory A);
//   - the two tiles ping-pong: while the softmax warps of one tile work on S_a, the tensor core computes S_b or P_b.V.
// TMEM (512 columns): S_a | S_b | O_a | O_b, 128 f32 columns each.  Shared memory: Q_a, Q_b, K x 2, V x 2 (192 KB).
// Roles (640 threads): warp 0 TMA producer, warp 1 issues every tensor-core product (S = Q.K^T and O += P.V of both tiles),
// warps 4..11 softmax of tile a, warps 12..19 softmax of tile b (two threads per query row, 64 keys each, as in the one-tile
// kernel); warps 2 and 3 only take part in the CTA-wide barriers.
// Per tile the chain S_g(j) -> softmax_g(j) -> P_g.V(j) -> S_g(j+1) is sequential (P overwrites S); the other tile fills the gaps.
// Items are numbered heaviest first (under a causal mask the late query rows visit the most key tiles) and dealt to the CTAs in
// rounds walked forwards and backwards in turn; the next item's Q, K_0, V_0 and first S products are under way while the softmax
// warps write the finished item's output (sixteen rows at a time through a shared-memory stage: coalesced stores).
// Measured on this chain (clock stamps of one CTA): S 890 clocks from issue until the softmax warps see it (512 of them the
// product), row maximum and its exchange 390, exponentials 1470 (the SFU alone would need 1024), store and publish 210, P.V 510.
// Variants that lost against this one: one thread per query row (no exchange, but one warp per scheduler cannot keep the SFU
// busy), P.V issued in four pieces as the exponentials complete (four barrier wake-ups cost more than the overlap gains),
// a separate issuing thread per tile (the tiles fall into step and want the tensor core, then the SFU, at the same time),
// busy polling with mbarrier.test_wait (steals issue slots from the other tile's softmax warps), a quarter of the
// exponentials as a packed cubic on the FMA pipe.
// Every mbarrier wait is time-bounded and reports through the device status word.
#include <cuda.h>
#include <math_constants.h>
#include <stdlib.h>

#include <algorithm>

#include "common.cuh"
#include "internal.h"
#include "tc_ptx.cuh"

namespace zyxb {

namespace {

constexpr int A2_BM = 128, A2_BN = 128, A2_D = 128;
constexpr int A2_THREADS = 640;
constexpr int A2_TILE = 128 * 128 * 2;                      // one 128 x 128 16-bit tile, 32 KB
constexpr int A2_Q_OFF = 0, A2_K_OFF = 2 * A2_TILE, A2_V_OFF = 4 * A2_TILE;
constexpr int A2_XCHG_OFF = 6 * A2_TILE;                    // [2 tiles][2 parities][2 halves][128 rows] f32 = 4 KB
constexpr int A2_STAGE_OFF = A2_XCHG_OFF + 4096;            // output staging: 16 softmax warps x (16 rows x 80 B: 64 B of data + padding)
constexpr int A2_STAGE_WARP = 16 * 80;
constexpr int A2_BAR_OFF = A2_STAGE_OFF + 16 * A2_STAGE_WARP;
constexpr int A2_SMEM_TOTAL = A2_BAR_OFF + 256;
enum { A2_ERR_PRODUCER = 16u, A2_ERR_MMA = 32u, A2_ERR_SOFTMAX = 64u, A2_ERR_ALIGN = 1024u };

struct Attn2Params {
  void* o; float* lse;
  uint32_t T, heads;
  uint32_t ldo;
  int64_t stride_o_batch;
  float scale_log2;
  int causal, rn, is_bf16;
  uint32_t n_bh;                // batch * heads
  uint32_t* status;
};

// D[tmem] (+)= A[tmem] . B[smem]: the A operand is read from tensor memory (128 lanes = rows, two 16-bit k-elements per column)
__device__ __forceinline__ void umma_f16_tmem_a(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// Clock stamps of the CTA with blockIdx.x == 0, for tuning (compiled in with -DZYXB_ATTN_TRACE, read back through
// zyxb_debug_attn_trace): role 0 the producer (index = work item), role 1 the issuing thread (index = key tile of this CTA),
// roles 3 / 4 lane 0 of the first softmax warp of each query tile; eight stamps per index, the first 32 indices.
#ifdef ZYXB_ATTN_TRACE
__device__ unsigned long long a2_trace[8192];
#define TR(role, j, k) do { if (blockIdx.x == 0 && (j) < 32) a2_trace[((role) * 32 + (j)) * 8 + (k)] = clock64(); } while (0)
#else
#define TR(role, j, k) do {} while (0)
#endif

// One thread's 64 scores of a tile -> P = 2^(s*scale - m) as 32 packed pairs of the 16-bit type, and their sum.  The
// multiply-subtract and the sum run two lanes per instruction (fma.rn.f32x2 / add.rn.f32x2); the exponentials are one SFU
// operation each.  DIAG: keys beyond `lim` (above the diagonal) give exactly zero.
template <bool BF16, bool DIAG>
__device__ __forceinline__ float exp_tile(const uint32_t (&r)[64], float scale, float neg_m, int32_t lim, uint32_t (&pk)[32]) {
  const uint64_t sc = f2_pack(scale, scale), nm = f2_pack(neg_m, neg_m);
  uint64_t acc[2] = {f2_pack(0.0f, 0.0f), f2_pack(0.0f, 0.0f)};
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float a, b;
    f2_unpack(f2_fma(f2_pack_bits(r[2 * i], r[2 * i + 1]), sc, nm), a, b);
    float e0 = ex2f(a), e1 = ex2f(b);
    if (DIAG) {
      e0 = 2 * i > lim ? 0.0f : e0;
      e1 = 2 * i + 1 > lim ? 0.0f : e1;
    }
    acc[i & 1] = f2_add(acc[i & 1], f2_pack(e0, e1));
    pk[i] = pack2_t<BF16>(e0, e1);
  }
  float s0, s1;
  f2_unpack(f2_add(acc[0], acc[1]), s0, s1);
  return s0 + s1;
}

__global__ void __launch_bounds__(A2_THREADS, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, Attn2Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {
    if (threadIdx.x == 0) atomicOr(p.status, A2_ERR_ALIGN);
    return;
  }
  uint8_t* base_ptr = smem_raw;
  const uint32_t bar = base + A2_BAR_OFF;
  const uint32_t q_full = bar;
  auto k_full = [&](int s) { return bar + 8u * (1 + s); };
  auto v_full = [&](int s) { return bar + 8u * (3 + s); };
  auto k_empty = [&](int s) { return bar + 8u * (5 + s); };    // both tiles' S products of the K tile in stage s have finished
  auto v_empty = [&](int s) { return bar + 8u * (7 + s); };    // both tiles' P.V products of the V tile in stage s have finished
  auto s_full = [&](int g) { return bar + 8u * (9 + g); };     // S_g(j) is in TMEM
  auto p_full = [&](int g) { return bar + 8u * (11 + g); };    // P_g(j) is in TMEM (and O_g rescaled if it had to be)
  auto pv_done = [&](int g) { return bar + 8u * (13 + g); };   // P_g.V(j) has finished: S_g / P_g may be overwritten, O_g is current
  const uint32_t q_empty = bar + 8u * 15;                      // every S product of a work item has finished: its Q tiles may be overwritten
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + A2_BAR_OFF + 8 * 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // A work item is one (batch, head, 256 query rows).  Items are numbered heaviest first (under a causal mask the late query
  // rows visit the most key tiles; all (batch, head) pairs of one query block, then the next lighter block) and a CTA takes
  // one item of every round of gridDim.x items: with one CTA per SM every SM gets the same mix, the load of the next
  // item's Q, K_0 and V_0 and its first S products run under the previous item's last softmax and its output stores, and
  // barriers, TMEM and tensor maps are set up once.  All barrier phases are counted across items (tile counters).
  const uint32_t n_super = p.T / (2 * A2_BM), n_items = n_super * p.n_bh;
  // the i-th item of this CTA: rounds of gridDim.x items, walked forwards and backwards in turn, so that the CTA that took the
  // heaviest item of one round takes the lightest of the next (plain strides gave the first CTA 70 key tiles and the last 54)
  auto nth_item = [&](uint32_t i) { return i * gridDim.x + ((i & 1) ? gridDim.x - 1 - blockIdx.x : blockIdx.x); };
  auto item_qs = [&](uint32_t item) { const uint32_t y = item / p.n_bh; return p.causal ? n_super - 1 - y : y; };
  auto item_bh = [&](uint32_t item) { return item % p.n_bh; };
  // key tiles query tile g of block qs visits: tile a = 2*qs sees 0 .. 2*qs, tile b = 2*qs + 1 sees one more
  auto kv_tiles = [&](uint32_t qs, int g) { return p.causal ? 2 * qs + 1 + (uint32_t)g : p.T / A2_BN; };

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full(s), 1); mbar_init(v_full(s), 1); mbar_init(k_empty(s), 1); mbar_init(v_empty(s), 1);
      mbar_init(s_full(s), 1); mbar_init(p_full(s), 8); mbar_init(pv_done(s), 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  constexpr uint32_t TMEM_COLS = 512;
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  auto tmem_s = [&](int g) { return tmem_base + (uint32_t)g * A2_BN; };
  auto tmem_o = [&](int g) { return tmem_base + 2 * A2_BN + (uint32_t)g * A2_D; };

  if (warp == 0) {
    // ---------------------------------- TMA producer ----------------------------------
    if (lane == 0) {
      uint32_t t = 0, it = 0, q_issued = 0;                  // K / V tiles and items issued so far by this CTA
      bool ok = true;
      for (uint32_t item = nth_item(0); item < n_items && ok; item = nth_item(++it)) {
        const uint32_t qs = item_qs(item), bh = item_bh(item), b = bh / p.heads, h = bh % p.heads;
        if (it > 0 && !mbar_wait(q_empty, (it - 1) & 1, abort_flag, p.status, A2_ERR_PRODUCER)) { ok = false; break; }
        TR(0, it, 0);
        mbar_expect_tx(q_full, 2 * A2_TILE);
        for (int g = 0; g < 2; ++g)
          for (int c = 0; c < 2; ++c)
            tma_load_4d(base + A2_Q_OFF + g * A2_TILE + c * (A2_TILE / 2), &map_q, q_full, c * 64, (int)((2 * qs + g) * A2_BM), (int)h, (int)b);
        ++q_issued;
        const uint32_t n_kv = kv_tiles(qs, 1);
        for (uint32_t j = 0; j < n_kv; ++j, ++t) {
          const int s = (int)(t & 1);
          const uint32_t free_parity = ((t >> 1) & 1) ^ 1;
          if (!mbar_wait(k_empty(s), free_parity, abort_flag, p.status, A2_ERR_PRODUCER)) { ok = false; break; }
          mbar_expect_tx(k_full(s), A2_TILE);
          for (int c = 0; c < 2; ++c)
            tma_load_4d(base + A2_K_OFF + s * A2_TILE + c * (A2_TILE / 2), &map_k, k_full(s), c * 64, (int)(j * A2_BN), (int)h, (int)b);
          if (!mbar_wait(v_empty(s), free_parity, abort_flag, p.status, A2_ERR_PRODUCER)) {
            // K of this tile is in flight: wait (bounded) for it below like for the others
            ok = false; ++t; break;
          }
          mbar_expect_tx(v_full(s), A2_TILE);
          for (int kb = 0; kb < 2; ++kb)
            for (int c = 0; c < 2; ++c)
              tma_load_4d(base + A2_V_OFF + s * A2_TILE + kb * (A2_TILE / 2) + c * (A2_TILE / 4), &map_v, v_full(s), c * 64,
                          (int)(j * A2_BN) + kb * 64, (int)h, (int)b);
        }
      }
      if (!ok) {   // drain: wait (bounded) for copies still in flight so none lands after the CTA has gone
        const uint64_t t0 = global_timer_ns();
        for (uint32_t i = 0; i < 2 && i < t; ++i) {
          const uint32_t j = t - 1 - i;
          while (!mbar_try_wait(k_full(j & 1), (j >> 1) & 1) && global_timer_ns() - t0 < TC_WAIT_NS) {}
          while (!mbar_try_wait(v_full(j & 1), (j >> 1) & 1) && global_timer_ns() - t0 < TC_WAIT_NS) {}
        }
        if (q_issued) while (!mbar_try_wait(q_full, (q_issued - 1) & 1) && global_timer_ns() - t0 < TC_WAIT_NS) {}
      }
    }
  } else if (warp == 1) {
    // ---------------------------------- every tensor-core product of the CTA ----------------------------------
    // One thread issues S_a(0), S_b(0) and then, per key tile, P_a.V, S_a(next), P_b.V, S_b(next).  The tensor core executes
    // one thread's products in issue order, so S_g(j+1), which overwrites P_g(j), needs no barrier between it and P_g(j).V:
    // it is queued right behind it.  The fixed alternation also keeps the two tiles half a period apart.
    if (lane == 0) {
      const bool bf16 = p.is_bf16 != 0;
      const uint32_t idesc_s = make_idesc(bf16, false, false, A2_BM, A2_BN);
      const uint32_t idesc_pv = make_idesc(bf16, false, true, A2_BM, A2_D);     // P (from TMEM, K-major) x V (N-major)
      auto issue_s = [&](int g, int s) {
        const uint32_t q_addr = base + A2_Q_OFF + g * A2_TILE, k_addr = base + A2_K_OFF + s * A2_TILE;
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(tmem_s(g), make_smem_desc(q_addr + c * (A2_TILE / 2) + kk * 32, 16, 1024),
                     make_smem_desc(k_addr + c * (A2_TILE / 2) + kk * 32, 16, 1024), idesc_s, (c | kk) != 0 ? 1u : 0u);
        umma_commit(s_full(g));
      };
      uint32_t t0 = 0, it = 0, done[2] = {0, 0};             // key tiles of earlier items; items; per query tile: P tiles of earlier items
      bool ok = true;
      for (uint32_t item = nth_item(0); item < n_items && ok; item = nth_item(++it)) {
        const uint32_t qs = item_qs(item);
        const uint32_t n_g[2] = {kv_tiles(qs, 0), kv_tiles(qs, 1)}, n_kv = n_g[1];
        if (!mbar_wait(q_full, it & 1, abort_flag, p.status, A2_ERR_MMA) ||
            !mbar_wait(k_full((int)(t0 & 1)), (t0 >> 1) & 1, abort_flag, p.status, A2_ERR_MMA)) { ok = false; break; }
        tc_fence_after();
        issue_s(0, (int)(t0 & 1));
        issue_s(1, (int)(t0 & 1));
        umma_commit(k_empty((int)(t0 & 1)));
        if (n_kv == 1) umma_commit(q_empty);
        for (uint32_t j = 0; j < n_kv && ok; ++j) {
          const uint32_t t = t0 + j;
          const int s = (int)(t & 1), sn = s ^ 1;
          if (!mbar_wait(v_full(s), (t >> 1) & 1, abort_flag, p.status, A2_ERR_MMA)) { ok = false; break; }
          TR(1, t, 0);
          bool k_ready = false, s_issued = false;
          for (int g = 0; g < 2 && ok; ++g) {
            if (j >= n_g[g]) continue;
            if (!mbar_wait(p_full(g), (done[g] + j) & 1, abort_flag, p.status, A2_ERR_MMA)) { ok = false; break; }
            tc_fence_after();
            TR(1, t, 1 + g);
            const uint32_t v_addr = base + A2_V_OFF + s * A2_TILE;
#pragma unroll
            for (int kb = 0; kb < 2; ++kb)       // 64 keys per k-block of V
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)     // 16 keys per instruction = 8 columns of packed P
                umma_f16_tmem_a(tmem_o(g), tmem_s(g) + (uint32_t)(kb * 32 + kk * 8),
                                make_smem_desc(v_addr + kb * (A2_TILE / 2) + kk * (16 * 128), A2_TILE / 4, 1024), idesc_pv,
                                (j != 0 || (kb | kk) != 0) ? 1u : 0u);
            umma_commit(pv_done(g));
            if (j + 1 < n_g[g]) {
              if (!k_ready && !mbar_wait(k_full(sn), ((t + 1) >> 1) & 1, abort_flag, p.status, A2_ERR_MMA)) { ok = false; break; }
              k_ready = true;
              tc_fence_after();
              issue_s(g, sn);
              s_issued = true;
            }
          }
          if (!ok) break;
          umma_commit(v_empty(s));
          if (s_issued) umma_commit(k_empty(sn));
          if (j + 2 == n_kv) umma_commit(q_empty);           // the item's last S product (tile b, key tile n_kv - 1) has just been issued
          TR(1, t, 3);
        }
        t0 += n_kv; done[0] += n_g[0]; done[1] += n_g[1];
      }
    }
  } else if (warp >= 4) {
    // ---------------------------------- softmax warps ----------------------------------
    const int g = (warp - 4) >> 3;                           // which query tile
    const uint32_t quarter = (uint32_t)(warp & 3);           // TMEM lanes this warp may access
    const int half = ((warp - 4) >> 2) & 1;                  // keys 0..63 or 64..127 of a tile
    const uint32_t row = quarter * 32 + lane;
    const uint32_t lane_addr = (quarter * 32u) << 16;
    const bool bf16 = p.is_bf16 != 0;
    float* xchg = reinterpret_cast<float*>(base_ptr + A2_XCHG_OFF) + g * 512;       // [2 parities][2 halves][128 rows]
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + g * 4 + (int)quarter) : "memory"); };
    uint32_t cnt = 0;                                        // key tiles this query tile has processed in earlier items
    bool ok = true;
    for (uint32_t it = 0, item = nth_item(0); item < n_items && ok; item = nth_item(++it)) {
      const uint32_t qs = item_qs(item), bh = item_bh(item), b = bh / p.heads, h = bh % p.heads;
      const uint32_t qt = 2 * qs + (uint32_t)g;              // this group's query tile
      const uint32_t my_kv = kv_tiles(qs, g);
      float m = -CUDART_INF_F, l = 0.0f;
      for (uint32_t j = 0; j < my_kv && ok; ++j) {
        const uint32_t c = cnt + j;
        if (!mbar_wait(s_full(g), c & 1, abort_flag, p.status, A2_ERR_SOFTMAX)) { ok = false; break; }
        tc_fence_after();
        const bool tr = quarter == 0 && half == 0 && lane == 0;
        if (tr) TR(3 + g, c, 0);
        uint32_t r[64];
        {
          uint32_t (&r0)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[0]);
          uint32_t (&r1)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[32]);
          tmem_ld32(tmem_s(g) + lane_addr + half * 64, r0);
          tmem_ld32(tmem_s(g) + lane_addr + half * 64 + 32, r1);
        }
        tmem_ld_wait();
        tc_fence_before();                                     // the partner's P store below overwrites columns this thread has just read
        const bool diag = p.causal && j == qt;
        const int32_t lim = (int32_t)row - half * 64;
        float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
        if (!diag) {
#pragma unroll
          for (int i = 0; i < 64; i += 2) mx4[(i >> 1) & 3] = fmax3(mx4[(i >> 1) & 3], __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
        } else {
#pragma unroll
          for (int i = 0; i < 64; ++i) mx4[i & 3] = i > lim ? mx4[i & 3] : fmaxf(mx4[i & 3], __uint_as_float(r[i]));
        }
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        float* xm = xchg + (c & 1) * 256;
        xm[half * 128 + row] = mx;
        pair_sync();                                           // also: both halves hold their scores in registers, P may overwrite S
        tc_fence_after();
        mx = fmaxf(mx, xm[(half ^ 1) * 128 + row]);
        // lazy reference point (see attention_tcgen05.cu): it moves only when the maximum grew by more than 2^8 beyond it
        const float m_seen = fmaxf(m, mx * p.scale_log2);
        const bool same = !(m_seen - m > 8.0f);
        const float m_new = same ? m : m_seen;
        const float alpha = same ? 1.0f : ex2f(m - m_new);
        uint32_t pk[32];
        const float tile_sum = bf16 ? (diag ? exp_tile<true, true>(r, p.scale_log2, -m_new, lim, pk) : exp_tile<true, false>(r, p.scale_log2, -m_new, lim, pk))
                                    : (diag ? exp_tile<false, true>(r, p.scale_log2, -m_new, lim, pk) : exp_tile<false, false>(r, p.scale_log2, -m_new, lim, pk));
        // O_g is rescaled only when some row's reference point moved; the previous P_g.V has finished by then (S_g(j) was
        // issued after it), the wait only makes that visible to this thread
        if (j > 0 && !__all_sync(0xffffffffu, same)) {
          if (!mbar_wait(pv_done(g), (c - 1) & 1, abort_flag, p.status, A2_ERR_SOFTMAX)) { ok = false; break; }
          tc_fence_after();
#pragma unroll 1
          for (int ch = 0; ch < 2; ++ch) {
            uint32_t o[32];
            tmem_ld32(tmem_o(g) + lane_addr + half * 64 + ch * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(tmem_o(g) + lane_addr + half * 64 + ch * 32, o);
          }
        }
        // P_g: 64 keys = 32 packed columns, over the first 64 columns of S_g (keys 64*half ..)
        tmem_st32(tmem_s(g) + lane_addr + half * 32, pk);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full(g));
        if (tr) TR(3 + g, c, 1);
        l = l * alpha + tile_sum;
        m = m_new;
      }
      if (!ok || !mbar_wait(pv_done(g), (cnt + my_kv - 1) & 1, abort_flag, p.status, A2_ERR_SOFTMAX)) { ok = false; break; }
      tc_fence_after();
      if (quarter == 0 && half == 0 && lane == 0) TR(3 + g, cnt + my_kv - 1, 2);
      float* xl = xchg + ((cnt + my_kv) & 1) * 256;          // the parity the last tile did not use
      xl[half * 128 + row] = l;
      pair_sync();
      l += xl[(half ^ 1) * 128 + row];
      pair_sync();                                           // the next item's first tile writes its maxima into this slot
      const float inv = 1.0f / l;
      const bool rn = p.rn != 0;
      const uint64_t grow = (uint64_t)qt * A2_BM + row;
      // Output: a thread holds 64 consecutive values of its own row, so a plain store would touch 32 rows per instruction.
      // Sixteen rows at a time go through a small shared-memory stage and leave as eight rows x 64 contiguous bytes per
      // store instruction (a quarter of the memory transactions).
      uint16_t* obase = reinterpret_cast<uint16_t*>(p.o) + (int64_t)b * p.stride_o_batch + (int64_t)((uint64_t)qt * A2_BM + quarter * 32) * p.ldo +
                        (int64_t)h * A2_D + half * 64;
      uint8_t* stage = base_ptr + A2_STAGE_OFF + (warp - 4) * A2_STAGE_WARP;
#pragma unroll 1
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t o[32];
        tmem_ld32(tmem_o(g) + lane_addr + half * 64 + ch * 32, o);
        tmem_ld_wait();
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float a = __uint_as_float(o[2 * i]) * inv, c = __uint_as_float(o[2 * i + 1]) * inv;
          const uint16_t lo = bf16 ? f32_to_bf16(a, rn) : f32_to_f16(a, rn), hi = bf16 ? f32_to_bf16(c, rn) : f32_to_f16(c, rn);
          w[i] = (uint32_t)lo | ((uint32_t)hi << 16);
        }
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
          if ((lane >> 4) == pass) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
              *reinterpret_cast<uint4*>(stage + (lane & 15) * 80 + q * 16) = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int r16 = (lane >> 2) + 8 * i, chunk = lane & 3;
            const uint4 val = *reinterpret_cast<const uint4*>(stage + r16 * 80 + chunk * 16);
            *reinterpret_cast<uint4*>(obase + (int64_t)(pass * 16 + r16) * p.ldo + ch * 32 + chunk * 8) = val;
          }
          __syncwarp();
        }
      }
      if (p.lse && half == 0) p.lse[(uint64_t)bh * p.T + grow] = (m + log2f(l)) * 0.6931471805599453f;
      if (quarter == 0 && half == 0 && lane == 0) TR(3 + g, cnt + my_kv - 1, 3);
      // O_g has been read: the next item's first P_g.V (which overwrites it) is only issued after this warp's next arrival on p_full
      tc_fence_before();
      cnt += my_kv;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace

#ifdef ZYXB_ATTN_TRACE
extern "C" __attribute__((visibility("default"))) int zyxb_debug_attn_trace(unsigned long long* out, int n) {
  return (int)cudaMemcpyFromSymbol(out, a2_trace, sizeof(unsigned long long) * n);
}
#endif
bool attention_fwd2_supported(const zyxb_attention_desc& d) {
  static const bool off = getenv("ZYXB_ATTENTION_ONE_TILE") != nullptr;
  return !off && d.seq % (2 * A2_BM) == 0;
}

int launch_attention_fwd2(const zyxb_attention_desc& d, void* const* args, const LaunchCtx& lc, std::string& err) {
  const uint64_t E = d.heads * d.head_dim, ld = d.ld ? d.ld : E;
  const bool bf16 = d.dtype == ZYXB_BF16;
  CUtensorMap mq, mk, mv;
  const bool okm = encode_map(lc.tma_encode, &mq, bf16, args[0], d.head_dim, d.seq, ld, d.heads, d.head_dim, d.batch, d.seq * ld, A2_BM) &&
                   encode_map(lc.tma_encode, &mk, bf16, args[1], d.head_dim, d.seq, ld, d.heads, d.head_dim, d.batch, d.seq * ld, A2_BN) &&
                   encode_map(lc.tma_encode, &mv, bf16, args[2], d.head_dim, d.seq, ld, d.heads, d.head_dim, d.batch, d.seq * ld, 64);
  if (!okm) { err = "attention: cuTensorMapEncodeTiled rejected an operand"; return ZYXB_ERR_KERNEL_LAUNCH; }
  Attn2Params p{};
  p.o = args[3]; p.lse = reinterpret_cast<float*>(args[4]);
  p.T = (uint32_t)d.seq; p.heads = (uint32_t)d.heads; p.ldo = (uint32_t)ld; p.stride_o_batch = (int64_t)(d.seq * ld);
  const float scale = d.scale > 0.0f ? d.scale : 1.0f / sqrtf((float)d.head_dim);
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = d.causal ? 1 : 0; p.rn = lc.round_nearest ? 1 : 0; p.is_bf16 = bf16 ? 1 : 0; p.status = lc.status_word;
  static uint64_t configured = 0;
  {
    cudaError_t e = ensure_dynamic_smem(attn_fwd2_kernel, A2_SMEM_TOTAL, &configured);
    if (e != cudaSuccess) { err = std::string("attention: ") + cudaGetErrorString(e); return ZYXB_ERR_KERNEL_LAUNCH; }
  }
  p.n_bh = (uint32_t)(d.batch * d.heads);
  const uint64_t n_items = (uint64_t)p.n_bh * (d.seq / (2 * A2_BM));
  if (n_items > 0x7fffffffull) { err = "attention: too many work items"; return ZYXB_ERR_INCORRECT_KERNEL_ARG; }
  // one CTA per SM walks the items (ZYXB_ATTENTION_CTA_PER_ITEM: one CTA per item, as many CTAs as items)
  static const bool per_item = getenv("ZYXB_ATTENTION_CTA_PER_ITEM") != nullptr;
  const unsigned grid = (unsigned)(per_item ? n_items : std::min<uint64_t>(n_items, (uint64_t)lc.sm_count));
  attn_fwd2_kernel<<<grid, A2_THREADS, A2_SMEM_TOTAL, lc.stream>>>(mq, mk, mv, p);
  return check_launch(lc, err, "attention");
}

}  // namespace zyxb
