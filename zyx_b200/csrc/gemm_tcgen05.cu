// bf16 / f16 matmul on the 5th-generation tensor cores: tcgen05.mma accumulating f32 in TMEM,
// operands staged by TMA into 128-byte-swizzled shared memory, mbarrier pipeline.
//   C[b] = epi(alpha * op(A[b]) . op(B[b]) + bias)        Tensor::dot, zyx/src/tensor/mod.rs:1469-1490
// Products of bf16/f16 inputs are exact in f32 and the accumulator is f32, which is what the
// reference C backend computes (zyx/src/codegen/c.rs:616-629, reduce_ops.rs:52-60); only the
// summation order differs.
//
// One persistent CTA per SM, 320 threads:
//   warp 0      TMA producer   (one lane): fills a ring of STAGES {A tile, B tile} slots
//   warp 1      MMA issuer     (one lane): tcgen05.mma 128 x BN x 16 per instruction, 4 per k-block;
//                               tcgen05.commit releases the slot, and the accumulator when a tile is done
//   warps 2..9  epilogue       : tcgen05.ld the 128 x BN f32 accumulator (lane = row; two warps per TMEM
//                               lane quarter, each taking half of the columns), apply alpha / bias / ReLU /
//                               GELU / activation gradient, convert and store 64 bytes per thread per chunk
// The accumulator is double-buffered in TMEM (2 x BN columns) so the epilogue of tile i overlaps
// the MMAs of tile i+1.  Operands may be K-major (rows of K) or MN-major (rows of M or N) in
// memory: all four transposition cases of the descriptor are served without a transpose pass.
// Every CTA loads its own tiles with plain per-CTA TMA loads; no thread-block clusters are used.
//
// Every wait on an mbarrier is bounded by wall-clock time; a wait that runs out sets a bit in
// the device status word, raises the CTA's abort flag and the kernel drains and returns.
#include <cuda.h>

#include <stdlib.h>

#include <algorithm>

#include "common.cuh"
#include "eltwise_math.cuh"
#include "gemm.h"
#include "tc_ptx.cuh"

namespace zyxb {

constexpr int TC_BM = 128;          // UMMA M (cta_group::1): TMEM lane = row of the tile
constexpr int TC_BK = 64;           // 64 x 2 bytes = one 128-byte swizzle atom along K
constexpr int TC_UMMA_K = 16;
constexpr int TC_THREADS = 320;
constexpr int TC_EPI_THREADS = 256;

struct TcParams {
  const void* bias; const void* z; void* c; void* preact;
  uint32_t m, n, k, batch;
  uint32_t tiles_m, tiles_n;
  int64_t stride_c, stride_c_inner;   // elements between outer / inner batches of C
  uint32_t ldc;           // row pitch of C (and of z / preact), elements
  uint32_t batch_inner;   // matrix z = (z / batch_inner, z % batch_inner)
  float alpha;
  int epilogue;
  int rn;
  int is_bf16;
  int a_batched, b_batched;   // bit 0: the operand has an outer batch stride, bit 1: an inner one (else that map extent is 1)
  uint32_t* status;
  uint32_t* tile_counter;     // zeroed before the launch; CTAs draw tile indices from it
  int dynamic_tiles;          // 1: draw tiles from the counter; 0: CTA i takes tiles i, i + grid, ...
  int tri;                    // ZYXB_TRI_*: tiles above the diagonal are skipped / the k range of a tile is cut at it
};

template <int BN, int STAGES>
struct TcSmem {
  static constexpr int A_BYTES = TC_BM * TC_BK * 2;
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;   // + barriers + slack to align the base to 1024 B
};

enum { TC_ERR_PRODUCER = 1u, TC_ERR_MMA = 2u, TC_ERR_EPILOGUE = 4u };

template <bool A_MN, bool B_MN, int BN, int STAGES>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, TcParams p) {
  using SM = TcSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;          // swizzle atoms repeat every 1024 B
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t bar_base = base + SM::BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  // tile queue: the producer draws tile indices from a global counter and hands them to the MMA issuer
  // and the epilogue warps, so a CTA that starts late (SMs busy with a collective) simply takes fewer tiles
  constexpr int TQ = 4;
  constexpr uint32_t TILE_NONE = 0xffffffffu;
  auto tq_full = [&](int i) { return bar_base + 8u * (2 * STAGES + 4 + i); };
  auto tq_empty = [&](int i) { return bar_base + 8u * (2 * STAGES + 4 + TQ + i); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + SM::BAR_OFFSET + 8 * (2 * STAGES + 4 + 2 * TQ));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile uint32_t* tile_q = reinterpret_cast<volatile uint32_t*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * BN;                  // two accumulator buffers (power of two >= 32)

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), TC_EPI_THREADS); }
    for (int i = 0; i < TQ; ++i) { mbar_init(tq_full(i), 1); mbar_init(tq_empty(i), 1 + TC_EPI_THREADS); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const uint32_t tiles_per_batch = p.tiles_m * p.tiles_n;
  const uint32_t total_tiles = tiles_per_batch * p.batch;
  const uint32_t k_blocks = (p.k + TC_BK - 1) / TC_BK;
  constexpr uint32_t GROUP_M = 16;   // tiles that run together share A and B panels in L2
  auto tile_coords = [&](uint32_t t, uint32_t& bz, uint32_t& tm, uint32_t& tn) {
    bz = t / tiles_per_batch;
    const uint32_t r = t % tiles_per_batch;
    const uint32_t group_size = GROUP_M * p.tiles_n;
    const uint32_t g = r / group_size, first_m = g * GROUP_M;
    const uint32_t rows_in_group = min(GROUP_M, p.tiles_m - first_m);
    const uint32_t in_group = r % group_size;
    tm = first_m + in_group % rows_in_group;
    tn = in_group / rows_in_group;
  };
  // causal structure: is the tile wholly above the diagonal of a lower-triangular result, and which k-blocks of a
  // lower-triangular A (or of its transpose) can be non-zero for the rows of this tile
  auto tile_skipped = [&](uint32_t tm, uint32_t tn) { return p.tri == ZYXB_TRI_OUT_LOWER && tn * BN > tm * TC_BM + (TC_BM - 1); };
  auto k_range = [&](uint32_t tm, uint32_t& kb0, uint32_t& kb1) {
    kb0 = 0; kb1 = k_blocks;
    if (p.tri == ZYXB_TRI_A_LOWER) kb1 = min(k_blocks, ((tm + 1) * TC_BM + TC_BK - 1) / TC_BK);
    else if (p.tri == ZYXB_TRI_AT_LOWER) kb0 = min(k_blocks - 1, (tm * TC_BM) / TC_BK);
  };
  // consumer side of the tile queue (MMA issuer and every epilogue thread keep their own cursor)
  uint32_t tq_slot = 0, tq_phase = 0;
  auto next_tile = [&](uint32_t code) -> uint32_t {
    if (!mbar_wait(tq_full(tq_slot), tq_phase, abort_flag, p.status, code)) return TILE_NONE;
    const uint32_t t = tile_q[tq_slot];
    mbar_arrive(tq_empty(tq_slot));
    if (++tq_slot == TQ) { tq_slot = 0; tq_phase ^= 1; }
    return t;
  };

  if (warp == 0) {
    // ---------------------------------- TMA producer ----------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      uint32_t issued = 0;
      bool ok = true;
      // the index of the tile after this one is drawn while this one's loads are issued, so the round trip of
      // the atomic never stalls the ring
      uint32_t t_next = p.dynamic_tiles ? atomicAdd(p.tile_counter, 1u) : blockIdx.x;
      while (ok) {
        // publish the tile (a slot is free once the MMA issuer and all epilogue threads have read it)
        if (!mbar_wait(tq_empty(tq_slot), tq_phase ^ 1, abort_flag, p.status, TC_ERR_PRODUCER)) { ok = false; break; }
        uint32_t t, bz = 0, tm = 0, tn = 0;
        for (;;) {   // draw until a tile that has work (tiles above a causal diagonal are never published)
          t = t_next;
          if (t >= total_tiles) { t = TILE_NONE; break; }
          t_next = p.dynamic_tiles ? atomicAdd(p.tile_counter, 1u) : t + gridDim.x;
          tile_coords(t, bz, tm, tn);
          if (!tile_skipped(tm, tn)) break;
        }
        tile_q[tq_slot] = t;
        mbar_arrive(tq_full(tq_slot));
        if (++tq_slot == TQ) { tq_slot = 0; tq_phase ^= 1; }
        if (t == TILE_NONE) break;
        uint32_t kb0, kb1;
        k_range(tm, kb0, kb1);
        const int zo = (int)(bz / p.batch_inner), zi = (int)(bz % p.batch_inner);
        const int zao = p.a_batched & 1 ? zo : 0, zai = p.a_batched & 2 ? zi : 0;
        const int zbo = p.b_batched & 1 ? zo : 0, zbi = p.b_batched & 2 ? zi : 0;
        for (uint32_t kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, p.status, TC_ERR_PRODUCER)) { ok = false; break; }
          const uint32_t a_dst = base + stage * SM::STAGE_BYTES, b_dst = a_dst + SM::A_BYTES;
          mbar_expect_tx(full_bar(stage), SM::STAGE_BYTES);
          const int k0 = (int)(kb * TC_BK);
          if constexpr (A_MN) {   // A stored [k, m]: boxes of 64 m x 64 k
#pragma unroll
            for (int j = 0; j < TC_BM / 64; ++j)
              tma_load_4d(a_dst + j * (64 * TC_BK * 2), &tma_a, full_bar(stage), (int)(tm * TC_BM) + j * 64, k0, zai, zao);
          } else {                // A stored [m, k]: one box of 64 k x 128 m
            tma_load_4d(a_dst, &tma_a, full_bar(stage), k0, (int)(tm * TC_BM), zai, zao);
          }
          if constexpr (B_MN) {   // B stored [k, n]: boxes of 64 n x 64 k
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_4d(b_dst + j * (64 * TC_BK * 2), &tma_b, full_bar(stage), (int)(tn * BN) + j * 64, k0, zbi, zbo);
          } else {                // B stored [n, k]: one box of 64 k x BN n
            tma_load_4d(b_dst, &tma_b, full_bar(stage), k0, (int)(tn * BN), zbi, zbo);
          }
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // drain: wait (bounded) for the copies still in flight so none lands after the CTA has gone
        uint32_t s = stage, ph = phase;
        const uint32_t n_back = issued < (uint32_t)STAGES ? issued : (uint32_t)STAGES;
        for (uint32_t i = 0; i < n_back; ++i) {
          if (s == 0) { s = STAGES - 1; ph ^= 1; } else --s;
          const uint64_t t0 = global_timer_ns();
          while (!mbar_try_wait(full_bar(s), ph) && global_timer_ns() - t0 < TC_WAIT_NS) {}
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------- MMA issuer ----------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc(p.is_bf16 != 0, A_MN, B_MN, TC_BM, BN);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      while (ok) {
        const uint32_t t = next_tile(TC_ERR_MMA);
        if (t == TILE_NONE) break;
        uint32_t bz, tm, tn, kb0, kb1;
        tile_coords(t, bz, tm, tn);
        k_range(tm, kb0, kb1);
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, abort_flag, p.status, TC_ERR_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (uint32_t kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, TC_ERR_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = base + stage * SM::STAGE_BYTES, b_addr = a_addr + SM::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < TC_BK / TC_UMMA_K; ++kk) {
            // K-major: 16 K-elements = 32 B inside the swizzle atom; MN-major: 16 k-rows of 128 B = 2048 B
            const uint64_t adesc = A_MN ? make_smem_desc(a_addr + kk * (TC_UMMA_K * 128), 64 * TC_BK * 2, 1024)
                                        : make_smem_desc(a_addr + kk * (TC_UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(b_addr + kk * (TC_UMMA_K * 128), 64 * TC_BK * 2, 1024)
                                        : make_smem_desc(b_addr + kk * (TC_UMMA_K * 2), 16, 1024);
            umma_f16(d_tmem, adesc, bdesc, idesc, (kb != kb0 || kk != 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));                 // slot is free once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));                     // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ---------------------------------- epilogue (warps 2..9) ----------------------------------
    const int col_half = (warp - 2) >> 2;                // warps 2..5 take the left half of the columns, 6..9 the right
    const uint32_t quarter = (uint32_t)(warp & 3);       // TMEM lanes this warp may read: 32*quarter .. +31
    const uint32_t row_in_tile = quarter * 32 + lane;
    uint32_t acc = 0, acc_phase = 0;
    const bool rn = p.rn != 0, is_bf16 = p.is_bf16 != 0;
    const uint16_t* bias = reinterpret_cast<const uint16_t*>(p.bias);
    auto ld16 = [&](uint16_t h) { return is_bf16 ? bf16_to_f32(h) : f16_to_f32(h); };
    auto st16 = [&](float v) { return is_bf16 ? f32_to_bf16(v, rn) : f32_to_f16(v, rn); };
    auto cdt = [&](float v) { return ld16(is_bf16 ? f32_to_bf16(v, false) : f32_to_f16(v, false)); };
    const float calpha = cdt(p.alpha);
    const GeluConsts gc{cdt(0.5f), cdt(0.044715f), cdt(0.7978845608028654f)};
    bool ok = true;
    while (ok) {
      const uint32_t t = next_tile(TC_ERR_EPILOGUE);
      if (t == TILE_NONE) break;
      uint32_t bz, tm, tn;
      tile_coords(t, bz, tm, tn);
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, TC_ERR_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      const uint32_t row = tm * TC_BM + row_in_tile;
      const uint32_t col0 = tn * BN;
      const int64_t c_off = (int64_t)(bz / p.batch_inner) * p.stride_c + (int64_t)(bz % p.batch_inner) * p.stride_c_inner + (int64_t)row * p.ldc;
      uint16_t* crow = reinterpret_cast<uint16_t*>(p.c) + c_off;
      uint16_t* zrow = p.preact ? reinterpret_cast<uint16_t*>(p.preact) + c_off : nullptr;
#pragma unroll 1
      for (int ch = col_half * (BN / 64); ch < (col_half + 1) * (BN / 64); ++ch) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((quarter * 32u) << 16) + acc * BN + ch * 32, r);
        tmem_ld_wait();
        const uint32_t c = col0 + ch * 32;
        if (row < p.m && c < p.n) {
          const bool full = c + 32 <= p.n;               // n % 8 == 0 is guaranteed by the host
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          if (p.alpha != 1.0f) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= calpha;
          }
          if (p.epilogue >= ZYXB_EPI_BIAS && p.epilogue <= ZYXB_EPI_BIAS_GELU) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (full || c + q * 8 < p.n) {
                const Pack<uint16_t, 8> pk = load_pack<uint16_t, 8>(bias + c + q * 8);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[q * 8 + j] += ld16(pk.v[j]);
              }
            }
          }
          if (zrow) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (full || c + q * 8 < p.n) {
                Pack<uint16_t, 8> pk;
#pragma unroll
                for (int j = 0; j < 8; ++j) pk.v[j] = st16(v[q * 8 + j]);
                store_pack<uint16_t, 8>(zrow + c + q * 8, pk);
              }
            }
          }
          if (p.epilogue == ZYXB_EPI_ADD) {
            const uint16_t* zr = reinterpret_cast<const uint16_t*>(p.z) + c_off;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (full || c + q * 8 < p.n) {
                const Pack<uint16_t, 8> pk = load_pack_stream<uint16_t, 8>(zr + c + q * 8);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[q * 8 + j] += ld16(pk.v[j]);
              }
            }
          } else if (p.epilogue == ZYXB_EPI_MUL_RELU_GRAD || p.epilogue == ZYXB_EPI_MUL_GELU_GRAD) {
            // backward through the activation: multiply the input gradient by act'(z), z read once from HBM
            const uint16_t* zr = reinterpret_cast<const uint16_t*>(p.z) + c_off;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (full || c + q * 8 < p.n) {
                const Pack<uint16_t, 8> pk = load_pack_stream<uint16_t, 8>(zr + c + q * 8);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const float x = ld16(pk.v[j]);
                  float g;
                  if (p.epilogue == ZYXB_EPI_MUL_RELU_GRAD) g = x > 0.0f ? 1.0f : 0.0f;
                  else {
                    const float u = (x + x * x * x * gc.a) * gc.s;
                    const float e = fast_exp(u + u);
                    const float th = __fdividef(e - 1.0f, e + 1.0f);
                    g = gc.half * (th + 1.0f) + x * gc.half * (1.0f - th * th) * ((1.0f + 3.0f * gc.a * x * x) * gc.s);
                  }
                  v[q * 8 + j] *= g;
                }
              }
            }
          } else if (p.epilogue == ZYXB_EPI_BIAS_RELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = relu_ref(v[j]);
          } else if (p.epilogue == ZYXB_EPI_BIAS_GELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              // gelu_ref with the SFU exponential and a fast divide: within 2^-20 of the formula
              const float x = v[j];
              const float u = (x + x * x * x * gc.a) * gc.s;
              const float e = fast_exp(u + u);
              const float th = __fdividef(e - 1.0f, e + 1.0f);
              v[j] = x * gc.half * (th + 1.0f);
            }
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (full || c + q * 8 < p.n) {
              Pack<uint16_t, 8> pk;
#pragma unroll
              for (int j = 0; j < 8; ++j) pk.v[j] = st16(v[q * 8 + j]);
              store_pack<uint16_t, 8>(crow + c + q * 8, pk);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(tempty_bar(acc));                      // all epilogue threads arrive: the accumulator goes back to the MMA issuer
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
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
bool gemm_tc_supported(const GemmParams& p, int dtype, const LaunchCtx& lc) {
  if (dtype != ZYXB_BF16 && dtype != ZYXB_F16) return false;
  if (!lc.tma_encode) return false;
  // TMA: 16-byte aligned bases and row pitches; the epilogue stores 8 elements at a time
  const uint64_t a_inner = p.trans_a ? p.m : p.k, b_inner = p.trans_b ? p.k : p.n;
  if (a_inner % 8 || b_inner % 8 || p.n % 8) return false;
  if (p.lda % 8 || p.ldb % 8 || p.ldc % 8) return false;
  if (p.stride_a_inner % 8 || p.stride_b_inner % 8 || p.stride_c_inner % 8) return false;
  if (p.ldc > 0xffffffffull) return false;
  if ((uintptr_t)p.a % 16 || (uintptr_t)p.b % 16 || (uintptr_t)p.c % 16) return false;
  if (p.preact && (uintptr_t)p.preact % 16) return false;
  if (p.bias && (uintptr_t)p.bias % 16) return false;
  if (p.z && (uintptr_t)p.z % 16) return false;
  if ((p.stride_a % 8) || (p.stride_b % 8) || (p.stride_c % 8)) return false;
  if (p.m > 0x7fffff00ull || p.n > 0x7fffff00ull || p.k > 0x7fffff00ull || p.batch * p.batch_inner > 65535) return false;
  // tiny problems are latency-bound: the SIMT kernel has no descriptor set-up cost
  if (p.m * p.n * p.k < (1ull << 21) || p.m < 32) return false;
  return true;
}

template <bool A_MN, bool B_MN, int BN, int STAGES>
static cudaError_t launch_tc_variant(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& tp, unsigned grid, cudaStream_t s) {
  using SM = TcSmem<BN, STAGES>;
  static uint64_t configured = 0;
  auto kern = gemm_tc_kernel<A_MN, B_MN, BN, STAGES>;
  {
    cudaError_t e = ensure_dynamic_smem(kern, SM::TOTAL, &configured);
    if (e != cudaSuccess) return e;
  }
  kern<<<grid, TC_THREADS, SM::TOTAL, s>>>(ma, mb, tp);
  return cudaGetLastError();
}

template <int BN, int STAGES>
static cudaError_t launch_tc_bn(bool a_mn, bool b_mn, const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& tp, unsigned grid,
                                cudaStream_t s) {
  if (a_mn) return b_mn ? launch_tc_variant<true, true, BN, STAGES>(ma, mb, tp, grid, s) : launch_tc_variant<true, false, BN, STAGES>(ma, mb, tp, grid, s);
  return b_mn ? launch_tc_variant<false, true, BN, STAGES>(ma, mb, tp, grid, s) : launch_tc_variant<false, false, BN, STAGES>(ma, mb, tp, grid, s);
}

int launch_gemm_tc(const GemmParams& p, int dtype, const LaunchCtx& lc, std::string& err) {
  const bool bf16 = dtype == ZYXB_BF16;
  const bool a_mn = p.trans_a != 0;      // A stored [k, m]: M is the contiguous axis
  const bool b_mn = p.trans_b == 0;      // B stored [k, n]: N is the contiguous axis
  const int bn = p.n <= 128 ? 128 : 256;
  CUtensorMap ma, mb;
  const uint64_t sa = p.batch > 1 ? (uint64_t)p.stride_a : 0, sb = p.batch > 1 ? (uint64_t)p.stride_b : 0;
  const uint64_t sai = p.batch_inner > 1 ? (uint64_t)p.stride_a_inner : 0, sbi = p.batch_inner > 1 ? (uint64_t)p.stride_b_inner : 0;
  const bool oka = a_mn ? encode_map(lc.tma_encode, &ma, bf16, p.a, p.m, p.k, p.lda, p.batch_inner, sai, p.batch, sa, 64)
                        : encode_map(lc.tma_encode, &ma, bf16, p.a, p.k, p.m, p.lda, p.batch_inner, sai, p.batch, sa, TC_BM);
  const bool okb = b_mn ? encode_map(lc.tma_encode, &mb, bf16, p.b, p.n, p.k, p.ldb, p.batch_inner, sbi, p.batch, sb, 64)
                        : encode_map(lc.tma_encode, &mb, bf16, p.b, p.k, p.n, p.ldb, p.batch_inner, sbi, p.batch, sb, (uint32_t)bn);
  if (!oka || !okb) { err = "gemm: cuTensorMapEncodeTiled rejected an operand"; return ZYXB_ERR_KERNEL_LAUNCH; }
  TcParams tp{};
  tp.bias = p.bias; tp.z = p.z; tp.c = p.c; tp.preact = p.preact;
  tp.m = (uint32_t)p.m; tp.n = (uint32_t)p.n; tp.k = (uint32_t)p.k; tp.batch = (uint32_t)(p.batch * p.batch_inner);
  tp.batch_inner = (uint32_t)p.batch_inner; tp.ldc = (uint32_t)p.ldc; tp.stride_c_inner = p.stride_c_inner;
  tp.tiles_m = (uint32_t)((p.m + TC_BM - 1) / TC_BM); tp.tiles_n = (uint32_t)((p.n + bn - 1) / bn);
  tp.stride_c = p.stride_c; tp.alpha = p.alpha; tp.epilogue = p.epilogue; tp.rn = p.rn; tp.is_bf16 = bf16 ? 1 : 0;
  tp.status = lc.status_word; tp.tri = p.tri;
  // tile counters live in the words after the status word, used in rotation and zeroed in stream order
  // While a collective may be running beside the matmul (a communicator exists) some SMs are not available to
  // the persistent grid; drawing tiles from a counter lets the CTAs that do run share the work evenly.  Alone on
  // the GPU the fixed assignment is marginally faster (no atomic per tile).
  static const char* dyn_env = getenv("ZYXB_DYNAMIC_TILES");
  tp.dynamic_tiles = dyn_env ? (dyn_env[0] == '1') : ((lc.overlap_hint || p.tri != ZYXB_TRI_NONE) ? 1 : 0);   // causal tiles differ in cost
  tp.tile_counter = lc.status_word + 8 + (*lc.launch_counter % 48);
  if (tp.dynamic_tiles && cudaMemsetAsync(tp.tile_counter, 0, sizeof(uint32_t), lc.stream) != cudaSuccess) {
    err = "gemm: tile counter reset failed"; return ZYXB_ERR_KERNEL_LAUNCH;
  }
  tp.a_batched = (sa ? 1 : 0) | (sai ? 2 : 0);
  tp.b_batched = (sb ? 1 : 0) | (sbi ? 2 : 0);
  const uint64_t total = (uint64_t)tp.tiles_m * tp.tiles_n * tp.batch;
  ZYXB_CHECK_ARG(total < 0x7fffffffull, "gemm: too many tiles");
  const unsigned grid = (unsigned)std::min<uint64_t>(total, (uint64_t)lc.sm_count);
  cudaError_t e = bn == 256 ? launch_tc_bn<256, 4>(a_mn, b_mn, ma, mb, tp, grid, lc.stream)
                            : launch_tc_bn<128, 6>(a_mn, b_mn, ma, mb, tp, grid, lc.stream);
  if (e != cudaSuccess) { err = std::string("gemm_tcgen05: ") + cudaGetErrorString(e); return ZYXB_ERR_KERNEL_LAUNCH; }
  *lc.launch_counter += 1;
  return ZYXB_OK;
}

}  // namespace zyxb
