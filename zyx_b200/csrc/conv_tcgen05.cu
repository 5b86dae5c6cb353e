// 2-D convolution forward (Tensor::conv with groups = 1, zyx/src/tensor/mod.rs:2583-2680).
//   y[n,o,i,j] = bias[o] + sum_{c,r,s} x[n, c, i*stride_h + r*dil_h - pad_top, j*stride_w + s*dil_w - pad_left] * w[o,c,r,s]
//
// bf16 / f16 with enough work: implicit GEMM on the 5th-generation tensor cores.  The reference builds the im2col view
// by reshape / expand / permute (pool, mod.rs:2442) and multiplies it with the weights; here no such matrix exists:
//   prep   x [n,c,h,w] -> xt [n,h,w,cp] and w [o,c,kh,kw] -> wt [o, kh*kw, cp]  (channels innermost, cp = c rounded up
//          to 8 so that every TMA row pitch is a multiple of 16 bytes; the added channels are zeros)
//   GEMM   M = 128 output positions, N = BN output channels, K = kh*kw*cp walked as (tap, 64-channel block).  The A tile
//          of a k-block is one TMA load through an im2col-mode tensor map: its bounding box is the set of window origins
//          ([-pad, extent + pad - dilated filter extent]), its element strides are the convolution's strides, the load's
//          coordinates name the tile's first output position and its two offsets the filter tap; the hardware walks the
//          128 positions that follow in row-major order, across rows and images, and zero-fills the padding.  (Paddings
//          beyond the 8-bit corner fields of a rank-4 map use a tiled map instead: a TH x TW patch of one image per tile,
//          box {64, TW*stride, TH*stride}.)  One box {64 channels, 1 tap, BN filters} of wt is the B tile.  Both land
//          K-major in 128-byte-swizzled shared memory, exactly the layout of the matmul kernel's NT case.
//   store  TMEM lane = output position, so for one output channel the 32 lanes of a warp hold 32 neighbouring positions:
//          each warp store writes a run of the channels-first output directly, no transposition pass.
// One persistent CTA per SM, 320 threads: warp 0 TMA producer, warp 1 MMA issuer, warps 2..9 epilogue; the accumulator is
// double-buffered in TMEM.  Every mbarrier wait is bounded by wall-clock time and reports through the status word.
//
// Everything else (f32, i32, tiny problems, shapes the boxes cannot express): a direct kernel, one thread per output
// element, summing in the reference's order (c, then r, then s), so integer results are bit-exact.
#include <cuda.h>

#include <algorithm>
#include <vector>

#include "common.cuh"
#include "internal.h"
#include "tc_ptx.cuh"

namespace zyxb {

namespace {

constexpr int CV_BM = 128, CV_BK = 64, CV_UMMA_K = 16, CV_THREADS = 320, CV_EPI_THREADS = 256;

struct ConvGeom {
  uint32_t n, c, h, w, o, kh, kw, oh, ow;
  uint32_t sh, sw, dh, dw;
  int pt, pl;
};

struct ConvTcParams {
  const void* bias; void* y;
  ConvGeom g;
  uint32_t cp, cblocks;              // padded channels; 64-channel blocks per tap
  uint32_t tw, th, tw_shift;         // patch of output positions per tile: th * tw = 128
  uint32_t tiles_w, tiles_h, tiles_n;
  uint32_t positions, tiles_m;        // im2col mode: n*oh*ow output positions in tiles of 128 consecutive ones
  int rn, is_bf16;
  int channels_last;                  // y is [positions, o]: a lane's 32 filters are contiguous
  // Output placement: position (oy, ox) of the g.oh x g.ow result lands at (off_h + step_h*oy, off_w + step_w*ox) of a
  // full_h x full_w plane.  The identity (steps 1, offsets 0, full = oh x ow) for a convolution; one residue class of the
  // input positions for a phase of a strided convolution's input gradient.
  uint32_t full_h, full_w, step_h, step_w, off_h, off_w;
  int out_mapped;
  uint32_t* status;
};

// What a phase of a strided convolution's input gradient changes in the tensor-core launch (see launch_conv_dgrad).
struct ConvPhase {
  uint32_t r0, step_r, s0, step_s;    // the forward filter's taps this phase uses: r0 + t*step_r (t < kh of the phase), columns alike
  uint32_t fkh, fkw;                  // the forward filter's extents
  uint32_t full_h, full_w, step_h, step_w, off_h, off_w;
  int pad_bottom, pad_right;          // signed: a phase may ignore the last rows / columns of dy (and its first: negative pt / pl)
  bool x_ready;                       // the channels-innermost copy of the input already sits in scratch (an earlier phase wrote it)
};

template <int BN, int STAGES>
struct ConvSmem {
  static constexpr int A_BYTES = CV_BM * CV_BK * 2;
  static constexpr int B_BYTES = BN * CV_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;   // + barriers + slack to align the base to 1024 B
};

enum { CV_ERR_PRODUCER = 16384u, CV_ERR_MMA = 32768u, CV_ERR_EPILOGUE = 65536u };

// ---- prep: channels innermost ----------------------------------------------------------------------
// x [n][c][hw] -> xt [n][hw][cp], 32 x 32 tiles through shared memory; channels c..cp-1 are written as zeros
__global__ void conv_nhwc_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ xt, uint32_t c, uint32_t cp, uint32_t hw) {
  __shared__ uint16_t tile[32][33];
  const uint32_t n = blockIdx.z, p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const uint16_t* xs = x + (size_t)n * c * hw;
  uint16_t* xd = xt + (size_t)n * hw * cp;
  for (uint32_t j = threadIdx.y; j < 32; j += blockDim.y) {
    const uint32_t ci = c0 + j, p = p0 + threadIdx.x;
    tile[j][threadIdx.x] = (ci < c && p < hw) ? xs[(size_t)ci * hw + p] : (uint16_t)0;
  }
  __syncthreads();
  for (uint32_t j = threadIdx.y; j < 32; j += blockDim.y) {
    const uint32_t p = p0 + j, ci = c0 + threadIdx.x;
    if (p < hw && ci < cp) xd[(size_t)p * cp + ci] = tile[threadIdx.x][j];
  }
}

// The same for an even hw: 64 x 64 tiles moved as 32-bit words on both sides (two positions per word when read, two
// channels per word when written), so every warp access covers whole 128-byte lines.
__global__ void __launch_bounds__(256) conv_nhwc_pairs_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ xt, uint32_t c, uint32_t cp, uint32_t hw) {
  __shared__ __align__(4) uint16_t tile[64][66];
  const uint32_t n = blockIdx.z, p0 = blockIdx.x * 64, c0 = blockIdx.y * 64;
  const uint16_t* xs = x + (size_t)n * c * hw;
  uint16_t* xd = xt + (size_t)n * hw * cp;
#pragma unroll
  for (uint32_t i = 0; i < 8; ++i) {
    const uint32_t idx = i * 256 + threadIdx.x, cj = idx >> 5, pp = (idx & 31) * 2;
    const uint32_t ci = c0 + cj, p = p0 + pp;
    uint32_t v = 0;
    if (ci < c && p < hw) v = __ldcs(reinterpret_cast<const uint32_t*>(xs + (size_t)ci * hw + p));   // hw even: p + 1 < hw too
    *reinterpret_cast<uint32_t*>(&tile[cj][pp]) = v;
  }
  __syncthreads();
#pragma unroll
  for (uint32_t i = 0; i < 8; ++i) {
    const uint32_t idx = i * 256 + threadIdx.x, pj = idx >> 5, cc = (idx & 31) * 2;
    const uint32_t p = p0 + pj, ci = c0 + cc;
    if (p < hw && ci < cp) {                              // cp even: ci + 1 < cp too
      const uint32_t v = (uint32_t)tile[cc][pj] | ((uint32_t)tile[cc + 1][pj] << 16);
      *reinterpret_cast<uint32_t*>(xd + (size_t)p * cp + ci) = v;
    }
  }
}

// w [o][c][taps] -> wt [o][taps][cp].  flipped: the buffer holds the filter of the convolution whose input gradient this
// one computes, [c][o][taps], and is read transposed in (o, c) with the taps reversed.
__global__ void conv_weight_kernel(const uint16_t* __restrict__ w, uint16_t* __restrict__ wt, uint32_t c, uint32_t cp, uint32_t o_count,
                                   uint32_t taps, uint64_t total, int flipped) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const uint32_t ci = (uint32_t)(i % cp);
  const uint64_t ot = i / cp;
  const uint32_t tap = (uint32_t)(ot % taps);
  const uint64_t o = ot / taps;
  uint16_t v = 0;
  if (ci < c) v = flipped ? w[((uint64_t)ci * o_count + o) * taps + (taps - 1 - tap)] : w[(o * c + ci) * taps + tap];
  wt[i] = v;
}

// A phase of a strided input gradient: wt [o][nr*ns][cp] from the forward filter [c][o][fkh][fkw], transposed in (o, c),
// restricted to the taps (r0 + t*step_r, s0 + u*step_s) and reversed in (t, u).
__global__ void conv_weight_phase_kernel(const uint16_t* __restrict__ w, uint16_t* __restrict__ wt, uint32_t c, uint32_t cp, uint32_t o_count,
                                         uint32_t nr, uint32_t ns, uint32_t r0, uint32_t step_r, uint32_t s0, uint32_t step_s, uint32_t fkh, uint32_t fkw,
                                         uint64_t total) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const uint32_t ci = (uint32_t)(i % cp);
  const uint64_t ot = i / cp;
  const uint32_t tap = (uint32_t)(ot % (nr * ns));
  const uint64_t o = ot / (nr * ns);
  const uint32_t r = r0 + (nr - 1 - tap / ns) * step_r, sx = s0 + (ns - 1 - tap % ns) * step_s;
  wt[i] = ci < c ? w[((uint64_t)ci * o_count + o) * fkh * fkw + r * fkw + sx] : (uint16_t)0;
}

// ---- implicit GEMM ---------------------------------------------------------------------------------
template <int BN, int STAGES, bool IM2COL>
__global__ void __launch_bounds__(CV_THREADS, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap tma_x, const __grid_constant__ CUtensorMap tma_w, ConvTcParams p) {
  using SM = ConvSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;          // swizzle atoms repeat every 1024 B
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t bar_base = base + SM::BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + SM::BAR_OFFSET + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), CV_EPI_THREADS); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const ConvGeom& g = p.g;
  const uint32_t taps = g.kh * g.kw, k_blocks = taps * p.cblocks;
  const uint32_t total_tiles = (IM2COL ? p.tiles_m : g.n * p.tiles_h * p.tiles_w) * p.tiles_n;
  const uint32_t plane = g.oh * g.ow;
  // Filter blocks vary fastest: the CTAs that share a patch of the image run at the same time and meet in L2.
  // Tiled mode: the tile is a th x tw patch of image img at (oh0, ow0).  im2col mode: the tile is the 128 positions that
  // follow (img, oh0, ow0) in row-major order, across rows and images; m0 is the first one's flat index.
  auto tile_coords = [&](uint32_t t, uint32_t& tn, uint32_t& img, uint32_t& oh0, uint32_t& ow0, uint32_t& m0) {
    tn = t % p.tiles_n; t /= p.tiles_n;
    if constexpr (IM2COL) {
      m0 = t * CV_BM;
      img = m0 / plane;
      const uint32_t rem = m0 - img * plane;
      oh0 = rem / g.ow; ow0 = rem - oh0 * g.ow;
    } else {
      m0 = 0;
      ow0 = (t % p.tiles_w) * p.tw; t /= p.tiles_w;
      oh0 = (t % p.tiles_h) * p.th;
      img = t / p.tiles_h;
    }
  };

  if (warp == 0) {
    // ---------------------------------- TMA producer ----------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, issued = 0;
      bool ok = true;
      for (uint32_t t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        uint32_t tn, img, oh0, ow0, m0;
        tile_coords(t, tn, img, oh0, ow0, m0);
        const int x0 = (int)(ow0 * g.sw) - g.pl, y0 = (int)(oh0 * g.sh) - g.pt;
        for (uint32_t tap = 0; ok && tap < taps; ++tap) {
          const int r = (int)(tap / g.kw), s = (int)(tap % g.kw);
          for (uint32_t cb = 0; cb < p.cblocks; ++cb) {
            if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, p.status, CV_ERR_PRODUCER)) { ok = false; break; }
            const uint32_t a_dst = base + stage * SM::STAGE_BYTES, b_dst = a_dst + SM::A_BYTES;
            mbar_expect_tx(full_bar(stage), SM::STAGE_BYTES);
            // the channel coordinate (innermost) is a multiple of 64 elements: always on a 16-byte boundary
            if constexpr (IM2COL) tma_load_im2col_4d(a_dst, &tma_x, full_bar(stage), (int)(cb * CV_BK), x0, y0, (int)img, (uint16_t)(s * g.dw), (uint16_t)(r * g.dh));
            else tma_load_4d(a_dst, &tma_x, full_bar(stage), (int)(cb * CV_BK), x0 + s * (int)g.dw, y0 + r * (int)g.dh, (int)img);
            tma_load_4d(b_dst, &tma_w, full_bar(stage), (int)(cb * CV_BK), (int)tap, (int)(tn * BN), 0);
            ++issued;
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
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
      const uint32_t idesc = make_idesc(p.is_bf16 != 0, false, false, CV_BM, BN);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (uint32_t t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, abort_flag, p.status, CV_ERR_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (uint32_t kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, CV_ERR_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = base + stage * SM::STAGE_BYTES, b_addr = a_addr + SM::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < CV_BK / CV_UMMA_K; ++kk) {
            const uint64_t adesc = make_smem_desc(a_addr + kk * (CV_UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = make_smem_desc(b_addr + kk * (CV_UMMA_K * 2), 16, 1024);
            umma_f16(d_tmem, adesc, bdesc, idesc, (kb != 0 || kk != 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ---------------------------------- epilogue (warps 2..9) ----------------------------------
    const int col_half = (warp - 2) >> 2;
    const uint32_t quarter = (uint32_t)(warp & 3);
    const uint32_t row_in_tile = quarter * 32 + lane;
    const uint32_t ty = row_in_tile >> p.tw_shift, tx = row_in_tile & (p.tw - 1);
    uint32_t acc = 0, acc_phase = 0;
    const bool rn = p.rn != 0, is_bf16 = p.is_bf16 != 0;
    const uint16_t* bias = reinterpret_cast<const uint16_t*>(p.bias);
    uint16_t* y = reinterpret_cast<uint16_t*>(p.y);
    for (uint32_t t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      uint32_t tn, img, oh0, ow0, m0;
      tile_coords(t, tn, img, oh0, ow0, m0);
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, CV_ERR_EPILOGUE)) break;
      tc_fence_after();
      bool inside;
      uint16_t* ypos;          // channels-first: this lane's position in filter 0's plane
      size_t pos;              // flat index of the position over (image, row, column)
      size_t oplane = plane;   // elements between two filters' planes of the channels-first output
      if constexpr (IM2COL) {
        const uint32_t m = m0 + row_in_tile, im = m / plane;      // this lane's position: image im, offset m - im * plane in its plane
        inside = m < p.positions;
        ypos = y + (size_t)im * g.o * plane + (m - im * plane);
        pos = m;
        if (p.out_mapped) {
          const uint32_t rem = m - im * plane, oy = rem / g.ow, ox = rem - oy * g.ow;
          oplane = (size_t)p.full_h * p.full_w;
          pos = ((size_t)im * p.full_h + p.off_h + (size_t)p.step_h * oy) * p.full_w + p.off_w + (size_t)p.step_w * ox;
          ypos = y + (size_t)im * g.o * oplane + (pos - (size_t)im * oplane);
        }
      } else {
        const uint32_t oy = oh0 + ty, ox = ow0 + tx;
        inside = oy < g.oh && ox < g.ow;
        ypos = y + (size_t)img * g.o * plane + (size_t)oy * g.ow + ox;
        pos = ((size_t)img * g.oh + oy) * g.ow + ox;
        if (p.out_mapped) {
          oplane = (size_t)p.full_h * p.full_w;
          pos = ((size_t)img * p.full_h + p.off_h + (size_t)p.step_h * oy) * p.full_w + p.off_w + (size_t)p.step_w * ox;
          ypos = y + (size_t)img * g.o * oplane + (pos - (size_t)img * oplane);
        }
      }
#pragma unroll 1
      for (int ch = col_half * (BN / 64); ch < (col_half + 1) * (BN / 64); ++ch) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((quarter * 32u) << 16) + acc * BN + ch * 32, r);
        tmem_ld_wait();
        const uint32_t o0 = tn * BN + ch * 32;
        if (inside && o0 < g.o && p.channels_last) {
          // channels-last output: this lane's position is a row of g.o filters, 32 of them here
          uint16_t* yrow = y + pos * g.o + o0;
          const bool vec = (g.o % 8 == 0) && o0 + 32 <= g.o;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            Pack<uint16_t, 8> pk;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t o = o0 + q * 8 + j;
              float v = __uint_as_float(r[q * 8 + j]);
              if (bias && o < g.o) v += is_bf16 ? bf16_to_f32(bias[o]) : f16_to_f32(bias[o]);
              pk.v[j] = is_bf16 ? f32_to_bf16(v, rn) : f32_to_f16(v, rn);
            }
            if (vec) store_pack<uint16_t, 8>(yrow + q * 8, pk);
            else {
#pragma unroll
              for (int j = 0; j < 8; ++j) if (o0 + q * 8 + j < g.o) yrow[q * 8 + j] = pk.v[j];
            }
          }
        } else if (inside && o0 < g.o) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const uint32_t o = o0 + j;
            if (o < g.o) {
              float v = __uint_as_float(r[j]);
              if (bias) v += is_bf16 ? bf16_to_f32(bias[o]) : f16_to_f32(bias[o]);
              ypos[(size_t)o * oplane] = is_bf16 ? f32_to_bf16(v, rn) : f32_to_f16(v, rn);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(tempty_bar(acc));
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

// ---- direct kernel -----------------------------------------------------------------------------------
template <typename T>
__global__ void conv_direct_kernel(const typename Elem<T>::store_t* __restrict__ x, const typename Elem<T>::store_t* __restrict__ w,
                                   const typename Elem<T>::store_t* __restrict__ bias, typename Elem<T>::store_t* __restrict__ y,
                                   ConvGeom g, uint64_t total, int rn, int channels_last, int flipped) {
  using A = typename Elem<T>::acc_t;
  // element strides of x: channels-first [n,c,h,w] or channels-last [n,h,w,c]
  const uint64_t xs_c = channels_last ? 1 : (uint64_t)g.h * g.w, xs_p = channels_last ? g.c : 1;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
    uint32_t ox, oy, o;
    uint64_t n, q = i;
    if (channels_last) { o = (uint32_t)(q % g.o); q /= g.o; ox = (uint32_t)(q % g.ow); q /= g.ow; oy = (uint32_t)(q % g.oh); n = q / g.oh; }
    else { ox = (uint32_t)(q % g.ow); q /= g.ow; oy = (uint32_t)(q % g.oh); q /= g.oh; o = (uint32_t)(q % g.o); n = q / g.o; }
    A acc = 0;
    for (uint32_t c = 0; c < g.c; ++c) {
      const auto* xp = x + n * g.c * (uint64_t)g.h * g.w + c * xs_c;
      // flipped: the stored filter is [c][o][kh][kw] and tap (r, s) reads its (kh-1-r, kw-1-s)
      const auto* wp = w + (flipped ? ((uint64_t)c * g.o + o) : ((uint64_t)o * g.c + c)) * g.kh * g.kw;
      for (uint32_t r = 0; r < g.kh; ++r) {
        const int iy = (int)(oy * g.sh + r * g.dh) - g.pt;
        if (iy < 0 || iy >= (int)g.h) continue;           // zero padding contributes nothing
        for (uint32_t s = 0; s < g.kw; ++s) {
          const int ix = (int)(ox * g.sw + s * g.dw) - g.pl;
          if (ix < 0 || ix >= (int)g.w) continue;
          acc += (A)Elem<T>::load(xp[((uint64_t)iy * g.w + ix) * xs_p]) * (A)Elem<T>::load(wp[flipped ? (g.kh - 1 - r) * g.kw + (g.kw - 1 - s) : r * g.kw + s]);
        }
      }
    }
    if (bias) acc += (A)Elem<T>::load(bias[o]);
    y[i] = Elem<T>::store(acc, rn != 0);
  }
}

bool geometry(const zyxb_conv_desc& d, ConvGeom& g, std::string& err) {
  auto one = [](uint32_t v) { return v ? v : 1u; };
  const uint64_t lim = 1u << 24;
  if (!d.n || !d.c || !d.h || !d.w || !d.o || !d.kh || !d.kw) { err = "conv: every extent must be positive"; return false; }
  if (d.n > lim || d.c > lim || d.h > lim || d.w > lim || d.o > lim || d.kh > 4096 || d.kw > 4096 || d.pad_top > lim || d.pad_left > lim ||
      d.pad_bottom > lim || d.pad_right > lim || d.stride_h > lim || d.stride_w > lim || d.dil_h > lim || d.dil_w > lim) {
    err = "conv: extent too large"; return false;
  }
  g.n = (uint32_t)d.n; g.c = (uint32_t)d.c; g.h = (uint32_t)d.h; g.w = (uint32_t)d.w; g.o = (uint32_t)d.o; g.kh = (uint32_t)d.kh; g.kw = (uint32_t)d.kw;
  g.sh = one(d.stride_h); g.sw = one(d.stride_w); g.dh = one(d.dil_h); g.dw = one(d.dil_w);
  g.pt = (int)d.pad_top; g.pl = (int)d.pad_left;
  const int64_t eh = (int64_t)d.h + d.pad_top + d.pad_bottom - (int64_t)g.dh * (g.kh - 1) - 1;
  const int64_t ew = (int64_t)d.w + d.pad_left + d.pad_right - (int64_t)g.dw * (g.kw - 1) - 1;
  if (eh < 0 || ew < 0) { err = "conv: the dilated filter is larger than the padded input"; return false; }
  g.oh = (uint32_t)(eh / g.sh + 1); g.ow = (uint32_t)(ew / g.sw + 1);
  return true;
}

template <int BN, int STAGES, bool IM2COL>
cudaError_t launch_conv_tc(const CUtensorMap& mx, const CUtensorMap& mw, const ConvTcParams& tp, unsigned grid, cudaStream_t s) {
  using SM = ConvSmem<BN, STAGES>;
  static uint64_t configured = 0;
  auto kern = conv_tc_kernel<BN, STAGES, IM2COL>;
  {
    cudaError_t e = ensure_dynamic_smem(kern, SM::TOTAL, &configured);
    if (e != cudaSuccess) return e;
  }
  kern<<<grid, CV_THREADS, SM::TOTAL, s>>>(mx, mw, tp);
  return cudaGetLastError();
}

// The tensor-core path: returns 1 when it took the launch, 0 when the shape is not for it, < 0 on an error (err set).
int try_conv_tc(const zyxb_conv_desc& d, const ConvGeom& g, const void* x, const void* w, const void* bias, void* y, const LaunchCtx& lc,
                std::string& err, const ConvPhase* phase = nullptr) {
  static const bool off = getenv("ZYXB_NO_CONV_TC") != nullptr;
  if (off || !lc.tma_encode || (d.dtype != ZYXB_BF16 && d.dtype != ZYXB_F16)) return 0;
  // latency-bound problems and single-filter outputs stay on the direct kernel
  const uint64_t positions = (uint64_t)g.n * g.oh * g.ow, kdim = (uint64_t)g.c * g.kh * g.kw;
  if ((!phase && positions * g.o * kdim < (1ull << 22)) || g.o < 8 || positions < 128) return 0;
  if (g.sw > 8 || g.sh > 8) return 0;                     // element strides of a tensor map go up to 8
  // im2col-mode tensor map: 128 consecutive output positions per tile, whatever the image's width.  Its corners and tap
  // offsets are 8-bit fields for a rank-4 map.
  static const bool tiled_only = getenv("ZYXB_CONV_TILED") != nullptr;
  const int lo_w = -g.pl, lo_h = -g.pt;
  const int pad_r = phase ? phase->pad_right : (int)d.pad_right, pad_b = phase ? phase->pad_bottom : (int)d.pad_bottom;
  const int up_w = pad_r - (int)((g.kw - 1) * g.dw), up_h = pad_b - (int)((g.kh - 1) * g.dh);
  const bool im2col = !tiled_only && lc.tma_encode_im2col && lo_w >= -128 && lo_h >= -128 && lo_w <= 127 && lo_h <= 127 && up_w >= -128 && up_w <= 127 && up_h >= -128 &&
                      up_h <= 127 && (g.kw - 1) * g.dw <= 255 && (g.kh - 1) * g.dh <= 255 && positions < 0x7fffff00ull;
  // tiled-mode fallback: a th x tw patch of one image per tile, tw = the power of two that covers a row (at most 128)
  uint32_t tw = 8;
  while (tw < 128 && tw < g.ow) tw <<= 1;
  while (tw > 8 && tw * g.sw > 256) tw >>= 1;             // a TMA box spans at most 256 elements per dimension
  const uint32_t th = 128 / tw;
  if (!im2col && (tw * g.sw > 256 || th * g.sh > 256)) return 0;
  const uint32_t cp = (g.c + 7) / 8 * 8, taps = g.kh * g.kw;
  // channels-last input is read by TMA where it lies: its pitch (c elements) must already be a multiple of 16 bytes
  const bool in_place = d.channels_last != 0;
  if (in_place && (g.c % 8 || (uintptr_t)x % 16 || (uintptr_t)y % 16)) return 0;
  const size_t xt_bytes = in_place ? 0 : (size_t)g.n * g.h * g.w * cp * 2, wt_bytes = (size_t)g.o * taps * cp * 2;
  const size_t wt_off = (xt_bytes + 1023) / 1024 * 1024;
  if (wt_off + wt_bytes > lc.scratch_bytes) return 0;
  if ((uintptr_t)lc.scratch % 1024) return 0;
  uint16_t* xt = in_place ? reinterpret_cast<uint16_t*>(const_cast<void*>(x)) : reinterpret_cast<uint16_t*>(lc.scratch);
  uint16_t* wt = reinterpret_cast<uint16_t*>(reinterpret_cast<char*>(lc.scratch) + wt_off);
  const bool bf16 = d.dtype == ZYXB_BF16;
  const CUtensorMapDataType dt = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const int bn = g.o > 128 ? 256 : 128;
  CUtensorMap mx, mw;
  {
    cuuint64_t dims[4] = {cp, g.w, g.h, g.n};
    cuuint64_t strides[3] = {(cuuint64_t)cp * 2, (cuuint64_t)g.w * cp * 2, (cuuint64_t)g.h * g.w * cp * 2};
    cuuint32_t estr[4] = {1, g.sw, g.sh, 1};
    if (im2col) {
      // bounding box of the filter windows' first elements: [-pad, extent + pad - dilated filter extent] per dimension
      const int lower[2] = {lo_w, lo_h}, upper[2] = {up_w, up_h};
      if (reinterpret_cast<EncodeIm2colFn>(lc.tma_encode_im2col)(&mx, dt, 4, xt, dims, strides, lower, upper, 64, CV_BM, estr,
                                                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return 0;
    } else {
      cuuint32_t box[4] = {64, tw * g.sw, th * g.sh, 1};  // loads ceil(box / element stride) = tw x th positions
      if (reinterpret_cast<EncodeTiledFn>(lc.tma_encode)(&mx, dt, 4, xt, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return 0;
    }
    cuuint64_t wdims[4] = {cp, taps, g.o, 1};
    cuuint64_t wstrides[3] = {(cuuint64_t)cp * 2, (cuuint64_t)taps * cp * 2, (cuuint64_t)g.o * taps * cp * 2};
    cuuint32_t wbox[4] = {64, 1, (cuuint32_t)bn, 1};
    cuuint32_t one[4] = {1, 1, 1, 1};
    if (reinterpret_cast<EncodeTiledFn>(lc.tma_encode)(&mw, dt, 4, wt, wdims, wstrides, wbox, one, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                       CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return 0;
  }
  const uint32_t hw = g.h * g.w;
  if (in_place || (phase && phase->x_ready)) {}
  else if (hw % 2 == 0 && (uintptr_t)x % 4 == 0)
    conv_nhwc_pairs_kernel<<<dim3((hw + 63) / 64, (cp + 63) / 64, g.n), 256, 0, lc.stream>>>(reinterpret_cast<const uint16_t*>(x), xt, g.c, cp, hw);
  else
    conv_nhwc_kernel<<<dim3((hw + 31) / 32, (cp + 31) / 32, g.n), dim3(32, 8), 0, lc.stream>>>(reinterpret_cast<const uint16_t*>(x), xt, g.c, cp, hw);
  const uint64_t wtotal = (uint64_t)g.o * taps * cp;
  if (phase)
    conv_weight_phase_kernel<<<(unsigned)((wtotal + 255) / 256), 256, 0, lc.stream>>>(reinterpret_cast<const uint16_t*>(w), wt, g.c, cp, g.o, g.kh, g.kw, phase->r0,
                                                                                     phase->step_r, phase->s0, phase->step_s, phase->fkh, phase->fkw, wtotal);
  else
    conv_weight_kernel<<<(unsigned)((wtotal + 255) / 256), 256, 0, lc.stream>>>(reinterpret_cast<const uint16_t*>(w), wt, g.c, cp, g.o, taps, wtotal, d.flip_filter != 0);
  ConvTcParams tp{};
  tp.full_h = g.oh; tp.full_w = g.ow; tp.step_h = tp.step_w = 1;
  if (phase) {
    tp.full_h = phase->full_h; tp.full_w = phase->full_w; tp.step_h = phase->step_h; tp.step_w = phase->step_w;
    tp.off_h = phase->off_h; tp.off_w = phase->off_w; tp.out_mapped = 1;
  }
  tp.bias = bias; tp.y = y; tp.g = g; tp.cp = cp; tp.cblocks = (cp + CV_BK - 1) / CV_BK;
  tp.tw = tw; tp.th = th; tp.tw_shift = 0;
  while ((1u << tp.tw_shift) < tw) ++tp.tw_shift;
  tp.tiles_w = (g.ow + tw - 1) / tw; tp.tiles_h = (g.oh + th - 1) / th; tp.tiles_n = (g.o + bn - 1) / bn;
  tp.rn = lc.round_nearest ? 1 : 0; tp.is_bf16 = bf16 ? 1 : 0; tp.status = lc.status_word; tp.channels_last = in_place ? 1 : 0;
  tp.positions = (uint32_t)positions; tp.tiles_m = (uint32_t)((positions + CV_BM - 1) / CV_BM);
  const uint64_t total = (im2col ? (uint64_t)tp.tiles_m : (uint64_t)g.n * tp.tiles_h * tp.tiles_w) * tp.tiles_n;
  if (total >= 0x7fffffffull) { err = "conv: too many tiles"; return -ZYXB_ERR_INCORRECT_KERNEL_ARG; }
  const unsigned grid = (unsigned)std::min<uint64_t>(total, (uint64_t)lc.sm_count);
  cudaError_t e;
  if (im2col) e = bn == 256 ? launch_conv_tc<256, 4, true>(mx, mw, tp, grid, lc.stream) : launch_conv_tc<128, 6, true>(mx, mw, tp, grid, lc.stream);
  else e = bn == 256 ? launch_conv_tc<256, 4, false>(mx, mw, tp, grid, lc.stream) : launch_conv_tc<128, 6, false>(mx, mw, tp, grid, lc.stream);
  if (e != cudaSuccess) { err = std::string("conv_tcgen05: ") + cudaGetErrorString(e); return -ZYXB_ERR_KERNEL_LAUNCH; }
  *lc.launch_counter += (in_place || (phase && phase->x_ready)) ? 2 : 3;
  return 1;
}

template <typename T>
int launch_conv_direct(const ConvGeom& g, int channels_last, int flipped, const void* x, const void* w, const void* bias, void* y, const LaunchCtx& lc, std::string& err) {
  using S = typename Elem<T>::store_t;
  const uint64_t total = (uint64_t)g.n * g.o * g.oh * g.ow;
  const unsigned grid = (unsigned)std::min<uint64_t>((total + 255) / 256, (uint64_t)lc.sm_count * 16);
  conv_direct_kernel<T><<<grid, 256, 0, lc.stream>>>(reinterpret_cast<const S*>(x), reinterpret_cast<const S*>(w), reinterpret_cast<const S*>(bias),
                                                     reinterpret_cast<S*>(y), g, total, lc.round_nearest ? 1 : 0, channels_last, flipped);
  return check_launch(lc, err, "conv_direct");
}

// input gradient, direct form (any stride): dx[n,c,y,x] = sum over (o, r, s) of dy[n,o,i,j] * w[o,c,r,s] for the output
// positions (i, j) whose window element (r, s) is input position (y, x): i*stride_h + r*dil_h - pad_top = y, j alike
template <typename T>
__global__ void conv_dgrad_direct_kernel(const typename Elem<T>::store_t* __restrict__ dy, const typename Elem<T>::store_t* __restrict__ w,
                                         typename Elem<T>::store_t* __restrict__ dx, ConvGeom g, uint64_t total, int rn, int channels_last) {
  using A = typename Elem<T>::acc_t;
  const uint64_t ys_o = channels_last ? 1 : (uint64_t)g.oh * g.ow, ys_p = channels_last ? g.o : 1;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
    uint32_t ix, iy, c;
    uint64_t n, q = i;
    if (channels_last) { c = (uint32_t)(q % g.c); q /= g.c; ix = (uint32_t)(q % g.w); q /= g.w; iy = (uint32_t)(q % g.h); n = q / g.h; }
    else { ix = (uint32_t)(q % g.w); q /= g.w; iy = (uint32_t)(q % g.h); q /= g.h; c = (uint32_t)(q % g.c); n = q / g.c; }
    A acc = 0;
    for (uint32_t o = 0; o < g.o; ++o) {
      const auto* yp = dy + n * g.o * (uint64_t)g.oh * g.ow + o * ys_o;
      const auto* wp = w + ((uint64_t)o * g.c + c) * g.kh * g.kw;
      for (uint32_t r = 0; r < g.kh; ++r) {
        const int ty = (int)iy + g.pt - (int)(r * g.dh);
        if (ty < 0 || ty % (int)g.sh || ty / (int)g.sh >= (int)g.oh) continue;
        for (uint32_t s = 0; s < g.kw; ++s) {
          const int tx = (int)ix + g.pl - (int)(s * g.dw);
          if (tx < 0 || tx % (int)g.sw || tx / (int)g.sw >= (int)g.ow) continue;
          acc += (A)Elem<T>::load(yp[((uint64_t)(ty / (int)g.sh) * g.ow + (uint64_t)(tx / (int)g.sw)) * ys_p]) * (A)Elem<T>::load(wp[r * g.kw + s]);
        }
      }
    }
    dx[i] = Elem<T>::store(acc, rn != 0);
  }
}

template <typename T>
int launch_conv_dgrad_direct(const ConvGeom& g, int channels_last, const void* dy, const void* w, void* dx, const LaunchCtx& lc, std::string& err) {
  using S = typename Elem<T>::store_t;
  const uint64_t total = (uint64_t)g.n * g.c * g.h * g.w;
  const unsigned grid = (unsigned)std::min<uint64_t>((total + 255) / 256, (uint64_t)lc.sm_count * 16);
  conv_dgrad_direct_kernel<T><<<grid, 256, 0, lc.stream>>>(reinterpret_cast<const S*>(dy), reinterpret_cast<const S*>(w), reinterpret_cast<S*>(dx), g, total,
                                                           lc.round_nearest ? 1 : 0, channels_last);
  return check_launch(lc, err, "conv_dgrad_direct");
}

#include "conv_wgrad_impl.cuh"

}  // namespace

int validate_conv(const zyxb_conv_desc& d, std::string& err) {
  ZYXB_CHECK_ARG(d.dtype == ZYXB_BF16 || d.dtype == ZYXB_F16 || d.dtype == ZYXB_F32 || d.dtype == ZYXB_I32, "conv: dtype must be bf16, f16, f32 or i32");
  ConvGeom g;
  if (!geometry(d, g, err)) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  return ZYXB_OK;
}

int launch_conv(const zyxb_conv_desc& d, void* const* args, const uint64_t* arg_bytes, int n_args, const LaunchCtx& lc, std::string& err) {
  ConvGeom g;
  if (!geometry(d, g, err)) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  const int want = d.has_bias ? 4 : 3;
  ZYXB_CHECK_ARG(n_args == want, "conv: expects x, w [,bias] -> y");
  const uint64_t es = dtype_size(d.dtype);
  ZYXB_CHECK_ARG(arg_bytes[0] >= (uint64_t)g.n * g.c * g.h * g.w * es, "conv: x is smaller than [n, c, h, w]");
  ZYXB_CHECK_ARG(arg_bytes[1] >= (uint64_t)g.o * g.c * g.kh * g.kw * es, "conv: w is smaller than [o, c, kh, kw]");
  if (d.has_bias) ZYXB_CHECK_ARG(arg_bytes[2] >= (uint64_t)g.o * es, "conv: bias is smaller than [o]");
  ZYXB_CHECK_ARG(arg_bytes[want - 1] >= (uint64_t)g.n * g.o * g.oh * g.ow * es, "conv: y is smaller than [n, o, oh, ow]");
  const void* x = args[0];
  const void* w = args[1];
  const void* bias = d.has_bias ? args[2] : nullptr;
  void* y = args[want - 1];
  const int took = try_conv_tc(d, g, x, w, bias, y, lc, err);
  if (took < 0) return -took;
  if (took) return ZYXB_OK;
  switch (d.dtype) {
    case ZYXB_F32: return launch_conv_direct<float>(g, d.channels_last != 0, d.flip_filter != 0, x, w, bias, y, lc, err);
    case ZYXB_BF16: return launch_conv_direct<bf16_t>(g, d.channels_last != 0, d.flip_filter != 0, x, w, bias, y, lc, err);
    case ZYXB_F16: return launch_conv_direct<f16_t>(g, d.channels_last != 0, d.flip_filter != 0, x, w, bias, y, lc, err);
    default: return launch_conv_direct<int32_t>(g, d.channels_last != 0, d.flip_filter != 0, x, w, bias, y, lc, err);
  }
}

// One dimension of a phase of a strided input gradient.  Input positions y = a + stride*i (i < count) receive
//   dx[y] = sum over the taps r with (a + pad - r*dil) divisible by stride of dy[i + (a + pad - r*dil)/stride] * w[r].
// Those taps are r0 + t*step (t < taps) and their dy offsets q0 - t*dq, which makes the phase a stride-1 convolution of dy
// with the reversed sub-filter, dilation dq and padding (taps-1)*dq - q0 before / `after` behind.
struct PhaseDim {
  uint32_t count = 0, taps = 0, r0 = 0, step = 1, dq = 1;
  int64_t before = 0, after = 0;
};
PhaseDim phase_dim(uint32_t a, uint32_t extent, uint32_t out_extent, uint32_t k, uint32_t stride, uint32_t dil, int pad) {
  PhaseDim ph;
  if (a >= extent) return ph;
  ph.count = (extent - a + stride - 1) / stride;
  uint32_t gc = stride, t = dil % stride;                 // gcd(dil, stride)
  while (t) { const uint32_t u = gc % t; gc = t; t = u; }
  ph.step = stride / gc; ph.dq = dil / gc;
  int64_t q0 = 0;
  for (uint32_t r = 0; r < k; ++r) {
    const int64_t v = (int64_t)a + pad - (int64_t)r * dil;
    if (((v % (int64_t)stride) + stride) % stride) continue;
    ph.r0 = r; q0 = (v - (((v % (int64_t)stride) + stride) % stride)) / (int64_t)stride;
    ph.taps = (k - 1 - r) / ph.step + 1;
    break;
  }
  if (!ph.taps) return ph;
  ph.before = (int64_t)(ph.taps - 1) * ph.dq - q0;
  ph.after = (int64_t)ph.count + (int64_t)(ph.taps - 1) * ph.dq - ph.before - (int64_t)out_extent;
  return ph;
}

// Strided input gradient on the tensor cores: the input positions fall into stride_h * stride_w residue classes, and each
// class is a stride-1 convolution of dy with the sub-filter of the taps that reach it, its result written to that class's
// positions of dx (ConvPhase).  No zeros are multiplied: the phases together execute exactly the gradient's FLOPs.
// Returns 1 when every phase ran there, 0 when the shape is not for it (nothing useful written), < 0 on an error.
int try_conv_dgrad_phases(const zyxb_conv_desc& d, const ConvGeom& g, const void* dy, const void* w, void* dx, const LaunchCtx& lc, std::string& err) {
  if (d.dtype != ZYXB_BF16 && d.dtype != ZYXB_F16) return 0;
  if (g.sh > 8 || g.sw > 8 || (uint64_t)g.n * g.o * g.oh * g.ow * g.c * g.kh * g.kw < (1ull << 24)) return 0;
  std::vector<PhaseDim> ph_h, ph_w;
  bool empty = false;
  for (uint32_t a = 0; a < g.sh; ++a) ph_h.push_back(phase_dim(a, g.h, g.oh, g.kh, g.sh, g.dh, g.pt));
  for (uint32_t b = 0; b < g.sw; ++b) ph_w.push_back(phase_dim(b, g.w, g.ow, g.kw, g.sw, g.dw, g.pl));
  for (const std::vector<PhaseDim>* v : {&ph_h, &ph_w})
    for (const PhaseDim& q : *v) {
      if (q.count && !q.taps) empty = true;               // positions no window element ever covers: their gradient is zero
      // negative values crop dy instead of padding it: window origins then start later / end earlier, nothing else changes
      if (q.taps && (q.before < -(1 << 20) || q.after < -(1 << 20) || q.before > (1 << 20) || q.after > (1 << 20))) return 0;
    }
  if (empty) {
    const cudaError_t e = cudaMemsetAsync(dx, 0, (size_t)g.n * g.c * g.h * g.w * 2, lc.stream);
    if (e != cudaSuccess) { err = std::string("conv input gradient: ") + cudaGetErrorString(e); return -ZYXB_ERR_KERNEL_LAUNCH; }
  }
  bool x_ready = false;
  for (uint32_t a = 0; a < g.sh; ++a)
    for (uint32_t b = 0; b < g.sw; ++b) {
      const PhaseDim &H = ph_h[a], &W = ph_w[b];
      if (!H.count || !W.count || !H.taps || !W.taps) continue;
      zyxb_conv_desc f = d;                               // dtype and channels_last; the extents travel in the geometry
      f.has_bias = 0; f.flip_filter = 0;
      ConvGeom pg{};
      pg.n = g.n; pg.c = g.o; pg.h = g.oh; pg.w = g.ow; pg.o = g.c; pg.kh = H.taps; pg.kw = W.taps; pg.oh = H.count; pg.ow = W.count;
      pg.sh = pg.sw = 1; pg.dh = H.dq; pg.dw = W.dq; pg.pt = (int)H.before; pg.pl = (int)W.before;
      ConvPhase cp{};
      cp.pad_bottom = (int)H.after; cp.pad_right = (int)W.after;
      cp.r0 = H.r0; cp.step_r = H.step; cp.s0 = W.r0; cp.step_s = W.step; cp.fkh = g.kh; cp.fkw = g.kw;
      cp.full_h = g.h; cp.full_w = g.w; cp.step_h = g.sh; cp.step_w = g.sw; cp.off_h = a; cp.off_w = b;
      cp.x_ready = x_ready;
      const int took = try_conv_tc(f, pg, dy, w, nullptr, dx, lc, err, &cp);
      if (took < 0) return took;
      if (!took) return 0;                                // the caller's direct kernel rewrites every element
      x_ready = true;
    }
  return 1;
}

// Input gradient of the convolution the descriptor names: args dy, w -> dx.  With stride 1 it is itself a convolution
// (of dy, with the filter transposed in (o, c) and reversed in (r, s), padding dil*(k-1) - pad): the forward program with
// flip_filter, tensor cores included.  Other strides split into one such convolution per residue class of the input
// positions (try_conv_dgrad_phases); what neither takes runs the direct kernel.
int launch_conv_dgrad(const zyxb_conv_desc& d, void* const* args, const uint64_t* arg_bytes, int n_args, const LaunchCtx& lc, std::string& err) {
  ConvGeom g;
  if (!geometry(d, g, err)) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  ZYXB_CHECK_ARG(n_args == 3, "conv input gradient: expects dy, w -> dx");
  const uint64_t es = dtype_size(d.dtype);
  ZYXB_CHECK_ARG(arg_bytes[0] >= (uint64_t)g.n * g.o * g.oh * g.ow * es, "conv input gradient: dy is smaller than [n, o, oh, ow]");
  ZYXB_CHECK_ARG(arg_bytes[1] >= (uint64_t)g.o * g.c * g.kh * g.kw * es, "conv input gradient: w is smaller than [o, c, kh, kw]");
  ZYXB_CHECK_ARG(arg_bytes[2] >= (uint64_t)g.n * g.c * g.h * g.w * es, "conv input gradient: dx is smaller than [n, c, h, w]");
  const int64_t eh = (int64_t)g.dh * (g.kh - 1), ew = (int64_t)g.dw * (g.kw - 1);
  const bool as_conv = g.sh == 1 && g.sw == 1 && d.pad_top <= eh && d.pad_bottom <= eh && d.pad_left <= ew && d.pad_right <= ew;
  if (as_conv) {
    zyxb_conv_desc f = d;
    f.c = g.o; f.h = g.oh; f.w = g.ow; f.o = g.c;
    f.pad_top = (uint32_t)(eh - d.pad_top); f.pad_bottom = (uint32_t)(eh - d.pad_bottom);
    f.pad_left = (uint32_t)(ew - d.pad_left); f.pad_right = (uint32_t)(ew - d.pad_right);
    f.has_bias = 0; f.flip_filter = 1;
    void* fargs[3] = {args[0], args[1], args[2]};
    return launch_conv(f, fargs, arg_bytes, 3, lc, err);
  }
  if (!as_conv) {
    static const bool no_phases = getenv("ZYXB_NO_CONV_DGRAD_TC") != nullptr;
    const int took = no_phases ? 0 : try_conv_dgrad_phases(d, g, args[0], args[1], args[2], lc, err);
    if (took < 0) return -took;
    if (took) return ZYXB_OK;
  }
  const int cl = d.channels_last != 0;
  switch (d.dtype) {
    case ZYXB_F32: return launch_conv_dgrad_direct<float>(g, cl, args[0], args[1], args[2], lc, err);
    case ZYXB_BF16: return launch_conv_dgrad_direct<bf16_t>(g, cl, args[0], args[1], args[2], lc, err);
    case ZYXB_F16: return launch_conv_dgrad_direct<f16_t>(g, cl, args[0], args[1], args[2], lc, err);
    default: return launch_conv_dgrad_direct<int32_t>(g, cl, args[0], args[1], args[2], lc, err);
  }
}

int launch_conv_wgrad(const zyxb_conv_desc& d, void* const* args, const uint64_t* arg_bytes, int n_args, const LaunchCtx& lc, std::string& err) {
  ConvGeom g;
  if (!geometry(d, g, err)) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  ZYXB_CHECK_ARG(n_args == 3, "conv weight gradient: expects x, dy -> dw");
  const uint64_t es = dtype_size(d.dtype);
  ZYXB_CHECK_ARG(arg_bytes[0] >= (uint64_t)g.n * g.c * g.h * g.w * es, "conv weight gradient: x is smaller than [n, c, h, w]");
  ZYXB_CHECK_ARG(arg_bytes[1] >= (uint64_t)g.n * g.o * g.oh * g.ow * es, "conv weight gradient: dy is smaller than [n, o, oh, ow]");
  ZYXB_CHECK_ARG(arg_bytes[2] >= (uint64_t)g.o * g.c * g.kh * g.kw * es, "conv weight gradient: dw is smaller than [o, c, kh, kw]");
  const int took = try_conv_wgrad_tc(d, g, args[0], args[1], args[2], lc, err);
  if (took < 0) return -took;
  if (took) return ZYXB_OK;
  const int cl = d.channels_last != 0;
  switch (d.dtype) {
    case ZYXB_F32: return launch_conv_wgrad_direct<float>(g, cl, args[0], args[1], args[2], lc, err);
    case ZYXB_BF16: return launch_conv_wgrad_direct<bf16_t>(g, cl, args[0], args[1], args[2], lc, err);
    case ZYXB_F16: return launch_conv_wgrad_direct<f16_t>(g, cl, args[0], args[1], args[2], lc, err);
    default: return launch_conv_wgrad_direct<int32_t>(g, cl, args[0], args[1], args[2], lc, err);
  }
}

}  // namespace zyxb
