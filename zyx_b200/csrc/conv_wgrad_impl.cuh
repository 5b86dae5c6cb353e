// Weight gradient of the convolution in conv_tcgen05.cu (included there, inside its unnamed namespace):
//   dw[o,c,r,s] = sum over (n, i, j) of  dy[n,o,i,j] * x[n, c, i*stride_h + r*dil_h - pad_top, j*stride_w + s*dil_w - pad_left]
// the adjoint of Tensor::conv with respect to its filter (zyx/src/graph/autograd.rs: the expand of the filter over
// (n, i, j) turns into a sum over them).
//
// bf16 / f16 with enough work: per filter tap (r, s) this is a matmul  dw_tap [O x C] = dy_t^T [O x P] . X_tap [P x C]
// over the P = n*oh*ow output positions, with X_tap never materialised:
//   A  dy as [P][O] (positions outer): tiled TMA boxes {64 filters, 64 positions}, M-major in shared memory
//   B  x as [n,h,w,c]: im2col-mode TMA loads of 64 consecutive positions x 64 channels at the tap's offset, N-major
//   D  128 filters x BN channels f32 in TMEM
// The matrix is small (O x C per tap) and the sum long (P), so the positions are split over CTAs: CTA (tap, filter
// block, channel block, split) sums its range of positions and writes an f32 partial tile to scratch; a second kernel
// adds the partials in split order (deterministic) and stores dw [o,c,kh,kw] in the tensor dtype.
#pragma once

constexpr int WG_BK = 64;   // positions per k-block

struct ConvWgParams {
  float* partial;                     // [splits][taps][o_pad][c_pad] f32
  ConvGeom g;
  uint32_t positions, k_blocks, blocks_per_split, splits;
  uint32_t tiles_o, tiles_c, o_pad, c_pad;
  uint32_t o_ext, c_ext;              // extents of the two tensor maps' innermost dimensions (o and c rounded up to 8)
  int is_bf16;
  uint32_t* status;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(CV_THREADS, 1)
conv_wgrad_tc_kernel(const __grid_constant__ CUtensorMap tma_dy, const __grid_constant__ CUtensorMap tma_x, ConvWgParams p) {
  using SM = ConvSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
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
  const uint32_t taps = g.kh * g.kw, plane = g.oh * g.ow;
  const uint32_t total_tiles = taps * p.tiles_o * p.tiles_c * p.splits;
  // splits vary fastest: the CTAs of one (tap, filter block, channel block) run together and finish together
  auto tile_coords = [&](uint32_t t, uint32_t& split, uint32_t& tc, uint32_t& to, uint32_t& tap) {
    split = t % p.splits; t /= p.splits;
    tc = t % p.tiles_c; t /= p.tiles_c;
    to = t % p.tiles_o;
    tap = t / p.tiles_o;
  };
  auto kb_range = [&](uint32_t split, uint32_t& kb0, uint32_t& kb1) {
    kb0 = split * p.blocks_per_split;
    kb1 = min(p.k_blocks, kb0 + p.blocks_per_split);
  };

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, issued = 0;
      bool ok = true;
      for (uint32_t t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        uint32_t split, tc, to, tap, kb0, kb1;
        tile_coords(t, split, tc, to, tap);
        kb_range(split, kb0, kb1);
        const uint16_t off_w = (uint16_t)((tap % g.kw) * g.dw), off_h = (uint16_t)((tap / g.kw) * g.dh);
        for (uint32_t kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, p.status, CV_ERR_PRODUCER)) { ok = false; break; }
          const uint32_t a_dst = base + stage * SM::STAGE_BYTES, b_dst = a_dst + SM::A_BYTES;
          // Chunks of 64 filters / channels that lie wholly past the tensor's extent are not loaded: their shared memory
          // keeps whatever it held and feeds only rows / columns of the accumulator that nothing reads.
          uint32_t chunks = 0;
#pragma unroll
          for (int j = 0; j < CV_BM / 64; ++j) chunks += (to * CV_BM + j * 64 < p.o_ext) ? 1u : 0u;
#pragma unroll
          for (int j = 0; j < BN / 64; ++j) chunks += (tc * BN + j * 64 < p.c_ext) ? 1u : 0u;
          mbar_expect_tx(full_bar(stage), chunks * (64 * WG_BK * 2));
          const uint32_t pos0 = kb * WG_BK;                 // first position of the block: image, row, column
          const uint32_t img = pos0 / plane, rem = pos0 - img * plane, oy = rem / g.ow, ox = rem - oy * g.ow;
#pragma unroll
          for (int j = 0; j < CV_BM / 64; ++j)              // dy_t [P][O]: boxes of 64 filters x 64 positions
            if (to * CV_BM + j * 64 < p.o_ext)
              tma_load_4d(a_dst + j * (64 * WG_BK * 2), &tma_dy, full_bar(stage), (int)(to * CV_BM) + j * 64, (int)pos0, 0, 0);
#pragma unroll
          for (int j = 0; j < BN / 64; ++j)                 // 64 positions x 64 channels of x at the tap's offset
            if (tc * BN + j * 64 < p.c_ext)
              tma_load_im2col_4d(b_dst + j * (64 * WG_BK * 2), &tma_x, full_bar(stage), (int)(tc * BN) + j * 64, (int)(ox * g.sw) - g.pl,
                                 (int)(oy * g.sh) - g.pt, (int)img, off_w, off_h);
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
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
    if (lane == 0) {
      const uint32_t idesc = make_idesc(p.is_bf16 != 0, true, true, CV_BM, BN);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (uint32_t t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        uint32_t split, tc, to, tap, kb0, kb1;
        tile_coords(t, split, tc, to, tap);
        kb_range(split, kb0, kb1);
        if (kb0 >= kb1) continue;                            // nothing to sum: the epilogue writes zeros without waiting
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, abort_flag, p.status, CV_ERR_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (uint32_t kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, CV_ERR_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = base + stage * SM::STAGE_BYTES, b_addr = a_addr + SM::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < WG_BK / CV_UMMA_K; ++kk) {
            // both operands MN-major: 16 k-rows of 128 B = 2048 B per step; 64-element chunks along M / N are 8 KB apart
            const uint64_t adesc = make_smem_desc(a_addr + kk * (CV_UMMA_K * 128), 64 * WG_BK * 2, 1024);
            const uint64_t bdesc = make_smem_desc(b_addr + kk * (CV_UMMA_K * 128), 64 * WG_BK * 2, 1024);
            umma_f16(d_tmem, adesc, bdesc, idesc, (kb != kb0 || kk != 0) ? 1u : 0u);
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
    const int col_half = (warp - 2) >> 2;
    const uint32_t quarter = (uint32_t)(warp & 3);
    const uint32_t row_in_tile = quarter * 32 + lane;
    uint32_t acc = 0, acc_phase = 0;
    for (uint32_t t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      uint32_t split, tc, to, tap, kb0, kb1;
      tile_coords(t, split, tc, to, tap);
      kb_range(split, kb0, kb1);
      const bool empty = kb0 >= kb1;                        // a split past the last block: its partial is zero
      if (!empty) {
        if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, CV_ERR_EPILOGUE)) break;
        tc_fence_after();
      }
      const uint32_t o = to * CV_BM + row_in_tile;
      float* prow = p.partial + (((size_t)split * taps + tap) * p.o_pad + o) * p.c_pad + (size_t)tc * BN;
#pragma unroll 1
      for (int ch = col_half * (BN / 64); ch < (col_half + 1) * (BN / 64); ++ch) {
        uint32_t r[32];
        if (!empty) {
          tmem_ld32(tmem_base + ((quarter * 32u) << 16) + acc * BN + ch * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<uint4*>(prow + ch * 32 + q * 4) = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
      }
      if (!empty) {
        tc_fence_before();
        mbar_arrive(tempty_bar(acc));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
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

// dw[o][c][tap] = sum over the splits, in split order, of partial[split][tap][o][c]; stored in the tensor dtype
template <typename T>
__global__ void conv_wgrad_finish_kernel(const float* __restrict__ partial, typename Elem<T>::store_t* __restrict__ dw, uint32_t o_count, uint32_t c_count,
                                         uint32_t taps, uint32_t o_pad, uint32_t c_pad, uint32_t splits, int rn) {
  const uint64_t total = (uint64_t)o_count * c_count * taps;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
    // consecutive threads take consecutive channels of one (tap, filter): coalesced reads of the partials
    const uint32_t c = (uint32_t)(i % c_count);
    const uint64_t q = i / c_count;
    const uint32_t o = (uint32_t)(q % o_count), tap = (uint32_t)(q / o_count);
    float acc = 0.0f;
    for (uint32_t s = 0; s < splits; ++s) acc += partial[(((size_t)s * taps + tap) * o_pad + o) * c_pad + c];
    dw[((size_t)o * c_count + c) * taps + tap] = Elem<T>::store(acc, rn != 0);
  }
}

// direct form: one thread per filter element, summing over (n, i, j) in that order
template <typename T>
__global__ void conv_wgrad_direct_kernel(const typename Elem<T>::store_t* __restrict__ x, const typename Elem<T>::store_t* __restrict__ dy,
                                         typename Elem<T>::store_t* __restrict__ dw, ConvGeom g, uint64_t total, int rn, int channels_last) {
  using A = typename Elem<T>::acc_t;
  const uint64_t xs_c = channels_last ? 1 : (uint64_t)g.h * g.w, xs_p = channels_last ? g.c : 1;
  const uint64_t ys_o = channels_last ? 1 : (uint64_t)g.oh * g.ow, ys_p = channels_last ? g.o : 1;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t s = (uint32_t)(i % g.kw);
    uint64_t q = i / g.kw;
    const uint32_t r = (uint32_t)(q % g.kh); q /= g.kh;
    const uint32_t c = (uint32_t)(q % g.c);
    const uint32_t o = (uint32_t)(q / g.c);
    A acc = 0;
    for (uint32_t n = 0; n < g.n; ++n) {
      const auto* xp = x + (uint64_t)n * g.c * g.h * g.w + c * xs_c;
      const auto* yp = dy + (uint64_t)n * g.o * g.oh * g.ow + o * ys_o;
      for (uint32_t oy = 0; oy < g.oh; ++oy) {
        const int iy = (int)(oy * g.sh + r * g.dh) - g.pt;
        if (iy < 0 || iy >= (int)g.h) continue;
        for (uint32_t ox = 0; ox < g.ow; ++ox) {
          const int ix = (int)(ox * g.sw + s * g.dw) - g.pl;
          if (ix < 0 || ix >= (int)g.w) continue;
          acc += (A)Elem<T>::load(yp[((uint64_t)oy * g.ow + ox) * ys_p]) * (A)Elem<T>::load(xp[((uint64_t)iy * g.w + ix) * xs_p]);
        }
      }
    }
    dw[i] = Elem<T>::store(acc, rn != 0);
  }
}

template <int BN, int STAGES>
cudaError_t launch_conv_wgrad_tc(const CUtensorMap& mdy, const CUtensorMap& mx, const ConvWgParams& wp, unsigned grid, cudaStream_t s) {
  using SM = ConvSmem<BN, STAGES>;
  static uint64_t configured = 0;
  auto kern = conv_wgrad_tc_kernel<BN, STAGES>;
  {
    cudaError_t e = ensure_dynamic_smem(kern, SM::TOTAL, &configured);
    if (e != cudaSuccess) return e;
  }
  kern<<<grid, CV_THREADS, SM::TOTAL, s>>>(mdy, mx, wp);
  return cudaGetLastError();
}

// channels-first [n][ch][hw] -> [n][hw][chp] in scratch (shared by x and dy)
inline void conv_to_channels_last(const void* src, uint16_t* dst, uint32_t n, uint32_t ch, uint32_t chp, uint32_t hw, cudaStream_t s) {
  if (hw % 2 == 0 && (uintptr_t)src % 4 == 0)
    conv_nhwc_pairs_kernel<<<dim3((hw + 63) / 64, (chp + 63) / 64, n), 256, 0, s>>>(reinterpret_cast<const uint16_t*>(src), dst, ch, chp, hw);
  else
    conv_nhwc_kernel<<<dim3((hw + 31) / 32, (chp + 31) / 32, n), dim3(32, 8), 0, s>>>(reinterpret_cast<const uint16_t*>(src), dst, ch, chp, hw);
}

// The tensor-core path: 1 = took the launch, 0 = not for it, < 0 = error (err set).
int try_conv_wgrad_tc(const zyxb_conv_desc& d, const ConvGeom& g, const void* x, const void* dy, void* dw, const LaunchCtx& lc, std::string& err) {
  static const bool off = getenv("ZYXB_NO_CONV_TC") != nullptr;
  if (off || !lc.tma_encode || !lc.tma_encode_im2col || (d.dtype != ZYXB_BF16 && d.dtype != ZYXB_F16)) return 0;
  const uint64_t positions = (uint64_t)g.n * g.oh * g.ow, kdim = (uint64_t)g.c * g.kh * g.kw;
  if (positions * g.o * kdim < (1ull << 22) || positions < 512 || positions >= 0x7fffff00ull) return 0;
  if (g.sw > 8 || g.sh > 8) return 0;
  const int lo_w = -g.pl, lo_h = -g.pt;
  const int up_w = (int)d.pad_right - (int)((g.kw - 1) * g.dw), up_h = (int)d.pad_bottom - (int)((g.kh - 1) * g.dh);
  if (lo_w < -128 || lo_h < -128 || up_w < -128 || up_w > 127 || up_h < -128 || up_h > 127 || (g.kw - 1) * g.dw > 255 || (g.kh - 1) * g.dh > 255) return 0;
  const bool in_place = d.channels_last != 0;
  if (in_place && (g.c % 8 || g.o % 8 || (uintptr_t)x % 16 || (uintptr_t)dy % 16)) return 0;
  const uint32_t cp = (g.c + 7) / 8 * 8, op = (g.o + 7) / 8 * 8, taps = g.kh * g.kw;
  const int bn = g.c > 128 ? 256 : 128;
  ConvWgParams wp{};
  wp.g = g; wp.positions = (uint32_t)positions; wp.k_blocks = (uint32_t)((positions + WG_BK - 1) / WG_BK);
  wp.tiles_o = (g.o + CV_BM - 1) / CV_BM; wp.tiles_c = (g.c + bn - 1) / bn;
  wp.o_pad = wp.tiles_o * CV_BM; wp.c_pad = wp.tiles_c * bn; wp.o_ext = op; wp.c_ext = cp;
  // positions split so that the grid about fills the SMs, with at least eight k-blocks per split
  const uint32_t base_tiles = taps * wp.tiles_o * wp.tiles_c;
  uint32_t splits = std::max(1u, (uint32_t)lc.sm_count / base_tiles);
  splits = std::min(splits, std::max(1u, wp.k_blocks / 8));
  wp.blocks_per_split = (wp.k_blocks + splits - 1) / splits;
  wp.splits = (wp.k_blocks + wp.blocks_per_split - 1) / wp.blocks_per_split;
  wp.is_bf16 = d.dtype == ZYXB_BF16 ? 1 : 0; wp.status = lc.status_word;
  // scratch: [x channels-last] [dy channels-last] [partials]
  auto up = [](size_t v) { return (v + 1023) / 1024 * 1024; };
  const size_t xt_bytes = in_place ? 0 : up((size_t)g.n * g.h * g.w * cp * 2), dyt_bytes = in_place ? 0 : up((size_t)positions * op * 2);
  const size_t part_bytes = (size_t)wp.splits * taps * wp.o_pad * wp.c_pad * 4;
  if (xt_bytes + dyt_bytes + part_bytes > lc.scratch_bytes || (uintptr_t)lc.scratch % 1024) return 0;
  char* sc = reinterpret_cast<char*>(lc.scratch);
  uint16_t* xt = in_place ? reinterpret_cast<uint16_t*>(const_cast<void*>(x)) : reinterpret_cast<uint16_t*>(sc);
  uint16_t* dyt = in_place ? reinterpret_cast<uint16_t*>(const_cast<void*>(dy)) : reinterpret_cast<uint16_t*>(sc + xt_bytes);
  wp.partial = reinterpret_cast<float*>(sc + xt_bytes + dyt_bytes);
  const bool bf16 = d.dtype == ZYXB_BF16;
  const CUtensorMapDataType dt = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap mdy, mx;
  if (!encode_map(lc.tma_encode, &mdy, bf16, dyt, op, positions, op, 1, 0, 1, 0, WG_BK)) return 0;
  {
    cuuint64_t dims[4] = {cp, g.w, g.h, g.n};
    cuuint64_t strides[3] = {(cuuint64_t)cp * 2, (cuuint64_t)g.w * cp * 2, (cuuint64_t)g.h * g.w * cp * 2};
    cuuint32_t estr[4] = {1, g.sw, g.sh, 1};
    const int lower[2] = {lo_w, lo_h}, upper[2] = {up_w, up_h};
    if (reinterpret_cast<EncodeIm2colFn>(lc.tma_encode_im2col)(&mx, dt, 4, xt, dims, strides, lower, upper, 64, WG_BK, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return 0;
  }
  int n_kernels = 2;
  if (!in_place) {
    conv_to_channels_last(x, xt, g.n, g.c, cp, g.h * g.w, lc.stream);
    conv_to_channels_last(dy, dyt, g.n, g.o, op, g.oh * g.ow, lc.stream);
    n_kernels += 2;
  }
  const uint64_t total = (uint64_t)base_tiles * wp.splits;
  const unsigned grid = (unsigned)std::min<uint64_t>(total, (uint64_t)lc.sm_count);
  cudaError_t e = bn == 256 ? launch_conv_wgrad_tc<256, 4>(mdy, mx, wp, grid, lc.stream) : launch_conv_wgrad_tc<128, 6>(mdy, mx, wp, grid, lc.stream);
  if (e != cudaSuccess) { err = std::string("conv_wgrad_tcgen05: ") + cudaGetErrorString(e); return -ZYXB_ERR_KERNEL_LAUNCH; }
  const uint64_t n_out = (uint64_t)g.o * g.c * taps;
  const unsigned fgrid = (unsigned)std::min<uint64_t>((n_out + 255) / 256, (uint64_t)lc.sm_count * 8);
  const int rn = lc.round_nearest ? 1 : 0;
  if (bf16) conv_wgrad_finish_kernel<bf16_t><<<fgrid, 256, 0, lc.stream>>>(wp.partial, reinterpret_cast<uint16_t*>(dw), g.o, g.c, taps, wp.o_pad, wp.c_pad, wp.splits, rn);
  else conv_wgrad_finish_kernel<f16_t><<<fgrid, 256, 0, lc.stream>>>(wp.partial, reinterpret_cast<uint16_t*>(dw), g.o, g.c, taps, wp.o_pad, wp.c_pad, wp.splits, rn);
  if ((e = cudaGetLastError()) != cudaSuccess) { err = std::string("conv_wgrad_finish: ") + cudaGetErrorString(e); return -ZYXB_ERR_KERNEL_LAUNCH; }
  *lc.launch_counter += (uint64_t)n_kernels;
  return 1;
}

template <typename T>
int launch_conv_wgrad_direct(const ConvGeom& g, int channels_last, const void* x, const void* dy, void* dw, const LaunchCtx& lc, std::string& err) {
  using S = typename Elem<T>::store_t;
  const uint64_t total = (uint64_t)g.o * g.c * g.kh * g.kw;
  const unsigned grid = (unsigned)std::min<uint64_t>((total + 127) / 128, (uint64_t)lc.sm_count * 16);
  conv_wgrad_direct_kernel<T><<<grid, 128, 0, lc.stream>>>(reinterpret_cast<const S*>(x), reinterpret_cast<const S*>(dy), reinterpret_cast<S*>(dw), g, total,
                                                           lc.round_nearest ? 1 : 0, channels_last);
  return check_launch(lc, err, "conv_wgrad_direct");
}
