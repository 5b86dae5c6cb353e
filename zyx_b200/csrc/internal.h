// Host-side declarations shared by the API layer and the kernel launchers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/zyxb.h"

namespace zyxb {

// What a launcher needs to know about the device and the context it runs in.
struct LaunchCtx {
  cudaStream_t stream;
  bool round_nearest;       // bf16/f16 store mode (zyxb_config::round_nearest)
  int sm_count;
  uint32_t* status_word;    // device word: kernels OR an error bit into it when a bounded wait runs out
  void* scratch;            // per-device scratch memory owned by the context (partials of split reductions)
  size_t scratch_bytes;
  uint64_t* launch_counter; // host counter of kernels launched
  void* tma_encode;         // cuTensorMapEncodeTiled entry point (driver), or nullptr
  void* tma_encode_im2col;  // cuTensorMapEncodeIm2col entry point (driver), or nullptr
  int device;
  bool overlap_hint;        // collectives that occupy SMs (NCCL) may run beside the kernels: draw matmul tiles from a queue
};

// Every launcher validates the argument count and the byte size of each buffer before it
// launches anything: a bad argument is reported as ZYXB_ERR_INCORRECT_KERNEL_ARG, never as
// an out-of-bounds access on the device.
int launch_rowreduce(const zyxb_rowreduce_desc& d, void* const* args, const uint64_t* arg_bytes, int n_args,
                     const LaunchCtx& lc, std::string& err);
int launch_eltwise(const zyxb_eltwise_desc& d, void* const* args, const uint64_t* arg_bytes, int n_args,
                   const LaunchCtx& lc, std::string& err);
struct OptimState;  // numel copy + step counter, owned by the program
int launch_optim(const zyxb_optim_desc& d, const uint64_t* numel, uint64_t step, void* const* args,
                 const uint64_t* arg_bytes, int n_args, const LaunchCtx& lc, std::string& err);
int launch_gemm(const zyxb_gemm_desc& d, void* const* args, const uint64_t* arg_bytes, int n_args, const LaunchCtx& lc,
                std::string& err);

int launch_attention(const zyxb_attention_desc& d, void* const* args, const uint64_t* arg_bytes, int n_args, const LaunchCtx& lc,
                     std::string& err);
int launch_attention_bwd(const zyxb_attention_desc& d, void* const* args, const uint64_t* arg_bytes, int n_args, const LaunchCtx& lc,
                         std::string& err);
int validate_attention(const zyxb_attention_desc& d, std::string& err);
int launch_conv(const zyxb_conv_desc& d, void* const* args, const uint64_t* arg_bytes, int n_args, const LaunchCtx& lc, std::string& err);
int validate_conv(const zyxb_conv_desc& d, std::string& err);
int launch_conv_dgrad(const zyxb_conv_desc& d, void* const* args, const uint64_t* arg_bytes, int n_args, const LaunchCtx& lc, std::string& err);
int launch_conv_wgrad(const zyxb_conv_desc& d, void* const* args, const uint64_t* arg_bytes, int n_args, const LaunchCtx& lc, std::string& err);

// column sums with the partials in a fixed device array (no allocation anywhere on the path)
int launch_colsum_static(int dtype, const void* x, void* y, uint64_t rows, uint64_t cols, const LaunchCtx& lc, std::string& err);
uint64_t colsum_static_capacity();
bool colsum_static_ready(int cuda_device);
bool attention_fwd2_supported(const zyxb_attention_desc& d);
int launch_attention_fwd2(const zyxb_attention_desc& d, void* const* args, const LaunchCtx& lc, std::string& err);
int launch_bounded_wait_selftest(uint64_t limit_ns, uint32_t* out_gave_up_dev, const LaunchCtx& lc, std::string& err);

int validate_rowreduce(const zyxb_rowreduce_desc& d, std::string& err);
int validate_eltwise(const zyxb_eltwise_desc& d, std::string& err);
int validate_optim(const zyxb_optim_desc& d, std::string& err);
int validate_gemm(const zyxb_gemm_desc& d, std::string& err);

inline uint64_t dtype_size(int dtype) {
  switch (dtype) {
    case ZYXB_BF16: case ZYXB_F16: case ZYXB_U16: case ZYXB_I16: return 2;
    case ZYXB_F32: case ZYXB_U32: case ZYXB_I32: return 4;
    case ZYXB_F64: case ZYXB_U64: case ZYXB_I64: return 8;
    default: return 1;
  }
}

#define ZYXB_CHECK_ARG(cond, msg)                         \
  do {                                                    \
    if (!(cond)) {                                        \
      err = std::string(msg);                             \
      return ZYXB_ERR_INCORRECT_KERNEL_ARG;               \
    }                                                     \
  } while (0)

inline int check_launch(const LaunchCtx& lc, std::string& err, const char* what, int n_kernels = 1) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    err = std::string(what) + ": " + cudaGetErrorString(e);
    return ZYXB_ERR_KERNEL_LAUNCH;
  }
  *lc.launch_counter += (uint64_t)n_kernels;
  return ZYXB_OK;
}

}  // namespace zyxb
