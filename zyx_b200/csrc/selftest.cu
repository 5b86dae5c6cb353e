// The bounded-wait self-test: how a wait that can never be satisfied ends.
//
// Every spin-wait of the tensor-core kernels goes through mbar_wait (tc_ptx.cuh): it polls the mbarrier, looks at the wall
// clock every 1024 failed polls and, past its limit, raises the CTA's abort flag, ORs a code into the device status word and
// returns false; the kernel then drains what it has in flight and returns.  The host sees the word through
// zyxb_device_status, which reports ZYXB_ERR_KERNEL_SYNC - zyx's ErrorStatus::KernelSync (zyx/src/error.rs:151-152) - and the
// context stays usable.  This file makes exactly that happen on purpose, with a limit of a millisecond instead of two
// seconds: one CTA initialises one mbarrier that nothing ever arrives on (no copy in flight, no TMEM allocated) and one
// thread waits on it through the same mbar_wait.  Nothing traps, faults or spins past its limit.
#include <cuda_runtime.h>

#include <string>

#include "internal.h"
#include "tc_ptx.cuh"

namespace zyxb {

constexpr uint32_t SELFTEST_STATUS_CODE = 0x8000;

__global__ void bounded_wait_selftest_kernel(uint64_t limit_ns, uint32_t* status, uint32_t* out_gave_up) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_flag, status, SELFTEST_STATUS_CODE, limit_ns);
    *out_gave_up = ok ? 0u : 1u;
  }
}

int launch_bounded_wait_selftest(uint64_t limit_ns, uint32_t* out_gave_up_dev, const LaunchCtx& lc, std::string& err) {
  if (limit_ns == 0 || limit_ns > 100000000ull) { err = "selftest: the limit must be between 1 ns and 100 ms"; return ZYXB_ERR_INCORRECT_KERNEL_ARG; }
  bounded_wait_selftest_kernel<<<1, 32, 0, lc.stream>>>(limit_ns, lc.status_word, out_gave_up_dev);
  return check_launch(lc, err, "bounded wait self-test");
}

}  // namespace zyxb
