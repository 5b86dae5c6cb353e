#include "gemm.h"
namespace zyxb {
bool gemm_tc_supported(const GemmParams&, int, const LaunchCtx&) { return false; }
int launch_gemm_tc(const GemmParams&, int, const LaunchCtx&, std::string& err) { err = "no tensor-core path"; return ZYXB_ERR_KERNEL_LAUNCH; }
}
