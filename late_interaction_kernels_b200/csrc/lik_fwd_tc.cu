// tcgen05 forward (placeholder until the kernel lands).
#include "lik_common.cuh"
namespace lik {
bool fwd_tc_supported(const lik_fwd_args&) { return false; }
size_t fwd_tc_workspace(const lik_fwd_args&) { return 0; }
int launch_fwd_tc(const lik_fwd_args&, const float*, const float*, void*, size_t, cudaStream_t) {
  set_error("tcgen05 forward not built");
  return LIK_ERR_UNSUPPORTED;
}
}  // namespace lik
