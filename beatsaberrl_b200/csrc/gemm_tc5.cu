// placeholder until the tcgen05 engine lands
#include "kernels.cuh"
namespace bsrl {
bool linear_tc5_ok(const LinearArgs&) { return false; }
int linear_tc5(const LinearArgs&, cudaStream_t) {
  set_error("tcgen05 engine not built");
  return BSRL_ERR_UNSUPPORTED;
}
}  // namespace bsrl
