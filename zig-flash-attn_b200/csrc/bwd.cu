#include "common.h"
namespace b200fa {
size_t bwd_workspace_bytes(const b200fa_problem&) { return 0; }
int launch_bwd(const b200fa_bwd_args&, cudaStream_t) {
  set_error("backward not built yet");
  return B200FA_ERR_UNSUPPORTED;
}
}  // namespace b200fa
