#include "ttt_internal.h"
int ttt_launch_backward(const ttt_b200_bwd_args*, cudaStream_t, uint32_t*, uint64_t) {
  return ttt_set_error(TTT_B200_ERR_LAUNCH, "backward kernel not built yet");
}
