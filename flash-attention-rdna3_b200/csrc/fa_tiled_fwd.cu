// The tiled forward family of the tiled CUDA-core kernels (fa_tiled.cuh).
#include "fa_tiled.cuh"

namespace fa {

int launch_tiled_fwd(const fa_attn_params& p, cudaStream_t stream) {
  launch_tiled<kTiledFwd>(p, stream);
  return check_launch("tiled forward");
}

}  // namespace fa
