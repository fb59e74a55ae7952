// The tiled dq family of the tiled CUDA-core kernels (fa_tiled.cuh).
#include "fa_tiled.cuh"

namespace fa {

int launch_tiled_dq(const fa_attn_params& p, cudaStream_t stream) {
  launch_tiled<kTiledDq>(p, stream);
  return check_launch("tiled dq");
}

}  // namespace fa
