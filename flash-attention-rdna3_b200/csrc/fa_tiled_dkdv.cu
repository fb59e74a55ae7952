// The tiled dkdv family of the tiled CUDA-core kernels (fa_tiled.cuh).
#include "fa_tiled.cuh"

namespace fa {

int launch_tiled_dkdv(const fa_attn_params& p, cudaStream_t stream) {
  launch_tiled<kTiledDkdv>(p, stream);
  return check_launch("tiled dkdv");
}

}  // namespace fa
