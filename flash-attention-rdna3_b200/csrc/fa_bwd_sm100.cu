// placeholder until the tcgen05 backward lands
#include "fa_common.cuh"
namespace fa {
bool bwd_tcgen05_supported(const fa_attn_params&) { return false; }
int launch_bwd_tcgen05(const fa_attn_params&, cudaStream_t) { return set_error(FA_ERR_UNSUPPORTED, "not built"); }
}
