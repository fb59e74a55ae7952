// extern "C" entry points of the library: argument checks, choice of kernel family, error strings.
// Declarations and the reference launch sites they replace are in include/fa_b200.h.
#include <stdarg.h>
#include <stdio.h>

#include <nvtx3/nvToolsExt.h>

#include "fa_common.cuh"

namespace fa {

// NVTX range around a C entry point (host side: argument checks, tensor-map encoding, launches). Header-only NVTX:
// costs a null check per call unless a profiler is attached.
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
};

namespace {
thread_local char g_error[512] = "";
thread_local int g_path = FA_PATH_NONE;
}  // namespace

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

void set_path(int path) { g_path = path; }

namespace {


int check_attn(const fa_attn_params* p, bool backward, bool want_varlen) {
  if (p == nullptr) return set_error(FA_ERR_INVALID_ARGUMENT, "params is NULL");
  if (p->dtype != FA_F16 && p->dtype != FA_BF16 && p->dtype != FA_F32)
    return set_error(FA_ERR_INVALID_ARGUMENT, "unsupported dtype %d; expected float16, bfloat16, float32", p->dtype);
  if ((p->varlen != 0) != want_varlen)
    return set_error(FA_ERR_INVALID_ARGUMENT, "varlen flag does not match the entry point");
  if (p->batch <= 0 || p->heads_q <= 0 || p->heads_kv <= 0 || p->seqlen_q <= 0 || p->seqlen_k <= 0 || p->head_dim <= 0)
    return set_error(FA_ERR_INVALID_ARGUMENT, "batch, heads, sequence lengths and head_dim must be positive");
  if (p->heads_q % p->heads_kv != 0)
    return set_error(FA_ERR_INVALID_ARGUMENT, "query heads must be a multiple of key/value heads");
  // The reference's kernels want a power of two in [16, 512] and its Python layer pads the rest; here every width up
  // to 512 runs as it is (16-bit multiples of 8 up to 128 on the tensor-core kernels, the rest on CUDA cores).
  if (p->head_dim > 512)
    return set_error(FA_ERR_UNSUPPORTED, "head_dim %d not supported; expected at most 512", p->head_dim);
  if (p->q == nullptr || p->k == nullptr || p->v == nullptr || p->out == nullptr || p->lse == nullptr)
    return set_error(FA_ERR_INVALID_ARGUMENT, "q, k, v, out and lse must not be NULL");
  if (p->varlen) {
    if (p->cu_seqlens_q == nullptr || p->cu_seqlens_k == nullptr || p->total_q <= 0 || p->total_k <= 0)
      return set_error(FA_ERR_INVALID_ARGUMENT, "varlen needs cu_seqlens_q, cu_seqlens_k and positive totals");
    if (p->bias != nullptr || p->dropout_p > 0.f)
      return set_error(FA_ERR_UNSUPPORTED, "additive bias and dropout are dense-only");
  }
  if (p->window_left < -1 || p->window_right < -1)
    return set_error(FA_ERR_INVALID_ARGUMENT, "window values must be integers greater than or equal to -1");
  if (!(p->softcap >= 0.f)) return set_error(FA_ERR_INVALID_ARGUMENT, "softcap must be nonnegative");
  if (!(p->dropout_p >= 0.f && p->dropout_p < 1.f))
    return set_error(FA_ERR_INVALID_ARGUMENT, "dropout_p must satisfy 0 <= dropout_p < 1");
  if (p->bias != nullptr && p->bias_dtype != p->dtype && p->bias_dtype != FA_F32)
    return set_error(FA_ERR_INVALID_ARGUMENT, "bias dtype must match query dtype or be float32");
  if (backward) {
    if (p->dout == nullptr || p->delta == nullptr || p->dq == nullptr || p->dk == nullptr || p->dv == nullptr)
      return set_error(FA_ERR_INVALID_ARGUMENT, "dout, delta, dq, dk and dv must not be NULL");
  }
  if (p->force_path != FA_PATH_NONE && p->force_path != FA_PATH_TCGEN05 && p->force_path != FA_PATH_SIMT)
    return set_error(FA_ERR_INVALID_ARGUMENT, "force_path must be 0, FA_PATH_TCGEN05 or FA_PATH_SIMT");
  return 0;
}

int run_fwd(const fa_attn_params* p, void* stream, bool varlen) {
  int rc = check_attn(p, false, varlen);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool wide_ok = !varlen && fwd_wide_supported(*p);  // head dims above 256: dense problems that bring a workspace
  const bool tc_ok = wide_ok || fwd_tcgen05_supported(*p);
  if (p->force_path == FA_PATH_TCGEN05 && !tc_ok)
    return set_error(FA_ERR_UNSUPPORTED, "the tcgen05 forward needs fp16/bf16, a head_dim that is a multiple of 8 up to "
                                         "256 (up to 512 for dense problems without score modifiers that bring a "
                                         "ds_workspace), unit inner strides and 16-byte aligned rows");
  if (tc_ok && p->force_path != FA_PATH_SIMT) {
    set_path(FA_PATH_TCGEN05);
    return wide_ok ? launch_fwd_wide(*p, s) : launch_fwd_tcgen05(*p, s);
  }
  set_path(FA_PATH_SIMT);
  return launch_fwd_simt(*p, s);
}

int run_bwd(const fa_attn_params* p, void* stream, bool varlen) {
  int rc = check_attn(p, true, varlen);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int parts = p->bwd_parts == 0 ? (FA_BWD_DELTA | FA_BWD_DKDV | FA_BWD_DQ) : p->bwd_parts;
  if (parts & FA_BWD_DELTA) {
    rc = launch_bwd_delta(*p, s);
    if (rc) return rc;
  }
  if (!(parts & (FA_BWD_DKDV | FA_BWD_DQ))) return 0;
  const bool wide_ok = bwd_wide_supported(*p);  // head dims above 128: dense problems that bring a workspace
  const bool tc_ok = wide_ok || bwd_tcgen05_supported(*p);
  if (p->force_path == FA_PATH_TCGEN05 && !tc_ok)
    return set_error(FA_ERR_UNSUPPORTED, "the tcgen05 backward needs fp16/bf16, a head_dim that is a multiple of 8 up to "
                                         "128 (up to 512 for dense problems with a ds_workspace; above 256 without score modifiers), unit inner strides and "
                                         "16-byte aligned rows");
  if (tc_ok && p->force_path != FA_PATH_SIMT) {
    set_path(FA_PATH_TCGEN05);
    return wide_ok ? launch_bwd_wide(*p, parts, s) : launch_bwd_tcgen05(*p, parts, s);
  }
  set_path(FA_PATH_SIMT);
  return launch_bwd_simt(*p, parts, s);
}

}  // namespace
}  // namespace fa

extern "C" {

int32_t fa_abi_version(void) { return FA_B200_ABI_VERSION; }

int32_t fa_device_supported(int32_t device) {
  cudaDeviceProp prop;
  cudaError_t e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fa::set_error(FA_ERR_DEVICE, "cannot query CUDA device %d: %s", device, cudaGetErrorString(e));
  }
  if (prop.major != 10)
    return fa::set_error(FA_ERR_UNSUPPORTED, "fa_b200 supports compute capability 10.x (B200), got %d.%d", prop.major,
                         prop.minor);
  return 0;
}

const char* fa_last_error_string(void) { return fa::g_error; }
int32_t fa_last_path(void) { return fa::g_path; }

int32_t fa_fwd(const fa_attn_params* p, void* stream) {
  fa::NvtxRange r("fa_fwd");
  return fa::run_fwd(p, stream, false);
}
int32_t fa_varlen_fwd(const fa_attn_params* p, void* stream) {
  fa::NvtxRange r("fa_varlen_fwd");
  return fa::run_fwd(p, stream, true);
}
int32_t fa_bwd(const fa_attn_params* p, void* stream) {
  fa::NvtxRange r("fa_bwd");
  return fa::run_bwd(p, stream, false);
}
int32_t fa_varlen_bwd(const fa_attn_params* p, void* stream) {
  fa::NvtxRange r("fa_varlen_bwd");
  return fa::run_bwd(p, stream, true);
}

int32_t fa_bwd_delta(const fa_attn_params* p, void* stream) {
  fa::NvtxRange r("fa_bwd_delta");
  if (p == nullptr || p->out == nullptr || p->dout == nullptr || p->delta == nullptr)
    return fa::set_error(FA_ERR_INVALID_ARGUMENT, "delta needs out, dout and delta");
  if (p->batch <= 0 || p->heads_q <= 0 || p->seqlen_q <= 0 || p->head_dim <= 0)
    return fa::set_error(FA_ERR_INVALID_ARGUMENT, "batch, heads, sequence length and head_dim must be positive");
  return fa::launch_bwd_delta(*p, static_cast<cudaStream_t>(stream));
}

int32_t fa_decode_splitk(const fa_decode_params* p, void* stream) {
  fa::NvtxRange r("fa_decode_splitk");
  if (p == nullptr) return fa::set_error(FA_ERR_INVALID_ARGUMENT, "params is NULL");
  if (p->batch <= 0 || p->heads_q <= 0 || p->heads_kv <= 0 || p->seqlen_q <= 0 || p->seqlen_k <= 0)
    return fa::set_error(FA_ERR_INVALID_ARGUMENT, "batch, heads and sequence lengths must be positive");
  if (p->q == nullptr || p->k == nullptr || p->v == nullptr || p->out == nullptr)
    return fa::set_error(FA_ERR_INVALID_ARGUMENT, "q, k, v and out must not be NULL");
  return fa::launch_decode_splitk(*p, static_cast<cudaStream_t>(stream));
}

int32_t fa_combine(const fa_combine_params* p, void* stream) {
  fa::NvtxRange r("fa_combine");
  if (p == nullptr || p->o_partial == nullptr || p->lse_partial == nullptr || p->out == nullptr)
    return fa::set_error(FA_ERR_INVALID_ARGUMENT, "combine needs o_partial, lse_partial and out");
  return fa::launch_combine(*p, static_cast<cudaStream_t>(stream));
}

int32_t fa_peer_merge(const fa_peer_merge_params* p, void* stream) {
  fa::NvtxRange r("fa_peer_merge");
  if (p == nullptr) return fa::set_error(FA_ERR_INVALID_ARGUMENT, "params is NULL");
  return fa::launch_peer_merge(*p, static_cast<cudaStream_t>(stream));
}

int32_t fa_enable_peer_access(int32_t peer_device) {
  int dev = 0, can = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fa::set_error(FA_ERR_DEVICE, "cudaGetDevice failed: %s", cudaGetErrorString(e));
  if (dev == peer_device) return 0;
  e = cudaDeviceCanAccessPeer(&can, dev, peer_device);
  if (e != cudaSuccess || !can) {
    cudaGetLastError();
    return fa::set_error(FA_ERR_UNSUPPORTED, "device %d has no peer path to device %d", dev, peer_device);
  }
  e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();  // not an error for this call
    return 0;
  }
  if (e != cudaSuccess) return fa::set_error(FA_ERR_DEVICE, "cudaDeviceEnablePeerAccess failed: %s", cudaGetErrorString(e));
  return 0;
}

int32_t fa_decode_paged(const fa_paged_params* p, void* stream) {
  fa::NvtxRange r("fa_decode_paged");
  if (p == nullptr) return fa::set_error(FA_ERR_INVALID_ARGUMENT, "params is NULL");
  if (p->batch <= 0 || p->heads_q <= 0 || p->heads_kv <= 0 || p->num_blocks <= 0 || p->max_blocks <= 0)
    return fa::set_error(FA_ERR_INVALID_ARGUMENT, "paged batch, heads, blocks and block table width must be positive");
  if (p->q == nullptr || p->k_cache == nullptr || p->v_cache == nullptr || p->out == nullptr ||
      p->block_table == nullptr || p->context_lens == nullptr)
    return fa::set_error(FA_ERR_INVALID_ARGUMENT, "q, caches, block_table, context_lens and out must not be NULL");
  return fa::launch_decode_paged(*p, static_cast<cudaStream_t>(stream));
}

int64_t fa_workspace_bytes(int32_t kind, const void* params) {
  if (params == nullptr) return fa::set_error(FA_ERR_INVALID_ARGUMENT, "params is NULL");
  switch (kind) {
    case FA_WS_BWD_DELTA: {
      const fa_attn_params* p = static_cast<const fa_attn_params*>(params);
      if (p->heads_q <= 0 || (p->varlen ? p->total_q <= 0 : (p->batch <= 0 || p->seqlen_q <= 0)))
        return fa::set_error(FA_ERR_INVALID_ARGUMENT, "workspace query: sizes must be positive");
      return 4 * (int64_t)p->heads_q * (p->varlen ? (int64_t)p->total_q : (int64_t)p->batch * p->seqlen_q);
    }
    case FA_WS_BWD_DS: {
      const fa_attn_params* p = static_cast<const fa_attn_params*>(params);
      if (p->batch <= 0 || p->heads_q <= 0 || p->seqlen_q <= 0 || p->seqlen_k <= 0)
        return fa::set_error(FA_ERR_INVALID_ARGUMENT, "workspace query: sizes must be positive");
      if (p->head_dim > 512 || p->head_dim % 8) return 0;
      if (p->dtype == FA_F32) return (p->head_dim > 256 || p->varlen) ? 0 : fa::bwd_wide_workspace_bytes(*p);
      return p->head_dim > 128 ? fa::bwd_wide_workspace_bytes(*p) : fa::bwd_ds_workspace_bytes(*p);
    }
    case FA_WS_FWD_P: {
      const fa_attn_params* p = static_cast<const fa_attn_params*>(params);
      if (p->batch <= 0 || p->heads_q <= 0 || p->seqlen_q <= 0 || p->seqlen_k <= 0)
        return fa::set_error(FA_ERR_INVALID_ARGUMENT, "workspace query: sizes must be positive");
      if (p->head_dim % 8) return 0;
      if (p->dtype == FA_F32 ? p->head_dim > 256 : (p->head_dim <= 256 || p->head_dim > 512)) return 0;
      return fa::fwd_wide_workspace_bytes(*p);
    }
    case FA_WS_DECODE_O_PARTIAL:
    case FA_WS_DECODE_LSE_PARTIAL: {
      const fa_decode_params* p = static_cast<const fa_decode_params*>(params);
      if (p->batch <= 0 || p->heads_q <= 0 || p->seqlen_q <= 0 || p->head_dim <= 0 || p->num_splits < 1)
        return fa::set_error(FA_ERR_INVALID_ARGUMENT, "workspace query: sizes must be positive");
      if (p->num_splits == 1) return 0;
      const int64_t rows = (int64_t)p->num_splits * p->batch * p->heads_q * p->seqlen_q;
      return 4 * rows * (kind == FA_WS_DECODE_O_PARTIAL ? p->head_dim : 1);
    }
    case FA_WS_PAGED_O_PARTIAL:
    case FA_WS_PAGED_LSE_PARTIAL: {
      const fa_paged_params* p = static_cast<const fa_paged_params*>(params);
      if (p->batch <= 0 || p->heads_q <= 0 || p->head_dim <= 0 || p->num_splits < 1)
        return fa::set_error(FA_ERR_INVALID_ARGUMENT, "workspace query: sizes must be positive");
      if (p->num_splits == 1) return 0;
      const int64_t rows = (int64_t)p->num_splits * p->batch * p->heads_q;
      return 4 * rows * (kind == FA_WS_PAGED_O_PARTIAL ? p->head_dim : 1);
    }
  }
  return fa::set_error(FA_ERR_INVALID_ARGUMENT, "unknown workspace kind %d", kind);
}

void fa_test_decode_fault(uint32_t poll_limit, int32_t skip_tile) {
  fa::set_decode_fault_injection(poll_limit, skip_tile);
}

int32_t fa_tiny_fwd(const fa_tiny_params* p, void* stream) {
  fa::NvtxRange r("fa_tiny_fwd");
  if (p == nullptr || p->q == nullptr || p->k == nullptr || p->v == nullptr || p->out == nullptr)
    return fa::set_error(FA_ERR_INVALID_ARGUMENT, "tiny forward needs q, k, v and out");
  return fa::launch_tiny(*p, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
