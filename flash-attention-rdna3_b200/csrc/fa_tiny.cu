// FP32 short-sequence attention: head_dim 128, at most 32 keys, non-causal, optional additive bias.
// One warp per query row, registers only: each lane holds four consecutive head-dim elements of the
// query and of the accumulator, lane n ends up holding the score of key n, and the softmax is the
// plain two-pass form. A row whose scores are all -inf produces zeros.
// Semantics: fa_rdna3/kernels/tiny.py:10-85.
#include "fa_common.cuh"

namespace fa {
namespace {

__global__ void __launch_bounds__(128) tiny_fwd_kernel(const fa_tiny_params p) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int flat = blockIdx.x * 4 + warp;
  const int total = p.batch * p.heads * p.seqlen;
  if (flat >= total) return;
  const int i = flat % p.seqlen, h = (flat / p.seqlen) % p.heads, b = flat / (p.seqlen * p.heads);

  const float qs = p.softmax_scale * kLog2e;
  const float* qrow = p.q + (int64_t)b * p.q_strides[0] + (int64_t)h * p.q_strides[1] + (int64_t)i * p.q_strides[2];
  float q[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) q[e] = qrow[(int64_t)(lane * 4 + e) * p.q_strides[3]] * qs;

  float score = kNegInf;  // lane n keeps key n's score
  for (int n = 0; n < p.seqlen; ++n) {
    const float* krow =
        p.k + (int64_t)b * p.k_strides[0] + (int64_t)h * p.k_strides[1] + (int64_t)n * p.k_strides[2];
    float d = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) d += q[e] * krow[(int64_t)(lane * 4 + e) * p.k_strides[3]];
    for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
    if (p.bias != nullptr) {
      const int64_t off = (int64_t)b * p.bias_strides[0] + (int64_t)h * p.bias_strides[1] +
                          (int64_t)i * p.bias_strides[2] + (int64_t)n * p.bias_strides[3];
      d += load_as_float(p.bias, off, p.bias_dtype) * kLog2e;
    }
    if (lane == n) score = d;
  }
  float mx = score;
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  const float mx_safe = (mx == kNegInf) ? 0.f : mx;
  const float prob = (lane < p.seqlen && mx != kNegInf) ? exp2f(score - mx_safe) : 0.f;
  float den = prob;
  for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
  const float den_safe = (den == 0.f) ? 1.f : den;

  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int n = 0; n < p.seqlen; ++n) {
    const float pn = __shfl_sync(0xffffffffu, prob, n);
    const float* vrow =
        p.v + (int64_t)b * p.v_strides[0] + (int64_t)h * p.v_strides[1] + (int64_t)n * p.v_strides[2];
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[e] += pn * vrow[(int64_t)(lane * 4 + e) * p.v_strides[3]];
  }
  float* orow = p.out + (int64_t)b * p.o_strides[0] + (int64_t)h * p.o_strides[1] + (int64_t)i * p.o_strides[2];
#pragma unroll
  for (int e = 0; e < 4; ++e) orow[(int64_t)(lane * 4 + e) * p.o_strides[3]] = acc[e] / den_safe;
}

}  // namespace

int launch_tiny(const fa_tiny_params& p, cudaStream_t stream) {
  if (p.head_dim != 128) return set_error(FA_ERR_UNSUPPORTED, "tiny forward needs head_dim 128, got %d", p.head_dim);
  if (p.seqlen < 1 || p.seqlen > 32)
    return set_error(FA_ERR_UNSUPPORTED, "tiny forward needs 1 <= seqlen <= 32, got %d", p.seqlen);
  if (p.batch < 1 || p.heads < 1) return set_error(FA_ERR_INVALID_ARGUMENT, "tiny forward: empty batch or heads");
  const int total = p.batch * p.heads * p.seqlen;
  tiny_fwd_kernel<<<(total + 3) / 4, 128, 0, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "tiny forward launch failed: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace fa
