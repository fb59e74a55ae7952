// Per-sequence view of a dense or packed attention problem, the score modifiers of one (batch, head) and the
// backward's per-pair arithmetic: shared by the CUDA-core kernel files (fa_simt.cu, fa_tiled_*.cu).
#pragma once
#include "fa_common.cuh"

namespace fa {
namespace {

struct SeqView {
  int b, h, hk;
  int seqlen_q, seqlen_k;
  int64_t q_off, k_off, v_off, o_off, do_off, dq_off, dk_off, dv_off;  // element offsets of row 0, this head
  int64_t lse_off, delta_off;                                        // offset of row 0
  int64_t lse_row_stride, delta_row_stride;
};

__device__ __forceinline__ bool make_view(const fa_attn_params& P, int b, int h, SeqView* s) {
  s->b = b;
  s->h = h;
  const int group = P.heads_q / P.heads_kv;
  s->hk = h / group;
  int q_start = 0, k_start = 0;
  if (P.varlen) {
    bounded_sequence(P.cu_seqlens_q, b, P.total_q, &q_start, &s->seqlen_q);
    bounded_sequence(P.cu_seqlens_k, b, P.total_k, &k_start, &s->seqlen_k);
  } else {
    s->seqlen_q = P.seqlen_q;
    s->seqlen_k = P.seqlen_k;
  }
  const int64_t bq = P.varlen ? 0 : b, tq = q_start, tk = k_start;
  s->q_off = bq * P.q_strides[0] + (int64_t)h * P.q_strides[1] + tq * P.q_strides[2];
  s->k_off = bq * P.k_strides[0] + (int64_t)s->hk * P.k_strides[1] + tk * P.k_strides[2];
  s->v_off = bq * P.v_strides[0] + (int64_t)s->hk * P.v_strides[1] + tk * P.v_strides[2];
  s->o_off = bq * P.o_strides[0] + (int64_t)h * P.o_strides[1] + tq * P.o_strides[2];
  s->do_off = bq * P.do_strides[0] + (int64_t)h * P.do_strides[1] + tq * P.do_strides[2];
  s->dq_off = bq * P.dq_strides[0] + (int64_t)h * P.dq_strides[1] + tq * P.dq_strides[2];
  s->dk_off = bq * P.dk_strides[0] + (int64_t)s->hk * P.dk_strides[1] + tk * P.dk_strides[2];
  s->dv_off = bq * P.dv_strides[0] + (int64_t)s->hk * P.dv_strides[1] + tk * P.dv_strides[2];
  s->lse_off = bq * P.lse_strides[0] + (int64_t)h * P.lse_strides[1] + tq * P.lse_strides[2];
  s->delta_off = bq * P.delta_strides[0] + (int64_t)h * P.delta_strides[1] + tq * P.delta_strides[2];
  s->lse_row_stride = P.lse_strides[2];
  s->delta_row_stride = P.delta_strides[2];
  return true;
}

__device__ __forceinline__ ScoreMods make_mods(const fa_attn_params& P, const SeqView& s) {
  ScoreMods m;
  m.scale_log2 = P.softmax_scale * kLog2e;
  m.cap_log2 = P.softcap > 0.f ? P.softcap * kLog2e : 0.f;
  m.inv_cap_log2 = P.softcap > 0.f ? 1.f / m.cap_log2 : 0.f;
  m.alibi_slope_log2 = P.alibi_slopes ? P.alibi_slopes[s.h] * kLog2e : 0.f;
  m.bias = nullptr;
  m.bias_dtype = P.bias_dtype;
  m.bias_stride_m = P.bias_strides[2];
  m.bias_stride_n = P.bias_strides[3];
  if (P.bias) {
    const int64_t off = (int64_t)s.b * P.bias_strides[0] + (int64_t)s.h * P.bias_strides[1];
    const int esz = P.bias_dtype == FA_F32 ? 4 : 2;
    m.bias = reinterpret_cast<const char*>(P.bias) + off * esz;
  }
  m.causal = P.causal;
  m.window_left = P.window_left;
  m.window_right = P.window_right;
  m.seqlen_q = s.seqlen_q;
  m.seqlen_k = s.seqlen_k;
  m.dropout_p = P.dropout_p;
  m.inv_keep = P.dropout_p > 0.f ? 1.f / (1.f - P.dropout_p) : 1.f;
  m.dropout_seed = P.dropout_seed;
  m.dropout_base = ((uint64_t)s.b * (uint64_t)P.heads_q + (uint64_t)s.h) * (uint64_t)s.seqlen_q;
  return m;
}

// Probability and score-gradient factor of one (i, j) pair in the backward pass.
//   p      = exp2(logit - lse*log2e), 0 when masked or when the row's lse is -inf
//   p_drop = p with the dropout mask applied (what multiplies dO for dV)
//   ds     = p * (dp_dropped - delta) * (1 - tanh^2)         (fa_rdna3/kernels/_common.py:385-432)
struct PairGrad { float p_drop; float ds; };

__device__ __forceinline__ PairGrad pair_grad(const ScoreMods& mods, float raw_qk, float raw_dp, float lse,
                                              float delta, int i, int j) {
  PairGrad g{0.f, 0.f};
  if (!mods.keep(i, j) || lse == kNegInf) return g;
  float t;
  const float x = mods.logit(raw_qk, i, j, &t);
  const float p = exp2f(x - lse * kLog2e);
  float dp = raw_dp;
  float p_drop = p;
  if (mods.dropout_p > 0.f) {
    const bool kd = mods.dropout_keep(i, j);
    p_drop = kd ? p * mods.inv_keep : 0.f;
    dp = kd ? dp * mods.inv_keep : 0.f;
  }
  float ds = p * (dp - delta);
  if (mods.cap_log2 > 0.f) ds *= (1.f - t * t);
  g.p_drop = p_drop;
  g.ds = ds;
  return g;
}

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "%s launch failed: %s", what, cudaGetErrorString(e));
  return 0;
}

}  // namespace
}  // namespace fa
