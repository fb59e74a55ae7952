// CUDA-core attention kernels that accept everything the public API accepts: fp16 / bf16 / fp32,
// any head_dim up to 512, arbitrary strides, every score modifier, dense and packed layouts.
// They serve the shapes the tensor-core kernels do not take (fp32 inputs, head dims above 256 or not a multiple of 8, the backward above 128,
// non-unit inner strides) and compute in fp32 throughout. Two forms: shared-memory tiled kernels (fa_tiled.cuh,
// launched from here) once both sequences span a tile, and below that the kernels of this file, where one warp owns
// one query row (forward, dQ) or one key row (dK/dV) and its lanes take 32 keys (or queries) at a time.
//
// Semantics follow fa_rdna3/kernels/_common.py:233-508 (inner loops) and
// fa_rdna3/kernels/forward.py:154-161 (empty rows: O = 0, LSE = -inf).
#include "fa_simt_shared.cuh"

namespace fa {
namespace {

constexpr int kWarpsPerBlock = 4;
constexpr int kMaxD = 512;
constexpr int kMaxDPerLane = kMaxD / 32;

__device__ __forceinline__ float warp_max(float x) {
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
__device__ __forceinline__ float warp_sum(float x) {
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// Full dot product of a staged fp32 vector with one global row.
__device__ __forceinline__ float dot_row(const float* vec_s, const void* base, int64_t row_off, int64_t stride_d,
                                         int D, int dtype) {
  float acc = 0.f;
  for (int d = 0; d < D; ++d) acc += vec_s[d] * load_as_float(base, row_off + (int64_t)d * stride_d, dtype);
  return acc;
}

// ---------------------------------------------------------------------------------------------
// delta = rowsum(out * dout)           (fa_rdna3/kernels/backward.py:18-46)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kWarpsPerBlock * 32) simt_delta_kernel(const fa_attn_params P) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int i = blockIdx.x * kWarpsPerBlock + warp;
  const int b = blockIdx.y / P.heads_q, h = blockIdx.y % P.heads_q;
  SeqView s;
  make_view(P, b, h, &s);
  if (i >= s.seqlen_q) return;
  float acc = 0.f;
  for (int d = lane; d < P.head_dim; d += 32) {
    acc += load_as_float(P.out, s.o_off + (int64_t)i * P.o_strides[2] + (int64_t)d * P.o_strides[3], P.dtype) *
           load_as_float(P.dout, s.do_off + (int64_t)i * P.do_strides[2] + (int64_t)d * P.do_strides[3], P.dtype);
  }
  acc = warp_sum(acc);
  if (lane == 0) P.delta[s.delta_off + (int64_t)i * s.delta_row_stride] = acc;
}

// Same, for 16-bit rows of up to D (64, 128 or 256) contiguous elements, a multiple of 8: D/8 lanes cover one row with
// 16-byte loads (lanes past the row's width hold zeros), so a warp reduces 4, 2 or 1 rows at a time. HBM-bound: reads
// O and dO once.
template <typename T, int D>
__global__ void __launch_bounds__(256) delta_vec_kernel(const fa_attn_params P) {
  constexpr int LPR = D / 8;         // lanes per row
  constexpr int RPW = 32 / LPR;      // rows per warp and pass
  constexpr int kPasses = 4;         // rows per lane group: all eight 16-byte loads are issued before the first use
  // the dK/dV kernel launched behind this one waits inside for this grid to finish: its CTAs may set themselves up as
  // SMs free
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int i0 = (blockIdx.x * 8 + warp) * RPW * kPasses + lane / LPR;
  const int b = blockIdx.y / P.heads_q, h = blockIdx.y % P.heads_q;
  SeqView s;
  make_view(P, b, h, &s);
  uint4 ov[kPasses], dv[kPasses];
#pragma unroll
  for (int r = 0; r < kPasses; ++r) {
    const int i = i0 + r * RPW;
    ov[r] = dv[r] = make_uint4(0u, 0u, 0u, 0u);
    if (i < s.seqlen_q && (lane % LPR) * 8 < P.head_dim) {
      ov[r] = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(P.out) + s.o_off + (int64_t)i * P.o_strides[2] +
                                              (lane % LPR) * 8);
      dv[r] = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(P.dout) + s.do_off +
                                              (int64_t)i * P.do_strides[2] + (lane % LPR) * 8);
    }
  }
#pragma unroll
  for (int r = 0; r < kPasses; ++r) {
    const int i = i0 + r * RPW;
    const uint32_t ow[4] = {ov[r].x, ov[r].y, ov[r].z, ov[r].w}, dw[4] = {dv[r].x, dv[r].y, dv[r].z, dv[r].w};
    float acc = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = DType<T>::unpack2(ow[e]), c = DType<T>::unpack2(dw[e]);
      acc += a.x * c.x + a.y * c.y;
    }
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (i < s.seqlen_q && lane % LPR == 0) P.delta[s.delta_off + (int64_t)i * s.delta_row_stride] = acc;
  }
}

// ---------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kWarpsPerBlock * 32) simt_fwd_kernel(const fa_attn_params P) {
  __shared__ float q_s[kWarpsPerBlock][kMaxD];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int i = blockIdx.x * kWarpsPerBlock + warp;
  const int b = blockIdx.y / P.heads_q, h = blockIdx.y % P.heads_q;
  const int D = P.head_dim;
  SeqView s;
  make_view(P, b, h, &s);
  if (i >= s.seqlen_q) return;
  const ScoreMods mods = make_mods(P, s);

  for (int d = lane; d < D; d += 32)
    q_s[warp][d] = load_as_float(P.q, s.q_off + (int64_t)i * P.q_strides[2] + (int64_t)d * P.q_strides[3], P.dtype);
  __syncwarp();

  int lo, hi;
  key_range_for_rows(mods, i, i, &lo, &hi);
  float m = kNegInf, l = 0.f;
  float acc[kMaxDPerLane];
#pragma unroll
  for (int r = 0; r < kMaxDPerLane; ++r) acc[r] = 0.f;

  for (int j0 = lo; j0 < hi; j0 += 32) {
    const int j = j0 + lane;
    float x = kNegInf;
    if (j < hi) {
      const float raw = dot_row(q_s[warp], P.k, s.k_off + (int64_t)j * P.k_strides[2], P.k_strides[3], D, P.dtype);
      x = mods.logit(raw, i, j, nullptr);
      if (!mods.keep(i, j)) x = kNegInf;
    }
    const float m_new = fmaxf(m, warp_max(x));
    const float m_safe = (m_new == kNegInf) ? 0.f : m_new;
    const float alpha = exp2f(m - m_safe);
    float p = exp2f(x - m_safe);
    l = l * alpha + warp_sum(p);
    if (mods.dropout_p > 0.f && j < hi) p = mods.dropout_keep(i, j) ? p * mods.inv_keep : 0.f;
#pragma unroll
    for (int r = 0; r < kMaxDPerLane; ++r) acc[r] *= alpha;
    const int jn = min(32, hi - j0);
    for (int jj = 0; jj < jn; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      if (pj == 0.f) continue;
      const int64_t voff = s.v_off + (int64_t)(j0 + jj) * P.v_strides[2];
#pragma unroll
      for (int r = 0; r < kMaxDPerLane; ++r) {
        const int d = lane + 32 * r;
        if (d < D) acc[r] += pj * load_as_float(P.v, voff + (int64_t)d * P.v_strides[3], P.dtype);
      }
    }
    if (m_new != kNegInf) m = m_new;
  }

  const float l_safe = (l == 0.f) ? 1.f : l;
  const float inv = 1.f / l_safe;
#pragma unroll
  for (int r = 0; r < kMaxDPerLane; ++r) {
    const int d = lane + 32 * r;
    if (d < D)
      store_from_float(P.out, s.o_off + (int64_t)i * P.o_strides[2] + (int64_t)d * P.o_strides[3], P.dtype,
                       acc[r] * inv);
  }
  if (lane == 0) P.lse[s.lse_off + (int64_t)i * s.lse_row_stride] = m * kLn2 + logf(l_safe);
}


// ---------------------------------------------------------------------------------------------
// dQ: one warp per query row                         (fa_rdna3/kernels/backward.py:210-322)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kWarpsPerBlock * 32) simt_bwd_dq_kernel(const fa_attn_params P) {
  __shared__ float q_s[kWarpsPerBlock][kMaxD];
  __shared__ float do_s[kWarpsPerBlock][kMaxD];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int i = blockIdx.x * kWarpsPerBlock + warp;
  const int b = blockIdx.y / P.heads_q, h = blockIdx.y % P.heads_q;
  const int D = P.head_dim;
  SeqView s;
  make_view(P, b, h, &s);
  if (i >= s.seqlen_q) return;
  const ScoreMods mods = make_mods(P, s);
  for (int d = lane; d < D; d += 32) {
    q_s[warp][d] = load_as_float(P.q, s.q_off + (int64_t)i * P.q_strides[2] + (int64_t)d * P.q_strides[3], P.dtype);
    do_s[warp][d] =
        load_as_float(P.dout, s.do_off + (int64_t)i * P.do_strides[2] + (int64_t)d * P.do_strides[3], P.dtype);
  }
  __syncwarp();
  const float lse = P.lse[s.lse_off + (int64_t)i * s.lse_row_stride];
  const float delta = P.delta[s.delta_off + (int64_t)i * s.delta_row_stride];

  int lo, hi;
  key_range_for_rows(mods, i, i, &lo, &hi);
  float acc[kMaxDPerLane];
#pragma unroll
  for (int r = 0; r < kMaxDPerLane; ++r) acc[r] = 0.f;

  for (int j0 = lo; j0 < hi; j0 += 32) {
    const int j = j0 + lane;
    float ds = 0.f;
    if (j < hi) {
      const float raw = dot_row(q_s[warp], P.k, s.k_off + (int64_t)j * P.k_strides[2], P.k_strides[3], D, P.dtype);
      const float dp = dot_row(do_s[warp], P.v, s.v_off + (int64_t)j * P.v_strides[2], P.v_strides[3], D, P.dtype);
      ds = pair_grad(mods, raw, dp, lse, delta, i, j).ds;
    }
    const int jn = min(32, hi - j0);
    for (int jj = 0; jj < jn; ++jj) {
      const float dj = __shfl_sync(0xffffffffu, ds, jj);
      if (dj == 0.f) continue;
      const int64_t koff = s.k_off + (int64_t)(j0 + jj) * P.k_strides[2];
#pragma unroll
      for (int r = 0; r < kMaxDPerLane; ++r) {
        const int d = lane + 32 * r;
        if (d < D) acc[r] += dj * load_as_float(P.k, koff + (int64_t)d * P.k_strides[3], P.dtype);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kMaxDPerLane; ++r) {
    const int d = lane + 32 * r;
    if (d < D)
      store_from_float(P.dq, s.dq_off + (int64_t)i * P.dq_strides[2] + (int64_t)d * P.dq_strides[3], P.dtype,
                       acc[r] * P.softmax_scale);
  }
}

// ---------------------------------------------------------------------------------------------
// dK, dV: one warp per key row of one kv head; sums over the query heads of the group in registers,
// no atomics (fa_rdna3/kernels/backward.py:56-200).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kWarpsPerBlock * 32) simt_bwd_dkdv_kernel(const fa_attn_params P) {
  __shared__ float k_s[kWarpsPerBlock][kMaxD];
  __shared__ float v_s[kWarpsPerBlock][kMaxD];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int j = blockIdx.x * kWarpsPerBlock + warp;
  const int b = blockIdx.y / P.heads_kv, hk = blockIdx.y % P.heads_kv;
  const int D = P.head_dim;
  const int group = P.heads_q / P.heads_kv;
  SeqView s;
  make_view(P, b, hk * group, &s);
  if (j >= s.seqlen_k) return;
  for (int d = lane; d < D; d += 32) {
    k_s[warp][d] = load_as_float(P.k, s.k_off + (int64_t)j * P.k_strides[2] + (int64_t)d * P.k_strides[3], P.dtype);
    v_s[warp][d] = load_as_float(P.v, s.v_off + (int64_t)j * P.v_strides[2] + (int64_t)d * P.v_strides[3], P.dtype);
  }
  __syncwarp();

  float dk[kMaxDPerLane], dv[kMaxDPerLane];
#pragma unroll
  for (int r = 0; r < kMaxDPerLane; ++r) dk[r] = dv[r] = 0.f;

  for (int g = 0; g < group; ++g) {
    make_view(P, b, hk * group + g, &s);
    const ScoreMods mods = make_mods(P, s);
    int lo, hi;
    query_range_for_keys(mods, j, j, &lo, &hi);
    for (int i0 = lo; i0 < hi; i0 += 32) {
      const int i = i0 + lane;
      PairGrad pg{0.f, 0.f};
      if (i < hi) {
        const float raw = dot_row(k_s[warp], P.q, s.q_off + (int64_t)i * P.q_strides[2], P.q_strides[3], D, P.dtype);
        const float dp =
            dot_row(v_s[warp], P.dout, s.do_off + (int64_t)i * P.do_strides[2], P.do_strides[3], D, P.dtype);
        const float lse = P.lse[s.lse_off + (int64_t)i * s.lse_row_stride];
        const float delta = P.delta[s.delta_off + (int64_t)i * s.delta_row_stride];
        pg = pair_grad(mods, raw, dp, lse, delta, i, j);
      }
      const int in = min(32, hi - i0);
      for (int ii = 0; ii < in; ++ii) {
        const float pd = __shfl_sync(0xffffffffu, pg.p_drop, ii);
        const float ds = __shfl_sync(0xffffffffu, pg.ds, ii);
        if (pd == 0.f && ds == 0.f) continue;
        const int64_t qoff = s.q_off + (int64_t)(i0 + ii) * P.q_strides[2];
        const int64_t dooff = s.do_off + (int64_t)(i0 + ii) * P.do_strides[2];
#pragma unroll
        for (int r = 0; r < kMaxDPerLane; ++r) {
          const int d = lane + 32 * r;
          if (d < D) {
            dv[r] += pd * load_as_float(P.dout, dooff + (int64_t)d * P.do_strides[3], P.dtype);
            dk[r] += ds * load_as_float(P.q, qoff + (int64_t)d * P.q_strides[3], P.dtype);
          }
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kMaxDPerLane; ++r) {
    const int d = lane + 32 * r;
    if (d < D) {
      store_from_float(P.dk, s.dk_off + (int64_t)j * P.dk_strides[2] + (int64_t)d * P.dk_strides[3], P.dtype,
                       dk[r] * P.softmax_scale);
      store_from_float(P.dv, s.dv_off + (int64_t)j * P.dv_strides[2] + (int64_t)d * P.dv_strides[3], P.dtype, dv[r]);
    }
  }
}

// The tiled kernels (fa_tiled.cuh) pay off once both sequences span at least a tile; below that the one-warp-per-row
// kernels have more parallelism.
bool tiled_worthwhile(const fa_attn_params& p) { return p.seqlen_q >= 32 && p.seqlen_k >= 64; }

template <typename T, int D>
int launch_delta_vec(const fa_attn_params& p, cudaStream_t stream) {
  constexpr int rows_per_block = 8 * (32 / (D / 8)) * 4;  // eight warps, four passes each
  dim3 grid((p.seqlen_q + rows_per_block - 1) / rows_per_block, p.batch * p.heads_q);
  delta_vec_kernel<T, D><<<grid, 256, 0, stream>>>(p);
  return check_launch("delta");
}

bool rows_vectorisable(const void* ptr, const int64_t st[4]) {
  return st[3] == 1 && (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && st[0] % 8 == 0 && st[1] % 8 == 0 && st[2] % 8 == 0;
}

}  // namespace

int launch_bwd_delta(const fa_attn_params& p, cudaStream_t stream) {
  if ((p.dtype == FA_F16 || p.dtype == FA_BF16) && p.head_dim % 8 == 0 && p.head_dim <= 256 &&
      rows_vectorisable(p.out, p.o_strides) && rows_vectorisable(p.dout, p.do_strides)) {
    const int width = p.head_dim <= 64 ? 64 : (p.head_dim <= 128 ? 128 : 256);
    if (p.dtype == FA_F16)
      return width == 64    ? launch_delta_vec<__half, 64>(p, stream)
             : width == 128 ? launch_delta_vec<__half, 128>(p, stream)
                            : launch_delta_vec<__half, 256>(p, stream);
    return width == 64    ? launch_delta_vec<__nv_bfloat16, 64>(p, stream)
           : width == 128 ? launch_delta_vec<__nv_bfloat16, 128>(p, stream)
                          : launch_delta_vec<__nv_bfloat16, 256>(p, stream);
  }
  dim3 grid((p.seqlen_q + kWarpsPerBlock - 1) / kWarpsPerBlock, p.batch * p.heads_q);
  simt_delta_kernel<<<grid, kWarpsPerBlock * 32, 0, stream>>>(p);
  return check_launch("delta");
}

int launch_fwd_simt(const fa_attn_params& p, cudaStream_t stream) {
  if (p.head_dim > kMaxD) return set_error(FA_ERR_UNSUPPORTED, "head_dim %d exceeds %d", p.head_dim, kMaxD);
  if (tiled_worthwhile(p)) {
    return launch_tiled_fwd(p, stream);
  }
  dim3 grid((p.seqlen_q + kWarpsPerBlock - 1) / kWarpsPerBlock, p.batch * p.heads_q);
  simt_fwd_kernel<<<grid, kWarpsPerBlock * 32, 0, stream>>>(p);
  return check_launch("simt forward");
}

int launch_bwd_simt(const fa_attn_params& p, int parts, cudaStream_t stream) {
  if (p.head_dim > kMaxD) return set_error(FA_ERR_UNSUPPORTED, "head_dim %d exceeds %d", p.head_dim, kMaxD);
  if (tiled_worthwhile(p)) {
    if (parts & FA_BWD_DKDV) {
      int rc = launch_tiled_dkdv(p, stream);
      if (rc) return rc;
    }
    if (parts & FA_BWD_DQ) {
      return launch_tiled_dq(p, stream);
    }
    return 0;
  }
  if (parts & FA_BWD_DKDV) {
    dim3 gk((p.seqlen_k + kWarpsPerBlock - 1) / kWarpsPerBlock, p.batch * p.heads_kv);
    simt_bwd_dkdv_kernel<<<gk, kWarpsPerBlock * 32, 0, stream>>>(p);
    int rc = check_launch("simt dkdv");
    if (rc) return rc;
  }
  if (parts & FA_BWD_DQ) {
    dim3 gq((p.seqlen_q + kWarpsPerBlock - 1) / kWarpsPerBlock, p.batch * p.heads_q);
    simt_bwd_dq_kernel<<<gq, kWarpsPerBlock * 32, 0, stream>>>(p);
    return check_launch("simt dq");
  }
  return 0;
}

}  // namespace fa
