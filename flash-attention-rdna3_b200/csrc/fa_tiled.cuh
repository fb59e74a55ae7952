// Shared-memory tiled CUDA-core attention kernels (forward, dQ, dK/dV). Each of fa_tiled_fwd.cu, fa_tiled_dq.cu and
// fa_tiled_dkdv.cu instantiates one family, so the three compile side by side.
#pragma once
#include "fa_simt_shared.cuh"

namespace fa {
namespace {

// =============================================================================================
// Tiled forms of the three kernels above, used once the problem is larger than a tile. A CTA of 256 threads (16 x 16)
// owns 16*kRows rows (queries; keys in dK/dV) and walks the other sequence 64 rows at a time. Two primitives on
// shared-memory tiles do all the arithmetic in fp32 FMAs:
//   tile_abt: scores[16*kRows][64] = A[rows][D] . B[64 rows][D]^T, the head dimension staged 32 columns at a time;
//             thread (ty, tx) holds rows ty + 16a and columns tx + 16b in registers
//   tile_pb : acc[rows][D] += P[rows][64] . B[64 rows][D], P in shared memory, B staged 64 columns at a time;
//             thread (ty, tx) holds rows ty + 16a and columns 64c + 4tx + e
// Every operand is read once per tile pair instead of once per row pair, which is what separates these kernels from
// the one-warp-per-row forms (50-80x at 2048 tokens). Loads honour arbitrary strides and any of the three dtypes.
// =============================================================================================
constexpr int kTileThreads = 256;

struct __align__(16) TileSmem {
  float P[64][68];
  union {
    struct { float A[64][36]; float B[64][36]; } ab;
    float V[64][64];
  } u;
};

template <typename T>
__device__ __forceinline__ float ld_elem(const void* base, int64_t idx) {
  return DType<T>::to_float(reinterpret_cast<const T*>(base)[idx]);
}

// Two adjacent 16-bit elements with one 4-byte load (kPair kernels: unit inner stride, even outer strides and offsets).
template <typename T>
__device__ __forceinline__ float2 ld_pair(const void* base, int64_t idx) {
  return DType<T>::unpack2(*reinterpret_cast<const uint32_t*>(reinterpret_cast<const T*>(base) + idx));
}
template <>
__device__ __forceinline__ float2 ld_pair<float>(const void* base, int64_t idx) {
  return *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(base) + idx);
}

// Staging slot u of a thread -> (row, column) of a tile that is 1 << kLog2W columns wide. With kPair, slots 2v and
// 2v + 1 are the two halves of one 4-byte load.
template <bool kPair, int kLog2W>
__device__ __forceinline__ void stage_pos(int tid, int u, int* r, int* c) {
  if (kPair) {
    const int pidx = tid + (u >> 1) * kTileThreads;
    *r = pidx >> (kLog2W - 1);
    *c = ((pidx & ((1 << (kLog2W - 1)) - 1)) << 1) | (u & 1);
  } else {
    const int idx = tid + u * kTileThreads;
    *r = idx >> kLog2W;
    *c = idx & ((1 << kLog2W) - 1);
  }
}

template <typename T, bool kPair, int kLog2W, int kN>
__device__ __forceinline__ void stage_fetch(float (&reg)[kN], const void* base, int64_t off, int64_t rs, int64_t ds,
                                            int valid, int c0, int D) {
  const int tid = threadIdx.x;
  if (kPair) {
#pragma unroll
    for (int u = 0; u < kN; u += 2) {
      int r, c;
      stage_pos<true, kLog2W>(tid, u, &r, &c);
      float2 v = make_float2(0.f, 0.f);
      if (r < valid && c0 + c < D) v = ld_pair<T>(base, off + (int64_t)r * rs + (c0 + c));
      reg[u] = v.x;
      reg[u + 1] = v.y;
    }
  } else {
#pragma unroll
    for (int u = 0; u < kN; ++u) {
      int r, c;
      stage_pos<false, kLog2W>(tid, u, &r, &c);
      reg[u] = (r < valid && c0 + c < D) ? ld_elem<T>(base, off + (int64_t)r * rs + (int64_t)(c0 + c) * ds) : 0.f;
    }
  }
}

template <bool kPair, int kLog2W, int kN, int kStride>
__device__ __forceinline__ void stage_store(const float (&reg)[kN], float (*dst)[kStride]) {
  const int tid = threadIdx.x;
  if (kPair) {
#pragma unroll
    for (int u = 0; u < kN; u += 2) {
      int r, c;
      stage_pos<true, kLog2W>(tid, u, &r, &c);
      *reinterpret_cast<float2*>(&dst[r][c]) = make_float2(reg[u], reg[u + 1]);
    }
  } else {
#pragma unroll
    for (int u = 0; u < kN; ++u) {
      int r, c;
      stage_pos<false, kLog2W>(tid, u, &r, &c);
      dst[r][c] = reg[u];
    }
  }
}

template <typename T, int kRows, bool kPair>
__device__ __forceinline__ void tile_abt(const void* A, int64_t a_off, int64_t a_rs, int64_t a_ds, int a_valid,
                                         const void* B, int64_t b_off, int64_t b_rs, int64_t b_ds, int b_valid, int D,
                                         TileSmem& sm, float (&acc)[kRows][4]) {
  constexpr int BM = 16 * kRows;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
#pragma unroll
  for (int a = 0; a < kRows; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
  // Global loads run one 32-column chunk ahead of the arithmetic: chunk d0 + 32 is in flight (in registers) while
  // chunk d0 is multiplied out of shared memory.
  constexpr int kA = BM * 32 / kTileThreads, kB = 64 * 32 / kTileThreads;
  float ra[kA], rb[kB];
  auto fetch = [&](int d0) {
    stage_fetch<T, kPair, 5>(ra, A, a_off, a_rs, a_ds, a_valid, d0, D);
    stage_fetch<T, kPair, 5>(rb, B, b_off, b_rs, b_ds, b_valid, d0, D);
  };
  fetch(0);
  for (int d0 = 0; d0 < D; d0 += 32) {
    __syncthreads();  // whoever read the staging buffers (or P's neighbours in the union) before is done
    stage_store<kPair, 5>(ra, sm.u.ab.A);
    stage_store<kPair, 5>(rb, sm.u.ab.B);
    __syncthreads();
    if (d0 + 32 < D) fetch(d0 + 32);
#pragma unroll
    for (int d = 0; d < 32; d += 4) {
      float4 av[kRows], bv[4];
#pragma unroll
      for (int a = 0; a < kRows; ++a) av[a] = *reinterpret_cast<const float4*>(&sm.u.ab.A[ty + 16 * a][d]);
#pragma unroll
      for (int b = 0; b < 4; ++b) bv[b] = *reinterpret_cast<const float4*>(&sm.u.ab.B[tx + 16 * b][d]);
#pragma unroll
      for (int a = 0; a < kRows; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b)
          acc[a][b] += av[a].x * bv[b].x + av[a].y * bv[b].y + av[a].z * bv[b].z + av[a].w * bv[b].w;
    }
  }
}

template <typename T, int kRows, int kDC, bool kPair>
__device__ __forceinline__ void tile_pb(const void* B, int64_t b_off, int64_t b_rs, int64_t b_ds, int b_valid, int D,
                                        TileSmem& sm, float (&acc)[kDC][kRows][4]) {
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  constexpr int kV = 64 * 64 / kTileThreads;
  float rv[kV];
  auto fetch = [&](int c) { stage_fetch<T, kPair, 6>(rv, B, b_off, b_rs, b_ds, b_valid, c * 64, D); };
  fetch(0);
#pragma unroll
  for (int c = 0; c < kDC; ++c) {
    if (c * 64 < D) {
      __syncthreads();  // P is written, the previous chunk is consumed
      stage_store<kPair, 6>(rv, sm.u.V);
      __syncthreads();
      if (c + 1 < kDC && (c + 1) * 64 < D) fetch(c + 1);
#pragma unroll 4
      for (int k = 0; k < 64; k += 4) {
        float4 pv[kRows], bv[4];
#pragma unroll
        for (int a = 0; a < kRows; ++a) pv[a] = *reinterpret_cast<const float4*>(&sm.P[ty + 16 * a][k]);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) bv[kk] = *reinterpret_cast<const float4*>(&sm.u.V[k + kk][tx * 4]);
#pragma unroll
        for (int a = 0; a < kRows; ++a) {
          acc[c][a][0] += pv[a].x * bv[0].x + pv[a].y * bv[1].x + pv[a].z * bv[2].x + pv[a].w * bv[3].x;
          acc[c][a][1] += pv[a].x * bv[0].y + pv[a].y * bv[1].y + pv[a].z * bv[2].y + pv[a].w * bv[3].y;
          acc[c][a][2] += pv[a].x * bv[0].z + pv[a].y * bv[1].z + pv[a].z * bv[2].z + pv[a].w * bv[3].z;
          acc[c][a][3] += pv[a].x * bv[0].w + pv[a].y * bv[1].w + pv[a].z * bv[2].w + pv[a].w * bv[3].w;
        }
      }
    }
  }
}

// max / sum over the 16 threads (same ty) that share a row: lanes 16*(ty&1) + tx of one warp
__device__ __forceinline__ float row16_max(float x) {
  for (int o = 8; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
__device__ __forceinline__ float row16_sum(float x) {
  for (int o = 8; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

template <typename T, int kRows, int kDC, bool kPair>
__global__ void __launch_bounds__(kTileThreads, (kDC * kRows <= 8 ? 2 : 1)) tiled_fwd_kernel(const fa_attn_params P) {
  __shared__ TileSmem sm;
  constexpr int BM = 16 * kRows;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int i0 = (gridDim.x - 1 - blockIdx.x) * BM;  // long (causal) rows first: the short ones fill the last wave
  const int b = blockIdx.y / P.heads_q, h = blockIdx.y % P.heads_q;
  const int D = P.head_dim;
  SeqView s;
  make_view(P, b, h, &s);
  if (i0 >= s.seqlen_q) return;
  const ScoreMods mods = make_mods(P, s);
  int lo, hi;
  key_range_for_rows(mods, i0, min(i0 + BM, s.seqlen_q) - 1, &lo, &hi);

  float m[kRows], l[kRows], acc[kDC][kRows][4];
#pragma unroll
  for (int a = 0; a < kRows; ++a) {
    m[a] = kNegInf;
    l[a] = 0.f;
#pragma unroll
    for (int c = 0; c < kDC; ++c)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[c][a][e] = 0.f;
  }

  for (int j0 = lo; j0 < hi; j0 += 64) {
    float sc[kRows][4];
    tile_abt<T, kRows, kPair>(P.q, s.q_off + (int64_t)i0 * P.q_strides[2], P.q_strides[2], P.q_strides[3], s.seqlen_q - i0,
                       P.k, s.k_off + (int64_t)j0 * P.k_strides[2], P.k_strides[2], P.k_strides[3], s.seqlen_k - j0, D,
                       sm, sc);
#pragma unroll
    for (int a = 0; a < kRows; ++a) {
      const int i = i0 + ty + 16 * a;
      float mx = kNegInf;
#pragma unroll
      for (int bb = 0; bb < 4; ++bb) {
        const int j = j0 + tx + 16 * bb;
        float x = kNegInf;
        if (i < s.seqlen_q && mods.keep(i, j)) x = mods.logit(sc[a][bb], i, j, nullptr);
        sc[a][bb] = x;
        mx = fmaxf(mx, x);
      }
      const float m_new = fmaxf(m[a], row16_max(mx));
      const float m_safe = (m_new == kNegInf) ? 0.f : m_new;
      const float alpha = exp2f(m[a] - m_safe);
      float sum = 0.f;
#pragma unroll
      for (int bb = 0; bb < 4; ++bb) {
        float p = exp2f(sc[a][bb] - m_safe);
        sum += p;
        if (mods.dropout_p > 0.f && p != 0.f) p = mods.dropout_keep(i, j0 + tx + 16 * bb) ? p * mods.inv_keep : 0.f;
        sm.P[ty + 16 * a][tx + 16 * bb] = p;  // the previous readers of P passed a barrier inside tile_abt
      }
      l[a] = l[a] * alpha + row16_sum(sum);
#pragma unroll
      for (int c = 0; c < kDC; ++c)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[c][a][e] *= alpha;
      if (m_new != kNegInf) m[a] = m_new;
    }
    tile_pb<T, kRows, kDC, kPair>(P.v, s.v_off + (int64_t)j0 * P.v_strides[2], P.v_strides[2], P.v_strides[3],
                           s.seqlen_k - j0, D, sm, acc);
  }

#pragma unroll
  for (int a = 0; a < kRows; ++a) {
    const int i = i0 + ty + 16 * a;
    if (i >= s.seqlen_q) continue;
    const float l_safe = (l[a] == 0.f) ? 1.f : l[a];
    const float inv = 1.f / l_safe;
#pragma unroll
    for (int c = 0; c < kDC; ++c)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int d = c * 64 + tx * 4 + e;
        if (d < D)
          store_from_float(P.out, s.o_off + (int64_t)i * P.o_strides[2] + (int64_t)d * P.o_strides[3], P.dtype,
                           acc[c][a][e] * inv);
      }
    if (tx == 0) P.lse[s.lse_off + (int64_t)i * s.lse_row_stride] = m[a] * kLn2 + logf(l_safe);
  }
}

template <typename T, int kRows, int kDC, bool kPair>
__global__ void __launch_bounds__(kTileThreads, (kDC * kRows <= 8 ? 2 : 1)) tiled_bwd_dq_kernel(const fa_attn_params P) {
  __shared__ TileSmem sm;
  constexpr int BM = 16 * kRows;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int i0 = (gridDim.x - 1 - blockIdx.x) * BM;  // long (causal) rows first: the short ones fill the last wave
  const int b = blockIdx.y / P.heads_q, h = blockIdx.y % P.heads_q;
  const int D = P.head_dim;
  SeqView s;
  make_view(P, b, h, &s);
  if (i0 >= s.seqlen_q) return;
  const ScoreMods mods = make_mods(P, s);
  int lo, hi;
  key_range_for_rows(mods, i0, min(i0 + BM, s.seqlen_q) - 1, &lo, &hi);

  float lse[kRows], delta[kRows], acc[kDC][kRows][4];
#pragma unroll
  for (int a = 0; a < kRows; ++a) {
    const int i = i0 + ty + 16 * a;
    lse[a] = i < s.seqlen_q ? P.lse[s.lse_off + (int64_t)i * s.lse_row_stride] : kNegInf;
    delta[a] = i < s.seqlen_q ? P.delta[s.delta_off + (int64_t)i * s.delta_row_stride] : 0.f;
#pragma unroll
    for (int c = 0; c < kDC; ++c)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[c][a][e] = 0.f;
  }

  for (int j0 = lo; j0 < hi; j0 += 64) {
    float sc[kRows][4], dp[kRows][4];
    tile_abt<T, kRows, kPair>(P.q, s.q_off + (int64_t)i0 * P.q_strides[2], P.q_strides[2], P.q_strides[3], s.seqlen_q - i0,
                       P.k, s.k_off + (int64_t)j0 * P.k_strides[2], P.k_strides[2], P.k_strides[3], s.seqlen_k - j0, D,
                       sm, sc);
    tile_abt<T, kRows, kPair>(P.dout, s.do_off + (int64_t)i0 * P.do_strides[2], P.do_strides[2], P.do_strides[3],
                       s.seqlen_q - i0, P.v, s.v_off + (int64_t)j0 * P.v_strides[2], P.v_strides[2], P.v_strides[3],
                       s.seqlen_k - j0, D, sm, dp);
#pragma unroll
    for (int a = 0; a < kRows; ++a) {
      const int i = i0 + ty + 16 * a;
#pragma unroll
      for (int bb = 0; bb < 4; ++bb) {
        const int j = j0 + tx + 16 * bb;
        float ds = 0.f;
        if (i < s.seqlen_q) ds = pair_grad(mods, sc[a][bb], dp[a][bb], lse[a], delta[a], i, j).ds;
        sm.P[ty + 16 * a][tx + 16 * bb] = ds;
      }
    }
    tile_pb<T, kRows, kDC, kPair>(P.k, s.k_off + (int64_t)j0 * P.k_strides[2], P.k_strides[2], P.k_strides[3],
                           s.seqlen_k - j0, D, sm, acc);
  }

#pragma unroll
  for (int a = 0; a < kRows; ++a) {
    const int i = i0 + ty + 16 * a;
    if (i >= s.seqlen_q) continue;
#pragma unroll
    for (int c = 0; c < kDC; ++c)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int d = c * 64 + tx * 4 + e;
        if (d < D)
          store_from_float(P.dq, s.dq_off + (int64_t)i * P.dq_strides[2] + (int64_t)d * P.dq_strides[3], P.dtype,
                           acc[c][a][e] * P.softmax_scale);
      }
  }
}

// Rows of the tile are keys, columns are queries; the query heads of the group are summed in registers.
template <typename T, int kRows, int kDC, bool kPair>
__global__ void __launch_bounds__(kTileThreads, (kDC * kRows <= 4 ? 2 : 1)) tiled_bwd_dkdv_kernel(const fa_attn_params P) {
  __shared__ TileSmem sm;
  constexpr int BM = 16 * kRows;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int j0 = blockIdx.x * BM;
  const int b = blockIdx.y / P.heads_kv, hk = blockIdx.y % P.heads_kv;
  const int D = P.head_dim;
  const int group = P.heads_q / P.heads_kv;
  SeqView s;
  make_view(P, b, hk * group, &s);
  if (j0 >= s.seqlen_k) return;

  float dk[kDC][kRows][4], dv[kDC][kRows][4];
#pragma unroll
  for (int c = 0; c < kDC; ++c)
#pragma unroll
    for (int a = 0; a < kRows; ++a)
#pragma unroll
      for (int e = 0; e < 4; ++e) dk[c][a][e] = dv[c][a][e] = 0.f;

  for (int g = 0; g < group; ++g) {
    make_view(P, b, hk * group + g, &s);
    const ScoreMods mods = make_mods(P, s);
    int lo, hi;
    query_range_for_keys(mods, j0, min(j0 + BM, s.seqlen_k) - 1, &lo, &hi);
    for (int i0 = lo; i0 < hi; i0 += 64) {
      float sc[kRows][4], dp[kRows][4];
      tile_abt<T, kRows, kPair>(P.k, s.k_off + (int64_t)j0 * P.k_strides[2], P.k_strides[2], P.k_strides[3], s.seqlen_k - j0,
                         P.q, s.q_off + (int64_t)i0 * P.q_strides[2], P.q_strides[2], P.q_strides[3], s.seqlen_q - i0,
                         D, sm, sc);
      tile_abt<T, kRows, kPair>(P.v, s.v_off + (int64_t)j0 * P.v_strides[2], P.v_strides[2], P.v_strides[3], s.seqlen_k - j0,
                         P.dout, s.do_off + (int64_t)i0 * P.do_strides[2], P.do_strides[2], P.do_strides[3],
                         s.seqlen_q - i0, D, sm, dp);
      float lse_i[4], delta_i[4];
#pragma unroll
      for (int bb = 0; bb < 4; ++bb) {
        const int i = i0 + tx + 16 * bb;
        lse_i[bb] = i < s.seqlen_q ? P.lse[s.lse_off + (int64_t)i * s.lse_row_stride] : kNegInf;
        delta_i[bb] = i < s.seqlen_q ? P.delta[s.delta_off + (int64_t)i * s.delta_row_stride] : 0.f;
      }
#pragma unroll
      for (int a = 0; a < kRows; ++a) {
        const int j = j0 + ty + 16 * a;
#pragma unroll
        for (int bb = 0; bb < 4; ++bb) {
          const int i = i0 + tx + 16 * bb;
          PairGrad pg{0.f, 0.f};
          if (i < s.seqlen_q && j < s.seqlen_k) pg = pair_grad(mods, sc[a][bb], dp[a][bb], lse_i[bb], delta_i[bb], i, j);
          sm.P[ty + 16 * a][tx + 16 * bb] = pg.p_drop;
          sc[a][bb] = pg.ds;
        }
      }
      tile_pb<T, kRows, kDC, kPair>(P.dout, s.do_off + (int64_t)i0 * P.do_strides[2], P.do_strides[2], P.do_strides[3],
                             s.seqlen_q - i0, D, sm, dv);
      __syncthreads();  // every thread is done with the probabilities before the score gradients replace them
#pragma unroll
      for (int a = 0; a < kRows; ++a)
#pragma unroll
        for (int bb = 0; bb < 4; ++bb) sm.P[ty + 16 * a][tx + 16 * bb] = sc[a][bb];
      tile_pb<T, kRows, kDC, kPair>(P.q, s.q_off + (int64_t)i0 * P.q_strides[2], P.q_strides[2], P.q_strides[3],
                             s.seqlen_q - i0, D, sm, dk);
    }
  }

#pragma unroll
  for (int a = 0; a < kRows; ++a) {
    const int j = j0 + ty + 16 * a;
    if (j >= s.seqlen_k) continue;
#pragma unroll
    for (int c = 0; c < kDC; ++c)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int d = c * 64 + tx * 4 + e;
        if (d < D) {
          store_from_float(P.dk, s.dk_off + (int64_t)j * P.dk_strides[2] + (int64_t)d * P.dk_strides[3], P.dtype,
                           dk[c][a][e] * P.softmax_scale);
          store_from_float(P.dv, s.dv_off + (int64_t)j * P.dv_strides[2] + (int64_t)d * P.dv_strides[3], P.dtype,
                           dv[c][a][e]);
        }
      }
  }
}

enum TiledKind { kTiledFwd, kTiledDq, kTiledDkdv };

template <TiledKind kind, typename T, int kRows, int kDC, bool kPair>
void launch_tiled_one(const fa_attn_params& p, cudaStream_t stream) {
  constexpr int BM = 16 * kRows;
  if constexpr (kind == kTiledDkdv) {
    dim3 grid((p.seqlen_k + BM - 1) / BM, p.batch * p.heads_kv);
    tiled_bwd_dkdv_kernel<T, kRows, kDC, kPair><<<grid, kTileThreads, 0, stream>>>(p);
  } else {
    dim3 grid((p.seqlen_q + BM - 1) / BM, p.batch * p.heads_q);
    if constexpr (kind == kTiledFwd) tiled_fwd_kernel<T, kRows, kDC, kPair><<<grid, kTileThreads, 0, stream>>>(p);
    else tiled_bwd_dq_kernel<T, kRows, kDC, kPair><<<grid, kTileThreads, 0, stream>>>(p);
  }
}

// Rows per thread and 64-column chunks by head dimension; dK/dV carries two accumulators, so it narrows sooner.
template <TiledKind kind, typename T, bool kPair>
void launch_tiled_typed(const fa_attn_params& p, cudaStream_t stream) {
  const int D = p.head_dim;
  if (D <= 64) launch_tiled_one<kind, T, 4, 1, kPair>(p, stream);
  else if (D <= 128) launch_tiled_one<kind, T, 4, 2, kPair>(p, stream);
  else if (D <= 256) launch_tiled_one<kind, T, 4, 4, kPair>(p, stream);
  else launch_tiled_one<kind, T, 2, 8, kPair>(p, stream);
}

// Paired loads need 4-byte (16-bit types) or 8-byte (fp32) aligned element pairs everywhere a tile may start.
inline bool pair_loadable(const void* ptr, const int64_t st[4], int elem_bytes) {
  return ptr == nullptr || (st[3] == 1 && (reinterpret_cast<uintptr_t>(ptr) % (2 * elem_bytes)) == 0 && st[0] % 2 == 0 &&
                            st[1] % 2 == 0 && st[2] % 2 == 0);
}

template <TiledKind kind>
void launch_tiled(const fa_attn_params& p, cudaStream_t stream) {
  const int eb = p.dtype == FA_F32 ? 4 : 2;
  bool pair = p.head_dim % 2 == 0 && pair_loadable(p.q, p.q_strides, eb) && pair_loadable(p.k, p.k_strides, eb) &&
              pair_loadable(p.v, p.v_strides, eb);
  if (kind != kTiledFwd) pair = pair && pair_loadable(p.dout, p.do_strides, eb);
  if (p.dtype == FA_F16) {
    if (pair) launch_tiled_typed<kind, __half, true>(p, stream);
    else launch_tiled_typed<kind, __half, false>(p, stream);
  } else if (p.dtype == FA_BF16) {
    if (pair) launch_tiled_typed<kind, __nv_bfloat16, true>(p, stream);
    else launch_tiled_typed<kind, __nv_bfloat16, false>(p, stream);
  } else {
    launch_tiled_typed<kind, float, false>(p, stream);  // 4-byte loads already fill a 128-byte line per warp
  }
}

}  // namespace
}  // namespace fa
