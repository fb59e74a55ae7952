// Pieces the tcgen05 backward kernels share between translation units: the argument block, score modifiers and
// masks, the elementwise steps of the two phases (P from S, dS from dP), the layout of a tile in the dS workspace,
// and the work items of the persistent kernels. Everything is in an unnamed namespace: each translation unit gets
// its own copy.
#pragma once

#include "fa_common.cuh"
#include "fa_sm100.cuh"

namespace fa {
namespace {

constexpr int kBwdThreads = 320;
constexpr uint32_t kFull = 0xffffffffu;

struct BwdArgs {
  int varlen, batch, heads_q, heads_kv, seqlen_q, seqlen_k, total_q, total_k;
  int head_dim;  // the caller's; the kernels' D is 64 or 128 and the columns in between load as zeros
  const int32_t* cu_q;
  const int32_t* cu_k;
  const float* lse;
  int64_t l_sb, l_sh, l_ss;
  const float* delta;
  int64_t d_sb, d_sh, d_ss;
  void* dq;
  int64_t dq_sb, dq_sh, dq_ss;
  void* dk;
  int64_t dk_sb, dk_sh, dk_ss;
  void* dv;
  int64_t dv_sb, dv_sh, dv_ss;
  float softmax_scale, softcap;
  const void* bias;
  int bias_dtype;
  int64_t bias_sb, bias_sh, bias_sm, bias_sn;
  const float* alibi;
  int causal, wl, wr;
  float dropout_p;
  uint64_t seed;
  int num_tiles;
  int* status;
  // dS workspace (dense only, may be null): the dK/dV kernel stores every 128 x 128 dS^T tile it forms (16-bit,
  // [key][query], 32 KB) at tile index ((b * heads_q + h) * ds_kt + key tile) * ds_qt + query tile, and the dQ product
  // is then one GEMM over those tiles (bwd_dq_gemm_kernel) instead of a second pass that recomputes S and dP.
  void* ds_ws;
  int ds_kt, ds_qt;
  float* lse_out;  // forward kernels that share this block: where LSE is written
  // forward over P tiles: per (batch, head, query row of the padded 128-row tiles) the row maximum (log2 domain) the P
  // tiles are relative to and 1 / the row sum, which the product's epilogue applies. Null in the backward.
  float2* row_stats;
  int compact;  // dK/dV of a packed batch on the compact grid (kv head, key tile number): see find_packed_tile
  int after_delta;  // dK/dV was launched as a programmatic dependent of the delta kernel: wait for it before reading delta
};

__device__ __forceinline__ void report_timeout(int* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

__device__ __forceinline__ ScoreMods make_mods(const BwdArgs& a, int b, int h, int Sq, int Sk) {
  ScoreMods m;
  m.scale_log2 = a.softmax_scale * kLog2e;
  m.cap_log2 = a.softcap > 0.f ? a.softcap * kLog2e : 0.f;
  m.inv_cap_log2 = a.softcap > 0.f ? 1.f / m.cap_log2 : 0.f;
  m.alibi_slope_log2 = a.alibi ? a.alibi[h] * kLog2e : 0.f;
  m.bias = nullptr;
  m.bias_dtype = a.bias_dtype;
  m.bias_stride_m = a.bias_sm;
  m.bias_stride_n = a.bias_sn;
  if (a.bias) {
    const int esz = a.bias_dtype == FA_F32 ? 4 : 2;
    m.bias = reinterpret_cast<const char*>(a.bias) + ((int64_t)b * a.bias_sb + (int64_t)h * a.bias_sh) * esz;
  }
  m.causal = a.causal;
  m.window_left = a.wl;
  m.window_right = a.wr;
  m.seqlen_q = Sq;
  m.seqlen_k = Sk;
  m.dropout_p = a.dropout_p;
  m.inv_keep = a.dropout_p > 0.f ? 1.f / (1.f - a.dropout_p) : 1.f;
  m.dropout_seed = a.seed;
  m.dropout_base = ((uint64_t)b * (uint64_t)a.heads_q + (uint64_t)h) * (uint64_t)Sq;
  return m;
}

// True when some pair of query rows [r0, r0+nr) x keys [k0, k0+nk) may be masked by bounds, causal or window.
__device__ __forceinline__ bool block_needs_mask(const ScoreMods& m, int r0, int nr, int k0, int nk) {
  const int off = m.seqlen_k - m.seqlen_q;
  return (k0 + nk > m.seqlen_k) || (m.causal && (k0 + nk - 1 > r0 + off)) ||
         (m.window_left >= 0 && (k0 < r0 + nr - 1 + off - m.window_left)) ||
         (!m.causal && m.window_right >= 0 && (k0 + nk - 1 > r0 + off + m.window_right));
}

// General path (softcap / bias / ALiBi / dropout) for 32 consecutive elements of one accumulator row: element e is
// (query i0, key j0 + e) when kAlongKeys (dQ kernel), (query i0 + e, key j0) otherwise (dK/dV kernel). In: x = raw
// scores, g = raw dP. Out: x = probabilities as the dV product wants them (dropped and rescaled under dropout),
// g = dS. nl / nd hold -lse*log2(e) (or -inf) and -delta of the query: one value when kAlongKeys, 32 otherwise.
// Elements outside [e_lo, e_hi] are masked out.
template <bool kAlongKeys>
__device__ __forceinline__ void bwd_mods_chunk32(const ScoreMods& m, float (&x)[32], float (&g)[32], const float* nl,
                                                 const float* nd, int i0, int j0, int e_lo, int e_hi) {
  const uint32_t kept = mods_dropout_bits32<kAlongKeys>(m, i0, j0);
  const bool dropout = m.dropout_p > 0.f;
  const float inv_keep = m.inv_keep;
  if (dropout) {
#pragma unroll
    for (int e = 0; e < 32; ++e) g[e] = ((kept >> e) & 1u) ? g[e] * inv_keep : 0.f;
  }
#pragma unroll
  for (int e = 0; e < 32; ++e) g[e] += nd[kAlongKeys ? 0 : e];
  mods_logits32<kAlongKeys>(m, x, i0, j0, &g);  // g picks up the soft-cap chain factor
#pragma unroll
  for (int e = 0; e < 32; ++e) {
    const float p = (e >= e_lo && e <= e_hi) ? fast_exp2(x[e] + nl[kAlongKeys ? 0 : e]) : 0.f;
    x[e] = p;
    g[e] *= p;
  }
  if (dropout) {
#pragma unroll
    for (int e = 0; e < 32; ++e) x[e] = ((kept >> e) & 1u) ? x[e] * inv_keep : 0.f;
  }
}

// Converts a 32-column fp32 slice of a TMEM accumulator to 16-bit and writes it to a global row.
template <typename T>
__device__ __forceinline__ void store_row_slice(T* dst, const uint32_t (&o)[32], float scale, int cols) {
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    if (v * 8 >= cols) break;  // columns past the caller's head dimension do not exist
    uint4 pkt;
    pkt.x = DType<T>::pack2(__uint_as_float(o[v * 8 + 0]) * scale, __uint_as_float(o[v * 8 + 1]) * scale);
    pkt.y = DType<T>::pack2(__uint_as_float(o[v * 8 + 2]) * scale, __uint_as_float(o[v * 8 + 3]) * scale);
    pkt.z = DType<T>::pack2(__uint_as_float(o[v * 8 + 4]) * scale, __uint_as_float(o[v * 8 + 5]) * scale);
    pkt.w = DType<T>::pack2(__uint_as_float(o[v * 8 + 6]) * scale, __uint_as_float(o[v * 8 + 7]) * scale);
    *reinterpret_cast<uint4*>(dst + v * 8) = pkt;
  }
}

// A dS^T tile in the workspace is stored as 16 blocks of 8 queries; a block holds, key after key, the 16 bytes of
// that key's 8 values. A warp (32 consecutive keys) therefore writes 512 contiguous bytes per store, and the tile is,
// byte for byte, the unswizzled core-matrix layout the tensor core reads an operand "across its rows" from.
// Stores 32 consecutive queries (four blocks, 16 packed words) of one key row; dst points at the key's 16 bytes in the
// first of the four blocks.
__device__ __forceinline__ void store_ds32(uint8_t* dst, const uint32_t (&dsk)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // streaming store: the tile is read once, by a later kernel, and should not push operand tiles out of L2
    asm volatile("st.global.cs.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(dst + i * 2048), "r"(dsk[4 * i]), "r"(dsk[4 * i + 1]),
                 "r"(dsk[4 * i + 2]), "r"(dsk[4 * i + 3])
                 : "memory");
  }
}

// Item a persistent CTA takes in its round-th turn: rounds alternate direction over the CTAs ("snake"), so with
// items ordered longest first every CTA gets nearly the same total length. An index past the item count ends the
// CTA's walk (later rounds only hold larger indices).
__device__ __forceinline__ int snake_item(int round, int cta, int num_ctas) {
  return round * num_ctas + ((round & 1) ? num_ctas - 1 - cta : cta);
}

// Work item of the persistent dQ kernel: one 128-query tile of one (batch, head).
struct DqItem {
  int b, h, hk, q0, q_start, k_start, Sq, Sk, slo, n_total;
  bool valid;
};

__device__ __forceinline__ DqItem dq_item(const BwdArgs& a, int w) {
  DqItem it;
  const int bh_count = a.batch * a.heads_q;
  const int qtile = a.num_tiles - 1 - w / bh_count;  // items are dealt longest (causal) rows first
  const int bh = w % bh_count;
  it.b = bh / a.heads_q;
  it.h = bh % a.heads_q;
  it.hk = it.h / (a.heads_q / a.heads_kv);
  it.q_start = it.k_start = 0;
  it.Sq = a.seqlen_q;
  it.Sk = a.seqlen_k;
  if (a.varlen) {
    bounded_sequence(a.cu_q, it.b, a.total_q, &it.q_start, &it.Sq);
    bounded_sequence(a.cu_k, it.b, a.total_k, &it.k_start, &it.Sk);
  }
  it.q0 = qtile * 128;
  it.valid = it.q0 < it.Sq;
  it.slo = it.n_total = 0;
  if (it.valid) {
    const int off = it.Sk - it.Sq;
    const int r1 = min(it.q0 + 127, it.Sq - 1);
    int khi = it.Sk, klo = 0;
    if (a.causal) khi = min(khi, r1 + off + 1);
    else if (a.wr >= 0) khi = min(khi, r1 + off + a.wr + 1);
    if (a.wl >= 0) klo = max(0, it.q0 + off - a.wl);
    khi = max(khi, 0);
    const int slo = klo / 128, shi = (khi + 127) / 128;
    if (shi > slo) {
      it.slo = slo;
      it.n_total = shi - slo;
    }
  }
  return it;
}

// 32 raw scores of one row -> probabilities in place: p = exp2(s * scale_log2 + nlse2), zero outside [c_lo, c_hi]
// (columns numbered from col0) when kMasked.
template <bool kMasked>
__device__ __forceinline__ void probs_inplace(uint32_t (&s)[32], uint64_t sc2, uint64_t nl2, int col0, int c_lo, int c_hi) {
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    float x0, x1;
    unpack_f32x2(fma_f32x2(pack_u32x2(s[2 * e], s[2 * e + 1]), sc2, nl2), &x0, &x1);
    float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
    if (kMasked) {
      const int col = col0 + 2 * e;
      if (col < c_lo || col > c_hi) p0 = 0.f;
      if (col + 1 < c_lo || col + 1 > c_hi) p1 = 0.f;
    }
    s[2 * e] = __float_as_uint(p0);
    s[2 * e + 1] = __float_as_uint(p1);
  }
}

// 32 probabilities and raw dP values of one row -> 16 packed dS = p * (dp + ndelta).
template <typename T>
__device__ __forceinline__ void dscore_row(const uint32_t (&p)[32], const uint32_t (&dp)[32], uint64_t nd2,
                                           uint32_t (&dsk)[16]) {
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    float d0, d1;
    unpack_f32x2(mul_f32x2(pack_u32x2(p[2 * e], p[2 * e + 1]), add_f32x2(pack_u32x2(dp[2 * e], dp[2 * e + 1]), nd2)), &d0,
                 &d1);
    dsk[e] = DType<T>::pack2(d0, d1);
  }
}

inline int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace
}  // namespace fa
