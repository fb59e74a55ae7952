// Device-side helpers shared by every attention kernel: dtype conversion, the score-modifier chain
// (scale -> softcap -> bias -> ALiBi -> mask, in the order of fa_rdna3/kernels/_common.py:275-308),
// the dropout generator, and error bookkeeping for the C ABI.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../../include/fa_b200.h"

namespace fa {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ---------------------------------------------------------------------------------------------
// dtype helpers
// ---------------------------------------------------------------------------------------------
template <typename T> struct DType;
template <> struct DType<__half> {
  static constexpr int kFormat = 0;
  __device__ static __forceinline__ float to_float(__half x) { return __half2float(x); }
  __device__ static __forceinline__ __half from_float(float x) { return __float2half_rn(x); }
  __device__ static __forceinline__ uint32_t pack2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __device__ static __forceinline__ float2 unpack2(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
};
template <> struct DType<__nv_bfloat16> {
  static constexpr int kFormat = 1;
  __device__ static __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
  __device__ static __forceinline__ __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
  __device__ static __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __device__ static __forceinline__ float2 unpack2(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  }
};
template <> struct DType<float> {
  static constexpr int kFormat = 2;
  __device__ static __forceinline__ float to_float(float x) { return x; }
  __device__ static __forceinline__ float from_float(float x) { return x; }
};

__device__ __forceinline__ float load_as_float(const void* base, int64_t index, int dtype) {
  if (dtype == FA_F16) return __half2float(reinterpret_cast<const __half*>(base)[index]);
  if (dtype == FA_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[index]);
  return reinterpret_cast<const float*>(base)[index];
}

__device__ __forceinline__ void store_from_float(void* base, int64_t index, int dtype, float x) {
  if (dtype == FA_F16) reinterpret_cast<__half*>(base)[index] = __float2half_rn(x);
  else if (dtype == FA_BF16) reinterpret_cast<__nv_bfloat16*>(base)[index] = __float2bfloat16_rn(x);
  else reinterpret_cast<float*>(base)[index] = x;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

constexpr float kNegInf = -INFINITY;

// Three-input max and packed fp32x2 arithmetic (two fp32 lanes in one 64-bit register, one instruction).
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ uint64_t pack_u32x2(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float* lo, float* hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(*lo), "=f"(*hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// ---------------------------------------------------------------------------------------------
// Dropout generator: Philox-4x32-10 keyed by the 64-bit seed, counter = (lo32(offset), hi32(offset), 0, 0),
// first output word mapped to [0, 1) the way Triton's tl.rand does (the reference draws its mask with
// tl.rand(seed, offset), fa_rdna3/kernels/_common.py:338-339). An element is kept when u > p.
// ---------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ uint32_t philox_first_word(uint64_t seed, uint64_t offset) {
  uint32_t c0 = static_cast<uint32_t>(offset), c1 = static_cast<uint32_t>(offset >> 32), c2 = 0, c3 = 0;
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
  for (int r = 0; r < 10; ++r) {
    const uint64_t pa = static_cast<uint64_t>(0xD2511F53u) * c0;
    const uint64_t pb = static_cast<uint64_t>(0xCD9E8D57u) * c2;
    const uint32_t n0 = static_cast<uint32_t>(pb >> 32) ^ c1 ^ k0;
    const uint32_t n2 = static_cast<uint32_t>(pa >> 32) ^ c3 ^ k1;
    c1 = static_cast<uint32_t>(pb);
    c3 = static_cast<uint32_t>(pa);
    c0 = n0;
    c2 = n2;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c0;
}

__host__ __device__ __forceinline__ float philox_uniform(uint64_t seed, uint64_t offset) {
  int32_t x = static_cast<int32_t>(philox_first_word(seed, offset));
  if (x < 0) x = -x - 1;
  return static_cast<float>(x) * 4.6566127342e-10f;
}

// The same draw as a real call: the ten Philox rounds are about a hundred instructions, and the tensor-core kernels
// would otherwise inline them once per element of their unrolled tile loops (hundreds of copies that cost
// instruction-cache misses on every launch, dropout or not).
static __device__ __noinline__ float philox_uniform_call(uint64_t seed, uint64_t offset) {
  return philox_uniform(seed, offset);
}

// tanh(z) from one exp2 and one reciprocal of the special-function unit: 1 - 2 / (e^(2z) + 1). Absolute error about
// 3e-7 (exact limits -1 and 1 for large |z|), far inside the tolerance of a soft-capped logit.
__device__ __forceinline__ float fast_tanh(float z) {
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(z * 2.8853900817779268f));
  return 1.f - __fdividef(2.f, e + 1.f);
}

// ---------------------------------------------------------------------------------------------
// Score modifiers for one (batch, head): everything a kernel needs to turn a raw q.k dot product at
// (query row i, key column j) of one sequence into a log2-domain logit, or -inf when masked.
// ---------------------------------------------------------------------------------------------
struct ScoreMods {
  float scale_log2;      // softmax_scale * log2(e)
  float cap_log2;        // softcap * log2(e); 0 disables
  float inv_cap_log2;    // 1 / cap_log2 (0 when disabled)
  float alibi_slope_log2;// slope * log2(e); 0 disables
  const void* bias;      // already offset to this (batch, head); nullptr disables
  int bias_dtype;
  int64_t bias_stride_m, bias_stride_n;
  int causal, window_left, window_right;
  int seqlen_q, seqlen_k;  // of this sequence
  float dropout_p;         // 0 disables
  float inv_keep;
  uint64_t dropout_seed;
  uint64_t dropout_base;   // (batch * heads + head) * seqlen_q

  __device__ __forceinline__ bool keep(int i, int j) const {
    const int qpos = i + (seqlen_k - seqlen_q);
    bool k = j < seqlen_k;
    if (causal) k = k && (qpos >= j);
    if (window_left >= 0) k = k && (j >= qpos - window_left);
    if (window_right >= 0) k = k && (j <= qpos + window_right);
    return k;
  }

  // Unmasked logit in the log2 domain. tanh_out receives tanh(s / cap) when softcap is on (the
  // backward chain factor is 1 - tanh^2), else 0.
  __device__ __forceinline__ float logit(float raw, int i, int j, float* tanh_out) const {
    float s = raw * scale_log2;
    float t = 0.f;
    if (cap_log2 > 0.f) {
      t = fast_tanh(s * inv_cap_log2);
      s = cap_log2 * t;
    }
    if (bias != nullptr) {
      // rows/columns outside the sequence read nothing (the caller masks them afterwards)
      if (i < seqlen_q && j < seqlen_k)
        s += load_as_float(bias, static_cast<int64_t>(i) * bias_stride_m + static_cast<int64_t>(j) * bias_stride_n,
                           bias_dtype) * kLog2e;
    }
    if (alibi_slope_log2 != 0.f) {
      const int dist = j - i - (seqlen_k - seqlen_q);
      s -= alibi_slope_log2 * static_cast<float>(dist < 0 ? -dist : dist);
    }
    if (tanh_out) *tanh_out = t;
    return s;
  }

  __device__ __forceinline__ bool dropout_keep(int i, int j) const {
    const uint64_t offs = (dropout_base + static_cast<uint64_t>(i)) * static_cast<uint64_t>(seqlen_k) +
                          static_cast<uint64_t>(j);
    return philox_uniform_call(dropout_seed, offs) > dropout_p;
  }
};

// ---- chunk forms of the modifiers, for kernels that hold 32 consecutive scores of one accumulator row in registers.
// Element e is (query i0, key j0 + e) when kAlongKeys, (query i0 + e, key j0) otherwise. Every modifier is one compact
// unrolled block behind one warp-uniform branch, so a launch that uses none of them jumps over four small blocks
// instead of 32 interleaved ones (the per-element form made the instruction stream so sparse that fetch misses
// dominated the kernels).
template <bool kAlongKeys, typename B>
__device__ __forceinline__ void mods_add_bias32(const ScoreMods& m, float (&x)[32], int i0, int j0) {
  const B* base = reinterpret_cast<const B*>(m.bias) + static_cast<int64_t>(i0) * m.bias_stride_m +
                  static_cast<int64_t>(j0) * m.bias_stride_n;
  const int64_t step = kAlongKeys ? m.bias_stride_n : m.bias_stride_m;
  // rows/columns outside the sequence read nothing (the caller masks them afterwards)
  const int room = kAlongKeys ? (i0 < m.seqlen_q ? m.seqlen_k - j0 : 0) : (j0 < m.seqlen_k ? m.seqlen_q - i0 : 0);
#pragma unroll
  for (int e = 0; e < 32; ++e)
    if (e < room) x[e] += DType<B>::to_float(base[e * step]) * kLog2e;
}

// Raw scores -> unmasked logits in the log2 domain, in place. When chain != nullptr, (*chain)[e] is multiplied by the
// soft-cap chain factor 1 - tanh^2 (left alone when soft-capping is off).
template <bool kAlongKeys>
__device__ __forceinline__ void mods_logits32(const ScoreMods& m, float (&x)[32], int i0, int j0, float (*chain)[32]) {
  if (m.cap_log2 > 0.f) {
    const float cap = m.cap_log2, pre = m.scale_log2 * m.inv_cap_log2;
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      const float t = fast_tanh(x[e] * pre);
      x[e] = cap * t;
      if (chain) (*chain)[e] *= fmaf(-t, t, 1.f);
    }
  } else {
    const float sc = m.scale_log2;
#pragma unroll
    for (int e = 0; e < 32; ++e) x[e] *= sc;
  }
  if (m.bias != nullptr) {
    if (m.bias_dtype == FA_F16) mods_add_bias32<kAlongKeys, __half>(m, x, i0, j0);
    else if (m.bias_dtype == FA_BF16) mods_add_bias32<kAlongKeys, __nv_bfloat16>(m, x, i0, j0);
    else mods_add_bias32<kAlongKeys, float>(m, x, i0, j0);
  }
  if (m.alibi_slope_log2 != 0.f) {
    const float slope = m.alibi_slope_log2;
    const int d0 = j0 - i0 - (m.seqlen_k - m.seqlen_q);
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      const int d = kAlongKeys ? d0 + e : d0 - e;
      x[e] = fmaf(-slope, static_cast<float>(d < 0 ? -d : d), x[e]);
    }
  }
}

// Bit e set = element e survives dropout (all ones when dropout is off).
template <bool kAlongKeys>
__device__ __forceinline__ uint32_t mods_dropout_bits32(const ScoreMods& m, int i0, int j0) {
  if (!(m.dropout_p > 0.f)) return 0xffffffffu;
  uint32_t bits = 0u;
#pragma unroll 1
  for (int e = 0; e < 32; ++e)
    bits |= static_cast<uint32_t>(m.dropout_keep(kAlongKeys ? i0 : i0 + e, kAlongKeys ? j0 + e : j0)) << e;
  return bits;
}

// First and one-past-last key index any row of query rows [r0, r1] (inclusive, r1 < seqlen_q) may attend.
__device__ __forceinline__ void key_range_for_rows(const ScoreMods& m, int r0, int r1, int* lo, int* hi) {
  const int off = m.seqlen_k - m.seqlen_q;
  int h = m.seqlen_k;
  if (m.causal) h = min(h, r1 + off + 1);
  else if (m.window_right >= 0) h = min(h, r1 + off + m.window_right + 1);
  int l = 0;
  if (m.window_left >= 0) l = max(0, r0 + off - m.window_left);
  *lo = l;
  *hi = max(h, 0);
}

// First and one-past-last query row any key of [c0, c1] (inclusive, c1 < seqlen_k) may be attended by.
__device__ __forceinline__ void query_range_for_keys(const ScoreMods& m, int c0, int c1, int* lo, int* hi) {
  const int off = m.seqlen_k - m.seqlen_q;
  int l = 0;
  // keep needs qpos >= j (causal) or j <= qpos + right  =>  i >= j - off [- right]
  if (m.causal) l = max(l, c0 - off);
  else if (m.window_right >= 0) l = max(l, c0 - off - m.window_right);
  int h = m.seqlen_q;
  // keep needs j >= qpos - left  =>  i <= j - off + left
  if (m.window_left >= 0) h = min(h, c1 - off + m.window_left + 1);
  *lo = l;
  *hi = max(h, 0);
}

// Sequence bounds of packed batch entry b, clamped into storage (fa_rdna3/kernels/varlen.py:22-27).
__device__ __forceinline__ void bounded_sequence(const int32_t* cu, int b, int total, int* start, int* len) {
  int s = cu[b], e = cu[b + 1];
  s = min(max(s, 0), total);
  e = min(max(e, 0), total);
  *start = s;
  *len = max(e - s, 0);
}

// Packed batches on a compact grid. The host knows the total number of rows but not the lengths, so it launches
// ceil(total / rows_per_tile) + sequences CTAs per head (at least the sum of the sequences' tile counts) and CTA `t`
// finds its (sequence, tile) here: tiles are numbered by falling tile index (kLastFirst: query tiles, whose work under
// a causal mask grows with the index) or by rising tile index (key tiles of the dK/dV kernel, whose work falls with
// it), and among the sequences that have a given tile index by sequence number, so that the long tiles of the long
// sequences start first. seq is -1 for the few CTAs past the last tile. Every thread of the CTA calls it (each warp works it out for itself: 32
// sequences per ballot, at most kPackedMaxSequences); a grid of one CTA per (sequence, possible tile) instead costs
// about 0.9 us of an SM for every tile a sequence does not have.
constexpr int kPackedMaxSequences = 128;
struct PackedTile {
  int seq, tile;
};
template <bool kLastFirst>
__device__ __forceinline__ PackedTile find_packed_tile(const int32_t* cu, int nseq, int total_rows, int rows_per_tile,
                                                       int max_tiles, int t) {
  const int lane = threadIdx.x & 31;
  int tiles[kPackedMaxSequences / 32];
#pragma unroll
  for (int k = 0; k < kPackedMaxSequences / 32; ++k) {
    const int b = k * 32 + lane;
    tiles[k] = 0;
    if (b < nseq) {
      int start, len;
      bounded_sequence(cu, b, total_rows, &start, &len);
      tiles[k] = (len + rows_per_tile - 1) / rows_per_tile;
    }
  }
  PackedTile found = {-1, 0};
  int before = 0;  // tiles numbered before this index
  for (int step = 0; step < max_tiles; ++step) {
    const int idx = kLastFirst ? max_tiles - 1 - step : step;
    unsigned has[kPackedMaxSequences / 32];
    int n = 0;
#pragma unroll
    for (int k = 0; k < kPackedMaxSequences / 32; ++k) {
      has[k] = __ballot_sync(0xffffffffu, tiles[k] > idx);
      n += __popc(has[k]);
    }
    if (t < before + n) {
      int r = t - before;  // the r-th of the sequences that have this tile
#pragma unroll
      for (int k = 0; k < kPackedMaxSequences / 32; ++k) {
        const int c = __popc(has[k]);
        if (found.seq < 0 && r < c) {
          found.seq = k * 32 + (int)__fns(has[k], 0, r + 1);
          found.tile = idx;
        }
        r -= c;
      }
      break;
    }
    before += n;
  }
  return found;
}

// ---------------------------------------------------------------------------------------------
// Host-side error bookkeeping (definitions in fa_api.cu)
// ---------------------------------------------------------------------------------------------
int set_error(int code, const char* fmt, ...);
void set_path(int path);

// Per-family launchers implemented in their own translation units; all return 0 or a negative fa_error.
int launch_fwd_tcgen05(const fa_attn_params& p, cudaStream_t stream);   // fa_fwd_sm100.cu
bool fwd_tcgen05_supported(const fa_attn_params& p);
int launch_bwd_tcgen05(const fa_attn_params& p, int parts, cudaStream_t stream);   // fa_bwd_sm100.cu
bool bwd_tcgen05_supported(const fa_attn_params& p);
int64_t bwd_ds_workspace_bytes(const fa_attn_params& p);
int launch_bwd_wide(const fa_attn_params& p, int parts, cudaStream_t stream);      // fa_wide_sm100.cu
bool bwd_wide_supported(const fa_attn_params& p);
int64_t bwd_wide_workspace_bytes(const fa_attn_params& p);
int launch_fwd_wide(const fa_attn_params& p, cudaStream_t stream);
bool fwd_wide_supported(const fa_attn_params& p);
int64_t fwd_wide_workspace_bytes(const fa_attn_params& p);
int launch_fwd_simt(const fa_attn_params& p, cudaStream_t stream);      // fa_simt.cu
int launch_bwd_simt(const fa_attn_params& p, int parts, cudaStream_t stream);      // fa_simt.cu
int launch_tiled_fwd(const fa_attn_params& p, cudaStream_t stream);    // fa_tiled_fwd.cu
int launch_tiled_dq(const fa_attn_params& p, cudaStream_t stream);     // fa_tiled_dq.cu
int launch_tiled_dkdv(const fa_attn_params& p, cudaStream_t stream);   // fa_tiled_dkdv.cu
int launch_peer_merge(const fa_peer_merge_params& p, cudaStream_t stream);  // fa_decode.cu
int launch_bwd_delta(const fa_attn_params& p, cudaStream_t stream);     // fa_simt.cu
int launch_decode_splitk(const fa_decode_params& p, cudaStream_t stream);  // fa_decode.cu
int launch_combine(const fa_combine_params& p, cudaStream_t stream);       // fa_decode.cu
int launch_decode_paged(const fa_paged_params& p, cudaStream_t stream);    // fa_paged.cu
int launch_tiny(const fa_tiny_params& p, cudaStream_t stream);             // fa_tiny.cu
bool decode_tc_supported(const fa_decode_params& p);                       // fa_decode_sm100.cu
int launch_decode_tc(const fa_decode_params& p, cudaStream_t stream);
// `words` zeroed ticket words of the library's fixed array for launches that use this partial buffer, or nullptr (array
// used up, or first use on this device while the stream is being captured); every launch leaves its words at zero
unsigned int* decode_ticket_words(const void* partial_buffer, int words, cudaStream_t stream);
bool paged_tc_supported(const fa_paged_params& p);
int launch_paged_tc(const fa_paged_params& p, cudaStream_t stream);
void set_decode_fault_injection(uint32_t poll_limit, int skip_tile);

}  // namespace fa
