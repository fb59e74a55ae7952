// FlashAttention-2 backward for sm_100a as two tcgen05 kernels (delta = rowsum(O*dO) is computed
// before them). Accumulators live in tensor memory; operand tiles arrive by TMA; both kernels use
//   warps 0-3, 4-7  two compute groups, each owning 64 of the 128 score columns of a tile
//   warp 8          TMA producer (one lane)
//   warp 9          MMA issuer (one lane)
//
// dK/dV kernel: one CTA per 128-key tile of one (batch, kv head); K and V stay in shared memory and
// the CTA walks the query tiles of every query head of the GQA group (no atomics, fixed summation
// order). Per query tile:
//     S^T  = K Q^T          dP^T = V dO^T                  (M = keys, N = queries)
//     P^T  = exp2(S^T*c - lse[q]) ;  dS^T = P^T * (dP^T - delta[q])      (registers; lse/delta per column)
//     dV  += P^T dO         dK  += dS^T Q                  (A from TMEM, B = the same smem tiles, MN-major)
// TMEM: S^T [0,128) dP^T [128,256) dK [256,256+D) dV [256+D,256+2D).
//
// dQ kernel: one CTA per 128-query tile of one (batch, head); Q and dO stay resident, K/V stream:
//     S = Q K^T    dP = dO V^T    dS = P*(dP - delta[row])    dQ += dS K
// TMEM: S [0,128) dP [128,256) dQ [256,256+D).
//
// The 16-bit P^T / dS^T (and dS) operands overwrite the first 32 columns of the 64-column block of
// S^T / dP^T that the writing group itself owns, so no group overwrites data another group still reads.
//
// Math follows fa_rdna3/kernels/_common.py:347-508 and fa_rdna3/kernels/backward.py:56-322 (varlen:
// fa_rdna3/kernels/varlen.py:193-421): P recomputed from LSE, rows with LSE = -inf contribute nothing,
// softcap chain factor (1 - tanh^2), dropout regenerated from the same counters, dQ and dK scaled by
// softmax_scale at the end.
#include "fa_common.cuh"
#include "fa_sm100.cuh"
#include "fa_tma_host.h"

namespace fa {
namespace {

constexpr int kBwdThreads = 320;
constexpr uint32_t kFull = 0xffffffffu;

struct BwdArgs {
  int varlen, heads_q, heads_kv, seqlen_q, seqlen_k, total_q, total_k;
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
  int num_tiles_x;
  int* status;
};

__device__ __forceinline__ void report_timeout(int* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

__device__ __forceinline__ ScoreMods make_mods(const BwdArgs& a, int b, int h, int Sq, int Sk) {
  ScoreMods m;
  m.scale_log2 = a.softmax_scale * kLog2e;
  m.cap_log2 = a.softcap > 0.f ? a.softcap * kLog2e : 0.f;
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

// True when some (query, key) pair of the tile rows [r0, r0+127] x keys [k0, k0+127] may be masked.
__device__ __forceinline__ bool tile_needs_mask(const ScoreMods& m, int r0, int k0) {
  const int off = m.seqlen_k - m.seqlen_q;
  return (k0 + 128 > m.seqlen_k) || (r0 + 128 > m.seqlen_q) || (m.causal && (k0 + 127 > r0 + off)) ||
         (m.window_left >= 0 && (k0 < r0 + 127 + off - m.window_left)) ||
         (!m.causal && m.window_right >= 0 && (k0 + 127 > r0 + off + m.window_right));
}

// One score element of the backward pass. lse2 = lse*log2(e), or +inf for rows that contribute nothing.
template <bool kMods>
__device__ __forceinline__ void bwd_element(const ScoreMods& m, bool masked_tile, float raw_s, float raw_dp, float lse2,
                                            float delta, int i, int j, float* p_drop, float* ds) {
  float p, t = 0.f;
  if (kMods) {
    p = fast_exp2(m.logit(raw_s, i, j, &t) - lse2);
  } else {
    p = fast_exp2(fmaf(raw_s, m.scale_log2, -lse2));
  }
  if (masked_tile && !m.keep(i, j)) p = 0.f;
  float dp = raw_dp, pd = p;
  if (kMods && m.dropout_p > 0.f) {
    const bool kd = m.dropout_keep(i, j);
    pd = kd ? p * m.inv_keep : 0.f;
    dp = kd ? dp * m.inv_keep : 0.f;
  }
  float d = p * (dp - delta);
  if (kMods && m.cap_log2 > 0.f) d *= (1.f - t * t);
  *p_drop = pd;
  *ds = d;
}

// Converts a 32-column fp32 slice of a TMEM accumulator to 16-bit and writes it to a global row.
template <typename T>
__device__ __forceinline__ void store_row_slice(T* dst, const uint32_t (&o)[32], float scale) {
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    uint4 pkt;
    pkt.x = DType<T>::pack2(__uint_as_float(o[v * 8 + 0]) * scale, __uint_as_float(o[v * 8 + 1]) * scale);
    pkt.y = DType<T>::pack2(__uint_as_float(o[v * 8 + 2]) * scale, __uint_as_float(o[v * 8 + 3]) * scale);
    pkt.z = DType<T>::pack2(__uint_as_float(o[v * 8 + 4]) * scale, __uint_as_float(o[v * 8 + 5]) * scale);
    pkt.w = DType<T>::pack2(__uint_as_float(o[v * 8 + 6]) * scale, __uint_as_float(o[v * 8 + 7]) * scale);
    *reinterpret_cast<uint4*>(dst + v * 8) = pkt;
  }
}

__device__ __forceinline__ void compute_group_sync() {
  asm volatile("bar.sync 1, 256;" ::: "memory");  // the eight compute warps only
}

// =============================================================================================
// dK / dV
// =============================================================================================
template <typename T, int D, bool kMods>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_dkdv_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                const BwdArgs a) {
  constexpr int kChunks = D / 64;
  constexpr int kTileBytes = kChunks * 16384;
  constexpr int kStages = 2;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + kTileBytes;
  uint8_t* sQdO = smem + 2 * kTileBytes;  // [stage][Q | dO]
  __shared__ uint64_t kv_full, qdo_full[kStages], qdo_empty[kStages], s_full, p_full, acc_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ float lse_s[2][128], delta_s[2][128];

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int ktile = blockIdx.x;
  const int b = blockIdx.y / a.heads_kv, hk = blockIdx.y % a.heads_kv;
  const int group = a.heads_q / a.heads_kv;

  int q_start = 0, k_start = 0, Sq = a.seqlen_q, Sk = a.seqlen_k;
  if (a.varlen) {
    bounded_sequence(a.cu_q, b, a.total_q, &q_start, &Sq);
    bounded_sequence(a.cu_k, b, a.total_k, &k_start, &Sk);
  }
  const int k0 = ktile * 128;
  if (k0 >= Sk) return;
  const int tb = a.varlen ? 0 : b;

  // query-tile range; the mask geometry does not depend on the head
  ScoreMods mods = make_mods(a, b, hk * group, Sq, Sk);
  int ilo, ihi;
  query_range_for_keys(mods, k0, min(k0 + 127, Sk - 1), &ilo, &ihi);
  int tlo = ilo / 128, thi = (ihi + 127) / 128;
  if (thi <= tlo) tlo = thi = 0;
  const int tiles_per_head = thi - tlo;
  const int n_total = tiles_per_head * group;

  if (tid == 0) {
    mbar_init(&kv_full, 1);
    mbar_init(&s_full, 1);
    mbar_init(&p_full, 256);
    mbar_init(&acc_done, 1);
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
    }
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  constexpr uint32_t kColS = 0, kColDP = 128, kColDK = 256, kColDV = 256 + D;

  if (warp == 8) {
    if (lane == 0 && n_total > 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_do);
      mbar_arrive_expect_tx(&kv_full, 2 * kTileBytes);
#pragma unroll
      for (int c = 0; c < kChunks; ++c) {
        tma_load_4d(sK + c * 16384, &map_k, &kv_full, c * 64, k_start + k0, hk, tb);
        tma_load_4d(sV + c * 16384, &map_v, &kv_full, c * 64, k_start + k0, hk, tb);
      }
      for (int n = 0; n < n_total; ++n) {
        const int stage = n % kStages;
        if (!mbar_wait(&qdo_empty[stage], ((n / kStages) & 1) ^ 1)) {
          report_timeout(a.status, 201);
          break;
        }
        const int h = hk * group + n / tiles_per_head;
        const int row = q_start + (tlo + n % tiles_per_head) * 128;
        uint8_t* dst = sQdO + stage * 2 * kTileBytes;
        mbar_arrive_expect_tx(&qdo_full[stage], 2 * kTileBytes);
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
          tma_load_4d(dst + c * 16384, &map_q, &qdo_full[stage], c * 64, row, h, tb);
          tma_load_4d(dst + kTileBytes + c * 16384, &map_do, &qdo_full[stage], c * 64, row, h, tb);
        }
      }
    }
  } else if (warp == 9) {
    if (lane == 0 && n_total > 0) {
      constexpr uint32_t idesc_s = make_idesc(DType<T>::kFormat, 128, 128, 0, 0);
      constexpr uint32_t idesc_acc = make_idesc(DType<T>::kFormat, 128, D, 0, 1);
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), qdo_addr = smem_u32(sQdO);
      bool ok = mbar_wait(&kv_full, 0);
      if (!ok) report_timeout(a.status, 202);
      for (int n = 0; n < n_total && ok; ++n) {
        const int stage = n % kStages;
        if (!mbar_wait(&qdo_full[stage], (n / kStages) & 1)) {
          report_timeout(a.status, 203);
          break;
        }
        tc_fence_after_sync();
        const uint32_t q_addr = qdo_addr + stage * 2 * kTileBytes, do_addr = q_addr + kTileBytes;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
          mma_ss(tmem_base + kColS, make_smem_desc(k_addr + off, 16, 1024), make_smem_desc(q_addr + off, 16, 1024),
                 idesc_s, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
          mma_ss(tmem_base + kColDP, make_smem_desc(v_addr + off, 16, 1024), make_smem_desc(do_addr + off, 16, 1024),
                 idesc_s, kk > 0);
        }
        tc_commit(&s_full);
        if (!mbar_wait(&p_full, n & 1)) {
          report_timeout(a.status, 204);
          break;
        }
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {  // 16 queries per step
          const uint32_t a_col = (kk / 4) * 64 + (kk % 4) * 8;
          mma_ts(tmem_base + kColDV, tmem_base + kColS + a_col, make_smem_desc(do_addr + kk * 2048, 16384, 1024),
                 idesc_acc, !(n == 0 && kk == 0));
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t a_col = (kk / 4) * 64 + (kk % 4) * 8;
          mma_ts(tmem_base + kColDK, tmem_base + kColDP + a_col, make_smem_desc(q_addr + kk * 2048, 16384, 1024),
                 idesc_acc, !(n == 0 && kk == 0));
        }
        tc_commit(&qdo_empty[stage]);
        if (n == n_total - 1) tc_commit(&acc_done);
      }
    }
  } else {
    const int wg = warp / 4, w4 = warp % 4;
    const int ctid = tid;  // 0..255 among compute threads
    const int key_row = w4 * 32 + lane;
    const int j = k0 + key_row;
    const uint32_t lane_addr = static_cast<uint32_t>(w4 * 32) << 16;
    const uint32_t tS = tmem_base + lane_addr + kColS + wg * 64;
    const uint32_t tDP = tmem_base + lane_addr + kColDP + wg * 64;
    bool ok = true;

    for (int n = 0; n < n_total; ++n) {
      const int h = hk * group + n / tiles_per_head;
      const int q0 = (tlo + n % tiles_per_head) * 128;
      if (n % tiles_per_head == 0) mods = make_mods(a, b, h, Sq, Sk);
      // stage this tile's per-query LSE (log2 domain; +inf = contributes nothing) and delta
      if (ctid < 128) {
        const int i = q0 + ctid;
        float l2 = INFINITY, dl = 0.f;
        if (i < Sq) {
          const int64_t bo = a.varlen ? 0 : (int64_t)b;
          const float l = a.lse[bo * a.l_sb + (int64_t)h * a.l_sh + (int64_t)(q_start + i) * a.l_ss];
          l2 = (l == kNegInf) ? INFINITY : l * kLog2e;
          dl = a.delta[bo * a.d_sb + (int64_t)h * a.d_sh + (int64_t)(q_start + i) * a.d_ss];
        }
        lse_s[n & 1][ctid] = l2;
        delta_s[n & 1][ctid] = dl;
      }
      compute_group_sync();
      const bool w_ok = mbar_wait(&s_full, n & 1);
      if (!__all_sync(kFull, w_ok)) {
        report_timeout(a.status, 205);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      uint32_t s[64], dp[64];
      tmem_ld32(tS, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      tmem_ld32(tS + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
      tmem_ld32(tDP, *reinterpret_cast<uint32_t(*)[32]>(&dp[0]));
      tmem_ld32(tDP + 32, *reinterpret_cast<uint32_t(*)[32]>(&dp[32]));
      tc_wait_ld();
      const bool masked = tile_needs_mask(mods, q0, k0);
      uint32_t pk[32], dsk[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const int col = wg * 64 + 2 * c;
        float p0, p1, d0, d1;
        bwd_element<kMods>(mods, masked, __uint_as_float(s[2 * c]), __uint_as_float(dp[2 * c]), lse_s[n & 1][col],
                           delta_s[n & 1][col], q0 + col, j, &p0, &d0);
        bwd_element<kMods>(mods, masked, __uint_as_float(s[2 * c + 1]), __uint_as_float(dp[2 * c + 1]),
                           lse_s[n & 1][col + 1], delta_s[n & 1][col + 1], q0 + col + 1, j, &p1, &d1);
        pk[c] = DType<T>::pack2(p0, p1);
        dsk[c] = DType<T>::pack2(d0, d1);
      }
      tmem_st32(tS, pk);
      tmem_st32(tDP, dsk);
      tc_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&p_full);
    }

    // epilogue: group 0 writes dK (scaled), group 1 writes dV
    if (n_total > 0) {
      const bool w_ok = ok && mbar_wait(&acc_done, 0);
      if (!__all_sync(kFull, w_ok)) {
        if (ok) report_timeout(a.status, 206);
        ok = false;
      }
    }
    if (ok) {
      tc_fence_after_sync();
      const int64_t bo = a.varlen ? 0 : (int64_t)b;
      T* row_ptr = (wg == 0)
                       ? reinterpret_cast<T*>(a.dk) + bo * a.dk_sb + (int64_t)hk * a.dk_sh + (int64_t)(k_start + j) * a.dk_ss
                       : reinterpret_cast<T*>(a.dv) + bo * a.dv_sb + (int64_t)hk * a.dv_sh + (int64_t)(k_start + j) * a.dv_ss;
      const uint32_t tAcc = tmem_base + lane_addr + (wg == 0 ? kColDK : kColDV);
      const float sc = (wg == 0) ? a.softmax_scale : 1.f;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        if (n_total > 0) {
          tmem_ld32(tAcc + c * 32, o);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = 0u;
        }
        if (j < Sk) store_row_slice<T>(row_ptr + c * 32, o, sc);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem_base, 512);
}

// =============================================================================================
// dQ
// =============================================================================================
template <typename T, int D, bool kMods>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
              const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
              const BwdArgs a) {
  constexpr int kChunks = D / 64;
  constexpr int kTileBytes = kChunks * 16384;
  constexpr int kStages = 2;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = smem + kTileBytes;
  uint8_t* sKV = smem + 2 * kTileBytes;  // [stage][K | V]
  __shared__ uint64_t qdo_full, kv_full[kStages], kv_empty[kStages], s_full, ds_full, acc_done;
  __shared__ uint32_t tmem_base_s;

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int qtile = a.num_tiles_x - 1 - blockIdx.x;
  const int b = blockIdx.y / a.heads_q, h = blockIdx.y % a.heads_q;
  const int hk = h / (a.heads_q / a.heads_kv);

  int q_start = 0, k_start = 0, Sq = a.seqlen_q, Sk = a.seqlen_k;
  if (a.varlen) {
    bounded_sequence(a.cu_q, b, a.total_q, &q_start, &Sq);
    bounded_sequence(a.cu_k, b, a.total_k, &k_start, &Sk);
  }
  const int q0 = qtile * 128;
  if (q0 >= Sq) return;
  const int tb = a.varlen ? 0 : b;

  const ScoreMods mods = make_mods(a, b, h, Sq, Sk);
  int klo, khi;
  key_range_for_rows(mods, q0, min(q0 + 127, Sq - 1), &klo, &khi);
  int jlo = klo / 128, jhi = (khi + 127) / 128;
  if (jhi <= jlo) jlo = jhi = 0;
  const int n_total = jhi - jlo;

  if (tid == 0) {
    mbar_init(&qdo_full, 1);
    mbar_init(&s_full, 1);
    mbar_init(&ds_full, 256);
    mbar_init(&acc_done, 1);
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  constexpr uint32_t kColS = 0, kColDP = 128, kColDQ = 256;

  if (warp == 8) {
    if (lane == 0 && n_total > 0) {
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      mbar_arrive_expect_tx(&qdo_full, 2 * kTileBytes);
#pragma unroll
      for (int c = 0; c < kChunks; ++c) {
        tma_load_4d(sQ + c * 16384, &map_q, &qdo_full, c * 64, q_start + q0, h, tb);
        tma_load_4d(sdO + c * 16384, &map_do, &qdo_full, c * 64, q_start + q0, h, tb);
      }
      for (int n = 0; n < n_total; ++n) {
        const int stage = n % kStages;
        if (!mbar_wait(&kv_empty[stage], ((n / kStages) & 1) ^ 1)) {
          report_timeout(a.status, 301);
          break;
        }
        const int row = k_start + (jlo + n) * 128;
        uint8_t* dst = sKV + stage * 2 * kTileBytes;
        mbar_arrive_expect_tx(&kv_full[stage], 2 * kTileBytes);
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
          tma_load_4d(dst + c * 16384, &map_k, &kv_full[stage], c * 64, row, hk, tb);
          tma_load_4d(dst + kTileBytes + c * 16384, &map_v, &kv_full[stage], c * 64, row, hk, tb);
        }
      }
    }
  } else if (warp == 9) {
    if (lane == 0 && n_total > 0) {
      constexpr uint32_t idesc_s = make_idesc(DType<T>::kFormat, 128, 128, 0, 0);
      constexpr uint32_t idesc_acc = make_idesc(DType<T>::kFormat, 128, D, 0, 1);
      const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sdO), kv_addr = smem_u32(sKV);
      bool ok = mbar_wait(&qdo_full, 0);
      if (!ok) report_timeout(a.status, 302);
      for (int n = 0; n < n_total && ok; ++n) {
        const int stage = n % kStages;
        if (!mbar_wait(&kv_full[stage], (n / kStages) & 1)) {
          report_timeout(a.status, 303);
          break;
        }
        tc_fence_after_sync();
        const uint32_t k_addr = kv_addr + stage * 2 * kTileBytes, v_addr = k_addr + kTileBytes;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
          mma_ss(tmem_base + kColS, make_smem_desc(q_addr + off, 16, 1024), make_smem_desc(k_addr + off, 16, 1024),
                 idesc_s, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
          mma_ss(tmem_base + kColDP, make_smem_desc(do_addr + off, 16, 1024), make_smem_desc(v_addr + off, 16, 1024),
                 idesc_s, kk > 0);
        }
        tc_commit(&s_full);
        if (!mbar_wait(&ds_full, n & 1)) {
          report_timeout(a.status, 304);
          break;
        }
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {  // 16 keys per step
          const uint32_t a_col = (kk / 4) * 64 + (kk % 4) * 8;
          mma_ts(tmem_base + kColDQ, tmem_base + kColS + a_col, make_smem_desc(k_addr + kk * 2048, 16384, 1024),
                 idesc_acc, !(n == 0 && kk == 0));
        }
        tc_commit(&kv_empty[stage]);
        if (n == n_total - 1) tc_commit(&acc_done);
      }
    }
  } else {
    const int wg = warp / 4, w4 = warp % 4;
    const int q_row = w4 * 32 + lane;
    const int i = q0 + q_row;
    const uint32_t lane_addr = static_cast<uint32_t>(w4 * 32) << 16;
    const uint32_t tS = tmem_base + lane_addr + kColS + wg * 64;
    const uint32_t tDP = tmem_base + lane_addr + kColDP + wg * 64;
    const int64_t bo = a.varlen ? 0 : (int64_t)b;
    float lse2 = INFINITY, delta = 0.f;
    if (i < Sq) {
      const float l = a.lse[bo * a.l_sb + (int64_t)h * a.l_sh + (int64_t)(q_start + i) * a.l_ss];
      lse2 = (l == kNegInf) ? INFINITY : l * kLog2e;
      delta = a.delta[bo * a.d_sb + (int64_t)h * a.d_sh + (int64_t)(q_start + i) * a.d_ss];
    }
    bool ok = true;
    for (int n = 0; n < n_total; ++n) {
      const int k0 = (jlo + n) * 128;
      const bool w_ok = mbar_wait(&s_full, n & 1);
      if (!__all_sync(kFull, w_ok)) {
        report_timeout(a.status, 305);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      uint32_t s[64], dp[64];
      tmem_ld32(tS, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      tmem_ld32(tS + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
      tmem_ld32(tDP, *reinterpret_cast<uint32_t(*)[32]>(&dp[0]));
      tmem_ld32(tDP + 32, *reinterpret_cast<uint32_t(*)[32]>(&dp[32]));
      tc_wait_ld();
      const bool masked = tile_needs_mask(mods, q0, k0);
      uint32_t dsk[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const int col = k0 + wg * 64 + 2 * c;
        float p0, p1, d0, d1;
        bwd_element<kMods>(mods, masked, __uint_as_float(s[2 * c]), __uint_as_float(dp[2 * c]), lse2, delta, i, col, &p0,
                           &d0);
        bwd_element<kMods>(mods, masked, __uint_as_float(s[2 * c + 1]), __uint_as_float(dp[2 * c + 1]), lse2, delta, i,
                           col + 1, &p1, &d1);
        dsk[c] = DType<T>::pack2(d0, d1);
      }
      tmem_st32(tS, dsk);
      tc_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&ds_full);
    }

    if (n_total > 0) {
      const bool w_ok = ok && mbar_wait(&acc_done, 0);
      if (!__all_sync(kFull, w_ok)) {
        if (ok) report_timeout(a.status, 306);
        ok = false;
      }
    }
    if (ok) {
      tc_fence_after_sync();
      T* row_ptr = reinterpret_cast<T*>(a.dq) + bo * a.dq_sb + (int64_t)h * a.dq_sh + (int64_t)(q_start + i) * a.dq_ss;
      // each group writes half of the head dimension
      constexpr int kSlices = D / 32 / 2;
#pragma unroll
      for (int cc = 0; cc < kSlices; ++cc) {
        const int c = wg * kSlices + cc;
        uint32_t o[32];
        if (n_total > 0) {
          tmem_ld32(tmem_base + lane_addr + kColDQ + c * 32, o);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = 0u;
        }
        if (i < Sq) store_row_slice<T>(row_ptr + c * 32, o, a.softmax_scale);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem_base, 512);
}

template <typename T, int D, bool kMods>
int launch_typed(const fa_attn_params& p, const BwdArgs& a0, int parts, cudaStream_t stream) {
  constexpr int kTileBytes = (D / 64) * 16384;
  const int smem = 6 * kTileBytes + 1024;
  CUtensorMap mq, mk, mv, mdo;
  const int rows_q = p.varlen ? p.total_q : p.seqlen_q;
  const int rows_k = p.varlen ? p.total_k : p.seqlen_k;
  const int nb = p.varlen ? 1 : p.batch;
  int rc = make_tile_map(&mq, p.q, p.dtype, D, rows_q, p.heads_q, nb, p.q_strides[2], p.q_strides[1], p.q_strides[0]);
  if (rc) return rc;
  rc = make_tile_map(&mk, p.k, p.dtype, D, rows_k, p.heads_kv, nb, p.k_strides[2], p.k_strides[1], p.k_strides[0]);
  if (rc) return rc;
  rc = make_tile_map(&mv, p.v, p.dtype, D, rows_k, p.heads_kv, nb, p.v_strides[2], p.v_strides[1], p.v_strides[0]);
  if (rc) return rc;
  rc = make_tile_map(&mdo, p.dout, p.dtype, D, rows_q, p.heads_q, nb, p.do_strides[2], p.do_strides[1],
                     p.do_strides[0]);
  if (rc) return rc;

  auto kdkdv = bwd_dkdv_kernel<T, D, kMods>;
  auto kdq = bwd_dq_kernel<T, D, kMods>;
  cudaError_t e = cudaFuncSetAttribute(kdkdv, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(kdq, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "backward smem opt-in failed: %s", cudaGetErrorString(e));

  BwdArgs a = a0;
  if (parts & FA_BWD_DKDV) {
    a.num_tiles_x = (p.seqlen_k + 127) / 128;
    kdkdv<<<dim3(a.num_tiles_x, p.batch * p.heads_kv), kBwdThreads, smem, stream>>>(mq, mk, mv, mdo, a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "dK/dV launch failed: %s", cudaGetErrorString(e));
  }
  if (parts & FA_BWD_DQ) {
    a.num_tiles_x = (p.seqlen_q + 127) / 128;
    kdq<<<dim3(a.num_tiles_x, p.batch * p.heads_q), kBwdThreads, smem, stream>>>(mq, mk, mv, mdo, a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "dQ launch failed: %s", cudaGetErrorString(e));
  }
  return 0;
}

}  // namespace

bool bwd_tcgen05_supported(const fa_attn_params& p) {
  if (p.dtype != FA_F16 && p.dtype != FA_BF16) return false;
  if (p.head_dim != 64 && p.head_dim != 128) return false;
  const int64_t nb = p.varlen ? 1 : p.batch;
  const int64_t sq[3] = {nb, p.heads_q, p.varlen ? p.total_q : p.seqlen_q};
  const int64_t sk[3] = {nb, p.heads_kv, p.varlen ? p.total_k : p.seqlen_k};
  return tma_operand_ok(p.q, p.q_strides, sq) && tma_operand_ok(p.k, p.k_strides, sk) &&
         tma_operand_ok(p.v, p.v_strides, sk) && tma_operand_ok(p.dout, p.do_strides, sq) &&
         tma_operand_ok(p.dq, p.dq_strides, sq) && tma_operand_ok(p.dk, p.dk_strides, sk) &&
         tma_operand_ok(p.dv, p.dv_strides, sk);
}

int launch_bwd_tcgen05(const fa_attn_params& p, int parts, cudaStream_t stream) {
  BwdArgs a;
  a.varlen = p.varlen;
  a.heads_q = p.heads_q;
  a.heads_kv = p.heads_kv;
  a.seqlen_q = p.seqlen_q;
  a.seqlen_k = p.seqlen_k;
  a.total_q = p.total_q;
  a.total_k = p.total_k;
  a.cu_q = p.cu_seqlens_q;
  a.cu_k = p.cu_seqlens_k;
  a.lse = p.lse;
  a.l_sb = p.lse_strides[0];
  a.l_sh = p.lse_strides[1];
  a.l_ss = p.lse_strides[2];
  a.delta = p.delta;
  a.d_sb = p.delta_strides[0];
  a.d_sh = p.delta_strides[1];
  a.d_ss = p.delta_strides[2];
  a.dq = p.dq;
  a.dq_sb = p.dq_strides[0];
  a.dq_sh = p.dq_strides[1];
  a.dq_ss = p.dq_strides[2];
  a.dk = p.dk;
  a.dk_sb = p.dk_strides[0];
  a.dk_sh = p.dk_strides[1];
  a.dk_ss = p.dk_strides[2];
  a.dv = p.dv;
  a.dv_sb = p.dv_strides[0];
  a.dv_sh = p.dv_strides[1];
  a.dv_ss = p.dv_strides[2];
  a.softmax_scale = p.softmax_scale;
  a.softcap = p.softcap;
  a.bias = p.bias;
  a.bias_dtype = p.bias_dtype;
  a.bias_sb = p.bias_strides[0];
  a.bias_sh = p.bias_strides[1];
  a.bias_sm = p.bias_strides[2];
  a.bias_sn = p.bias_strides[3];
  a.alibi = p.alibi_slopes;
  a.causal = p.causal;
  a.wl = p.window_left;
  a.wr = p.window_right;
  a.dropout_p = p.dropout_p;
  a.seed = p.dropout_seed;
  a.num_tiles_x = 0;
  a.status = p.status;
  const bool mods = p.softcap > 0.f || p.bias != nullptr || p.alibi_slopes != nullptr || p.dropout_p > 0.f;
  const bool f16 = p.dtype == FA_F16;
  if (p.head_dim == 128) {
    if (f16) return mods ? launch_typed<__half, 128, true>(p, a, parts, stream) : launch_typed<__half, 128, false>(p, a, parts, stream);
    return mods ? launch_typed<__nv_bfloat16, 128, true>(p, a, parts, stream)
                : launch_typed<__nv_bfloat16, 128, false>(p, a, parts, stream);
  }
  if (f16) return mods ? launch_typed<__half, 64, true>(p, a, parts, stream) : launch_typed<__half, 64, false>(p, a, parts, stream);
  return mods ? launch_typed<__nv_bfloat16, 64, true>(p, a, parts, stream)
              : launch_typed<__nv_bfloat16, 64, false>(p, a, parts, stream);
}

}  // namespace fa
