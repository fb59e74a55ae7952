// FlashAttention-2 forward for sm_100a: tcgen05 MMAs with the score and output accumulators in tensor
// memory, K/V tiles streamed by TMA through a shared-memory ring, warp-specialised roles.
//
// One CTA owns 256 query rows (two 128-row tiles) of one (batch, head):
//   warps 0-3   softmax group for tile 0   (thread = one query row; TMEM lane = row)
//   warps 4-7   softmax group for tile 1
//   warp  8     TMA producer (one lane): Q once, then K_j, V_j, K_j+1, V_j+1 ... into the ring
//   warp  9     MMA issuer (one lane):   S_t = Q_t K_j^T,  O_t += P_t V_j
// The MMA order is QK0, QK1, then per key tile { PV0, QK0', PV1, QK1' } so that while one group runs
// its softmax the tensor core works for the other. P (16-bit) overwrites the first 64 columns of its
// S tile in TMEM and is consumed from there as the A operand of the PV MMA; V is used straight from
// the TMA-swizzled tile as an MN-major B operand. The running maximum is only refreshed (and O
// rescaled in TMEM) when it grows by more than 2^8, so the O round trip is rare.
//
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D).
//
// Semantics follow fa_rdna3/kernels/forward.py:28-164 and fa_rdna3/kernels/_common.py:233-345
// (varlen: fa_rdna3/kernels/varlen.py:42-149): modifier order, bottom-right causal alignment,
// O = 0 / LSE = -inf for rows with no visible key, natural-log LSE.
#include "fa_common.cuh"
#include "fa_sm100.cuh"
#include "fa_tma_host.h"
#include "fa_prof.cuh"

namespace fa {
namespace {

// Three warpgroups: two softmax groups and one group whose first two warps are the TMA producer and the MMA issuer
// (the other two only take part in the register hand-over and the final barrier).
constexpr int kFwdThreads = 384;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct FwdArgs {
  int varlen, heads_q, heads_kv, seqlen_q, seqlen_k, total_q, total_k;
  int head_dim;  // the caller's; the kernel's D is 64 or 128 and the columns in between load as zeros
  const int32_t* cu_q;
  const int32_t* cu_k;
  void* out;
  int64_t o_sb, o_sh, o_ss;
  float* lse;
  int64_t l_sb, l_sh, l_ss;
  float softmax_scale, softcap;
  const void* bias;
  int bias_dtype;
  int64_t bias_sb, bias_sh, bias_sm, bias_sn;
  const float* alibi;
  int causal, wl, wr;
  float dropout_p;
  uint64_t seed;
  int num_pairs;
  int batch;    // sequences of a packed batch
  int compact;  // packed batch on the compact grid (head, tile number): see find_packed_tile
  int* status;
};

__device__ __forceinline__ void report_timeout(int* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

// Multiplies this thread's row of the O accumulator (D fp32 columns in TMEM) by alpha.
template <int D>
__device__ __forceinline__ void rescale_o(uint32_t tO, float alpha) {
#pragma unroll
  for (int c = 0; c < D / 32; ++c) {
    uint32_t o[32];
    tmem_ld32(tO + c * 32, o);
    tc_wait_ld();
#pragma unroll
    for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
    tmem_st32(tO + c * 32, o);
  }
  tc_wait_st();
}

template <typename T, int D, bool kMods>
__global__ void __launch_bounds__(kFwdThreads, 1)
fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
           const __grid_constant__ CUtensorMap map_v, const FwdArgs a) {
  constexpr int kChunks = D / 64;
  constexpr int kTileBytes = kChunks * 16384;  // one 128-row operand tile (rows of 128 B, 128-byte swizzle)
  // Head dims above 128 ("wide"): one 128-row query tile per CTA with a 256-column O accumulator, the S tile
  // double-buffered in the 256 columns the second query tile would use, and one softmax group (the other idles).
  constexpr bool kWide = D > 128;
  constexpr int kQTiles = kWide ? 1 : 2;
  constexpr int kSlots = kWide ? 2 : (D == 128) ? 4 : 6;
  constexpr uint32_t kFull = 0xffffffffu;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + kQTiles * kTileBytes;
  __shared__ uint64_t q_full[2], kv_full[kSlots], kv_empty[kSlots], s_full[2], p_full[2], o_ready[2];
  __shared__ uint32_t tmem_base_s;

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  int pair = a.num_pairs - 1 - blockIdx.y;  // blocks are issued x-fastest: all the long (causal) tiles go first
  int b = blockIdx.x / a.heads_q, h = blockIdx.x % a.heads_q;
  if (a.compact) {
    const PackedTile pt = find_packed_tile<true>(a.cu_q, a.batch, a.total_q, kQTiles * 128, a.num_pairs, blockIdx.y);
    if (pt.seq < 0) return;  // uniform: nothing allocated yet
    b = pt.seq;
    pair = pt.tile;
    h = blockIdx.x;
  }
  const int hk = h / (a.heads_q / a.heads_kv);

  int q_start = 0, k_start = 0, Sq = a.seqlen_q, Sk = a.seqlen_k;
  if (a.varlen) {
    bounded_sequence(a.cu_q, b, a.total_q, &q_start, &Sq);
    bounded_sequence(a.cu_k, b, a.total_k, &k_start, &Sk);
  }
  const int row_base = pair * (kQTiles * 128);
  if (row_base >= Sq) return;  // uniform: nothing allocated yet
  const int tb = a.varlen ? 0 : b;  // batch coordinate of the tensor maps

  ScoreMods mods;
  mods.scale_log2 = a.softmax_scale * kLog2e;
  mods.cap_log2 = a.softcap > 0.f ? a.softcap * kLog2e : 0.f;
  mods.inv_cap_log2 = a.softcap > 0.f ? 1.f / mods.cap_log2 : 0.f;
  mods.alibi_slope_log2 = a.alibi ? a.alibi[h] * kLog2e : 0.f;
  mods.bias = nullptr;
  mods.bias_dtype = a.bias_dtype;
  mods.bias_stride_m = a.bias_sm;
  mods.bias_stride_n = a.bias_sn;
  if (a.bias) {
    const int esz = a.bias_dtype == FA_F32 ? 4 : 2;
    mods.bias = reinterpret_cast<const char*>(a.bias) + ((int64_t)b * a.bias_sb + (int64_t)h * a.bias_sh) * esz;
  }
  mods.causal = a.causal;
  mods.window_left = a.wl;
  mods.window_right = a.wr;
  mods.seqlen_q = Sq;
  mods.seqlen_k = Sk;
  mods.dropout_p = a.dropout_p;
  mods.inv_keep = a.dropout_p > 0.f ? 1.f / (1.f - a.dropout_p) : 1.f;
  mods.dropout_seed = a.seed;
  mods.dropout_base = ((uint64_t)b * (uint64_t)a.heads_q + (uint64_t)h) * (uint64_t)Sq;

  // key-tile range [lo, hi) of each query tile; a tile past the sequence end is inactive
  int lo[2], hi[2];
  bool active[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int r0 = row_base + t * 128;
    active[t] = r0 < Sq && t < kQTiles;
    lo[t] = hi[t] = 0;
    if (active[t]) {
      int klo, khi;
      key_range_for_rows(mods, r0, min(r0 + 127, Sq - 1), &klo, &khi);
      lo[t] = klo / 128;
      hi[t] = (khi + 127) / 128;
      if (hi[t] <= lo[t]) lo[t] = hi[t] = 0;
    }
  }
  const bool any0 = hi[0] > lo[0], any1 = hi[1] > lo[1];
  const int jlo = any0 && any1 ? min(lo[0], lo[1]) : (any0 ? lo[0] : lo[1]);
  const int jhi = any0 && any1 ? max(hi[0], hi[1]) : (any0 ? hi[0] : hi[1]);
  const bool any_work = any0 || any1;

  if (tid == 0) {
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      mbar_init(&q_full[t], 1);
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 128);
      mbar_init(&o_ready[t], 1);
    }
#pragma unroll
    for (int s = 0; s < kSlots; ++s) {
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

  // Register hand-over (every warp of a warpgroup executes the same instruction): the service group gives registers
  // back, the softmax groups take them so that a whole 128-column S row fits in registers. Per scheduler partition:
  // two softmax warps at 224 plus one service warp at 56 stay within the 512 registers per lane.
  if (warp >= 8) {
   asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
   if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && any_work) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (hi[t] > lo[t]) {
          mbar_arrive_expect_tx(&q_full[t], kTileBytes);
#pragma unroll
          for (int c = 0; c < kChunks; ++c)
            tma_load_4d(sQ + t * kTileBytes + c * 16384, &map_q, &q_full[t], c * 64, q_start + row_base + t * 128, h,
                        tb);
        }
      }
      int n = 0;
      bool ok = true;
      for (int j = jlo; j < jhi && ok; ++j) {
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          const int slot = n % kSlots;
          const uint32_t par = ((n / kSlots) & 1) ^ 1;
          if (!mbar_wait(&kv_empty[slot], par)) {
            report_timeout(a.status, 101);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&kv_full[slot], kTileBytes);
#pragma unroll
          for (int c = 0; c < kChunks; ++c)
            tma_load_4d(sKV + slot * kTileBytes + c * 16384, which == 0 ? &map_k : &map_v, &kv_full[slot], c * 64,
                        k_start + j * 128, hk, tb);
          ++n;
        }
      }
    }
   } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && any_work) {
      constexpr uint32_t idesc_qk = make_idesc(DType<T>::kFormat, 128, 128, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc(DType<T>::kFormat, 128, D, 0, 1);
      const uint32_t sq_addr = smem_u32(sQ), skv_addr = smem_u32(sKV);
      bool ok = true;
      PROF_DECL;
      auto slot_addr = [&](int n) { return skv_addr + (n % kSlots) * kTileBytes; };
      auto wait_full = [&](int n) {
        if (!mbar_wait(&kv_full[n % kSlots], (n / kSlots) & 1)) {
          report_timeout(a.status, 102);
          ok = false;
        }
      };
      auto in_range = [&](int t, int j) { return j >= lo[t] && j < hi[t]; };
      // sbuf: which 128-column S buffer (and s_full barrier) the tile uses: the query tile's own, or for wide head dims
      // the parity of the key tile
      auto issue_qk = [&](int t, int n, int sbuf) {
        const uint32_t qa = sq_addr + t * kTileBytes, ka = slot_addr(n);
        // descriptors as 32-bit halves: stepping along the tile is one add per operand (the issuing thread shares its
        // scheduler with two softmax warps, so every instruction it saves is tensor-pipe time)
        const uint32_t q_lo = smem_desc_lo(qa, 16), k_lo = smem_desc_lo(ka, 16);
        constexpr uint32_t hi = smem_desc_hi(1024);
        mma_ss_lo<0>(tmem_base + sbuf * 128, q_lo, hi, k_lo, hi, idesc_qk);
#pragma unroll
        for (int kk = 1; kk < D / 16; ++kk) {
          const uint32_t off = ((kk / 4) * 16384 + (kk % 4) * 32) >> 4;
          mma_ss_lo<1>(tmem_base + sbuf * 128, q_lo + off, hi, k_lo + off, hi, idesc_qk);
        }
        tc_commit(&s_full[sbuf]);
      };
      auto issue_pv = [&](int t, int n, bool first, int sbuf) {
        const uint32_t va = slot_addr(n);
        const uint32_t v_lo = smem_desc_lo(va, 16384);
        constexpr uint32_t hi = smem_desc_hi(1024);
        if (first) mma_ts_lo<0>(tmem_base + 256 + t * D, tmem_base + sbuf * 128, v_lo, hi, idesc_pv);
        else mma_ts_lo<1>(tmem_base + 256 + t * D, tmem_base + sbuf * 128, v_lo, hi, idesc_pv);
#pragma unroll
        for (int kk = 1; kk < 8; ++kk)
          mma_ts_lo<1>(tmem_base + 256 + t * D, tmem_base + sbuf * 128 + kk * 8, v_lo + kk * (2048 >> 4), hi, idesc_pv);
        tc_commit(&o_ready[t]);
      };

#pragma unroll
      for (int t = 0; t < 2; ++t)
        if (hi[t] > lo[t] && ok && !mbar_wait(&q_full[t], 0)) {
          report_timeout(a.status, 103);
          ok = false;
        }
      tc_fence_after_sync();
      if constexpr (kWide) {
        // One query tile: Q K^T of key tile i + 1 goes to the other S buffer before P V of tile i is issued, so it runs
        // while the softmax group works on tile i. Ring: K(i) and V(i) take the two slots in turn.
        if (ok) {
          wait_full(0);
          if (ok) {
            tc_fence_after_sync();
            issue_qk(0, 0, 0);
            tc_commit(&kv_empty[0]);
          }
        }
        for (int j = jlo; j < jhi && ok; ++j) {
          const int i = j - jlo, nv = 2 * i + 1, nk_next = 2 * i + 2;
          if (j + 1 < jhi) {
            wait_full(nk_next);
            if (!ok) break;
            tc_fence_after_sync();
            issue_qk(0, nk_next, (i + 1) & 1);
            tc_commit(&kv_empty[nk_next % kSlots]);
          }
          wait_full(nv);
          if (!ok) break;
          if (!mbar_wait(&p_full[0], i & 1)) {
            report_timeout(a.status, 104);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          issue_pv(0, nv, i == 0, i & 1);
          tc_commit(&kv_empty[nv % kSlots]);
        }
      } else {
      if (ok) {
        wait_full(0);
        if (ok) {
          tc_fence_after_sync();
          if (in_range(0, jlo)) issue_qk(0, 0, 0);
          if (in_range(1, jlo)) issue_qk(1, 0, 1);
          tc_commit(&kv_empty[0 % kSlots]);
        }
      }
      for (int j = jlo; j < jhi && ok; ++j) {
        const int nk = 2 * (j - jlo), nv = nk + 1, nk_next = nk + 2;
        const bool have_next = j + 1 < jhi;
        PROF_MARK(2);
        wait_full(nv);
        if (!ok) break;
        if (have_next) {
          wait_full(nk_next);
          if (!ok) break;
        }
        tc_fence_after_sync();
        PROF_MARK(0);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (in_range(t, j)) {
            PROF_MARK(2);
            if (!mbar_wait(&p_full[t], (j - lo[t]) & 1)) {
              report_timeout(a.status, 104);
              ok = false;
              break;
            }
            PROF_MARK(1);
            tc_fence_after_sync();
            issue_pv(t, nv, j == lo[t], t);
          }
          if (t == 1) tc_commit(&kv_empty[nv % kSlots]);
          if (have_next && in_range(t, j + 1)) issue_qk(t, nk_next, t);
          if (t == 1 && have_next) tc_commit(&kv_empty[nk_next % kSlots]);
        }
      }
      }
      PROF_MARK(2);
      PROF_FLUSH(2, true);
    }
   }
  } else {
    // ------------------------------------------------------------------ softmax groups
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int t = warp / 4, w4 = warp % 4;
    const int r_tile = w4 * 32 + lane;
    const int row = row_base + t * 128 + r_tile;
    const int r0 = row_base + t * 128;
    const uint32_t lane_addr = static_cast<uint32_t>(w4 * 32) << 16;
    const uint32_t tS_own = tmem_base + lane_addr + t * 128;
    const uint32_t tO = tmem_base + lane_addr + 256 + t * D;
    const int off = Sk - Sq;

    // scalars instead of runtime-indexed arrays (those would live in local memory)
    const bool active_t = t ? active[1] : active[0];
    const int lo_t = t ? lo[1] : lo[0];
    const int n_tiles = (t ? hi[1] : hi[0]) - lo_t;

    if (active_t) {
      float m_used = kNegInf, l = 0.f;
      bool ok = true;
      PROF_DECL;
      for (int it = 0; it < n_tiles; ++it) {
        const int j = lo_t + it;
        PROF_MARK(7);
        // wide head dims: the S tile alternates between the two 128-column buffers with the key tile
        const uint32_t tS = kWide ? tmem_base + lane_addr + (it & 1) * 128 : tS_own;
        bool w_ok = kWide ? mbar_wait(&s_full[it & 1], (it >> 1) & 1) : mbar_wait(&s_full[t], it & 1);
        if (w_ok && it > 0) w_ok = mbar_wait(&o_ready[t], (it - 1) & 1);
        if (!__all_sync(kFull, w_ok)) {
          report_timeout(a.status, 105);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        PROF_MARK(0);

        const int k0 = j * 128;
        const bool tile_masked = (k0 + 128 > Sk) || (a.causal && (k0 + 127 > r0 + off)) ||
                                 (a.wl >= 0 && (k0 < r0 + 127 + off - a.wl)) ||
                                 (!a.causal && a.wr >= 0 && (k0 + 127 > r0 + off + a.wr));
        // Every mask (key bound, causal, window) keeps one interval [c_lo, c_hi] of this row's 128 columns.
        int c_lo = 0, c_hi = 127;
        if (tile_masked) {
          c_hi = min(c_hi, Sk - 1 - k0);
          if (a.causal) c_hi = min(c_hi, row + off - k0);
          else if (a.wr >= 0) c_hi = min(c_hi, row + off + a.wr - k0);
          if (a.wl >= 0) c_lo = max(0, row + off - a.wl - k0);
        }

        if (kMods) {
          // General path (softcap, bias, ALiBi, dropout): 32 columns at a time in rolled loops, so the code stays
          // small; the transformed logits go back to TMEM in place between the maximum and the exponentials.
          float m_tile = kNegInf;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld32(tS + c * 32, r);
            tc_wait_ld_regs(r);
            float(&x)[32] = *reinterpret_cast<float(*)[32]>(&r[0]);
            mods_logits32<true>(mods, x, row, k0 + c * 32, nullptr);
            if (tile_masked) {
#pragma unroll
              for (int e = 0; e < 32; ++e)
                if (c * 32 + e < c_lo || c * 32 + e > c_hi) x[e] = kNegInf;
            }
#pragma unroll
            for (int e = 0; e < 32; e += 2) m_tile = fmax3(m_tile, x[e], x[e + 1]);
            tmem_st32(tS + c * 32, r);
          }
          tc_wait_st();
          PROF_MARK(2);
          const float m_new = fmaxf(m_used, m_tile);
          const bool grow = m_new > m_used + kRescaleThreshold;
          if (__any_sync(kFull, grow)) {
            const float alpha = (m_new == kNegInf) ? 1.f : exp2f(m_used - m_new);
            l *= alpha;
            if (it > 0) rescale_o<D>(tO, alpha);
            m_used = m_new;
          }
          const float m_eff = (m_used == kNegInf) ? 0.f : m_used;
          PROF_MARK(3);
          float sum = 0.f;
          const float inv_keep = mods.inv_keep;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32], pk[16];
            tmem_ld32(tS + c * 32, r);
            const uint32_t kept = mods_dropout_bits32<true>(mods, row, k0 + c * 32);
            tc_wait_ld_regs(r);
            float(&x)[32] = *reinterpret_cast<float(*)[32]>(&r[0]);
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              x[e] = fast_exp2(x[e] - m_eff);
              sum += x[e];
            }
            if (mods.dropout_p > 0.f) {  // the row sum above is of the undropped probabilities
#pragma unroll
              for (int e = 0; e < 32; ++e) x[e] = ((kept >> e) & 1u) ? x[e] * inv_keep : 0.f;
            }
#pragma unroll
            for (int e = 0; e < 16; ++e) pk[e] = DType<T>::pack2(x[2 * e], x[2 * e + 1]);
            // the 16-bit chunk lands on columns [16c, 16c+16): all of them already read
            tmem_st16(tS + c * 16, pk);
          }
          l += sum;
        } else {
          // Fast path: the whole S row (128 fp32 values) is read from TMEM once and stays in registers between
          // the maximum and the exponentials.
          uint32_t r[128];
#pragma unroll
          for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
          float mx[4] = {kNegInf, kNegInf, kNegInf, kNegInf};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            // wait::ld covers every load issued so far; naming the chunk pins its uses behind the wait
            if (c == 0) tc_wait_ld_regs(*reinterpret_cast<uint32_t(*)[32]>(&r[0]));
            else asm volatile("" : "+r"(r[c * 32]), "+r"(r[c * 32 + 31]));
            if (tile_masked) {
#pragma unroll
              for (int e = 0; e < 32; ++e)
                if (c * 32 + e < c_lo || c * 32 + e > c_hi) r[c * 32 + e] = __float_as_uint(kNegInf);
            }
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
#pragma unroll
              for (int u = 0; u < 4; ++u)
                mx[u] = fmax3(mx[u], __uint_as_float(r[c * 32 + e + 2 * u]), __uint_as_float(r[c * 32 + e + 2 * u + 1]));
            }
          }
          const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * mods.scale_log2;  // scale > 0 here
          PROF_MARK(2);
          const float m_new = fmaxf(m_used, m_tile);
          const bool grow = m_new > m_used + kRescaleThreshold;
          if (__any_sync(kFull, grow)) {
            const float alpha = (m_new == kNegInf) ? 1.f : exp2f(m_used - m_new);
            l *= alpha;
            if (it > 0) rescale_o<D>(tO, alpha);
            m_used = m_new;
          }
          const float m_eff = (m_used == kNegInf) ? 0.f : m_used;
          PROF_MARK(3);

          // p = exp2(s*scale - m) with packed fp32x2 FMA/ADD, 32 columns at a time; the 16-bit P chunk goes to
          // columns [16c, 16c+16) of the S tile.
          const uint64_t sc2 = pack_f32x2(mods.scale_log2, mods.scale_log2);
          const uint64_t nm2 = pack_f32x2(-m_eff, -m_eff);
          uint64_t acc2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const uint64_t x2 = fma_f32x2(pack_u32x2(r[c * 32 + 2 * e], r[c * 32 + 2 * e + 1]), sc2, nm2);
              float x0, x1;
              unpack_f32x2(x2, &x0, &x1);
              const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
              acc2[e & 3] = add_f32x2(acc2[e & 3], pack_f32x2(p0, p1));
              pk[e] = DType<T>::pack2(p0, p1);
            }
            tmem_st16(tS + c * 16, pk);
          }
          float s0, s1;
          unpack_f32x2(add_f32x2(add_f32x2(acc2[0], acc2[1]), add_f32x2(acc2[2], acc2[3])), &s0, &s1);
          l += s0 + s1;
        }
        PROF_MARK(4);
        tc_wait_st();
        tc_fence_before_sync();
        mbar_arrive(&p_full[t]);
        PROF_MARK(5);
      }

      // epilogue: O / l -> global, LSE
      T* orow = reinterpret_cast<T*>(a.out) + (a.varlen ? 0 : (int64_t)b * a.o_sb) + (int64_t)h * a.o_sh +
                (int64_t)(q_start + row) * a.o_ss;
      if (n_tiles > 0) {
        bool w_ok = ok && mbar_wait(&o_ready[t], (n_tiles - 1) & 1);
        if (!__all_sync(kFull, w_ok)) {
          if (ok) report_timeout(a.status, 106);
          ok = false;
        }
      }
      if (ok) {
        tc_fence_after_sync();
        const float l_safe = (l == 0.f) ? 1.f : l;
        const float inv = 1.f / l_safe;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          if (n_tiles > 0) {
            tmem_ld32(tO + c * 32, o);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = 0u;
          }
          if (row < Sq) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 pkt;
              pkt.x = DType<T>::pack2(__uint_as_float(o[v * 8 + 0]) * inv, __uint_as_float(o[v * 8 + 1]) * inv);
              pkt.y = DType<T>::pack2(__uint_as_float(o[v * 8 + 2]) * inv, __uint_as_float(o[v * 8 + 3]) * inv);
              pkt.z = DType<T>::pack2(__uint_as_float(o[v * 8 + 4]) * inv, __uint_as_float(o[v * 8 + 5]) * inv);
              pkt.w = DType<T>::pack2(__uint_as_float(o[v * 8 + 6]) * inv, __uint_as_float(o[v * 8 + 7]) * inv);
              if (c * 32 + v * 8 < a.head_dim) *reinterpret_cast<uint4*>(orow + c * 32 + v * 8) = pkt;
            }
          }
        }
        if (row < Sq) {
          float* lrow = a.lse + (a.varlen ? 0 : (int64_t)b * a.l_sb) + (int64_t)h * a.l_sh +
                        (int64_t)(q_start + row) * a.l_ss;
          *lrow = (l == 0.f) ? kNegInf : (m_used * kLn2 + logf(l));
        }
      }
      PROF_MARK(6);
      PROF_FLUSH(t, lane == 0 && w4 == 0);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem_base, 512);
}

template <typename T, int D, bool kMods>
int launch_typed(const fa_attn_params& p, const FwdArgs& a, cudaStream_t stream) {
  constexpr int kChunks = D / 64;
  constexpr int kTileBytes = kChunks * 16384;
  constexpr int kQTiles = D > 128 ? 1 : 2;
  constexpr int kSlots = D > 128 ? 2 : (D == 128) ? 4 : 6;
  const int smem = (kQTiles + kSlots) * kTileBytes + 1024;
  CUtensorMap mq, mk, mv;
  const int rows_q = p.varlen ? p.total_q : p.seqlen_q;
  const int rows_k = p.varlen ? p.total_k : p.seqlen_k;
  const int nb = p.varlen ? 1 : p.batch;
  int rc = make_tile_map(&mq, p.q, p.dtype, p.head_dim, rows_q, p.heads_q, nb, p.q_strides[2], p.q_strides[1], p.q_strides[0]);
  if (rc) return rc;
  rc = make_tile_map(&mk, p.k, p.dtype, p.head_dim, rows_k, p.heads_kv, nb, p.k_strides[2], p.k_strides[1], p.k_strides[0]);
  if (rc) return rc;
  rc = make_tile_map(&mv, p.v, p.dtype, p.head_dim, rows_k, p.heads_kv, nb, p.v_strides[2], p.v_strides[1], p.v_strides[0]);
  if (rc) return rc;
  auto kern = fwd_kernel<T, D, kMods>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "forward smem opt-in failed: %s", cudaGetErrorString(e));
  dim3 grid(p.batch * p.heads_q, a.num_pairs);
  if (a.compact) grid = dim3(p.heads_q, (p.total_q + kQTiles * 128 - 1) / (kQTiles * 128) + p.batch);
  kern<<<grid, kFwdThreads, smem, stream>>>(mq, mk, mv, a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "forward launch failed: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace

PROF_DEFINE_READER(fa_debug_read_prof)

bool fwd_tcgen05_supported(const fa_attn_params& p) {
  if (p.dtype != FA_F16 && p.dtype != FA_BF16) return false;
  if (p.head_dim < 8 || p.head_dim > 256 || p.head_dim % 8) return false;  // narrower rows are zero-filled by TMA
  const int64_t nb = p.varlen ? 1 : p.batch;
  const int64_t sq[3] = {nb, p.heads_q, p.varlen ? p.total_q : p.seqlen_q};
  const int64_t sk[3] = {nb, p.heads_kv, p.varlen ? p.total_k : p.seqlen_k};
  if (!tma_operand_ok(p.q, p.q_strides, sq) || !tma_operand_ok(p.k, p.k_strides, sk) ||
      !tma_operand_ok(p.v, p.v_strides, sk))
    return false;
  if (!tma_operand_ok(p.out, p.o_strides, sq)) return false;  // 16-byte vector stores need the same alignment
  return true;
}

int launch_fwd_tcgen05(const fa_attn_params& p, cudaStream_t stream) {
  FwdArgs a;
  a.varlen = p.varlen;
  a.heads_q = p.heads_q;
  a.head_dim = p.head_dim;
  a.heads_kv = p.heads_kv;
  a.seqlen_q = p.seqlen_q;
  a.seqlen_k = p.seqlen_k;
  a.total_q = p.total_q;
  a.total_k = p.total_k;
  a.cu_q = p.cu_seqlens_q;
  a.cu_k = p.cu_seqlens_k;
  a.out = p.out;
  a.o_sb = p.o_strides[0];
  a.o_sh = p.o_strides[1];
  a.o_ss = p.o_strides[2];
  a.lse = p.lse;
  a.l_sb = p.lse_strides[0];
  a.l_sh = p.lse_strides[1];
  a.l_ss = p.lse_strides[2];
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
  a.num_pairs = p.head_dim > 128 ? (p.seqlen_q + 127) / 128 : (p.seqlen_q + 255) / 256;  // CTAs along the queries
  a.status = p.status;
  a.batch = p.batch;
  a.compact = (p.varlen && p.batch <= kPackedMaxSequences) ? 1 : 0;
  const bool mods = p.softcap > 0.f || p.bias != nullptr || p.alibi_slopes != nullptr || p.dropout_p > 0.f ||
                    !(p.softmax_scale > 0.f);
  const bool f16 = p.dtype == FA_F16;
  if (p.head_dim > 128) {
    if (f16) return mods ? launch_typed<__half, 256, true>(p, a, stream) : launch_typed<__half, 256, false>(p, a, stream);
    return mods ? launch_typed<__nv_bfloat16, 256, true>(p, a, stream)
                : launch_typed<__nv_bfloat16, 256, false>(p, a, stream);
  }
  if (p.head_dim > 64) {
    if (f16) return mods ? launch_typed<__half, 128, true>(p, a, stream) : launch_typed<__half, 128, false>(p, a, stream);
    return mods ? launch_typed<__nv_bfloat16, 128, true>(p, a, stream)
                : launch_typed<__nv_bfloat16, 128, false>(p, a, stream);
  }
  if (f16) return mods ? launch_typed<__half, 64, true>(p, a, stream) : launch_typed<__half, 64, false>(p, a, stream);
  return mods ? launch_typed<__nv_bfloat16, 64, true>(p, a, stream)
              : launch_typed<__nv_bfloat16, 64, false>(p, a, stream);
}

}  // namespace fa
