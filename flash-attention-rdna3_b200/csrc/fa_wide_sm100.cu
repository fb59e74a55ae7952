// Attention on tcgen05 for the head dims the fused kernels have no room for, dense problems with a workspace:
// the backward above 128 (up to 256) and the forward above 256 (up to 512). Both are taken apart into plain products
// whose 128 x 128 16-bit tiles (P, dS) pass through a scratch buffer in the layout an MMA reads its operand in.
//
// Backward, head dims 129-256.
// dK and dV of a 128-key tile are 2 x 256 fp32 accumulator columns, all of tensor memory, so the fused form of
// fa_bwd_sm100.cu does not fit. Here the backward is taken apart into the products it consists of:
//
//   1. bwd_wide_scores_kernel   S = Q K^T, dP = dO V^T (contraction over the whole head dim), then
//                               P = exp2(S*c - lse), dS = P * (dP - delta); both 128 x 128 tiles go to the workspace as
//                               16-bit operands, already in the layout the tensor core reads them in.
//   2. bwd_wide_gemm_kernel     dV = P^T dO, dK = dS^T Q, dQ = dS K: three plain products over those tiles, one
//                               persistent launch whose work items are (product, output tile).
//
// Five tile products for five algorithmic ones (nothing is recomputed), fixed summation order, no atomics. The price
// is memory traffic: 64 KB written per tile pair and 96 KB read, which the B200's HBM and L2 take at about the rate
// the tensor pipe produces them.
//
// A tile in the workspace holds dS (or P) of 128 queries x 128 keys as 16 blocks of 8 keys; a block holds, query
// after query, the 16 bytes of that query's 8 values: a warp of the scores kernel (32 consecutive queries) writes 512
// contiguous bytes per store, and the tile is, byte for byte, the unswizzled core-matrix layout of an MMA operand:
// read along its 16-byte rows (contraction over keys) it is the A operand of dQ = dS K, read across them (contraction
// over queries) it is the A operand of dK = dS^T Q and dV = P^T dO.
// Tile index: ((batch * heads_q + head) * key_tiles + key tile) * query_tiles + query tile; the P tiles follow the dS
// tiles. Math as in fa_bwd_sm100.cu (fa_rdna3/kernels/_common.py:347-508, fa_rdna3/kernels/backward.py:56-322).
//
// Forward, head dims 257-512: the output accumulator of 128 rows alone is 512 columns, all of tensor memory, so there
// is no room for a score tile beside it. Three steps (fa_rdna3/kernels/forward.py:28-164 computes the same O and LSE
// in one kernel):
//   1. fwd_wide_kernel<stats>   S = Q K^T, online row maximum and sum -> LSE
//   2. fwd_wide_kernel<probs>   S = Q K^T again, P = exp2(S*c - row maximum) -> P tiles in the workspace (the largest
//                               entry of a row is exactly 1, as in the fused kernels)
//   3. bwd_wide_gemm_kernel     O = (P V) / row sum, the same product as dQ = dS K, once per half of the head dim
// Rows that see no key get LSE = -inf and O = 0.
#include "fa_bwd_shared.cuh"
#include "fa_tma_host.h"

namespace fa {
namespace {

constexpr int kWD = 256;              // compiled head dim; narrower rows load as zeros
constexpr int kTileWs = 32768;        // one 128 x 128 16-bit tile in the workspace
constexpr int kWideGemmThreads = 224;

// Key tiles [slo, slo + n) that the 128-query tile qt sees (dense problem). Every kernel of this file derives its
// loops from this one function, so the tiles that are read are exactly the tiles that were written.
__device__ __forceinline__ void key_tiles_of(const BwdArgs& a, int qt, int* slo, int* n) {
  const int q0 = qt * 128, off = a.seqlen_k - a.seqlen_q;
  const int r1 = min(q0 + 127, a.seqlen_q - 1);
  int khi = a.seqlen_k, klo = 0;
  if (a.causal) khi = min(khi, r1 + off + 1);
  else if (a.wr >= 0) khi = min(khi, r1 + off + a.wr + 1);
  if (a.wl >= 0) klo = max(0, q0 + off - a.wl);
  khi = max(khi, 0);
  const int lo = klo / 128, hi = (khi + 127) / 128;
  *slo = hi > lo ? lo : 0;
  *n = hi > lo ? hi - lo : 0;
}

// Query tiles [qlo, qlo + n) that see key tile kt: the inverse of key_tiles_of (the ranges move monotonically with
// the query tile, so the set is an interval).
__device__ __forceinline__ void query_tiles_of(const BwdArgs& a, int kt, int* qlo, int* n) {
  int lo = 0, hi = a.ds_qt - 1, s, c;
  for (; lo <= hi; ++lo) {
    key_tiles_of(a, lo, &s, &c);
    if (kt >= s && kt < s + c) break;
  }
  for (; hi >= lo; --hi) {
    key_tiles_of(a, hi, &s, &c);
    if (kt >= s && kt < s + c) break;
  }
  *qlo = lo;
  *n = hi >= lo ? hi - lo + 1 : 0;
}

__device__ __forceinline__ void compute_sync_256() {
  asm volatile("bar.sync 1, 256;" ::: "memory");  // the eight compute warps
}

__device__ __forceinline__ int64_t ws_tile(const BwdArgs& a, int b, int h, int kt, int qt) {
  return (((int64_t)b * a.heads_q + h) * a.ds_kt + kt) * a.ds_qt + qt;
}

// =============================================================================================
// 1. scores -> P and dS tiles
// =============================================================================================
// Persistent CTAs walk 128-query tiles of one (batch, head), longest first. Q and dO of the item (64 KB each) stay in
// shared memory; K and V stream in pieces of 64 columns (128 keys x 64 columns, 16 KB) through a ring of six slots,
// the pieces of K first, then those of V, each released by the commit of the four MMAs that read it. S and dP are both double
// buffered in tensor memory (4 x 128 columns), and a buffer goes back to the MMA thread as soon as the compute warps
// hold it in registers, so the products of step g + 1 run under the elementwise work of step g.
//   warps 0-7   compute: thread = one query row; group wg = warp / 4 owns key columns [64 wg, 64 wg + 64) of a step
//   warp  8     TMA producer (one lane)          warp 9     MMA issuer (one lane)
template <int D>
struct WideSmem {
  static constexpr int kTileBytes = (D / 64) * 16384;  // Q or dO of the item
  static constexpr int kOffQ = 0;
  static constexpr int kOffDo = kTileBytes;
  static constexpr int kOffRing = 2 * kTileBytes;
  static constexpr int kChunks = D / 64;               // 64-column pieces: the unit of the ring
  static constexpr int kSlotBytes = 16384;
  static constexpr int kSlots = (232448 - 2048 - 2 * kTileBytes) / kSlotBytes > 8 ? 8 : (232448 - 2048 - 2 * kTileBytes) / kSlotBytes;
  static constexpr int kOffBars = kOffRing + kSlots * kSlotBytes;
  static constexpr int kNumBars = 10 + 2 * kSlots;
  static constexpr int kOffTmemPtr = kOffBars + kNumBars * 8;
  static constexpr int kBytes = kOffTmemPtr + 8 + 1024;  // + slack to round the base up to 1024
  static_assert(kBytes <= 232448, "shared memory plan exceeds one CTA's 227 KB");
};

struct ScoreItem {
  int b, h, hk, qt, slo, n;
};

__device__ __forceinline__ ScoreItem score_item(const BwdArgs& a, int w) {
  ScoreItem it;
  const int bh_count = a.batch * a.heads_q;
  it.qt = a.ds_qt - 1 - w / bh_count;  // longest (causal) rows first
  const int bh = w % bh_count;
  it.b = bh / a.heads_q;
  it.h = bh % a.heads_q;
  it.hk = it.h / (a.heads_q / a.heads_kv);
  key_tiles_of(a, it.qt, &it.slo, &it.n);
  return it;
}

template <typename T, int D, bool kMods>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_wide_scores_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                       const BwdArgs a) {
  using L = WideSmem<D>;
  constexpr int kSlots = L::kSlots, kChunks = L::kChunks;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::kOffQ;
  uint8_t* sDo = smem + L::kOffDo;
  uint8_t* sRing = smem + L::kOffRing;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBars);
  uint64_t* qdo_full = bars + 0;
  uint64_t* qdo_empty = bars + 1;
  uint64_t* s_full = bars + 2;    // [2]
  uint64_t* s_free = bars + 4;    // [2]
  uint64_t* dp_full = bars + 6;   // [2]
  uint64_t* dp_free = bars + 8;   // [2]
  uint64_t* ring_full = bars + 10;
  uint64_t* ring_empty = ring_full + kSlots;
  uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(smem + L::kOffTmemPtr);

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int n_items = a.ds_qt * a.batch * a.heads_q;

  // The product kernel launched behind this one may set itself up while the last CTAs here drain (it waits inside).
  grid_launch_dependents();
  if (tid == 0) {
    mbar_init(qdo_full, 1);
    mbar_init(qdo_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 256);
      mbar_init(&dp_full[i], 1);
      mbar_init(&dp_free[i], 256);
    }
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(&ring_full[i], 1);
      mbar_init(&ring_empty[i], 1);
    }
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_s;
  constexpr uint32_t kColS = 0, kColDP = 256;

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      int r = 0;     // ring entries issued so far
      int used = 0;  // items that used the pipeline so far
      bool ok = true;
      for (int round = 0; ok; ++round) {
        const int w = snake_item(round, blockIdx.x, gridDim.x);
        if (w >= n_items) break;
        const ScoreItem it = score_item(a, w);
        if (it.n == 0) continue;
        for (int n = 0; n < it.n && ok; ++n) {
          const int row = (it.slo + n) * 128;
#pragma unroll 1
          for (int j = 0; j < 2 * kChunks && ok; ++j, ++r) {  // the pieces of K, then those of V
            const int st = r % kSlots;
            if (!mbar_wait(&ring_empty[st], ((r / kSlots) & 1) ^ 1)) {
              report_timeout(a.status, 601);
              ok = false;
              break;
            }
            uint8_t* dst = sRing + st * L::kSlotBytes;
            mbar_arrive_expect_tx(&ring_full[st], L::kSlotBytes);
            tma_load_4d(dst, j < kChunks ? &map_k : &map_v, &ring_full[st], (j % kChunks) * 64, row, it.hk, it.b);
            if (n == 0 && j == 0) {
              // Q and dO of the item behind its first half tile: the MMAs of the previous item that read the old
              // ones need nothing further from this thread, so this wait cannot block the ring
              if (!mbar_wait(qdo_empty, (used & 1) ^ 1)) {
                report_timeout(a.status, 600);
                ok = false;
                break;
              }
              mbar_arrive_expect_tx(qdo_full, 2 * L::kTileBytes);
#pragma unroll
              for (int c = 0; c < D / 64; ++c) tma_load_4d(sQ + c * 16384, &map_q, qdo_full, c * 64, it.qt * 128, it.h, it.b);
#pragma unroll
              for (int c = 0; c < D / 64; ++c) tma_load_4d(sDo + c * 16384, &map_do, qdo_full, c * 64, it.qt * 128, it.h, it.b);
            }
          }
        }
        ++used;
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(DType<T>::kFormat, 128, 128, 0, 0);
      constexpr uint32_t hi = smem_desc_hi(1024);
      const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sDo), ring_addr = smem_u32(sRing);
      int g = 0, r = 0, used = 0;
      bool ok = true;
      auto wait_or_report = [&](uint64_t* bar, int parity, int code) {
        if (!ok) return;
        if (!mbar_wait(bar, parity)) {
          report_timeout(a.status, code);
          ok = false;
        }
      };
      // [128 queries x 128 keys] (+)= A[:, piece] B[:, piece]^T: 64 columns of the head dim, four MMAs
      auto piece_product = [&](uint32_t col, uint32_t a_addr, bool first) {
        const int st = r % kSlots;
        wait_or_report(&ring_full[st], (r / kSlots) & 1, 603);
        if (!ok) return;
        tc_fence_after_sync();
        const uint32_t a_lo = smem_desc_lo(a_addr, 16), b_lo = smem_desc_lo(ring_addr + st * L::kSlotBytes, 16);
        if (first) mma_ss_lo<0>(tmem_base + col, a_lo, hi, b_lo, hi, idesc);
        else mma_ss_lo<1>(tmem_base + col, a_lo, hi, b_lo, hi, idesc);
#pragma unroll
        for (int kk = 1; kk < 4; ++kk) mma_ss_lo<1>(tmem_base + col, a_lo + kk * 2, hi, b_lo + kk * 2, hi, idesc);
        tc_commit(&ring_empty[st]);
        ++r;
      };
      for (int round = 0; ok; ++round) {
        const int w = snake_item(round, blockIdx.x, gridDim.x);
        if (w >= n_items) break;
        const ScoreItem it = score_item(a, w);
        if (it.n == 0) continue;
        wait_or_report(qdo_full, used & 1, 602);
        for (int n = 0; n < it.n && ok; ++n, ++g) {
          const int buf = g & 1;
          wait_or_report(&s_free[buf], ((g >> 1) & 1) ^ 1, 604);  // the compute warps hold the old S in registers
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < kChunks; ++c) piece_product(kColS + buf * 128, q_addr + c * 16384, c == 0);
          if (!ok) break;
          tc_commit(&s_full[buf]);
          wait_or_report(&dp_free[buf], ((g >> 1) & 1) ^ 1, 605);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < kChunks; ++c) piece_product(kColDP + buf * 128, do_addr + c * 16384, c == 0);
          if (!ok) break;
          tc_commit(&dp_full[buf]);
        }
        if (ok) tc_commit(qdo_empty);  // every MMA that reads this item's Q / dO is issued
        ++used;
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warps
    const int wg = warp / 4, w4 = warp % 4;
    const int q_row = w4 * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(w4 * 32) << 16;
    uint8_t* ws_ds = reinterpret_cast<uint8_t*>(a.ds_ws);
    uint8_t* ws_p = ws_ds + (int64_t)a.batch * a.heads_q * a.ds_kt * a.ds_qt * kTileWs;
    const int thread_off = wg * 8 * 2048 + q_row * 16;  // this thread's 16 bytes in the first block of its columns
    int g = 0;
    bool ok = true;
    for (int round = 0; ok; ++round) {
      const int w = snake_item(round, blockIdx.x, gridDim.x);
      if (w >= n_items) break;
      const ScoreItem it = score_item(a, w);
      if (it.n == 0) continue;
      const int q0 = it.qt * 128, i = q0 + q_row;
      const ScoreMods mods = make_mods(a, it.b, it.h, a.seqlen_q, a.seqlen_k);
      const int off = a.seqlen_k - a.seqlen_q;
      float nlse2 = kNegInf, ndelta = 0.f;  // -lse*log2(e) (-inf = the row contributes nothing) and -delta
      if (i < a.seqlen_q) {
        const float l = a.lse[(int64_t)it.b * a.l_sb + (int64_t)it.h * a.l_sh + (int64_t)i * a.l_ss];
        nlse2 = (l == kNegInf) ? kNegInf : -l * kLog2e;
        ndelta = -a.delta[(int64_t)it.b * a.d_sb + (int64_t)it.h * a.d_sh + (int64_t)i * a.d_ss];
      }
      const uint64_t sc2 = pack_f32x2(mods.scale_log2, mods.scale_log2);
      const uint64_t nl2 = pack_f32x2(nlse2, nlse2), nd2 = pack_f32x2(ndelta, ndelta);

      for (int n = 0; n < it.n; ++n, ++g) {
        const int buf = g & 1, kt = it.slo + n, ks = kt * 128;
        const uint32_t tS = tmem_base + lane_addr + kColS + buf * 128 + wg * 64;
        const uint32_t tDP = tmem_base + lane_addr + kColDP + buf * 128 + wg * 64;
        const int64_t tile = ws_tile(a, it.b, it.h, kt, it.qt) * kTileWs + thread_off;
        uint8_t* p_dst = ws_p + tile;
        uint8_t* ds_dst = ws_ds + tile;
        // keys this query row keeps: one interval [c_lo, c_hi] of the step's 128 columns
        const bool masked = block_needs_mask(mods, q0, 128, ks, 128);
        int c_lo = 0, c_hi = 127;
        if (masked) {
          c_hi = min(c_hi, a.seqlen_k - 1 - ks);
          if (a.causal) c_hi = min(c_hi, i + off - ks);
          else if (a.wr >= 0) c_hi = min(c_hi, i + off + a.wr - ks);
          if (a.wl >= 0) c_lo = max(0, i + off - a.wl - ks);
        }
        if (!__all_sync(kFull, mbar_wait(&s_full[buf], (g >> 1) & 1))) {
          report_timeout(a.status, 606);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (!kMods) {
          // ---- P = exp2(S * c - lse[row]); the S buffer goes back as soon as it is in registers
          uint32_t p0[32], p1[32], pk[16];
          tmem_ld32(tS, p0);
          tmem_ld32(tS + 32, p1);
          tc_wait_ld_regs(p0);
          tc_wait_ld_regs(p1);
          tc_fence_before_sync();
          mbar_arrive(&s_free[buf]);
          if (masked) {
            probs_inplace<true>(p0, sc2, nl2, wg * 64, c_lo, c_hi);
            probs_inplace<true>(p1, sc2, nl2, wg * 64 + 32, c_lo, c_hi);
          } else {
            probs_inplace<false>(p0, sc2, nl2, wg * 64, c_lo, c_hi);
            probs_inplace<false>(p1, sc2, nl2, wg * 64 + 32, c_lo, c_hi);
          }
#pragma unroll
          for (int e = 0; e < 16; ++e) pk[e] = DType<T>::pack2(__uint_as_float(p0[2 * e]), __uint_as_float(p0[2 * e + 1]));
          store_ds32(p_dst, pk);
#pragma unroll
          for (int e = 0; e < 16; ++e) pk[e] = DType<T>::pack2(__uint_as_float(p1[2 * e]), __uint_as_float(p1[2 * e + 1]));
          store_ds32(p_dst + 4 * 2048, pk);

          // ---- dS = P * (dP - delta[row])
          if (!__all_sync(kFull, mbar_wait(&dp_full[buf], (g >> 1) & 1))) {
            report_timeout(a.status, 607);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          uint32_t d0[32], d1[32];
          tmem_ld32(tDP, d0);
          tmem_ld32(tDP + 32, d1);
          tc_wait_ld_regs(d0);
          tc_wait_ld_regs(d1);
          tc_fence_before_sync();
          mbar_arrive(&dp_free[buf]);
          dscore_row<T>(p0, d0, nd2, pk);
          store_ds32(ds_dst, pk);
          dscore_row<T>(p1, d1, nd2, pk);
          store_ds32(ds_dst + 4 * 2048, pk);
        } else {
          // ---- general path (softcap / bias / ALiBi / dropout), 32 columns per (rolled) pass
          if (!__all_sync(kFull, mbar_wait(&dp_full[buf], (g >> 1) & 1))) {
            report_timeout(a.status, 607);
            ok = false;
            break;
          }
          tc_fence_after_sync();
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t sv[32], dp[32], pk[16];
            tmem_ld32(tS + c * 32, sv);
            tmem_ld32(tDP + c * 32, dp);
            tc_wait_ld_regs(sv);
            tc_wait_ld_regs(dp);
            if (c == 1) {
              tc_fence_before_sync();
              mbar_arrive(&s_free[buf]);
              mbar_arrive(&dp_free[buf]);
            }
            const int col0 = wg * 64 + c * 32;
            float(&x)[32] = *reinterpret_cast<float(*)[32]>(&sv[0]);
            float(&gr)[32] = *reinterpret_cast<float(*)[32]>(&dp[0]);
            bwd_mods_chunk32<true>(mods, x, gr, &nlse2, &ndelta, i, ks + col0, c_lo - col0, c_hi - col0);
#pragma unroll
            for (int e = 0; e < 16; ++e) pk[e] = DType<T>::pack2(x[2 * e], x[2 * e + 1]);
            store_ds32(p_dst + c * 4 * 2048, pk);
#pragma unroll
            for (int e = 0; e < 16; ++e) pk[e] = DType<T>::pack2(gr[2 * e], gr[2 * e + 1]);
            store_ds32(ds_dst + c * 4 * 2048, pk);
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem_base, 512);
}

// =============================================================================================
// forward for head dims above 256: row statistics, then normalised P tiles
// =============================================================================================
// The same persistent structure as the scores kernel above with one product per step: Q of the item resident
// (8 pieces of 64 columns, 128 KB), K streamed piece by piece through a ring of six 16 KB slots, S double-buffered in
// tensor memory. Statistics mode: every thread keeps the running maximum and sum of its 64 columns of every step; the
// two column halves of a row are joined through shared memory at the end of the item; LSE and the pair (row maximum,
// 1 / row sum) are written. Probabilities mode: P = exp2(S * c - row maximum) goes to the workspace as a 16-bit tile
// (the layout of the dS tiles above); the product's epilogue divides by the row sum in fp32.
// The backward of these widths runs the same kernel twice more (Q and dO, 128 KB each, cannot both be resident as in
// the scores kernel above): once over (Q, K) for P = exp2(S * c - lse), once over (dO, V), where the accumulator is dP
// and the compute warps read their P back from its tile to form dS = P * (dP - delta); then the three products, one
// launch per 256 columns of the head dim.
struct FwdWideSmem {
  static constexpr int kD = 512;
  static constexpr int kTileBytes = (kD / 64) * 16384;
  static constexpr int kOffRing = kTileBytes;
  static constexpr int kSlotBytes = 16384;
  static constexpr int kSlots = 6;
  static constexpr int kOffStats = kOffRing + kSlots * kSlotBytes;  // [128 rows] (max, sum) of compute group 1
  static constexpr int kOffBars = kOffStats + 128 * 8;
  static constexpr int kNumBars = 6 + 2 * kSlots;
  static constexpr int kOffTmemPtr = kOffBars + kNumBars * 8;
  static constexpr int kBytes = kOffTmemPtr + 8 + 1024;
  static_assert(kBytes <= 232448, "shared memory plan exceeds one CTA's 227 KB");
};

enum WideMode {
  kModeStats = 0,     // forward: row maximum and sum -> LSE and (maximum, 1 / sum)
  kModeProbsMax = 1,  // forward: P = exp2(S * c - row maximum) -> tiles in the first region of the workspace
  kModeProbsLse = 2,  // backward: P = exp2(S * c - lse) -> tiles in the second region
  kModeDScores = 3    // backward, with dO and V in the places of Q and K: dS = P * (dP - delta) -> tiles in the first region
};

// TIn = float: Q and K are fp32 tiles (a piece is 32 columns, the same 128 bytes per row) and the product is a tf32 MMA;
// T is then the 16-bit type of the P tiles.
template <typename T, int kMode, typename TIn = T>
__global__ void __launch_bounds__(kBwdThreads, 1)
fwd_wide_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const BwdArgs a) {
  using L = FwdWideSmem;
  constexpr int kSlots = L::kSlots, kChunks = L::kD / 64;
  constexpr int kPieceCols = 128 / (int)sizeof(TIn);  // columns of a 128-byte piece
  constexpr bool kTf32 = sizeof(TIn) == 4;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sRing = smem + L::kOffRing;
  float2* stats_s = reinterpret_cast<float2*>(smem + L::kOffStats);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBars);
  uint64_t* q_full = bars + 0;
  uint64_t* q_empty = bars + 1;
  uint64_t* s_full = bars + 2;  // [2]
  uint64_t* s_free = bars + 4;  // [2]
  uint64_t* ring_full = bars + 6;
  uint64_t* ring_empty = ring_full + kSlots;
  uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(smem + L::kOffTmemPtr);

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int n_items = a.ds_qt * a.batch * a.heads_q;

  grid_launch_dependents();  // the kernel behind this one sets itself up early and waits inside
  if (tid == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 256);
    }
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(&ring_full[i], 1);
      mbar_init(&ring_empty[i], 1);
    }
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_base_s, 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_s;
  // every mode but the first reads what the kernel launched before it wrote (statistics, delta, P tiles)
  if (kMode != kModeStats) grid_dependency_wait();

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&map_k);
      int r = 0, used = 0;
      bool ok = true;
      for (int round = 0; ok; ++round) {
        const int w = snake_item(round, blockIdx.x, gridDim.x);
        if (w >= n_items) break;
        const ScoreItem it = score_item(a, w);
        if (it.n == 0) continue;
        for (int n = 0; n < it.n && ok; ++n) {
          const int row = (it.slo + n) * 128;
#pragma unroll 1
          for (int j = 0; j < kChunks && ok; ++j, ++r) {
            const int st = r % kSlots;
            if (!mbar_wait(&ring_empty[st], ((r / kSlots) & 1) ^ 1)) {
              report_timeout(a.status, 621);
              ok = false;
              break;
            }
            mbar_arrive_expect_tx(&ring_full[st], L::kSlotBytes);
            tma_load_4d(sRing + st * L::kSlotBytes, &map_k, &ring_full[st], j * kPieceCols, row, it.hk, it.b);
            if (n == 0 && j == 0) {  // Q of the item behind its first K piece (see the scores kernel)
              if (!mbar_wait(q_empty, (used & 1) ^ 1)) {
                report_timeout(a.status, 620);
                ok = false;
                break;
              }
              mbar_arrive_expect_tx(q_full, L::kTileBytes);
#pragma unroll
              for (int c = 0; c < kChunks; ++c) tma_load_4d(sQ + c * 16384, &map_q, q_full, c * kPieceCols, it.qt * 128, it.h, it.b);
            }
          }
        }
        ++used;
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(DType<TIn>::kFormat, 128, 128, 0, 0);
      constexpr uint32_t hi = smem_desc_hi(1024);
      const uint32_t q_addr = smem_u32(sQ), ring_addr = smem_u32(sRing);
      int g = 0, r = 0, used = 0;
      bool ok = true;
      for (int round = 0; ok; ++round) {
        const int w = snake_item(round, blockIdx.x, gridDim.x);
        if (w >= n_items) break;
        const ScoreItem it = score_item(a, w);
        if (it.n == 0) continue;
        if (!mbar_wait(q_full, used & 1)) {
          report_timeout(a.status, 622);
          break;
        }
        for (int n = 0; n < it.n && ok; ++n, ++g) {
          const int buf = g & 1;
          if (!mbar_wait(&s_free[buf], ((g >> 1) & 1) ^ 1)) {  // the compute warps hold the old S in registers
            report_timeout(a.status, 624);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          for (int c = 0; c < kChunks && ok; ++c, ++r) {
            const int st = r % kSlots;
            if (!mbar_wait(&ring_full[st], (r / kSlots) & 1)) {
              report_timeout(a.status, 623);
              ok = false;
              break;
            }
            tc_fence_after_sync();
            const uint32_t a_lo = smem_desc_lo(q_addr + c * 16384, 16), b_lo = smem_desc_lo(ring_addr + st * L::kSlotBytes, 16);
            if (kTf32) {  // 8 fp32 columns (32 bytes) per instruction
              if (c == 0) mma_ss_lo_tf32<0>(tmem_base + buf * 128, a_lo, hi, b_lo, hi, idesc);
              else mma_ss_lo_tf32<1>(tmem_base + buf * 128, a_lo, hi, b_lo, hi, idesc);
#pragma unroll
              for (int kk = 1; kk < 4; ++kk)
                mma_ss_lo_tf32<1>(tmem_base + buf * 128, a_lo + kk * 2, hi, b_lo + kk * 2, hi, idesc);
            } else {  // 16 sixteen-bit columns (32 bytes) per instruction
              if (c == 0) mma_ss_lo<0>(tmem_base + buf * 128, a_lo, hi, b_lo, hi, idesc);
              else mma_ss_lo<1>(tmem_base + buf * 128, a_lo, hi, b_lo, hi, idesc);
#pragma unroll
              for (int kk = 1; kk < 4; ++kk) mma_ss_lo<1>(tmem_base + buf * 128, a_lo + kk * 2, hi, b_lo + kk * 2, hi, idesc);
            }
            tc_commit(&ring_empty[st]);
          }
          if (ok) tc_commit(&s_full[buf]);
        }
        if (ok) tc_commit(q_empty);  // every MMA that reads this item's Q is issued
        ++used;
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warps
    const int wg = warp / 4, w4 = warp % 4;
    const int q_row = w4 * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(w4 * 32) << 16;
    constexpr bool kProbs = kMode == kModeProbsMax || kMode == kModeProbsLse;
    uint8_t* ws_first = reinterpret_cast<uint8_t*>(a.ds_ws);
    uint8_t* ws_second = ws_first + (int64_t)a.batch * a.heads_q * a.ds_kt * a.ds_qt * kTileWs;
    uint8_t* ws_p = kMode == kModeProbsMax ? ws_first : ws_second;
    const int thread_off = wg * 8 * 2048 + q_row * 16;
    const float scale_log2 = a.softmax_scale * kLog2e;
    int g = 0;
    bool ok = true;
    for (int round = 0; ok; ++round) {
      const int w = snake_item(round, blockIdx.x, gridDim.x);
      if (w >= n_items) break;
      const ScoreItem it = score_item(a, w);
      const int q0 = it.qt * 128, i = q0 + q_row;
      const int64_t lse_idx = (int64_t)it.b * a.l_sb + (int64_t)it.h * a.l_sh + (int64_t)i * a.l_ss;
      float2* stat = a.row_stats == nullptr ? nullptr : a.row_stats + ((int64_t)it.b * a.heads_q + it.h) * (a.ds_qt * 128) + i;
      if (it.n == 0) {  // rows that see no key
        if (kMode == kModeStats && wg == 0 && i < a.seqlen_q) a.lse_out[lse_idx] = kNegInf;
        continue;
      }
      const ScoreMods mods = make_mods(a, it.b, it.h, a.seqlen_q, a.seqlen_k);
      const int off = a.seqlen_k - a.seqlen_q;
      float nlse2 = kNegInf;  // minus the row maximum (or lse); -inf for rows that keep nothing (their P is 0)
      float ndelta = 0.f;
      if (kMode == kModeProbsMax && i < a.seqlen_q) {
        const float m = stat->x;
        nlse2 = (m == kNegInf) ? kNegInf : -m;
      }
      if (kMode == kModeProbsLse && i < a.seqlen_q) {
        const float l = a.lse[lse_idx];
        nlse2 = (l == kNegInf) ? kNegInf : -l * kLog2e;
      }
      if (kMode == kModeDScores && i < a.seqlen_q)
        ndelta = -a.delta[(int64_t)it.b * a.d_sb + (int64_t)it.h * a.d_sh + (int64_t)i * a.d_ss];
      const uint64_t sc2 = pack_f32x2(scale_log2, scale_log2), nl2 = pack_f32x2(nlse2, nlse2);
      float m_run = kNegInf, l_run = 0.f;  // statistics of this thread's columns, log2 domain

      for (int n = 0; n < it.n; ++n, ++g) {
        const int buf = g & 1, kt = it.slo + n, ks = kt * 128;
        const uint32_t tS = tmem_base + lane_addr + buf * 128 + wg * 64;
        const bool masked = block_needs_mask(mods, q0, 128, ks, 128);
        int c_lo = 0, c_hi = 127;
        if (masked) {
          c_hi = min(c_hi, a.seqlen_k - 1 - ks);
          if (a.causal) c_hi = min(c_hi, i + off - ks);
          else if (a.wr >= 0) c_hi = min(c_hi, i + off + a.wr - ks);
          if (a.wl >= 0) c_lo = max(0, i + off - a.wl - ks);
        }
        if (!__all_sync(kFull, mbar_wait(&s_full[buf], (g >> 1) & 1))) {
          report_timeout(a.status, 626);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        uint32_t p0[32], p1[32];
        tmem_ld32(tS, p0);
        tmem_ld32(tS + 32, p1);
        tc_wait_ld_regs(p0);
        tc_wait_ld_regs(p1);
        tc_fence_before_sync();
        mbar_arrive(&s_free[buf]);
        if (kProbs) {
          uint32_t pk[16];
          if (masked) {
            probs_inplace<true>(p0, sc2, nl2, wg * 64, c_lo, c_hi);
            probs_inplace<true>(p1, sc2, nl2, wg * 64 + 32, c_lo, c_hi);
          } else {
            probs_inplace<false>(p0, sc2, nl2, wg * 64, c_lo, c_hi);
            probs_inplace<false>(p1, sc2, nl2, wg * 64 + 32, c_lo, c_hi);
          }
          uint8_t* p_dst = ws_p + ws_tile(a, it.b, it.h, kt, it.qt) * kTileWs + thread_off;
#pragma unroll
          for (int e = 0; e < 16; ++e) pk[e] = DType<T>::pack2(__uint_as_float(p0[2 * e]), __uint_as_float(p0[2 * e + 1]));
          store_ds32(p_dst, pk);
#pragma unroll
          for (int e = 0; e < 16; ++e) pk[e] = DType<T>::pack2(__uint_as_float(p1[2 * e]), __uint_as_float(p1[2 * e + 1]));
          store_ds32(p_dst + 4 * 2048, pk);
        } else if (kMode == kModeDScores) {
          // the accumulator holds dP; P comes back from its tile (this thread's own 16-byte pieces, zero where masked)
          const int64_t tile = ws_tile(a, it.b, it.h, kt, it.qt) * kTileWs + thread_off;
          const uint8_t* p_src = ws_second + tile;
          uint8_t* ds_dst = ws_first + tile;
          const uint64_t nd2 = pack_f32x2(ndelta, ndelta);
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t (&dp)[32] = c == 0 ? p0 : p1;
            uint32_t pk[16], dsk[16];
#pragma unroll
            for (int b4 = 0; b4 < 4; ++b4) {
              const uint4 v = *reinterpret_cast<const uint4*>(p_src + (c * 4 + b4) * 2048);
              pk[4 * b4] = v.x;
              pk[4 * b4 + 1] = v.y;
              pk[4 * b4 + 2] = v.z;
              pk[4 * b4 + 3] = v.w;
            }
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const float2 pf = DType<T>::unpack2(pk[e]);
              float d0, d1;
              unpack_f32x2(mul_f32x2(pack_f32x2(pf.x, pf.y), add_f32x2(pack_u32x2(dp[2 * e], dp[2 * e + 1]), nd2)), &d0, &d1);
              dsk[e] = DType<T>::pack2(d0, d1);
            }
            store_ds32(ds_dst + c * 4 * 2048, dsk);
          }
        } else {
          // maximum of the kept columns, then the sum relative to the new running maximum
          float mt = kNegInf;
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int c0 = wg * 64 + e, c1 = c0 + 32;
            const float x0 = (!masked || (c0 >= c_lo && c0 <= c_hi)) ? __uint_as_float(p0[e]) : kNegInf;
            const float x1 = (!masked || (c1 >= c_lo && c1 <= c_hi)) ? __uint_as_float(p1[e]) : kNegInf;
            p0[e] = __float_as_uint(x0);
            p1[e] = __float_as_uint(x1);
            mt = fmaxf(mt, fmaxf(x0, x1));
          }
          mt *= scale_log2;  // softmax_scale > 0 on this path
          const float m_new = fmaxf(m_run, mt);
          if (m_new != kNegInf) {
            float sum = 0.f;
#pragma unroll
            for (int e = 0; e < 32; ++e)
              sum += fast_exp2(__uint_as_float(p0[e]) * scale_log2 - m_new) + fast_exp2(__uint_as_float(p1[e]) * scale_log2 - m_new);
            l_run = l_run * fast_exp2(m_run - m_new) + sum;
            m_run = m_new;
          }
        }
      }
      if (!ok) break;
      if (kMode == kModeStats) {
        // join the two column halves of every row: group 1 hands its pair over, group 0 writes LSE
        float2* slot = stats_s + q_row;
        if (wg == 1) *slot = make_float2(m_run, l_run);
        compute_sync_256();
        if (wg == 0) {
          const float2 other = *slot;
          const float M = fmaxf(m_run, other.x);
          float lse = kNegInf, inv = 0.f;
          if (M != kNegInf) {
            const float Lsum = l_run * fast_exp2(m_run - M) + other.y * fast_exp2(other.x - M);
            lse = (M + log2f(Lsum)) * kLn2;
            inv = 1.f / Lsum;
          }
          if (i < a.seqlen_q) a.lse_out[lse_idx] = lse;
          *stat = make_float2(M, inv);  // rows past the sequence end lie inside the padded array
        }
        compute_sync_256();  // the slots may be written again
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem_base, 256);
}

// =============================================================================================
// 2. the three products over the tiles
// =============================================================================================
// Persistent CTAs walk work items (product, output tile of 128 rows x head dim): first the dV tiles, then the dK
// tiles (both by key tile, longest first, all query heads of the kv head's group summed in the item), then the dQ
// tiles. Per step the producer brings one workspace tile (untiled bulk copy, 32 KB) and the matching 128 rows of dO, Q
// or K (TMA, 64 KB), each through a ring of its own (three tile slots, two operand slots: the tiles come from HBM and
// want more requests in flight than the operands, which come from L2); the MMA thread accumulates into one of two
// accumulators in tensor memory (2 x 256 columns), so that four epilogue warps write one output tile while the next
// one accumulates.
//   warps 0-3   epilogue (thread = one output row = one TMEM lane)
//   warp  4     tile producer (one lane)     warp 5     MMA issuer (one lane)     warp 6     operand producer (one lane)
enum WideRole { kRoleDV = 0, kRoleDK = 1, kRoleDQ = 2 };

template <int D>
struct GemmSmem {
  static constexpr int kOpBytes = (D / 64) * 16384;  // 128 rows of the streamed operand
  static constexpr int kOpSlots = 2;
  static constexpr int kTileSlots = (232448 - 2048 - kOpSlots * kOpBytes) / kTileWs > 5 ? 5 : (232448 - 2048 - kOpSlots * kOpBytes) / kTileWs;
  static constexpr int kOffOp = kTileSlots * kTileWs;
  static constexpr int kBytes = kOffOp + kOpSlots * kOpBytes + 1024;
};

struct GemmItem {
  int role, b, head, t;  // head: kv head (dV, dK) or query head (dQ); t: key tile (dV, dK) or query tile (dQ)
  int lo, per_head, n;   // first streamed tile, streamed tiles per query head, steps in all
};

// parts: FA_BWD_DKDV adds the dV and dK items, FA_BWD_DQ the dQ items
__device__ __forceinline__ int gemm_item_count(const BwdArgs& a, int parts) {
  return ((parts & FA_BWD_DKDV) ? 2 * a.ds_kt * a.batch * a.heads_kv : 0) +
         ((parts & FA_BWD_DQ) ? a.ds_qt * a.batch * a.heads_q : 0);
}

__device__ __forceinline__ GemmItem gemm_item(const BwdArgs& a, int parts, int w) {
  GemmItem it;
  const int nkv = (parts & FA_BWD_DKDV) ? a.ds_kt * a.batch * a.heads_kv : 0;
  if (w < 2 * nkv) {
    it.role = w < nkv ? kRoleDV : kRoleDK;
    const int idx = w < nkv ? w : w - nkv;
    const int bh_count = a.batch * a.heads_kv;
    it.t = idx / bh_count;  // causal: the first key tiles are seen by the most queries
    it.b = (idx % bh_count) / a.heads_kv;
    it.head = (idx % bh_count) % a.heads_kv;
    query_tiles_of(a, it.t, &it.lo, &it.per_head);
    it.n = it.per_head * (a.heads_q / a.heads_kv);
  } else {
    it.role = kRoleDQ;
    const int idx = w - 2 * nkv;
    const int bh_count = a.batch * a.heads_q;
    it.t = a.ds_qt - 1 - idx / bh_count;
    it.b = (idx % bh_count) / a.heads_q;
    it.head = (idx % bh_count) % a.heads_q;
    key_tiles_of(a, it.t, &it.lo, &it.per_head);
    it.n = it.per_head;
  }
  return it;
}

// Converts a 32-column fp32 slice of a TMEM accumulator to the output type and writes it to a global row.
template <typename TO>
__device__ __forceinline__ void store_out_slice(TO* dst, const uint32_t (&o)[32], float scale, int cols) {
  store_row_slice<TO>(dst, o, scale, cols);
}
template <>
__device__ __forceinline__ void store_out_slice<float>(float* dst, const uint32_t (&o)[32], float scale, int cols) {
#pragma unroll
  for (int v = 0; v < 8; ++v) {
    if (v * 4 >= cols) break;  // columns past the caller's head dimension do not exist
    *reinterpret_cast<float4*>(dst + v * 4) =
        make_float4(__uint_as_float(o[v * 4]) * scale, __uint_as_float(o[v * 4 + 1]) * scale,
                    __uint_as_float(o[v * 4 + 2]) * scale, __uint_as_float(o[v * 4 + 3]) * scale);
  }
}

// T: the 16-bit type of the tiles and of the streamed operand; TO: the type of the output rows.
template <typename T, int D, typename TO = T>
__global__ void __launch_bounds__(kWideGemmThreads, 1)
bwd_wide_gemm_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_do, const BwdArgs a, const int parts) {
  using L = GemmSmem<D>;
  constexpr int kTS = L::kTileSlots, kOS = L::kOpSlots;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t t_full[kTS], t_empty[kTS], o_full[kOS], o_empty[kOS], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int n_items = gemm_item_count(a, parts);
  constexpr uint32_t kCols = 2 * D;  // two accumulators

  if (tid == 0) {
    for (int i = 0; i < kTS; ++i) {
      mbar_init(&t_full[i], 1);
      mbar_init(&t_empty[i], 1);
    }
    for (int i = 0; i < kOS; ++i) {
      mbar_init(&o_full[i], 1);
      mbar_init(&o_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 128);
    }
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(&tmem_base_s, kCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  // Launched as a programmatic dependent of the scores kernel, whose tiles it reads: everything above overlaps that
  // kernel's tail, everything below waits for it to have completed.
  grid_dependency_wait();

  if (warp == 4 || warp == 6) {
    if (lane == 0) {
      const bool tiles = warp == 4;  // this thread's ring: workspace tiles or operand rows
      if (!tiles) {
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_do);
      }
      const uint8_t* ws_ds = reinterpret_cast<const uint8_t*>(a.ds_ws);
      const uint8_t* ws_p = ws_ds + (int64_t)a.batch * a.heads_q * a.ds_kt * a.ds_qt * kTileWs;
      const int group = a.heads_q / a.heads_kv;
      int g = 0;  // ring entries issued so far
      bool ok = true;
      for (int round = 0; ok; ++round) {
        const int w = snake_item(round, blockIdx.x, gridDim.x);
        if (w >= n_items) break;
        const GemmItem it = gemm_item(a, parts, w);
        for (int n = 0; n < it.n; ++n, ++g) {
          const uint8_t* tile;
          const CUtensorMap* map;
          int row, head;
          if (it.role == kRoleDQ) {
            const int kt = it.lo + n;
            tile = ws_ds + ws_tile(a, it.b, it.head, kt, it.t) * kTileWs;
            map = &map_k;
            row = kt * 128;
            head = it.head / group;
          } else {
            const int h = it.head * group + n / it.per_head, qt = it.lo + n % it.per_head;
            tile = (it.role == kRoleDV ? ws_p : ws_ds) + ws_tile(a, it.b, h, it.t, qt) * kTileWs;
            map = it.role == kRoleDV ? &map_do : &map_q;
            row = qt * 128;
            head = h;
          }
          if (tiles) {
            const int st = g % kTS;
            if (!mbar_wait(&t_empty[st], ((g / kTS) & 1) ^ 1)) {
              report_timeout(a.status, 611);
              ok = false;
              break;
            }
            mbar_arrive_expect_tx(&t_full[st], kTileWs);
            bulk_load_stream(smem + st * kTileWs, tile, kTileWs, &t_full[st]);
          } else {
            const int st = g % kOS;
            if (!mbar_wait(&o_empty[st], ((g / kOS) & 1) ^ 1)) {
              report_timeout(a.status, 615);
              ok = false;
              break;
            }
            uint8_t* dst = smem + L::kOffOp + st * L::kOpBytes;
            mbar_arrive_expect_tx(&o_full[st], L::kOpBytes);
#pragma unroll
            for (int c = 0; c < D / 64; ++c) tma_load_4d(dst + c * 16384, map, &o_full[st], c * 64, row, head, it.b);
          }
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      // the streamed operand (dO, Q or K rows) is read across its rows: N = head dim, contraction over the 128 rows
      constexpr uint32_t hi_b = smem_desc_hi(1024);
      // the workspace tile, unswizzled core matrices of 8 queries x 16 bytes (8 keys), blocks of 8 keys 2048 bytes apart:
      //   dQ (rows = queries, contraction over keys): read along its 16-byte rows; 8 keys on = 2048 bytes (leading
      //      offset), 8 queries on = 128 bytes (stride offset); 16 keys per instruction = 4096 bytes
      //   dV, dK (rows = keys, contraction over queries): read across them; 8 queries on = 128 bytes (leading offset),
      //      8 keys on = 2048 bytes (stride offset); 16 queries per instruction = 256 bytes
      constexpr uint32_t idesc_dq = make_idesc(DType<T>::kFormat, 128, D, 0, 1);
      constexpr uint32_t idesc_kv = make_idesc(DType<T>::kFormat, 128, D, 1, 1);
      constexpr uint32_t hi_dq = smem_desc_hi_noswizzle(128), hi_kv = smem_desc_hi_noswizzle(2048);
      const uint32_t base = smem_u32(smem);
      int g = 0, used = 0;
      bool ok = true;
      for (int round = 0; ok; ++round) {
        const int w = snake_item(round, blockIdx.x, gridDim.x);
        if (w >= n_items) break;
        const GemmItem it = gemm_item(a, parts, w);
        if (it.n == 0) continue;
        const int buf = used & 1;
        if (!mbar_wait(&acc_empty[buf], ((used >> 1) & 1) ^ 1)) {  // the epilogue has read this accumulator out
          report_timeout(a.status, 612);
          break;
        }
        tc_fence_after_sync();
        const bool dq = it.role == kRoleDQ;
        const uint32_t idesc = dq ? idesc_dq : idesc_kv, hi_a = dq ? hi_dq : hi_kv;
        const uint32_t a_lbo = dq ? 2048u : 128u, a_step = dq ? (4096u >> 4) : (256u >> 4);
        const uint32_t acc = tmem_base + buf * D;
        for (int n = 0; n < it.n; ++n, ++g) {
          const int ts = g % kTS, os = g % kOS;
          if (!mbar_wait(&t_full[ts], (g / kTS) & 1) || !mbar_wait(&o_full[os], (g / kOS) & 1)) {
            report_timeout(a.status, 613);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_lo = smem_desc_lo(base + ts * kTileWs, a_lbo);
          const uint32_t b_lo = smem_desc_lo(base + L::kOffOp + os * L::kOpBytes, 16384);
          if (n == 0) mma_ss_lo<0>(acc, a_lo, hi_a, b_lo, hi_b, idesc);
          else mma_ss_lo<1>(acc, a_lo, hi_a, b_lo, hi_b, idesc);
#pragma unroll
          for (int kk = 1; kk < 8; ++kk)  // 16 rows of the streamed operand per instruction
            mma_ss_lo<1>(acc, a_lo + kk * a_step, hi_a, b_lo + kk * (2048 >> 4), hi_b, idesc);
          tc_commit(&t_empty[ts]);
          tc_commit(&o_empty[os]);
        }
        if (!ok) break;
        tc_commit(&acc_full[buf]);
        ++used;
      }
    }
  } else if (warp < 4) {
    const int r = warp * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    int used = 0;
    for (int round = 0;; ++round) {
      const int w = snake_item(round, blockIdx.x, gridDim.x);
      if (w >= n_items) break;
      const GemmItem it = gemm_item(a, parts, w);
      const int row = it.t * 128 + r;
      TO* row_ptr;
      int rows;
      float scale = a.softmax_scale;
      if (it.role == kRoleDQ) {
        row_ptr = reinterpret_cast<TO*>(a.dq) + (int64_t)it.b * a.dq_sb + (int64_t)it.head * a.dq_sh + (int64_t)row * a.dq_ss;
        rows = a.seqlen_q;
        if (a.row_stats != nullptr && it.n > 0)  // forward: O = (P V) / row sum (tiles nothing reaches have no entry)
          scale = a.row_stats[((int64_t)it.b * a.heads_q + it.head) * (a.ds_qt * 128) + row].y;
      } else if (it.role == kRoleDK) {
        row_ptr = reinterpret_cast<TO*>(a.dk) + (int64_t)it.b * a.dk_sb + (int64_t)it.head * a.dk_sh + (int64_t)row * a.dk_ss;
        rows = a.seqlen_k;
      } else {
        row_ptr = reinterpret_cast<TO*>(a.dv) + (int64_t)it.b * a.dv_sb + (int64_t)it.head * a.dv_sh + (int64_t)row * a.dv_ss;
        rows = a.seqlen_k;
        scale = 1.f;
      }
      const int buf = used & 1;
      if (it.n > 0) {
        if (!__all_sync(kFull, mbar_wait(&acc_full[buf], (used >> 1) & 1))) {
          report_timeout(a.status, 614);
          break;
        }
        tc_fence_after_sync();
      }
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        if (it.n > 0) {
          tmem_ld32(tmem_base + lane_addr + buf * D + c * 32, o);
          tc_wait_ld_regs(o);
        } else {  // rows that nothing reaches: the gradient is zero
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = 0u;
        }
        if (row < rows) store_out_slice<TO>(row_ptr + c * 32, o, scale, a.head_dim - c * 32);
      }
      if (it.n > 0) {
        tc_fence_before_sync();
        mbar_arrive(&acc_empty[buf]);
        ++used;
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, kCols);
}

// The products kernel over the tiles in a.ds_ws. dependent: launched as a programmatic dependent of the kernel before
// it on the stream (which wrote the tiles and releases its dependents early).
template <typename T, int D, typename TO = T>
int launch_products(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mdo, const BwdArgs& a, int parts,
                    bool dependent, cudaStream_t stream) {
  auto kern = bwd_wide_gemm_kernel<T, D, TO>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<D>::kBytes);
  if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "products smem opt-in failed: %s", cudaGetErrorString(e));
  const int sms = sm_count();
  const int n_items = ((parts & FA_BWD_DKDV) ? 2 * a.ds_kt * a.batch * a.heads_kv : 0) +
                      ((parts & FA_BWD_DQ) ? a.ds_qt * a.batch * a.heads_q : 0);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_items < sms ? n_items : sms);
  cfg.blockDim = dim3(kWideGemmThreads);
  cfg.dynamicSmemBytes = GemmSmem<D>::kBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr = {};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  if (dependent) {  // its CTAs may set themselves up while the last CTAs of that kernel drain (they wait inside)
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  }
  e = cudaLaunchKernelEx(&cfg, kern, mq, mk, mdo, a, parts);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "products launch failed: %s", cudaGetErrorString(e));
  return 0;
}

template <typename T, int D, bool kMods>
int launch_wide_typed(const fa_attn_params& p, const BwdArgs& a, int parts, cudaStream_t stream) {
  auto map_of = [&](CUtensorMap* m, const void* ptr, int rows, int heads, const int64_t* st) {
    return make_tile_map(m, ptr, p.dtype, p.head_dim, rows, heads, p.batch, st[2], st[1], st[0], 128);
  };
  CUtensorMap mq, mk, mv, mdo;
  int rc = map_of(&mq, p.q, p.seqlen_q, p.heads_q, p.q_strides);
  if (!rc) rc = map_of(&mk, p.k, p.seqlen_k, p.heads_kv, p.k_strides);
  if (!rc) rc = map_of(&mv, p.v, p.seqlen_k, p.heads_kv, p.v_strides);
  if (!rc) rc = map_of(&mdo, p.dout, p.seqlen_q, p.heads_q, p.do_strides);
  if (rc) return rc;
  cudaError_t e;
  const int sms = sm_count();
  if (parts & FA_BWD_DKDV) {
    auto kern = bwd_wide_scores_kernel<T, D, kMods>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, WideSmem<D>::kBytes);
    if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "backward smem opt-in failed: %s", cudaGetErrorString(e));
    const int n_items = a.ds_qt * p.batch * p.heads_q;
    kern<<<dim3(n_items < sms ? n_items : sms), kBwdThreads, WideSmem<D>::kBytes, stream>>>(mq, mk, mv, mdo, a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "backward scores launch failed: %s", cudaGetErrorString(e));
  }
  return launch_products<T, D>(mq, mk, mdo, a, parts, (parts & FA_BWD_DKDV) != 0, stream);
}


template <typename T>
int launch_fwd_wide_typed(const fa_attn_params& p, const BwdArgs& a0, cudaStream_t stream) {
  CUtensorMap mq, mk;
  int rc = make_tile_map(&mq, p.q, p.dtype, p.head_dim, p.seqlen_q, p.heads_q, p.batch, p.q_strides[2], p.q_strides[1],
                         p.q_strides[0], 128);
  if (!rc) rc = make_tile_map(&mk, p.k, p.dtype, p.head_dim, p.seqlen_k, p.heads_kv, p.batch, p.k_strides[2],
                              p.k_strides[1], p.k_strides[0], 128);
  if (rc) return rc;
  const int sms = sm_count();
  const int n_items = a0.ds_qt * p.batch * p.heads_q;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_items < sms ? n_items : sms);
  cfg.blockDim = dim3(kBwdThreads);
  cfg.dynamicSmemBytes = FwdWideSmem::kBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr = {};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cudaError_t e;
  {  // 1. row statistics -> LSE
    auto kern = fwd_wide_kernel<T, kModeStats>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdWideSmem::kBytes);
    if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, kern, mq, mk, a0);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "forward statistics launch failed: %s", cudaGetErrorString(e));
  }
  {  // 2. normalised P tiles; set up while the statistics kernel drains
    auto kern = fwd_wide_kernel<T, kModeProbsMax>;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdWideSmem::kBytes);
    if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, kern, mq, mk, a0);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "forward probabilities launch failed: %s", cudaGetErrorString(e));
  }
  // 3. O = P V, the product dQ = dS K with V in the place of K, O in the place of dQ and no scale; one launch per
  //    256 columns of the head dim
  for (int col0 = 0; col0 < p.head_dim; col0 += kWD) {
    const int width = p.head_dim - col0 < kWD ? p.head_dim - col0 : kWD;
    const T* v = reinterpret_cast<const T*>(p.v) + col0;
    CUtensorMap mv;
    rc = make_tile_map(&mv, v, p.dtype, width, p.seqlen_k, p.heads_kv, p.batch, p.v_strides[2], p.v_strides[1],
                       p.v_strides[0], 128);
    if (rc) return rc;
    BwdArgs a = a0;
    a.head_dim = width;
    a.softmax_scale = 1.f;
    a.dq = reinterpret_cast<T*>(p.out) + col0;
    a.dq_sb = p.o_strides[0];
    a.dq_sh = p.o_strides[1];
    a.dq_ss = p.o_strides[2];
    rc = launch_products<T, kWD>(mv, mv, mv, a, FA_BWD_DQ, true, stream);
    if (rc) return rc;
  }
  return 0;
}

// fp32 inputs: an operand rounded to fp16 once, rows made contiguous, for the products over the 16-bit tiles.
__global__ void __launch_bounds__(256) convert_rows_f16_kernel(const float* src, int64_t sb, int64_t sh, int64_t ss,
                                                               __half* dst, int heads, int rows, int head_dim, int64_t total8) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int per_row = head_dim / 8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % per_row);
    const int64_t row_flat = i / per_row;
    const int r = (int)(row_flat % rows), h = (int)((row_flat / rows) % heads);
    const int64_t b = row_flat / ((int64_t)rows * heads);
    const float* p = src + b * sb + (int64_t)h * sh + (int64_t)r * ss + c * 8;
    const float4 x = *reinterpret_cast<const float4*>(p), y = *reinterpret_cast<const float4*>(p + 4);
    uint4 o;
    o.x = DType<__half>::pack2(x.x, x.y);
    o.y = DType<__half>::pack2(x.z, x.w);
    o.z = DType<__half>::pack2(y.x, y.y);
    o.w = DType<__half>::pack2(y.z, y.w);
    *reinterpret_cast<uint4*>(dst + row_flat * head_dim + c * 8) = o;
  }
}

// Forward for fp32 inputs (head dims to 256): Q K^T as tf32 MMAs on the fp32 tiles, P as fp16 tiles, V rounded to fp16,
// O and LSE in fp32.
int launch_fwd_wide_f32(const fa_attn_params& p, const BwdArgs& a0, cudaStream_t stream) {
  CUtensorMap mq, mk;
  int rc = make_tile_map_f32(&mq, p.q, p.head_dim, p.seqlen_q, p.heads_q, p.batch, p.q_strides[2], p.q_strides[1],
                             p.q_strides[0], 128);
  if (!rc) rc = make_tile_map_f32(&mk, p.k, p.head_dim, p.seqlen_k, p.heads_kv, p.batch, p.k_strides[2], p.k_strides[1],
                                  p.k_strides[0], 128);
  if (rc) return rc;
  // V in fp16 behind the P tiles and the row statistics
  __half* v16 = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(a0.row_stats) +
                                          (int64_t)p.batch * p.heads_q * a0.ds_qt * 128 * 8);
  const int64_t total8 = (int64_t)p.batch * p.heads_kv * p.seqlen_k * (p.head_dim / 8);
  const int sms = sm_count();
  const int64_t want = (total8 + 255) / 256;
  convert_rows_f16_kernel<<<(int)(want < 8 * sms ? want : 8 * sms), 256, 0, stream>>>(
      reinterpret_cast<const float*>(p.v), p.v_strides[0], p.v_strides[1], p.v_strides[2], v16, p.heads_kv, p.seqlen_k,
      p.head_dim, total8);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "forward V conversion launch failed: %s", cudaGetErrorString(e));
  const int n_items = a0.ds_qt * p.batch * p.heads_q;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_items < sms ? n_items : sms);
  cfg.blockDim = dim3(kBwdThreads);
  cfg.dynamicSmemBytes = FwdWideSmem::kBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr = {};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  {
    auto kern = fwd_wide_kernel<__half, kModeStats, float>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdWideSmem::kBytes);
    if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, kern, mq, mk, a0);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "forward statistics launch failed: %s", cudaGetErrorString(e));
  }
  {
    auto kern = fwd_wide_kernel<__half, kModeProbsMax, float>;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdWideSmem::kBytes);
    if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, kern, mq, mk, a0);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "forward probabilities launch failed: %s", cudaGetErrorString(e));
  }
  CUtensorMap mv;
  rc = make_tile_map(&mv, v16, FA_F16, p.head_dim, p.seqlen_k, p.heads_kv, p.batch, p.head_dim,
                     (int64_t)p.seqlen_k * p.head_dim, (int64_t)p.heads_kv * p.seqlen_k * p.head_dim, 128);
  if (rc) return rc;
  BwdArgs a = a0;
  a.softmax_scale = 1.f;
  a.dq = p.out;
  a.dq_sb = p.o_strides[0];
  a.dq_sh = p.o_strides[1];
  a.dq_ss = p.o_strides[2];
  return launch_products<__half, kWD, float>(mv, mv, mv, a, FA_BWD_DQ, true, stream);
}

// Backward for fp32 inputs (head dims to 256, no score modifier): S and dP as tf32 products on the fp32 tiles, P and dS
// as fp16 tiles, Q, K and dO rounded to fp16 for the three products, fp32 gradients.
int launch_bwd_wide_f32(const fa_attn_params& p, const BwdArgs& a0, int parts, cudaStream_t stream) {
  const int sms = sm_count();
  cudaError_t e;
  int rc;
  const int64_t tiles = (int64_t)p.batch * p.heads_q * a0.ds_kt * a0.ds_qt;
  const int64_t nq = (int64_t)p.batch * p.heads_q * p.seqlen_q * p.head_dim;
  const int64_t nk = (int64_t)p.batch * p.heads_kv * p.seqlen_k * p.head_dim;
  __half* q16 = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(p.ds_workspace) + 2 * tiles * kTileWs);
  __half* do16 = q16 + nq;
  __half* k16 = do16 + nq;
  if (parts & FA_BWD_DKDV) {
    auto convert = [&](const void* src, const int64_t* st, __half* dst, int heads, int rows) {
      const int64_t total8 = (int64_t)p.batch * heads * rows * (p.head_dim / 8);
      const int64_t want = (total8 + 255) / 256;
      convert_rows_f16_kernel<<<(int)(want < 8 * sms ? want : 8 * sms), 256, 0, stream>>>(
          reinterpret_cast<const float*>(src), st[0], st[1], st[2], dst, heads, rows, p.head_dim, total8);
    };
    convert(p.q, p.q_strides, q16, p.heads_q, p.seqlen_q);
    convert(p.dout, p.do_strides, do16, p.heads_q, p.seqlen_q);
    convert(p.k, p.k_strides, k16, p.heads_kv, p.seqlen_k);
    e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "backward conversion launch failed: %s", cudaGetErrorString(e));
    CUtensorMap mq, mk, mv, mdo;
    auto map32 = [&](CUtensorMap* m, const void* ptr, int rows, int heads, const int64_t* st) {
      return make_tile_map_f32(m, ptr, p.head_dim, rows, heads, p.batch, st[2], st[1], st[0], 128);
    };
    rc = map32(&mq, p.q, p.seqlen_q, p.heads_q, p.q_strides);
    if (!rc) rc = map32(&mk, p.k, p.seqlen_k, p.heads_kv, p.k_strides);
    if (!rc) rc = map32(&mv, p.v, p.seqlen_k, p.heads_kv, p.v_strides);
    if (!rc) rc = map32(&mdo, p.dout, p.seqlen_q, p.heads_q, p.do_strides);
    if (rc) return rc;
    const int n_items = a0.ds_qt * p.batch * p.heads_q;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_items < sms ? n_items : sms);
    cfg.blockDim = dim3(kBwdThreads);
    cfg.dynamicSmemBytes = FwdWideSmem::kBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    {
      auto kern = fwd_wide_kernel<__half, kModeProbsLse, float>;
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdWideSmem::kBytes);
      if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, kern, mq, mk, a0);
      if (e == cudaSuccess) e = cudaGetLastError();
      if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "backward probabilities launch failed: %s", cudaGetErrorString(e));
    }
    {
      auto kern = fwd_wide_kernel<__half, kModeDScores, float>;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdWideSmem::kBytes);
      if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, kern, mdo, mv, a0);
      if (e == cudaSuccess) e = cudaGetLastError();
      if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "backward dS launch failed: %s", cudaGetErrorString(e));
    }
  }
  CUtensorMap mq, mk, mdo;
  auto map16 = [&](CUtensorMap* m, const __half* ptr, int rows, int heads) {
    return make_tile_map(m, ptr, FA_F16, p.head_dim, rows, heads, p.batch, p.head_dim, (int64_t)rows * p.head_dim,
                         (int64_t)heads * rows * p.head_dim, 128);
  };
  rc = map16(&mq, q16, p.seqlen_q, p.heads_q);
  if (!rc) rc = map16(&mk, k16, p.seqlen_k, p.heads_kv);
  if (!rc) rc = map16(&mdo, do16, p.seqlen_q, p.heads_q);
  if (rc) return rc;
  return launch_products<__half, kWD, float>(mq, mk, mdo, a0, parts, (parts & FA_BWD_DKDV) != 0, stream);
}

// Backward for head dims above 256: P tiles, then dS tiles, then the products once per 256 columns.
template <typename T>
int launch_bwd_vwide_typed(const fa_attn_params& p, const BwdArgs& a0, int parts, cudaStream_t stream) {
  auto map_of = [&](CUtensorMap* m, const void* ptr, int width, int rows, int heads, const int64_t* st) {
    return make_tile_map(m, ptr, p.dtype, width, rows, heads, p.batch, st[2], st[1], st[0], 128);
  };
  const int sms = sm_count();
  cudaError_t e;
  int rc;
  if (parts & FA_BWD_DKDV) {
    CUtensorMap mq, mk, mv, mdo;
    rc = map_of(&mq, p.q, p.head_dim, p.seqlen_q, p.heads_q, p.q_strides);
    if (!rc) rc = map_of(&mk, p.k, p.head_dim, p.seqlen_k, p.heads_kv, p.k_strides);
    if (!rc) rc = map_of(&mv, p.v, p.head_dim, p.seqlen_k, p.heads_kv, p.v_strides);
    if (!rc) rc = map_of(&mdo, p.dout, p.head_dim, p.seqlen_q, p.heads_q, p.do_strides);
    if (rc) return rc;
    const int n_items = a0.ds_qt * p.batch * p.heads_q;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_items < sms ? n_items : sms);
    cfg.blockDim = dim3(kBwdThreads);
    cfg.dynamicSmemBytes = FwdWideSmem::kBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    {
      auto kern = fwd_wide_kernel<T, kModeProbsLse>;
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdWideSmem::kBytes);
      if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, kern, mq, mk, a0);
      if (e == cudaSuccess) e = cudaGetLastError();
      if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "backward probabilities launch failed: %s", cudaGetErrorString(e));
    }
    {
      auto kern = fwd_wide_kernel<T, kModeDScores>;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdWideSmem::kBytes);
      if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, kern, mdo, mv, a0);
      if (e == cudaSuccess) e = cudaGetLastError();
      if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "backward dS launch failed: %s", cudaGetErrorString(e));
    }
  }
  for (int col0 = 0; col0 < p.head_dim; col0 += kWD) {
    const int width = p.head_dim - col0 < kWD ? p.head_dim - col0 : kWD;
    CUtensorMap mq, mk, mdo;
    rc = map_of(&mq, reinterpret_cast<const T*>(p.q) + col0, width, p.seqlen_q, p.heads_q, p.q_strides);
    if (!rc) rc = map_of(&mk, reinterpret_cast<const T*>(p.k) + col0, width, p.seqlen_k, p.heads_kv, p.k_strides);
    if (!rc) rc = map_of(&mdo, reinterpret_cast<const T*>(p.dout) + col0, width, p.seqlen_q, p.heads_q, p.do_strides);
    if (rc) return rc;
    BwdArgs a = a0;
    a.head_dim = width;
    a.dq = reinterpret_cast<T*>(p.dq) + col0;
    a.dk = reinterpret_cast<T*>(p.dk) + col0;
    a.dv = reinterpret_cast<T*>(p.dv) + col0;
    rc = launch_products<T, kWD>(mq, mk, mdo, a, parts, (parts & FA_BWD_DKDV) != 0 || col0 > 0, stream);
    if (rc) return rc;
  }
  return 0;
}

}  // namespace

namespace {
// An fp32 operand (batch, head, row, dim) TMA can read: unit inner stride, 16-byte aligned base and rows.
bool tma_operand_ok_f32(const void* ptr, const int64_t strides[4], const int64_t sizes[3]) {
  if (ptr == nullptr || (reinterpret_cast<uintptr_t>(ptr) & 15) || strides[3] != 1) return false;
  for (int i = 0; i < 3; ++i)
    if (sizes[i] > 1 && (strides[i] <= 0 || (strides[i] % 4) != 0)) return false;
  return true;
}
}  // namespace

// Head dims above 128 up to 512, dense, 16-bit, with a workspace for the P and dS tiles; above 256 without score
// modifiers only. fp32 inputs that bring a workspace opt into tf32 / fp16 products (head dims to 256, no modifier).
bool bwd_wide_supported(const fa_attn_params& p) {
  if (p.varlen || p.ds_workspace == nullptr) return false;
  if (p.dtype == FA_F32) {
    if (p.head_dim < 8 || p.head_dim > kWD || p.head_dim % 8) return false;
    if (p.softcap > 0.f || p.bias != nullptr || p.alibi_slopes != nullptr || p.dropout_p > 0.f || !(p.softmax_scale > 0.f))
      return false;
    const int64_t fq[3] = {p.batch, p.heads_q, p.seqlen_q};
    const int64_t fk[3] = {p.batch, p.heads_kv, p.seqlen_k};
    return tma_operand_ok_f32(p.q, p.q_strides, fq) && tma_operand_ok_f32(p.k, p.k_strides, fk) &&
           tma_operand_ok_f32(p.v, p.v_strides, fk) && tma_operand_ok_f32(p.dout, p.do_strides, fq) &&
           tma_operand_ok_f32(p.dq, p.dq_strides, fq) && tma_operand_ok_f32(p.dk, p.dk_strides, fk) &&
           tma_operand_ok_f32(p.dv, p.dv_strides, fk);
  }
  if (p.dtype != FA_F16 && p.dtype != FA_BF16) return false;
  if (p.head_dim <= 128 || p.head_dim > 512 || p.head_dim % 8) return false;
  if (p.head_dim > kWD && (p.softcap > 0.f || p.bias != nullptr || p.alibi_slopes != nullptr || p.dropout_p > 0.f ||
                           !(p.softmax_scale > 0.f)))
    return false;
  const int64_t sq[3] = {p.batch, p.heads_q, p.seqlen_q};
  const int64_t sk[3] = {p.batch, p.heads_kv, p.seqlen_k};
  return tma_operand_ok(p.q, p.q_strides, sq) && tma_operand_ok(p.k, p.k_strides, sk) &&
         tma_operand_ok(p.v, p.v_strides, sk) && tma_operand_ok(p.dout, p.do_strides, sq) &&
         tma_operand_ok(p.dq, p.dq_strides, sq) && tma_operand_ok(p.dk, p.dk_strides, sk) &&
         tma_operand_ok(p.dv, p.dv_strides, sk);
}

// One dS tile and one P tile of 32 KB per (batch, query head, key tile, query tile).
int64_t bwd_wide_workspace_bytes(const fa_attn_params& p) {
  if (p.varlen) return 0;
  const int64_t tiles = (int64_t)p.batch * p.heads_q * ((p.seqlen_k + 127) / 128) * ((p.seqlen_q + 127) / 128);
  int64_t bytes = 2 * tiles * kTileWs;
  if (p.dtype == FA_F32)  // Q, dO and K rounded to fp16
    bytes += 2 * ((int64_t)p.batch * p.head_dim * (2 * (int64_t)p.heads_q * p.seqlen_q + (int64_t)p.heads_kv * p.seqlen_k));
  return bytes;
}

int launch_bwd_wide(const fa_attn_params& p, int parts, cudaStream_t stream) {
  const int64_t need = bwd_wide_workspace_bytes(p);
  if (p.ds_workspace_bytes < need)
    return set_error(FA_ERR_INVALID_ARGUMENT, "ds_workspace holds %lld bytes, this problem needs %lld",
                     (long long)p.ds_workspace_bytes, (long long)need);
  if (reinterpret_cast<uintptr_t>(p.ds_workspace) & 1023)
    return set_error(FA_ERR_INVALID_ARGUMENT, "ds_workspace must be aligned to 1024 bytes");
  BwdArgs a = {};
  a.varlen = 0;
  a.batch = p.batch;
  a.heads_q = p.heads_q;
  a.heads_kv = p.heads_kv;
  a.head_dim = p.head_dim;
  a.seqlen_q = p.seqlen_q;
  a.seqlen_k = p.seqlen_k;
  a.total_q = p.total_q;
  a.total_k = p.total_k;
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
  a.status = p.status;
  a.ds_ws = p.ds_workspace;
  a.ds_kt = (p.seqlen_k + 127) / 128;
  a.ds_qt = (p.seqlen_q + 127) / 128;
  if (p.dtype == FA_F32) return launch_bwd_wide_f32(p, a, parts, stream);
  if (p.head_dim > kWD)
    return p.dtype == FA_F16 ? launch_bwd_vwide_typed<__half>(p, a, parts, stream)
                             : launch_bwd_vwide_typed<__nv_bfloat16>(p, a, parts, stream);
  const bool mods = p.softcap > 0.f || p.bias != nullptr || p.alibi_slopes != nullptr || p.dropout_p > 0.f;
  if (p.dtype == FA_F16)
    return mods ? launch_wide_typed<__half, 256, true>(p, a, parts, stream)
                : launch_wide_typed<__half, 256, false>(p, a, parts, stream);
  return mods ? launch_wide_typed<__nv_bfloat16, 256, true>(p, a, parts, stream)
              : launch_wide_typed<__nv_bfloat16, 256, false>(p, a, parts, stream);
}

// Forward for head dims above 256 up to 512: dense, 16-bit, no score modifier, with a workspace for the P tiles.
bool fwd_wide_supported(const fa_attn_params& p) {
  if (p.varlen || p.ds_workspace == nullptr || p.lse == nullptr) return false;
  if (p.softcap > 0.f || p.bias != nullptr || p.alibi_slopes != nullptr || p.dropout_p > 0.f) return false;
  if (!(p.softmax_scale > 0.f)) return false;
  if (p.dtype == FA_F32) {
    // fp32 inputs that bring a workspace opt into tf32 / fp16 products (head dims to 256)
    if (p.head_dim < 8 || p.head_dim > 256 || p.head_dim % 8) return false;
    const int64_t fq[3] = {p.batch, p.heads_q, p.seqlen_q};
    const int64_t fk[3] = {p.batch, p.heads_kv, p.seqlen_k};
    return tma_operand_ok_f32(p.q, p.q_strides, fq) && tma_operand_ok_f32(p.k, p.k_strides, fk) &&
           tma_operand_ok_f32(p.v, p.v_strides, fk) && tma_operand_ok_f32(p.out, p.o_strides, fq);
  }
  if (p.dtype != FA_F16 && p.dtype != FA_BF16) return false;
  if (p.head_dim <= 256 || p.head_dim > 512 || p.head_dim % 8) return false;
  const int64_t sq[3] = {p.batch, p.heads_q, p.seqlen_q};
  const int64_t sk[3] = {p.batch, p.heads_kv, p.seqlen_k};
  return tma_operand_ok(p.q, p.q_strides, sq) && tma_operand_ok(p.k, p.k_strides, sk) &&
         tma_operand_ok(p.v, p.v_strides, sk) && tma_operand_ok(p.out, p.o_strides, sq);
}

// One P tile of 32 KB per (batch, query head, key tile, query tile), then 8 bytes per query row of the padded tiles.
int64_t fwd_wide_workspace_bytes(const fa_attn_params& p) {
  if (p.varlen) return 0;
  const int64_t qt = (p.seqlen_q + 127) / 128;
  const int64_t tiles = (int64_t)p.batch * p.heads_q * ((p.seqlen_k + 127) / 128) * qt;
  int64_t bytes = tiles * kTileWs + (int64_t)p.batch * p.heads_q * qt * 128 * 8;
  if (p.dtype == FA_F32) bytes += (int64_t)p.batch * p.heads_kv * p.seqlen_k * p.head_dim * 2;  // V rounded to fp16
  return bytes;
}

int launch_fwd_wide(const fa_attn_params& p, cudaStream_t stream) {
  const int64_t need = fwd_wide_workspace_bytes(p);
  if (p.ds_workspace_bytes < need)
    return set_error(FA_ERR_INVALID_ARGUMENT, "ds_workspace holds %lld bytes, this problem needs %lld",
                     (long long)p.ds_workspace_bytes, (long long)need);
  if (reinterpret_cast<uintptr_t>(p.ds_workspace) & 1023)
    return set_error(FA_ERR_INVALID_ARGUMENT, "ds_workspace must be aligned to 1024 bytes");
  BwdArgs a = {};
  a.batch = p.batch;
  a.heads_q = p.heads_q;
  a.heads_kv = p.heads_kv;
  a.head_dim = p.head_dim;
  a.seqlen_q = p.seqlen_q;
  a.seqlen_k = p.seqlen_k;
  a.lse = p.lse;
  a.lse_out = p.lse;
  a.l_sb = p.lse_strides[0];
  a.l_sh = p.lse_strides[1];
  a.l_ss = p.lse_strides[2];
  a.softmax_scale = p.softmax_scale;
  a.causal = p.causal;
  a.wl = p.window_left;
  a.wr = p.window_right;
  a.status = p.status;
  a.ds_ws = p.ds_workspace;
  a.ds_kt = (p.seqlen_k + 127) / 128;
  a.ds_qt = (p.seqlen_q + 127) / 128;
  a.row_stats = reinterpret_cast<float2*>(reinterpret_cast<uint8_t*>(p.ds_workspace) +
                                          (int64_t)p.batch * p.heads_q * a.ds_kt * a.ds_qt * kTileWs);
  if (p.dtype == FA_F32) return launch_fwd_wide_f32(p, a, stream);
  return p.dtype == FA_F16 ? launch_fwd_wide_typed<__half>(p, a, stream) : launch_fwd_wide_typed<__nv_bfloat16>(p, a, stream);
}

}  // namespace fa
