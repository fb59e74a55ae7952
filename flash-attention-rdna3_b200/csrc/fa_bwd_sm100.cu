// FlashAttention-2 backward for sm_100a as two tcgen05 kernels (delta = rowsum(O*dO) is computed
// before them). Accumulators live in tensor memory; operand tiles arrive by TMA. Both kernels walk their
// streamed operand in steps of 128 rows, so every MMA is 128 x 128 x 16 or 128 x D x 16 (N = 64 would run the
// tensor pipe at half rate), and split the elementwise work of a step into two phases that overlap MMAs of the
// neighbouring steps:   phase 1  P = exp2(S*c - lse)      phase 2  dS = P * (dP - delta)
//   warps 0-3   compute group 0: columns [0,64) of every step   (thread = one TMEM lane = one row)
//   warps 4-7   compute group 1: columns [64,128)
//   warp  8     TMA producer (one lane)
//   warp  9     MMA issuer (one lane)
//
// dK/dV kernel: one CTA per 128-key tile of one (batch, kv head); K and V stay in shared memory and
// the CTA walks 128-query steps of every query head of the GQA group (no atomics, fixed summation order):
//     S^T  = K Q^T          dP^T = V dO^T                  (M = 128 keys, N = 128 queries)
//     P^T  = exp2(S^T*c - lse[q]) ;  dS^T = P^T * (dP^T - delta[q])      (lse/delta per column, staged in smem)
//     dV  += P^T dO         dK  += dS^T Q                  (A from TMEM, B = the same smem tiles, MN-major)
// TMEM: S^T [0,128); dP^T, then P^T and dS^T [128,256); dK [256,256+D); dV [256+D,256+2D).
//
// dQ kernel: persistent CTAs walking 128-query tiles; Q and dO stay resident, K/V stream in 128-key steps:
//     S = Q K^T    dP = dO V^T    dS = P*(dP - delta[row])    dQ += dS K
// TMEM: S buffers [0,128) [128,256); dP [256,384); dQ [384,384+D).
//
// The 16-bit P^T / dS^T (and dS) operands overwrite fp32 score columns of their own group's half, only over columns
// the writing thread has already consumed.
//
// Math follows fa_rdna3/kernels/_common.py:347-508 and fa_rdna3/kernels/backward.py:56-322 (varlen:
// fa_rdna3/kernels/varlen.py:193-421): P recomputed from LSE, rows with LSE = -inf contribute nothing,
// softcap chain factor (1 - tanh^2), dropout regenerated from the same counters, dQ and dK scaled by
// softmax_scale at the end.
#include "fa_bwd_shared.cuh"
#include "fa_tma_host.h"
#include "fa_prof.cuh"

namespace fa {
namespace {


// =============================================================================================
// dK / dV
// =============================================================================================
// 32 raw scores of one row -> 16 packed 16-bit probabilities: p = exp2(s * scale_log2 + nlse[col]) with columns outside
// [c_lo, c_hi] (numbered from col0) zeroed when kMasked. nlse points at the 32 per-column values in shared memory.
template <typename T, bool kMasked>
__device__ __forceinline__ void probs_chunk(const uint32_t (&s)[32], const float* nlse, uint64_t sc2, int col0, int c_lo,
                                            int c_hi, uint32_t* pk) {
#pragma unroll
  for (int e4 = 0; e4 < 8; ++e4) {  // four columns at a time: one 16-byte read
    const float4 nl = *reinterpret_cast<const float4*>(nlse + e4 * 4);
    const float nls[4] = {nl.x, nl.y, nl.z, nl.w};
#pragma unroll
    for (int e2 = 0; e2 < 2; ++e2) {
      const int e = e4 * 2 + e2;
      const uint64_t x2 = fma_f32x2(pack_u32x2(s[2 * e], s[2 * e + 1]), sc2, pack_f32x2(nls[2 * e2], nls[2 * e2 + 1]));
      float x0, x1;
      unpack_f32x2(x2, &x0, &x1);
      float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
      if (kMasked) {
        const int col = col0 + 2 * e;
        if (col < c_lo || col > c_hi) p0 = 0.f;
        if (col + 1 < c_lo || col + 1 > c_hi) p1 = 0.f;
      }
      pk[e] = DType<T>::pack2(p0, p1);
    }
  }
}

// 32 raw dP values of one row and the matching packed probabilities -> 16 packed dS = p * (dp + ndelta[col]).
template <typename T>
__device__ __forceinline__ void dscore_chunk(const uint32_t (&dp)[32], const float* ndelta, const uint32_t* pk,
                                             uint32_t (&dsk)[16]) {
#pragma unroll
  for (int e4 = 0; e4 < 8; ++e4) {
    const float4 nd = *reinterpret_cast<const float4*>(ndelta + e4 * 4);
    const float nds[4] = {nd.x, nd.y, nd.z, nd.w};
#pragma unroll
    for (int e2 = 0; e2 < 2; ++e2) {
      const int e = e4 * 2 + e2;
      const float2 pf = DType<T>::unpack2(pk[e]);
      const uint64_t dd = add_f32x2(pack_u32x2(dp[2 * e], dp[2 * e + 1]), pack_f32x2(nds[2 * e2], nds[2 * e2 + 1]));
      float d0, d1;
      unpack_f32x2(mul_f32x2(pack_f32x2(pf.x, pf.y), dd), &d0, &d1);
      dsk[e] = DType<T>::pack2(d0, d1);
    }
  }
}


// Shared-memory plan of the dK/dV kernel; everything is dynamic so that the tiles can take (almost) all of it.
template <int D>
struct DkdvSmem {
  static constexpr int kChunks = D / 64;
  static constexpr int kTileBytes = kChunks * 16384;  // one 128-row operand tile
  static constexpr int kQStages = D == 128 ? 3 : 4;   // Q lives from S^T of its step to dK of the same step
  static constexpr int kDoStages = D == 128 ? 2 : 3;
  static constexpr int kOffK = 0;
  static constexpr int kOffV = kTileBytes;
  static constexpr int kOffQ = 2 * kTileBytes;
  static constexpr int kOffDo = kOffQ + kQStages * kTileBytes;
  static constexpr int kOffStage = kOffDo + kDoStages * kTileBytes;  // two sets of 128 x (-lse*log2e), 128 x (-delta)
  static constexpr int kOffBars = kOffStage + 2 * 256 * 4;
  static constexpr int kNumBars = 8 + 2 * kQStages + 2 * kDoStages;
  static constexpr int kOffTmemPtr = kOffBars + kNumBars * 8;
  static constexpr int kBytes = kOffTmemPtr + 8;  // the dynamic region is declared 1024-byte aligned (and checked)
  static_assert(kBytes <= 232448, "dK/dV shared memory plan exceeds one CTA's 227 KB");
};

__device__ __forceinline__ void compute_sync() {
  asm volatile("bar.sync 1, 256;" ::: "memory");  // the eight compute warps
}

// One CTA per 128-key tile of one (batch, kv head). Step i of the pipe (128 queries; all MMAs issued by one thread, in
// this order):
//     S^T(i+1) = K Q(i+1)^T       as soon as the compute warps hold S^T(i) in registers (start of phase 1 of step i)
//     dV  += P^T(i) dO(i)         needs phase 1 of step i and dP^T(i) read into registers
//     dK  += dS^T(i) Q(i)         needs phase 2 of step i
//     dP^T(i+1) = V dO(i+1)^T     overwrites P^T(i) and dS^T(i)
// The 16-bit P^T and dS^T of a group both live in that group's 64 dP^T columns (first and second 32), which a thread
// overwrites only after it has read its dP^T values; the S^T columns are therefore free during the whole of phase 1
// and the next scores are formed behind it, off the phase 1 -> dV -> S^T -> phase 1 chain. All 512 TMEM columns are in
// use without double buffering: S^T [0,128), dP^T/P^T/dS^T [128,256), dK [256,256+D), dV [256+D,256+2D).
// With score modifiers (kMods) both score tiles are consumed in one pass, P^T stays in its S^T columns and S^T(i+1)
// follows dV(i) instead.
template <typename T, int D, bool kMods>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_dkdv_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                const BwdArgs a) {
  using L = DkdvSmem<D>;
  constexpr int kChunks = L::kChunks;
  constexpr int kTileBytes = L::kTileBytes;
  constexpr int kQS = L::kQStages, kDS = L::kDoStages;

  // The 128-byte swizzle wants tiles on 1 KB boundaries and the plan leaves no room to round the base up.
  extern __shared__ __align__(1024) uint8_t smem_dkdv[];
  uint8_t* smem = smem_dkdv;
  if ((smem_u32(smem) & 1023u) != 0) {  // never seen; leave before anything is set up rather than run past the end
    if (threadIdx.x == 0) report_timeout(a.status, 211);
    return;
  }
  uint8_t* sK = smem + L::kOffK;
  uint8_t* sV = smem + L::kOffV;
  uint8_t* sQ = smem + L::kOffQ;
  uint8_t* sDo = smem + L::kOffDo;
  float* stage_s = reinterpret_cast<float*>(smem + L::kOffStage);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBars);
  uint64_t* k_full = bars + 0;
  uint64_t* v_full = bars + 1;
  uint64_t* s_full = bars + 2;
  uint64_t* p_full = bars + 3;
  uint64_t* dp_full = bars + 4;
  uint64_t* ds_full = bars + 5;
  uint64_t* acc_done = bars + 6;
  uint64_t* s_free = bars + 7;
  uint64_t* q_full = bars + 8;
  uint64_t* q_empty = q_full + kQS;
  uint64_t* do_full = q_empty + kQS;
  uint64_t* do_empty = do_full + kDS;
  uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(smem + L::kOffTmemPtr);

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  int ktile = blockIdx.y;
  int b = blockIdx.x / a.heads_kv, hk = blockIdx.x % a.heads_kv;
  const int group = a.heads_q / a.heads_kv;

  int q_start = 0, k_start = 0, Sq = a.seqlen_q, Sk = a.seqlen_k;
  if (a.varlen) {
    bounded_sequence(a.cu_q, b, a.total_q, &q_start, &Sq);
    bounded_sequence(a.cu_k, b, a.total_k, &k_start, &Sk);
  }
  // The dQ kernel launched behind this one needs none of its results: let its CTAs take over SMs as they free up.
  grid_launch_dependents();
  PROF_STAMP(3);
  if (a.compact) {
    const PackedTile pt = find_packed_tile<false>(a.cu_k, a.batch, a.total_k, 128, a.num_tiles, blockIdx.y);
    if (pt.seq < 0) return;
    b = pt.seq;
    ktile = pt.tile;
    hk = blockIdx.x;
    bounded_sequence(a.cu_q, b, a.total_q, &q_start, &Sq);
    bounded_sequence(a.cu_k, b, a.total_k, &k_start, &Sk);
  }
  const int k0 = ktile * 128;
  if (k0 >= Sk) return;
  const int tb = a.varlen ? 0 : b;

  // 128-query steps that can see this key tile; the mask geometry does not depend on the head
  ScoreMods mods = make_mods(a, b, hk * group, Sq, Sk);
  int ilo, ihi;
  query_range_for_keys(mods, k0, min(k0 + 127, Sk - 1), &ilo, &ihi);
  int slo = ilo / 128, shi = (ihi + 127) / 128;
  if (shi <= slo) slo = shi = 0;
  const int steps_per_head = shi - slo;
  const int n_total = steps_per_head * group;

  if (tid == 0) {
    mbar_init(k_full, 1);
    mbar_init(v_full, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 256);
    mbar_init(dp_full, 1);
    mbar_init(ds_full, 256);
    mbar_init(acc_done, 1);
    mbar_init(s_free, 256);
    for (int i = 0; i < kQS; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    for (int i = 0; i < kDS; ++i) {
      mbar_init(&do_full[i], 1);
      mbar_init(&do_empty[i], 1);
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
  constexpr uint32_t kColS = 0, kColDP = 128, kColDK = 256, kColDV = 256 + D;

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_total > 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_do);
      auto load_tile = [&](uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int row, int head) {
        mbar_arrive_expect_tx(bar, kTileBytes);
#pragma unroll
        for (int c = 0; c < kChunks; ++c) tma_load_4d(dst + c * 16384, map, bar, c * 64, row, head, tb);
      };
      load_tile(sK, &map_k, k_full, k_start + k0, hk);
      int h = hk * group, step = 0;
      for (int n = 0; n < n_total; ++n) {
        const int row = q_start + (slo + step) * 128;
        const int qs = n % kQS, ds = n % kDS;
        if (!mbar_wait(&q_empty[qs], ((n / kQS) & 1) ^ 1)) {
          report_timeout(a.status, 201);
          break;
        }
        load_tile(sQ + qs * kTileBytes, &map_q, &q_full[qs], row, h);
        if (n == 0) load_tile(sV, &map_v, v_full, k_start + k0, hk);
        if (!mbar_wait(&do_empty[ds], ((n / kDS) & 1) ^ 1)) {
          report_timeout(a.status, 207);
          break;
        }
        load_tile(sDo + ds * kTileBytes, &map_do, &do_full[ds], row, h);
        if (++step == steps_per_head) {
          step = 0;
          ++h;
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_total > 0) {
      constexpr uint32_t idesc_s = make_idesc(DType<T>::kFormat, 128, 128, 0, 0);
      constexpr uint32_t idesc_acc = make_idesc(DType<T>::kFormat, 128, D, 0, 1);
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), q_base = smem_u32(sQ), do_base = smem_u32(sDo);
      bool ok = true;
      PROF_DECL;
      auto wait_or_report = [&](uint64_t* bar, int parity, int code) {
        if (!ok) return;
        if (!mbar_wait(bar, parity)) {
          report_timeout(a.status, code);
          ok = false;
        }
      };
      auto scores = [&](uint32_t col, uint32_t a_addr, uint32_t b_addr) {  // [128 keys x 128 queries] = A B^T over D
        // descriptors as 32-bit halves: one add per operand and instruction (the issuing thread shares its scheduler
        // with compute warps, so its instruction count is tensor-pipe time)
        const uint32_t a_lo = smem_desc_lo(a_addr, 16), b_lo = smem_desc_lo(b_addr, 16);
        constexpr uint32_t hi = smem_desc_hi(1024);
        mma_ss_lo<0>(tmem_base + col, a_lo, hi, b_lo, hi, idesc_s);
#pragma unroll
        for (int kk = 1; kk < D / 16; ++kk) {
          const uint32_t o = ((kk / 4) * 16384 + (kk % 4) * 32) >> 4;
          mma_ss_lo<1>(tmem_base + col, a_lo + o, hi, b_lo + o, hi, idesc_s);
        }
      };
      auto accumulate = [&](uint32_t col_acc, uint32_t col_a, uint32_t b_addr, bool first) {  // += A^(tmem) B over queries
        // 16 queries per instruction; each group's operand sits in its own half
        const uint32_t b_lo = smem_desc_lo(b_addr, 16384);
        constexpr uint32_t hi = smem_desc_hi(1024);
        if (first) mma_ts_lo<0>(tmem_base + col_acc, tmem_base + col_a, b_lo, hi, idesc_acc);
        else mma_ts_lo<1>(tmem_base + col_acc, tmem_base + col_a, b_lo, hi, idesc_acc);
#pragma unroll
        for (int kk = 1; kk < 8; ++kk)
          mma_ts_lo<1>(tmem_base + col_acc, tmem_base + col_a + (kk / 4) * 64 + (kk % 4) * 8, b_lo + kk * (2048 >> 4), hi,
                       idesc_acc);
      };

      wait_or_report(k_full, 0, 202);
      wait_or_report(&q_full[0], 0, 203);
      if (ok) {
        tc_fence_after_sync();
        scores(kColS, k_addr, q_base);
        tc_commit(s_full);
      }
      wait_or_report(v_full, 0, 202);
      wait_or_report(&do_full[0], 0, 203);
      if (ok) {
        tc_fence_after_sync();
        scores(kColDP, v_addr, do_base);
        tc_commit(dp_full);
      }
      PROF_MARK(0);
      for (int n = 0; n < n_total && ok; ++n) {
        const int qs = n % kQS, ds = n % kDS;
        const int qs1 = (n + 1) % kQS, ds1 = (n + 1) % kDS;
        const bool more = n + 1 < n_total;
        // Plain path: P^T and dS^T both sit in the dP^T columns (the first and the second 32 of each group's 64), so
        // the S^T columns are free as soon as the compute warps hold step n's scores in registers and the next
        // scores are formed during phase 1 instead of behind dV. Modified scores: P^T stays in its S^T columns.
        constexpr uint32_t kColP = kMods ? kColS : kColDP, kColDs = kMods ? kColDP : kColDP + 32;
        // the next step's tiles were requested steps ago: ask for both now, look at the answers when they are needed
        const bool q_there = more && mbar_test(&q_full[qs1], ((n + 1) / kQS) & 1);
        const bool do_there = more && mbar_test(&do_full[ds1], ((n + 1) / kDS) & 1);
        if (!kMods && more) {
          wait_or_report(s_free, n & 1, 210);
          if (!q_there) wait_or_report(&q_full[qs1], ((n + 1) / kQS) & 1, 203);
          PROF_MARK(3);
          if (!ok) break;
          tc_fence_after_sync();
          scores(kColS, k_addr, q_base + qs1 * kTileBytes);
          tc_commit(s_full);
          PROF_MARK(2);
        }
        wait_or_report(p_full, n & 1, 204);
        PROF_MARK(1);
        if (!ok) break;
        tc_fence_after_sync();
        accumulate(kColDV, kColP, do_base + ds * kTileBytes, n == 0);
        tc_commit(&do_empty[ds]);
        PROF_MARK(2);
        if (kMods && more) {
          if (!q_there) wait_or_report(&q_full[qs1], ((n + 1) / kQS) & 1, 203);
          PROF_MARK(3);
          if (!ok) break;
          tc_fence_after_sync();
          scores(kColS, k_addr, q_base + qs1 * kTileBytes);
          tc_commit(s_full);
          PROF_MARK(2);
        }
        wait_or_report(ds_full, n & 1, 208);
        PROF_MARK(4);
        if (!ok) break;
        tc_fence_after_sync();
        accumulate(kColDK, kColDs, q_base + qs * kTileBytes, n == 0);
        tc_commit(&q_empty[qs]);
        PROF_MARK(2);
        if (more) {
          if (!do_there) wait_or_report(&do_full[ds1], ((n + 1) / kDS) & 1, 203);
          PROF_MARK(3);
          if (!ok) break;
          tc_fence_after_sync();
          scores(kColDP, v_addr, do_base + ds1 * kTileBytes);
          tc_commit(dp_full);
          PROF_MARK(2);
        }
      }
      if (ok) tc_commit(acc_done);
      PROF_FLUSH(2, true);
    }
  } else {
    // ------------------------------------------------------------------ compute warps
    // thread = one key row (TMEM lane); group wg owns query columns [64 wg, 64 wg + 64) of every step
    const int wg = warp / 4, w4 = warp % 4;
    const int key_row = w4 * 32 + lane;
    const int j = k0 + key_row;
    const uint32_t lane_addr = static_cast<uint32_t>(w4 * 32) << 16;
    const uint32_t tS = tmem_base + lane_addr + kColS + wg * 64;
    const uint32_t tDP = tmem_base + lane_addr + kColDP + wg * 64;
    const int off = Sk - Sq;
    const int64_t bo = a.varlen ? 0 : (int64_t)b;
    bool ok = true;
    PROF_DECL;
    // threads 0-127 fetch -lse*log2(e) (-inf = contributes nothing), threads 128-255 fetch -delta, of query tid & 127.
    // Head and step are carried along instead of divided out of n, and the address is kept as a pointer: with two
    // compute warps per scheduler a chain of dependent integer instructions costs its full latency every step.
    const bool is_lse = tid < 128;
    const int64_t st_sh = is_lse ? a.l_sh : a.d_sh, st_ss = is_lse ? a.l_ss : a.d_ss;
    const int f_i0 = slo * 128 + (tid & 127);
    const float* f_head = (is_lse ? a.lse + bo * a.l_sb : a.delta + bo * a.d_sb) + (int64_t)(hk * group) * st_sh +
                          (int64_t)(q_start + f_i0) * st_ss;
    const float* f_ptr = f_head;
    int f_i = f_i0, f_step = 0;
    // The raw value is returned and only converted when it is published a step later: anything computed from it here
    // would wait for the load, a trip to L2, in every step.
    auto fetch_row_stat = [&]() {  // the next step's value; advances the position
      float val = is_lse ? kNegInf : 0.f;
      if (f_i < Sq) val = *f_ptr;
      if (++f_step == steps_per_head) {
        f_step = 0;
        f_head += st_sh;
        f_ptr = f_head;
        f_i = f_i0;
      } else {
        f_ptr += 128 * st_ss;
        f_i += 128;
      }
      return val;
    };
    // Launched behind the delta kernel with the programmatic attribute, this CTA may be running before that kernel has
    // finished: everything so far (and the loads of K, V, Q, dO and the first scores, which other warps are at) needs
    // nothing of it; delta is first read here. (Without that kind of launch the wait returns at once.)
    if (a.after_delta && !is_lse) grid_dependency_wait();
    float staged = n_total > 0 ? fetch_row_stat() : 0.f;
    const int64_t ds_head_stride = (int64_t)a.ds_kt * a.ds_qt * 32768;
    uint8_t* ds_head = a.ds_ws == nullptr
                           ? nullptr
                           : reinterpret_cast<uint8_t*>(a.ds_ws) +
                                 (((int64_t)b * a.heads_q + hk * group) * a.ds_kt + ktile) * a.ds_qt * 32768 +
                                 wg * 8 * 2048 + key_row * 16;
    int h = hk * group, step = 0;

    for (int n = 0; n < n_total; ++n) {
      const int q0 = (slo + step) * 128;
      const int par = n & 1;
      if (kMods) mods = make_mods(a, b, h, Sq, Sk);
      // publish -lse*log2(e) / -delta of this step's 128 queries (fetched one step ahead), then fetch the next
      // (two sets in turn: a thread may still be reading step n - 1's values; nobody is behind that, because everybody
      // passed the barrier of step n - 1)
      float* nlse_s = stage_s + (n & 1) * 256;  // nlse_s[0,128) then ndelta_s[0,128)
      float* ndelta_s = nlse_s + 128;
      nlse_s[tid] = is_lse ? ((staged == kNegInf) ? kNegInf : -staged * kLog2e) : -staged;
      compute_sync();
      if (n + 1 < n_total) staged = fetch_row_stat();
      PROF_MARK(6);
      bool w_ok = mbar_wait(s_full, par);
      if (kMods) w_ok = mbar_wait(dp_full, par) && w_ok;
      if (!__all_sync(kFull, w_ok)) {
        report_timeout(a.status, 205);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      PROF_MARK(0);

      // queries this key row keeps: one interval [c_lo, c_hi] of the step's 128 columns
      const bool masked = block_needs_mask(mods, q0, 128, k0, 128);
      int c_lo = 0, c_hi = 127;
      if (masked) {
        if (a.causal) c_lo = max(c_lo, j - off - q0);
        else if (a.wr >= 0) c_lo = max(c_lo, j - off - a.wr - q0);
        if (a.wl >= 0) c_hi = min(c_hi, j - off + a.wl - q0);
        if (j >= Sk) c_hi = -1;
      }
      const uint64_t sc2 = pack_f32x2(mods.scale_log2, mods.scale_log2);
      // this thread's key row in the first of its eight query blocks of the step's dS^T tile, if there is a workspace
      uint8_t* ds_row = ds_head == nullptr ? nullptr : ds_head + (int64_t)(slo + step) * 32768;
      if (++step == steps_per_head) {  // for the next iteration
        step = 0;
        ++h;
        if (ds_head != nullptr) ds_head += ds_head_stride;
      }

      if (!kMods) {
        // ---- phase 1: P^T = exp2(S^T * c - lse[q]) in registers; the S^T columns go back to the MMA thread at once
        uint32_t pk[32];
        {
          uint32_t s0[32], s1[32];
          tmem_ld32(tS, s0);
          tmem_ld32(tS + 32, s1);
          tc_wait_ld_regs(s0);
          tc_wait_ld_regs(s1);
          tc_fence_before_sync();
          mbar_arrive(s_free);
          const float* nl = nlse_s + wg * 64;
          if (masked) probs_chunk<T, true>(s0, nl, sc2, wg * 64, c_lo, c_hi, &pk[0]);
          else probs_chunk<T, false>(s0, nl, sc2, wg * 64, c_lo, c_hi, &pk[0]);
          if (masked) probs_chunk<T, true>(s1, nl + 32, sc2, wg * 64 + 32, c_lo, c_hi, &pk[16]);
          else probs_chunk<T, false>(s1, nl + 32, sc2, wg * 64 + 32, c_lo, c_hi, &pk[16]);
        }
        PROF_MARK(4);

        // ---- phase 2: dP^T into registers, then P^T (16-bit) over the first half of this group's dP^T columns and
        // dS^T = P^T * (dP^T - delta[q]) over the second half
        const bool d_ok = mbar_wait(dp_full, par);
        if (!__all_sync(kFull, d_ok)) {
          report_timeout(a.status, 209);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        PROF_MARK(1);
        uint32_t dsk0[16], dsk1[16];
        {
          uint32_t d0[32], d1[32];
          tmem_ld32(tDP, d0);
          tmem_ld32(tDP + 32, d1);
          tc_wait_ld_regs(d0);
          tc_wait_ld_regs(d1);
          tmem_st16(tDP, *reinterpret_cast<uint32_t(*)[16]>(&pk[0]));
          tmem_st16(tDP + 16, *reinterpret_cast<uint32_t(*)[16]>(&pk[16]));
          tc_wait_st();
          tc_fence_before_sync();
          mbar_arrive(p_full);
          const float* nd = ndelta_s + wg * 64;
          dscore_chunk<T>(d0, nd, &pk[0], dsk0);
          tmem_st16(tDP + 32, dsk0);
          dscore_chunk<T>(d1, nd + 32, &pk[16], dsk1);
          tmem_st16(tDP + 48, dsk1);
        }
        tc_wait_st();
        tc_fence_before_sync();
        mbar_arrive(ds_full);
        if (ds_row != nullptr) {  // behind the hand-over, so the stores are off the dP -> dS -> dK chain
          store_ds32(ds_row, dsk0);
          store_ds32(ds_row + 4 * 2048, dsk1);
        }
        PROF_MARK(5);
      } else {
        // ---- general path: both products at once, 32 columns per (rolled) pass
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t s[32], dp[32];
          tmem_ld32(tS + c * 32, s);
          tmem_ld32(tDP + c * 32, dp);
          tc_wait_ld_regs(s);
          tc_wait_ld_regs(dp);
          const int col0 = wg * 64 + c * 32;
          float(&x)[32] = *reinterpret_cast<float(*)[32]>(&s[0]);
          float(&gr)[32] = *reinterpret_cast<float(*)[32]>(&dp[0]);
          bwd_mods_chunk32<false>(mods, x, gr, nlse_s + col0, ndelta_s + col0, q0 + col0, j, c_lo - col0, c_hi - col0);
          uint32_t pkk[16], dsk[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            pkk[e] = DType<T>::pack2(x[2 * e], x[2 * e + 1]);
            dsk[e] = DType<T>::pack2(gr[2 * e], gr[2 * e + 1]);
          }
          tmem_st16(tS + c * 16, pkk);
          tmem_st16(tDP + c * 16, dsk);
          if (ds_row != nullptr) store_ds32(ds_row + c * 4 * 2048, dsk);
        }
        tc_wait_st();
        tc_fence_before_sync();
        mbar_arrive(p_full);
        mbar_arrive(ds_full);
      }
    }
    PROF_FLUSH(wg, lane == 0 && w4 == 0);

    // epilogue: group 0 writes dK (scaled), group 1 writes dV
    if (n_total > 0) {
      const bool w_ok = ok && mbar_wait(acc_done, 0);
      if (!__all_sync(kFull, w_ok)) {
        if (ok) report_timeout(a.status, 206);
        ok = false;
      }
    }
    if (ok) {
      tc_fence_after_sync();
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
          tc_wait_ld_regs(o);
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = 0u;
        }
        if (j < Sk) store_row_slice<T>(row_ptr + c * 32, o, sc, a.head_dim - c * 32);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem_base, 512);
  PROF_STAMP(7);
}

// =============================================================================================
// dQ
// =============================================================================================

// Shared-memory plan of the dQ kernel (all dynamic).
template <int D>
struct DqSmem {
  static constexpr int kChunks = D / 64;
  static constexpr int kTileBytes = kChunks * 16384;  // one 128-row operand tile
  static constexpr int kKStages = D == 128 ? 3 : 4;   // K lives from S of its step to dQ of the same step (two steps later)
  static constexpr int kVStages = D == 128 ? 2 : 3;
  static constexpr int kOffQ = 0;
  static constexpr int kOffDo = kTileBytes;
  static constexpr int kOffK = 2 * kTileBytes;
  static constexpr int kOffV = kOffK + kKStages * kTileBytes;
  static constexpr int kOffBars = kOffV + kVStages * kTileBytes;
  static constexpr int kNumBars = 9 + 2 * kKStages + 2 * kVStages;
  static constexpr int kOffTmemPtr = kOffBars + kNumBars * 8;
  static constexpr int kBytes = kOffTmemPtr + 8 + 1024;  // + slack to round the base up to 1024
  static_assert(kBytes <= 232448, "dQ shared memory plan exceeds one CTA's 227 KB");
};


// Persistent: gridDim.x CTAs (one per SM) each walk items snake_item(0), snake_item(1), ... Q and dO of the item stay
// in shared memory; K/V stream in 128-key steps through two rings. All pipeline counters (ring positions, score
// buffer parity) run on across items, so the producer prefetches the next item's operands and the MMA warp starts
// its score MMAs while the compute warps still write out dQ. One thread issues, per step i (g = global step):
//     dP(i+1) = dO V(i+1)^T       after the compute warps have read dP(i)
//     dQ    += dS(i) K(i)         dS(i) sits in score buffer g & 1
//     S(i+2)  = Q K(i+2)^T        into the same buffer, behind dQ(i) in the pipe
// so phase 1 of step i+1 (P from S, kept in registers) never waits and phase 2 (dS = P * (dP - delta), written over
// the score buffer) finds dP(i+1) ready. TMEM: S buffers [0,128) [128,256); dP [256,384); dQ [384,384+D).
template <typename T, int D, bool kMods>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
              const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
              const BwdArgs a) {
  using L = DqSmem<D>;
  constexpr int kChunks = L::kChunks;
  constexpr int kTileBytes = L::kTileBytes;
  constexpr int kKS = L::kKStages, kVS = L::kVStages;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::kOffQ;
  uint8_t* sDo = smem + L::kOffDo;
  uint8_t* sK = smem + L::kOffK;
  uint8_t* sV = smem + L::kOffV;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBars);
  uint64_t* qdo_full = bars + 0;
  uint64_t* qdo_empty = bars + 1;
  uint64_t* dp_full = bars + 2;
  uint64_t* acc_done = bars + 3;
  uint64_t* acc_free = bars + 4;
  uint64_t* s_full = bars + 5;   // [2]
  uint64_t* ds_full = bars + 7;  // [2]
  uint64_t* k_full = bars + 9;
  uint64_t* k_empty = k_full + kKS;
  uint64_t* v_full = k_empty + kKS;
  uint64_t* v_empty = v_full + kVS;
  uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(smem + L::kOffTmemPtr);

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int n_items = a.num_tiles * a.batch * a.heads_q;

  if (tid == 0) {
    mbar_init(qdo_full, 1);
    mbar_init(qdo_empty, 1);
    mbar_init(dp_full, 1);
    mbar_init(acc_done, 1);
    mbar_init(acc_free, 256);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&ds_full[i], 256);
    }
    for (int i = 0; i < kKS; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    for (int i = 0; i < kVS; ++i) {
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
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
  constexpr uint32_t kColS = 0, kColDP = 256, kColDQ = 384;

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      int g = 0;     // global step counter (ring positions)
      int used = 0;  // items that used the pipeline so far
      bool ok = true;
      for (int round = 0; ok; ++round) {
        const int w = snake_item(round, blockIdx.x, gridDim.x);
        if (w >= n_items) break;
        const DqItem it = dq_item(a, w);
        if (!it.valid || it.n_total == 0) continue;
        const int tb = a.varlen ? 0 : it.b;
        auto load_tile = [&](uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int row, int head) {
#pragma unroll
          for (int c = 0; c < kChunks; ++c) tma_load_4d(dst + c * 16384, map, bar, c * 64, row, head, tb);
        };
        for (int n = 0; n < it.n_total; ++n, ++g) {
          const int ks = g % kKS, vs = g % kVS;
          const int row = it.k_start + (it.slo + n) * 128;
          if (!mbar_wait(&k_empty[ks], ((g / kKS) & 1) ^ 1)) {
            report_timeout(a.status, 301);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&k_full[ks], kTileBytes);
          load_tile(sK + ks * kTileBytes, &map_k, &k_full[ks], row, it.hk);
          if (!mbar_wait(&v_empty[vs], ((g / kVS) & 1) ^ 1)) {
            report_timeout(a.status, 308);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&v_full[vs], kTileBytes);
          load_tile(sV + vs * kTileBytes, &map_v, &v_full[vs], row, it.hk);
          if (n == 0) {  // after the first K/V tiles, whose ring slots free up before the previous item's Q/dO do
            if (!mbar_wait(qdo_empty, (used & 1) ^ 1)) {
              report_timeout(a.status, 300);
              ok = false;
              break;
            }
            mbar_arrive_expect_tx(qdo_full, 2 * kTileBytes);
            load_tile(sQ, &map_q, qdo_full, it.q_start + it.q0, it.h);
            load_tile(sDo, &map_do, qdo_full, it.q_start + it.q0, it.h);
          }
        }
        ++used;
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(DType<T>::kFormat, 128, 128, 0, 0);
      constexpr uint32_t idesc_acc = make_idesc(DType<T>::kFormat, 128, D, 0, 1);
      const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sDo), k_base = smem_u32(sK), v_base = smem_u32(sV);
      int g0 = 0, used = 0;
      bool ok = true;
      PROF_DECL;
      auto wait_or_report = [&](uint64_t* bar, int parity, int code) {
        if (!ok) return;
        if (!mbar_wait(bar, parity)) {
          report_timeout(a.status, code);
          ok = false;
        }
      };
      auto scores = [&](uint32_t col, uint32_t a_addr, uint32_t b_addr) {  // [128 queries x 128 keys] = A B^T over D
        // descriptors as 32-bit halves: one add per operand and instruction (the issuing thread shares its scheduler
        // with compute warps, so its instruction count is tensor-pipe time)
        const uint32_t a_lo = smem_desc_lo(a_addr, 16), b_lo = smem_desc_lo(b_addr, 16);
        constexpr uint32_t hi = smem_desc_hi(1024);
        mma_ss_lo<0>(tmem_base + col, a_lo, hi, b_lo, hi, idesc_s);
#pragma unroll
        for (int kk = 1; kk < D / 16; ++kk) {
          const uint32_t o = ((kk / 4) * 16384 + (kk % 4) * 32) >> 4;
          mma_ss_lo<1>(tmem_base + col, a_lo + o, hi, b_lo + o, hi, idesc_s);
        }
      };
      auto issue_s = [&](int g) {  // S of global step g into score buffer g & 1
        wait_or_report(&k_full[g % kKS], (g / kKS) & 1, 303);
        if (!ok) return;
        tc_fence_after_sync();
        scores(kColS + (g & 1) * 128, q_addr, k_base + (g % kKS) * kTileBytes);
        tc_commit(&s_full[g & 1]);
      };
      auto issue_dp = [&](int g) {
        wait_or_report(&v_full[g % kVS], (g / kVS) & 1, 309);
        if (!ok) return;
        tc_fence_after_sync();
        scores(kColDP, do_addr, v_base + (g % kVS) * kTileBytes);
        tc_commit(dp_full);
        tc_commit(&v_empty[g % kVS]);
      };

      for (int round = 0; ok; ++round) {
        const int w = snake_item(round, blockIdx.x, gridDim.x);
        if (w >= n_items) break;
        const DqItem it = dq_item(a, w);
        if (!it.valid || it.n_total == 0) continue;
        const int n = it.n_total;
        PROF_MARK(5);
        wait_or_report(qdo_full, used & 1, 302);
        if (!ok) break;
        tc_fence_after_sync();
        issue_s(g0);
        issue_dp(g0);
        if (ok && n == 1) tc_commit(qdo_empty);  // every MMA that reads Q / dO is issued: they may be replaced
        if (n > 1) issue_s(g0 + 1);
        PROF_MARK(0);
        for (int i = 0; i < n && ok; ++i) {
          const int g = g0 + i;
          wait_or_report(&ds_full[g & 1], (g >> 1) & 1, 304);
          if (i == 0 && used > 0) wait_or_report(acc_free, (used - 1) & 1, 307);  // previous dQ has been read out
          PROF_MARK(1);
          if (!ok) break;
          tc_fence_after_sync();
          if (i + 1 < n) {
            issue_dp(g + 1);
            if (ok && i + 2 == n) tc_commit(qdo_empty);
            PROF_MARK(3);
          }
          if (!ok) break;
          const uint32_t kb = k_base + (g % kKS) * kTileBytes;
          {  // 16 keys per instruction; each compute group's dS sits in its own half
            const uint32_t kb_lo = smem_desc_lo(kb, 16384), ds_col = tmem_base + kColS + (g & 1) * 128;
            constexpr uint32_t hi = smem_desc_hi(1024);
            if (i == 0) mma_ts_lo<0>(tmem_base + kColDQ, ds_col, kb_lo, hi, idesc_acc);
            else mma_ts_lo<1>(tmem_base + kColDQ, ds_col, kb_lo, hi, idesc_acc);
#pragma unroll
            for (int kk = 1; kk < 8; ++kk)
              mma_ts_lo<1>(tmem_base + kColDQ, ds_col + (kk / 4) * 64 + (kk % 4) * 8, kb_lo + kk * (2048 >> 4), hi, idesc_acc);
          }
          tc_commit(&k_empty[g % kKS]);
          PROF_MARK(2);
          if (i + 2 < n) {
            issue_s(g + 2);
            PROF_MARK(4);
          }
        }
        if (ok) tc_commit(acc_done);
        g0 += n;
        ++used;
      }
      PROF_FLUSH(2, true);
    }
  } else {
    // ------------------------------------------------------------------ compute warps
    // thread = one query row (TMEM lane); group wg owns key columns [64 wg, 64 wg + 64) of every step
    const int wg = warp / 4, w4 = warp % 4;
    const int q_row = w4 * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(w4 * 32) << 16;
    const uint32_t tDP = tmem_base + lane_addr + kColDP + wg * 64;
    int g0 = 0, used = 0;
    bool ok = true;
    PROF_DECL;
    // -lse*log2(e) (-inf = the row contributes nothing) and -delta of this thread's query row of an item
    auto row_stats = [&](const DqItem& it, float& nlse2, float& ndelta) {
      const int i = it.q0 + q_row;
      const int64_t bo = a.varlen ? 0 : (int64_t)it.b;
      nlse2 = kNegInf;
      ndelta = 0.f;
      if (i < it.Sq) {
        const float l = a.lse[bo * a.l_sb + (int64_t)it.h * a.l_sh + (int64_t)(it.q_start + i) * a.l_ss];
        nlse2 = (l == kNegInf) ? kNegInf : -l * kLog2e;
        ndelta = -a.delta[bo * a.d_sb + (int64_t)it.h * a.d_sh + (int64_t)(it.q_start + i) * a.d_ss];
      }
    };
    float pre_nlse2 = kNegInf, pre_ndelta = 0.f;
    int pre_round = -1;

    for (int round = 0; ok; ++round) {
      const int w = snake_item(round, blockIdx.x, gridDim.x);
      if (w >= n_items) break;
      const DqItem it = dq_item(a, w);
      if (!it.valid) continue;
      const int i = it.q0 + q_row;
      const int64_t bo = a.varlen ? 0 : (int64_t)it.b;
      T* row_ptr = reinterpret_cast<T*>(a.dq) + bo * a.dq_sb + (int64_t)it.h * a.dq_sh + (int64_t)(it.q_start + i) * a.dq_ss;
      constexpr int kSlices = D / 32 / 2;  // each group writes half of the head dimension
      if (it.n_total == 0) {  // rows that see no key: dQ = 0
        if (i < it.Sq) {
          uint32_t z[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) z[e] = 0u;
#pragma unroll
          for (int cc = 0; cc < kSlices; ++cc) store_row_slice<T>(row_ptr + (wg * kSlices + cc) * 32, z, 0.f, a.head_dim - (wg * kSlices + cc) * 32);
        }
        continue;
      }
      const ScoreMods mods = make_mods(a, it.b, it.h, it.Sq, it.Sk);
      const int off = it.Sk - it.Sq;
      float nlse2 = pre_nlse2, ndelta = pre_ndelta;
      if (pre_round != round) row_stats(it, nlse2, ndelta);
      const uint64_t sc2 = pack_f32x2(mods.scale_log2, mods.scale_log2);
      const uint64_t nl2 = pack_f32x2(nlse2, nlse2), nd2 = pack_f32x2(ndelta, ndelta);
      PROF_MARK(6);

      for (int n = 0; n < it.n_total; ++n) {
        const int g = g0 + n;
        const int ks = (it.slo + n) * 128;
        const uint32_t tS = tmem_base + lane_addr + kColS + (g & 1) * 128 + wg * 64;
        bool w_ok = mbar_wait(&s_full[g & 1], (g >> 1) & 1);
        if (kMods) w_ok = mbar_wait(dp_full, g & 1) && w_ok;
        if (!__all_sync(kFull, w_ok)) {
          report_timeout(a.status, 305);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        PROF_MARK(0);
        // keys this query row keeps: one interval [c_lo, c_hi] of the step's 128 columns
        const bool masked = block_needs_mask(mods, it.q0, 128, ks, 128);
        int c_lo = 0, c_hi = 127;
        if (masked) {
          c_hi = min(c_hi, it.Sk - 1 - ks);
          if (a.causal) c_hi = min(c_hi, i + off - ks);
          else if (a.wr >= 0) c_hi = min(c_hi, i + off + a.wr - ks);
          if (a.wl >= 0) c_lo = max(0, i + off - a.wl - ks);
        }
        if (!kMods) {
          // ---- phase 1: P = exp2(S * c - lse[row]), kept in registers
          uint32_t p0[32], p1[32];
          tmem_ld32(tS, p0);
          tc_wait_ld_regs(p0);
          tmem_ld32(tS + 32, p1);  // in flight while the first half is processed
          if (masked) probs_inplace<true>(p0, sc2, nl2, wg * 64, c_lo, c_hi);
          else probs_inplace<false>(p0, sc2, nl2, wg * 64, c_lo, c_hi);
          tc_wait_ld_regs(p1);
          if (masked) probs_inplace<true>(p1, sc2, nl2, wg * 64 + 32, c_lo, c_hi);
          else probs_inplace<false>(p1, sc2, nl2, wg * 64 + 32, c_lo, c_hi);
          PROF_MARK(4);

          // ---- phase 2: dS = P * (dP - delta[row]) -> 16-bit, over the score buffer
          const bool d_ok = mbar_wait(dp_full, g & 1);
          if (!__all_sync(kFull, d_ok)) {
            report_timeout(a.status, 310);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          PROF_MARK(1);
          uint32_t d0[32], d1[32], dsk[16];
          tmem_ld32(tDP, d0);
          tc_wait_ld_regs(d0);
          tmem_ld32(tDP + 32, d1);
          dscore_row<T>(p0, d0, nd2, dsk);
          tmem_st16(tS, dsk);
          tc_wait_ld_regs(d1);
          dscore_row<T>(p1, d1, nd2, dsk);
          tmem_st16(tS + 16, dsk);
        } else {
          // ---- general path, 32 columns per (rolled) pass
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t sv[32], dp[32];
            tmem_ld32(tS + c * 32, sv);
            tmem_ld32(tDP + c * 32, dp);
            tc_wait_ld_regs(sv);
            tc_wait_ld_regs(dp);
            const int col0 = wg * 64 + c * 32;
            float(&x)[32] = *reinterpret_cast<float(*)[32]>(&sv[0]);
            float(&gr)[32] = *reinterpret_cast<float(*)[32]>(&dp[0]);
            bwd_mods_chunk32<true>(mods, x, gr, &nlse2, &ndelta, i, ks + col0, c_lo - col0, c_hi - col0);
            uint32_t dsk[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) dsk[e] = DType<T>::pack2(gr[2 * e], gr[2 * e + 1]);
            tmem_st16(tS + c * 16, dsk);
          }
        }
        tc_wait_st();
        tc_fence_before_sync();
        mbar_arrive(&ds_full[g & 1]);
        PROF_MARK(5);
      }
      if (!ok) break;

      {  // fetch the next item's row statistics now; the loads complete behind the epilogue
        const int w2 = snake_item(round + 1, blockIdx.x, gridDim.x);
        if (w2 < n_items) {
          const DqItem it2 = dq_item(a, w2);
          if (it2.valid && it2.n_total > 0) {
            row_stats(it2, pre_nlse2, pre_ndelta);
            pre_round = round + 1;
          }
        }
      }
      // epilogue of the item: dQ * softmax_scale -> global, then hand the accumulator back
      const bool w_ok = mbar_wait(acc_done, used & 1);
      if (!__all_sync(kFull, w_ok)) {
        report_timeout(a.status, 306);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      PROF_MARK(2);
#pragma unroll
      for (int cc = 0; cc < kSlices; ++cc) {
        const int c = wg * kSlices + cc;
        uint32_t o[32];
        tmem_ld32(tmem_base + lane_addr + kColDQ + c * 32, o);
        tc_wait_ld_regs(o);
        if (cc == kSlices - 1) {
          tc_fence_before_sync();
          mbar_arrive(acc_free);  // this thread's last read of dQ is in registers
        }
        if (i < it.Sq) store_row_slice<T>(row_ptr + c * 32, o, a.softmax_scale, a.head_dim - c * 32);
      }
      PROF_MARK(3);
      g0 += it.n_total;
      ++used;
    }
    PROF_FLUSH(wg, lane == 0 && w4 == 0);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem_base, 512);
  PROF_STAMP(7);
}

// =============================================================================================
// dQ from the dS workspace
// =============================================================================================
// dQ = dS K as one GEMM over the dS^T tiles the dK/dV kernel stored: no score or dP product is recomputed (8 MMAs per
// 128 x 128 tile pair instead of 24). Persistent CTAs walk 128-query tiles of one (batch, head), longest first; per
// key tile the producer brings the dS^T tile [key][query] (32 KB) and the K tile [key][d] into a ring, and the MMA
// thread accumulates dQ[query][d] += dS K with BOTH operands read across their rows (M and N are the contiguous
// directions). Two accumulators in TMEM alternate between items, so four epilogue warps write one tile out while the
// next one accumulates. HBM-bound: reads the workspace once.
//   warps 0-3   epilogue (thread = one query row = one TMEM lane)
//   warp  4     dS^T tile producer (one lane)    warp 5     MMA issuer (one lane)    warp 6     K tile producer (one lane)
// The dS^T tiles come from HBM (each is read once), the K tiles from L2: the two run through rings of their own, five
// tile slots and two K slots, so that four or five HBM requests of 32 KB are in flight per SM whatever the K ring does
// (with both in one three-stage ring the kernel was bound by the latency of two requests in flight: 3.6 TB/s).
constexpr int kGemmThreads = 224;

template <int D>
struct DqGemmSmem {
  static constexpr int kKBytes = (D / 64) * 16384;  // one 128-key K tile
  static constexpr int kTileSlots = 5;
  static constexpr int kKSlots = D == 128 ? 2 : 3;
  static constexpr int kOffK = kTileSlots * 32768;
  static constexpr int kBytes = kOffK + kKSlots * kKBytes + 1024;
};

template <typename T, int D>
__global__ void __launch_bounds__(kGemmThreads, 1)
bwd_dq_gemm_kernel(const __grid_constant__ CUtensorMap map_k, const BwdArgs a) {
  using L = DqGemmSmem<D>;
  constexpr int kTS = L::kTileSlots, kKS = L::kKSlots;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t t_full[kTS], t_empty[kTS], k_full[kKS], k_empty[kKS], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int n_items = a.num_tiles * a.batch * a.heads_q;
  constexpr uint32_t kCols = 2 * D;  // two accumulators

  if (tid == 0) {
    for (int i = 0; i < kTS; ++i) {
      mbar_init(&t_full[i], 1);
      mbar_init(&t_empty[i], 1);
    }
    for (int i = 0; i < kKS; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
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
  // Launched as a programmatic dependent of the dK/dV kernel, whose tiles it reads: everything above overlaps that
  // kernel's tail, everything below waits for it to have completed.
  grid_dependency_wait();

  if (warp == 4 || warp == 6) {
    if (lane == 0) {
      const bool tiles = warp == 4;  // this thread's ring: dS^T tiles or K tiles
      if (!tiles) tma_prefetch_desc(&map_k);
      int g = 0;  // ring entries issued so far
      bool ok = true;
      for (int round = 0; ok; ++round) {
        const int w = snake_item(round, blockIdx.x, gridDim.x);
        if (w >= n_items) break;
        const DqItem it = dq_item(a, w);
        if (!it.valid || it.n_total == 0) continue;
        const int64_t tile0 = (((int64_t)it.b * a.heads_q + it.h) * a.ds_kt) * a.ds_qt + it.q0 / 128;
        for (int n = 0; n < it.n_total; ++n, ++g) {
          const int kt = it.slo + n;
          if (tiles) {
            const int st = g % kTS;
            if (!mbar_wait(&t_empty[st], ((g / kTS) & 1) ^ 1)) {
              report_timeout(a.status, 501);
              ok = false;
              break;
            }
            mbar_arrive_expect_tx(&t_full[st], 32768);
            bulk_load_stream(smem + st * 32768, reinterpret_cast<const uint8_t*>(a.ds_ws) + (tile0 + (int64_t)kt * a.ds_qt) * 32768,
                             32768, &t_full[st]);
          } else {
            const int st = g % kKS;
            if (!mbar_wait(&k_empty[st], ((g / kKS) & 1) ^ 1)) {
              report_timeout(a.status, 505);
              ok = false;
              break;
            }
            uint8_t* dst = smem + L::kOffK + st * L::kKBytes;
            mbar_arrive_expect_tx(&k_full[st], L::kKBytes);
#pragma unroll
            for (int c = 0; c < D / 64; ++c)
              tma_load_4d(dst + c * 16384, &map_k, &k_full[st], c * 64, it.k_start + kt * 128, it.hk, it.b);
          }
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(DType<T>::kFormat, 128, D, 1, 1);  // both operands read across their rows
      constexpr uint32_t hi = smem_desc_hi(1024);
      // unswizzled operand read across its rows: the leading offset is the step between core matrices along the
      // contraction (8 keys on: 128 bytes), the stride offset the step along the rows (8 queries on: 2048 bytes)
      constexpr uint32_t kDsLbo = 128, kDsSbo = 2048;
      constexpr uint32_t hi_ds = smem_desc_hi_noswizzle(kDsSbo);
      const uint32_t base = smem_u32(smem);
      int g = 0, used = 0;
      bool ok = true;
      for (int round = 0; ok; ++round) {
        const int w = snake_item(round, blockIdx.x, gridDim.x);
        if (w >= n_items) break;
        const DqItem it = dq_item(a, w);
        if (!it.valid || it.n_total == 0) continue;
        const int buf = used & 1;
        if (!mbar_wait(&acc_empty[buf], ((used >> 1) & 1) ^ 1)) {  // the epilogue has read this accumulator out
          report_timeout(a.status, 502);
          break;
        }
        tc_fence_after_sync();
        for (int n = 0; n < it.n_total; ++n, ++g) {
          const int ts = g % kTS, ks = g % kKS;
          if (!mbar_wait(&t_full[ts], (g / kTS) & 1) || !mbar_wait(&k_full[ks], (g / kKS) & 1)) {
            report_timeout(a.status, 503);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          // dS^T: unswizzled core matrices; a step of 16 keys is 256 bytes. K: the TMA tile, as V in the forward.
          const uint32_t ds_lo = smem_desc_lo(base + ts * 32768, kDsLbo);
          const uint32_t k_lo = smem_desc_lo(base + L::kOffK + ks * L::kKBytes, 16384);
          if (n == 0) mma_ss_lo<0>(tmem_base + buf * D, ds_lo, hi_ds, k_lo, hi, idesc);
          else mma_ss_lo<1>(tmem_base + buf * D, ds_lo, hi_ds, k_lo, hi, idesc);
#pragma unroll
          for (int kk = 1; kk < 8; ++kk)  // 16 keys per instruction
            mma_ss_lo<1>(tmem_base + buf * D, ds_lo + kk * (256 >> 4), hi_ds, k_lo + kk * (2048 >> 4), hi, idesc);
          tc_commit(&t_empty[ts]);
          tc_commit(&k_empty[ks]);
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
      const DqItem it = dq_item(a, w);
      if (!it.valid) continue;
      const int i = it.q0 + r;
      T* row_ptr = reinterpret_cast<T*>(a.dq) + (a.varlen ? 0 : (int64_t)it.b * a.dq_sb) + (int64_t)it.h * a.dq_sh +
                   (int64_t)(it.q_start + i) * a.dq_ss;
      const int buf = used & 1;
      if (it.n_total > 0) {
        if (!__all_sync(kFull, mbar_wait(&acc_full[buf], (used >> 1) & 1))) {
          report_timeout(a.status, 504);
          break;
        }
        tc_fence_after_sync();
      }
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        if (it.n_total > 0) {
          tmem_ld32(tmem_base + lane_addr + buf * D + c * 32, o);
          tc_wait_ld_regs(o);
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = 0u;
        }
        if (i < it.Sq) store_row_slice<T>(row_ptr + c * 32, o, a.softmax_scale, a.head_dim - c * 32);
      }
      if (it.n_total > 0) {
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


template <typename T, int D, bool kMods>
int launch_typed(const fa_attn_params& p, const BwdArgs& a0, int parts, cudaStream_t stream) {
  const int rows_q = p.varlen ? p.total_q : p.seqlen_q;
  const int rows_k = p.varlen ? p.total_k : p.seqlen_k;
  const int nb = p.varlen ? 1 : p.batch;
  auto map_of = [&](CUtensorMap* m, const void* ptr, int rows, int heads, const int64_t* st, int box_rows) {
    return make_tile_map(m, ptr, p.dtype, p.head_dim, rows, heads, nb, st[2], st[1], st[0], box_rows);
  };
  cudaError_t e;
  BwdArgs a = a0;
  if (parts & FA_BWD_DKDV) {
    CUtensorMap mq, mk, mv, mdo;
    int rc = map_of(&mq, p.q, rows_q, p.heads_q, p.q_strides, 128);
    if (!rc) rc = map_of(&mk, p.k, rows_k, p.heads_kv, p.k_strides, 128);
    if (!rc) rc = map_of(&mv, p.v, rows_k, p.heads_kv, p.v_strides, 128);
    if (!rc) rc = map_of(&mdo, p.dout, rows_q, p.heads_q, p.do_strides, 128);
    if (rc) return rc;
    auto kern = bwd_dkdv_kernel<T, D, kMods>;
    constexpr int smem_dkdv = DkdvSmem<D>::kBytes;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dkdv);
    if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "backward smem opt-in failed: %s", cudaGetErrorString(e));
    a.num_tiles = (p.seqlen_k + 127) / 128;
    dim3 grid(p.batch * p.heads_kv, a.num_tiles);
    a.compact = (p.varlen && p.batch <= kPackedMaxSequences) ? 1 : 0;
    if (a.compact) grid = dim3(p.heads_kv, (p.total_k + 127) / 128 + p.batch);
    // Behind the delta kernel of the same call the CTAs may start as that kernel's CTAs leave their SMs (they wait
    // inside, where delta is first read) - unless the dQ kernel that follows is the recomputing one, which is itself
    // let loose early on the grounds that delta was complete before this kernel started.
    const bool early = (parts & FA_BWD_DELTA) && !((parts & FA_BWD_DQ) && a.ds_ws == nullptr);
    a.after_delta = early ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kBwdThreads);
    cfg.dynamicSmemBytes = smem_dkdv;
    cfg.stream = stream;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    if (early) {
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
    }
    e = cudaLaunchKernelEx(&cfg, kern, mq, mk, mv, mdo, a);
    a.compact = 0;  // the dQ kernels walk their own item list
    a.after_delta = 0;
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "dK/dV launch failed: %s", cudaGetErrorString(e));
  }
  if ((parts & FA_BWD_DQ) && a.ds_ws != nullptr) {
    // the dK/dV kernel of this (or of an earlier) call left every dS^T tile in the workspace: dQ is one GEMM over them
    CUtensorMap mk;
    int rc = map_of(&mk, p.k, rows_k, p.heads_kv, p.k_strides, 128);
    if (rc) return rc;
    auto kern = bwd_dq_gemm_kernel<T, D>;
    constexpr int smem_gemm = DqGemmSmem<D>::kBytes;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_gemm);
    if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "backward smem opt-in failed: %s", cudaGetErrorString(e));
    a.num_tiles = (p.seqlen_q + 127) / 128;
    const int n_items = a.num_tiles * p.batch * p.heads_q;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_items < sm_count() ? n_items : sm_count());
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = smem_gemm;
    cfg.stream = stream;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    if (parts & FA_BWD_DKDV) {  // its CTAs may set themselves up while the last dK/dV CTAs drain (they wait inside)
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
    }
    e = cudaLaunchKernelEx(&cfg, kern, mk, a);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "dQ (workspace) launch failed: %s", cudaGetErrorString(e));
  } else if (parts & FA_BWD_DQ) {
    CUtensorMap mq, mk, mv, mdo;
    int rc = map_of(&mq, p.q, rows_q, p.heads_q, p.q_strides, 128);
    if (!rc) rc = map_of(&mk, p.k, rows_k, p.heads_kv, p.k_strides, 128);
    if (!rc) rc = map_of(&mv, p.v, rows_k, p.heads_kv, p.v_strides, 128);
    if (!rc) rc = map_of(&mdo, p.dout, rows_q, p.heads_q, p.do_strides, 128);
    if (rc) return rc;
    auto kern = bwd_dq_kernel<T, D, kMods>;
    constexpr int smem_dq = DqSmem<D>::kBytes;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dq);
    if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "backward smem opt-in failed: %s", cudaGetErrorString(e));
    a.num_tiles = (p.seqlen_q + 127) / 128;
    const int n_items = a.num_tiles * p.batch * p.heads_q;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_items < sm_count() ? n_items : sm_count());
    cfg.blockDim = dim3(kBwdThreads);
    cfg.dynamicSmemBytes = smem_dq;
    cfg.stream = stream;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    if (parts & FA_BWD_DKDV) {
      // dQ reads nothing the dK/dV kernel writes, and that kernel started only after delta was complete: its CTAs
      // may begin while the last dK/dV CTAs drain.
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
    }
    e = cudaLaunchKernelEx(&cfg, kern, mq, mk, mv, mdo, a);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "dQ launch failed: %s", cudaGetErrorString(e));
  }
  return 0;
}

}  // namespace

PROF_DEFINE_READER(fa_debug_read_prof_bwd)

bool bwd_tcgen05_supported(const fa_attn_params& p) {
  if (p.dtype != FA_F16 && p.dtype != FA_BF16) return false;
  if (p.head_dim < 8 || p.head_dim > 128 || p.head_dim % 8) return false;  // narrower rows are zero-filled by TMA
  const int64_t nb = p.varlen ? 1 : p.batch;
  const int64_t sq[3] = {nb, p.heads_q, p.varlen ? p.total_q : p.seqlen_q};
  const int64_t sk[3] = {nb, p.heads_kv, p.varlen ? p.total_k : p.seqlen_k};
  return tma_operand_ok(p.q, p.q_strides, sq) && tma_operand_ok(p.k, p.k_strides, sk) &&
         tma_operand_ok(p.v, p.v_strides, sk) && tma_operand_ok(p.dout, p.do_strides, sq) &&
         tma_operand_ok(p.dq, p.dq_strides, sq) && tma_operand_ok(p.dk, p.dk_strides, sk) &&
         tma_operand_ok(p.dv, p.dv_strides, sk);
}

// Bytes of the dS workspace for a dense problem: one 32 KB tile per (batch, query head, key tile, query tile). Zero
// for problems the workspace form does not take (packed sequences).
int64_t bwd_ds_workspace_bytes(const fa_attn_params& p) {
  if (p.varlen) return 0;
  const int64_t tiles = (int64_t)p.batch * p.heads_q * ((p.seqlen_k + 127) / 128) * ((p.seqlen_q + 127) / 128);
  return tiles * 32768;
}

int launch_bwd_tcgen05(const fa_attn_params& p, int parts, cudaStream_t stream) {
  BwdArgs a = {};
  a.varlen = p.varlen;
  a.batch = p.batch;
  a.heads_q = p.heads_q;
  a.head_dim = p.head_dim;
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
  a.num_tiles = 0;
  a.status = p.status;
  a.ds_ws = nullptr;
  a.ds_kt = (p.seqlen_k + 127) / 128;
  a.ds_qt = (p.seqlen_q + 127) / 128;
  if (p.ds_workspace != nullptr && !p.varlen) {
    const int64_t need = bwd_ds_workspace_bytes(p);
    if (p.ds_workspace_bytes < need)
      return set_error(FA_ERR_INVALID_ARGUMENT, "ds_workspace holds %lld bytes, this problem needs %lld",
                       (long long)p.ds_workspace_bytes, (long long)need);
    if (reinterpret_cast<uintptr_t>(p.ds_workspace) & 1023)
      return set_error(FA_ERR_INVALID_ARGUMENT, "ds_workspace must be aligned to 1024 bytes");
    a.ds_ws = p.ds_workspace;
  }
  const bool mods = p.softcap > 0.f || p.bias != nullptr || p.alibi_slopes != nullptr || p.dropout_p > 0.f;
  const bool f16 = p.dtype == FA_F16;
  if (p.head_dim > 64) {
    if (f16)
      return mods ? launch_typed<__half, 128, true>(p, a, parts, stream)
                  : launch_typed<__half, 128, false>(p, a, parts, stream);
    return mods ? launch_typed<__nv_bfloat16, 128, true>(p, a, parts, stream)
                : launch_typed<__nv_bfloat16, 128, false>(p, a, parts, stream);
  }
  if (f16)
    return mods ? launch_typed<__half, 64, true>(p, a, parts, stream)
                : launch_typed<__half, 64, false>(p, a, parts, stream);
  return mods ? launch_typed<__nv_bfloat16, 64, true>(p, a, parts, stream)
              : launch_typed<__nv_bfloat16, 64, false>(p, a, parts, stream);
}

}  // namespace fa
