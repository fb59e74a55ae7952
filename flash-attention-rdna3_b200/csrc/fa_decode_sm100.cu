// Split-K decode (dense and paged KV) for sm_100a with TMA-fed tiles and tcgen05 MMAs.
//
// Decode is bound by reading K and V once from HBM. TMA moves whole 128-key tiles (or whole pages) into
// shared memory with no register or LSU traffic and keeps several tiles in flight per SM; the query
// rows that share a kv head (GQA group x seqlen_q, at most 128) are padded to one 128-row MMA tile, so
// scores and P.V for a tile cost two short bursts of tcgen05.mma whatever the group size, and grouped
// queries read K/V exactly once.
//
// One CTA = one contiguous range of 128-key tiles of one (batch, kv head). The range is dealt to two
// independent streams (even / odd tiles), each with its own softmax warpgroup, S and O accumulators in
// TMEM and K/V slots in shared memory, so one stream's softmax overlaps the other's MMAs and loads:
//   warps 0-3 / 4-7  softmax of stream 0 / 1 (thread = query row = TMEM lane; rows >= R idle along)
//   warp 8           TMA producer (one lane); paged: one box per page, looked up in the block table
//   warp 9           MMA issuer (one lane)
// Each stream ends with a normalised fp32 partial and a natural-log LSE (-inf when it saw no key), written
// as partial number 2 * blockIdx.x + stream; the LSE merge kernel combines all partials of a row.
//
// Paged safety (fa_rdna3/kernels/paged.py:37-63): context lengths are clamped to the table capacity;
// page ids outside the pool are never dereferenced (the TMA box is aimed past the pool and reads zeros);
// keys past the context are masked, and V rows past the context are never loaded (the last, ragged page
// is fetched token by token), so stale cache contents cannot reach the output.
#include "fa_common.cuh"
#include "fa_sm100.cuh"
#include "fa_tma_host.h"
#include "fa_prof.cuh"

#include <mutex>
#include <unordered_map>
#include <utility>

namespace fa {

int launch_combine_internal(int rows, int D, int splits, const float* o_partial, int64_t o_split_stride,
                            int64_t o_row_stride, const float* lse_partial, int64_t lse_split_stride,
                            int64_t lse_row_stride, void* out, int out_dtype, int n1, int n2, int64_t os0,
                            int64_t os1, int64_t os2, int64_t osd, float* lse_out, cudaStream_t stream,
                            bool dependent);

namespace {

constexpr int kThreads = 320;
constexpr uint32_t kFull = 0xffffffffu;
constexpr float kRescaleThreshold = 8.0f;

struct DecArgs {
  int paged;
  int batch, heads_q, heads_kv, group, seqlen_q, rows;  // rows = query rows sharing a kv head
  int seqlen_k;                                         // dense
  // paged
  int block_size, max_blocks, num_blocks, first_block, block_step;
  int tpt;  // tokens per unit: a unit is tpt consecutive tokens of one page, all kv heads (tpt * heads_kv rows)
  int upp;  // units per page  = block_size / tpt
  int upt;  // units per tile  = 128 / (tpt * heads_kv) when a page is one unit, else 1
  const int32_t* block_table;
  int64_t bt_sb, bt_sk;
  const int32_t* context_lens;
  int64_t cl_stride;
  float softmax_scale;
  int num_partials;  // partial slots per row: 2 * gridDim.x, or the caller's capacity when balanced
  int balanced;      // paged: gridDim.x CTAs are dealt to the sequences in proportion to their tile counts
  int spread;        // paged, 8 kv heads, 16 tokens per tile: query heads are spread over the four lane quarters (see below)
  float* o_partial;
  float* lse_partial;
  int* status;
  uint32_t poll_limit;  // polls before a barrier wait is declared lost (kWaitPollLimit unless a test shortens it)
  int skip_tile;        // test hook: the producer leaves out the loads of this tile of every CTA (-1: none)
  // dense, merge inside the kernel: the last CTA of a (batch, kv head) to finish combines that head's partials.
  // tickets == nullptr: the caller launches the merge kernel instead.
  unsigned int* tickets;  // dense: one word per (batch, kv head), zero between launches (atomicInc wraps it back);
                          // paged (balanced, cooperative launch): two words per sequence, arrivals and departures
  float* lse_out;         // paged merge inside the kernel: merged LSE per (batch, head), may be null
  void* out;
  int out_dtype;
  int64_t o_sb, o_sh, o_ss, o_sd;
};

__device__ __forceinline__ void report_timeout(int* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

template <int D>
__device__ __forceinline__ void rescale_o(uint32_t tO, float alpha) {
#pragma unroll
  for (int c = 0; c < D / 32; ++c) {
    uint32_t o[32];
    tmem_ld32(tO + c * 32, o);
    tc_wait_ld_regs(o);
#pragma unroll
    for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
    tmem_st32(tO + c * 32, o);
  }
  tc_wait_st();
}

// Paged decode, balanced mode: the grid is one row of CTAs (one per SM) and every CTA works out, from the context
// lengths alone, which sequence it serves: each sequence gets one CTA, the rest are dealt in proportion to the
// sequences' tile counts (never more than one CTA per two tiles, never more than the partial buffer has slots for).
// Every CTA computes the same table, so no host read-back of the context lengths and no second launch is needed.
// Returns false for a CTA that is left over. batch <= kBalancedMaxBatch and batch <= gridDim.x (checked on the host).
constexpr int kBalancedMaxBatch = 256;

__device__ __forceinline__ int paged_tiles_of(const DecArgs& a, int b, int* ctx_out, int* pages_out) {
  const int bs = a.block_size;
  int ctx = a.context_lens[(int64_t)b * a.cl_stride];
  ctx = (int)min((int64_t)max(ctx, 0), (int64_t)a.max_blocks * bs);
  const int nblk = (ctx + bs - 1) / bs;
  const int pages = (nblk > a.first_block) ? (nblk - a.first_block + a.block_step - 1) / a.block_step : 0;
  *ctx_out = ctx;
  *pages_out = pages;
  return (pages * a.upp + a.upt - 1) / a.upt;
}

// `scratch` is shared memory nobody uses yet (the tile ring), at least 4 * (2 * kBalancedMaxBatch + 4) bytes.
__device__ __forceinline__ bool balanced_assignment(const DecArgs& a, void* scratch, int* b_out, int* x_out, int* n_out) {
  long long& total_s = *reinterpret_cast<long long*>(scratch);
  int* tiles_s = reinterpret_cast<int*>(scratch) + 2;
  int* first_s = tiles_s + kBalancedMaxBatch;
  const int tid = threadIdx.x, G = gridDim.x, B = a.batch;
  if (tid < B) {
    int ctx, pages;
    tiles_s[tid] = paged_tiles_of(a, tid, &ctx, &pages);
  }
  __syncthreads();
  if (tid < 32) {
    long long t = 0;
    for (int i = tid; i < B; i += 32) t += tiles_s[i];
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (tid == 0) total_s = t;
  }
  __syncthreads();
  const long long T = total_s;
  const int spare = G - B;  // CTAs beyond the one every sequence gets
  if (tid < B) {
    const int tl = tiles_s[tid];
    int n = 1 + (T > 0 ? (int)((long long)spare * tl / T) : 0);
    n = min(n, max(1, tl / 2));
    n = min(n, max(1, a.num_partials / 2));
    tiles_s[tid] = n;  // from here on: CTAs of the sequence
  }
  __syncthreads();
  if (tid < 32) {  // exclusive prefix sums, eight sequences per lane
    const int per = (B + 31) / 32;
    int sum = 0;
    for (int i = tid * per; i < min(B, (tid + 1) * per); ++i) sum += tiles_s[i];
    int incl = sum;
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (tid >= o) incl += v;
    }
    int run = incl - sum;
    for (int i = tid * per; i < min(B, (tid + 1) * per); ++i) {
      first_s[i] = run;
      run += tiles_s[i];
    }
    if (tid == 31) first_s[B] = incl;
  }
  __syncthreads();
  const int c = blockIdx.x;
  const bool mine = c < first_s[B];
  int lo = 0, hi = B - 1;  // last sequence whose first CTA is <= c
  while (lo < hi) {
    const int mid = (lo + hi + 1) / 2;
    if (first_s[mid] <= c) lo = mid;
    else hi = mid - 1;
  }
  *b_out = lo;
  *x_out = c - first_s[lo];
  *n_out = tiles_s[lo];
  __syncthreads();  // the scratch goes back to its owner
  return mine;
}

// Spread mode of the paged kernel (8 kv heads, 16 tokens x 8 heads per tile, at most 4 query heads per kv head):
// column c of a score tile is (token c / 8, kv head c % 8), so a query row only wants every eighth column. With all
// query rows in the first lane quarter one warp walks 128 columns per row and masks 112 of them; instead the rows of
// kv heads 2w and 2w + 1 sit in lane quarter w (Q is loaded as four boxes), every softmax warp picks the 16 columns of
// each of its rows out of the tile (a switch on the row's kv head, two cases per warp, compile-time register indices)
// and works on those alone. pick<HK> takes the four columns of one 32-column chunk, place<HK> puts four probabilities
// back as 16-bit halves of an otherwise zero chunk of P.
template <int HK, int C>
__device__ __forceinline__ void pick_cols(const uint32_t (&r)[32], float (&x)[16]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) x[4 * C + j] = __uint_as_float(r[HK + 8 * j]);
}
template <typename T, int HK, int C>
__device__ __forceinline__ void place_cols(uint32_t (&pk)[16], const float (&p)[16]) {
#pragma unroll
  for (int j = 0; j < 4; ++j)
    pk[4 * j + HK / 2] = (HK & 1) ? DType<T>::pack2(0.f, p[4 * C + j]) : DType<T>::pack2(p[4 * C + j], 0.f);
}
// the two switches on the row's kv head, for chunk C of the tile
template <int C>
__device__ __forceinline__ void pick_chunk(int hk, const uint32_t (&r)[32], float (&x)[16]) {
  switch (hk) {
    case 0: pick_cols<0, C>(r, x); break;
    case 1: pick_cols<1, C>(r, x); break;
    case 2: pick_cols<2, C>(r, x); break;
    case 3: pick_cols<3, C>(r, x); break;
    case 4: pick_cols<4, C>(r, x); break;
    case 5: pick_cols<5, C>(r, x); break;
    case 6: pick_cols<6, C>(r, x); break;
    default: pick_cols<7, C>(r, x); break;
  }
}
template <typename T, int C>
__device__ __forceinline__ void place_chunk(int hk, uint32_t (&pk)[16], const float (&p)[16]) {
  switch (hk) {
    case 0: place_cols<T, 0, C>(pk, p); break;
    case 1: place_cols<T, 1, C>(pk, p); break;
    case 2: place_cols<T, 2, C>(pk, p); break;
    case 3: place_cols<T, 3, C>(pk, p); break;
    case 4: place_cols<T, 4, C>(pk, p); break;
    case 5: place_cols<T, 5, C>(pk, p); break;
    case 6: place_cols<T, 6, C>(pk, p); break;
    default: place_cols<T, 7, C>(pk, p); break;
  }
}

template <typename T, int D, bool kPaged>
__global__ void __launch_bounds__(kThreads, 1)
decode_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_v_row,
                 const DecArgs a) {
  constexpr int kChunks = D / 64;
  constexpr int kTileBytes = kChunks * 16384;
  // Head dim 256 ("wide", dense caches only): TMEM holds one 256-column O accumulator beside the two S buffers, so one
  // softmax group walks every tile (the S tile still alternates between the two buffers, which lets Q K^T of the next
  // tile run ahead) and the CTA emits one partial; K and V (64 KB each) take the two ring slots in turn.
  constexpr bool kWide = D > 128;
  static_assert(!(kWide && kPaged), "the paged kernel is not built for head dims above 128");
  constexpr int kSlots = kWide ? 2 : (D == 128) ? 6 : 10;  // ring of 128-key tiles: K_t, V_t, K_t+1, V_t+1, ...

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sRing = smem + kTileBytes;
  __shared__ uint64_t q_full, full[kSlots], empty[kSlots], s_full[2], p_full[2], o_ready[2];
  __shared__ uint32_t tmem_base_s;
  // paged: readable tokens of each unit of tile t, in entry t % 8. The producer is at most three tiles ahead of the
  // Q K^T products and a tile's softmax has read its entry before the product three tiles on is even issued, so eight
  // entries never hold two live tiles.
  __shared__ int nval_s[8][16];

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  // The merge kernel launched behind this one is set up while the last CTAs here drain; it waits for the whole grid.
  grid_launch_dependents();
  PROF_STAMP(3);
  auto wait = [&](uint64_t* bar, uint32_t parity) { return mbar_wait_limit(bar, parity, a.poll_limit); };
  // dense: one CTA row per (batch, kv head). paged: one per batch entry; a tile interleaves all kv heads
  // (row = token * heads_kv + head), which is how a page lies in memory, so a page is fetched with few large boxes.
  int b = kPaged ? blockIdx.y : blockIdx.y / a.heads_kv;
  const int hk = kPaged ? 0 : blockIdx.y % a.heads_kv;
  int cta_x = blockIdx.x, ctas_b = gridDim.x;  // this CTA's index among the CTAs of its (batch[, kv head]) row
  if (kPaged && a.balanced) {
    if (!balanced_assignment(a, sRing, &b, &cta_x, &ctas_b)) return;  // uniform: nothing allocated yet
  }

  // keys seen by this call, in local order, and this CTA's tile range
  int nkeys = a.seqlen_k, ctx = 0, nlocal_pages = 0, tiles_total;
  if (kPaged) {
    tiles_total = paged_tiles_of(a, b, &ctx, &nlocal_pages);
  } else {
    tiles_total = (nkeys + 127) / 128;
  }
  const int tiles_per_cta = (tiles_total + ctas_b - 1) / ctas_b;
  const int jlo = min(cta_x * tiles_per_cta, tiles_total);
  const int jhi = min(jlo + tiles_per_cta, tiles_total);
  const int ntiles = jhi - jlo;

  if (tid == 0) {
    mbar_init(&q_full, 1);
#pragma unroll
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 128);
      mbar_init(&o_ready[s], 1);
    }
    mbar_fence_init();
  }
  if (kPaged && jhi == tiles_total) {
    // V tiles (the odd slots: kSlots is even) may be read at rows no load ever wrote: tokens past the context in the
    // sequence's last tile. Only the CTA that owns that tile can meet them before full tiles have filled its slots:
    // it starts its V slots from zeros (every other CTA only ever reads rows a load of real, finite data wrote).
    static_assert(kSlots % 2 == 0, "K and V tiles must keep to their own slots");
    for (int i = tid; i < (kSlots / 2) * (kTileBytes / 16); i += kThreads) {
      const int slot = 2 * (i / (kTileBytes / 16)) + 1, w = i % (kTileBytes / 16);
      reinterpret_cast<uint4*>(sRing + slot * kTileBytes)[w] = make_uint4(0, 0, 0, 0);
    }
    fence_proxy_async_smem();
  }
  // paged: lane u < upt of the producer warp holds the page id and the token counts of unit u of a tile. The look-up is
  // split in two so that the table read never stalls the producer: `request` only issues the load of the raw id (for
  // the tile after the one being queued), `resolve` turns it into box coordinates an iteration later. The first
  // request is made here, so that its load runs behind the TMEM allocation and the barrier set-up.
  constexpr int kNoPage = -0x7fffffff;  // no page behind this unit (past the context, past this lane's units)
  auto request = [&](int t) -> int {
    int id = kNoPage;
    if (kPaged) {
      const int u = (jlo + t) * a.upt + lane;  // local unit index
      const int lp = u / a.upp;
      if (t < ntiles && lane < a.upt && lp < nlocal_pages)
        id = a.block_table[(int64_t)b * a.bt_sb + (int64_t)(a.first_block + lp * a.block_step) * a.bt_sk];
    }
    return id;
  };
  auto resolve = [&](int t, int id, int* phys_out, int* nvalid_out, int* tokoff_out) {
    int phys = a.num_blocks, nvalid = 0, tokoff = 0;
    if (kPaged && id != kNoPage) {
      const int u = (jlo + t) * a.upt + lane;
      const int lb = a.first_block + (u / a.upp) * a.block_step;
      tokoff = (u % a.upp) * a.tpt;
      nvalid = max(0, min(a.tpt, ctx - (lb * a.block_size + tokoff)));
      if (id >= 0 && id < a.num_blocks) phys = id;
      else nvalid = -nvalid;  // present but unreadable: box aimed past the pool reads zeros, keys masked
    }
    *phys_out = phys;
    *nvalid_out = nvalid;
    *tokoff_out = tokoff;
  };
  int id_next = kNoPage;
  if (kPaged && warp == 8 && ntiles > 0) id_next = request(0);
  if (warp == 9) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer (whole warp; lane 0 issues)
    if (ntiles > 0) {
      if (lane == 0) {
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        if (kPaged && a.spread) {
          // four boxes of 2 * group rows: the query heads of kv heads 2w, 2w + 1 to rows 32w... (the rows in between
          // stay as they are: their lanes never look at their scores and hand in zero probabilities)
          mbar_arrive_expect_tx(&q_full, 4 * 2 * a.group * 128 * kChunks);
          for (int w = 0; w < 4; ++w)
#pragma unroll
            for (int c = 0; c < kChunks; ++c)
              tma_load_4d(sQ + c * 16384 + w * 4096, &map_q, &q_full, c * 64, w * 2 * a.group, hk, b);
        } else {
          mbar_arrive_expect_tx(&q_full, kTileBytes);
#pragma unroll
          for (int c = 0; c < kChunks; ++c) tma_load_4d(sQ + c * 16384, &map_q, &q_full, c * 64, 0, hk, b);
        }
      }
      const int unit_rows_bytes = kPaged ? a.tpt * a.heads_kv * 128 : 0;
      // One unit per tile (a page of at least 128 rows, or exactly one): lane 0 does everything and the warp-wide
      // steps (vote, byte count, barriers between lanes) drop out; they cost more than the two boxes they serve.
      const bool single = kPaged && a.upt == 1;
      bool ok = true;
      PROF_DECL;
      for (int t = 0; t < ntiles && ok && (!single || lane == 0); ++t) {
        int phys, nvalid, tokoff;
        resolve(t, id_next, &phys, &nvalid, &tokoff);
        if (kPaged) id_next = request(t + 1);  // in flight while this tile is queued; not looked at before the next turn
        for (int which = 0; which < 2 && ok; ++which) {
          const int n = 2 * t + which, slot = n % kSlots;
          uint8_t* dst = sRing + slot * kTileBytes;
          bool w_ok = true;
          PROF_MARK(1);  // issuing
          if (lane == 0) w_ok = wait(&empty[slot], ((n / kSlots) & 1) ^ 1);
          if (!single) w_ok = __shfl_sync(kFull, w_ok, 0);
          PROF_MARK(0);  // waiting for a free slot
          if (!w_ok) {
            if (lane == 0) report_timeout(a.status, 401);
            ok = false;
            break;
          }
          if (t == a.skip_tile) continue;  // test hook: this tile never arrives, its consumers' waits run out
          if (!kPaged) {
            if (lane == 0) {
              mbar_arrive_expect_tx(&full[slot], kTileBytes);
#pragma unroll
              for (int c = 0; c < kChunks; ++c)
                tma_load_4d(dst + c * 16384, which == 0 ? &map_k : &map_v, &full[slot], c * 64, (jlo + t) * 128, hk, b);
            }
            continue;
          }
          // paged: bytes this tile delivers, token counts for the softmax groups, then the boxes
          PROF_MARK(2);  // from the slot wait to here (look-up of the next tile included)
          const int present = nvalid < 0 ? -nvalid : nvalid;  // tokens inside the context
          const int readable = nvalid > 0 ? nvalid : 0;       // ... that may be used
          int mybytes = (which == 0) ? (present > 0 ? a.tpt : 0) : present;
          mybytes *= a.heads_kv * 128 * kChunks;
          if (!single) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mybytes += __shfl_xor_sync(kFull, mybytes, o);
          }
          if (which == 0 && lane < 16) nval_s[t & 7][lane] = readable;
          if (!single) __syncwarp();
          if (lane == 0) mbar_arrive_expect_tx(&full[slot], (uint32_t)mybytes);
          if (!single) __syncwarp();
          PROF_MARK(3);  // byte count, token counts, expect_tx
          // every lane issues the boxes of its own unit, so the copies of a tile are queued in parallel
          if (lane < a.upt && present > 0) {
            uint8_t* udst = dst + lane * unit_rows_bytes;
            if (which == 0 || present == a.tpt) {
#pragma unroll
              for (int c = 0; c < kChunks; ++c)
                tma_load_4d(udst + c * 16384, which == 0 ? &map_k : &map_v, &full[slot], c * 64, 0, tokoff, phys);
            } else {
              for (int tok = 0; tok < present; ++tok)
#pragma unroll
                for (int c = 0; c < kChunks; ++c)
                  tma_load_4d(udst + c * 16384 + tok * a.heads_kv * 128, &map_v_row, &full[slot], c * 64, 0, tokoff + tok,
                              phys);
            }
          }
          if (!single) __syncwarp();
          PROF_MARK(4);  // queueing the boxes
        }
      }
      PROF_MARK(1);
      PROF_FLUSH(2, lane == 0);
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && ntiles > 0) {
      constexpr uint32_t idesc_qk = make_idesc(DType<T>::kFormat, 128, 128, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc(DType<T>::kFormat, 128, D, 0, 1);
      const uint32_t q_addr = smem_u32(sQ), ring_addr = smem_u32(sRing);
      bool ok = wait(&q_full, 0);
      if (!ok) report_timeout(a.status, 403);
      PROF_DECL;

      auto issue_qk = [&](int t) {  // tile t goes to stream t & 1
        const int n = 2 * t, slot = n % kSlots, s = t & 1;
        PROF_MARK(3);
        if (!wait(&full[slot], (n / kSlots) & 1)) {
          report_timeout(a.status, 404);
          ok = false;
          return;
        }
        PROF_MARK(0);  // waiting for a K tile
        tc_fence_after_sync();
        const uint32_t k_addr = ring_addr + slot * kTileBytes;
        {  // descriptors as 32-bit halves, one add per operand and instruction (this thread's issue slots are the
           // stream's latency)
          const uint32_t q_lo = smem_desc_lo(q_addr, 16), k_lo = smem_desc_lo(k_addr, 16);
          constexpr uint32_t hi = smem_desc_hi(1024);
          mma_ss_lo<0>(tmem_base + s * 128, q_lo, hi, k_lo, hi, idesc_qk);
#pragma unroll
          for (int kk = 1; kk < D / 16; ++kk) {
            const uint32_t off = ((kk / 4) * 16384 + (kk % 4) * 32) >> 4;
            mma_ss_lo<1>(tmem_base + s * 128, q_lo + off, hi, k_lo + off, hi, idesc_qk);
          }
        }
        tc_commit(&s_full[s]);
        tc_commit(&empty[slot]);
        PROF_MARK(1);  // issuing Q K^T
      };

      if (ok) issue_qk(0);
      if (ok && ntiles > 1) issue_qk(1);
      for (int t = 0; t < ntiles && ok; ++t) {
        const int n = 2 * t + 1, slot = n % kSlots, s = t & 1;
        PROF_MARK(3);
        if (!wait(&full[slot], (n / kSlots) & 1)) {
          report_timeout(a.status, 405);
          break;
        }
        PROF_MARK(4);  // waiting for a V tile
        if (!wait(&p_full[s], (t >> 1) & 1)) {
          report_timeout(a.status, 405);
          break;
        }
        PROF_MARK(2);  // waiting for P
        tc_fence_after_sync();
        const uint32_t v_addr = ring_addr + slot * kTileBytes;
        {
          const uint32_t v_lo = smem_desc_lo(v_addr, 16384), o_col = tmem_base + 256 + (kWide ? 0 : s * D);
          constexpr uint32_t hi = smem_desc_hi(1024);
          if (t < (kWide ? 1 : 2)) mma_ts_lo<0>(o_col, tmem_base + s * 128, v_lo, hi, idesc_pv);  // the stream's first tile
          else mma_ts_lo<1>(o_col, tmem_base + s * 128, v_lo, hi, idesc_pv);
#pragma unroll
          for (int kk = 1; kk < 8; ++kk)
            mma_ts_lo<1>(o_col, tmem_base + s * 128 + kk * 8, v_lo + kk * (2048 >> 4), hi, idesc_pv);
        }
        tc_commit(&o_ready[kWide ? 0 : s]);
        tc_commit(&empty[slot]);
        PROF_MARK(3);  // issuing P V
        if (t + 2 < ntiles) issue_qk(t + 2);
      }
      PROF_FLUSH(1, true);
    }
  } else {
    // ------------------------------------------------------------------ softmax of stream s
    const int s = warp / 4, w4 = warp % 4;
    const int row = w4 * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(w4 * 32) << 16;
    const uint32_t tS_own = tmem_base + lane_addr + s * 128;
    const uint32_t tO = tmem_base + lane_addr + 256 + (kWide ? 0 : s * D);
    const int n_mine = kWide ? (s == 0 ? ntiles : 0) : (ntiles + 1 - s) / 2;
    const bool spread = kPaged && a.spread;
    // warps whose 32 rows are all padding only keep the barriers moving (spread: every warp has rows)
    const bool warp_active = spread || w4 * 32 < a.rows;
    // spread: this lane's kv head and whether the lane holds a query row at all
    // (lanes without a row take the second head's case, so that a warp runs two cases of the switches, not eight)
    const int sp_hk = 2 * w4 + min(lane / max(a.group, 1), 1);
    const bool sp_row = spread && lane < 2 * a.group;
    const float scale_log2 = a.softmax_scale * kLog2e;
    float m_used = kNegInf, l = 0.f;
    bool ok = true;
    PROF_DECL;
    // paged: columns of this row's kv head when every token of the tile is readable
    uint32_t full_pat[4] = {0u, 0u, 0u, 0u};
    const int my_hk = kPaged ? min(row, a.heads_q - 1) / a.group : 0;
    if (kPaged) {
      for (int tok = 0; tok < a.upt * a.tpt; ++tok) {
        const int c = tok * a.heads_kv + my_hk;
#pragma unroll
        for (int w = 0; w < 4; ++w)
          if ((c >> 5) == w) full_pat[w] |= 1u << (c & 31);
      }
    }

    for (int i = 0; i < n_mine; ++i) {
      const int t = kWide ? i : 2 * i + s, j = jlo + t;
      const int sb = kWide ? (i & 1) : s;  // S buffer and its barriers
      const uint32_t tS = kWide ? tmem_base + lane_addr + sb * 128 : tS_own;
      PROF_MARK(5);
      bool w_ok = wait(&s_full[sb], kWide ? (i >> 1) & 1 : i & 1);
      PROF_MARK(0);  // waiting for S
      if (w_ok && i > 0) w_ok = wait(&o_ready[s], (i - 1) & 1);
      PROF_MARK(6);  // waiting for the previous P V
      if (!__all_sync(kFull, w_ok)) {
        report_timeout(a.status, 406);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      // validity of the tile's 128 columns for this row as a bit mask
      uint32_t vmask[4] = {kFull, kFull, kFull, kFull};
      int nv_first = 0;  // paged: readable tokens of the tile's first unit (all there is in spread mode)
      if (kPaged) {
        // column = (unit * tpt + token) * heads_kv + kv head: this row only sees the columns of its own kv head,
        // and of those only the readable tokens
        const int* nval = nval_s[t & 7];
        nv_first = nval[0];
        bool all_full = true;
        for (int u = 0; u < a.upt && !spread; ++u) all_full = all_full && (nval[u] == a.tpt);
#pragma unroll
        for (int w = 0; w < 4; ++w) vmask[w] = full_pat[w];
        if (!all_full) {
          vmask[0] = vmask[1] = vmask[2] = vmask[3] = 0u;
          for (int u = 0; u < a.upt; ++u) {
            const int nv = nval[u];
            for (int tok = 0; tok < nv; ++tok) {
              const int c = (u * a.tpt + tok) * a.heads_kv + my_hk;
#pragma unroll
              for (int w = 0; w < 4; ++w)
                if ((c >> 5) == w) vmask[w] |= 1u << (c & 31);
            }
          }
        }
      } else if (j * 128 + 128 > nkeys) {
        const int nv = nkeys - j * 128;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const int left = nv - w * 32;
          vmask[w] = left >= 32 ? kFull : (left <= 0 ? 0u : ((1u << left) - 1u));
        }
      }
      const bool masked = (vmask[0] & vmask[1] & vmask[2] & vmask[3]) != kFull;
      PROF_MARK(1);  // validity mask, slot release
      if (spread) {
        // the 16 scores of this row: column 8 * token + kv head of every chunk
        const int nv = nv_first;
        float x[16];
        {
          uint32_t r[32];
          tmem_ld32(tS, r);
          tc_wait_ld_regs(r);
          pick_chunk<0>(sp_hk, r, x);
          tmem_ld32(tS + 32, r);
          tc_wait_ld_regs(r);
          pick_chunk<1>(sp_hk, r, x);
          tmem_ld32(tS + 64, r);
          tc_wait_ld_regs(r);
          pick_chunk<2>(sp_hk, r, x);
          tmem_ld32(tS + 96, r);
          tc_wait_ld_regs(r);
          pick_chunk<3>(sp_hk, r, x);
        }
        float m_tile = kNegInf;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (!sp_row || j >= nv) x[j] = kNegInf;  // lanes without a row and tokens past the context
          m_tile = fmaxf(m_tile, x[j]);
        }
        PROF_MARK(2);
        m_tile *= scale_log2;  // softmax_scale > 0 on this path
        const float m_new = fmaxf(m_used, m_tile);
        const bool grow = m_new > m_used + kRescaleThreshold;
        if (__any_sync(kFull, grow)) {
          const float alpha = (m_new == kNegInf) ? 1.f : exp2f(m_used - m_new);
          l *= alpha;
          if (i > 0) rescale_o<D>(tO, alpha);
          m_used = m_new;
        }
        const float m_eff = (m_used == kNegInf) ? 0.f : m_used;
        PROF_MARK(3);
        float pr[16], sum = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          pr[j] = fast_exp2(x[j] * scale_log2 - m_eff);
          sum += pr[j];
        }
        l += sum;
        {
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) pk[e] = 0u;
          place_chunk<T, 0>(sp_hk, pk, pr);
          tmem_st16(tS, pk);
#pragma unroll
          for (int e = 0; e < 16; ++e) pk[e] = 0u;
          place_chunk<T, 1>(sp_hk, pk, pr);
          tmem_st16(tS + 16, pk);
#pragma unroll
          for (int e = 0; e < 16; ++e) pk[e] = 0u;
          place_chunk<T, 2>(sp_hk, pk, pr);
          tmem_st16(tS + 32, pk);
#pragma unroll
          for (int e = 0; e < 16; ++e) pk[e] = 0u;
          place_chunk<T, 3>(sp_hk, pk, pr);
          tmem_st16(tS + 48, pk);
        }
        tc_wait_st();
        PROF_MARK(4);
      } else if (warp_active) {
        // pass 1: row maximum
        float mx[4] = {kNegInf, kNegInf, kNegInf, kNegInf};
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t r[64];
          tmem_ld32(tS + half * 64, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
          tmem_ld32(tS + half * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
          tc_wait_ld_regs(*reinterpret_cast<uint32_t(*)[32]>(&r[0]));
          tc_wait_ld_regs(*reinterpret_cast<uint32_t(*)[32]>(&r[32]));
          if (masked) {
#pragma unroll
            for (int c = 0; c < 64; ++c)
              if (!((vmask[half * 2 + c / 32] >> (c & 31)) & 1u)) r[c] = __float_as_uint(kNegInf);
          }
#pragma unroll
          for (int c = 0; c < 64; c += 8)
#pragma unroll
            for (int u = 0; u < 4; ++u)
              mx[u] = fmax3(mx[u], __uint_as_float(r[c + 2 * u]), __uint_as_float(r[c + 2 * u + 1]));
        }
        float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        PROF_MARK(2);  // pass 1
        m_tile *= scale_log2;  // softmax_scale > 0 on this path
        const float m_new = fmaxf(m_used, m_tile);
        const bool grow = m_new > m_used + kRescaleThreshold;
        if (__any_sync(kFull, grow)) {
          const float alpha = (m_new == kNegInf) ? 1.f : exp2f(m_used - m_new);
          l *= alpha;
          if (i > 0) rescale_o<D>(tO, alpha);
          m_used = m_new;
        }
        const float m_eff = (m_used == kNegInf) ? 0.f : m_used;
        PROF_MARK(3);  // rescale

        // pass 2: p = exp2(s*scale - m), 32 columns at a time, P written over consumed S columns
        const uint64_t sc2 = pack_f32x2(scale_log2, scale_log2);
        const uint64_t nm2 = pack_f32x2(-m_eff, -m_eff);
        uint64_t acc2[4] = {0ull, 0ull, 0ull, 0ull};
        uint32_t rb[2][32];
        tmem_ld32(tS, rb[0]);
        tc_wait_ld_regs(rb[0]);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (c < 3) tmem_ld32(tS + (c + 1) * 32, rb[(c + 1) & 1]);
          uint32_t (&r)[32] = rb[c & 1];
          if (masked) {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (!((vmask[c] >> e) & 1u)) r[e] = __float_as_uint(kNegInf);
          }
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const uint64_t x2 = fma_f32x2(pack_u32x2(r[2 * e], r[2 * e + 1]), sc2, nm2);
            float x0, x1;
            unpack_f32x2(x2, &x0, &x1);
            const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
            acc2[e & 3] = add_f32x2(acc2[e & 3], pack_f32x2(p0, p1));
            pk[e] = DType<T>::pack2(p0, p1);
          }
          tmem_st16(tS + c * 16, pk);
          if (c < 3) tc_wait_ld_regs(rb[(c + 1) & 1]);
        }
        float s0, s1;
        unpack_f32x2(add_f32x2(add_f32x2(acc2[0], acc2[1]), add_f32x2(acc2[2], acc2[3])), &s0, &s1);
        l += s0 + s1;
        tc_wait_st();
        PROF_MARK(4);  // pass 2
      } else {
        // padding-only warp: P rows of its lanes must still be finite zeros for the MMA
        uint32_t z[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) z[e] = 0u;
        tmem_st32(tS, z);
        tmem_st32(tS + 32, z);
        tc_wait_st();
      }
      tc_fence_before_sync();
      mbar_arrive(&p_full[sb]);
    }

    PROF_MARK(5);
    PROF_FLUSH(0, s == 0 && w4 == 0 && lane == 0);
    // epilogue: normalised fp32 partial and LSE of this stream
    if (n_mine > 0) {
      const bool w_ok = ok && wait(&o_ready[s], (n_mine - 1) & 1);
      if (!__all_sync(kFull, w_ok)) {
        if (ok) report_timeout(a.status, 407);
        ok = false;
      }
    }
    if (warp_active && !(kWide && s == 1)) {
      tc_fence_after_sync();
      const int part = kWide ? cta_x : 2 * cta_x + s;
      const int g = row / a.seqlen_q, sq = row % a.seqlen_q;
      const int h = spread ? sp_hk * a.group + lane % a.group : (kPaged ? row : hk * a.group + g);
      const bool has_row = spread ? sp_row : row < a.rows;
      int64_t flat_o, flat_l;
      if (kPaged) {  // (batch, heads_q, partials, D) and (batch, heads_q, partials)
        flat_l = ((int64_t)b * a.heads_q + h) * a.num_partials + part;
        flat_o = flat_l * D;
      } else {       // (partials, batch, heads_q, seqlen_q, D) and (partials, batch, heads_q, seqlen_q)
        flat_l = (((int64_t)part * a.batch + b) * a.heads_q + h) * a.seqlen_q + sq;
        flat_o = flat_l * D;
      }
      // A stream that gave up on a wait hands in an empty partial (zeros, LSE = -inf), which the merge ignores;
      // the status word carries the failure.
      if (!ok) l = 0.f;
      const float l_safe = (l == 0.f) ? 1.f : l;
      const float inv = 1.f / l_safe;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        if (n_mine > 0 && ok) {
          tmem_ld32(tO + c * 32, o);
          tc_wait_ld_regs(o);
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = 0u;
        }
        if (has_row) {
          float4* dst = reinterpret_cast<float4*>(a.o_partial + flat_o + c * 32);
#pragma unroll
          for (int v = 0; v < 8; ++v)
            dst[v] = make_float4(__uint_as_float(o[4 * v]) * inv, __uint_as_float(o[4 * v + 1]) * inv,
                                 __uint_as_float(o[4 * v + 2]) * inv, __uint_as_float(o[4 * v + 3]) * inv);
        }
      }
      if (has_row) a.lse_partial[flat_l] = (l == 0.f) ? kNegInf : (m_used * kLn2 + logf(l));
    }
    if (!kPaged && a.tickets != nullptr) __threadfence();  // this thread's partial is visible before the ticket is taken
  }

  if (kPaged && a.balanced && cta_x == 0 && a.tickets == nullptr) {
    // the slots of this sequence that no CTA writes must not take part in the merge: LSE = -inf
    const int used = 2 * ctas_b, spare = a.num_partials - used;
    for (int i = tid; i < a.heads_q * spare; i += kThreads)
      a.lse_partial[((int64_t)b * a.heads_q + i / spare) * a.num_partials + used + i % spare] = kNegInf;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem_base, 512);
  PROF_STAMP(7);

  if (kPaged && a.tickets != nullptr) {
    // Merge inside the kernel, balanced mode under a cooperative launch (all CTAs are resident, so waiting for the
    // others is legitimate): a CTA announces its partials, waits - with a bound - until all ctas_b CTAs of its sequence
    // have done so, then merges the rows cta_x, cta_x + ctas_b, ... of the sequence (the LSE-weighted sum of
    // fa_rdna3/kernels/decode.py:101-122 over the 2 * ctas_b partials that were written). The last CTA to leave puts
    // the two counters back to zero; nobody can still be polling then, because a CTA only leaves after its wait ended.
    __shared__ int all_here;
    unsigned int* arrive = a.tickets + 2 * b;
    unsigned int* depart = arrive + 1;
    __threadfence();  // this thread's partial is visible device-wide before the CTA is counted
    __syncthreads();
    if (tid == 0) {
      atomicAdd(arrive, 1u);
      bool seen = false;
      for (uint32_t i = 0; i < a.poll_limit; ++i) {
        unsigned int v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(arrive) : "memory");
        if (v >= (unsigned int)ctas_b) {
          seen = true;
          break;
        }
        __nanosleep(100);
      }
      if (!seen) report_timeout(a.status, 408);
      all_here = seen ? 1 : 0;
    }
    __syncthreads();
    if (all_here) {
      const int P = 2 * ctas_b, lane4 = tid % 32, grp = tid / 32;  // ten groups of 32 lanes; a lane owns four columns
      float* w_s = reinterpret_cast<float*>(smem);                         // [P] weights (P <= 2 * 148)
      float* part_s = w_s + 320;                                           // [10]
      float4* red_s = reinterpret_cast<float4*>(smem + 2048);              // [10][32]
      for (int r = cta_x; r < a.heads_q; r += ctas_b) {
        const int64_t row0 = ((int64_t)b * a.heads_q + r) * a.num_partials;
        const float ls = tid < P ? __ldcg(a.lse_partial + row0 + tid) : kNegInf;
        float M = ls;
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(kFull, M, o));
        if (lane4 == 0) part_s[grp] = M;
        __syncthreads();
        M = lane4 < kThreads / 32 ? part_s[lane4] : kNegInf;
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(kFull, M, o));
        const float Ms = (M == kNegInf) ? 0.f : M;
        const float w = (ls == kNegInf) ? 0.f : expf(ls - Ms);
        if (tid < P) w_s[tid] = w;
        float den = w;
        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(kFull, den, o);
        __syncthreads();  // everyone has read part_s; the weights are in place
        if (lane4 == 0) part_s[grp] = den;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (lane4 < D / 4) {
          const float4* src = reinterpret_cast<const float4*>(a.o_partial + row0 * D) + lane4;
#pragma unroll 4
          for (int sp = grp; sp < P; sp += kThreads / 32) {
            const float ws = w_s[sp];
            if (ws == 0.f) continue;
            const float4 v = __ldcg(src + (int64_t)sp * (D / 4));
            acc.x += ws * v.x;
            acc.y += ws * v.y;
            acc.z += ws * v.z;
            acc.w += ws * v.w;
          }
        }
        red_s[grp * 32 + lane4] = acc;
        __syncthreads();
        float den_all = lane4 < kThreads / 32 ? part_s[lane4] : 0.f;
        for (int o = 16; o > 0; o >>= 1) den_all += __shfl_xor_sync(kFull, den_all, o);
        const float inv = 1.f / ((den_all == 0.f) ? 1.f : den_all);
        if (tid < D) {
          const float* col = reinterpret_cast<const float*>(red_s) + tid;  // element tid of every group's row
          float num = 0.f;
#pragma unroll
          for (int g2 = 0; g2 < kThreads / 32; ++g2) num += col[g2 * 128];
          store_from_float(a.out, (int64_t)b * a.o_sb + (int64_t)r * a.o_sh + (int64_t)tid * a.o_sd, a.out_dtype, num * inv);
        }
        if (tid == 0 && a.lse_out != nullptr)
          a.lse_out[(int64_t)b * a.heads_q + r] = (den_all == 0.f) ? kNegInf : (Ms + logf(den_all));
        __syncthreads();  // the staging arrays are free for the next row
      }
    }
    if (tid == 0 && atomicAdd(depart, 1u) == (unsigned int)ctas_b - 1u) {
      *arrive = 0u;
      *depart = 0u;
      __threadfence();
    }
  }

  if (!kPaged && a.tickets != nullptr) {
    // Merge inside the kernel: every CTA of this (batch, kv head) takes a ticket once its partials are written; the
    // one that draws the last ticket sees all of them and writes the output rows (the LSE-weighted sum of
    // fa_rdna3/kernels/decode.py:101-122). Nobody waits for anybody. atomicInc wraps the word back to zero.
    __shared__ int is_last;
    if (tid == 0) is_last = atomicInc(&a.tickets[blockIdx.y], gridDim.x - 1) == gridDim.x - 1;
    __syncthreads();
    if (is_last) {
      __threadfence();
      // The ring is idle by now: its first bytes hold the weights and the cross-group sums. Threads are spread over
      // (partial group, row, four columns) so that the partial reads of a small problem are all in flight at once.
      const int P = a.num_partials, n_items = a.rows * (D / 4);
      const int64_t split_rows = (int64_t)a.batch * a.heads_q * a.seqlen_q;  // rows of one partial
      float* w_s = reinterpret_cast<float*>(smem);               // [rows][P] LSE, then weight
      float* inv_s = w_s + a.rows * P;                            // [rows] 1 / sum of weights
      float4* red_s = reinterpret_cast<float4*>(smem + 16384);    // [groups][n_items]
      auto partial_row = [&](int r) {
        const int g = r / a.seqlen_q, sq = r % a.seqlen_q;
        return ((int64_t)b * a.heads_q + hk * a.group + g) * a.seqlen_q + sq;
      };
      for (int i = tid; i < a.rows * P; i += kThreads)
        w_s[i] = __ldcg(a.lse_partial + (i % P) * split_rows + partial_row(i / P));
      __syncthreads();
      for (int r = tid; r < a.rows; r += kThreads) {
        float M = kNegInf, den = 0.f;
        for (int sp = 0; sp < P; ++sp) M = fmaxf(M, w_s[r * P + sp]);
        const float Ms = (M == kNegInf) ? 0.f : M;
        for (int sp = 0; sp < P; ++sp) {
          const float ls = w_s[r * P + sp];
          const float w = (ls == kNegInf) ? 0.f : expf(ls - Ms);
          w_s[r * P + sp] = w;
          den += w;
        }
        inv_s[r] = 1.f / ((den == 0.f) ? 1.f : den);
      }
      __syncthreads();
      const int groups = n_items >= kThreads ? 1 : min(P, kThreads / n_items);
      for (int it0 = 0; it0 < n_items; it0 += kThreads) {  // one pass unless rows * D / 4 exceeds the CTA
        const int grp = groups == 1 ? 0 : tid / n_items;
        const int item = groups == 1 ? it0 + tid : tid % n_items;
        const bool mine = item < n_items && grp < groups;
        const int r = mine ? item / (D / 4) : 0, d4 = item % (D / 4);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (mine) {
          const float4* src = reinterpret_cast<const float4*>(a.o_partial + partial_row(r) * D) + d4;
#pragma unroll 4
          for (int sp = grp; sp < P; sp += groups) {
            const float w = w_s[r * P + sp];
            const float4 v = __ldcg(src + sp * split_rows * (D / 4));
            acc.x += w * v.x;
            acc.y += w * v.y;
            acc.z += w * v.z;
            acc.w += w * v.w;
          }
        }
        if (groups > 1) {
          if (mine) red_s[grp * n_items + item] = acc;
          __syncthreads();
          if (mine && grp == 0)
            for (int g2 = 1; g2 < groups; ++g2) {
              const float4 v = red_s[g2 * n_items + item];
              acc.x += v.x;
              acc.y += v.y;
              acc.z += v.z;
              acc.w += v.w;
            }
        }
        if (mine && grp == 0) {
          const float inv = inv_s[r];
          const int g = r / a.seqlen_q, sq = r % a.seqlen_q, h = hk * a.group + g;
          const int64_t obase =
              (int64_t)b * a.o_sb + (int64_t)h * a.o_sh + (int64_t)sq * a.o_ss + (int64_t)(d4 * 4) * a.o_sd;
          store_from_float(a.out, obase, a.out_dtype, acc.x * inv);
          store_from_float(a.out, obase + a.o_sd, a.out_dtype, acc.y * inv);
          store_from_float(a.out, obase + 2 * a.o_sd, a.out_dtype, acc.z * inv);
          store_from_float(a.out, obase + 3 * a.o_sd, a.out_dtype, acc.w * inv);
        }
      }
    }
  }
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Tensor map over a paged cache (dim, kv head, token in page, page) with a box of 64 x heads_kv x box_tokens x 1:
// box_tokens tokens of one page, all kv heads, land as rows token * heads_kv + head.
int make_page_map(CUtensorMap* map, const void* ptr, int dtype, int D, int heads_kv, int block_size, int num_blocks,
                  const int64_t st[4], int box_tokens) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (enc == nullptr) return set_error(FA_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)heads_kv, (cuuint64_t)block_size, (cuuint64_t)num_blocks};
  auto bytes = [&](int64_t s, int64_t n) { return (cuuint64_t)((n > 1 && s > 0) ? s : D) * 2; };
  const cuuint64_t strides[3] = {bytes(st[2], heads_kv), bytes(st[1], block_size), bytes(st[0], num_blocks)};
  const cuuint32_t box[4] = {64, (cuuint32_t)heads_kv, (cuuint32_t)box_tokens, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = (dtype == FA_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = enc(map, dt, 4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(FA_ERR_LAUNCH, "cuTensorMapEncodeTiled (paged cache) failed with code %d", (int)r);
  return 0;
}

constexpr int kCooperativeRefused = 1;  // launch_kernel: the cooperative launch was not accepted, nothing was launched

template <typename T, int D, bool kPaged>
int launch_kernel(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mvr,
                  const DecArgs& a, int ctas, cudaStream_t stream) {
  constexpr int kTileBytes = (D / 64) * 16384;
  constexpr int kSlots = D > 128 ? 2 : (D == 128) ? 6 : 10;
  const int smem = (1 + kSlots) * kTileBytes + 1024;
  auto kern = decode_tc_kernel<T, D, kPaged>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "decode smem opt-in failed: %s", cudaGetErrorString(e));
  const dim3 grid(ctas, kPaged ? (a.balanced ? 1 : a.batch) : a.batch * a.heads_kv);
  if (kPaged && a.tickets != nullptr) {
    // the CTAs of a sequence wait for one another before they merge: only under a launch that guarantees that all of
    // them are resident
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeCooperative;
    attr.val.cooperative = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kern, mq, mk, mv, mvr, a);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      return kCooperativeRefused;  // the caller launches the two-kernel form instead
    }
    return 0;
  }
  kern<<<grid, kThreads, smem, stream>>>(mq, mk, mv, mvr, a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "tcgen05 decode launch failed: %s", cudaGetErrorString(e));
  return 0;
}

template <bool kPaged>
int dispatch(int dtype, int D, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
             const CUtensorMap& mvr, const DecArgs& a, int ctas, cudaStream_t stream) {
  if (D == 256) {
    if constexpr (!kPaged) {
      return dtype == FA_F16 ? launch_kernel<__half, 256, false>(mq, mk, mv, mvr, a, ctas, stream)
                             : launch_kernel<__nv_bfloat16, 256, false>(mq, mk, mv, mvr, a, ctas, stream);
    } else {
      return set_error(FA_ERR_UNSUPPORTED, "paged tcgen05 decode takes head_dim 64 or 128");
    }
  }
  if (dtype == FA_F16)
    return D == 128 ? launch_kernel<__half, 128, kPaged>(mq, mk, mv, mvr, a, ctas, stream)
                    : launch_kernel<__half, 64, kPaged>(mq, mk, mv, mvr, a, ctas, stream);
  return D == 128 ? launch_kernel<__nv_bfloat16, 128, kPaged>(mq, mk, mv, mvr, a, ctas, stream)
                  : launch_kernel<__nv_bfloat16, 64, kPaged>(mq, mk, mv, mvr, a, ctas, stream);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Ticket words of the in-kernel merge: a fixed array inside the library image (zero when the module is loaded, and
// every finished launch leaves its words at zero again), so the library never allocates. Launches that may run at the
// same time (different streams) must not share words; such launches use different partial buffers, so each partial
// buffer address gets a region of its own, for good, of as many words as its problem needs (rounded up to 16): 256 KB
// serve some thousand buffers. Once the array is used up, further buffers simply keep the separate merge kernel.
// Regions are never handed to a second buffer, so a captured graph that holds a region pointer stays valid whatever
// runs later; a buffer that comes back with a larger problem gets a new, larger region.
constexpr int kTicketWordsTotal = 64 * 1024, kTicketWords = 1024, kTicketDevices = 64;
static __device__ __align__(256) unsigned int g_ticket_words[kTicketWordsTotal];

struct TicketTable {
  unsigned int* base = nullptr;  // device address of g_ticket_words in this device's context
  std::unordered_map<const void*, std::pair<int, int>> region;  // partial buffer -> (first word, words)
  int next = 0;
};
std::mutex g_ticket_mutex;
TicketTable g_ticket_table[kTicketDevices];

// `words` ticket words for this partial buffer on the current device, or nullptr (array used up, or its address is not
// known yet and cannot be asked for because the stream is being captured).
unsigned int* ticket_region(const void* partial_buffer, int words, bool capturing) {
  int dev = 0;
  if (words <= 0 || words > kTicketWords) return nullptr;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kTicketDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_ticket_mutex);
  TicketTable& tab = g_ticket_table[dev];
  if (tab.base == nullptr) {
    if (capturing) return nullptr;
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_ticket_words) != cudaSuccess || ptr == nullptr) {
      (void)cudaGetLastError();
      return nullptr;
    }
    tab.base = static_cast<unsigned int*>(ptr);
  }
  auto it = tab.region.find(partial_buffer);
  if (it != tab.region.end() && it->second.second >= words) return tab.base + it->second.first;
  const int take = (words + 15) & ~15;
  if (tab.next + take > kTicketWordsTotal) return nullptr;
  tab.region[partial_buffer] = std::make_pair(tab.next, take);
  unsigned int* out = tab.base + tab.next;
  tab.next += take;
  return out;
}

// Whether the current device takes cooperative launches (asked once per device).
bool cooperative_launch_ok() {
  static int cached[kTicketDevices] = {};  // 0 unknown, 1 yes, 2 no
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kTicketDevices) return false;
  if (cached[dev] == 0) {
    int v = 0;
    cached[dev] = (cudaDeviceGetAttribute(&v, cudaDevAttrCooperativeLaunch, dev) == cudaSuccess && v) ? 1 : 2;
  }
  return cached[dev] == 1;
}

// Test hook (fa_test_decode_fault): poll limit and tile to leave out for the next tensor-core decode launch of this
// thread; consumed by that launch.
thread_local uint32_t g_fault_poll_limit = 0;
thread_local int g_fault_skip_tile = -1;

void take_fault_injection(DecArgs* a) {
  a->poll_limit = g_fault_poll_limit ? g_fault_poll_limit : kWaitPollLimit;
  a->skip_tile = g_fault_skip_tile;
  g_fault_poll_limit = 0;
  g_fault_skip_tile = -1;
}

}  // namespace

// Dense split-K decode on the tcgen05 path. Head dims 64 and 128: num_splits must be even, each CTA produces two
// partials. Head dim 256: one partial per CTA, any num_splits >= 2.
bool decode_tc_supported(const fa_decode_params& p) {
  if (p.dtype != FA_F16 && p.dtype != FA_BF16) return false;
  if (p.head_dim != 64 && p.head_dim != 128 && p.head_dim != 256) return false;
  if (!(p.softmax_scale > 0.f)) return false;
  if (p.num_splits < 2 || p.o_partial == nullptr || p.lse_partial == nullptr) return false;
  if (p.head_dim != 256 && (p.num_splits & 1)) return false;
  if (p.heads_kv <= 0 || p.heads_q % p.heads_kv) return false;
  const int group = p.heads_q / p.heads_kv;
  if (group * p.seqlen_q > 128) return false;
  const int64_t sk[3] = {p.batch, p.heads_kv, p.seqlen_k};
  if (!tma_operand_ok(p.k, p.k_strides, sk) || !tma_operand_ok(p.v, p.v_strides, sk)) return false;
  // the query rows of one kv head must form one strided row sequence
  if (!aligned16(p.q) || p.q_strides[3] != 1) return false;
  if (p.seqlen_q > 1 && group > 1 && p.q_strides[1] != p.q_strides[2] * p.seqlen_q) return false;
  const int64_t row_stride = p.seqlen_q > 1 ? p.q_strides[2] : p.q_strides[1];
  if (group * p.seqlen_q > 1 && (row_stride <= 0 || row_stride % 8)) return false;
  if (p.heads_kv > 1 && ((p.q_strides[1] * group) % 8 || p.q_strides[1] <= 0)) return false;
  if (p.batch > 1 && (p.q_strides[0] % 8 || p.q_strides[0] <= 0)) return false;
  return true;
}

int launch_decode_tc(const fa_decode_params& p, cudaStream_t stream) {
  const int group = p.heads_q / p.heads_kv, rows = group * p.seqlen_q, D = p.head_dim;
  const int64_t row_stride = p.seqlen_q > 1 ? p.q_strides[2] : p.q_strides[1];
  CUtensorMap mq, mk, mv;
  int rc = make_tile_map(&mq, p.q, p.dtype, D, rows, p.heads_kv, p.batch, row_stride, p.q_strides[1] * group,
                         p.q_strides[0]);
  if (!rc) rc = make_tile_map(&mk, p.k, p.dtype, D, p.seqlen_k, p.heads_kv, p.batch, p.k_strides[2], p.k_strides[1],
                              p.k_strides[0]);
  if (!rc) rc = make_tile_map(&mv, p.v, p.dtype, D, p.seqlen_k, p.heads_kv, p.batch, p.v_strides[2], p.v_strides[1],
                              p.v_strides[0]);
  if (rc) return rc;
  DecArgs a = {};
  a.paged = 0;
  a.batch = p.batch;
  a.heads_q = p.heads_q;
  a.heads_kv = p.heads_kv;
  a.group = group;
  a.seqlen_q = p.seqlen_q;
  a.rows = rows;
  a.seqlen_k = p.seqlen_k;
  a.softmax_scale = p.softmax_scale;
  a.num_partials = p.num_splits;
  a.o_partial = p.o_partial;
  a.lse_partial = p.lse_partial;
  a.status = p.status;
  take_fault_injection(&a);
  // Small merges run inside the decode kernel (one launch instead of two); large ones (many rows x many partials
  // through one CTA) keep the merge kernel, which spreads the rows over the GPU.
  a.tickets = nullptr;
  if ((int64_t)rows * D * p.num_splits <= 65536 && (int64_t)p.batch * p.heads_kv <= kTicketWords && D % 4 == 0) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    const bool capturing = cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone;
    a.tickets = ticket_region(p.o_partial, p.batch * p.heads_kv, capturing);
  }
  a.out = p.out;
  a.out_dtype = p.dtype;
  a.o_sb = p.o_strides[0];
  a.o_sh = p.o_strides[1];
  a.o_ss = p.o_strides[2];
  a.o_sd = p.o_strides[3];
  rc = dispatch<false>(p.dtype, D, mq, mk, mv, mv, a, D == 256 ? p.num_splits : p.num_splits / 2, stream);
  if (rc) return rc;
  if (a.tickets != nullptr) return 0;
  const int nrows = p.batch * p.heads_q * p.seqlen_q;
  return launch_combine_internal(nrows, D, p.num_splits, p.o_partial, (int64_t)nrows * D, D, p.lse_partial, nrows, 1,
                                 p.out, p.dtype, p.heads_q, p.seqlen_q, p.o_strides[0], p.o_strides[1], p.o_strides[2],
                                 p.o_strides[3], nullptr, stream, true);
}

unsigned int* decode_ticket_words(const void* partial_buffer, int words, cudaStream_t stream) {
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  const bool capturing = cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone;
  return ticket_region(partial_buffer, words, capturing);
}

bool paged_tc_supported(const fa_paged_params& p) {
  if (p.dtype != FA_F16 && p.dtype != FA_BF16) return false;
  if (p.head_dim != 64 && p.head_dim != 128) return false;
  if (!(p.softmax_scale > 0.f)) return false;
  if (p.num_splits < 2 || (p.num_splits & 1) || p.o_partial == nullptr || p.lse_partial == nullptr) return false;
  if (p.heads_kv <= 0 || p.heads_q % p.heads_kv || p.heads_q > 128) return false;  // one MMA row per query head
  if (p.block_size < 1 || (p.block_size & (p.block_size - 1))) return false;
  if (p.heads_kv > 128 || (p.heads_kv & (p.heads_kv - 1))) return false;           // rows per token must divide 128
  if (p.block_size * p.heads_kv < 8) return false;                                  // at most 16 units per tile
  if (!aligned16(p.k_cache) || !aligned16(p.v_cache) || !aligned16(p.q)) return false;
  if (p.k_strides[3] != 1 || p.v_strides[3] != 1 || p.q_strides[2] != 1) return false;
  for (int i = 0; i < 3; ++i)
    if (p.k_strides[i] <= 0 || p.k_strides[i] % 8 || p.v_strides[i] <= 0 || p.v_strides[i] % 8) return false;
  const int group = p.heads_q / p.heads_kv;
  if (p.heads_q > 1 && (p.q_strides[1] <= 0 || p.q_strides[1] % 8)) return false;
  if (p.batch > 1 && (p.q_strides[0] <= 0 || p.q_strides[0] % 8)) return false;
  (void)group;
  return true;
}

int launch_paged_tc(const fa_paged_params& p, cudaStream_t stream) {
  const int group = p.heads_q / p.heads_kv, D = p.head_dim;
  CUtensorMap mq, mk, mv, mvr;
  // unit = tpt tokens of one page with all kv heads (tpt * heads_kv <= 128 rows); a tile holds upt units
  const int tpt = p.block_size * p.heads_kv <= 128 ? p.block_size : 128 / p.heads_kv;
  const int upp = p.block_size / tpt;
  const int upt = upp == 1 ? 128 / (tpt * p.heads_kv) : 1;
  // spread mode (see pick_cols): 8 kv heads, a tile of 16 tokens x 8 heads, at most 4 query heads per kv head
  const bool spread = p.heads_kv == 8 && tpt == 16 && upt == 1 && group <= 4;
  int rc = make_tile_map(&mq, p.q, p.dtype, D, p.heads_q, 1, p.batch, p.q_strides[1], 0, p.q_strides[0],
                         spread ? 2 * group : 128);
  if (!rc) rc = make_page_map(&mk, p.k_cache, p.dtype, D, p.heads_kv, p.block_size, p.num_blocks, p.k_strides, tpt);
  if (!rc) rc = make_page_map(&mv, p.v_cache, p.dtype, D, p.heads_kv, p.block_size, p.num_blocks, p.v_strides, tpt);
  if (!rc) rc = make_page_map(&mvr, p.v_cache, p.dtype, D, p.heads_kv, p.block_size, p.num_blocks, p.v_strides, 1);
  if (rc) return rc;
  DecArgs a = {};
  a.paged = 1;
  a.batch = p.batch;
  a.heads_q = p.heads_q;
  a.heads_kv = p.heads_kv;
  a.group = group;
  a.seqlen_q = 1;
  a.rows = p.heads_q;
  a.tpt = tpt;
  a.upp = upp;
  a.upt = upt;
  a.block_size = p.block_size;
  a.max_blocks = p.max_blocks;
  a.num_blocks = p.num_blocks;
  a.first_block = p.first_block;
  a.block_step = p.block_step;
  a.block_table = p.block_table;
  a.bt_sb = p.bt_strides[0];
  a.bt_sk = p.bt_strides[1];
  a.context_lens = p.context_lens;
  a.cl_stride = p.cl_stride;
  a.softmax_scale = p.softmax_scale;
  a.num_partials = p.num_splits;
  a.o_partial = p.o_partial;
  a.lse_partial = p.lse_partial;
  a.status = p.status;
  a.spread = spread ? 1 : 0;
  take_fault_injection(&a);
  int ctas = p.num_splits / 2;
  if (p.balance) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      return set_error(FA_ERR_DEVICE, "cannot query the SM count of the current device");
    if (p.batch > kBalancedMaxBatch || p.batch > sms)
      return set_error(FA_ERR_UNSUPPORTED, "balanced paged decode takes at most %d sequences (and at most one per SM)",
                       kBalancedMaxBatch);
    a.balanced = 1;
    ctas = sms;
  }
  // Balanced mode merges inside the kernel when the launch can be cooperative (every CTA resident, so the CTAs of a
  // sequence may wait for one another), there is a ticket region for this partial buffer and the stream is not being
  // captured; otherwise the merge kernel follows.
  if (p.balance && 2 * ctas <= kThreads && 2 * p.batch <= kTicketWords) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    const bool capturing = cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone;
    if (!capturing && cooperative_launch_ok()) {
      a.tickets = ticket_region(p.o_partial, 2 * p.batch, false);
      a.out = p.out;
      a.out_dtype = p.out_is_f32 ? (int)FA_F32 : p.dtype;
      a.o_sb = p.o_strides[0];
      a.o_sh = p.o_strides[1];
      a.o_sd = p.o_strides[2];
      a.lse_out = p.lse_out;
    }
  }
  rc = dispatch<true>(p.dtype, D, mq, mk, mv, mvr, a, ctas, stream);
  if (rc == kCooperativeRefused) {
    a.tickets = nullptr;
    rc = dispatch<true>(p.dtype, D, mq, mk, mv, mvr, a, ctas, stream);
  }
  if (rc) return rc;
  if (a.tickets != nullptr) return 0;
  const int nrows = p.batch * p.heads_q;
  return launch_combine_internal(nrows, D, p.num_splits, p.o_partial, D, (int64_t)p.num_splits * D, p.lse_partial, 1,
                                 p.num_splits, p.out, p.out_is_f32 ? (int)FA_F32 : p.dtype, p.heads_q, 1, p.o_strides[0],
                                 p.o_strides[1], 0, p.o_strides[2], p.lse_out, stream, true);
}

PROF_DEFINE_READER(fa_debug_read_prof_decode)

void set_decode_fault_injection(uint32_t poll_limit, int skip_tile) {
  g_fault_poll_limit = poll_limit;
  g_fault_skip_tile = skip_tile;
}

}  // namespace fa
