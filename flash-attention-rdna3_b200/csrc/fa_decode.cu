// Split-K decode and the LSE merge. Memory-bound: every K and V byte is read once with 128-bit
// loads, dot products run on the CUDA cores, and the lanes that share a key reduce with shuffles.
//
// One CTA streams one contiguous key slice of one (batch, kv head) for up to R query rows that share
// that kv head (the rows of the GQA group times seqlen_q), so grouped queries read K/V once.
// A "worker" is the set of lanes that covers one key row with 16-byte loads; each worker keeps its
// own running (max, sum, accumulator) and the workers of a CTA are merged through shared memory.
//
// Semantics: fa_rdna3/kernels/decode.py:13-125 (partials are normalised, LSE is natural-log and -inf
// for an empty slice; the merge ignores -inf partials and returns zeros when every slice is empty).
#include <mutex>

#include "fa_common.cuh"

namespace fa {
namespace {

constexpr int kDecodeThreads = 256;
constexpr int kKeysPerIter = 4;

struct DecodeArgs {
  fa_decode_params p;
  int group;
  int rows_total;      // group * seqlen_q
  int keys_per_split;
  unsigned int* tickets;  // one word per (batch, kv head, row block): the merge runs inside the kernel; or nullptr
};

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
  const float2 a = DType<T>::unpack2(raw.x), b = DType<T>::unpack2(raw.y), c = DType<T>::unpack2(raw.z),
               d = DType<T>::unpack2(raw.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

// Shared by the dense and paged kernels: merges the per-worker states in shared memory and writes
// either the final output row (single split, no LSE wanted) or a normalised fp32 partial plus LSE.
//   sm layout: [worker][row][D + 2] floats: acc[D], m (log2 domain), l.
template <int D, int R>
__device__ __forceinline__ void merge_workers_and_store(const float* sm, int workers, int rows_here, int tid,
                                                        int nthreads, float* opart_rows[R], float* lse_rows[R],
                                                        void* out_rows[R], int out_dtype, int64_t out_stride_d) {
  constexpr int kRow = D + 2;
  for (int idx = tid; idx < rows_here * D; idx += nthreads) {
    const int r = idx / D, d = idx % D;
    float M = kNegInf;
    for (int w = 0; w < workers; ++w) M = fmaxf(M, sm[(w * R + r) * kRow + D]);
    const float Ms = (M == kNegInf) ? 0.f : M;
    float num = 0.f, den = 0.f;
    for (int w = 0; w < workers; ++w) {
      const float* st = sm + (w * R + r) * kRow;
      const float sc = exp2f(st[D] - Ms);
      num += sc * st[d];
      den += sc * st[D + 1];
    }
    const float den_safe = (den == 0.f) ? 1.f : den;
    const float o = num / den_safe;
    if (opart_rows[r] != nullptr) opart_rows[r][d] = o;
    else store_from_float(out_rows[r], (int64_t)d * out_stride_d, out_dtype, o);
    if (d == 0 && lse_rows[r] != nullptr) lse_rows[r][0] = (den == 0.f) ? kNegInf : (M * kLn2 + logf(den));
  }
}

// Streaming core shared by the dense and the paged kernel. A worker (LPK lanes) keeps, for each of R query
// rows, the running maximum m (log2 domain), the sum l and its slice of the accumulator.
template <typename T, int D, int R>
struct Stream {
  static constexpr int LPK = (D / 8 < 32) ? D / 8 : 32;  // lanes per key row
  static constexpr int CH = D / (8 * LPK);               // 16-byte chunks per lane per key
  static constexpr int WORKERS = kDecodeThreads / LPK;
  static constexpr int E = CH * 8;                        // head-dim elements per lane

  float q[R][E];
  float m[R], l[R], acc[R][E];

  __device__ __forceinline__ void init() {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      m[r] = kNegInf;
      l[r] = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) acc[r][e] = 0.f;
    }
  }

  // Folds kKeysPerIter keys (raw 16-byte chunks of K and V, already in registers) into the state.
  __device__ __forceinline__ void consume(const uint4 (&kraw)[kKeysPerIter][CH], const uint4 (&vraw)[kKeysPerIter][CH],
                                          const bool (&valid)[kKeysPerIter]) {
    float s[kKeysPerIter][R];
#pragma unroll
    for (int u = 0; u < kKeysPerIter; ++u) {
      float kf[E];
#pragma unroll
      for (int c = 0; c < CH; ++c) unpack8<T>(kraw[u][c], *reinterpret_cast<float(*)[8]>(&kf[c * 8]));
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) d += q[r][e] * kf[e];
        s[u][r] = d;
      }
    }
#pragma unroll
    for (int o = LPK / 2; o > 0; o >>= 1)
#pragma unroll
      for (int u = 0; u < kKeysPerIter; ++u)
#pragma unroll
        for (int r = 0; r < R; ++r) s[u][r] += __shfl_xor_sync(0xffffffffu, s[u][r], o);

    float pr[kKeysPerIter][R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float mt = m[r];
#pragma unroll
      for (int u = 0; u < kKeysPerIter; ++u) {
        if (!valid[u]) s[u][r] = kNegInf;
        mt = fmaxf(mt, s[u][r]);
      }
      const float ms = (mt == kNegInf) ? 0.f : mt;
      const float alpha = fast_exp2(m[r] - ms);
      float sum = 0.f;
#pragma unroll
      for (int u = 0; u < kKeysPerIter; ++u) {
        pr[u][r] = fast_exp2(s[u][r] - ms);
        sum += pr[u][r];
      }
      l[r] = l[r] * alpha + sum;
#pragma unroll
      for (int e = 0; e < E; ++e) acc[r][e] *= alpha;
      m[r] = mt;
    }
#pragma unroll
    for (int u = 0; u < kKeysPerIter; ++u) {
      float vf[E];
#pragma unroll
      for (int c = 0; c < CH; ++c) unpack8<T>(vraw[u][c], *reinterpret_cast<float(*)[8]>(&vf[c * 8]));
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int e = 0; e < E; ++e) acc[r][e] += pr[u][r] * vf[e];
    }
  }

  // Publishes the worker state to shared memory: [worker][row][D + 2] floats.
  __device__ __forceinline__ void publish(float* sm, int worker, int wl) const {
    constexpr int kRow = D + 2;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float* st = sm + (worker * R + r) * kRow;
#pragma unroll
      for (int c = 0; c < CH; ++c)
#pragma unroll
        for (int e = 0; e < 8; ++e) st[(c * LPK + wl) * 8 + e] = acc[r][c * 8 + e];
      if (wl == 0) {
        st[D] = m[r];
        st[D + 1] = l[r];
      }
    }
  }
};

// Walks keys [n_start, n_end) of one CTA with register double-buffering: the loads of the next group of keys are
// in flight while the current group is folded in. `issue(base, kraw, vraw, valid)` fills the raw chunks of the
// keys base + u * WORKERS + worker (zeros and valid = false for keys it must not read).
template <typename S, typename Issue>
__device__ __forceinline__ void stream_keys(S& st, int n_start, int n_end, Issue issue) {
  constexpr int kStride = S::WORKERS * kKeysPerIter;
  uint4 kA[kKeysPerIter][S::CH], vA[kKeysPerIter][S::CH], kB[kKeysPerIter][S::CH], vB[kKeysPerIter][S::CH];
  bool validA[kKeysPerIter], validB[kKeysPerIter];
  issue(n_start, kA, vA, validA);
  for (int base = n_start; base < n_end; base += 2 * kStride) {
    issue(base + kStride, kB, vB, validB);
    st.consume(kA, vA, validA);
    issue(base + 2 * kStride, kA, vA, validA);
    st.consume(kB, vB, validB);
  }
}

template <typename T, int D, int R>
__global__ void __launch_bounds__(kDecodeThreads, 2) decode_splitk_kernel(const DecodeArgs a) {
  using S = Stream<T, D, R>;
  constexpr int LPK = S::LPK, CH = S::CH, WORKERS = S::WORKERS;
  extern __shared__ float sm[];

  const fa_decode_params& p = a.p;
  const int tid = threadIdx.x;
  const int worker = tid / LPK, wl = tid % LPK;
  const int split = blockIdx.x;
  const int b = blockIdx.y / p.heads_kv, hk = blockIdx.y % p.heads_kv;
  const int row0 = blockIdx.z * R;
  const int rows_here = min(R, a.rows_total - row0);

  const int n_start = min(split * a.keys_per_split, p.seqlen_k);
  const int n_end = min(n_start + a.keys_per_split, p.seqlen_k);

  const T* kbase = reinterpret_cast<const T*>(p.k) + (int64_t)b * p.k_strides[0] + (int64_t)hk * p.k_strides[1];
  const T* vbase = reinterpret_cast<const T*>(p.v) + (int64_t)b * p.v_strides[0] + (int64_t)hk * p.v_strides[1];

  S st;
  st.init();
  // this lane's slice of each query row, pre-scaled into the log2 domain
  const float qscale = p.softmax_scale * kLog2e;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int row = row0 + r;
    const int g = row / p.seqlen_q, sq = row % p.seqlen_q;
    const T* qrow = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_strides[0] +
                    (int64_t)(hk * a.group + g) * p.q_strides[1] + (int64_t)sq * p.q_strides[2];
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int d = (c * LPK + wl) * 8 + e;
        st.q[r][c * 8 + e] = (r < rows_here) ? DType<T>::to_float(qrow[(int64_t)d * p.q_strides[3]]) * qscale : 0.f;
      }
  }

  const int64_t ksk = p.k_strides[2], vsk = p.v_strides[2];
  stream_keys(st, n_start, n_end,
              [&](int base, uint4 (&kraw)[kKeysPerIter][CH], uint4 (&vraw)[kKeysPerIter][CH], bool (&valid)[kKeysPerIter]) {
#pragma unroll
                for (int u = 0; u < kKeysPerIter; ++u) {
                  const int key = base + u * WORKERS + worker;
                  valid[u] = key < n_end;
#pragma unroll
                  for (int c = 0; c < CH; ++c) {
                    const int d = (c * LPK + wl) * 8;
                    kraw[u][c] = valid[u] ? ldg_stream(kbase + (int64_t)key * ksk + d) : make_uint4(0, 0, 0, 0);
                    vraw[u][c] = valid[u] ? ldg_stream(vbase + (int64_t)key * vsk + d) : make_uint4(0, 0, 0, 0);
                  }
                }
              });

  st.publish(sm, worker, wl);
  __syncthreads();

  float* opart_rows[R];
  float* lse_rows[R];
  void* out_rows[R];
  const bool direct = (p.num_splits == 1);
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int row = row0 + ((r < rows_here) ? r : 0);
    const int g = row / p.seqlen_q, sq = row % p.seqlen_q;
    const int h = hk * a.group + g;
    const int64_t flat = (((int64_t)split * p.batch + b) * p.heads_q + h) * p.seqlen_q + sq;
    opart_rows[r] = direct ? nullptr : p.o_partial + flat * D;
    lse_rows[r] = direct ? nullptr : p.lse_partial + flat;
    out_rows[r] = reinterpret_cast<T*>(p.out) + (int64_t)b * p.o_strides[0] + (int64_t)h * p.o_strides[1] +
                  (int64_t)sq * p.o_strides[2];
  }
  merge_workers_and_store<D, R>(sm, WORKERS, rows_here, tid, kDecodeThreads, opart_rows, lse_rows, out_rows,
                                p.dtype, p.o_strides[3]);

  // Merge inside the kernel: every CTA of these rows takes a ticket behind its partials (atomicInc wraps the word
  // back to zero), and the one that draws the last ticket merges all splits (the rule of combine_kernel) and writes
  // the output rows. Nobody waits for anybody; it saves the launch of the merge kernel, which for a short decode is a
  // sixth of the call.
  if (!direct && a.tickets != nullptr) {
    __shared__ int last_s;
    __threadfence();
    __syncthreads();
    if (tid == 0) last_s = atomicInc(a.tickets + (blockIdx.z * gridDim.y + blockIdx.y), gridDim.x - 1) == gridDim.x - 1;
    __syncthreads();
    if (last_s) {
      __threadfence();
      const int64_t stride_l = (int64_t)p.batch * p.heads_q * p.seqlen_q, stride_o = stride_l * D;
      for (int idx = tid; idx < rows_here * D; idx += kDecodeThreads) {
        const int r = idx / D, d = idx % D;
        const float* l0 = lse_rows[r] - (int64_t)split * stride_l;
        const float* o0 = opart_rows[r] - (int64_t)split * stride_o + d;
        float M = kNegInf;
        for (int s = 0; s < p.num_splits; ++s) M = fmaxf(M, __ldcg(l0 + s * stride_l));
        const float Ms = (M == kNegInf) ? 0.f : M;
        float num = 0.f, den = 0.f;
        for (int s = 0; s < p.num_splits; ++s) {
          const float ls = __ldcg(l0 + s * stride_l);
          const float w = (ls == kNegInf) ? 0.f : expf(ls - Ms);
          den += w;
          if (w != 0.f) num += w * __ldcg(o0 + s * stride_o);
        }
        store_from_float(out_rows[r], (int64_t)d * p.o_strides[3], p.dtype, num / ((den == 0.f) ? 1.f : den));
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Paged-KV decode (fa_rdna3/kernels/paged.py:17-89): one query row per (batch, query head); keys live
// in fixed-size physical pages reached through a per-sequence block table. One CTA serves one
// (split, batch, kv head) and all query heads of that kv head's group, so a page slice is read once
// per group instead of once per query head. Out-of-range context lengths are clamped and invalid
// page ids are skipped without being dereferenced (paged.py:37-38, 58-63).
// ---------------------------------------------------------------------------------------------
struct PagedArgs {
  fa_paged_params p;
  int group;
};

template <typename T, int D, int R>
__global__ void __launch_bounds__(kDecodeThreads, 2) decode_paged_kernel(const PagedArgs a) {
  using S = Stream<T, D, R>;
  constexpr int LPK = S::LPK, CH = S::CH, WORKERS = S::WORKERS;
  extern __shared__ float sm[];

  const fa_paged_params& p = a.p;
  const int tid = threadIdx.x;
  const int worker = tid / LPK, wl = tid % LPK;
  const int split = blockIdx.x;
  const int b = blockIdx.y / p.heads_kv, hk = blockIdx.y % p.heads_kv;
  const int row0 = blockIdx.z * R;
  const int rows_here = min(R, a.group - row0);
  const int bs = p.block_size;

  int ctx = p.context_lens[(int64_t)b * p.cl_stride];
  const int64_t cap = (int64_t)p.max_blocks * bs;
  ctx = (int)min((int64_t)max(ctx, 0), cap);
  const int nblk = (ctx + bs - 1) / bs;
  // logical blocks of this call: first_block, first_block + block_step, ...
  const int nlocal = (nblk > p.first_block) ? (nblk - p.first_block + p.block_step - 1) / p.block_step : 0;
  const int per = nlocal / p.num_splits, extra = nlocal % p.num_splits;
  const int blk_begin = split * per + min(split, extra);
  const int blk_end = blk_begin + per + (split < extra ? 1 : 0);
  const int n_start = blk_begin * bs, n_end = blk_end * bs;  // local key indices

  S st;
  st.init();
  const float qscale = p.softmax_scale * kLog2e;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const T* qrow = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_strides[0] +
                    (int64_t)(hk * a.group + row0 + r) * p.q_strides[1];
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int d = (c * LPK + wl) * 8 + e;
        st.q[r][c * 8 + e] = (r < rows_here) ? DType<T>::to_float(qrow[(int64_t)d * p.q_strides[2]]) * qscale : 0.f;
      }
  }

  const T* kc = reinterpret_cast<const T*>(p.k_cache) + (int64_t)hk * p.k_strides[2];
  const T* vc = reinterpret_cast<const T*>(p.v_cache) + (int64_t)hk * p.v_strides[2];
  const int32_t* table = p.block_table + (int64_t)b * p.bt_strides[0];

  stream_keys(st, n_start, n_end,
              [&](int base, uint4 (&kraw)[kKeysPerIter][CH], uint4 (&vraw)[kKeysPerIter][CH], bool (&valid)[kKeysPerIter]) {
#pragma unroll
                for (int u = 0; u < kKeysPerIter; ++u) {
                  const int key = base + u * WORKERS + worker;
                  valid[u] = false;
                  int64_t koff = 0, voff = 0;
                  if (key < n_end) {
                    const int lb = p.first_block + (key / bs) * p.block_step;
                    const int within = key % bs;
                    const int phys = table[(int64_t)lb * p.bt_strides[1]];
                    if (lb * bs + within < ctx && phys >= 0 && phys < p.num_blocks) {
                      valid[u] = true;
                      koff = (int64_t)phys * p.k_strides[0] + (int64_t)within * p.k_strides[1];
                      voff = (int64_t)phys * p.v_strides[0] + (int64_t)within * p.v_strides[1];
                    }
                  }
#pragma unroll
                  for (int c = 0; c < CH; ++c) {
                    const int d = (c * LPK + wl) * 8;
                    kraw[u][c] = valid[u] ? ldg_stream(kc + koff + d) : make_uint4(0, 0, 0, 0);
                    vraw[u][c] = valid[u] ? ldg_stream(vc + voff + d) : make_uint4(0, 0, 0, 0);
                  }
                }
              });

  st.publish(sm, worker, wl);
  __syncthreads();

  float* opart_rows[R];
  float* lse_rows[R];
  void* out_rows[R];
  const bool direct = (p.num_splits == 1);
  const int out_dtype = p.out_is_f32 ? (int)FA_F32 : p.dtype;
  const int esz = (out_dtype == FA_F32) ? 4 : 2;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int h = hk * a.group + row0 + ((r < rows_here) ? r : 0);
    const int64_t flat = ((int64_t)b * p.heads_q + h) * p.num_splits + split;
    opart_rows[r] = direct ? nullptr : p.o_partial + flat * D;
    lse_rows[r] = direct ? (p.lse_out ? p.lse_out + (int64_t)b * p.heads_q + h : nullptr) : p.lse_partial + flat;
    out_rows[r] = reinterpret_cast<char*>(p.out) + ((int64_t)b * p.o_strides[0] + (int64_t)h * p.o_strides[1]) * esz;
  }
  merge_workers_and_store<D, R>(sm, WORKERS, rows_here, tid, kDecodeThreads, opart_rows, lse_rows, out_rows,
                                out_dtype, p.o_strides[2]);
}

// ---------------------------------------------------------------------------------------------
// LSE merge (fa_rdna3/kernels/decode.py:80-125).
// ---------------------------------------------------------------------------------------------
struct CombineArgs {
  int rows, D, splits;
  const float* o_partial; int64_t o_split_stride, o_row_stride;
  const float* lse_partial; int64_t lse_split_stride, lse_row_stride;
  void* out; int out_dtype;
  int n1, n2;                       // row = (i0 * n1 + i1) * n2 + i2
  int64_t os0, os1, os2, osd;       // element strides of out for (i0, i1, i2, d)
  float* lse_out;
  // multi-GPU merge: partial s (s != wait_skip) may be read once wait_flags[s] >= wait_value (raised by rank s over
  // NVLink after its stores); null for every other use
  const int* wait_flags;
  int wait_count, wait_skip, wait_value;
  int* status;
};

// Bounded wait of a merge CTA for the partials other GPUs deliver. Returns false (and records it) when a flag did not
// arrive in about a second; the CTA then writes nothing.
__device__ __forceinline__ bool wait_for_peers(const CombineArgs& a) {
  __shared__ int lost;
  if (threadIdx.x == 0) lost = 0;
  __syncthreads();
  const int t = threadIdx.x;
  if (t < a.wait_count && t != a.wait_skip) {
    bool seen = false;
    for (uint32_t i = 0; i < (1u << 22); ++i) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(a.wait_flags + t) : "memory");
      if (v >= a.wait_value) {
        seen = true;
        break;
      }
      __nanosleep(200);
    }
    if (!seen) {
      lost = 1;
      if (a.status != nullptr) atomicCAS(a.status, 0, 701);
    }
  }
  __syncthreads();
  return lost == 0;
}

// One 256-thread CTA per output row. The merge weights of all partials are computed once into shared memory;
// then eight groups of 32 lanes each take every eighth partial (independent loads, all in flight together)
// and the group sums are added through shared memory.
constexpr int kCombineThreads = 256;
constexpr int kCombineMaxD = 512;

__global__ void __launch_bounds__(kCombineThreads) combine_kernel(const CombineArgs a) {
  // Launched as a programmatic dependent of the kernel that writes the partials, this CTA may already be resident
  // while that kernel drains; it goes on once that grid has completed (at once when launched the ordinary way).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (a.wait_flags != nullptr && !wait_for_peers(a)) return;
  __shared__ float w_s[kCombineThreads];
  __shared__ __align__(16) float red_s[8][kCombineMaxD];  // written as float4
  __shared__ float stat_s[2];
  const int tid = threadIdx.x, grp = tid / 32, lane = tid % 32;
  const int row = blockIdx.x;
  const float* lse_row = a.lse_partial + (int64_t)row * a.lse_row_stride;
  const float* o_row = a.o_partial + (int64_t)row * a.o_row_stride;

  // maximum LSE over the partials (the first warp; splits beyond 256 are walked with a stride)
  if (grp == 0) {
    float M = kNegInf;
    for (int s = lane; s < a.splits; s += 32) M = fmaxf(M, lse_row[(int64_t)s * a.lse_split_stride]);
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    if (lane == 0) stat_s[0] = (M == kNegInf) ? 0.f : M;
  }
  __syncthreads();
  const float Ms = stat_s[0];

  float4 acc4[kCombineMaxD / 128];  // this lane's float4 slots: d4 = lane + 32 * k
#pragma unroll
  for (int k = 0; k < kCombineMaxD / 128; ++k) acc4[k] = make_float4(0.f, 0.f, 0.f, 0.f);
  float den = 0.f;
  const int nd4 = a.D / 4;
  for (int s0 = 0; s0 < a.splits; s0 += kCombineThreads) {
    __syncthreads();
    const int sw = s0 + tid;
    float w = 0.f;
    if (sw < a.splits) {
      const float ls = lse_row[(int64_t)sw * a.lse_split_stride];
      w = (ls == kNegInf) ? 0.f : expf(ls - Ms);
    }
    w_s[tid] = w;
    __syncthreads();
    const int n_here = min(kCombineThreads, a.splits - s0);
    for (int s = grp; s < n_here; s += 8) {
      const float ws = w_s[s];
      den += ws;
      if (ws == 0.f) continue;
      const float4* src = reinterpret_cast<const float4*>(o_row + (int64_t)(s0 + s) * a.o_split_stride);
#pragma unroll
      for (int k = 0; k < kCombineMaxD / 128; ++k) {
        const int d4 = lane + 32 * k;
        if (d4 < nd4) {
          const float4 v = src[d4];
          acc4[k].x += ws * v.x;
          acc4[k].y += ws * v.y;
          acc4[k].z += ws * v.z;
          acc4[k].w += ws * v.w;
        }
      }
    }
  }
#pragma unroll
  for (int k = 0; k < kCombineMaxD / 128; ++k) {
    const int d4 = lane + 32 * k;
    if (d4 < nd4) *reinterpret_cast<float4*>(&red_s[grp][d4 * 4]) = acc4[k];
  }
  // every group saw a disjoint set of partials: the denominators add up across groups
  if (lane == 0) w_s[grp] = den;
  __syncthreads();
  float den_all = 0.f;
#pragma unroll
  for (int g = 0; g < 8; ++g) den_all += w_s[g];
  const float den_safe = (den_all == 0.f) ? 1.f : den_all;
  const int i2 = row % a.n2, i1 = (row / a.n2) % a.n1, i0 = row / (a.n2 * a.n1);
  const int64_t obase = (int64_t)i0 * a.os0 + (int64_t)i1 * a.os1 + (int64_t)i2 * a.os2;
  for (int d = tid; d < a.D; d += kCombineThreads) {
    float num = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) num += red_s[g][d];
    store_from_float(a.out, obase + (int64_t)d * a.osd, a.out_dtype, num / den_safe);
  }
  if (tid == 0 && a.lse_out != nullptr) a.lse_out[row] = (den_all == 0.f) ? kNegInf : (Ms + logf(den_all));
}

// The same merge for many partials of a narrow row (head_dim <= 128, 16 to 1024 partials): 1024 threads per output
// row, so that 32 groups of lanes each take every 32nd partial and all partial rows of a merge of up to 32 x 8
// partials are in flight within a few load round trips (the 256-thread form walks them eight at a time).
constexpr int kCombineWideThreads = 1024;
constexpr int kCombineWideMaxSplits = 1024;

__global__ void __launch_bounds__(kCombineWideThreads) combine_wide_kernel(const CombineArgs a) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // see combine_kernel
  __shared__ float w_s[kCombineWideMaxSplits];
  __shared__ float4 red_s[32][32];
  __shared__ float part_s[32];
  const int tid = threadIdx.x, grp = tid / 32, lane = tid % 32;
  const int row = blockIdx.x;
  const float* lse_row = a.lse_partial + (int64_t)row * a.lse_row_stride;
  const float* o_row = a.o_partial + (int64_t)row * a.o_row_stride;

  const float ls = tid < a.splits ? lse_row[(int64_t)tid * a.lse_split_stride] : kNegInf;
  float M = ls;
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
  if (lane == 0) part_s[grp] = M;
  __syncthreads();
  M = part_s[lane];
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
  const float Ms = (M == kNegInf) ? 0.f : M;
  const float w = (ls == kNegInf) ? 0.f : expf(ls - Ms);
  if (tid < a.splits) w_s[tid] = w;
  float den = w;
  for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
  __syncthreads();  // everyone has read part_s; the weights are in place
  if (lane == 0) part_s[grp] = den;

  const int nd4 = a.D / 4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (lane < nd4) {
#pragma unroll 4
    for (int s = grp; s < a.splits; s += 32) {
      const float ws = w_s[s];
      if (ws == 0.f) continue;
      const float4 v = reinterpret_cast<const float4*>(o_row + (int64_t)s * a.o_split_stride)[lane];
      acc.x += ws * v.x;
      acc.y += ws * v.y;
      acc.z += ws * v.z;
      acc.w += ws * v.w;
    }
  }
  red_s[grp][lane] = acc;
  __syncthreads();
  float den_all = part_s[lane];
  for (int o = 16; o > 0; o >>= 1) den_all += __shfl_xor_sync(0xffffffffu, den_all, o);
  const float den_safe = (den_all == 0.f) ? 1.f : den_all;
  if (tid < a.D) {
    const float* col = reinterpret_cast<const float*>(&red_s[0][0]) + tid;  // element tid of every group's row
    float num = 0.f;
#pragma unroll
    for (int g = 0; g < 32; ++g) num += col[g * 128];
    const int i2 = row % a.n2, i1 = (row / a.n2) % a.n1, i0 = row / (a.n2 * a.n1);
    const int64_t obase = (int64_t)i0 * a.os0 + (int64_t)i1 * a.os1 + (int64_t)i2 * a.os2;
    store_from_float(a.out, obase + (int64_t)tid * a.osd, a.out_dtype, num / den_safe);
  }
  if (tid == 0 && a.lse_out != nullptr) a.lse_out[row] = (den_all == 0.f) ? kNegInf : (Ms + logf(den_all));
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "%s launch failed: %s", what, cudaGetErrorString(e));
  return 0;
}

template <typename T, int D, int R>
int launch_split_typed(const DecodeArgs& a, cudaStream_t stream) {
  constexpr int LPK = (D / 8 < 32) ? D / 8 : 32;
  constexpr int WORKERS = kDecodeThreads / LPK;
  const size_t smem = sizeof(float) * WORKERS * R * (D + 2);
  auto kern = decode_splitk_kernel<T, D, R>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "decode smem opt-in failed: %s", cudaGetErrorString(e));
  }
  dim3 grid(a.p.num_splits, a.p.batch * a.p.heads_kv, (a.rows_total + R - 1) / R);
  kern<<<grid, kDecodeThreads, smem, stream>>>(a);
  return check_launch("split-K decode");
}

template <typename T, int D>
int launch_split_rows(const DecodeArgs& a, cudaStream_t stream) {
  if (a.rows_total == 1) return launch_split_typed<T, D, 1>(a, stream);
  if (a.rows_total == 2) return launch_split_typed<T, D, 2>(a, stream);
  if (D >= 256) return launch_split_typed<T, D, 2>(a, stream);
  return launch_split_typed<T, D, 4>(a, stream);
}

template <typename T>
int launch_split_dim(const DecodeArgs& a, cudaStream_t stream) {
  switch (a.p.head_dim) {
    case 16: return launch_split_rows<T, 16>(a, stream);
    case 32: return launch_split_rows<T, 32>(a, stream);
    case 64: return launch_split_rows<T, 64>(a, stream);
    case 128: return launch_split_rows<T, 128>(a, stream);
    case 256: return launch_split_rows<T, 256>(a, stream);
    case 512: return launch_split_rows<T, 512>(a, stream);
  }
  return set_error(FA_ERR_UNSUPPORTED, "decode head_dim %d is not a supported power of two", a.p.head_dim);
}

template <typename T, int D, int R>
int launch_paged_typed(const PagedArgs& a, cudaStream_t stream) {
  constexpr int LPK = (D / 8 < 32) ? D / 8 : 32;
  constexpr int WORKERS = kDecodeThreads / LPK;
  const size_t smem = sizeof(float) * WORKERS * R * (D + 2);
  auto kern = decode_paged_kernel<T, D, R>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "paged smem opt-in failed: %s", cudaGetErrorString(e));
  }
  dim3 grid(a.p.num_splits, a.p.batch * a.p.heads_kv, (a.group + R - 1) / R);
  kern<<<grid, kDecodeThreads, smem, stream>>>(a);
  return check_launch("paged decode");
}

template <typename T, int D>
int launch_paged_rows(const PagedArgs& a, cudaStream_t stream) {
  if (a.group == 1) return launch_paged_typed<T, D, 1>(a, stream);
  if (a.group == 2) return launch_paged_typed<T, D, 2>(a, stream);
  if (D >= 256) return launch_paged_typed<T, D, 2>(a, stream);
  return launch_paged_typed<T, D, 4>(a, stream);
}

template <typename T>
int launch_paged_dim(const PagedArgs& a, cudaStream_t stream) {
  switch (a.p.head_dim) {
    case 16: return launch_paged_rows<T, 16>(a, stream);
    case 32: return launch_paged_rows<T, 32>(a, stream);
    case 64: return launch_paged_rows<T, 64>(a, stream);
    case 128: return launch_paged_rows<T, 128>(a, stream);
    case 256: return launch_paged_rows<T, 256>(a, stream);
    case 512: return launch_paged_rows<T, 512>(a, stream);
  }
  return set_error(FA_ERR_UNSUPPORTED, "paged head_dim %d is not a supported power of two", a.p.head_dim);
}

}  // namespace

int launch_combine_internal(int rows, int D, int splits, const float* o_partial, int64_t o_split_stride,
                            int64_t o_row_stride, const float* lse_partial, int64_t lse_split_stride,
                            int64_t lse_row_stride, void* out, int out_dtype, int n1, int n2, int64_t os0,
                            int64_t os1, int64_t os2, int64_t osd, float* lse_out, cudaStream_t stream,
                            bool dependent) {
  CombineArgs a{rows, D, splits, o_partial, o_split_stride, o_row_stride, lse_partial, lse_split_stride,
                lse_row_stride, out, out_dtype, n1, n2, os0, os1, os2, osd, lse_out, nullptr, 0, 0, 0, nullptr};
  if (D > kCombineMaxD || D % 4 || o_split_stride % 4 || o_row_stride % 4 ||
      (reinterpret_cast<uintptr_t>(o_partial) & 15))
    return set_error(FA_ERR_UNSUPPORTED, "combine needs head_dim <= %d, and 16-byte aligned partial rows", kCombineMaxD);
  // dependent: the kernel launched just before on this stream writes the partials and releases its dependents early,
  // so these CTAs are set up while its last CTAs drain instead of after the grid has gone
  const bool wide = D <= 128 && splits >= 16 && splits <= kCombineWideMaxSplits;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows);
  cfg.blockDim = dim3(wide ? kCombineWideThreads : kCombineThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr = {};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  if (dependent) {
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  }
  const cudaError_t e = wide ? cudaLaunchKernelEx(&cfg, combine_wide_kernel, a) : cudaLaunchKernelEx(&cfg, combine_kernel, a);
  if (e != cudaSuccess) return set_error(FA_ERR_LAUNCH, "combine launch failed: %s", cudaGetErrorString(e));
  return check_launch("combine");
}

// ---------------------------------------------------------------------------------------------
// multi-GPU merge without a collective
// ---------------------------------------------------------------------------------------------
struct PeerPushArgs {
  const float4* src;
  int64_t n4;
  float4* dst[FA_MAX_PEERS];
  int* flag[FA_MAX_PEERS];
  int rank, epoch;
};

// One CTA per peer: copies this rank's slot into the peer's buffer (plain 16-byte stores over NVLink), makes the
// stores visible system-wide, then raises the peer's flag for this rank.
__global__ void __launch_bounds__(1024) peer_push_kernel(const PeerPushArgs a) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int peer = blockIdx.x < a.rank ? blockIdx.x : blockIdx.x + 1;
  float4* dst = a.dst[peer];
  for (int64_t i = threadIdx.x; i < a.n4; i += blockDim.x) dst[i] = a.src[i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(a.flag[peer]), "r"(a.epoch) : "memory");
}

int launch_peer_merge(const fa_peer_merge_params& p, cudaStream_t stream) {
  if (p.world < 1 || p.world > FA_MAX_PEERS || p.rank < 0 || p.rank >= p.world)
    return set_error(FA_ERR_INVALID_ARGUMENT, "peer merge: world must be in [1, %d] and rank inside it", FA_MAX_PEERS);
  if (p.rows <= 0 || p.head_dim <= 0 || p.head_dim % 4 || p.head_dim > kCombineMaxD || p.epoch <= 0)
    return set_error(FA_ERR_INVALID_ARGUMENT, "peer merge: rows, head_dim (multiple of 4) and epoch must be positive");
  if (p.slot_floats < (int64_t)p.rows * (p.head_dim + 1) || p.slot_floats % 4)
    return set_error(FA_ERR_INVALID_ARGUMENT, "peer merge: a slot holds rows * (head_dim + 1) floats, a multiple of four");
  for (int r = 0; r < p.world; ++r)
    if (p.peer_base[r] == nullptr || p.peer_flags[r] == nullptr || (reinterpret_cast<uintptr_t>(p.peer_base[r]) & 15))
      return set_error(FA_ERR_INVALID_ARGUMENT, "peer merge: buffer %d is NULL or not 16-byte aligned", r);
  if (p.out == nullptr) return set_error(FA_ERR_INVALID_ARGUMENT, "peer merge: out is NULL");
  float* local = p.peer_base[p.rank];
  if (p.world > 1) {
    PeerPushArgs a = {};
    a.src = reinterpret_cast<const float4*>(local + (int64_t)p.rank * p.slot_floats);
    a.n4 = p.slot_floats / 4;
    for (int r = 0; r < p.world; ++r) {
      a.dst[r] = reinterpret_cast<float4*>(p.peer_base[r] + (int64_t)p.rank * p.slot_floats);
      a.flag[r] = p.peer_flags[r] + p.rank;
    }
    a.rank = p.rank;
    a.epoch = p.epoch;
    peer_push_kernel<<<p.world - 1, 1024, 0, stream>>>(a);
    int rc = check_launch("peer push");
    if (rc) return rc;
  }
  CombineArgs c{p.rows, p.head_dim, p.world, local, p.slot_floats, p.head_dim, local + (int64_t)p.rows * p.head_dim,
                p.slot_floats, 1, p.out, p.out_dtype, 1, p.rows, 0, 0, p.out_row_stride, 1, p.lse_out,
                p.world > 1 ? p.peer_flags[p.rank] : nullptr, p.world, p.rank, p.epoch, p.status};
  combine_kernel<<<p.rows, kCombineThreads, 0, stream>>>(c);
  return check_launch("peer merge");
}

int launch_combine(const fa_combine_params& p, cudaStream_t stream) {
  if (p.rows <= 0 || p.head_dim <= 0 || p.num_splits <= 0)
    return set_error(FA_ERR_INVALID_ARGUMENT, "combine: rows, head_dim and num_splits must be positive");
  return launch_combine_internal(p.rows, p.head_dim, p.num_splits, p.o_partial, p.o_split_stride, p.o_row_stride,
                                 p.lse_partial, p.lse_split_stride, p.lse_row_stride, p.out, p.out_dtype, 1, p.rows,
                                 0, 0, p.out_row_stride, 1, p.lse_out, stream, false);
}

int launch_decode_splitk(const fa_decode_params& p, cudaStream_t stream) {
  if (p.dtype != FA_F16 && p.dtype != FA_BF16)
    return set_error(FA_ERR_UNSUPPORTED, "decode supports float16 and bfloat16 only");
  if (p.heads_kv <= 0 || p.heads_q % p.heads_kv != 0)
    return set_error(FA_ERR_INVALID_ARGUMENT, "query heads must be a multiple of key/value heads");
  if (p.num_splits < 1) return set_error(FA_ERR_INVALID_ARGUMENT, "num_splits must be at least 1");
  if (p.k_strides[3] != 1 || p.v_strides[3] != 1 || p.k_strides[2] % 8 || p.v_strides[2] % 8 ||
      p.k_strides[1] % 8 || p.v_strides[1] % 8 || p.k_strides[0] % 8 || p.v_strides[0] % 8 ||
      (reinterpret_cast<uintptr_t>(p.k) & 15) || (reinterpret_cast<uintptr_t>(p.v) & 15))
    return set_error(FA_ERR_UNSUPPORTED, "decode needs K/V with unit inner stride and 16-byte aligned rows");
  if (p.num_splits > 1 && (p.o_partial == nullptr || p.lse_partial == nullptr))
    return set_error(FA_ERR_INVALID_ARGUMENT, "decode with several splits needs partial buffers");
  const bool tc_ok = decode_tc_supported(p);
  if (p.force_path == FA_PATH_TCGEN05 && !tc_ok)
    return set_error(FA_ERR_UNSUPPORTED, "tcgen05 decode needs fp16/bf16, head_dim 64/128/256, <= 128 rows per kv head, "
                                         "TMA-compatible strides and num_splits >= 2 (even below head_dim 256)");
  // Head dim 256 has room for two 64 KB ring slots only, so its tensor-core kernel streams at about 4 TB/s; it wins
  // once a kv head serves four or more query rows (the CUDA-core kernel is then bound by its FMAs: 2.7 TB/s at a group
  // of four) and loses below that (5.8 TB/s on CUDA cores with one row per kv head).
  const bool tc_pays = p.head_dim != 256 || (p.heads_q / p.heads_kv) * p.seqlen_q >= 4;
  if (tc_ok && p.force_path != FA_PATH_SIMT && (tc_pays || p.force_path == FA_PATH_TCGEN05)) {
    set_path(FA_PATH_TCGEN05);
    return launch_decode_tc(p, stream);
  }
  set_path(FA_PATH_SIMT);
  DecodeArgs a;
  a.p = p;
  a.group = p.heads_q / p.heads_kv;
  a.rows_total = a.group * p.seqlen_q;
  const int blocks64 = (p.seqlen_k + 63) / 64;
  a.keys_per_split = ((blocks64 + p.num_splits - 1) / p.num_splits) * 64;
  a.tickets = nullptr;
  {
    // rows per CTA as launch_split_rows chooses them; one ticket word per (batch, kv head, row block)
    const int rows_per_cta = a.rows_total <= 2 ? a.rows_total : (p.head_dim >= 256 ? 2 : 4);
    const int64_t words = (int64_t)p.batch * p.heads_kv * ((a.rows_total + rows_per_cta - 1) / rows_per_cta);
    if (p.num_splits > 1 && p.num_splits <= 64 && words <= 1024)
      a.tickets = decode_ticket_words(p.o_partial, (int)words, stream);
  }
  int rc = (p.dtype == FA_F16) ? launch_split_dim<__half>(a, stream) : launch_split_dim<__nv_bfloat16>(a, stream);
  if (rc) return rc;
  if (p.num_splits > 1 && a.tickets == nullptr) {
    const int rows = p.batch * p.heads_q * p.seqlen_q;
    rc = launch_combine_internal(rows, p.head_dim, p.num_splits, p.o_partial, (int64_t)rows * p.head_dim, p.head_dim,
                                 p.lse_partial, rows, 1, p.out, p.dtype, p.heads_q, p.seqlen_q, p.o_strides[0],
                                 p.o_strides[1], p.o_strides[2], p.o_strides[3], nullptr, stream, false);
  }
  return rc;
}

int launch_decode_paged(const fa_paged_params& p, cudaStream_t stream) {
  if (p.dtype != FA_F16 && p.dtype != FA_BF16)
    return set_error(FA_ERR_UNSUPPORTED, "paged decode supports float16 and bfloat16 only");
  if (p.heads_kv <= 0 || p.heads_q % p.heads_kv != 0)
    return set_error(FA_ERR_INVALID_ARGUMENT, "query heads must be a multiple of cache heads");
  if (p.num_splits < 1 || p.block_size < 1 || p.block_step < 1 || p.first_block < 0)
    return set_error(FA_ERR_INVALID_ARGUMENT, "paged decode: bad num_splits / block_size / block range");
  if (p.k_strides[3] != 1 || p.v_strides[3] != 1 || p.k_strides[0] % 8 || p.k_strides[1] % 8 || p.k_strides[2] % 8 ||
      p.v_strides[0] % 8 || p.v_strides[1] % 8 || p.v_strides[2] % 8 ||
      (reinterpret_cast<uintptr_t>(p.k_cache) & 15) || (reinterpret_cast<uintptr_t>(p.v_cache) & 15))
    return set_error(FA_ERR_UNSUPPORTED, "paged decode needs caches with unit inner stride and 16-byte aligned rows");
  if (p.num_splits > 1 && (p.o_partial == nullptr || p.lse_partial == nullptr))
    return set_error(FA_ERR_INVALID_ARGUMENT, "paged decode with several splits needs partial buffers");
  const bool tc_ok = paged_tc_supported(p);
  if (p.force_path == FA_PATH_TCGEN05 && !tc_ok)
    return set_error(FA_ERR_UNSUPPORTED, "tcgen05 paged decode needs fp16/bf16, head_dim 64/128, block_size <= 128, "
                                         "TMA-compatible strides and an even num_splits >= 2");
  if (tc_ok && p.force_path != FA_PATH_SIMT) {
    set_path(FA_PATH_TCGEN05);
    return launch_paged_tc(p, stream);
  }
  set_path(FA_PATH_SIMT);
  PagedArgs a;
  a.p = p;
  a.group = p.heads_q / p.heads_kv;
  int rc = (p.dtype == FA_F16) ? launch_paged_dim<__half>(a, stream) : launch_paged_dim<__nv_bfloat16>(a, stream);
  if (rc) return rc;
  if (p.num_splits > 1) {
    const int rows = p.batch * p.heads_q;
    rc = launch_combine_internal(rows, p.head_dim, p.num_splits, p.o_partial, p.head_dim,
                                 (int64_t)p.num_splits * p.head_dim, p.lse_partial, 1, p.num_splits, p.out,
                                 p.out_is_f32 ? (int)FA_F32 : p.dtype, p.heads_q, 1, p.o_strides[0], p.o_strides[1], 0,
                                 p.o_strides[2], p.lse_out, stream, false);
  }
  return rc;
}

// ---------------------------------------------------------------------------------------------
// Split-K decode for callers that cannot allocate device memory.
//
// Some callers of a decode step may not allocate device memory (no cudaMalloc, nothing that allocates) where
// they run attention: code that executes inside a serving engine's pre-sized arena, a plug-in that is only
// handed input and output buffers, or a caller in a latency-critical loop where an allocator call (and the
// device synchronisation it can imply) is not acceptable. Split-K decode needs scratch for the per-slice
// partial results; this variant keeps that scratch in a fixed array that is part of the library image.
//
// The array lives in every GPU context that loads the library, from load until exit: kNoAllocScratchFloats
// floats (8 MiB). A problem needs num_splits * batch * heads_q * seqlen_q * (head_dim + 1) floats and is
// rejected when that is more. All calls on a device share the array and it keeps what the last call wrote,
// so two calls whose kernels may overlap on the GPU (different streams, or graphs replayed concurrently)
// race; calls on one stream are safe. Nothing in it has to start from zero: every slice of every row writes
// its partial and its LSE before the merge reads them.
//
// In host code the array's name is only a handle, not a device address. The first call on a device (with
// that device current) asks the runtime for the real address with cudaGetSymbolAddress and caches it per
// device; make that first call before any stream capture starts.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr size_t kNoAllocScratchFloats = size_t(2) << 20;  // 2 Mi floats = 8 MiB
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];

constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {};
std::mutex g_noalloc_mutex;

// Device address of the scratch array in the current device's context, or nullptr with the error set.
float* noalloc_scratch_for_current_device() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_error(FA_ERR_DEVICE, "cannot identify the current CUDA device: %s", cudaGetErrorString(e));
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      set_error(FA_ERR_DEVICE, "cudaGetSymbolAddress failed for the decode scratch array: %s", cudaGetErrorString(e));
      return nullptr;
    }
    g_noalloc_ptr[dev] = static_cast<float*>(ptr);
  }
  return g_noalloc_ptr[dev];
}

}  // namespace

int launch_decode_splitk_noalloc(const fa_decode_params& p, cudaStream_t stream) {
  if (p.num_splits < 1) return set_error(FA_ERR_INVALID_ARGUMENT, "num_splits must be at least 1");
  const size_t rows = (size_t)p.batch * p.heads_q * p.seqlen_q;
  const size_t need = (size_t)p.num_splits * rows * ((size_t)p.head_dim + 1);
  if (need > kNoAllocScratchFloats)
    return set_error(FA_ERR_UNSUPPORTED,
                     "decode without allocation: num_splits*batch*heads_q*seqlen_q*(head_dim+1) = %zu floats exceeds the "
                     "built-in scratch of %zu floats; use fewer splits or fa_decode_splitk with caller scratch",
                     need, kNoAllocScratchFloats);
  float* scratch = noalloc_scratch_for_current_device();
  if (scratch == nullptr) return FA_ERR_DEVICE;
  fa_decode_params q = p;
  q.o_partial = scratch;                                        // (num_splits, rows, head_dim)
  q.lse_partial = scratch + (size_t)p.num_splits * rows * p.head_dim;  // (num_splits, rows)
  return launch_decode_splitk(q, stream);
}

}  // namespace fa

extern "C" int32_t fa_decode_splitk_noalloc(const fa_decode_params* p, void* stream) {
  if (p == nullptr) return fa::set_error(FA_ERR_INVALID_ARGUMENT, "params is NULL");
  if (p->batch <= 0 || p->heads_q <= 0 || p->heads_kv <= 0 || p->seqlen_q <= 0 || p->seqlen_k <= 0 || p->head_dim <= 0)
    return fa::set_error(FA_ERR_INVALID_ARGUMENT, "batch, heads, sequence lengths and head_dim must be positive");
  if (p->q == nullptr || p->k == nullptr || p->v == nullptr || p->out == nullptr)
    return fa::set_error(FA_ERR_INVALID_ARGUMENT, "q, k, v and out must not be NULL");
  return fa::launch_decode_splitk_noalloc(*p, static_cast<cudaStream_t>(stream));
}
