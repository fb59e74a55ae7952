/*
 * fa_b200 — C ABI of the B200 (sm_100a) attention library.
 *
 * The reference project (chelokot/flash-attention-rdna3, package fa_rdna3) has no FFI: its Python
 * launch glue calls Triton kernels directly. Each entry point below replaces one of those launch
 * sites; the comment on it names the launch it stands for (paths are relative to the reference
 * repository). The Python package fa_b200 binds these symbols with ctypes and is the only caller
 * the library needs, but any host language that can pass plain pointers can use it.
 *
 * Conventions
 *  - Every pointer is a device pointer unless stated otherwise. The caller owns every buffer: the
 *    library allocates nothing and frees nothing (outputs and scratch are passed in, the way the reference
 *    allocates them with torch.empty before a launch; fa_workspace_bytes gives the scratch sizes). The two
 *    fixed arrays the library does use (the scratch of fa_decode_splitk_noalloc and the ticket words of the
 *    in-kernel decode merge) are part of its image.
 *  - Strides are in ELEMENTS of the tensor's dtype, one per dimension, as in the reference kernels'
 *    signatures (e.g. fa_rdna3/kernels/forward.py:30-40).
 *  - `stream` is a cudaStream_t passed as void*; work is enqueued on it and the call returns without
 *    synchronising.
 *  - Return value: 0 on success, a negative FA_ERR_* code otherwise; fa_last_error_string() gives a
 *    message for the calling thread's last failure. Nothing throws.
 *  - `status` fields point at one int32 in device memory that a kernel sets non-zero when one of its
 *    bounded internal waits ran out (the kernel then abandons its tile and exits); may be NULL.
 */
#ifndef FA_B200_H_
#define FA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FA_B200_ABI_VERSION 3

#if defined(__GNUC__)
#define FA_API __attribute__((visibility("default")))
#else
#define FA_API
#endif

enum fa_dtype { FA_F16 = 0, FA_BF16 = 1, FA_F32 = 2 };

enum fa_error {
  FA_OK = 0,
  FA_ERR_INVALID_ARGUMENT = -1,
  FA_ERR_UNSUPPORTED = -2,
  FA_ERR_LAUNCH = -3,
  FA_ERR_DEVICE = -4
};

/* Which kernel family served the last fa_fwd / fa_bwd call (diagnostics and tests). */
enum fa_path { FA_PATH_NONE = 0, FA_PATH_TCGEN05 = 1, FA_PATH_SIMT = 2 };

/*
 * Dense or packed (varlen) attention problem; shared by forward and backward.
 *
 * Dense layout: q (batch, heads_q, seqlen_q, head_dim); k, v (batch, heads_kv, seqlen_k, head_dim);
 * lse/delta (batch, heads_q, seqlen_q). Stride arrays are ordered (batch, head, seq, dim).
 * Varlen layout (varlen != 0): q (total_q, heads_q, head_dim), k, v (total_k, heads_kv, head_dim),
 * lse/delta (heads_q, total_q); stride arrays keep the (batch, head, seq, dim) order with the batch
 * stride ignored and the `seq` stride being the token stride; `batch` is the number of sequences and
 * seqlen_q / seqlen_k are max_seqlen_q / max_seqlen_k. cu_seqlens_* hold batch + 1 int32 entries and
 * are clamped into [0, total] by the kernels (fa_rdna3/kernels/varlen.py:22-27).
 *
 * head_dim: any width up to 512. fp16 / bf16 widths that are a multiple of 8 up to 256 (forward) or 128 (backward),
 * with unit inner stride and 16-byte aligned rows, run on the fused tensor-core kernels as they are: the tensor maps
 * fill the columns up to 64, 128 or 256 with zeros, so the padding the reference does in Python
 * (fa_rdna3/interface.py:386-396) needs no copy here. Dense problems that bring a ds_workspace also run on the tensor
 * cores above those widths, up to 512 (above 256 without softcap, bias, ALiBi or dropout), as separate products over
 * 16-bit tiles kept in that workspace. Everything else (fp32, odd strides, those widths without a
 * workspace or with packed sequences) runs on the CUDA-core kernels.
 */
typedef struct fa_attn_params {
  int32_t dtype;            /* fa_dtype of q, k, v, out, dout, dq, dk, dv */
  int32_t varlen;
  int32_t batch, heads_q, heads_kv, seqlen_q, seqlen_k, head_dim;
  int32_t total_q, total_k; /* varlen only */
  const int32_t* cu_seqlens_q;
  const int32_t* cu_seqlens_k;

  const void* q; int64_t q_strides[4];
  const void* k; int64_t k_strides[4];
  const void* v; int64_t v_strides[4];
  void* out;     int64_t o_strides[4];
  float* lse;    int64_t lse_strides[3];   /* (batch, head, seq); varlen: (unused, head, token) */

  /* backward only */
  const void* dout; int64_t do_strides[4];
  float* delta;     int64_t delta_strides[3];
  void* dq; int64_t dq_strides[4];
  void* dk; int64_t dk_strides[4];
  void* dv; int64_t dv_strides[4];

  /* score modifiers, applied in the reference's order: scale, softcap, bias, ALiBi, mask
     (fa_rdna3/kernels/_common.py:275-308) */
  float softmax_scale;
  float softcap;            /* 0 disables */
  const void* bias;         /* may be NULL; broadcast dims carry stride 0 */
  int32_t bias_dtype;       /* fa_dtype of bias */
  int64_t bias_strides[4];  /* (batch, head, seq_q, seq_k) */
  const float* alibi_slopes;/* (heads_q,) fp32, may be NULL */
  int32_t causal;           /* bottom-right aligned */
  int32_t window_left;      /* -1 = unbounded */
  int32_t window_right;     /* -1 = unbounded */
  float dropout_p;          /* dense only */
  uint64_t dropout_seed;

  int32_t* status;          /* device int32 or NULL */
  int32_t force_path;       /* 0 = automatic, else an fa_path to force (tests) */
  int32_t bwd_parts;        /* fa_bwd only: 0 = everything, else a mask of FA_BWD_* parts to run
                               (lets a caller time or schedule the three kernels separately) */
  /* fa_bwd, dense, tensor-core kernels only; may be NULL. Scratch of fa_workspace_bytes(FA_WS_BWD_DS, p) bytes,
     aligned to 1024. With it the dK/dV kernel stores every 128 x 128 tile of dS it forms (16-bit) and dQ = dS K is one
     GEMM over those tiles; without it a second kernel recomputes the scores and dP for dQ (7 tile products instead of
     5, no scratch). Same arithmetic on the same 16-bit dS either way, same fixed summation order, no atomics. The
     size grows with seqlen_q * seqlen_k (2 bytes per score of every query head): meant for training shapes where
     that is affordable; the Python layer uses it up to a cap and the reference never materialises anything.
     Head dims above 128 (to 512; above 256 without score modifiers): the scratch holds P and dS (4 bytes per score)
     and is what puts the backward on the tensor cores at all. fa_fwd, dense, head dims above 256 (to 512), no score modifier: scratch of
     fa_workspace_bytes(FA_WS_FWD_P, p) bytes for the P tiles (2 bytes per score); without it the forward of those
     widths runs on the CUDA-core kernels. fa_fwd, dense, fp32 inputs, head dims to 256, no score modifier: passing a
     scratch of FA_WS_FWD_P bytes opts into tensor-core products (Q K^T in tf32, P V in fp16 with V rounded to fp16,
     about 1e-3 absolute error on unit-variance inputs); without it fp32 inputs are computed in exact fp32. */
  void* ds_workspace;
  int64_t ds_workspace_bytes;
} fa_attn_params;

enum fa_bwd_part { FA_BWD_DELTA = 1, FA_BWD_DKDV = 2, FA_BWD_DQ = 4 };

/* Split-K decode: q (batch, heads_q, seqlen_q, head_dim), k/v (batch, heads_kv, seqlen_k, head_dim).
   Two kernel families: with fp16/bf16, head_dim 64 or 128, at most 128 query rows per kv head, TMA-compatible
   strides and an EVEN num_splits >= 2 the TMA + tcgen05 kernel runs (num_splits / 2 CTAs per (batch, kv head),
   two partials each); head_dim 256 runs on it with any num_splits >= 2 (one partial per CTA); anything else runs
   on the CUDA-core kernel.
   o_partial (num_splits, batch, heads_q, seqlen_q, head_dim) fp32 contiguous and
   lse_partial (num_splits, batch, heads_q, seqlen_q) fp32 contiguous are caller-allocated scratch. */
typedef struct fa_decode_params {
  int32_t dtype;
  int32_t batch, heads_q, heads_kv, seqlen_q, seqlen_k, head_dim;
  const void* q; int64_t q_strides[4];
  const void* k; int64_t k_strides[4];
  const void* v; int64_t v_strides[4];
  void* out;     int64_t o_strides[4];
  float softmax_scale;
  int32_t num_splits;
  float* o_partial;
  float* lse_partial;
  int32_t force_path;  /* 0 = automatic; FA_PATH_TCGEN05 (needs an even num_splits >= 2) or FA_PATH_SIMT */
  int32_t* status;     /* device int32 or NULL; set by the tensor-core kernel when a bounded wait ran out (the
                          abandoned slice then contributes an empty partial: zeros with LSE = -inf) */
} fa_decode_params;

/* LSE-weighted merge of `num_splits` partial results for `rows` independent rows.
   o_partial element (s, r, d) at o_partial[s*o_split_stride + r*o_row_stride + d];
   lse_partial element (s, r) at lse_partial[s*lse_split_stride + r*lse_row_stride].
   out row r at out + r*out_row_stride (elements of out_dtype); lse_out (fp32, may be NULL) gets the
   merged log-sum-exp per row. */
typedef struct fa_combine_params {
  int32_t out_dtype;
  int32_t rows, head_dim, num_splits;
  const float* o_partial; int64_t o_split_stride, o_row_stride;
  const float* lse_partial; int64_t lse_split_stride, lse_row_stride;
  void* out; int64_t out_row_stride;
  float* lse_out;
} fa_combine_params;

/* Multi-GPU merge of per-rank partials without a collective (no counterpart in the reference, which is single-GPU;
   the merge rule is fa_rdna3/kernels/decode.py:101-122). Every rank owns a buffer of `world` slots of slot_floats
   floats (a slot: rows * head_dim partial values, then rows LSEs) and `world` int32 flags, mapped into every other
   rank's address space (CUDA IPC or any other peer mapping: the caller's business). A call copies this rank's slot
   `rank` of its own buffer into slot `rank` of every peer's buffer with ordinary stores over NVLink, then raises
   flag `rank` there to `epoch`; a second kernel waits (bounded; a lost wait sets `status` and leaves out unwritten)
   until every flag of the local buffer has reached `epoch` and merges the local slots into `out`. Only stores cross
   the link; nothing here reads peer memory, and no TMA or multicast instruction is involved. `epoch` must grow with
   every call on a buffer; callers alternate between two buffers so that a fast rank cannot overwrite a slot a slow
   rank is still merging. */
#define FA_MAX_PEERS 16
typedef struct fa_peer_merge_params {
  int32_t world, rank;
  int32_t out_dtype, rows, head_dim;
  int32_t epoch;
  int64_t slot_floats;
  float* peer_base[FA_MAX_PEERS];     /* peer_base[r]: rank r's buffer as this process addresses it; [rank] = local */
  int32_t* peer_flags[FA_MAX_PEERS];  /* likewise the flag arrays */
  void* out; int64_t out_row_stride;
  float* lse_out;                     /* may be NULL */
  int32_t* status;                    /* may be NULL */
} fa_peer_merge_params;

/* Paged-KV decode: q (batch, heads_q, head_dim); caches (num_blocks, block_size, heads_kv, head_dim);
   block_table int32 (batch, max_blocks) and context_lens int32 (batch) with arbitrary strides.
   first_block / block_step restrict the call to logical blocks first_block, first_block + block_step, ...
   (a KV shard of a multi-GPU decode; 0 and 1 for the whole context).
   With num_splits == 1 and lse_out == NULL the result goes straight to out; otherwise
   o_partial (batch, heads_q, num_splits, head_dim) fp32 and lse_partial (batch, heads_q, num_splits) fp32
   are caller-allocated scratch and the merged result is written to out (and lse_out if not NULL). */
typedef struct fa_paged_params {
  int32_t dtype;
  int32_t batch, heads_q, heads_kv, head_dim;
  int32_t num_blocks, block_size, max_blocks;
  const void* q; int64_t q_strides[3];
  const void* k_cache; int64_t k_strides[4];
  const void* v_cache; int64_t v_strides[4];
  const int32_t* block_table; int64_t bt_strides[2];
  const int32_t* context_lens; int64_t cl_stride;
  void* out; int64_t o_strides[3];
  float softmax_scale;
  int32_t num_splits;
  int32_t first_block, block_step;
  float* o_partial;
  float* lse_partial;
  float* lse_out;           /* (batch, heads_q) fp32 contiguous or NULL */
  int32_t out_is_f32;       /* write out as fp32 regardless of dtype (shard partials) */
  int32_t force_path;       /* 0 = automatic; FA_PATH_TCGEN05 (needs an even num_splits >= 2) or FA_PATH_SIMT */
  int32_t* status;          /* device int32 or NULL, as in fa_decode_params */
  int32_t balance;          /* tensor-core kernel only. 0: num_splits / 2 CTAs per sequence, each sequence cut into
                               equal parts. 1: one CTA per SM, dealt to the sequences on the device in proportion to
                               their (clamped) context lengths, so ragged batches keep every SM busy without a host
                               read-back of context_lens; num_splits is then the number of partial slots per
                               sequence in o_partial / lse_partial (2 per CTA; 2 x SM count is always enough) and
                               batch may be at most 256 and at most the SM count. */
} fa_paged_params;

/* FP32 short-sequence attention: q, k, v, out (batch, heads, seqlen <= 32, 128), optional bias. */
typedef struct fa_tiny_params {
  int32_t batch, heads, seqlen, head_dim;
  const float* q; int64_t q_strides[4];
  const float* k; int64_t k_strides[4];
  const float* v; int64_t v_strides[4];
  float* out;     int64_t o_strides[4];
  const void* bias; int32_t bias_dtype; int64_t bias_strides[4];
  float softmax_scale;
} fa_tiny_params;

/* Library / device queries. */
FA_API int32_t fa_abi_version(void);
/* 0 when `device` is a compute-capability-10.x GPU, else a negative code (replaces the gfx1100 gate,
   fa_rdna3/_validation.py:22-37). */
FA_API int32_t fa_device_supported(int32_t device);
FA_API const char* fa_last_error_string(void);
/* fa_path of the calling thread's last fa_fwd / fa_bwd / fa_varlen_* call. */
FA_API int32_t fa_last_path(void);

/* Bytes of caller-provided scratch an entry point needs for the problem in `params` (the struct of that entry
   point), or a negative fa_error. The reference sizes the same buffers inline with torch.empty
   (fa_rdna3/interface.py:217-220 delta, :451-455 split-K partials, :696-699 paged partials). */
enum fa_workspace_kind {
  FA_WS_BWD_DELTA = 1,          /* fa_attn_params   -> delta */
  FA_WS_DECODE_O_PARTIAL = 2,   /* fa_decode_params -> o_partial (0 when num_splits == 1) */
  FA_WS_DECODE_LSE_PARTIAL = 3, /* fa_decode_params -> lse_partial */
  FA_WS_PAGED_O_PARTIAL = 4,    /* fa_paged_params  -> o_partial */
  FA_WS_PAGED_LSE_PARTIAL = 5,  /* fa_paged_params  -> lse_partial */
  FA_WS_BWD_DS = 6,             /* fa_attn_params   -> ds_workspace of fa_bwd (optional; 0 when the problem cannot use one) */
  FA_WS_FWD_P = 7               /* fa_attn_params   -> ds_workspace of fa_fwd (16-bit head dims above 256, fp32 to 256; else 0) */
};
FA_API int64_t fa_workspace_bytes(int32_t kind, const void* params);

/* Dense forward: writes out and lse. Replaces the _attention_forward launch,
   fa_rdna3/interface.py:154-199 (kernel fa_rdna3/kernels/forward.py:28-164). */
FA_API int32_t fa_fwd(const fa_attn_params* p, void* stream);

/* delta = rowsum(out * dout). Replaces the _attention_bwd_preprocess launch,
   fa_rdna3/interface.py:225-233 (kernel fa_rdna3/kernels/backward.py:18-46); varlen form
   fa_rdna3/interface.py:530-538. */
FA_API int32_t fa_bwd_delta(const fa_attn_params* p, void* stream);

/* Dense backward: computes delta, then dk/dv and dq. Replaces the three launches of
   fa_rdna3/interface.py:202-277 (kernels fa_rdna3/kernels/backward.py:56-322). */
FA_API int32_t fa_bwd(const fa_attn_params* p, void* stream);

/* Packed variable-length forward / backward (p->varlen must be 1). Replace
   fa_rdna3/interface.py:482-511 and :514-580 (kernels fa_rdna3/kernels/varlen.py:42-421). */
FA_API int32_t fa_varlen_fwd(const fa_attn_params* p, void* stream);
FA_API int32_t fa_varlen_bwd(const fa_attn_params* p, void* stream);

/* Split-K decode (partials + merge). Replaces the _attention_split and _attention_combine launches,
   fa_rdna3/interface.py:457-478 (kernels fa_rdna3/kernels/decode.py:13-125). */
FA_API int32_t fa_decode_splitk(const fa_decode_params* p, void* stream);

/* The same split-K decode for callers that must not allocate device memory (code running inside a pre-sized
   arena, plug-ins that only receive input and output buffers, latency-critical loops). It has no counterpart
   in the reference, which always allocates its partial buffers with torch.empty (fa_rdna3/interface.py:451-455).
   p->o_partial and p->lse_partial are ignored: the partials go to an 8 MiB array built into the library, which
   every GPU that loads the library holds until exit. The call is refused (FA_ERR_UNSUPPORTED) when
   num_splits * batch * heads_q * seqlen_q * (head_dim + 1) exceeds 2 Mi floats. It calls no allocator.
   All calls on a device share that array: calls whose kernels can overlap on the GPU race, calls on one stream
   do not. The first call on each device looks the array's address up (cudaGetSymbolAddress) with that device
   current; make it before any stream capture begins. */
FA_API int32_t fa_decode_splitk_noalloc(const fa_decode_params* p, void* stream);

/* Stand-alone LSE merge; also merges per-GPU shard partials. Replaces the _attention_combine launch,
   fa_rdna3/kernels/decode.py:80-125. */
FA_API int32_t fa_combine(const fa_combine_params* p, void* stream);

/* See fa_peer_merge_params. */
FA_API int32_t fa_peer_merge(const fa_peer_merge_params* p, void* stream);

/* Lets kernels of the current device store into memory of `peer_device` (cudaDeviceEnablePeerAccess; already enabled
   counts as success). Returns FA_ERR_UNSUPPORTED when the two devices have no peer path. */
FA_API int32_t fa_enable_peer_access(int32_t peer_device);

/* Paged-KV decode. Replaces the _attention_decode_paged (+ combine) launches,
   fa_rdna3/interface.py:703-727 (kernel fa_rdna3/kernels/paged.py:17-89). */
FA_API int32_t fa_decode_paged(const fa_paged_params* p, void* stream);

/* Test hook, no counterpart in the reference: makes the NEXT tensor-core decode launch (dense or paged) of the
   calling thread use `poll_limit` polls per barrier wait (0 = the default, about a second) and leave out the
   loads of tile `skip_tile` of every CTA (-1 = none), so that a wait runs out, the kernel leaves through its
   normal exit and the status word is set. Nothing faults and nothing hangs. */
FA_API void fa_test_decode_fault(uint32_t poll_limit, int32_t skip_tile);

/* FP32 short-sequence forward. Replaces the _attention_tiny_forward launch,
   fa_rdna3/interface.py:84-104 (kernel fa_rdna3/kernels/tiny.py:10-85). */
FA_API int32_t fa_tiny_fwd(const fa_tiny_params* p, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FA_B200_H_ */
