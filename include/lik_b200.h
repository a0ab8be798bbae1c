/*
 * lik_b200.h — C ABI of the B200 (sm_100a) MaxSim engine.
 *
 * The reference project (hcompai/late-interaction-kernels) is pure Python: its
 * GPU work is Triton kernels launched from Python launcher functions, so it has
 * no FFI of its own.  Each entry point below replaces one of those launchers;
 * the comment above it names the launcher (file:line inside the reference
 * repository) whose behaviour it reproduces.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the name ends in _host;
 *   - the caller allocates inputs, outputs and workspaces; the library never
 *     allocates device memory and never synchronises.  State it keeps per
 *     process: the error text of each thread, one auxiliary stream and two events
 *     per device for the backward (created on first use, see lik_maxsim_bwd), a
 *     count of the kernels it launched (lik_launch_count), and the device address
 *     of the built-in scratch array of lik_maxsim_fwd_static;
 *   - launches go to the cudaStream_t passed as lik_stream_t;
 *   - return value: LIK_OK or a negative lik_status; lik_last_error() gives the
 *     text for the calling thread;
 *   - data-dependent problems found on the device (a pair index out of range, a
 *     query longer than the argmax stride, a bounded wait that gave up) never
 *     trap: the kernel ORs a LIK_DEV_* bit into *status (if non-NULL), skips the
 *     offending work and returns.
 */
#ifndef LIK_B200_H
#define LIK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* lik_stream_t; /* cudaStream_t */

enum lik_dtype { LIK_F32 = 0, LIK_F16 = 1, LIK_BF16 = 2, LIK_E4M3 = 3 };

enum lik_status {
  LIK_OK = 0,
  LIK_ERR_INVALID = -1,     /* bad argument (NULL pointer, negative size, unknown enum) */
  LIK_ERR_UNSUPPORTED = -2, /* valid request this build has no kernel for */
  LIK_ERR_CUDA = -3,        /* a CUDA runtime/driver call failed */
  LIK_ERR_WORKSPACE = -4    /* workspace too small (see the *_workspace function) */
};

/* bits OR-ed into the device status word */
enum lik_dev_status {
  LIK_DEV_PAIR_RANGE = 1,   /* pair_q / pair_d entry outside [0, n_seq) */
  LIK_DEV_ARGMAX_STRIDE = 2,/* a query has more tokens than argmax_stride */
  LIK_DEV_WAIT_TIMEOUT = 4, /* a bounded mbarrier wait expired inside the tensor-core kernel */
  LIK_DEV_CODE_RANGE = 8,   /* PLAID centroid code outside [0, n_centroids) (read as centroid 0) */
  LIK_DEV_LEN_RANGE = 16,   /* a length exceeds the padded extent (clamped) */
  LIK_DEV_INTERNAL = 32     /* a kernel's own consistency check failed (the access was skipped) */
};

enum lik_normalize { LIK_NORM_NONE = 0, LIK_NORM_Q = 1, LIK_NORM_D = 2, LIK_NORM_BOTH = 3, LIK_NORM_ROUNDED = 4 };

enum lik_pairing {
  LIK_PAIR_CROSS = 0,   /* every query against every document: scores[i * d.n_seq + j] */
  LIK_PAIR_GROUPED = 1, /* document j belongs to query j / group: scores[j]            */
  LIK_PAIR_LIST = 2     /* explicit list: scores[p] = MaxSim(q[pair_q[p]], d[pair_d[p]]) */
};

/*
 * One side of a MaxSim problem: token sequences stored as rows of one matrix.
 *   padded layout (cu == NULL): sequence i occupies rows [i*seq_stride, i*seq_stride + max_len);
 *       token t of it is valid when t < lens[i] (lens optional) and mask[row] != 0 (mask optional).
 *   packed layout (cu != NULL): sequence i occupies rows [cu[i], cu[i+1]).
 * mask and scale are indexed by row number, like data.
 */
typedef struct lik_seqs {
  const void* data;     /* [n_rows, dim] row-major */
  int64_t row_stride;   /* elements between consecutive rows */
  int64_t n_rows;       /* rows addressable from data */
  int32_t n_seq;
  int32_t max_len;      /* padded: stored length; packed: upper bound used to size per-query buffers */
  int64_t seq_stride;   /* padded: rows between sequence starts */
  const int32_t* cu;    /* packed: [n_seq + 1] */
  const int32_t* lens;  /* padded, optional: [n_seq] */
  const uint8_t* mask;  /* padded, optional: [n_rows] */
  const float* scale;   /* optional per-token dequantisation scale: [n_rows] */
  float scale_scalar;   /* multiplies every token (1.0f when unused) */
  int32_t reserved;
} lik_seqs;

/* ------------------------------------------------------------------------- */
/* Forward.  Replaces _run_forward (forward.py:228-346), _varlen_forward        */
/* (varlen.py:271-364), _scatter_forward (score_pairs.py:281-341) and the FP8   */
/* launcher maxsim_inference_fp8 (fp8.py:234-422).                              */
/*   scores[p] = sum_{valid s} max_{valid t} <q_s, d_t> * scales                */
/*   argmax (optional) [n_scores, argmax_stride] int32: winning token of the    */
/*   document for every query token, relative to the document start; -1 when    */
/*   the document has no valid token, and for positions >= the query length.    */
/* normalize: bit 0 (LIK_NORM_Q) / bit 1 (LIK_NORM_D): divide the query /       */
/* document tokens by max(||x||, 1e-12) as part of the call (fused L2 norm).   */
/* By default the scoring kernel multiplies the raw dot products by fp32       */
/* inverse norms, so scores and winners follow the fp32 oracle (reference.py). */
/* With LIK_NORM_ROUNDED (bit 2) and 16-bit inputs the operands are instead    */
/* normalised in fp32 and rounded back to their type into workspace copies,    */
/* which is what the reference's GPU kernel does (forward.py:120-126) and is   */
/* faster; near-ties may then pick another winner, so it is meant for search.  */
/* ------------------------------------------------------------------------- */
typedef struct lik_fwd_args {
  lik_seqs q, d;
  int32_t dtype; /* lik_dtype of q.data and d.data */
  int32_t dim;
  int32_t pairing;
  int32_t group; /* LIK_PAIR_GROUPED: documents per query */
  const int32_t* pair_q;
  const int32_t* pair_d;
  int64_t n_pairs; /* LIK_PAIR_LIST */
  int32_t normalize;
  int32_t engine; /* 0 = automatic, 1 = force the portable fp32 kernel, 2 = force the tcgen05 kernel */
  float* scores;
  int32_t* argmax;
  int32_t argmax_stride;
  int32_t reserved;
  void* workspace;
  size_t workspace_bytes;
  int32_t* status;
} lik_fwd_args;

size_t lik_maxsim_fwd_workspace(const lik_fwd_args* args);
int lik_maxsim_fwd(const lik_fwd_args* args, lik_stream_t stream);

/*
 * lik_maxsim_fwd_static — the same forward for callers that have no way to hand over device
 * scratch.  (No counterpart in the reference; added for this library.)
 *
 * Some embedders of this ABI run inside a host that owns all device memory — a serving runtime
 * with a fixed memory plan, a plugin sandbox that forbids cudaMalloc, a process that must not touch
 * the allocator while a CUDA graph pool is live.  They can pass inputs and outputs they were given,
 * but they cannot allocate the workspace lik_maxsim_fwd asks for.  This entry point takes the same
 * argument struct, ignores args->workspace / workspace_bytes and uses a scratch array that is part
 * of the library's device image instead (LIK_STATIC_SCRATCH_BYTES, resident on every GPU that loads
 * the library until the process exits).  It allocates nothing and frees nothing.
 *
 * Limits and rules:
 *   - problems whose lik_maxsim_fwd_workspace() exceeds LIK_STATIC_SCRATCH_BYTES are refused with
 *     LIK_ERR_WORKSPACE (roughly: fused L2 norm over more than 4 M token rows, or very long queries
 *     against very many documents);
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress);
 *     make that first call outside any stream capture, with the device current;
 *   - all calls on a device share the one array.  Its previous contents are never relied on (every
 *     region is rewritten before it is read, nothing needs zeroing), but two calls whose kernels
 *     overlap on the GPU — different streams, no ordering — would race on it: serialise them.
 */
#define LIK_STATIC_SCRATCH_BYTES (16u << 20)
int lik_maxsim_fwd_static(const lik_fwd_args* args, lik_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Backward.  Replaces maxsim_backward_unified (backward/unified.py:205-289),   */
/* maxsim_backward_lowmem (backward/lowmem.py:205-322), the varlen backward     */
/* (varlen.py:389-449) and the pair-list backward (score_pairs.py:356-420).     */
/*   grad_q[row(i,s)] = sum_p g[p] * d[row(j_p, argmax[p,s])]                   */
/*   grad_d[row(j,t)] = sum_{p,s : argmax[p,s]=t} g[p] * q[row(i_p,s)]          */
/* normalize: bit LIK_NORM_Q / LIK_NORM_D = that side was L2-normalised by the  */
/* forward; its Jacobian (autograd.py:213-225) is applied inside the kernels     */
/* (LIK_NORM_BOTH for maxsim(normalize=True); LIK_NORM_D alone for a projected    */
/* document head).  grad_q / grad_d are [n_rows, dim] contiguous.                */
/* deterministic != 0 (CROSS and GROUPED pairing): destination-owned reduction, */
/* grads written once in grad_dtype, bitwise reproducible.  deterministic == 0: */
/* fp32 atomics into the workspace followed by a finalise pass.                 */
/* ------------------------------------------------------------------------- */
typedef struct lik_bwd_args {
  lik_seqs q, d;
  int32_t dtype;
  int32_t dim;
  int32_t pairing;
  int32_t group;
  const int32_t* pair_q;
  const int32_t* pair_d;
  int64_t n_pairs;
  int32_t normalize;
  int32_t deterministic;
  const float* grad_scores;
  const int32_t* argmax;
  int32_t argmax_stride;
  int32_t grad_dtype; /* lik_dtype of grad_q / grad_d (F32, F16 or BF16) */
  void* grad_q;       /* may be NULL to skip */
  void* grad_d;       /* may be NULL to skip */
  void* workspace;
  size_t workspace_bytes;
  int32_t* status;
} lik_bwd_args;

size_t lik_maxsim_bwd_workspace(const lik_bwd_args* args);
/* All work is ordered after what `stream` already holds and before anything enqueued on it afterwards.
 * When both gradients are requested on a large problem, the grad_q kernel is enqueued on a stream the
 * library creates once per device (event fork from `stream`, event join back into it), so that it runs
 * beside the grad_d kernels; callers only ever synchronise with `stream`. */
int lik_maxsim_bwd(const lik_bwd_args* args, lik_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Top-k.  Replaces the torch.topk / cat / topk merge loop of maxsim_topk        */
/* (topk.py:41-86) and retrieve (retrieve.py:254-310).                          */
/* lik_topk_rows: per row of scores [n_rows, n_cols] (row stride ld) keep the k */
/* best as (score, index + index_offset), sorted best first; ties go to the     */
/* lower index.  k <= LIK_TOPK_MAX.  If merge != 0 the k entries already in      */
/* out_scores/out_index take part (running merge across chunks).  Entries with  */
/* index < 0 are padding.                                                       */
/* lik_topk_merge: cand_* are [n_lists, n_rows, k]; result is the top k of the  */
/* union per row (used for per-CTA partial lists and for the all-gathered       */
/* per-GPU lists of the sharded retrieve).                                      */
/* ------------------------------------------------------------------------- */
#define LIK_TOPK_MAX 8192
int lik_topk_rows(const float* scores, int64_t n_rows, int64_t n_cols, int64_t ld, int32_t k, int32_t largest,
                  int64_t index_offset, int32_t merge, float* out_scores, int64_t* out_index, lik_stream_t stream);
int lik_topk_merge(const float* cand_scores, const int64_t* cand_index, int32_t n_lists, int64_t n_rows, int32_t k,
                   int32_t largest, float* out_scores, int64_t* out_index, lik_stream_t stream);

/* ------------------------------------------------------------------------- */
/* PLAID.                                                                       */
/* lik_plaid_decompress: emb = centroids[code] + bucket_weights[bucket(f)],     */
/* optional L2 norm, written as out_dtype rows [n_tokens, dim] — the            */
/* decompress stage of _maxsim_residual_kernel (plaid.py:236-284) and           */
/* _maxsim_residual_varlen_kernel (plaid.py:684-829), run once per token instead*/
/* of once per (query, document) program.  Bit layout: feature f is in byte     */
/* f / (8/nbits), bit offset (f % (8/nbits)) * nbits (reference.py:124-139).     */
/* lik_plaid_approx: replaces plaid_approx_score (plaid.py:82-136).             */
/* lik_plaid_bwd_dq: replaces _maxsim_residual_bwd_dQ_kernel + the Q Jacobian    */
/* (plaid.py:310-401, 596-605).                                                 */
/* ------------------------------------------------------------------------- */
typedef struct lik_plaid_index {
  const int32_t* codes;       /* [n_tokens] */
  const uint8_t* residuals;   /* [n_tokens, packed_dim], packed_dim = ceil(dim*nbits/8) */
  int64_t n_tokens;
  const void* centroids;      /* [n_centroids, dim] */
  int32_t centroid_dtype;     /* LIK_F32 / LIK_F16 / LIK_BF16 */
  int32_t n_centroids;
  const float* bucket_weights;/* [1 << nbits] */
  int32_t nbits;              /* 2, 4 or 8 */
  int32_t dim;
} lik_plaid_index;

int lik_plaid_decompress(const lik_plaid_index* index, int64_t token_begin, int64_t token_count, int32_t normalize,
                         void* out, int32_t out_dtype, int32_t* status, lik_stream_t stream);
int lik_plaid_approx(const float* qcs, int32_t n_centroids, int32_t lq, const int32_t* codes, int64_t n_docs,
                     int32_t max_ld, const int64_t* doc_lengths, float* out, lik_stream_t stream);
/* grad_q [n_q, lq, dim] fp32 from argmax [n_q, n_docs, lq] over a padded index (row of doc j token t = j*max_ld + t) */
int lik_plaid_bwd_dq(const lik_plaid_index* index, int32_t max_ld, int64_t n_docs, const void* q, int32_t q_dtype,
                     int32_t n_q, int32_t lq, const float* grad_scores, const int32_t* argmax, int32_t normalize,
                     float* grad_q, lik_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Scoring fused with the per-query top-k.  Replaces the chunk loop of          */
/* maxsim_topk (topk.py:41-86: score a chunk, torch.topk, cat, torch.topk) and  */
/* of retrieve (retrieve.py:194-310) by ONE pass of the scoring kernel over all */
/* documents: no [n_q, n_docs] and no [n_q, chunk] score matrix exists; every   */
/* (query, document) score is offered to a candidate list of its query straight */
/* from the accumulator epilogue, lists are cut back to their k best as they    */
/* fill, and a merge kernel writes the k best per query, best first, ties to    */
/* the lower document index (the order lik_topk_rows uses).                     */
/* args: a lik_fwd_args with LIK_PAIR_CROSS pairing; scores / argmax unused.    */
/* Supported (lik_maxsim_fwd_topk_supported() == 1): bf16 / fp16 / e4m3 inputs  */
/* the tcgen05 kernel takes, padded queries of at most 128 tokens, k <= 128.    */
/* Anything else: use lik_maxsim_fwd per chunk + lik_topk_rows.                 */
/* out_index = document index + index_offset.  Fewer than k documents: the      */
/* remaining entries are (-inf / +inf, -1).                                     */
/* ------------------------------------------------------------------------- */
/* A corpus that does not sit in memory as one matrix is scored piece by piece into the SAME workspace:  */
/* every call but the first sets LIK_TOPK_CONTINUE (keep the candidate lists of the earlier pieces),     */
/* every call but the last sets LIK_TOPK_PARTIAL (no merge, nothing written to out_*); doc_base is the   */
/* index of the piece's first document (pieces in ascending order, same queries, same k).                */
enum lik_topk_flags { LIK_TOPK_CONTINUE = 1, LIK_TOPK_PARTIAL = 2 };
typedef struct lik_topk_spec {
  int32_t k;
  int32_t largest;      /* 0: the k smallest scores */
  int64_t index_offset;
  float* out_scores;    /* [q.n_seq, k] */
  int64_t* out_index;   /* [q.n_seq, k] */
  int32_t flags;        /* lik_topk_flags */
  int32_t doc_base;     /* added to the document index of this call's documents */
} lik_topk_spec;

int lik_maxsim_fwd_topk_supported(const lik_fwd_args* args, const lik_topk_spec* topk);
size_t lik_maxsim_fwd_topk_workspace(const lik_fwd_args* args, const lik_topk_spec* topk);
int lik_maxsim_fwd_topk(const lik_fwd_args* args, const lik_topk_spec* topk, lik_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Scoring straight from a compressed index: ONE kernel gathers centroid rows,  */
/* unpacks the residual codes, adds bucket weights, normalises, rounds to the   */
/* operand type and feeds the tensor cores (the decode stage runs in the        */
/* kernel's producer warps and writes the operand tiles into shared memory).    */
/* Replaces _maxsim_residual_forward (plaid.py:404-515) and the launcher of     */
/* maxsim_residual_varlen (plaid.py:832-963); with topk != NULL the scores go   */
/* into the same fused top-k as above instead of a [n_q, n_docs] matrix.        */
/* args: q = the queries (bf16 or fp16); d describes the document layout only   */
/* (d.data == NULL, rows = tokens of the index: packed cu or padded lens);      */
/* normalize bit LIK_NORM_D = normalise the decoded tokens, LIK_NORM_Q = the    */
/* queries.  Supported: width a multiple of 16 and at most 128, 16-byte aligned */
/* centroid rows.  Otherwise decode with lik_plaid_decompress and score the     */
/* rows with lik_maxsim_fwd: both ways give the same bits.                      */
/* ------------------------------------------------------------------------- */
int lik_plaid_fwd_supported(const lik_fwd_args* args, const lik_plaid_index* index, const lik_topk_spec* topk);
size_t lik_plaid_fwd_workspace(const lik_fwd_args* args, const lik_plaid_index* index, const lik_topk_spec* topk);
int lik_plaid_fwd(const lik_fwd_args* args, const lik_plaid_index* index, const lik_topk_spec* topk, lik_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Document head in front of MaxSim.  Replaces the forward launcher of          */
/* maxsim_from_hidden (fused_head.py:262-330, kernel fused_head.py:40-260):     */
/*   scores[i, j] = MaxSim(q_i, normalize(h_j @ w^T + bias))                    */
/* One kernel: the projection of a 128-token tile runs on the tensor cores      */
/* into tensor memory, is rounded to the operand type (plus bias), written to   */
/* shared memory as the operand of the scoring MMA, and scored against the      */
/* resident queries; the projected tokens never reach device memory.  The       */
/* inverse norms come from the rounded values and are applied in fp32 to the    */
/* raw dot products, as lik_maxsim_fwd does with LIK_NORM_D.                    */
/*   q: padded queries [n_seq * max_len, d_out] (no mask, no lens); at most two */
/*      128-row tiles of whole queries.   h: padded documents [n_rows, d_model] */
/*      (mask / lens optional).   w [d_out, d_model], bias [d_out] or NULL, all */
/*      of `dtype` (LIK_BF16 or LIK_F16); d_out a multiple of 32 up to 128.     */
/*   argmax (optional) [n_q * n_d, argmax_stride] as for lik_maxsim_fwd.        */
/* lik_maxsim_hidden_fwd_supported says whether this kernel takes the problem;  */
/* callers project with a GEMM and call lik_maxsim_fwd otherwise.               */
/* ------------------------------------------------------------------------- */
typedef struct lik_hidden_fwd_args {
  lik_seqs q;          /* projected queries */
  lik_seqs h;          /* hidden states of the document tokens */
  const void* w;       /* [d_out, d_model] */
  int64_t w_stride;    /* elements between rows of w */
  const void* bias;    /* [d_out] or NULL */
  int32_t dtype;
  int32_t d_model;
  int32_t d_out;
  int32_t normalize;   /* LIK_NORM_D or LIK_NORM_NONE */
  float* scores;       /* [q.n_seq, h.n_seq] */
  int32_t* argmax;
  int32_t argmax_stride;
  int32_t reserved;
  void* workspace;
  size_t workspace_bytes;
  int32_t* status;
} lik_hidden_fwd_args;

int lik_maxsim_hidden_fwd_supported(const lik_hidden_fwd_args* args);
size_t lik_maxsim_hidden_fwd_workspace(const lik_hidden_fwd_args* args);
int lik_maxsim_hidden_fwd(const lik_hidden_fwd_args* args, lik_stream_t stream);

/* Backward of the document head (fused_head.py:332-456): only winning tokens carry gradient, so the  */
/* backward gathers them into "compact" documents, runs lik_maxsim_bwd on those and scatters the rows  */
/* of grad_h back.                                                                                     */
/* lik_hidden_winners: per document j, the distinct winners over all (query, query token), ascending:  */
/*   counts[j] of them (at most `slots`, which must be >= min(n_q * lq, ld)); rows[j * slots + p] =     */
/*   j * ld + token of compact slot p (unused slots repeat the document's first row);                   */
/*   compact_argmax [n_q, n_d, lq] = position of each winner inside its compact document (-1: none);    */
/*   bitmap / prefix [n_d, ceil(ld / 32)]: which tokens won, and how many winners precede each word.    */
/* lik_hidden_scatter_rows: grad_h [n_d * ld rows of row_bytes] = the compact row of every winning     */
/*   token (compact_rows [n_d * slots rows]), zeros elsewhere; every row is written exactly once.       */
int lik_hidden_winners(const int32_t* argmax, int32_t n_q, int32_t n_d, int32_t lq, int32_t ld, int32_t slots,
                       int32_t* compact_argmax, int64_t* rows, int32_t* counts, uint32_t* bitmap, int32_t* prefix,
                       int32_t* status, lik_stream_t stream);
int lik_hidden_scatter_rows(const void* compact_rows, int64_t row_bytes, int32_t n_d, int32_t ld, int32_t slots,
                            const uint32_t* bitmap, const int32_t* prefix, void* grad_h, lik_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Utilities                                                                    */
/* ------------------------------------------------------------------------- */
/* out[r] = 1 / max(||x_r||, eps) for every row; the fused-normalise kernels take these. */
int lik_row_inv_norm(const void* data, int32_t dtype, int64_t n_rows, int32_t dim, int64_t row_stride, float eps,
                     float* out, lik_stream_t stream);
/* Self-test of the bounded waits: every wait inside the tensor-core kernel (on a TMA stage, an accumulator, the unit
 * ring) gives up after a cycle limit, raises LIK_DEV_WAIT_TIMEOUT, lets the CTA drain and return.  This launches one
 * thread that runs that same wait on a barrier nothing arrives at, with limit_cycles (at most 2e8, a tenth of a
 * second) as its limit.  result (device, int32[3]) = {what the wait returned (0 = gave up), the CTA's abort flag,
 * cycles spent}.  Nothing faults, traps or hangs.  (No counterpart in the reference, whose length checks trap.) */
int lik_selftest_wait_timeout(int64_t limit_cycles, int32_t* status, int32_t* result, lik_stream_t stream);
const char* lik_last_error(void);
/* kernels this library has launched in this process so far (all threads, all devices) */
uint64_t lik_launch_count(void);
int lik_version(void);
/* 1 when the device the calling thread has current is sm_100 (tcgen05 kernels usable) */
int lik_device_supported(void);

#ifdef __cplusplus
}
#endif
#endif /* LIK_B200_H */
