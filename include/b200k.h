/*
 * b200k — C ABI of the B200 (sm_100a) dense-contraction kernel library.
 *
 * This is the boundary that replaces the native launch path underneath iree-turbine's
 * operator surface.  In the reference every custom op ends in
 * `eager_dispatch` (iree/turbine/runtime/op_reg/eager.py:58-206), which JIT-compiles an IREE
 * module (runtime/op_reg/compiler.py:105-220), imports torch tensors through dlpack
 * (runtime/device.py:561-591) and invokes the VM after a host-side stream synchronize
 * (runtime/invoke.py:28-75, runtime/device.py:158-162).  For the Wave kernel templates the same
 * role is played by the `wave_runtime` native module named in requirements-wave-runtime.txt:2.
 * The functions below take what that path takes after marshalling: raw device pointers,
 * sizes, strides, scalars and the caller's CUDA stream.
 *
 * Conventions
 *   - All pointers are device pointers unless a comment says "host".
 *   - `stream` is a `cudaStream_t` passed as `void*` (0 = the legacy default stream).
 *     Every launch is asynchronous on that stream; no function synchronizes the host.
 *   - The library never allocates or frees tensor memory.  Outputs and workspaces are
 *     allocated by the caller (see the *_workspace_bytes queries).
 *   - Every function returns a b200k_status.  Arguments are validated before any launch;
 *     on failure nothing has been enqueued.  b200k_last_error() returns a thread-local
 *     human-readable message for the most recent non-OK status on the calling thread.
 *   - No exceptions cross this boundary and nothing aborts the process.
 */
#ifndef B200K_H_
#define B200K_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200K_ABI_VERSION 3

typedef enum b200k_status {
  B200K_OK = 0,
  B200K_ERR_BAD_SHAPE = -1,        /* a dimension is non-positive or unsupported          */
  B200K_ERR_BAD_ALIGN = -2,        /* a pointer or stride violates the 16-byte rules       */
  B200K_ERR_BAD_DTYPE = -3,        /* dtype combination not implemented                    */
  B200K_ERR_UNSUPPORTED_ARCH = -4, /* current device is not compute capability 10.x        */
  B200K_ERR_CUDA = -5,             /* a CUDA runtime / driver call failed                  */
  B200K_ERR_NULL = -6,             /* a required pointer is NULL                           */
  B200K_ERR_TIMEOUT = -7,          /* reported through the status word: a device wait gave up */
  B200K_ERR_WORKSPACE = -8         /* workspace too small                                  */
} b200k_status;

typedef enum b200k_dtype {
  B200K_F16 = 0,
  B200K_BF16 = 1,
  B200K_F32 = 2,
  B200K_E4M3 = 3 /* float8_e4m3fn */
} b200k_dtype;

/* ---- library ---------------------------------------------------------------------- */

/* Returns B200K_ABI_VERSION of the built library. */
int b200k_abi_version(void);

/* Thread-local message describing the last non-OK status returned on this thread. */
const char* b200k_last_error(void);

/* Human-readable name of a status code. */
const char* b200k_status_string(int status);

/*
 * Device status word.  Kernels that wait on barriers bound every wait; when one gives up the
 * kernel ORs a non-zero code into this word and exits cleanly.  The word lives in device
 * memory owned by the caller (4 bytes, zero-initialised by the caller).  Passing NULL in the
 * args structs is allowed; the code is then dropped.  Bits: 0 GEMM wait gave up, 1 attention
 * forward wait gave up, 2 block-table entry outside the pool, 3 a seq_lens entry was cut to
 * max_seq_len, 4 the bounded-wait self-test, 5 a split-K GEMM found itself in a cluster of another
 * size than it was launched for (nothing written), 6 attention backward wait gave up.
 */

/* ---- GEMM:  C[M,N] = A[M,K] * B[N,K]^T  ------------------------------------------- */
/*
 * Replaces the Wave GEMM template launch (A row-major M x K, B stored N x K, fp32
 * accumulate).  The same NT convention is what the reference's GEMMForward computes with
 * transpose_b (iree/turbine/kernel/boo/op_exports/gemm.py:217-230).
 *
 *   in_dtype  F16 | BF16  -> out_dtype F32 | F16 | BF16
 *   in_dtype  E4M3        -> out_dtype BF16 | F32, result multiplied by (*scale_a) * (*scale_b)
 *
 * lda / ldb / ldc are row strides in ELEMENTS.  A, B: 16-byte aligned base, row stride a
 * multiple of 16 bytes.  C: base aligned to 16 bytes, ldc * sizeof(out) a multiple of 16.
 * K tails, M tails and N tails are handled (out-of-range operand elements read as zero).
 *
 * The kernel is launched as a programmatic dependent launch: its barrier set-up and tensor-memory
 * allocation may overlap the end of the previous kernel of the stream, and it waits for that
 * kernel before reading an operand or writing C, so the caller sees plain stream order.
 */
enum { B200K_ACT_NONE = 0, B200K_ACT_RELU = 1, B200K_ACT_GELU = 2 /* erf form */, B200K_ACT_SILU = 3 };

typedef struct b200k_gemm_args {
  const void* a;
  const void* b;
  void* c;
  int64_t m, n, k;
  int64_t lda, ldb, ldc;
  int32_t in_dtype;
  int32_t out_dtype;
  const float* scale_a; /* device scalar, E4M3 only, may be NULL (= 1.0) */
  const float* scale_b; /* device scalar, E4M3 only, may be NULL (= 1.0) */
  int32_t* status;      /* device status word, may be NULL */
  int32_t tile_n;       /* 0 = choose; else 128 or 256 */
  int32_t tile_m;       /* 0 = choose; else 128 or 256 (256 needs tile_n 256 or 0) */
  /* Optional fused epilogue (the bias / activation tail of a linear layer, cf. the reference's
   * ops/templates/test_linear_trailing_optional_biased.mlir):  C = act(A B^T * scales + bias[n]).
   * bias: device vector of n elements, NULL = none; activation: B200K_ACT_*. */
  const void* bias;
  int32_t bias_dtype; /* F32 | F16 | BF16 */
  int32_t activation;
  /* Operand storage, F16 / BF16 only (0, 0 = the NT form above).  a_km != 0: A is stored [K, M]
   * (lda = its row stride >= M), i.e. the product uses A^T of the stored matrix; b_kn != 0: B is
   * stored [K, N] (ldb >= N).  With these the four BLAS forms and the two backward products of
   * the NT form (dA = dC B: b_kn; dB = dC^T A: a_km and b_kn; kernel/boo/op_exports/gemm.py:233-270)
   * run without repacking an operand. */
  int32_t a_km;
  int32_t b_kn;
  /* Batched product (aten::bmm, which the reference's BOO layer lists beside mm and addmm,
   * kernel/boo/op_exports/registry.py:99-104): batch > 1 independent problems of the same shape,
   * problem i reading a + i * a_batch_stride, b + i * b_batch_stride and writing c + i *
   * c_batch_stride (strides in ELEMENTS; the A / B strides multiples of 16 bytes).  All problems'
   * tiles go through one persistent launch.  batch 0 or 1 = a single problem (strides ignored). */
  int64_t batch;
  int64_t a_batch_stride, b_batch_stride, c_batch_stride;
  /* Split-K: 0 = the library decides, 1 = never, 2 / 4 / 8 = that many CTAs (one thread-block
   * cluster) share every 128-row output tile, each summing a slice of K; the fp32 partial tiles
   * stay in the CTAs' shared memory and are added in rank order through distributed shared
   * memory, so no scratch is needed and a result is reproducible bit for bit.  For problems whose
   * whole tiles would leave most SMs idle (few output tiles, long K: weight gradients, narrow
   * projections).  Not available with tile_m 256 or in b200k_gemm_nt_allgather. */
  int32_t split_k;
  int32_t reserved;
} b200k_gemm_args;

int b200k_gemm_nt(const b200k_gemm_args* args, void* stream);

/*
 * Column-parallel GEMM fused with the all-gather of its result (the exchange step of the fp8
 * GEMM when it is sharded over N across the GPUs of one box; no counterpart in the reference,
 * which has no collective call site).  The rank computes C[:, col_offset : col_offset + n] from
 * its rows of B and writes every tile directly into the FULL matrix of each rank listed in
 * peer_c (its own included) through peer-mapped memory: every staged piece of a tile (32 rows x
 * 128 bytes) leaves as one bulk tensor store per rank (plain_stores: as 16-byte stores; multicast_c:
 * as one multimem store).  The transfer overlaps the math tile by tile and no staging copy or
 * separate collective is needed.  Only stores cross to other GPUs; nothing is loaded from a peer.
 *
 *   gemm        the local problem (a, b, m, n = shard width, k, lda, ldb, dtypes, scales);
 *               gemm.c and gemm.ldc are ignored
 *   peer_c[i]   base of rank i's full [m, peer_ldc] output, addressable from this device
 *   peer_ldc    row pitch of the full matrix in elements; col_offset: first column of the shard
 * Row pitch, column offset and shard width must be multiples of 16 bytes.  Completion on this
 * stream only means this rank's stores were issued and are visible at system scope after a
 * stream synchronize; readers on other ranks need a cross-rank barrier after that.
 */
typedef struct b200k_gemm_allgather_args {
  b200k_gemm_args gemm;
  void* peer_c[8];
  int32_t num_peers;
  int32_t self_index;  /* this rank's position in peer_c: peers are written in the order self + 1,
                          self + 2, ..., self, so that at any moment the ranks aim at different
                          destinations */
  int64_t peer_ldc;
  int64_t col_offset;
  void* multicast_c;   /* optional: the NVSwitch multicast address of the same matrix (one
                          multimem.st then reaches every rank, the switch replicates it); NULL =
                          one store per peer */
  int32_t plain_stores; /* 0: every staged 32-row x 128-byte piece goes to each rank as one bulk tensor
                           store (TMA) through a tensor map over that rank's matrix; != 0: as 16-byte
                           stores issued by the epilogue warps.  Ignored with multicast_c. */
  int32_t reserved;
} b200k_gemm_allgather_args;

int b200k_gemm_nt_allgather(const b200k_gemm_allgather_args* args, void* stream);

/* ---- attention forward (vanilla and causal) ---------------------------------------- */
/*
 * Replaces the Wave vanilla / causal attention template launch.
 * O = softmax(scale * Q K^T [+ causal mask]) V per (batch, head); fp32 scores, running max
 * and running sum; output in the input dtype.  The blockwise online-softmax structure is the
 * one stated in the reference's tests/kernel/fused_attention_test.py:43-77, with natural-base
 * softmax semantics as in aten::scaled_dot_product_attention (which the reference rewrites
 * SDPA variants to, iree/turbine/kernel/boo/fusion/replacement.py:239-290).
 *
 * Layout: Q [batch, q_heads, seq_q, head_dim], K/V [batch, kv_heads, seq_kv, head_dim],
 * O like Q; innermost dimension contiguous; strides below are in ELEMENTS.
 * q_heads must be a multiple of kv_heads (query head h reads kv head h / (q_heads/kv_heads)).
 * head_dim must be 128 or 64.  Causal masking aligns the last query with the last key
 * (query i sees keys j <= i + seq_kv - seq_q).
 *
 * Two kernels implement the call.  B200K_ATTN_ONE_TILE: a work item is one 128-row query tile,
 * two softmax warpgroups take alternate KV steps (head_dim 128 only).  B200K_ATTN_TILE_PAIR: a
 * work item is a pair of query tiles that share every K/V tile, one softmax warpgroup each; causal
 * problems are dealt out in (heavy, light) couples of equal cost.  B200K_ATTN_AUTO picks the pair
 * kernel for head_dim 64 and for causal problems whose couples fill the SMs evenly, else the
 * one-tile kernel (the measured winner in each case).  Results of the two agree within rounding
 * of the 16-bit probabilities, not bitwise.
 */
enum { B200K_ATTN_AUTO = 0, B200K_ATTN_ONE_TILE = 1, B200K_ATTN_TILE_PAIR = 2 };

typedef struct b200k_attention_args {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  int32_t batch, q_heads, kv_heads, seq_q, seq_kv, head_dim;
  int64_t q_stride_b, q_stride_h, q_stride_s;
  int64_t k_stride_b, k_stride_h, k_stride_s;
  int64_t v_stride_b, v_stride_h, v_stride_s;
  int64_t o_stride_b, o_stride_h, o_stride_s;
  int32_t dtype; /* F16 | BF16 */
  int32_t causal;
  float scale;
  int32_t* status; /* device status word, may be NULL */
  float* lse;      /* optional output [batch, q_heads, seq_q] (contiguous fp32), may be NULL:
                      ln sum_j exp(scale * q_i . k_j) over the visible keys, -inf for a row that sees
                      none; b200k_attention_bwd takes it to skip recomputing the row statistics */
  int32_t kernel;  /* B200K_ATTN_AUTO | B200K_ATTN_ONE_TILE | B200K_ATTN_TILE_PAIR */
  int32_t reserved;
} b200k_attention_args;

int b200k_attention_fwd(const b200k_attention_args* args, void* stream);

/*
 * Attention backward: given q, k, v, the forward output o and its gradient d_o (layouts, head
 * grouping, causal alignment and scale as in b200k_attention_fwd), writes
 *   d_q [batch, q_heads, seq_q, head_dim],  d_k and d_v [batch, kv_heads, seq_kv, head_dim]
 * (head_dim 128 or 64; for grouped-query heads d_k / d_v are summed over the query heads of a group).  Nothing but o is
 * needed from the forward call: the row statistics are recomputed.  No atomics are used; results
 * do not depend on the grid.  workspace: device memory, 16-byte aligned, at least
 * b200k_attention_bwd_workspace_bytes(args) bytes (two fp32 values per query row); contents need
 * not be preserved between calls.
 * The reference lists attention backward beside its GEMM backward (kernel/boo/op_exports/gemm.py:233-270,
 * wrapped as in kernel/boo/ops/conv.py:313-372) without a kernel of its own; the formulas are the
 * ones torch.autograd derives for softmax(scale * q k^T) v.
 */
typedef struct b200k_attention_bwd_args {
  const void* q;
  const void* k;
  const void* v;
  const void* o;
  const void* d_o;
  void* d_q;
  void* d_k;
  void* d_v;
  void* workspace;
  uint64_t workspace_bytes;
  int32_t batch, q_heads, kv_heads, seq_q, seq_kv, head_dim;
  int64_t q_stride_b, q_stride_h, q_stride_s;
  int64_t k_stride_b, k_stride_h, k_stride_s;
  int64_t v_stride_b, v_stride_h, v_stride_s;
  int64_t o_stride_b, o_stride_h, o_stride_s;
  int64_t do_stride_b, do_stride_h, do_stride_s;
  int64_t dq_stride_b, dq_stride_h, dq_stride_s;
  int64_t dk_stride_b, dk_stride_h, dk_stride_s;
  int64_t dv_stride_b, dv_stride_h, dv_stride_s;
  int32_t dtype; /* F16 | BF16 */
  int32_t causal;
  float scale;
  int32_t reserved;
  int32_t* status;  /* device status word, may be NULL; bit 6 = a bounded wait ran out */
  const float* lse; /* optional: the lse output of b200k_attention_fwd for the same q, k, v; NULL =
                       recompute the row statistics (one more pass over K in the dQ kernel) */
} b200k_attention_bwd_args;

uint64_t b200k_attention_bwd_workspace_bytes(const b200k_attention_bwd_args* args);
int b200k_attention_bwd(const b200k_attention_bwd_args* args, void* stream);

/*
 * Attention forward over a PAGED K/V cache (prefill, or a chunk of it, after its K/V rows have been
 * appended with b200k_kv_append): same computation as b200k_attention_fwd, with
 *   K/V of sequence b, token t  =  cache[block_table[b * block_table_stride + t / page_size], h, t % page_size, :]
 * and seq_lens[b] <= max_seq_kv keys for sequence b.  The seq_q queries of a sequence are its last
 * seq_q tokens: with causal != 0 query i sees keys j <= i + seq_lens[b] - seq_q.  A sequence with
 * no visible key yields zeros.  k_cache / v_cache: [num_pages, kv_heads, page_size, head_dim] with
 * contiguous rows, page_size in {16, 32, 64, 128}, head_dim 128 or 64.  Whole pages are fetched, so the rows of a
 * sequence's last page past seq_lens[b] must hold finite values (they are masked, but 0 * NaN is
 * NaN).  A block-table entry outside the pool reads as zeros and sets status bit 2 (value 4).
 * The reference has no call site for this; its layout is the decode path's.
 */
typedef struct b200k_paged_attention_args {
  const void* q;
  const void* k_cache;
  const void* v_cache;
  void* o;
  const int32_t* block_table;
  const int32_t* seq_lens;
  int32_t batch, q_heads, kv_heads, seq_q, max_seq_kv, head_dim;
  int32_t page_size, num_pages, block_table_stride, reserved;
  int64_t q_stride_b, q_stride_h, q_stride_s;
  int64_t o_stride_b, o_stride_h, o_stride_s;
  int64_t kv_page_stride, kv_head_stride;
  int32_t dtype; /* F16 | BF16 */
  int32_t causal;
  float scale;
  int32_t kernel;  /* B200K_ATTN_AUTO | B200K_ATTN_ONE_TILE | B200K_ATTN_TILE_PAIR */
  int32_t* status; /* device status word, may be NULL */
} b200k_paged_attention_args;

int b200k_paged_attention_fwd(const b200k_paged_attention_args* args, void* stream);

/* ---- decode / paged-decode attention (split-KV + reduction) ------------------------ */
/*
 * Replaces the Wave decode and paged-decode attention template launches: one query token per
 * sequence against that sequence's KV history, grouped-query heads, phase 1 over KV chunks
 * followed by a reduction kernel that merges the per-chunk (max, sum, partial output).
 *
 * q            [num_seqs, q_heads, head_dim]                       (contiguous)
 * o            [num_seqs, q_heads, head_dim]                       (contiguous, dtype of q)
 * seq_lens     int32 [num_seqs]; a zero-length sequence yields zeros.  The lengths are device data,
 *              so the kernels bound them themselves: an entry above max_seq_len is treated as
 *              max_seq_len (status bit 3 is set), a negative one as 0.
 *
 * block_table != NULL  (paged):
 *   k_cache/v_cache [num_pages, kv_heads, page_size, head_dim]; token t of sequence s lives in
 *   page block_table[s * block_table_stride + t / page_size], row t % page_size.
 * block_table == NULL  (contiguous):
 *   k_cache/v_cache [num_seqs, kv_heads, kv_seq_stride/head_dim rows, head_dim]; token t of
 *   sequence s is at  s * kv_batch_stride + h * kv_head_stride + t * head_dim  (elements).
 *
 * head_dim must be 128 or 64, page_size a multiple of 16, chunk_tokens a multiple of 64 (0 = choose).
 * workspace: b200k_decode_workspace_bytes() bytes, 256-byte aligned; contents are scratch.
 */
typedef struct b200k_decode_args {
  const void* q;
  const void* k_cache;
  const void* v_cache;
  const int32_t* block_table;
  const int32_t* seq_lens;
  void* o;
  void* workspace;
  uint64_t workspace_bytes;
  int32_t num_seqs, q_heads, kv_heads, head_dim;
  int32_t page_size;          /* paged only */
  int32_t num_pages;          /* paged only: pages in the pool (bounds check of table entries) */
  int32_t block_table_stride; /* paged only: entries per sequence row */
  int32_t max_seq_len;        /* upper bound of seq_lens (sizes the grid and the workspace) */
  int64_t kv_batch_stride;    /* contiguous only, elements */
  int64_t kv_head_stride;     /* paged: elements between kv heads inside a page (page_size*head_dim);
                                 contiguous: elements between kv heads of one sequence */
  int64_t kv_page_stride;     /* paged only: elements between pages */
  int32_t dtype;              /* F16 | BF16 */
  int32_t chunk_tokens;       /* KV tokens per split; 0 = choose */
  float scale;
  int32_t reserved;
  int32_t* status;            /* device status word, may be NULL; bit 3 (value 8) = a seq_lens entry was
                                 larger than max_seq_len and was cut to it */
} b200k_decode_args;

/* Bytes of scratch the call needs for the given problem (depends on num_seqs, q_heads,
 * head_dim, max_seq_len and chunk_tokens only). */
uint64_t b200k_decode_workspace_bytes(const b200k_decode_args* args);

/* The chunk size the library would choose for chunk_tokens == 0. */
int32_t b200k_decode_default_chunk(const b200k_decode_args* args);

int b200k_decode_attention(const b200k_decode_args* args, void* stream);

/*
 * Decode attention for callers that cannot supply scratch memory.
 * (No counterpart in the reference: its runtime always owns allocation.)
 *
 * Same arguments, same kernels and same results as b200k_decode_attention, except that
 * args->workspace and args->workspace_bytes are ignored: the split-KV partial results go into a
 * fixed array that is part of the library image.  Meant for hosts that pass a plug-in only its
 * input and output buffers and keep all device allocation to themselves, and for request paths
 * that must not call cudaMalloc (it can stall the device and can fail under fragmentation).
 * The call performs no cudaMalloc / cudaFree and calls no allocating routine.
 *
 *  - Limit: the problem's b200k_decode_workspace_bytes() must not exceed
 *    B200K_DECODE_STATIC_SCRATCH_BYTES, otherwise B200K_ERR_WORKSPACE is returned and nothing is
 *    launched (raise chunk_tokens or split the batch).  The array is reserved on every GPU that
 *    loads the library, for the life of the process.
 *  - The first call on each device looks up the array's device address (once, cached); make
 *    that first call outside any stream capture.
 *  - All calls on a device share the one array and it keeps whatever the previous call left.
 *    The kernels never depend on old contents, but two calls whose kernels overlap on the GPU
 *    (different streams, no ordering) race on it: order such calls.
 */
#define B200K_DECODE_STATIC_SCRATCH_BYTES (32u << 20)
int b200k_decode_attention_static(const b200k_decode_args* args, void* stream);

/*
 * Gathers the K or V rows of every sequence through the block table into a contiguous buffer
 *   out[s, h, t, :] = cache[block_table[s, t / page_size], h, t % page_size, :]
 * with out laid out [num_seqs, kv_heads, max_seq_len, head_dim].  Rows t >= seq_lens[s] are
 * left untouched.  It uses the same address function as the paged decode kernel and exists so
 * that the index arithmetic can be checked bit-for-bit against a host gather.
 */
int b200k_paged_gather(const void* cache, const int32_t* block_table, const int32_t* seq_lens, void* out,
                       int32_t num_seqs, int32_t kv_heads, int32_t head_dim, int32_t page_size, int32_t num_pages,
                       int32_t block_table_stride, int32_t max_seq_len, int64_t kv_page_stride,
                       int64_t kv_head_stride, int32_t elem_bytes, void* stream);

/*
 * KV-cache append (the step before decode; the reference's decode templates assume a cache that
 * some other kernel has filled, it has no call site of its own for this):
 *   cache[block_table[s, p / page_size], h, p % page_size, :] = new[s, t, h, :],  p = positions[s] + t
 * for t in [0, new_tokens), for K and V alike.  k_new / v_new: [num_seqs, new_tokens, kv_heads,
 * head_dim] contiguous; caches and block table as in b200k_decode_args (paged form).  The address
 * function is the decode kernel's.  A row whose block-table entry is negative, outside the pool
 * or beyond the table is not written; status bit 2 (value 4) is OR-ed into *status (optional).
 */
int b200k_kv_append(const void* k_new, const void* v_new, void* k_cache, void* v_cache, const int32_t* block_table,
                    const int32_t* positions, int32_t num_seqs, int32_t new_tokens, int32_t kv_heads, int32_t head_dim,
                    int32_t page_size, int32_t num_pages, int32_t block_table_stride, int64_t kv_page_stride,
                    int64_t kv_head_stride, int32_t elem_bytes, int32_t* status, void* stream);

/* ---- per-tensor fp8 quantisation helper -------------------------------------------- */
/*
 * scale = max|x| / 448 (1.0 if the tensor is all zero), y = e4m3(x / scale).
 * x: float32 [n]; y: e4m3 [n]; scale_out: device float; amax_scratch: device uint32 (zeroed by
 * the call).  Two launches on `stream`.
 */
int b200k_quantize_e4m3(const float* x, void* y, float* scale_out, uint32_t* amax_scratch, int64_t n, void* stream);

/* ---- self-test of the bounded device-side wait -------------------------------------- */
/*
 * Every barrier wait in the kernels of this library is bounded: when one runs out the kernel sets
 * a shared abort word, all of its roles leave through the common exit, and a code is OR-ed into the
 * caller's status word (the reference has no counterpart: its kernels are generated and it reports
 * failures from the host side of the VM invoke, runtime/invoke.py:62-70).  This entry exercises
 * that exit in isolation: a small kernel waits limit_us microseconds (1 .. 100000) on a barrier on
 * which nobody arrives, returns, and ORs bit 4 (value 16) into *status.  The context stays usable.
 */
int b200k_selftest_bounded_wait(int32_t* status, uint32_t limit_us, void* stream);

/* ---- host-buffer convenience entry points (copies inside the call) ------------------ */
/*
 * Same operations with HOST pointers: the call stages inputs to the device buffers given in
 * `dev` (same struct, device pointers, caller-allocated), launches, and copies the output back
 * to the host pointer, all on `stream`, then returns without synchronizing.  Host buffers
 * should be pinned for the copies to be asynchronous.
 * The copy-back runs on a stream the library keeps per device, ordered with two events that all
 * calls on that device share: call these two functions from ONE host thread per device at a time
 * (calls on different devices are independent).  b200k_gemm_nt_host takes the [M, K] x [N, K]
 * storage only (a_km and b_kn are rejected); the row
 * pitches of both images are checked against the row lengths before any copy.
 */
int b200k_gemm_nt_host(const b200k_gemm_args* host, const b200k_gemm_args* dev, void* stream);
int b200k_attention_fwd_host(const b200k_attention_args* host, const b200k_attention_args* dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200K_H_ */
