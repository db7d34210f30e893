/*
 * hapx - C ABI of the B200-native executor for HAP's uneven collectives and
 * ratio-sharded tensor ops.
 *
 * Every entry point takes plain pointers and sizes (no torch types) so that the
 * reference's Python layer (collectives.py) can bind it with ctypes, and any
 * other host language with its own FFI.  Each declaration cites the reference
 * interface it stands in for, by path inside the reference project.
 *
 * Conventions
 *  - All functions return 0 on success or a negative hapx_status code;
 *    hapx_last_error() returns a thread-local message for the last failure.
 *  - A tensor of shape S sharded on dimension `dim` is described as
 *    (outer, extent, inner): outer = prod(S[:dim]), inner = prod(S[dim+1:]);
 *    rank r holds extent lengths[r].  All tensors are contiguous.
 *  - Pointer-array arguments (`dst`, `src`) have one entry per LOCAL rank of the
 *    communicator: exactly one for a one-process-per-GPU communicator, `world`
 *    for a local (single-device emulation) communicator.
 *  - Work is enqueued on `stream` (a cudaStream_t); results are usable on that
 *    stream without further synchronisation, as with the NCCL calls the
 *    reference makes (comment at collectives.py:47).
 *  - All ranks must issue the same sequence of collective calls.
 *  - No entry point falls back to the CPU.
 */
#ifndef HAPX_H
#define HAPX_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HAPX_MAX_WORLD 16
#define HAPX_IPC_HANDLE_BYTES 64

typedef struct hapx_comm hapx_comm;
typedef void* hapx_stream; /* cudaStream_t */

enum hapx_status {
  HAPX_OK = 0,
  HAPX_ERR_ARGUMENT = -1,    /* bad pointer, world size, dimension ...            */
  HAPX_ERR_EXTENT = -2,      /* sharding lengths inconsistent with the geometry  */
  HAPX_ERR_DTYPE = -3,       /* dtype not supported by this operation            */
  HAPX_ERR_CUDA = -4,        /* a CUDA runtime call failed                       */
  HAPX_ERR_PEER_TIMEOUT = -5,/* a bounded device-side wait on a peer ran out     */
  HAPX_ERR_STAGING = -6,     /* input is outside the peer-visible heap and does
                                not fit the staging area                         */
  HAPX_ERR_STATE = -7        /* communicator not ready (peers not opened, ...)   */
};

enum hapx_dtype {
  HAPX_F32 = 0, HAPX_BF16 = 1, HAPX_F16 = 2, HAPX_F64 = 3,
  /* copy-only element types (gather / slice / all-to-all) */
  HAPX_B8 = 4, HAPX_B16 = 5, HAPX_B32 = 6, HAPX_B64 = 7
};

/* Entry point selection that mirrors the reference's two strategies.  Both
 * return identical values. */
enum hapx_mode {
  HAPX_MODE_PADDING = 0,   /* collectives.py:14-29, 88-103  (all_gather / reduce_scatter)              */
  HAPX_MODE_GROUP_CALL = 1 /* collectives.py:31-66, 105-140 (all_gather_by_group_call / reduce_scatter_by_group_call) */
};

const char* hapx_last_error(void);
int hapx_version(void);

/* Number of kernels this library has launched in this process (all communicators). */
int64_t hapx_launch_count(void);

/* ---- extents ---------------------------------------------------------------
 * Replaces hap.rs:3536-3559 (fn sharding_round; Python export hap.rs:211-218).
 * Writes `world` integer extents that sum to full_length. */
int hapx_sharding_round(int64_t full_length, const double* ratios, int world, int64_t* out_lengths);

/* ---- communicator ------------------------------------------------------------
 * Replaces dist.init_process_group('nccl', rank=...) at worker.py:18 as far as
 * the collectives below are concerned: one peer-visible heap per rank, mapped
 * into every other rank's address space, plus the flag words the kernels use to
 * synchronise over NVLink.  The heap's first bytes are a control block, followed
 * by a staging area of `stage_bytes` (for inputs that live outside the heap) and
 * the user area (hapx_comm_heap) from which callers may carve zero-copy tensors.
 */
int hapx_comm_create(hapx_comm** out, int world, int rank, int device, size_t heap_bytes, size_t stage_bytes);
/* `world` virtual ranks on ONE device, driven by one process: every collective
 * is a single cooperative launch over all ranks' data.  For single-GPU testing. */
int hapx_comm_create_local(hapx_comm** out, int world, int device, size_t heap_bytes, size_t stage_bytes);
/* Exchange step of a one-process-per-GPU communicator: get this rank's 64-byte
 * handle, all-gather the handles with any host transport, open the peers. */
int hapx_comm_ipc_handle(hapx_comm* c, void* out_handle);
int hapx_comm_open_peers(hapx_comm* c, const void* handles /* world * 64 bytes, rank order */);
/* Alternative to open_peers when the caller maps peer heaps itself. */
int hapx_comm_attach_peer(hapx_comm* c, int peer, void* mapped_base);
/* Tear-down.  hapx_comm_destroy closes the mappings of the peers' heaps and frees this rank's own
 * heap.  Freeing a heap that a peer still has mapped is undefined, so ranks that run as separate
 * processes should tear down in two phases: every rank calls hapx_comm_close_peers, all ranks meet at
 * a host barrier of the caller's, then every rank calls hapx_comm_destroy. */
int hapx_comm_close_peers(hapx_comm* c);
int hapx_comm_destroy(hapx_comm* c);
int hapx_comm_world(hapx_comm* c, int* world, int* n_local, int* first_rank);
/* User area of local rank `local_index`'s heap. */
int hapx_comm_heap(hapx_comm* c, int local_index, void** base, size_t* bytes);
/* Upper bound for device-side waits on peers, in milliseconds.  Default 600000 (ten minutes: a
 * peer that is merely late - logging, a checkpoint, a data stall - must not be mistaken for a dead
 * one), or the value of the environment variable HAPX_TIMEOUT_MS when the communicator is created.
 * When a wait runs out the kernel skips its data movement (its outputs stay unwritten) and leaves an
 * error behind that every later collective call on the communicator returns as
 * HAPX_ERR_PEER_TIMEOUT, without synchronising, until hapx_comm_check has reported and cleared it. */
int hapx_comm_set_timeout_ms(hapx_comm* c, int ms);
/* The same test the collectives make on entry, by itself: HAPX_ERR_PEER_TIMEOUT if a kernel of an
 * earlier call has given up on a peer.  Reads one word of pinned host memory; no synchronisation,
 * so it only sees kernels that have already run. */
int hapx_comm_poll(hapx_comm* c);
/* Number of collectives launched on this communicator so far. */
int hapx_comm_calls_issued(hapx_comm* c, int64_t* calls);
/* Cap the CTAs per rank that a collective launches (0 = one full wave). */
int hapx_comm_set_max_ctas(hapx_comm* c, int ctas);
/* Forms of all_reduce above 256 KiB:
 *   0  two launches: every rank reduces its slice of an even split into a peer-visible buffer, then all gather;
 *   1  the same in ONE launch (reduce the own slice, announce it, gather all slices);
 *   2  one launch in which the owner of a slice writes its sums straight into every rank's output when every
 *      output lies in its rank's peer-visible heap and the byte count is a multiple of 16 (the in-place all_reduce
 *      of a heap-resident gradient bucket): each byte crosses the links once per direction and there is no second
 *      phase.  The ranks settle inside the kernel whether all outputs qualify; if not, the launch proceeds as form 1.
 *  -1  the default: 2 between processes (1 for tensors above 128 MiB on more than 4 GPUs, where writing into seven
 *      peers at once measured slower), 0 in the single-device emulation (no launch or flag latency to save there).
 * Every rank of a communicator must use the same setting. */
int hapx_comm_set_fused_all_reduce(hapx_comm* c, int mode);
/* Calls issued on different streams are ordered with an event by default.  Turn that off
 * (on = 0) while the caller captures its stream into a CUDA graph and keeps all calls on that one
 * stream: event records / waits against streams outside the capture would invalidate it. */
int hapx_comm_set_stream_ordering(hapx_comm* c, int on);
/* Synchronises the device and reports (then clears) the status words the kernels
 * leave behind: 0, or HAPX_ERR_PEER_TIMEOUT with details in hapx_last_error(). */
int hapx_comm_check(hapx_comm* c);

/* ---- collectives ---------------------------------------------------------------
 * all_gather: replaces AllGather.forward (collectives.py:14-20),
 * AllGatherByGroupCall.forward (:31-50), ReduceScatter.backward (:98-103) and
 * ReduceScatterByGroupCall.backward (:123-140).
 * src[i]: (outer, lengths[rank_i], inner); dst[i]: (outer, sum(lengths), inner). */
int hapx_all_gather(hapx_comm* c, void* const* dst, const void* const* src, int dtype,
                    int64_t outer, int64_t inner, const int64_t* lengths, int mode, hapx_stream stream);

/* reduce_scatter: replaces ReduceScatter.forward (collectives.py:88-96),
 * ReduceScatterByGroupCall.forward (:105-121), AllGather.backward (:22-29) and
 * AllGatherByGroupCall.backward (:52-66).
 * src[i]: (outer, sum(lengths), inner) partial; dst[i]: (outer, lengths[rank_i], inner)
 * = out_dtype(scale * sum over ranks), accumulated in fp32 in rank order.
 * The input is never modified (the group-call reference overwrites it). */
int hapx_reduce_scatter(hapx_comm* c, void* const* dst, const void* const* src, int in_dtype, int out_dtype,
                        double scale, int64_t outer, int64_t inner, const int64_t* lengths, int mode,
                        hapx_stream stream);

/* all_reduce: replaces AllReduce.forward/backward (collectives.py:73-84) and
 * Replicate.backward (:176-180).  dst[i] = out_dtype(scale * sum_r src_r), n elements.
 * dst[i] may equal src[i] when in_dtype == out_dtype. */
int hapx_all_reduce(hapx_comm* c, void* const* dst, const void* const* src, int in_dtype, int out_dtype,
                    double scale, int64_t n, hapx_stream stream);

/* all_to_all: replaces AllToAll.forward/backward (collectives.py:152-166).
 * The tensor is viewed as (a, X1, b, X2, c) where X1/X2 are the lower/higher of
 * (split_dim, cat_dim); split_is_first != 0 when split_dim < cat_dim.
 * src[i] has extent sum(split_lengths) on the split dim and cat_lengths[rank_i]
 * on the cat dim; dst[i] has split_lengths[rank_i] and sum(cat_lengths). */
int hapx_all_to_all(hapx_comm* c, void* const* dst, const void* const* src, int dtype,
                    int64_t a, int64_t b, int64_t cc, int split_is_first,
                    const int64_t* split_lengths, const int64_t* cat_lengths, hapx_stream stream);

/* dynamic_slice: replaces collectives.py:146-148 (split + getitem + contiguous)
 * and the placeholder sharding emitted at hap.rs:2511-2515.  Purely local.
 * src: (outer, sum(lengths), inner); dst: (outer, lengths[rank], inner). */
int hapx_dynamic_slice(void* dst, const void* src, int dtype, int64_t outer, int64_t inner,
                       const int64_t* lengths, int world, int rank, hapx_stream stream);
/* Its autograd dual: dst (outer, sum(lengths), inner) = zeros with slice `rank` = src. */
int hapx_dynamic_slice_backward(void* dst, const void* src, int dtype, int64_t outer, int64_t inner,
                                const int64_t* lengths, int world, int rank, hapx_stream stream);

/* One-sided read: copy `bytes` bytes that start `peer_offset` bytes into the USER AREA of rank
 * `peer`'s heap (hapx_comm_heap) into local memory at dst, with the copy kernel of the collectives
 * (16-byte peer loads over NVLink) and no handshake: the caller orders it against the peer's writes
 * (a host barrier, or a collective in between).  No counterpart in the reference; it is the
 * primitive the collectives are built from, exposed for measuring the peer-copy rate of a link
 * (the denominator the all_gather / reduce_scatter fractions are quoted against) and for callers
 * that manage their own synchronisation.  One-process-per-GPU communicators only. */
int hapx_comm_get(hapx_comm* c, int peer, size_t peer_offset, void* dst, size_t bytes, hapx_stream stream);

/* ---- ratio-sharded F.linear on the tensor cores --------------------------------------------
 * Replace the F.linear nodes the planner emits (hap.rs:1030-1037; sharding variants
 * hap.rs:2787-2816: data parallel = uneven m, column parallel = uneven n) and their autograd
 * backward.  bfloat16 operands, fp32 accumulation; m, n, k are the extents of THIS rank's
 * shard and may be any positive numbers (rows of every operand must be 16-byte multiples:
 * k % 8 == 0 for forward, n % 8 == 0 and k % 8 == 0 for dgrad / wgrad).  All tensors
 * contiguous row-major.  out_dtype: HAPX_BF16 or HAPX_F32.
 *   forward: y[m,n] = act(x[m,k] * w[n,k]^T + bias[n])     epilogue: 0 none, 1 relu, 2 gelu(erf), 3 sigmoid
 *   dgrad  : dx[m,k] = g[m,n] * w[n,k]
 *   wgrad  : dw[n,k] = g[m,n]^T * x[m,k];  dbias[n] = column sums of g (either output may be null) */
int hapx_linear_forward(void* y, const void* x, const void* w, const void* bias, int dtype, int out_dtype,
                        int64_t m, int64_t n, int64_t k, int epilogue, hapx_stream stream);
int hapx_linear_dgrad(void* dx, const void* g, const void* w, int dtype, int out_dtype,
                      int64_t m, int64_t n, int64_t k, hapx_stream stream);
int hapx_linear_wgrad(void* dw, void* dbias, const void* g, const void* x, int dtype, int out_dtype,
                      int64_t m, int64_t n, int64_t k, hapx_stream stream);
/* Batched contraction behind the expert einsums the planner emits for MoE layers (torch.einsum
 * codes "bsd,bsec->becd", "edh,becd->bech", "ehd,bech->becd", "becd,bsec->bsd": hap.rs:2255-2276,
 * models.py:356-364) and their backward.  For every batch entry (b_out, b_in):
 *     D[m, n] = sum_k A(m, k) * B(n, k)          bfloat16 operands, fp32 accumulation
 * An operand is "K-major" when k is its contiguous index (element (r, k) at r * ld + k) or
 * "MN-major" when m / n is (element (r, k) at k * ld + r); ld and the batch strides are in elements
 * and must be multiples of 8.  A batch_out stride of 0 shares the operand across b_out (expert
 * weights).  D is row-major with pitch ldd.  A MN-major together with B K-major is not built. */
int hapx_gemm_batched(void* d, const void* a, const void* b, int out_dtype, int a_mn_major, int b_mn_major,
                      int64_t m, int64_t n, int64_t kc, int64_t lda, int64_t ldb, int64_t ldd,
                      int64_t batch_in, int64_t batch_out, int64_t a_stride_in, int64_t a_stride_out,
                      int64_t b_stride_in, int64_t b_stride_out, int64_t d_stride_in, int64_t d_stride_out,
                      hapx_stream stream);
/* Synchronises the device and reports (then clears) an error left by a GEMM kernel whose
 * bounded barrier wait ran out. */
int hapx_gemm_status(void);

/* Sparse form of the two einsums that move tokens into expert slots and back ("bsd,bsec->becd" and
 * "becd,bsec->bsd", models.py:353-366) for dense (batch, seq, expert * capacity) tensors as the gating
 * functions build them (models.py:477-502): every slot of a batch entry holds at most one token, every
 * token sits in at most two slots.  bfloat16 data, row width D a multiple of 8.
 *   hapx_moe_index: one pass over dense [B, S, EC]: slot_token [B, EC] (-1 = empty) and slot_weight
 *       [B, EC]; token_slot [B, S, 2] (-1 = unused) and token_weight [B, S, 2].
 *   hapx_moe_rows_from_tokens: rows[b, slot, :] = slot_weight * x[b, slot_token, :] (0 for an empty
 *       slot; slot_weight null = 1).  The dispatch einsum; the gradient of the combine einsum w.r.t.
 *       the expert outputs (x = the output gradient).
 *   hapx_moe_tokens_from_rows: y[b, s, :] = sum_k token_weight_k * rows[b, token_slot_k, :]
 *       (token_weight null = 1).  The combine einsum; the gradient of the dispatch einsum w.r.t. x.
 *   hapx_moe_weight_grad: d_dense [B, S, EC] = 0 except d_dense[b, s, slot_k(s)] =
 *       <rows[b, slot_k(s), :], dy[b, s, :]>: the gradient of the combine weights at the positions the
 *       gating function reads it back from. */
int hapx_moe_index(const void* dense, int32_t* slot_token, float* slot_weight, int32_t* token_slot, float* token_weight,
                   int64_t B, int64_t S, int64_t EC, hapx_stream stream);
int hapx_moe_rows_from_tokens(void* rows, const void* x, const int32_t* slot_token, const float* slot_weight, int64_t B,
                              int64_t S, int64_t EC, int64_t D, hapx_stream stream);
int hapx_moe_tokens_from_rows(void* y, const void* rows, const int32_t* token_slot, const float* token_weight, int64_t B,
                              int64_t S, int64_t EC, int64_t D, hapx_stream stream);
int hapx_moe_weight_grad(void* d_dense, const void* rows, const void* dy, const int32_t* token_slot, int64_t B, int64_t S,
                         int64_t EC, int64_t D, hapx_stream stream);
/* The same three with explicit layouts, so that no copy stands between the gathers and their neighbours:
 * token tensors (x, y, dy) are addressed as base + b * stride_b + s * stride_s (elements, multiples of 8; rows of D
 * contiguous elements) - e.g. a (b, s, d) view of sequence-major memory; `rows_capacity` > 0 says that the
 * (b, e, c, d) row tensor lies in expert-major memory (e, b, c, d) with c = rows_capacity, the layout the expert
 * GEMMs work on (0: batch-major, as above). */
int hapx_moe_rows_from_tokens_strided(void* rows, const void* x, const int32_t* slot_token, const float* slot_weight, int64_t B, int64_t S,
                                      int64_t EC, int64_t D, int64_t x_stride_b, int64_t x_stride_s, int64_t rows_capacity, hapx_stream stream);
int hapx_moe_tokens_from_rows_strided(void* y, const void* rows, const int32_t* token_slot, const float* token_weight, int64_t B, int64_t S,
                                      int64_t EC, int64_t D, int64_t y_stride_b, int64_t y_stride_s, int64_t rows_capacity, hapx_stream stream);
int hapx_moe_weight_grad_strided(void* d_dense, const void* rows, const void* dy, const int32_t* token_slot, int64_t B, int64_t S, int64_t EC,
                                 int64_t D, int64_t dy_stride_b, int64_t dy_stride_s, int64_t rows_capacity, hapx_stream stream);

/* ---- multi-head self-attention on a batch shard ---------------------------------------------
 * Replace the attention core of F.multi_head_attention_forward as emitted at hap.rs:1297-1329
 * (query = key = value, packed in-projection, no bias_k/bias_v, no key padding mask; only the
 * batch dimension N is sharded, hap.rs:2903-2926).  All tensors bfloat16, (L, N, E) layout:
 *   qkv  [L, N, 3E]  output of the packed in-projection (E = H * D);   out [L, N, E]
 *   probs      [N*H, L, Lp] bf16, Lp = L rounded up to 8: softmax output, kept for backward
 *   scores_ws  [N*H, L, Lp] fp32 scratch;   ds_ws [N*H, L, Lp] bf16 scratch (backward)
 * forward : out = softmax(Q K^T / sqrt(D) + mask) V.  causal != 0 masks keys after the query
 *           (the -inf upper-triangular mask of models.py:72); mask = optional additive [L, L] fp32.
 * backward: dqkv [L, N, 3E] from dout [L, N, E].  No dropout on this path (head dimensions other
 * than 64 without dropout; for D = 64 see the fused entry points below).
 * Limits: L <= 1024, D % 8 == 0. */
int hapx_attention_forward(void* out, void* probs, void* scores_ws, const void* qkv, int64_t L, int64_t N, int64_t H,
                           int64_t D, int causal, const float* mask, hapx_stream stream);
int hapx_attention_backward(void* dqkv, void* dscores_ws, void* ds_ws, const void* dout, const void* probs,
                            const void* qkv, int64_t L, int64_t N, int64_t H, int64_t D, hapx_stream stream);

/* Fused form of the same attention core for head dimension D = 64 (every benchmark configuration):
 * one kernel computes S = Q K^T in tensor memory, the online softmax, the dropout on the
 * probabilities (dropout_p of the attention node, hap.rs:1257, 1307, 1319; 0.1 in config.py:33) and
 * O = P V, so nothing of size L x L is written to memory; only lse2 [N*H, L] fp32 (the rows'
 * log-sum-exp in the log2 domain) is kept for backward.  backward recomputes the probabilities per
 * tile and regenerates the dropout mask from (generator state, call_id) - see the dropout section -
 * so it must run in the same iteration (before the next hapx_rng_advance) with the same call_id,
 * causal flag and mask.  delta_ws: N*H*L floats of scratch.  out is the forward's output.
 * Deterministic: no atomics, every output element is written by one thread block.
 * mask_flag (optional, with a mask tensor): a device word written by hapx_attention_classify_mask,
 * non-zero when the mask tensor is exactly the causal mask (0 on and below the diagonal, -inf
 * above, as models.py:72 builds it); the kernels then skip the key tiles the causal rule excludes
 * and never read the tensor.  The word is read on the device, so nothing synchronises with the host;
 * classify a mask tensor once and pass the word to every layer's forward and backward.
 * hapx_attention_dropout_mask writes the keep mask [N*H, L, L] as bytes (for tests). */
int hapx_attention_classify_mask(const float* mask, int64_t L, unsigned* flag, hapx_stream stream);
int hapx_attention_fused_forward(void* out, float* lse2, const void* qkv, int64_t L, int64_t N, int64_t H, int64_t D,
                                 int causal, const float* mask, const unsigned* mask_flag, double dropout_p, uint64_t call_id,
                                 hapx_stream stream);
int hapx_attention_fused_backward(void* dqkv, float* delta_ws, const void* dout, const void* out, const float* lse2,
                                  const void* qkv, int64_t L, int64_t N, int64_t H, int64_t D, int causal, const float* mask,
                                  const unsigned* mask_flag, double dropout_p, uint64_t call_id, hapx_stream stream);
int hapx_attention_dropout_mask(unsigned char* mask, int64_t L, int64_t N, int64_t H, double dropout_p, uint64_t call_id,
                                hapx_stream stream);

/* ---- dropout ---------------------------------------------------------------------------------
 * Replaces the torch.nn.functional.dropout(input, p) nodes the planner emits (hap.rs:1446-1464;
 * the encoder layers of models.py:40,74,83-88 are built with config.py:33 dropout = 0.1) and supplies
 * the random bits for the dropout on the attention probabilities (dropout_p of the attention node,
 * hap.rs:1257, 1307, 1319).  The generator is counter based: a mask is a pure function of
 * (seed, iteration counter, call_id, element index), so backward passes regenerate it instead of
 * storing it.  Seed and iteration counter live in device memory, one pair per device:
 * hapx_rng_seed sets the seed and zeroes the counter, hapx_rng_advance adds one to the counter (a
 * one-thread kernel: recorded into a CUDA graph it advances on every replay).  Call hapx_rng_advance
 * once per training iteration; call_id distinguishes the dropout sites within an iteration.
 * The first use on a device allocates the 16-byte state: make it outside any stream capture.
 * hapx_dropout: y[i] = keep(i) ? x[i] / (1 - p) : 0 over n elements of HAPX_BF16 or HAPX_F32
 * (y may equal x).  The backward pass is the same call on the incoming gradient with the same
 * call_id in the same iteration.  hapx_dropout_mask writes keep(i) as bytes (for tests). */
int hapx_rng_seed(uint64_t seed, hapx_stream stream);
int hapx_rng_advance(hapx_stream stream);
int hapx_dropout(void* y, const void* x, int dtype, int64_t n, double p, uint64_t call_id, hapx_stream stream);
int hapx_dropout_mask(unsigned char* mask, int64_t n, double p, uint64_t call_id, hapx_stream stream);
/* The same dropout fused with its neighbours in the reference's encoder layers (one pass over memory
 * instead of two or three; p = 0 is allowed and gives the bare operation):
 *   hapx_dropout_add : y = residual + dropout(x)            x + dropout1(sa(x)), x + dropout2(ff(x))
 *   hapx_act_dropout : y = dropout(act(x))                  dropout(activation(linear1(x)));  act 1 = relu, 2 = gelu (erf)
 * backward of dropout_add w.r.t. x is hapx_dropout on the incoming gradient (w.r.t. residual: the
 * identity); backward of act_dropout is hapx_act_dropout_backward with `saved` = the forward's OUTPUT
 * for relu (an element is non-zero iff it was active and kept: no mask is regenerated) and the
 * forward's INPUT for gelu. */
int hapx_dropout_add(void* y, const void* x, const void* residual, int dtype, int64_t n, double p, uint64_t call_id,
                     hapx_stream stream);
int hapx_act_dropout(void* y, const void* x, int dtype, int64_t n, int act, double p, uint64_t call_id, hapx_stream stream);
int hapx_act_dropout_backward(void* dx, const void* dy, const void* saved, int dtype, int64_t n, int act, double p,
                              uint64_t call_id, hapx_stream stream);

/* all_reduce that allocates nothing.  No counterpart in the reference.
 * Same values as hapx_all_reduce on a local (single-device) communicator of `world` virtual
 * ranks, but without a communicator: all scratch (control blocks, staged inputs, reduced
 * slices) is a 16 MiB device array built into the library, so the call performs no cudaMalloc /
 * cudaFree.  The array is part of the library's device code: the driver reserves it when it loads
 * that code on a device, which with lazy loading is the FIRST call on the device - make one warm-up
 * call per device while memory is still available; only from then on is nothing reserved any more.
 * For hosts that cannot allocate when the
 * collective is due (all device memory already owned by another allocator, or a thread that
 * must not take cudaMalloc's device-wide synchronisation).
 * dst[r], src[r]: n elements each, r = 0..world-1, src 16-byte aligned or not (inputs are
 * copied into the scratch first); dst[r] may equal src[r].
 * Limits: world <= 8; 4096 + round256(n*in_size) + round256(slice*out_size) <= 2 MiB, where
 * slice = ceil(n/world) rounded up to 16 bytes (about 460 000 float32 elements at world 8);
 * beyond that the call returns HAPX_ERR_STAGING.
 * The first call on a device resolves the array's device address; make it outside any stream
 * capture.  Calls share the array: calls whose kernels overlap on the GPU race.
 * A bounded wait inside the kernels that runs out leaves the outputs unwritten and a status word in
 * the array, which stays there until hapx_local_all_reduce_noalloc_status reads it. */
int hapx_local_all_reduce_noalloc(int world, void* const* dst, const void* const* src, int in_dtype, int out_dtype,
                                  double scale, int64_t n, hapx_stream stream);
/* Synchronises the current device and reports (then clears) a wait that ran out in an earlier
 * hapx_local_all_reduce_noalloc on it: 0 or HAPX_ERR_PEER_TIMEOUT.  No counterpart in the reference. */
int hapx_local_all_reduce_noalloc_status(void);

/* ---- step tail: gradient clipping + Adam over the local parameter shards ----------
 * Replaces torch.nn.utils.clip_grad_norm_(dmodel.parameters(), 0.5) and optimizer.step() of
 * the reference's iteration (worker.py:74, 76; optimizer created at worker.py:47 as
 * torch.optim.Adam with default betas / eps) by multi-tensor kernels that never synchronise
 * with the host.  The norm is the 2-norm over the shards THIS rank holds, as in the reference
 * (no collective).
 *
 * `state`: HAPX_OPTIM_STATE_FLOATS floats of device memory owned by the caller, zero-filled
 * once before the first step: [0] steps taken so far, [1] last gradient norm, [2] last clip
 * coefficient, [8...] partial sums of squares.
 *
 * hapx_grad_sqnorm adds the sum of squares of `n` gradient tensors (numel[i] elements of
 * `dtype`, HAPX_F32 or HAPX_BF16) into the state; reset != 0 starts a new sum.  Call it once
 * per dtype group, the first with reset = 1.
 * hapx_clip_adam_apply scales every gradient by min(1, max_norm / (norm + 1e-6)) (max_norm <= 0:
 * no clipping, the state's sum is not read), then applies the Adam update in fp32 and rounds
 * once: exp_avg, exp_avg_sq and params have `dtype`; gradients are left unmodified (the
 * reference's clip_grad_norm_ scales them in place).  advance_step != 0 increments the step
 * count after the update: pass it on the last group of an iteration. */
#define HAPX_OPTIM_STATE_FLOATS 2056
int hapx_grad_sqnorm(int n, const void* const* grads, const int64_t* numel, int dtype, float* state, int reset,
                     hapx_stream stream);
int hapx_clip_adam_apply(int n, void* const* params, const void* const* grads, void* const* exp_avg,
                         void* const* exp_avg_sq, const int64_t* numel, int dtype, double lr, double beta1, double beta2,
                         double eps, double weight_decay, double max_norm, float* state, int advance_step,
                         hapx_stream stream);

/* ---- loss: log_softmax + nll_loss(reduction='sum') in one pass ---------------------
 * Replaces the pair of fx nodes the planner emits for the models' loss (hap.rs:1808
 * log_softmax, hap.rs:1858 nll_loss; models.py:116-117): logits [rows][classes] (row pitch
 * `pitch` elements, HAPX_F32 or HAPX_BF16), int64 targets [rows].
 * forward writes row_lse[r] = logsumexp(logits[r]) and row_loss[r] = row_lse[r] -
 * logits[r][target[r]] (fp32); the loss is the sum of row_loss.  A target outside
 * [0, classes), such as torch's ignore_index -100, gives a zero loss and a zero gradient row.
 * backward writes grad_logits[r][c] = *grad_out * (exp(logits[r][c] - row_lse[r]) - [c == target[r]])
 * in the logits' dtype; grad_out is a device scalar. */
int hapx_nll_logsoftmax_forward(const void* logits, const int64_t* targets, float* row_loss, float* row_lse, int dtype,
                                int64_t rows, int64_t classes, int64_t pitch, hapx_stream stream);
int hapx_nll_logsoftmax_backward(const void* logits, const int64_t* targets, const float* row_lse, const float* grad_out,
                                 void* grad_logits, int dtype, int64_t rows, int64_t classes, int64_t pitch,
                                 int64_t grad_pitch, hapx_stream stream);

/* ---- gradient of an embedding lookup ----------------------------------------------------
 * Replaces the backward pass of the torch.nn.functional.embedding nodes (the models look their tokens up with
 * it, models.py:66-71): dweight[v, :] = sum of grad[i, :] over the positions i with idx[i] == v, added in
 * ascending order of position in float32 (bit-reproducible; no sort, no atomics), all other rows zero.
 * dweight: V x E, grad: n x E of `dtype` (HAPX_F32 / HAPX_BF16), idx: n int64; E a multiple of 8 in [8, 2048],
 * n <= 2^20 (the kernel compares every position with every other one). */
int hapx_embedding_backward(void* dweight, const void* grad, const int64_t* idx, int dtype, int64_t n, int64_t V, int64_t E,
                            hapx_stream stream);

/* ---- layer_norm over the last dimension ---------------------------------------------
 * Replaces the torch.nn.functional.layer_norm nodes of the Transformer programs (planner
 * handler hap.rs:1637-1660; nn.LayerNorm of the reference's encoder layers, models.py:319-320).
 * x, y, dy, dx: [rows][E] contiguous, gamma / beta: [E] (beta may be null), all of `dtype`
 * (HAPX_F32 or HAPX_BF16); E a multiple of 8, at most 2048.  mean / rstd: fp32 [rows], written
 * by forward and read by backward.
 * backward needs `partial`: 2 * E * hapx_layer_norm_backward_blocks(rows, E) floats of scratch;
 * dgamma / dbeta may be null.  The parameter gradients are summed in a fixed order. */
int hapx_layer_norm_forward(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd, int dtype,
                            int64_t rows, int64_t E, double eps, hapx_stream stream);
int hapx_layer_norm_backward_blocks(int64_t rows, int64_t E);
int hapx_layer_norm_backward(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd, void* dx,
                             void* dgamma, void* dbeta, float* partial, int dtype, int64_t rows, int64_t E,
                             hapx_stream stream);
/* The same with a second gradient of x added to dx in the same pass (`add`: rows x E of the data type, or
 * NULL): the gradient that reaches x through the residual connection around the normalised branch of a
 * pre-LN block, which autograd would otherwise add with a kernel of its own. */
int hapx_layer_norm_backward_add(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd, const void* add,
                                 void* dx, void* dgamma, void* dbeta, float* partial, int dtype, int64_t rows, int64_t E,
                                 hapx_stream stream);

/* ---- diagnostics ----------------------------------------------------------------
 * No counterpart in the reference.  Walks the kernels' tiling of ONE rank's pull over
 * HOST buffers (op: 0 gather, 1 all-to-all, 2 slice, 3 slice-backward), bounds-checking
 * every byte range and counting in `cover` (optional, dst_bytes long) how often each
 * output byte is written.  It exists so that CPU-only tests can validate the index
 * arithmetic of a geometry; it is not a compute path and takes no device pointers. */
int hapx_debug_host_walk(int op, int world, int rank, int elem_size, int64_t a, int64_t b, int64_t cc,
                         int split_is_first, const int64_t* l1, const int64_t* l2,
                         const void* const* src_per_rank, const size_t* src_bytes, void* dst, size_t dst_bytes,
                         unsigned char* cover);

#ifdef __cplusplus
}
#endif
#endif /* HAPX_H */
