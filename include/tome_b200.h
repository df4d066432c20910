/*
 * tome_b200 -- C ABI of the B200 (sm_100a) log-probability library.
 *
 * The library replaces one path of feitreim/Tome: LM-head logits -> per-token
 * log-probabilities of the sampled tokens (GRPO rollout / reference-logprob path).
 * The reference implements that path as MLX expressions and one Metal kernel
 * that MLX JIT-compiles; it has no FFI of its own, so every entry point below
 * cites the reference Python code whose arithmetic it replaces.
 *
 * Conventions
 *   - every pointer named "device" points to CUDA device memory owned by the caller;
 *     the library allocates nothing and keeps no device state between calls (the one
 *     exception is the fixed scratch array of tome_lmhead_logprob_static, described there);
 *   - calls are asynchronous on `stream` (a cudaStream_t passed as void*; NULL is the
 *     legacy default stream); no call synchronises the host with the device;
 *   - the return value is a tome_status: 0 = success, negative = an argument was
 *     rejected on the host before anything was launched, positive = a CUDA runtime
 *     error.  Conditions that only the device can see (a target index outside
 *     [0, vocab), a bounded wait that ran out) are OR-ed as TOME_DEV_* bits into the
 *     optional caller-owned `dev_status` word (device memory, int32, zero it before
 *     the first call; nullable); kernels never trap;
 *   - dtype codes: TOME_F32 = 0, TOME_BF16 = 1;
 *   - all index arithmetic is 64-bit.
 */
#ifndef TOME_B200_H_
#define TOME_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TOME_B200_VERSION 100

enum tome_dtype { TOME_F32 = 0, TOME_BF16 = 1 };

enum tome_status {
  TOME_OK = 0,
  TOME_ERR_NULL_POINTER = -1,
  TOME_ERR_MISALIGNED = -2,
  TOME_ERR_BAD_DTYPE = -3,
  TOME_ERR_BAD_SHAPE = -4,
  TOME_ERR_BAD_STRIDE = -5,
  TOME_ERR_WORKSPACE_TOO_SMALL = -6,
  TOME_ERR_BAD_TEMPERATURE = -7,
  TOME_ERR_UNSUPPORTED = -8,
  TOME_ERR_TOO_LARGE = -9,
  TOME_ERR_CUDA = 1
};

/* bits OR-ed into *dev_status by kernels */
#define TOME_DEV_TARGET_OUT_OF_RANGE 1
#define TOME_DEV_TIMEOUT 2
#define TOME_DEV_RAGGED_OVERFLOW 4 /* windows cover more positions than the packed arrays hold */
#define TOME_DEV_BLOCK_OUT_OF_RANGE 8 /* a block-table entry outside [0, num_blocks) */
#define TOME_DEV_NO_CANDIDATE 16 /* sampling: a row without a single logit that is not NaN */

/* Library version (TOME_B200_VERSION of the build). */
int32_t tome_version(void);

/* Static, human-readable name of a status code. */
const char* tome_status_string(int32_t status);

/* Detail text of the last non-zero status returned on the calling thread. */
const char* tome_last_error_string(void);

/*
 * Self-test of the bounded waits: launches a one-CTA kernel that waits on an mbarrier nothing
 * ever arrives on, gives up after limit_cycles SM clock cycles (<= 2e9), ORs TOME_DEV_TIMEOUT
 * into *dev_status (nullable) and writes 1 to *out_gave_up (device int32, nullable), then exits
 * normally.  This is the path every device-side wait of the library takes when it runs out
 * (no counterpart in the reference).
 */
int32_t tome_selftest_bounded_wait(int64_t limit_cycles, int32_t* dev_status,
                                   int32_t* out_gave_up, void* stream);

/*
 * Selective log-softmax: out_logprob[i] = x[i, targets[i]]/T - logsumexp_j(x[i, j]/T), fp32.
 * Replaces local_compute_logprobs (mlx-impl/node.py:400-404) and the
 * "fused_log_softmax(...) then lp[b, token]" pattern of the policy call sites
 * (mlx-impl/node.py:558-571, 590-605, 331-340, 356-373).
 *
 *   logits        device, [rows, vocab], row r starts at element r*row_stride (row_stride >= vocab)
 *   dtype         TOME_F32 or TOME_BF16
 *   targets       device int32 [rows], each in [0, vocab); a target outside the range
 *                 gives NaN in that row and sets TOME_DEV_TARGET_OUT_OF_RANGE
 *   temperature   > 0 and finite (the "temperature or 1.0" convention of node.py is the caller's)
 *   out_logprob   device fp32 [rows]
 *   out_lse       device fp32 [rows] or NULL: logsumexp_j(x/T)
 *   out_target_raw device fp32 [rows] or NULL: the gathered logit x[i, targets[i]],
 *                 converted to fp32 without scaling (bit-exact copy of the input element)
 * One pass over the logits; accumulation in fp32.
 */
int32_t tome_selective_logprob(const void* logits, int32_t dtype, int64_t rows, int64_t vocab,
                               int64_t row_stride, const int32_t* targets, float temperature,
                               float* out_logprob, float* out_lse, float* out_target_raw,
                               int32_t* dev_status, void* stream);

/*
 * Full-matrix log-softmax with the order of operations of the reference's Metal kernel
 * (mlx-impl/model.py:16-66, wrapper fused_log_softmax model.py:77-89):
 *   out[i, j] = T(float(x[i, j]) * (1/temperature)) - T(max + log(sum exp(...))), in dtype T.
 *   out       device, same dtype as logits, [rows, vocab] with row stride out_row_stride
 *   out_lse   device fp32 [rows] or NULL
 */
int32_t tome_log_softmax_full(const void* logits, int32_t dtype, int64_t rows, int64_t vocab,
                              int64_t row_stride, float temperature, void* out,
                              int64_t out_row_stride, float* out_lse, int32_t* dev_status,
                              void* stream);

/*
 * GRPO dual scoring: per-token log-probs of the policy and of the reference model on a
 * ragged window of each sequence, and the masked k3 KL estimate
 *   kl = exp(r - p) - (r - p) - 1,  r = reference logprob, p = policy logprob.
 * The window is the completion slice of _process_ref_logprobs_batched
 * (mlx-impl/node.py:446-451): positions [starts[i], starts[i] + lengths[i]) of sequence i.
 * The KL formula has no counterpart in the reference (the external trainer forms it).
 *
 *   policy_logits, ref_logits  device, [n_seq * seq_len, vocab], row stride row_stride, same dtype
 *   targets   device int32 [n_seq * seq_len]
 *   lengths   device int32 [n_seq]; clamped to [0, seq_len - start]
 *   starts    device int32 [n_seq] or NULL (all zero)
 *   out_*     device fp32 [n_seq * seq_len]; positions outside the window are written as 0
 * Rows outside the windows are never read.  n_seq <= 1024 per call.
 */
int32_t tome_dual_logprob_kl(const void* policy_logits, const void* ref_logits, int32_t dtype,
                             int64_t n_seq, int64_t seq_len, int64_t vocab, int64_t row_stride,
                             const int32_t* targets, const int32_t* lengths,
                             const int32_t* starts, float temperature, float* out_lp_policy,
                             float* out_lp_ref, float* out_kl, int32_t* dev_status,
                             void* stream);

/*
 * Ragged selective log-softmax, packed to the wire layout: scores the window
 * [starts[i], starts[i] + lengths[i]) of every sequence of ONE model and writes the results
 * back to back, sequence after sequence, which is the layout of Completion.ref_log_probs
 * (scheduler/proto/inference.proto:108-112).  Replaces the per-sequence loop of
 * _process_ref_logprobs_batched (mlx-impl/node.py:446-458: slice, local_compute_logprobs,
 * .tolist(), extend).
 *
 *   logits          device, [n_seq * seq_len, vocab], row stride row_stride
 *   targets_packed  device int32 [packed_capacity]: the completion tokens of sequence 0, then of
 *                   sequence 1, ... (one per scored position)
 *   packed_capacity entries in targets_packed and in the packed outputs; if the windows cover
 *                   more positions, only the first packed_capacity are scored and
 *                   TOME_DEV_RAGGED_OVERFLOW is set
 *   lengths, starts as in tome_dual_logprob_kl (starts nullable); n_seq <= 1024 per call
 *   out_logprob_packed  device fp32 [packed_capacity]
 *   out_lse_packed      device fp32 [packed_capacity] or NULL
 *   out_offsets     device int32 [n_seq + 1] or NULL: offset of each sequence in the packed
 *                   arrays (exclusive prefix sums of the clamped lengths)
 * Rows outside the windows are never read.
 */
int32_t tome_ragged_logprob(const void* logits, int32_t dtype, int64_t n_seq, int64_t seq_len,
                            int64_t vocab, int64_t row_stride, const int32_t* targets_packed,
                            int64_t packed_capacity, const int32_t* lengths,
                            const int32_t* starts, float temperature,
                            float* out_logprob_packed, float* out_lse_packed,
                            int32_t* out_offsets, int32_t* dev_status, void* stream);

/*
 * Top-k temperature sampling fused with the sampled token's log-prob, one row per sequence.
 * Replaces the per-sequence host loop of the rollout (mlx-impl/node.py:593-610):
 * _sample_token (node.py:894-907: top-k of logits / temperature, categorical draw) followed by
 * float(fused_log_softmax(...)[b, token]) (node.py:590, 605), without a host round trip.
 *
 *   temperature  > 0: draw from softmax over the top_k logits / temperature; the log-prob is of
 *                the FULL-vocabulary softmax at that temperature.  0: argmax (first maximum),
 *                scored at temperature 1 (node.py:597-603 with "temperature or 1.0")
 *   top_k        1..64 (the reference uses 20); clipped to vocab
 *   seed, offset select the random stream: the draw of row i depends only on
 *                (seed, offset, i).  The generator is Philox-4x32-10, not MLX's, so parity with
 *                the reference is distributional, not bitwise
 *   out_tokens   device int32 [rows]; out_logprob device fp32 [rows]
 *   out_topk_idx device int32 [rows, top_k] or NULL, out_topk_val device fp32 [rows, top_k] or
 *                NULL: the top-k (value descending, ties by ascending index), raw logits
 */
int32_t tome_sample_topk_logprob(const void* logits, int32_t dtype, int64_t rows, int64_t vocab,
                                 int64_t row_stride, float temperature, int32_t top_k,
                                 uint64_t seed, uint64_t offset, int32_t* out_tokens,
                                 float* out_logprob, int32_t* out_topk_idx, float* out_topk_val,
                                 int32_t* dev_status, void* stream);

/*
 * The same call with caller-owned scratch, which lets batches of a few hundred rows and more
 * (fp32: from 149, bf16: from 297) take a path
 * whose pass over the logits is a plain streaming pass (it keeps the row's sum, finds the
 * row's top-k threshold on the way and notes where the logits that reach it sit; those are
 * fetched again, ranked and drawn from, by a second kernel or between the first one's copies).  Same results as tome_sample_topk_logprob: the
 * draw depends on the row's top-k only.  tome_sample_workspace_bytes returns the bytes that
 * path needs for the batch, or 0 if a batch of that shape would not take it whatever its
 * dtype (then workspace may be NULL).  workspace must be 16-byte aligned; its contents need
 * no initialisation.  A row without a single logit that is not NaN gets token -1, log-prob
 * NaN and TOME_DEV_NO_CANDIDATE (both entry points).
 */
size_t tome_sample_workspace_bytes(int64_t rows, int64_t vocab);
int32_t tome_sample_topk_logprob_ws(const void* logits, int32_t dtype, int64_t rows,
                                    int64_t vocab, int64_t row_stride, float temperature,
                                    int32_t top_k, uint64_t seed, uint64_t offset,
                                    int32_t* out_tokens, float* out_logprob,
                                    int32_t* out_topk_idx, float* out_topk_val, void* workspace,
                                    size_t ws_bytes, int32_t* dev_status, void* stream);

/*
 * Fused LM head + selective log-prob: logits = hidden @ weight^T are formed tile by tile
 * on the tensor cores and reduced on the fly; no logits buffer exists.
 * Replaces "x @ embed_tokens.weight.T" (mlx-impl/model.py:538) followed by
 * local_compute_logprobs (mlx-impl/node.py:400-404).
 *
 *   hidden       device bf16 [rows, hidden_dim], contiguous, 16-byte aligned, hidden_dim % 8 == 0
 *   weight       device bf16 [vocab_local, hidden_dim], contiguous (a row shard of the head)
 *   vocab_offset global vocabulary index of weight row 0 (0 when unsharded)
 *   targets      device int32 [rows], GLOBAL vocabulary indices
 *   workspace    device scratch of at least tome_lmhead_workspace_bytes(...) bytes, 16-byte aligned
 *
 * tome_lmhead_partials writes the shard's triple per row (all device fp32 [rows]):
 *   out_m = max_j(x_j)/T, out_s = sum_j exp(x_j/T - out_m), out_t = x_target/T if the
 *   shard owns the target, else 0.
 * tome_lmhead_logprob (unsharded: vocab_offset 0, vocab_local = vocab) writes
 *   out_logprob = x_target/T - lse and out_lse (nullable).
 */
size_t tome_lmhead_workspace_bytes(int64_t rows, int64_t hidden_dim, int64_t vocab_local);

/* flags of the fused LM-head calls */
#define TOME_LMHEAD_ROUND_LOGITS_BF16 1 /* round each logit to bf16 before reducing, as the
                                           reference's materialised bf16 logits are (model.py:538) */

int32_t tome_lmhead_partials(const void* hidden, const void* weight, int64_t rows,
                             int64_t hidden_dim, int64_t vocab_local, int64_t vocab_offset,
                             const int32_t* targets, float temperature, int32_t flags,
                             float* out_m, float* out_s, float* out_t, void* workspace,
                             size_t workspace_bytes, int32_t* dev_status, void* stream);

int32_t tome_lmhead_logprob(const void* hidden, const void* weight, int64_t rows,
                            int64_t hidden_dim, int64_t vocab, const int32_t* targets,
                            float temperature, int32_t flags, float* out_logprob,
                            float* out_lse, void* workspace, size_t workspace_bytes,
                            int32_t* dev_status, void* stream);

/*
 * Final RMSNorm of the model, the step before the head (RMSNorm, mlx-impl/model.py:336-343,
 * applied at model.py:536): out = bf16(float(x) * rsqrt(mean(x^2) + eps) * float(weight)).
 *   x, out  device bf16 [rows, dim], contiguous, 16-byte aligned (may not alias), dim % 8 == 0
 *   weight  device bf16 [dim]
 */
int32_t tome_rmsnorm_bf16(const void* x, const void* weight, int64_t rows, int64_t dim, float eps,
                          void* out, void* stream);

/*
 * tome_lmhead_logprob without a workspace argument and without any allocation.
 * (No counterpart in the reference: MLX owns all memory there.)
 *
 * Some hosts cannot hand this library a scratch buffer: a serving process whose device
 * memory is entirely reserved by another framework's pool (so a cudaMalloc of its own would
 * fail or fragment the pool), a latency-critical loop that must not hit the implicit device
 * synchronisation of cudaMalloc/cudaFree, or a foreign-language binding that has no device
 * allocator at all.  For them the partial-triple scratch lives in a fixed array inside the
 * library's device image, tome_lmhead_static_scratch_bytes() = 8 MiB per GPU that loads
 * the library, held until the process exits.  Inputs and outputs are still the caller's.
 *
 *   - Sizes whose scratch need (tome_lmhead_workspace_bytes) exceeds the array are rejected
 *     with TOME_ERR_TOO_LARGE; Qwen3-0.6B head shape fits up to 16384 rows per call.
 *   - The first call on each device looks the array's device address up (with that device
 *     current) and remembers it; make that first call before any stream capture begins.
 *   - All calls on a device share the one array and it keeps the previous call's contents.
 *     Nothing in it has to start at zero (each call overwrites every slot it later reads), but
 *     two calls that overlap in time on the same GPU (different streams, or different host
 *     threads) race on it: serialise them on one stream.
 *   - Calls no cudaMalloc, cudaFree or other allocating routine.
 * Arguments and results are those of tome_lmhead_logprob, without `flags` (the logits are
 * always reduced un-rounded; TOME_LMHEAD_ROUND_LOGITS_BF16 needs the workspace variant) and
 * without the workspace pair.
 */
size_t tome_lmhead_static_scratch_bytes(void);

int32_t tome_lmhead_logprob_static(const void* hidden, const void* weight, int64_t rows,
                                   int64_t hidden_dim, int64_t vocab, const int32_t* targets,
                                   float temperature, float* out_logprob, float* out_lse,
                                   int32_t* dev_status, void* stream);

/*
 * Paged KV cache: gather and update (byte-exact data movement; adjacent to the log-prob path,
 * used when the rollout restores or persists a shared prompt prefix).
 * Pool layout [num_blocks, heads, block_size, head_dim]; block_tables int32 [batch, max_blocks];
 * elem_bytes 2 (bf16/fp16) or 4; head_dim * elem_bytes must be a multiple of 16.
 *
 * tome_gather_paged_kv replaces gather_paged_kv (mlx-impl/paged_kv.py:57-116):
 *   out[b, h, s, :] = pool[block_tables[b, s / block_size], h, s % block_size, :] for
 *   s < offsets[b], and 0 for offsets[b] <= s < max_seq_len; out is [batch, heads, max_seq_len,
 *   head_dim].
 * tome_update_paged_kv replaces update_paged_kv (mlx-impl/paged_kv.py:6-54), IN PLACE on the
 * pool (the reference returns new arrays): the first lengths[b] (NULL: new_len) tokens of
 *   new[b] are written block_size at a time; piece i goes to the START of physical block
 *   block_tables[b, (offsets[b] + i * block_size) / block_size]; pieces past the end of the
 *   table are dropped.  Sequences that share a physical block write it concurrently.
 * A table entry outside [0, num_blocks) is skipped (gather writes zeros) and sets
 * TOME_DEV_BLOCK_OUT_OF_RANGE.
 */
int32_t tome_gather_paged_kv(const int32_t* block_tables, const int32_t* offsets,
                             const void* k_pool, const void* v_pool, int32_t elem_bytes,
                             int64_t batch, int64_t heads, int64_t head_dim, int32_t block_size,
                             int32_t max_blocks, int32_t num_blocks, int64_t max_seq_len,
                             void* k_out, void* v_out, int32_t* dev_status, void* stream);

int32_t tome_update_paged_kv(const void* k_new, const void* v_new, const int32_t* block_tables,
                             const int32_t* offsets, const int32_t* lengths, void* k_pool,
                             void* v_pool, int32_t elem_bytes, int64_t batch, int64_t heads,
                             int64_t new_len, int64_t head_dim, int32_t block_size,
                             int32_t max_blocks, int32_t num_blocks, int32_t* dev_status,
                             void* stream);

/*
 * Combine per-shard triples into log-probs (the step after the vocab-parallel exchange;
 * no counterpart in the reference, which has no sharded head):
 *   M = max_p m[p], S = sum_p s[p] * exp(m[p] - M), lse = M + log S,
 *   out_logprob = sum_q t[q] - lse.
 *   m, s   device fp32, part p of row i at m[p * ms_part_stride + i], n_parts parts
 *   t      device fp32, part q of row i at t[q * t_part_stride + i], n_t_parts parts
 *          (1 when the exchange already summed the target column)
 *   out_lse nullable
 */
int32_t tome_combine_triples(const float* m, const float* s, int64_t ms_part_stride,
                             int32_t n_parts, const float* t, int64_t t_part_stride,
                             int32_t n_t_parts, int64_t rows, float* out_logprob,
                             float* out_lse, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TOME_B200_H_ */
