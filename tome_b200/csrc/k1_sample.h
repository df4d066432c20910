// Internal interface of the streaming kernel's sampling mode (see k1_logprob.cu, MODE = SAMPLE),
// the large-batch sampling path of k4_sample.cu: it streams the logits once at HBM speed, keeps
// the row's (max, sum-exp), derives the row's top-k threshold from the logits as they pass,
// notes where the logits that reach it sit, and its producer warp turns those notes into the
// exact top-k, a drawn token and its log-prob while the next rows stream.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tome {

// A row holds at least two 16-byte vectors and fewer than 2^27 of them (rows may start anywhere
// on the element grid: vector numbers count from a row's first 16-byte boundary, and the
// elements outside its boundaries count as one more, short, vector).
bool k1_sample_eligible(const void* logits, int32_t dtype, int64_t vocab, int64_t row_stride);

// Lists the kernel keeps per row (one per consumer warp), entries a list holds, and the
// distance (in 16-byte vectors) between the four vectors one entry speaks of.
int k1_sample_lists_per_row();
int k1_sample_list_capacity();
int k1_sample_vector_stride();
// Most parts a row of this length may be cut into (1, 2 or 4): every part gets a bulk copy.
int k1_sample_max_parts(int64_t vocab, int32_t dtype);

struct K1SampleArgs {
  bool finish_in_kernel;    // the producer warp finishes the rows (else only the notes are left)
  int32_t parts;            // 1, 2 or 4 work items per row (more than 1: not with finish_in_kernel)
  float temperature;        // as asked for: 0 = greedy (argmax, scored at temperature 1)
  int32_t top_k;
  uint64_t seed, offset;
  int32_t* out_tokens;      // [rows]
  float* out_logprob;       // [rows]
  int32_t* out_topk_idx;    // nullable, [rows, top_k]
  float* out_topk_val;      // nullable, [rows, top_k]
  // scratch, all device memory
  float* row_thr;           // [rows, parts]
  float* lse;               // [rows] (parts == 1)
  float2* part_ms;          // [rows, parts] (parts > 1)
  int32_t* cand_count;      // [rows, parts, lists]
  uint2* cand_entry;        // [rows, parts, lists, list capacity]
  int32_t* marked;          // one word: rows left to the row kernel (with finish_in_kernel it
                            // must be ZERO before the launch; without, the kernel clears it)
  int32_t* marked_rows;     // [rows]: their indices
};

// Always left in the scratch, per row: row_thr, a value that at least min(top_k, vocab) logits
// of the row reach; lse = logsumexp(x / temperature); L = k1_sample_lists_per_row() lists of
// entries {(v << 4) | mask, largest}: bit j of the mask says that the 16-byte vector number
// v + j * k1_sample_vector_stride() of the row holds a logit >= the threshold in force when it
// passed (never above row_thr, so every logit >= row_thr sits in a vector some entry names; the
// elements outside the row's first and last 16-byte boundary count as one more, short, vector), and
// `largest` is the float bits of the largest logit of the entry's four vectors (NaN if one of
// them holds a NaN); cand_count (list capacity + 1 if a list ran over).
// With finish_in_kernel the kernel also writes token and log-prob (and the optional top-k
// lists) of every row it can finish; the others (a list that ran over, too many logits at the
// threshold, fewer than top_k logits that are not NaN) are counted in *marked and listed in
// marked_rows.
// With parts > 1 every part of a row is a work item of its own (small batches: more CTAs than
// rows): it leaves its own threshold (a value that at least min(top_k, vocab) logits of the PART
// reach, hence of the row: the largest of a row's part thresholds serves as row_thr), its own
// lists (vector numbers count from the row's start) and, instead of lse, the pair (max,
// sum of 2^((x - max) * log2(e) / temperature)) of the part in part_ms.
int32_t k1_launch_sample(const void* logits, int32_t dtype, int64_t rows, int64_t vocab,
                         int64_t row_stride, const K1SampleArgs& args, int32_t* dev_status,
                         cudaStream_t stream);

}  // namespace tome
