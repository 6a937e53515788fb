/*
 * leat_sampler.h -- C ABI of the B200 token sampler (libleat_sampler.so).
 *
 * The library replaces leat's token-sampling path.  In leat that path is a Python function
 * boundary, not an FFI: leat/ops.py:496-515 asks leat/kernels/ for `argmax` and `cutoff`, and
 * leat/sampler.py:31-55 (`sample`) composes them.  Each entry point below names the reference
 * interface it stands in for.  All pointers are device pointers unless stated otherwise, all
 * matrices are row-major, every call is asynchronous on `stream`, allocates nothing and makes no
 * host synchronisation, so a call can be recorded into a CUDA graph (option values live on the
 * device, as leat/sampler.py:39-40 wants them: one captured graph serves every value).
 *
 * Return value: 0, or a negative LEAT_E_* for an argument error found on the host (nothing is
 * launched).  Conditions found on the device are OR-ed into the caller's `status` word as
 * LEAT_STATUS_* bits; no kernel traps.
 */
#ifndef LEAT_SAMPLER_H
#define LEAT_SAMPLER_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct leat_sampler leat_sampler_t;
typedef struct leat_shard leat_shard_t;
typedef void* leat_stream_t; /* a cudaStream_t */

enum {
  LEAT_OK = 0,
  LEAT_E_ARGUMENT = -1,  /* null pointer, bad shape, bad broadcast row count */
  LEAT_E_CAPACITY = -2,  /* rows / vocab / width beyond what the handle was created for */
  LEAT_E_WORKSPACE = -3, /* workspace too small or misaligned */
  LEAT_E_CUDA = -4,      /* a CUDA runtime call failed; see leat_sampler_last_cuda_error() */
  LEAT_E_DEVICE = -5     /* the handle belongs to another device than the current one */
};

/* bits of the device status word */
enum {
  LEAT_STATUS_FALLBACK = 1,  /* a row took the exact multi-pass path (informational) */
  LEAT_STATUS_TRUNCATED = 2, /* a row had more survivors than out_width; probabilities clipped */
  LEAT_STATUS_INTERNAL = 4,  /* an internal bound was exceeded; the row's id is -1 */
  LEAT_STATUS_PEER = 8       /* vocabulary shards: another rank's hand-over did not arrive within the wait's limit */
};

/* flags */
enum {
  LEAT_FLAG_DIVIDE = 1,        /* scores = logits / T as an IEEE quotient instead of logits * (1 / T) */
  LEAT_FLAG_NO_FALLBACK = 2,   /* caller promises every row has 0 < top_k <= k_max (or is greedy): the
                                  multi-pass routine is not run; a row that needs it gets id -1
                                  and LEAT_STATUS_INTERNAL */
  LEAT_FLAG_LOGITS_BF16 = 4,   /* `logits` points at bfloat16 values (the lm_head's own output) */
  LEAT_FLAG_LOGITS_F16 = 8,    /* `logits` points at float16 values */
  LEAT_FLAG_CLEAR_STATUS = 16  /* the call clears the status word before its kernels OR into it (saves
                                  the caller a fill of its own) */
};

/* Arguments of leat_sample; stands in for the arguments of sample() at leat/sampler.py:31-34. */
typedef struct leat_sample_args {
  /* logits (rows, vocab), row b at element b * row_stride: float32, or bfloat16 / float16 with
     LEAT_FLAG_LOGITS_BF16 / LEAT_FLAG_LOGITS_F16 (any shape float32 logits may have; 16-byte
     aligned rows of a multiple of 8 tokens, at least 16384 of them, without a dense seen mask are
     the fast case, everything else is streamed with two-byte loads) */
  const void* logits;
  int32_t rows;
  int32_t vocab;
  int64_t row_stride;
  /* options (options_rows, 5) float32 rows of [temperature, top_k, top_p, min_p, presence_penalty]
     (Sampling.values(), leat/sampler.py:23-25); options_rows is `rows` or 1 (one row for all).
     NULL: every row is greedy. */
  const float* options;
  int32_t options_rows;
  /* seed (seed_rows,) uint32 and position (position_rows,) int32, each `rows` or 1; used by the
     hashed Gumbel-max draw (leat/sampler.py:58-64) when `uniform` is NULL */
  const uint32_t* seed;
  int32_t seed_rows;
  const int32_t* position;
  int32_t position_rows;
  /* seen (rows, vocab) bytes, non-zero where presence_penalty applies (leat/sampler.py:48-49), row
     b at seen + b * seen_stride; or NULL */
  const uint8_t* seen;
  int64_t seen_stride;
  /* extension: history (rows, history_cap) int32 token ids of which the first history_len[b] count
     (history_len NULL: all history_cap); gives per-token counts; or NULL */
  const int32_t* history;
  const int32_t* history_len;
  int32_t history_cap;
  /* extension: penalties (penalties_rows, 3) float32 rows of [repetition, presence, frequency];
     replaces the options' presence column; NULL: [1, options[4], 0], the reference's behaviour */
  const float* penalties;
  int32_t penalties_rows;
  /* extension: uniform (rows,) float32 in [0, 1): draw by inverse CDF over the survivors instead
     of hashed Gumbel-max; NULL: the reference's draw */
  const float* uniform;
  /* first token id of this vocabulary slice (0 for a whole vocabulary): added to every id written
     and hashed, subtracted from history ids */
  int32_t vocab_offset;
  /* size of the whole vocabulary when `vocab` is one slice of it (0: `vocab` is the whole) */
  int32_t vocab_total;
  uint32_t flags;
  /* outputs; any but out_ids may be NULL */
  int32_t* out_ids;      /* (rows,) the token per row: what sample() returns as (B, 1) */
  int32_t* out_greedy;   /* (rows,) argmax of the penalised logits, first index on ties */
  float* out_cut;        /* (rows,) the cut of leat/ops.py:503-515 */
  int32_t* out_kept;     /* (rows,) number of survivors (scores >= cut); 0 for greedy rows */
  float* out_probs;      /* (rows, out_width) survivor probabilities, likeliest first, 0-padded */
  int32_t* out_prob_ids; /* (rows, out_width) their ids, -1-padded */
  int32_t out_width;
  int32_t* status;       /* one int32, OR-ed with LEAT_STATUS_*; may be NULL */
  /* extension: the model's soft cap on its logits, logits = tanh(logits / cap) * cap
     (leat/model.py:419-423), applied here to the few logits that reach a row's floor instead of by
     a pass of its own over (rows, vocab); 0: none.  Evaluated in double precision and rounded to
     float32.  Rows that cannot take the list path are then settled by the multi-pass routine. */
  float softcap;
  /* the position of every row when `position` is NULL (leat/sampler.py:41-42 takes an int too) */
  int32_t position_scalar;
} leat_sample_args;

/* Bytes of device workspace a handle needs for calls of up to max_rows x max_vocab with
   top_k <= k_max on the single-pass path (k_max <= 1024).  No reference counterpart: leat's
   kernels allocate their scratch per call (leat/kernels/argmax.py:57-59, cutoff.py:163-170). */
size_t leat_sampler_workspace_bytes(int32_t max_rows, int32_t max_vocab, int32_t k_max);

/* Builds a handle over caller-owned device memory `workspace` (256-byte aligned, at least
   leat_sampler_workspace_bytes(...) bytes) on CUDA device `device`; clears the workspace on the
   default stream and waits for it.  The handle itself is a small host object. */
int leat_sampler_create(void* workspace, size_t bytes, int32_t device, int32_t max_rows,
                        int32_t max_vocab, int32_t k_max, leat_sampler_t** out);
int leat_sampler_destroy(leat_sampler_t* handle);

/* Launch shape override, for tests that run one input through several shapes: threads per block (128, 256 or 512; 0 = automatic) and
   blocks per row (0 = automatic). */
int leat_sampler_tune(leat_sampler_t* handle, int32_t threads, int32_t slices);
/* The filter path (floor per row, one streaming filter, finish from the row's list) is taken for
   16-byte aligned rows of at least 16384 tokens without a dense seen mask; 0 turns it off and every
   row goes through the fused kernel (for tests that run one input through both). */
int leat_sampler_tune_filter(leat_sampler_t* handle, int32_t enabled);
/* The launch shape the handle would use for (rows, vocab): writes threads, slices, blocks. */
int leat_sampler_plan(const leat_sampler_t* handle, int32_t rows, int32_t vocab, int32_t history_cap,
                      int32_t* threads, int32_t* slices, int32_t* shared_bytes);
/* Number of kernels the last call on this handle launched (host counter). */
int leat_sampler_last_launches(const leat_sampler_t* handle);
/* Measurement aid.  While enabled, the kernels of a call on this handle record, in the workspace,
   when their first block began and their last block ended (the GPU's nanosecond timer), also inside
   a captured CUDA graph.  leat_sampler_kernel_times waits for the device and writes twelve offsets in
   milliseconds from the first begin of the last call: begin and end of filter_kernel,
   finish_list_kernel (a shard's: shard_select_kernel), sample_kernel, floor_kernel,
   shard_finish_kernel and shard_result_kernel (-1, -1 for a kernel the call did not launch).  Kernels of
   one call overlap (each is a programmatic dependent of the one before), which the offsets show. */
int leat_sampler_time_kernels(leat_sampler_t* handle, int32_t enabled);
int leat_sampler_kernel_times(leat_sampler_t* handle, float* milliseconds);
/* Text of the last CUDA error seen by this library on this thread (host pointer, static). */
const char* leat_sampler_last_cuda_error(void);

/* sample(): leat/sampler.py:31-55 (presence -> temperature -> cut -> draw -> argmax), plus the
   extensions the arguments describe. */
int leat_sample(leat_sampler_t* handle, const leat_sample_args* args, leat_stream_t stream);

/* leat_sample() without a handle or a workspace, for callers that cannot allocate device memory:
   a server whose memory pool is already fully committed, a foreign-language binding that only
   receives device pointers and owns no allocator, or a step that must not pay cudaMalloc's
   device-wide synchronisation.  It has no counterpart in the reference (leat's kernels allocate
   their scratch per call).  The scratch the blocks of a row exchange lives in a fixed array of
   about 1.1 MB inside the library, held by every GPU that loads the library until the process
   exits.  Limits: rows <= 64 and vocab <= 262144, else LEAT_E_CAPACITY; float32 logits only
   (LEAT_FLAG_LOGITS_BF16 / _F16: LEAT_E_ARGUMENT); rows with top_k <= 64 take the single pass,
   rows with a larger top_k (or none, with top_p < 1) are settled by the slower multi-pass routine,
   as with a handle created for k_max = 64.  The caller still passes every input and output buffer.
   The first call on a device looks up the array's device address and raises the kernels'
   shared-memory limit (under a lock: threads may race to it), so make that first call outside any
   stream capture.  All calls on a device share the one array: calls that overlap on the GPU
   (different streams) race; issue them on one stream or order them.  Calls cudaMalloc, cudaFree
   or any allocating routine nowhere. */
int leat_sample_static(const leat_sample_args* args, leat_stream_t stream);

/* ops.argmax(): leat/ops.py:496-500 and leat/kernels/argmax.py:48-61.  x (rows, vocab) float32 ->
   out (rows,) int32, the first index of each row's largest value (a NaN is never the largest; a row
   of nothing but -inf and NaN answers 0).  One launch that streams x once for 16-byte aligned rows of
   a multiple of four values, at least 4096 of them; the sampler's greedy path otherwise. */
int leat_argmax(leat_sampler_t* handle, const float* x, int32_t rows, int32_t vocab,
                int64_t row_stride, int32_t* out, int32_t* status, leat_stream_t stream);

/* ops.cutoff(): leat/ops.py:503-515 with the exact _cutoff of :518-529 (not the 2048-bin
   approximation of leat/kernels/cutoff.py).  scores (rows, vocab) float32 and top_k, top_p, min_p
   (rows,) float32 -> cut (rows,) float32, -inf where no option is set. */
int leat_cutoff(leat_sampler_t* handle, const float* scores, int32_t rows, int32_t vocab,
                int64_t row_stride, const float* top_k, const float* top_p, const float* min_p,
                float* cut, int32_t* status, leat_stream_t stream);

/* The accept loop of a speculative step: leat/engine.py:612-626.  drafted (n, drafts) and sampled
   (n, drafts + 1) int32 -> accepted (n,) = the first j with drafted[j] != sampled[j], else
   drafts; tokens (n, drafts + 1) = sampled[0..accepted], -1 after.  With `greedy` non-NULL
   (n, drafts + 1), the variant: a draft is accepted while it equals greedy[j], and tokens =
   drafted[0..accepted) then sampled[accepted]. */
int leat_verify_draft(const int32_t* drafted, const int32_t* sampled, const int32_t* greedy,
                      int32_t n, int32_t drafts, int32_t* accepted, int32_t* tokens,
                      leat_stream_t stream);

/* What follows a speculative step's verification on the device, so that the next step needs no
   host round trip (leat/engine.py:609-631, :677-686): sequence i ran its last token and `drafts`
   drafts, of which `accepted[i]` are kept.  Its slot's history (leat_b200's sparse form of leat's
   `_seen` mask: ids (slots, capacity) int32 used as a ring, count (slots,) int32) takes the tokens
   that were run up to the kept row, last[i] then drafted[i, 0..accepted[i]), markup left out (text
   (vocab,) bytes, non-zero = a penalty may lower the token; NULL: every token), as
   `_seen_rows[row]` holds them; next[i] = sampled[i, accepted[i]], the token the next step runs;
   row[i] = i * (drafts + 1) + accepted[i], the row whose hidden state the slot keeps. */
int leat_settle_draft(const int32_t* accepted, const int32_t* last, const int32_t* drafted, const int32_t* sampled,
                      const int32_t* slots, int32_t n, int32_t drafts, int32_t* history_ids, int32_t* history_count,
                      int32_t capacity, const uint8_t* text, int32_t vocab, int32_t* next, int32_t* row,
                      leat_stream_t stream);

/* Vocabulary shards (no reference counterpart: leat runs one model per GPU, leat/server.py:427-428).
   leat_topk_local runs the first half of leat_sample on this rank's slice of the vocabulary
   (args->vocab = slice width, args->vocab_offset = its first id) and writes, per row, the slice's
   candidates: every (score, global id) at or above the slice's top_k-th score, up to `cap` of
   them, unordered; count (rows,) is their number, or -1 when the slice cannot be reduced to `cap`
   candidates.  best (rows,) holds the slice's greedy candidate as a packed 64-bit key (penalised
   logit, id).  The args' outputs are ignored. */
int leat_topk_local(leat_sampler_t* handle, const leat_sample_args* args, float* cand_value,
                    int32_t* cand_id, int32_t* cand_count, uint64_t* best, int32_t cap,
                    leat_stream_t stream);

/* Second half: samples each row from the candidates of `parts` slices laid out part-major, as an
   all-gather leaves them: cand_value / cand_id (parts, rows, cap), cand_count (parts, rows), best
   (parts, rows).  Uses args->options, seed, position, uniform, flags and outputs; args->logits is
   ignored and args->vocab is the whole vocabulary's size. */
int leat_sample_from_candidates(leat_sampler_t* handle, const leat_sample_args* args,
                                const float* cand_value, const int32_t* cand_id,
                                const int32_t* cand_count, const uint64_t* best, int32_t parts,
                                int32_t cap, leat_stream_t stream);

/* The same from packed records, so that one all-gather moves everything a rank hands over.  A
   rank's record is leat_candidate_record_bytes(rows, cap) bytes: cand_value (rows, cap) float32 at
   offset 0, then cand_id, cand_count and best at the offsets leat_candidate_record_layout()
   returns (the caller points leat_topk_local at them).  `records` holds `parts` records back to
   back, as the all-gather leaves them. */
size_t leat_candidate_record_bytes(int32_t rows, int32_t cap);
int leat_candidate_record_layout(int32_t rows, int32_t cap, size_t* id_at, size_t* count_at, size_t* best_at);
int leat_sample_from_records(leat_sampler_t* handle, const leat_sample_args* args, const void* records,
                             int32_t parts, int32_t cap, leat_stream_t stream);

/* Vocabulary shards that exchange candidates over peer memory instead of a collective (no reference
   counterpart, like the entries above).  Every rank owns a slice of the vocabulary and a share of
   the rows.  A step is three calls on every rank, on one stream, all ranks taking the same steps in
   the same order:

     leat_shard_select  filters the rank's slice (args as for leat_topk_local) and stores each row's
                        candidates straight into the exchange region of the rank that owns the row
     leat_shard_finish  finishes the rows this rank owns from every rank's candidates (waiting, with a
                        limit, for their arrival) and stores the results into every rank's region
     leat_shard_result  waits (with a limit) for every owner's results and writes them to args'
                        out_ids, out_greedy, out_cut, out_kept (rows,), the same on every rank

   args of the last two: rows, options, seed, position, uniform, flags as for the select; vocab (or
   vocab_total) the whole vocabulary's size; logits ignored; out_probs is not supported.  Pass
   LEAT_FLAG_CLEAR_STATUS to the select only.  A wait that runs out (a rank that never took the
   step) ORs LEAT_STATUS_PEER | LEAT_STATUS_INTERNAL into the status word and the ids read -1; the
   kernels end, nothing hangs.

   Regions: leat_shard_region_bytes(rows, cap, world) bytes per rank, zeroed, each mapped into every
   rank's address space: leat_peer_alloc makes one with cudaMalloc and returns its 64-byte
   inter-process handle, leat_peer_open maps another process's (peer access is enabled as needed);
   ranks in one process may pass plain pointers.  leat_shard_create takes the `world` region
   pointers as this process sees them (index = rank); all ranks must have zeroed their regions
   before any rank's first step.  Only stores cross NVLink; every rank reads its own region. */
size_t leat_shard_region_bytes(int32_t rows, int32_t cap, int32_t world);
int leat_peer_alloc(size_t bytes, void** ptr, unsigned char* handle64);
int leat_peer_open(const unsigned char* handle64, void** ptr);
int leat_peer_close(void* ptr);
int leat_peer_free(void* ptr);
int leat_shard_create(leat_sampler_t* handle, int32_t rank, int32_t world, int32_t rows, int32_t cap,
                      void* const* regions, leat_shard_t** out);
int leat_shard_destroy(leat_shard_t* shard);
int leat_shard_select(leat_shard_t* shard, const leat_sample_args* args, leat_stream_t stream);
int leat_shard_finish(leat_shard_t* shard, const leat_sample_args* args, leat_stream_t stream);
int leat_shard_result(leat_shard_t* shard, const leat_sample_args* args, leat_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* LEAT_SAMPLER_H */
