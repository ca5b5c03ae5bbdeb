/* zipage_b200 host control plane — C ABI.
 *
 * A native request scheduler and page (block) manager with the behaviour of the reference's
 * Python ones, step for step: zipage/engine/scheduler.py:10-167 (Scheduler),
 * zipage/engine/block_manager.py:26-210 (BlockManager), zipage/engine/sequence.py:14-119
 * (Sequence state).  At 2048 concurrent requests the reference spends 1.6 to 4 ms of Python per
 * decode step in schedule() + postprocess() alone, before it builds the step's index lists
 * (zipage/engine/model_runner.py:633-675) — the same order as the GPU time of the step itself.
 * Here a step is two C calls on arrays (schedule, postprocess) and one more that fills the
 * runner's input arrays for the whole batch (zp_sched_decode_inputs / zp_sched_compress_inputs).
 *
 * Plain host code: no CUDA call, no device pointer.  Sequences are addressed by the handle
 * zp_sched_add() returns (a small non-negative integer, never reused).  Every function returns
 * a count or 0 on success and a negative ZP_SCHED_ERR_* code on failure; zp_sched_last_error()
 * holds the message (per thread).  Every call on a scheduler object takes that object's lock, so
 * calls from two threads are serialised (the reference engine's asynchronous mode calls
 * postprocess from its compression thread, zipage_engine.py:88-96).
 */
#ifndef ZIPAGE_B200_HOST_H
#define ZIPAGE_B200_HOST_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ZP_SCHED_ERR_ARG (-1)       /* null pointer, bad handle, capacity too small */
#define ZP_SCHED_ERR_STATE (-2)     /* the reference would raise here (an assert of its code) */

/* Sequence status codes (zipage/engine/sequence.py:8-11). */
#define ZP_SEQ_WAITING 0
#define ZP_SEQ_RUNNING 1
#define ZP_SEQ_FINISHED 2

/* The fields of zipage/config.py the scheduler reads (scheduler.py:11-27). */
typedef struct zp_sched_config {
  int32_t num_blocks;              /* config.num_kvcache_blocks */
  int32_t block_size;              /* config.kvcache_block_size */
  int32_t max_blocks_per_seq;      /* config.max_cache_blocks_per_seq + 1 */
  int32_t enable_prefix_cache;
  int32_t max_num_seqs;
  int32_t max_num_batched_tokens;
  int32_t eos;
  int32_t max_concurrency;         /* number of observation-window (query) slots */
  int32_t enable_hybrid_engine;
  int32_t query_cache_len;
} zp_sched_config;

const char* zp_sched_last_error(void);

void* zp_sched_create(const zp_sched_config* cfg);
void zp_sched_destroy(void* sched);

/* Scheduler.add(Sequence(token_ids, sampling_params)) (scheduler.py:32-33, sequence.py:18-37):
 * the new sequence goes to the back of the waiting queue.  Returns its handle. */
int zp_sched_add(void* sched, const int32_t* token_ids, int n_tokens, float temperature, int max_tokens,
                 int ignore_eos);

/* Scheduler.schedule() (scheduler.py:47-124): writes the handles of the scheduled sequences in
 * order and whether the step is a prefill.  Returns how many. */
int zp_sched_schedule(void* sched, int32_t* out_handles, int capacity, int32_t* is_prefill);

/* Scheduler.postprocess(seqs, token_ids) (scheduler.py:143-167); token_ids may be null (the
 * call after a compression).  `now` is the wall-clock time stored as time_prefilled /
 * time_finished.  Returns how many of the sequences finished in this call and writes their
 * handles to finished_out (room for n; may be null). */
int zp_sched_postprocess(void* sched, const int32_t* handles, int n, const int32_t* token_ids, double now,
                         int32_t* finished_out);

/* Scheduler.preempt(seq) (scheduler.py:136-141). */
int zp_sched_preempt(void* sched, int handle);

/* What ModelRunner.prepare_prefill does to the sequences it ran (model_runner.py:387):
 * num_cached_tokens = len(seq). */
int zp_sched_mark_prefilled(void* sched, const int32_t* handles, int n);

/* Frees the token list of a finished sequence (its scalar state stays readable). */
int zp_sched_release(void* sched, int handle);

/* out[0..7] = waiting, running, free blocks, used blocks, free query slots, used query slots,
 * sequences ever added, 1 if Scheduler.is_finished(). */
int zp_sched_counts(void* sched, int32_t out[8]);

/* Scalar state of one sequence, out[0..15] = status, num_tokens, num_prompt_tokens,
 * num_cached_tokens, last_token, query_id, require_compress, compressed, prefilled, max_tokens,
 * ignore_eos, len(block_table), len(new_block_table), len(block_to_release), 0, 0. */
int zp_sched_seq_info(void* sched, int handle, int32_t out[16]);
/* The same for n sequences: out[n][16]. */
int zp_sched_seq_info_batch(void* sched, const int32_t* handles, int n, int32_t* out);
/* times[0..1] = time_prefilled, time_finished; temperature */
int zp_sched_seq_times(void* sched, int handle, double times[2], float* temperature);
int zp_sched_seq_set_num_cached(void* sched, int handle, int num_cached_tokens);

/* One list of a sequence: which = 0 block_table, 1 new_block_table, 2 block_to_release,
 * 3 token_ids.  Returns its length (also when out is null or too small: nothing is written then). */
int zp_sched_seq_list(void* sched, int handle, int which, int32_t* out, int capacity);

/* Order of a queue: which = 0 waiting, 1 running (handles), 2 free blocks, 3 free query slots.
 * Returns its length; writes only when it fits. */
int zp_sched_queue(void* sched, int which, int32_t* out, int capacity);

/* Block state, out[0..1] = ref_count, 1 if the block carries a hash; *hash = that hash
 * (block_manager.py:9-23). */
int zp_sched_block_info(void* sched, int block_id, int32_t out[2], uint64_t* hash);

/* BlockManager.compute_hash (block_manager.py:45-51): XXH64 of the optional 8-byte prefix hash
 * followed by the tokens as little-endian int64. */
uint64_t zp_sched_hash_tokens(const int32_t* token_ids, int n, int has_prefix, uint64_t prefix);

/* Inputs of one decode step for n scheduled sequences, what ModelRunner.prepare_decode builds one
 * Python list element at a time (model_runner.py:633-675): last token, number of tokens, query
 * slot and the block table padded with -1 to `table_width` columns.  Returns the widest table. */
int zp_sched_decode_inputs(void* sched, const int32_t* handles, int n, int32_t* input_ids,
                           int32_t* num_tokens, int32_t* query_ids, int32_t* block_tables, int table_width);

/* The sampling temperatures of n sequences (ModelRunner.prepare_sample, model_runner.py:692-697). */
int zp_sched_temperatures(void* sched, const int32_t* handles, int n, float* out);

/* Inputs of one prefill step (ModelRunner.prepare_prefill, model_runner.py:352-422).
 * zp_sched_prefill_sizes: out[0..3] = new tokens of all n sequences, window rows they store,
 * max_seqlen_q, max_seqlen_k.  zp_sched_prefill_inputs fills input_ids / positions / slot_mapping
 * (one entry per new token), cu_seqlens_q / cu_seqlens_k (n + 1 entries) and the window-store
 * triples (row of the flattened batch, query slot, window index; three int32 each), marks the
 * sequences prefilled (num_cached_tokens = len) and returns the number of triples. */
int zp_sched_prefill_sizes(void* sched, const int32_t* handles, int n, int32_t out[4]);
int zp_sched_prefill_inputs(void* sched, const int32_t* handles, int n, int32_t* input_ids, int32_t* positions,
                            int32_t* slot_mapping, int32_t* cu_seqlens_q, int32_t* cu_seqlens_k,
                            int32_t* query_triples);

/* The handles among `handles` whose sequence has require_compress set, in order (the filter of
 * zipage_engine.py:101-105).  Returns how many. */
int zp_sched_compress_due(void* sched, const int32_t* handles, int n, int32_t* out_handles);

/* Inputs of one compression for n sequences with require_compress set (model_runner.py:424-463):
 * block tables padded with -1, the last page written as -(id)-2; the destination pages
 * (new_block_table, `target_width` columns); query slots; 1 where the sequence was compressed
 * before.  Returns the widest table. */
int zp_sched_compress_inputs(void* sched, const int32_t* handles, int n, int32_t* tables, int table_width,
                             int32_t* targets, int target_width, int32_t* query_ids, uint8_t* compressed);

#ifdef __cplusplus
}
#endif
#endif /* ZIPAGE_B200_HOST_H */
