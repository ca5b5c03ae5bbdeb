/*
 * libzipage_b200 — C ABI of the compressed-PagedAttention hot path for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes raw DEVICE pointers, explicit sizes/strides (in ELEMENTS unless the
 * name says bytes) and a CUDA stream (cudaStream_t passed as void*; NULL = legacy default
 * stream).  Calls are asynchronous with respect to the host, never synchronise the device, keep
 * no global mutable state (safe to call from several host threads on different streams) and,
 * unless stated otherwise, allocate nothing: scratch memory is passed in by the caller and its
 * size comes from the matching *_workspace_bytes query.
 *
 * Return value: ZP_OK (0) or a negative ZP_ERR_* code; zp_last_error() then returns a
 * thread-local description.  There is no CPU fallback.
 *
 * Layouts (the reference's, unchanged):
 *   K/V cache    [L, P, BS, Hkv, D]   L layers (a chunk), P pages, BS = 256 slots per page
 *   query cache  [L, C, QCL, Hq, D]   observation window: last QCL queries of each sequence
 *   score cache  [L, P, BS, Hkv]
 *   scores/flags [L, B, Hkv, NB, BS]  B sequences of the call, NB = padded table length
 *   block_table  [B, NB] int32        -1 padding, id >= 0 page, -(id)-2 = last page of the sequence
 *   target table [B, NT] int32        destination pages of the compaction (NT = budget + 1)
 * Only the two leading strides of a cache (layer, page) are free; the rest is contiguous.
 * dtype codes select the cache element type T.
 */
#ifndef ZIPAGE_B200_H_
#define ZIPAGE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ZP_OK 0
#define ZP_ERR_INVALID_ARGUMENT (-1)
#define ZP_ERR_CUDA (-2)
#define ZP_ERR_UNSUPPORTED (-3)
#define ZP_ERR_WORKSPACE (-4)

#define ZP_DTYPE_BF16 0
#define ZP_DTYPE_F32 1
#define ZP_DTYPE_F16 2

/* kernel families a call may use: ZP_IMPL_AUTO picks tcgen05 kernels for 16-bit caches with
 * head_dim 128 and the portable SIMT kernels otherwise (fp32 caches always use SIMT fp32 maths). */
#define ZP_IMPL_AUTO 0
#define ZP_IMPL_SIMT 1
#define ZP_IMPL_TCGEN05 2

const char* zp_last_error(void);
int zp_version(void);

/* The tcgen05 kernels bound every wait on a barrier; a wait that runs out makes the kernel return
 * early and raises a device-side error word (no reference counterpart: the reference has no such
 * kernels).  This call synchronises the device, stores the word in *code_out (0 = no error; else an
 * internal code naming the wait) and clears it when reset != 0. */
int zp_device_error(int* code_out, int reset);
/* The same word without a device-wide synchronisation: a 4-byte copy into host_out (pinned host
 * memory) ordered on `stream`; the caller reads *host_out after it has synchronised that stream.
 * The word is not cleared.  (No reference counterpart.) */
int zp_device_error_async(int* host_out, void* stream);

/* Replaces store_kvcache, zipage/layers/attention.py:12-50.
 * key/value [N, Hkv, D] (row stride given), caches contiguous [P*BS, Hkv, D];
 * row i goes to flat slot slot_mapping[i]; slot -1 is skipped. */
int zp_store_kv(const void* key, const void* value, void* k_cache, void* v_cache,
                const int32_t* slot_mapping, int n_tokens, int num_kv_heads, int head_dim,
                int64_t key_stride0, int64_t value_stride0, int dtype, void* stream);

/* Replaces store_query_cache, zipage/kernel/store_query_cache.py:7-68.
 * query [n_query_rows, Hq, D]; query_cache [cache_seqs, window_len, Hq, D] (one layer); triples
 * [n_triples, 3] int32 = (row of query, query_id, window index).  valid_count: NULL, or a device
 * word holding how many leading triples are valid (a list built on the device into a buffer of
 * fixed capacity, as zp_prepare_decode leaves it): the rest are not read.  A triple that names
 * no row of `query` or no slot of the cache is skipped. */
int zp_store_query(const void* query, void* query_cache, const int32_t* triples, int n_triples,
                   int num_heads, int head_dim, int64_t query_stride0, int64_t cache_stride_seq,
                   int64_t cache_stride_slot, int dtype, const int32_t* valid_count,
                   int n_query_rows, int cache_seqs, int window_len, void* stream);

/* Replaces attention_score, zipage/kernel/attention_score.py:8-250 (kernel + torch glue), without
 * the [L,B,Hq,QCL,NB,BS] logits buffer: softmax over the sequence of the window queries' logits,
 * max over the query heads of a KV group, mean (reduce_mode 0) or max (1) over the window rows.
 * scores_out [L,B,Hkv,NB,BS] T (padded pages get 0).  logits_out is NULL or a
 * [L,B,Hq,QCL,NB,BS] T buffer that receives the masked logits (return_logits=True). */
int zp_window_score(const void* k_cache, const void* query_cache, const int32_t* seq_idx,
                    const int32_t* block_table, void* scores_out, void* logits_out, int L, int B,
                    int NB, int Hq, int Hkv, int D, int QCL, int BS, int64_t k_stride_layer,
                    int64_t k_stride_page, int64_t q_stride_layer, int64_t q_stride_seq,
                    float softmax_scale, int reduce_mode, int dtype, int impl, void* stream);

/* Same as zp_window_score with scratch.  The tcgen05 kernel handles 128 window rows (G*QCL) per
 * pass; larger windows (e.g. 8 query heads per KV head with a 32-token window) take several passes
 * whose per-key sums meet in this workspace (zp_window_score_workspace_bytes + 256; 0 bytes when
 * one pass suffices).  Without a sufficient workspace such shapes run on the portable SIMT kernel. */
size_t zp_window_score_workspace_bytes(int L, int B, int NB, int Hq, int Hkv, int QCL);
int zp_window_score_ws(const void* k_cache, const void* query_cache, const int32_t* seq_idx,
                       const int32_t* block_table, void* scores_out, void* logits_out, int L, int B,
                       int NB, int Hq, int Hkv, int D, int QCL, int BS, int64_t k_stride_layer,
                       int64_t k_stride_page, int64_t q_stride_layer, int64_t q_stride_seq,
                       float softmax_scale, int reduce_mode, int dtype, int impl, void* workspace,
                       size_t workspace_bytes, void* stream);

/* Replaces global_score, zipage/kernel/global_score.py:8-120 (activate 0 = max, 1 = sum), plus the
 * optional max-normalisation that precedes it, zipage/engine/model_runner.py:482-487
 * (max_norm != 0: scores are first divided by their per-(layer, seq, head) maximum).
 * scores [L,B,Hkv,NB,BS] and score_cache [L,P,BS,Hkv] are both updated in place. */
int zp_global_score(void* scores, void* score_cache, const int32_t* block_table,
                    const uint8_t* compressed, int L, int B, int NB, int Hkv, int BS,
                    int64_t sc_stride_layer, int64_t sc_stride_page, float decay, int activate,
                    int max_norm, int dtype, void* stream);

/* Replaces key_norm, zipage/kernel/key_norm.py:8-113: norm_out [L,B,Hkv,NB,BS] T, floor 1e-6
 * (padded pages hold the floor). */
int zp_key_norm(const void* k_cache, const int32_t* block_table, void* norm_out, int L, int B,
                int NB, int Hkv, int D, int BS, int64_t k_stride_layer, int64_t k_stride_page,
                float eps, int dtype, void* stream);

/* Replaces the kernels of lightning_redudancy_score (zipage/kernel/lightning_redudancy_score.py:
 * 10-169) and raw_redudancy_score (zipage/kernel/raw_redudancy_score.py:10-155, :218): cosine
 * similarity of key pairs (same page / whole sequence), diagonal zeroed, per column the entry of
 * the latest row above `threshold` zeroed, row sums.  logits_out [L,B,Hkv,NB,BS] T, padded pages
 * -inf.  The exact form needs scratch: zp_redundancy_exact_workspace_bytes(L,B,NB,Hkv,BS). */
int zp_redundancy_lightning(const void* k_cache, const int32_t* block_table, void* logits_out,
                            int L, int B, int NB, int Hkv, int D, int BS, int64_t k_stride_layer,
                            int64_t k_stride_page, float threshold, int dtype, int impl,
                            void* stream);
size_t zp_redundancy_exact_workspace_bytes(int L, int B, int NB, int Hkv, int BS);
int zp_redundancy_exact(const void* k_cache, const int32_t* block_table, void* logits_out, int L,
                        int B, int NB, int Hkv, int D, int BS, int64_t k_stride_layer,
                        int64_t k_stride_page, float threshold, int dtype, int impl,
                        void* workspace, size_t workspace_bytes, void* stream);

/* The torch epilogue of both redundancy functions (lightning :248-252, raw :226-229): in place,
 * logits / (temperature * divisor), minus the row maximum, softmax over the sequence, each step
 * rounded to T.  per_sequence_len != 0: divisor = BS * (#valid pages) (exact form), else BS. */
int zp_redundancy_softmax(void* logits_inout, const int32_t* block_table, int L, int B, int NB,
                          int Hkv, int BS, float temperature, int per_sequence_len, int dtype,
                          void* stream);

/* Selection parameters of zp_select (zipage/engine/model_runner.py:499-602). */
typedef struct zp_select_params {
  int32_t top_k;               /* rows kept per (layer, seq, head): BS * budget              */
  int32_t query_cache_len;     /* window length: last QCL slots of the last page <- +inf      */
  int32_t pooling_size;        /* 0 = no pooling, else odd kernel of max_pool1d (reference: 5) */
  int32_t continues_pooling;   /* pool sequences that were compressed before as well          */
  int32_t use_redundancy;      /* 0 none, 1 lightning (divisor BS), 2 exact (divisor length)   */
  int32_t redundancy_max_norm; /* divide the redundancy by its maximum (global score+max_norm) */
  int32_t sink_len;            /* 0 = off, else first sink_len tokens <- +inf                 */
  int32_t pad_mask;            /* padded pages <- -inf (model_runner.py:592-593); 0 = leave    */
  float redundancy_lambda;           /* lambda                                              */
  float redundancy_one_minus_lambda; /* 1 - lambda, evaluated in double by the caller        */
  float redundancy_temperature;
} zp_select_params;

/* Replaces the pooling / combine / sink / window_mask / pad mask / topk_mask stages
 * (zipage/engine/model_runner.py:499-602, zipage/kernel/window_mask.py:8-72,
 * zipage/kernel/utils.py:21-36).  scores [L,B,Hkv,NB,BS] T (after the global-score stage) and
 * red_logits (same shape, output of zp_redundancy_*; NULL when use_redundancy == 0) are read;
 * keep_out [L,B,Hkv,NB,BS] uint8 receives 1 for the top_k entries of every row — equal scores go
 * to the LOWEST index.  final_out is NULL or receives the selection scores (T). */
int zp_select(const void* scores, const void* red_logits, const int32_t* block_table,
              const uint8_t* compressed, uint8_t* keep_out, void* final_out, int L, int B, int NB,
              int Hkv, int BS, const zp_select_params* params, int dtype, void* stream);

/* Replaces compress_kv (zipage/kernel/compress_kv.py:8-141) and compress_score
 * (zipage/kernel/compress_score.py:8-99): stable forward compaction of the kept rows of every
 * (layer, seq, head) into the pages of target_table, in place.  score_cache may be NULL (then
 * only K/V move); k_cache/v_cache may be NULL (then only the score cache moves).  Requires, as the
 * reference does, that a destination never lies after the row being read (block_manager.py:129-169)
 * and that no more than NT*BS rows are kept. */
int zp_compact(void* k_cache, void* v_cache, void* score_cache, const uint8_t* keep,
               const int32_t* block_table, const int32_t* target_table, int L, int B, int NB,
               int NT, int Hkv, int D, int BS, int64_t kv_stride_layer, int64_t kv_stride_page,
               int64_t sc_stride_layer, int64_t sc_stride_page, int dtype, void* stream);

/* Parameters of zp_compress_batch: the switches ModelRunner.compress reads
 * (zipage/config.py:22-46, zipage/engine/model_runner.py:51-71). */
typedef struct zp_compress_params {
  int32_t budget_blocks;       /* pages kept per sequence; top_k = BS * budget_blocks          */
  int32_t query_cache_len;
  int32_t use_global_score;    /* merge with / persist to score_cache                          */
  int32_t max_norm;            /* divide scores (and redundancy) by their row maximum           */
  int32_t redundancy;          /* 0 none, 1 lightning, 2 exact                                  */
  int32_t pooling_size;        /* 0 = off, else odd max-pool kernel (reference: 5)              */
  int32_t continues_pooling;
  int32_t sink_len;            /* 0 = off                                                       */
  float decay_factor;
  float redundancy_lambda;
  float redundancy_one_minus_lambda;
  float redundancy_temperature;
  float redundancy_threshold;  /* reference default 0.5                                         */
  float softmax_scale;         /* <= 0: head_dim^-0.5                                           */
} zp_compress_params;

/* Replaces one layer-chunk iteration of ModelRunner.compress, zipage/engine/model_runner.py:466-622,
 * as ONE call: window scoring -> [global score] -> [redundancy] -> pooling/combine/masks/top-k ->
 * in-place compaction of K, V (and the score cache) -> optional device-side table update
 * (new_table [B, NT], context_len [B], next_slot [B]; pass NULL to skip).  Scratch comes from the
 * caller: zp_compress_batch_workspace_bytes(L, B, NB, Hkv, BS, dtype, redundancy). */
size_t zp_compress_batch_workspace_bytes(int L, int B, int NB, int Hkv, int BS, int dtype, int redundancy);
int zp_compress_batch(void* k_cache, void* v_cache, const void* query_cache, void* score_cache,
                      const int32_t* query_ids, const int32_t* block_table,
                      const int32_t* target_table, const uint8_t* compressed, int32_t* new_table,
                      int32_t* context_len, int32_t* next_slot, int L, int B, int NB, int NT, int Hq,
                      int Hkv, int D, int QCL, int BS, int64_t kv_stride_layer, int64_t kv_stride_page,
                      int64_t q_stride_layer, int64_t q_stride_seq, int64_t sc_stride_layer,
                      int64_t sc_stride_page, const zp_compress_params* params, int dtype, int impl,
                      void* workspace, size_t workspace_bytes, void* stream);

/* Device-side table update after a compaction (no reference kernel: the reference does this on
 * the host in zipage/engine/scheduler.py:150-156 and model_runner.py:633-675).  For each sequence:
 * new_table[b, :] = target_table[b, :]; context_len[b] = BS*(NT-1) + 1;
 * next_slot[b] = target_table[b, NT-1] * BS (the slot the next token's K/V is stored to). */
int zp_update_tables(const int32_t* target_table, int32_t* new_table, int32_t* context_len,
                     int32_t* next_slot, int B, int NT, int new_table_stride, int BS, void* stream);

/* Replaces flash_attn_with_kvcache as called at zipage/layers/attention.py:95-103: one query token
 * per sequence over its paged K/V.  q,out [B, Hq, D]; caches [P, BS, Hkv, D] (page stride given);
 * cache_seqlens [B]; block_table [B, NBmax] (-1 padded).  Scratch from
 * zp_paged_decode_workspace_bytes.  With too little scratch for the split-KV form the call still
 * succeeds, runs one block per (sequence, kv head) and leaves a note in zp_last_error. */
size_t zp_paged_decode_workspace_bytes(int B, int Hq, int D, int max_splits);
int zp_paged_decode(const void* q, const void* k_cache, const void* v_cache,
                    const int32_t* cache_seqlens, const int32_t* block_table, void* out, int B,
                    int NBmax, int Hq, int Hkv, int D, int BS, int64_t kv_stride_page,
                    float softmax_scale, int dtype, void* workspace, size_t workspace_bytes,
                    void* stream);

/* No counterpart in the reference.  zp_paged_decode for callers that cannot hand over a workspace
 * because they must not allocate device memory when they decode (an engine that gave all free
 * memory to the KV cache, a latency-critical thread that cannot take cudaMalloc's implicit
 * synchronisation).  The split-KV partial results go to a 4 MiB array built into the library
 * (every GPU that loads the library holds it until exit); the call performs no allocation of any
 * kind.  Batches whose split scratch exceeds zp_paged_decode_noalloc_max_scratch_bytes() are
 * rejected with ZP_ERR_WORKSPACE.  The first call on each device looks up the array's device
 * address (cudaGetSymbolAddress) and should therefore be made before any stream capture starts.
 * All calls on a device share the array: it keeps the last call's partials (every entry a call
 * reads is written by that call first, so nothing needs clearing), and two calls whose kernels
 * overlap on the GPU (different streams) race on it — serialise them. */
size_t zp_paged_decode_noalloc_max_scratch_bytes(void);
int zp_paged_decode_noalloc(const void* q, const void* k_cache, const void* v_cache,
                            const int32_t* cache_seqlens, const int32_t* block_table, void* out,
                            int B, int NBmax, int Hq, int Hkv, int D, int BS,
                            int64_t kv_stride_page, float softmax_scale, int dtype, void* stream);

/* Replaces flash_attn_varlen_func as called at zipage/layers/attention.py:79-93: causal
 * (bottom-right aligned) variable-length attention.  q,out [sum_q, Hq, D].  block_table == NULL:
 * k,v dense [sum_k, Hkv, D]; else k,v are the paged caches [P, BS, Hkv, D] and block_table
 * [B, NBmax] lists each sequence's pages. */
int zp_varlen_prefill(const void* q, const void* k, const void* v, const int32_t* cu_seqlens_q,
                      const int32_t* cu_seqlens_k, const int32_t* block_table, void* out, int B,
                      int max_seqlen_q, int NBmax, int Hq, int Hkv, int D, int BS,
                      int64_t kv_stride_page, float softmax_scale, int dtype, void* stream);

/* zp_varlen_prefill with the row counts of q (total_q) and, for dense k/v, of k and v (total_k),
 * which the tcgen05 kernel needs for its tensor maps (tiles that run past a tensor's end read
 * zeros instead of memory behind it), and a choice of kernel family: ZP_IMPL_AUTO picks the
 * tcgen05 kernel for 16-bit tensors with head_dim 128 (pages: a multiple of 128 keys) and the
 * kernels of zp_varlen_prefill otherwise; ZP_IMPL_SIMT always takes the latter; ZP_IMPL_TCGEN05
 * fails with ZP_ERR_UNSUPPORTED where the tcgen05 kernel cannot run. */
int zp_varlen_prefill_ex(const void* q, const void* k, const void* v, const int32_t* cu_seqlens_q,
                         const int32_t* cu_seqlens_k, const int32_t* block_table, void* out, int B,
                         int max_seqlen_q, int NBmax, int Hq, int Hkv, int D, int BS,
                         int64_t kv_stride_page, float softmax_scale, int total_q, int total_k,
                         int impl, int dtype, void* stream);

/* ---- Per-step ops around the attention path (the rows next to the compression path) -------- */

/* Replaces RMSNorm.forward, third_party/nanovllm/layers/layernorm.py:16-50 (both branches).
 * x [n_rows, hidden] (row stride given), weight [hidden], out [n_rows, hidden] (row stride given).
 * residual == NULL: out = T(T(x * rsqrt(mean(x^2) + eps)) * weight).
 * residual != NULL ([n_rows, hidden] contiguous): s = x + residual in fp32, residual_out = T(s)
 * (may be the residual buffer itself), out from the UNROUNDED s as the reference does.
 * out may be x.  hidden <= 2048 16-byte vectors. */
int zp_rms_norm(const void* x, const void* residual, const void* weight, void* out,
                void* residual_out, int n_rows, int hidden, int64_t x_stride, int64_t out_stride,
                float eps, int dtype, void* stream);

/* Replaces SiluAndMul.forward, third_party/nanovllm/layers/activation.py:11-14.
 * x [n_rows, 2*inter] contiguous -> out [n_rows, inter] = T(T(silu(x[:, :inter])) * x[:, inter:]). */
int zp_silu_and_mul(const void* x, void* out, int n_rows, int inter, int dtype, void* stream);

/* Replaces, in one launch, the q/k normalisation and rotation of Qwen3Attention.forward
 * (third_party/nanovllm/models/qwen3.py:75-79: RMSNorm over each q and k head, layernorm.py:17-26,
 * then apply_rotary_emb, rotary_embedding.py:8-16 and :92-103) and the two cache writes of
 * Attention.forward (zipage/layers/attention.py:72-77: store_kvcache, store_query_cache).
 * qkv [n_tokens, (Hq + 2*Hkv) * D] (row stride given) = the fused projection's output;
 * positions [n_tokens] int64; cos_sin [max_position, D] fp32 (cos in the first half of a row, sin
 * in the second: RotaryEmbedding.cos_sin_cache); q_weight, k_weight [D].
 * q_out [n_tokens, Hq, D]; k_out [n_tokens, Hkv, D] or NULL (decode reads K from the cache).
 * slot_mapping [n_tokens] or NULL: flat cache slot of each token (-1 = skip); k_cache / v_cache
 * contiguous [P*BS, Hkv, D] (one layer).  triples [n_triples, 3] int32 (row, query_id, window
 * index) -> query_cache [C, QCL, Hq, D] (one layer; strides in elements).  n_triples_device: NULL,
 * or a device word with the number of valid triples (as zp_prepare_decode leaves it), in which case
 * n_triples is only an upper bound (the rows of `triples`) and no host read-back is needed. */
int zp_qk_norm_rope_store(const void* qkv, const int64_t* positions, const float* cos_sin,
                          const void* q_weight, const void* k_weight, float eps, void* q_out,
                          void* k_out, void* k_cache, void* v_cache, const int32_t* slot_mapping,
                          void* query_cache, const int32_t* triples, int n_triples,
                          const int32_t* n_triples_device, int n_tokens,
                          int Hq, int Hkv, int D, int64_t qkv_stride, int64_t cache_stride_seq,
                          int64_t cache_stride_slot, int dtype, void* stream);

/* Replaces Sampler.calculate_probs + Sampler.sample, zipage/layers/sampler.py:17-31.
 * logits [n_rows, vocab] T, temperatures [n_rows] fp32; tokens_out [n_rows] int64 =
 * argmax(softmax(fp32 logits / T) / max(noise, 1e-10)), lowest index on ties.  noise [n_rows,
 * vocab] fp32 holds the Exp(1) draws (the reference makes them with Tensor.exponential_); with
 * noise == NULL they come from a counter-based generator keyed by (seed, row, index), which is a
 * different stream of draws than torch's. */
int zp_sample(const void* logits, const float* temperatures, const float* noise,
              int64_t* tokens_out, int n_rows, int vocab, uint64_t seed, int dtype, void* stream);

/* Replaces the host loop of ModelRunner.prepare_decode, zipage/engine/model_runner.py:633-675
 * (with get_query_slot_mapping, :319-350), from device-resident state, so that a decode step
 * needs no host-built lists: num_tokens [B] (len(seq)), block_tables [B, table_width] (-1 padded,
 * e.g. as zp_update_tables leaves them), query_ids [B] (-1 = no window buffer).
 * positions_out [B] int64 = num_tokens - 1; context_lens_out [B]; slot_mapping_out [B];
 * triples_out [B, 3] (the first *n_triples_out rows are valid, in sequence order). */
int zp_prepare_decode(const int32_t* num_tokens, const int32_t* block_tables,
                      const int32_t* query_ids, int B, int table_width, int query_cache_len,
                      int block_size, int64_t* positions_out, int32_t* context_lens_out,
                      int32_t* slot_mapping_out, int32_t* triples_out, int32_t* n_triples_out,
                      void* stream);

/* ---- tensor-parallel all-reduce over NVLink peer memory (one process per GPU, one node) ----------
 * Replaces dist.all_reduce(y) of RowParallelLinear.forward, third_party/nanovllm/layers/linear.py:
 * 149-153 (o_proj and down_proj of every decoder block), and, fused with it, the
 * RMSNorm.add_rms_forward that consumes the reduced tensor (third_party/nanovllm/layers/layernorm.py:
 * 28-40, called at third_party/nanovllm/models/qwen3.py:146-152).  The sum is taken in fp32 in rank
 * order and rounded to T once, so every rank holds the same bits.
 *
 * Set-up, once per rank: zp_comm_create allocates this rank's segment (flags + 2 x (world + 1)
 * message areas of max_bytes) with cudaMalloc; the ranks exchange the 64-byte handles of zp_comm_ipc_handle by
 * any host channel and map each other's segment with zp_comm_open_peer (CUDA IPC), or map the
 * segments themselves and pass the pointers to zp_comm_attach_peer.  All ranks must make the same
 * sequence of calls with the same sizes.  Every device-side wait ends after timeout_ms: the call's
 * result is then undefined, zp_comm_status reports ZP_COMM_TIMEOUT and the communicator must be
 * destroyed and created again; the CUDA context stays usable. */
typedef struct zp_comm zp_comm;
#define ZP_COMM_OK 0
#define ZP_COMM_TIMEOUT 1
int zp_comm_create(int rank, int world, size_t max_bytes, int timeout_ms, zp_comm** comm_out);
int zp_comm_segment(zp_comm* comm, void** ptr_out, size_t* bytes_out);
int zp_comm_ipc_handle(zp_comm* comm, void* handle64_out);
int zp_comm_open_peer(zp_comm* comm, int peer, const void* handle64);
int zp_comm_attach_peer(zp_comm* comm, int peer, void* segment);
int zp_comm_status(zp_comm* comm, int* status_out);   /* synchronous 4-byte read */
int zp_comm_destroy(zp_comm* comm);
/* out[i] = T(sum over ranks of in[i]); count elements, count * sizeof(T) a multiple of 16 and at
 * most max_bytes; in == out allowed.  algo: 0 = by size and world, 1 = one-shot (every rank gets
 * all inputs, one meeting), 2 = two-shot (reduce-scatter into every rank's result area, then a
 * local read; two meetings), 3 = flagged lines (one-shot with the epoch stored beside every
 * payload word instead of a meeting; at most 2 MiB; the default up to 512 KiB on up to 4 ranks). */
int zp_all_reduce(zp_comm* comm, const void* in, void* out, int64_t count, int dtype, int algo,
                  void* stream);
/* x = all-reduce(in) [rows, hidden]; s = x + residual; residual_out = T(s);
 * out = T(T(s * rsqrt(mean(s^2) + eps)) * weight) — zp_all_reduce followed by zp_rms_norm with a
 * residual, in one launch.  out may alias in, residual_out may alias residual. */
int zp_all_reduce_add_rms_norm(zp_comm* comm, const void* in, const void* residual, const void* weight,
                               void* out, void* residual_out, int64_t rows, int hidden, float eps,
                               int dtype, int algo, void* stream);

/* Replaces ParallelLMHead's gather of the vocabulary shards to rank 0 (zipage/layers/embed_head.py:
 * 27-34: dist.gather + torch.cat) followed by Sampler.forward on rank 0 (zipage/layers/sampler.py:
 * 17-31): every rank runs the exponential race on its own shard logits[:, rank*Vs:(rank+1)*Vs]
 * and the ranks exchange, per row, 8 bytes of softmax statistics and 8 bytes of (value, index)
 * (each as one 16-byte line that carries the call's epoch beside the payload: no meeting) —
 * one launch per rank, no library collective, every rank ends with the same tokens_out [n_rows].
 * noise: this rank's shard [n_rows, Vs] of the Exp(1) draws, or NULL for the generator of
 * zp_sample (keyed by the global index: the same draws whatever the sharding).
 * comm's max_bytes must be at least 16 * min(n_rows, 4 * SM count). */
int zp_sample_sharded(zp_comm* comm, const void* logits, const float* temperatures, const float* noise,
                      int64_t* tokens_out, int n_rows, int vocab_shard, uint64_t seed, int dtype,
                      void* stream);

/* Test support, not a serving path: the ranks of a world (2, 4 or 8) as ONE cooperative launch on
 * one GPU — grid (blocks, world), every block resident, rank r = comms[r] (all created in this
 * process on the current device, each with the others' segments attached by zp_comm_attach_peer).
 * Runs the same per-rank code as zp_all_reduce (fused = 0; rows x row_elems elements) or
 * zp_all_reduce_add_rms_norm (fused = 1), for world sizes with no multi-GPU machine at hand.
 * ins / outs / residual_outs: one pointer per rank; residual and weight are shared.  algo 1 or 2. */
int zp_all_reduce_emulated(zp_comm* const* comms, int world, const void* const* ins, void* const* outs,
                           const void* residual, const void* weight, void* const* residual_outs,
                           int64_t rows, int row_elems, float eps, int dtype, int algo, int fused,
                           void* stream);

/* Test support, as zp_all_reduce_emulated: zp_sample_sharded for every rank of a world as one
 * cooperative launch on one GPU.  logits_shards[r] [n_rows, vocab_shard], noise_shards (NULL, or
 * one [n_rows, vocab_shard] fp32 pointer per rank), tokens_outs[r] [n_rows] int64. */
int zp_sample_sharded_emulated(zp_comm* const* comms, int world, const void* const* logits_shards,
                               const float* temperatures, const float* const* noise_shards,
                               int64_t* const* tokens_outs, int n_rows, int vocab_shard, uint64_t seed,
                               int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ZIPAGE_B200_H_ */
