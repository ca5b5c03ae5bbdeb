// The whole compression op of one layer chunk behind a single C entry point: it sequences the
// stage kernels on the caller's stream with scratch carved out of the caller's workspace.
#include "zp_common.cuh"

namespace {
inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }
}

extern "C" size_t zp_compress_batch_workspace_bytes(int L, int B, int NB, int Hkv, int BS, int dtype,
                                                    int redundancy) {
  const size_t n = (size_t)L * B * Hkv * NB * BS;
  const size_t es = zp::dtype_size(dtype);
  // scores + keep flags + room for up to two passes of window-score partial sums (fp32)
  size_t total = align256(n * es) /* scores */ + align256(n) /* keep flags */ + 256;
  if (dtype != ZP_DTYPE_F32) total += align256(2 * n * sizeof(float) + 256);
  if (redundancy) total += align256(n * es);  /* redundancy logits */
  if (redundancy == 2) total += align256(zp_redundancy_exact_workspace_bytes(L, B, NB, Hkv, BS));
  return total;
}

extern "C" int zp_compress_batch(void* k_cache, void* v_cache, const void* query_cache, void* score_cache,
                                 const int32_t* query_ids, const int32_t* block_table,
                                 const int32_t* target_table, const uint8_t* compressed,
                                 int32_t* new_table, int32_t* context_len, int32_t* next_slot, int L, int B,
                                 int NB, int NT, int Hq, int Hkv, int D, int QCL, int BS,
                                 int64_t kv_stride_layer, int64_t kv_stride_page, int64_t q_stride_layer,
                                 int64_t q_stride_seq, int64_t sc_stride_layer, int64_t sc_stride_page,
                                 const zp_compress_params* pr, int dtype, int impl, void* workspace,
                                 size_t workspace_bytes, void* stream) {
  if (L * B == 0) return ZP_OK;
  ZP_REQUIRE(pr && workspace, "zp_compress_batch: null pointer");
  ZP_REQUIRE(!pr->use_global_score || score_cache, "zp_compress_batch: global score needs a score cache");
  ZP_REQUIRE(NT >= pr->budget_blocks, "zp_compress_batch: target table shorter than the budget");
  const size_t need = zp_compress_batch_workspace_bytes(L, B, NB, Hkv, BS, dtype, pr->redundancy);
  if (workspace_bytes < need) {
    zp::set_error("zp_compress_batch: workspace of %zu bytes, %zu needed", workspace_bytes, need);
    return ZP_ERR_WORKSPACE;
  }
  const size_t n = (size_t)L * B * Hkv * NB * BS;
  const size_t es = zp::dtype_size(dtype);
  char* w = reinterpret_cast<char*>(((uintptr_t)workspace + 255) & ~(uintptr_t)255);
  void* scores = w; w += align256(n * es);
  uint8_t* keep = reinterpret_cast<uint8_t*>(w); w += align256(n);
  void* red = nullptr;
  if (pr->redundancy) { red = w; w += align256(n * es); }
  void* red_ws = w;
  void* win_ws = nullptr;
  size_t win_ws_bytes = 0;
  if (dtype != ZP_DTYPE_F32) {  // placed last: the exact-redundancy scratch (if any) comes first
    char* e = reinterpret_cast<char*>(red_ws);
    if (pr->redundancy == 2) e += align256(zp_redundancy_exact_workspace_bytes(L, B, NB, Hkv, BS));
    win_ws = e; win_ws_bytes = 2 * n * sizeof(float) + 256;
  }
  const float scale = pr->softmax_scale > 0.f ? pr->softmax_scale : 1.0f / sqrtf((float)D);

  int rc = zp_window_score_ws(k_cache, query_cache, query_ids, block_table, scores, nullptr, L, B, NB, Hq,
                              Hkv, D, QCL, BS, kv_stride_layer, kv_stride_page, q_stride_layer, q_stride_seq,
                              scale, 0, dtype, impl, win_ws, win_ws_bytes, stream);
  if (rc) return rc;
  if (pr->use_global_score) {
    rc = zp_global_score(scores, score_cache, block_table, compressed, L, B, NB, Hkv, BS, sc_stride_layer,
                         sc_stride_page, pr->decay_factor, 0, pr->max_norm, dtype, stream);
    if (rc) return rc;
  }
  if (pr->redundancy == 1) {
    rc = zp_redundancy_lightning(k_cache, block_table, red, L, B, NB, Hkv, D, BS, kv_stride_layer,
                                 kv_stride_page, pr->redundancy_threshold, dtype, impl, stream);
  } else if (pr->redundancy == 2) {
    rc = zp_redundancy_exact(k_cache, block_table, red, L, B, NB, Hkv, D, BS, kv_stride_layer,
                             kv_stride_page, pr->redundancy_threshold, dtype, impl, red_ws,
                             zp_redundancy_exact_workspace_bytes(L, B, NB, Hkv, BS), stream);
  }
  if (rc) return rc;
  zp_select_params sp;
  sp.top_k = BS * pr->budget_blocks;
  sp.query_cache_len = pr->query_cache_len;
  sp.pooling_size = pr->pooling_size;
  sp.continues_pooling = pr->continues_pooling;
  sp.use_redundancy = pr->redundancy;
  sp.redundancy_max_norm = pr->use_global_score && pr->max_norm;
  sp.sink_len = pr->sink_len;
  sp.pad_mask = 1;
  sp.redundancy_lambda = pr->redundancy_lambda;
  sp.redundancy_one_minus_lambda = pr->redundancy_one_minus_lambda;
  sp.redundancy_temperature = pr->redundancy_temperature;
  rc = zp_select(scores, red, block_table, compressed, keep, nullptr, L, B, NB, Hkv, BS, &sp, dtype, stream);
  if (rc) return rc;
  rc = zp_compact(k_cache, v_cache, pr->use_global_score ? score_cache : nullptr, keep, block_table,
                  target_table, L, B, NB, NT, Hkv, D, BS, kv_stride_layer, kv_stride_page, sc_stride_layer,
                  sc_stride_page, dtype, stream);
  if (rc) return rc;
  if (new_table) rc = zp_update_tables(target_table, new_table, context_len, next_slot, B, NT, NT, BS, stream);
  return rc;
}
