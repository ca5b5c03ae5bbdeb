// Cache writes: this step's K/V rows into the paged cache, window queries into the
// observation-window buffer.  Pure copies; 16-byte vector accesses.
#include "zp_common.cuh"

namespace zp {

// One block per token row; the row (Hkv*D elements) is copied as int4 vectors.
__global__ void store_kv_kernel(const char* __restrict__ key, const char* __restrict__ value,
                                char* __restrict__ k_cache, char* __restrict__ v_cache,
                                const int32_t* __restrict__ slot_mapping, int64_t key_stride_b,
                                int64_t value_stride_b, int row_bytes) {
  const int i = blockIdx.x;
  const int slot = slot_mapping[i];
  if (slot == -1) return;
  const char* ks = key + (int64_t)i * key_stride_b;
  const char* vs = value + (int64_t)i * value_stride_b;
  char* kd = k_cache + (int64_t)slot * row_bytes;
  char* vd = v_cache + (int64_t)slot * row_bytes;
  for (int o = threadIdx.x * 16; o < row_bytes; o += blockDim.x * 16) {
    st16(kd + o, ld16(ks + o));
    st16(vd + o, ld16(vs + o));
  }
}

// One block per triple.  Rows past *valid_count (when given) and triples that do not name a row of
// `query` and a slot of the cache are skipped: a capacity-sized triple buffer whose tail was never
// written (the device-built list of a replayed decode graph) stores nothing from that tail.
__global__ void store_query_kernel(const char* __restrict__ query, char* __restrict__ query_cache,
                                   const int32_t* __restrict__ triples, int64_t q_stride_b,
                                   int64_t c_stride_seq_b, int64_t c_stride_slot_b, int row_bytes,
                                   const int32_t* __restrict__ valid_count, int n_query_rows,
                                   int cache_seqs, int window_len) {
  const int i = blockIdx.x;
  if (valid_count && i >= *valid_count) return;
  const int row = triples[3 * i], qid = triples[3 * i + 1], idx = triples[3 * i + 2];
  if (row < 0 || row >= n_query_rows || qid < 0 || qid >= cache_seqs || idx < 0 || idx >= window_len) return;
  const char* src = query + (int64_t)row * q_stride_b;
  char* dst = query_cache + (int64_t)qid * c_stride_seq_b + (int64_t)idx * c_stride_slot_b;
  for (int o = threadIdx.x * 16; o < row_bytes; o += blockDim.x * 16) st16(dst + o, ld16(src + o));
}

}  // namespace zp

extern "C" int zp_store_kv(const void* key, const void* value, void* k_cache, void* v_cache,
                           const int32_t* slot_mapping, int n_tokens, int num_kv_heads,
                           int head_dim, int64_t key_stride0, int64_t value_stride0, int dtype,
                           void* stream) {
  if (n_tokens == 0) return ZP_OK;
  ZP_REQUIRE(key && value && k_cache && v_cache && slot_mapping, "zp_store_kv: null pointer");
  const size_t es = zp::dtype_size(dtype);
  const int row_bytes = (int)(num_kv_heads * head_dim * es);
  ZP_REQUIRE(row_bytes % 16 == 0 && (key_stride0 * es) % 16 == 0 && (value_stride0 * es) % 16 == 0,
             "zp_store_kv: rows must be multiples of 16 bytes");
  ZP_REQUIRE(((uintptr_t)key | (uintptr_t)value | (uintptr_t)k_cache | (uintptr_t)v_cache) % 16 == 0,
             "zp_store_kv: pointers must be 16-byte aligned");
  const int threads = row_bytes / 16 >= 128 ? 128 : (row_bytes / 16 >= 64 ? 64 : 32);
  zp::store_kv_kernel<<<n_tokens, threads, 0, (cudaStream_t)stream>>>(
      (const char*)key, (const char*)value, (char*)k_cache, (char*)v_cache, slot_mapping,
      key_stride0 * (int64_t)es, value_stride0 * (int64_t)es, row_bytes);
  return zp::check_launch("zp_store_kv");
}

extern "C" int zp_store_query(const void* query, void* query_cache, const int32_t* triples,
                              int n_triples, int num_heads, int head_dim, int64_t query_stride0,
                              int64_t cache_stride_seq, int64_t cache_stride_slot, int dtype,
                              const int32_t* valid_count, int n_query_rows, int cache_seqs,
                              int window_len, void* stream) {
  if (n_triples == 0) return ZP_OK;
  ZP_REQUIRE(query && query_cache && triples, "zp_store_query: null pointer");
  const size_t es = zp::dtype_size(dtype);
  const int row_bytes = (int)(num_heads * head_dim * es);
  ZP_REQUIRE(row_bytes % 16 == 0 && (query_stride0 * es) % 16 == 0 &&
                 (cache_stride_seq * es) % 16 == 0 && (cache_stride_slot * es) % 16 == 0,
             "zp_store_query: rows must be multiples of 16 bytes");
  ZP_REQUIRE(((uintptr_t)query | (uintptr_t)query_cache) % 16 == 0,
             "zp_store_query: pointers must be 16-byte aligned");
  zp::store_query_kernel<<<n_triples, 128, 0, (cudaStream_t)stream>>>(
      (const char*)query, (char*)query_cache, triples, query_stride0 * (int64_t)es,
      cache_stride_seq * (int64_t)es, cache_stride_slot * (int64_t)es, row_bytes, valid_count,
      n_query_rows, cache_seqs, window_len);
  return zp::check_launch("zp_store_query");
}
