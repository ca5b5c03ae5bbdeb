// In-place compaction of the kept K / V rows (and score-cache scalars) of every
// (layer, sequence, kv head) into the pages of the target table, plus the device-side table update.
//
// One block per unit.  The keep flags are scanned once into a list of source token indices (kept
// rows in table order).  Row j of that list moves to slot (j % BS) of page target[j / BS].  Rows
// are moved in chunks of consecutive j: every thread first loads its part of the chunk into
// registers, the block synchronises, then stores.  Because a destination never lies after the
// row being read in table order (the engine's guarantee, which the reference's serial walk also
// relies on), a store of chunk c can only overwrite rows of chunks <= c, all of which have been
// read by then.  Rows that already sit at their destination are skipped.
// Heads of one page row are adjacent 16-byte-aligned segments, so the units of one sequence touch
// disjoint bytes and run concurrently.
#include "zp_common.cuh"

namespace zp {

constexpr int CP_THREADS = 256;
constexpr int CP_UNROLL = 4;  // rows per thread-group per pass

struct CpArgs {
  char* k;
  char* v;
  char* sc;
  const uint8_t* keep;
  const int32_t* block_table;
  const int32_t* target;
  int L, B, NB, NT, Hkv, BS;
  int row_bytes;       // D * elem size
  int elem_bytes;
  int64_t kv_stride_layer_b, kv_stride_page_b, sc_stride_layer_b, sc_stride_page_b;
};

__global__ void __launch_bounds__(CP_THREADS) compact_kernel(const CpArgs a) {
  extern __shared__ int s_src[];          // [NT*BS] source token index of destination row j
  int* s_pages = s_src + a.NT * a.BS;     // [NB] decoded source page ids (-1 padded)
  int* s_tgt = s_pages + a.NB;            // [NT]
  __shared__ int warp_tot[CP_THREADS / 32];
  __shared__ int sh_running;

  const int unit = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int h = unit % a.Hkv, b = (unit / a.Hkv) % a.B, l = unit / (a.Hkv * a.B);
  const int N = a.NB * a.BS, cap = a.NT * a.BS;
  for (int i = tid; i < a.NB; i += CP_THREADS) {
    const PageRef pr = decode_page(a.block_table[(int64_t)b * a.NB + i]);
    s_pages[i] = pr.valid ? pr.id : -1;
  }
  for (int i = tid; i < a.NT; i += CP_THREADS) s_tgt[i] = a.target[(int64_t)b * a.NT + i];
  if (tid == 0) sh_running = 0;
  __syncthreads();

  // ---- scan the keep flags into the source list ----
  const uint8_t* flags = a.keep + (int64_t)unit * N;
  for (int base = 0; base < N; base += CP_THREADS) {
    const int i = base + tid;
    const bool on = i < N && flags[i] != 0 && s_pages[i / a.BS] >= 0;
    const uint32_t bal = __ballot_sync(0xffffffffu, on);
    if (lane == 0) warp_tot[w] = __popc(bal);
    __syncthreads();
    int pos = sh_running;
    for (int j = 0; j < w; ++j) pos += warp_tot[j];
    pos += __popc(bal & ((1u << lane) - 1u));
    if (on && pos < cap) s_src[pos] = i;
    __syncthreads();
    if (tid == 0) {
      int t = 0;
      for (int j = 0; j < CP_THREADS / 32; ++j) t += warp_tot[j];
      sh_running += t;
    }
    __syncthreads();
  }
  const int kept = min(sh_running, cap);

  // ---- K and V rows ----
  if (a.k) {
    const int vpr = a.row_bytes / 16;            // 16-byte vectors per row
    const int groups = CP_THREADS / vpr;         // rows moved side by side
    const int g = tid / vpr, vec = tid % vpr;
    const int rows_per_pass = groups * CP_UNROLL;
    const int64_t head_off = (int64_t)h * a.row_bytes + vec * 16;
    const int64_t slot_stride = (int64_t)a.Hkv * a.row_bytes;
    char* kl = a.k + (int64_t)l * a.kv_stride_layer_b;
    char* vl = a.v + (int64_t)l * a.kv_stride_layer_b;
    for (int j0 = 0; j0 < kept; j0 += rows_per_pass) {
      int4 kr[CP_UNROLL], vr[CP_UNROLL];
      int64_t doff[CP_UNROLL];
      bool mv[CP_UNROLL];
#pragma unroll
      for (int u = 0; u < CP_UNROLL; ++u) {
        const int j = j0 + u * groups + g;
        mv[u] = false;
        if (g < groups && j < kept) {
          const int src = s_src[j];
          const int64_t soff = (int64_t)s_pages[src / a.BS] * a.kv_stride_page_b +
                               (int64_t)(src % a.BS) * slot_stride + head_off;
          doff[u] = (int64_t)s_tgt[j / a.BS] * a.kv_stride_page_b +
                    (int64_t)(j % a.BS) * slot_stride + head_off;
          mv[u] = soff != doff[u];
          if (mv[u]) { kr[u] = ld16(kl + soff); vr[u] = ld16(vl + soff); }
        }
      }
      __syncthreads();
#pragma unroll
      for (int u = 0; u < CP_UNROLL; ++u)
        if (mv[u]) { st16(kl + doff[u], kr[u]); st16(vl + doff[u], vr[u]); }
      __syncthreads();
    }
  }

  // ---- score-cache scalars [page][slot][head] ----
  if (a.sc) {
    char* sl = a.sc + (int64_t)l * a.sc_stride_layer_b;
    const int64_t slot_stride = (int64_t)a.Hkv * a.elem_bytes;
    for (int j0 = 0; j0 < kept; j0 += CP_THREADS) {
      const int j = j0 + tid;
      bool mv = false;
      int64_t doff = 0;
      uint32_t val = 0;
      if (j < kept) {
        const int src = s_src[j];
        const int64_t soff = (int64_t)s_pages[src / a.BS] * a.sc_stride_page_b +
                             (int64_t)(src % a.BS) * slot_stride + (int64_t)h * a.elem_bytes;
        doff = (int64_t)s_tgt[j / a.BS] * a.sc_stride_page_b + (int64_t)(j % a.BS) * slot_stride +
               (int64_t)h * a.elem_bytes;
        mv = soff != doff;
        if (mv) val = a.elem_bytes == 4 ? *reinterpret_cast<const uint32_t*>(sl + soff)
                                        : *reinterpret_cast<const uint16_t*>(sl + soff);
      }
      __syncthreads();
      if (mv) {
        if (a.elem_bytes == 4) *reinterpret_cast<uint32_t*>(sl + doff) = val;
        else *reinterpret_cast<uint16_t*>(sl + doff) = (uint16_t)val;
      }
      __syncthreads();
    }
  }
}

__global__ void update_tables_kernel(const int32_t* __restrict__ target, int32_t* __restrict__ new_table,
                                     int32_t* __restrict__ context_len, int32_t* __restrict__ next_slot,
                                     int B, int NT, int new_table_stride, int BS) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  for (int i = 0; i < new_table_stride; ++i)
    new_table[(int64_t)b * new_table_stride + i] = i < NT ? target[(int64_t)b * NT + i] : -1;
  if (context_len) context_len[b] = BS * (NT - 1) + 1;
  if (next_slot) next_slot[b] = target[(int64_t)b * NT + NT - 1] * BS;
}

}  // namespace zp

extern "C" int zp_compact(void* k_cache, void* v_cache, void* score_cache, const uint8_t* keep,
                          const int32_t* block_table, const int32_t* target_table, int L, int B,
                          int NB, int NT, int Hkv, int D, int BS, int64_t kv_stride_layer,
                          int64_t kv_stride_page, int64_t sc_stride_layer, int64_t sc_stride_page,
                          int dtype, void* stream) {
  if (L * B == 0) return ZP_OK;
  ZP_REQUIRE(keep && block_table && target_table, "zp_compact: null pointer");
  ZP_REQUIRE((k_cache == nullptr) == (v_cache == nullptr), "zp_compact: K and V go together");
  ZP_REQUIRE(k_cache || score_cache, "zp_compact: nothing to compact");
  ZP_REQUIRE(dtype == ZP_DTYPE_BF16 || dtype == ZP_DTYPE_F16 || dtype == ZP_DTYPE_F32,
             "zp_compact: unknown dtype code %d", dtype);
  const int es = (int)zp::dtype_size(dtype);
  zp::CpArgs a;
  a.k = (char*)k_cache; a.v = (char*)v_cache; a.sc = (char*)score_cache;
  a.keep = keep; a.block_table = block_table; a.target = target_table;
  a.L = L; a.B = B; a.NB = NB; a.NT = NT; a.Hkv = Hkv; a.BS = BS;
  a.row_bytes = D * es; a.elem_bytes = es;
  a.kv_stride_layer_b = kv_stride_layer * es; a.kv_stride_page_b = kv_stride_page * es;
  a.sc_stride_layer_b = sc_stride_layer * es; a.sc_stride_page_b = sc_stride_page * es;
  if (k_cache) {
    ZP_REQUIRE(a.row_bytes % 16 == 0 && a.row_bytes / 16 <= zp::CP_THREADS &&
                   zp::CP_THREADS % (a.row_bytes / 16) == 0,
               "zp_compact: head_dim %d not supported", D);
    ZP_REQUIRE(((uintptr_t)k_cache | (uintptr_t)v_cache) % 16 == 0 && a.kv_stride_layer_b % 16 == 0 &&
                   a.kv_stride_page_b % 16 == 0,
               "zp_compact: K/V caches must be 16-byte aligned");
  }
  const size_t smem = sizeof(int) * ((size_t)NT * BS + NB + NT);
  if (smem > 200 * 1024) {
    zp::set_error("zp_compact: target of %d pages too large", NT);
    return ZP_ERR_UNSUPPORTED;
  }
  auto kern = zp::compact_kernel;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { zp::set_error("zp_compact: %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  }
  kern<<<L * B * Hkv, zp::CP_THREADS, smem, (cudaStream_t)stream>>>(a);
  return zp::check_launch("zp_compact");
}

extern "C" int zp_update_tables(const int32_t* target_table, int32_t* new_table, int32_t* context_len,
                                int32_t* next_slot, int B, int NT, int new_table_stride, int BS,
                                void* stream) {
  if (B == 0) return ZP_OK;
  ZP_REQUIRE(target_table && new_table, "zp_update_tables: null pointer");
  ZP_REQUIRE(new_table_stride >= NT, "zp_update_tables: new table narrower than the target");
  zp::update_tables_kernel<<<(B + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
      target_table, new_table, context_len, next_slot, B, NT, new_table_stride, BS);
  return zp::check_launch("zp_update_tables");
}
