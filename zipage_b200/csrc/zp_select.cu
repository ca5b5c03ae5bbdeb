// Pooling, redundancy combine, sink / window / padding masks and the ragged top-k, fused:
// one block per (layer, sequence, kv head) row of N = NB*BS scores held in shared memory.
//
// Top-k: 4-pass (8 bits per pass) radix select of the k-th largest score on order-preserving
// 32-bit keys, then a keep flag for everything above it plus the first (k - #above) entries equal
// to it IN INDEX ORDER — equal scores are resolved towards the lowest index.
#include "zp_common.cuh"

namespace zp {

constexpr int SEL_THREADS = 256;

__device__ __forceinline__ uint32_t order_key(float v) {
  v += 0.0f;  // -0 -> +0 so that the two zeros compare equal
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct SelArgs {
  const void* scores;
  const void* red;
  const int32_t* block_table;
  const uint8_t* compressed;
  uint8_t* keep;
  void* final_out;
  int L, B, NB, Hkv, BS;
  zp_select_params sp;
};

// RED_SMEM: the scaled redundancy logits of the row are staged in shared memory ([N] more
// elements).  Without it they are recomputed from global memory in each of the three passes that
// need them (same arithmetic, same rounding points), which halves the shared memory a row needs:
// the form used for tables too long for both arrays.
template <typename T, bool RED_SMEM>
__global__ void __launch_bounds__(SEL_THREADS) select_kernel(const SelArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int N = a.NB * a.BS;
  T* sS = reinterpret_cast<T*>(smem_raw);       // [N] scores -> final
  T* sR = sS + N;                               // [N] redundancy (only if staged)
  __shared__ float red[32];
  __shared__ int hist[256];
  __shared__ int warp_tot[SEL_THREADS / 32];
  __shared__ uint32_t sh_prefix;
  __shared__ int sh_krem, sh_last_page, sh_nvalid, sh_running;

  const int unit = blockIdx.x, tid = threadIdx.x;
  const int b = (unit / a.Hkv) % a.B;
  const T* gS = reinterpret_cast<const T*>(a.scores) + (int64_t)unit * N;
  const int32_t* table = a.block_table + (int64_t)b * a.NB;

  if (tid == 0) {
    int lastp = -1, nv = 0;
    for (int pg = 0; pg < a.NB; ++pg) {
      const int e = table[pg];
      nv += e != -1;
      if (e < -1) lastp = pg;
    }
    sh_last_page = lastp; sh_nvalid = nv;
  }

  // ---- scores, with max pooling along the token axis (-inf outside the row) ----
  const bool pool = a.sp.pooling_size > 1 && (a.sp.continues_pooling || !a.compressed[b]);
  const int rad = a.sp.pooling_size / 2;
  for (int i = tid; i < N; i += SEL_THREADS) {
    float v;
    if (pool) {
      v = -INFINITY;
      const int lo = max(i - rad, 0), hi = min(i + rad, N - 1);
      for (int j = lo; j <= hi; ++j) v = fmaxf(v, Elem<T>::to_f32(gS[j]));
    } else {
      v = Elem<T>::to_f32(gS[i]);
    }
    sS[i] = Elem<T>::from_f32(v);
  }
  __syncthreads();

  // ---- redundancy: softmax over the sequence of logits/(temperature*divisor), then combine ----
  if (a.sp.use_redundancy) {
    const T* gR = reinterpret_cast<const T*>(a.red) + (int64_t)unit * N;
    const float divisor = a.sp.redundancy_temperature *
                          (float)(a.sp.use_redundancy == 2 ? sh_nvalid * a.BS : a.BS);
    // scaled logit of token i: from shared memory when staged, else recomputed
    auto scaled = [&](int i) -> float {
      return RED_SMEM ? Elem<T>::to_f32(sR[i]) : round_to<T>(Elem<T>::to_f32(gR[i]) / divisor);
    };
    float m = -INFINITY;
    for (int i = tid; i < N; i += SEL_THREADS) {
      const float v = round_to<T>(Elem<T>::to_f32(gR[i]) / divisor);
      if (RED_SMEM) sR[i] = Elem<T>::from_f32(v);
      m = fmaxf(m, v);
    }
    m = block_max(m, red);
    float z = 0.f;
    for (int i = tid; i < N; i += SEL_THREADS) z += expf(round_to<T>(scaled(i) - m));
    z = block_sum(z, red);
    // the largest probability belongs to the largest logit: exp(0) / z
    const float pm = round_to<T>(1.0f / z);
    for (int i = tid; i < N; i += SEL_THREADS) {
      float pr = round_to<T>(expf(round_to<T>(scaled(i) - m)) / z);
      if (a.sp.redundancy_max_norm) pr = round_to<T>(pr / pm);
      const float x = round_to<T>(Elem<T>::to_f32(sS[i]) * a.sp.redundancy_lambda);
      const float y = round_to<T>(pr * a.sp.redundancy_one_minus_lambda);
      sS[i] = Elem<T>::from_f32(x - y);
    }
    __syncthreads();
  }

  // ---- sink, window and padding masks ----
  for (int i = tid; i < N; i += SEL_THREADS) {
    const int pg = i / a.BS, s = i % a.BS;
    float v = Elem<T>::to_f32(sS[i]);
    if (i < a.sp.sink_len) v = INFINITY;
    if (pg == sh_last_page && s >= a.BS - a.sp.query_cache_len) v = INFINITY;
    if (a.sp.pad_mask && table[pg] == -1) v = -INFINITY;
    sS[i] = Elem<T>::from_f32(v);
    if (a.final_out)
      reinterpret_cast<T*>(a.final_out)[(int64_t)unit * N + i] = Elem<T>::from_f32(v);
  }
  __syncthreads();

  uint8_t* keep = a.keep + (int64_t)unit * N;
  const int k = a.sp.top_k;
  if (k >= N) {
    for (int i = tid; i < N; i += SEL_THREADS) keep[i] = 1;
    return;
  }
  if (k <= 0) {
    for (int i = tid; i < N; i += SEL_THREADS) keep[i] = 0;
    return;
  }

  // ---- radix select of the k-th largest key ----
  if (tid == 0) { sh_prefix = 0u; sh_krem = k; }
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    hist[tid] = 0;  // SEL_THREADS == 256 bins
    __syncthreads();
    const uint32_t prefix = sh_prefix;
    const uint32_t pmask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = tid; i < N; i += SEL_THREADS) {
      const uint32_t key = order_key(Elem<T>::to_f32(sS[i]));
      if ((key & pmask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
    }
    __syncthreads();
    if (tid < 32) {
      // lane j owns bins 255-8j .. 248-8j (descending); find the bin holding the k_rem-th entry
      int c[8], tot = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) { c[j] = hist[255 - 8 * tid - j]; tot += c[j]; }
      int incl = tot;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (tid >= o) incl += t;
      }
      const int excl = incl - tot, krem = sh_krem;
      if (excl < krem && krem <= incl) {
        int run = excl;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (run < krem && krem <= run + c[j]) {
            sh_prefix = prefix | ((uint32_t)(255 - 8 * tid - j) << shift);
            sh_krem = krem - run;
          }
          run += c[j];
        }
      }
    }
    __syncthreads();
  }
  const uint32_t kth = sh_prefix;
  const int need_eq = sh_krem;  // entries equal to the k-th key that are kept (lowest indices)

  // ---- keep flags; equal entries ranked in index order ----
  if (tid == 0) sh_running = 0;
  __syncthreads();
  const int lane = tid & 31, w = tid >> 5;
  for (int base = 0; base < N; base += SEL_THREADS) {
    const int i = base + tid;
    uint32_t key = 0u;
    bool eq = false;
    if (i < N) { key = order_key(Elem<T>::to_f32(sS[i])); eq = key == kth; }
    const uint32_t bal = __ballot_sync(0xffffffffu, eq);
    if (lane == 0) warp_tot[w] = __popc(bal);
    __syncthreads();
    int before = sh_running;
    for (int j = 0; j < w; ++j) before += warp_tot[j];
    const int rank = before + __popc(bal & ((1u << lane) - 1u));
    if (i < N) keep[i] = (key > kth || (eq && rank < need_eq)) ? 1 : 0;
    __syncthreads();
    if (tid == 0) {
      int t = 0;
      for (int j = 0; j < SEL_THREADS / 32; ++j) t += warp_tot[j];
      sh_running += t;
    }
    __syncthreads();
  }
}

}  // namespace zp

extern "C" int zp_select(const void* scores, const void* red_logits, const int32_t* block_table,
                         const uint8_t* compressed, uint8_t* keep_out, void* final_out, int L, int B,
                         int NB, int Hkv, int BS, const zp_select_params* params, int dtype,
                         void* stream) {
  if (L * B == 0) return ZP_OK;
  ZP_REQUIRE(scores && block_table && compressed && keep_out && params, "zp_select: null pointer");
  ZP_REQUIRE(!params->use_redundancy || red_logits, "zp_select: redundancy logits missing");
  ZP_REQUIRE(params->pooling_size == 0 || params->pooling_size % 2 == 1,
             "zp_select: pooling_size must be odd");
  ZP_REQUIRE(params->query_cache_len >= 0 && params->query_cache_len <= BS,
             "zp_select: bad query_cache_len");
  const int N = NB * BS;
  // A row lives in shared memory: N scores, plus N scaled redundancy logits when they fit as well
  // (else they are recomputed per pass).  200 KB hold 102 400 16-bit or 51 200 fp32 scores:
  // tables of up to 400 / 200 pages of 256 tokens.
  const size_t row = (size_t)N * zp::dtype_size(dtype);
  const bool red_smem = params->use_redundancy && 2 * row <= 200 * 1024;
  const size_t smem = red_smem ? 2 * row : row;
  if (smem > 200 * 1024) {
    zp::set_error("zp_select: %d tokens per row need %zu bytes of shared memory (max 204800)", N, smem);
    return ZP_ERR_UNSUPPORTED;
  }
  zp::SelArgs a;
  a.scores = scores; a.red = red_logits; a.block_table = block_table; a.compressed = compressed;
  a.keep = keep_out; a.final_out = final_out;
  a.L = L; a.B = B; a.NB = NB; a.Hkv = Hkv; a.BS = BS; a.sp = *params;
  ZP_DISPATCH_DTYPE(dtype, T, {
    void (*kern)(const zp::SelArgs) = red_smem ? zp::select_kernel<T, true> : zp::select_kernel<T, false>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) { zp::set_error("zp_select: %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
    }
    kern<<<L * B * Hkv, zp::SEL_THREADS, smem, (cudaStream_t)stream>>>(a);
  });
  return zp::check_launch("zp_select");
}
