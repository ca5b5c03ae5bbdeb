// Key-similarity redundancy: key norms, the similarity row sums with the "latest similar key is
// exempt" rule (lightning = same page only, exact = whole sequence), and the softmax epilogue.
// This file holds the portable SIMT kernels (fp32 maths, any cache dtype).
//
// How the exemption is computed.  The reference zeroes, in every column n of S = K^ K^T, the entry
// of the LARGEST row m with S[m,n] > threshold, then sums rows.  S is symmetric, so reading row n
// instead of column n: c(n) = the largest column with S[n,c] > threshold and v(n) = S[n,c(n)];
// the zeroed entry of column n is (c(n), n) and its value is v(n).  Hence
//     logits[m] = rowsum(S)[m] - sum over { n : c(n) = m } of v(n),
// which needs only row-wise state while the columns stream by.
#include "zp_common.cuh"

namespace zp {

constexpr int RD_THREADS = 256;
constexpr int RD_CT = 64;  // columns per tile

// Load `nrows` keys (slots slot0..) of one head from a page, normalise, store fp32 rows of LD.
// One warp per key row; norm = max(T(sqrt(sum k^2)), T(eps)) as key_norm.py:53-56,112.
template <typename T, int D>
__device__ __forceinline__ void load_normalised_rows(const T* __restrict__ kpage, int h, int Hkv,
                                                     int slot0, int nrows, float* __restrict__ dst,
                                                     float eps_t) {
  constexpr int LD = D + 4;
  constexpr int EPL = D / 32;  // elements per lane
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int r = w; r < nrows; r += nw) {
    const T* src = kpage + ((int64_t)(slot0 + r) * Hkv + h) * D + lane * EPL;
    float v[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) v[j] = Elem<T>::to_f32(src[j]);
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) ss = fmaf(v[j], v[j], ss);
    ss = warp_sum(ss);
    const float nrm = fmaxf(round_to<T>(sqrtf(ss)), eps_t);
#pragma unroll
    for (int j = 0; j < EPL; ++j) dst[r * LD + lane * EPL + j] = v[j] / nrm;
  }
}

struct RdParams {
  const void* k_cache;
  const int32_t* block_table;
  void* logits_out;   // lightning: written here; exact: written by the finalize kernel
  float* rowsum;      // exact only: [units][NB*BS]
  long long* sub;     // exact only: [units][NB*BS], zeroed before the launch
  int L, B, NB, Hkv, BS;
  int64_t k_stride_layer, k_stride_page;
  float threshold, eps;
  int exact;
};

// One block per (unit, row page).  Rows: the page's BS (=256) keys, resident in shared memory.
// Thread (ty,tx) owns rows rb*64 + ty*4 + a (rb,a < 4) and, of each 64-column tile, columns
// tx + 16c (c < 4).
template <typename T, int D>
__global__ void __launch_bounds__(RD_THREADS, 1) redundancy_rows_kernel(const RdParams p) {
  constexpr int LD = D + 4;
  extern __shared__ __align__(16) float smem[];
  float* sR = smem;                    // [256][LD] normalised row keys
  float* sC = sR + 256 * LD;           // [64][LD]  normalised column keys
  float* sSum = sC + RD_CT * LD;       // [256]
  float* sVal = sSum + 256;            // [256]
  int* sCol = reinterpret_cast<int*>(sVal + 256);  // [256]

  const int mp = blockIdx.x % p.NB;
  const int unit = blockIdx.x / p.NB;
  const int h = unit % p.Hkv, b = (unit / p.Hkv) % p.B, l = unit / (p.Hkv * p.B);
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int32_t* table = p.block_table + (int64_t)b * p.NB;
  const PageRef rp = decode_page(table[mp]);
  T* lout = reinterpret_cast<T*>(p.logits_out) + ((int64_t)unit * p.NB + mp) * p.BS;
  if (!rp.valid) {
    if (!p.exact)
      for (int s = tid; s < p.BS; s += RD_THREADS) lout[s] = Elem<T>::from_f32(-INFINITY);
    return;
  }
  const T* kbase = reinterpret_cast<const T*>(p.k_cache) + (int64_t)l * p.k_stride_layer;
  const float eps_t = round_to<T>(p.eps);
  load_normalised_rows<T, D>(kbase + (int64_t)rp.id * p.k_stride_page, h, p.Hkv, 0, 256, sR, eps_t);

  float rsum[4][4], bval[4][4];
  int bcol[4][4];
#pragma unroll
  for (int rb = 0; rb < 4; ++rb)
#pragma unroll
    for (int a = 0; a < 4; ++a) { rsum[rb][a] = 0.f; bval[rb][a] = 0.f; bcol[rb][a] = -1; }

  const int pg_lo = p.exact ? 0 : mp, pg_hi = p.exact ? p.NB : mp + 1;
  for (int pg = pg_lo; pg < pg_hi; ++pg) {
    const PageRef cp = decode_page(table[pg]);
    if (!cp.valid) continue;
    const T* cpage = kbase + (int64_t)cp.id * p.k_stride_page;
    for (int s0 = 0; s0 < p.BS; s0 += RD_CT) {
      __syncthreads();
      load_normalised_rows<T, D>(cpage, h, p.Hkv, s0, RD_CT, sC, eps_t);
      __syncthreads();
#pragma unroll
      for (int rb = 0; rb < 4; ++rb) {
        float acc[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int c = 0; c < 4; ++c) acc[a][c] = 0.f;
        const float* rbase = sR + (rb * 64 + ty * 4) * LD;
#pragma unroll 4
        for (int d = 0; d < D; d += 4) {
          float4 cv[4], rv[4];
#pragma unroll
          for (int c = 0; c < 4; ++c) cv[c] = *reinterpret_cast<const float4*>(sC + (tx + 16 * c) * LD + d);
#pragma unroll
          for (int a = 0; a < 4; ++a) rv[a] = *reinterpret_cast<const float4*>(rbase + a * LD + d);
#pragma unroll
          for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              acc[a][c] = fmaf(rv[a].x, cv[c].x, acc[a][c]);
              acc[a][c] = fmaf(rv[a].y, cv[c].y, acc[a][c]);
              acc[a][c] = fmaf(rv[a].z, cv[c].z, acc[a][c]);
              acc[a][c] = fmaf(rv[a].w, cv[c].w, acc[a][c]);
            }
        }
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          const int m = mp * p.BS + rb * 64 + ty * 4 + a;  // token index in table order
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int n = pg * p.BS + s0 + tx + 16 * c;
            const float s = (n == m) ? 0.f : acc[a][c];
            rsum[rb][a] += s;
            if (s > p.threshold) { bcol[rb][a] = n; bval[rb][a] = s; }
          }
        }
      }
    }
  }
  // combine the 16 column groups of each row (lanes of one half-warp)
#pragma unroll
  for (int rb = 0; rb < 4; ++rb)
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      float s = rsum[rb][a], v = bval[rb][a];
      int c = bcol[rb][a];
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) {
        s += __shfl_xor_sync(0xffffffffu, s, o);
        const int c2 = __shfl_xor_sync(0xffffffffu, c, o);
        const float v2 = __shfl_xor_sync(0xffffffffu, v, o);
        if (c2 > c) { c = c2; v = v2; }
      }
      if (tx == 0) {
        const int r = rb * 64 + ty * 4 + a;
        sSum[r] = s; sCol[r] = c; sVal[r] = v;
      }
    }
  __syncthreads();
  const int m = tid;  // 256 threads, 256 rows
  if (!p.exact) {
    const int me = mp * p.BS + m;
    float subtract = 0.f;
    for (int n = 0; n < 256; ++n)
      if (sCol[n] == me) subtract += sVal[n];
    lout[m] = Elem<T>::from_f32(sSum[m] - subtract);
  } else {
    const int64_t base = (int64_t)unit * p.NB * p.BS;
    p.rowsum[base + mp * p.BS + m] = sSum[m];
    if (sCol[m] >= 0) {
      const long long fx = __float2ll_rn(sVal[m] * 4294967296.f);  // exact for |v| >= 2^-9
      atomicAdd(reinterpret_cast<unsigned long long*>(p.sub + base + sCol[m]), (unsigned long long)fx);
    }
  }
}

// exact form: logits = T(rowsum - sub), padded pages -inf.  With `rn` (the tcgen05 path), `rowsum`
// holds k_m . w and the row sum is rn_m * (k_m . w) - S[m,m] (stats: rn at [0,total), S[m,m] at
// [total, 2*total)).
template <typename T>
__global__ void redundancy_finalize_kernel(const float* __restrict__ rowsum,
                                           const long long* __restrict__ sub,
                                           const float* __restrict__ rn,
                                           const int32_t* __restrict__ block_table,
                                           T* __restrict__ logits, int B, int NB, int Hkv, int BS,
                                           int64_t total) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int pg = (int)((i / BS) % NB);
  const int b = (int)((i / ((int64_t)BS * NB * Hkv)) % B);
  if (block_table[(int64_t)b * NB + pg] == -1) { logits[i] = Elem<T>::from_f32(-INFINITY); return; }
  const float s = (float)((double)sub[i] * (1.0 / 4294967296.0));
  const float rs = rn ? rn[i] * rowsum[i] - rn[total + i] : rowsum[i];
  logits[i] = Elem<T>::from_f32(rs - s);
}

// One warp per key: norm_out = max(T(sqrt(sum k^2)), T(eps)); padded pages get T(eps).
template <typename T, int D>
__global__ void key_norm_kernel(const T* __restrict__ k_cache, const int32_t* __restrict__ block_table,
                                T* __restrict__ out, int B, int NB, int Hkv, int BS,
                                int64_t k_stride_layer, int64_t k_stride_page, float eps) {
  constexpr int EPL = D / 32;
  const int pg = blockIdx.x % NB, unit = blockIdx.x / NB;
  const int h = unit % Hkv, b = (unit / Hkv) % B, l = unit / (Hkv * B);
  const PageRef pr = decode_page(block_table[(int64_t)b * NB + pg]);
  T* o = out + ((int64_t)unit * NB + pg) * BS;
  const float eps_t = round_to<T>(eps);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (!pr.valid) {
    for (int s = threadIdx.x; s < BS; s += blockDim.x) o[s] = Elem<T>::from_f32(eps_t);
    return;
  }
  const T* kpage = k_cache + (int64_t)l * k_stride_layer + (int64_t)pr.id * k_stride_page;
  for (int r = w; r < BS; r += nw) {
    const T* src = kpage + ((int64_t)r * Hkv + h) * D + lane * EPL;
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) { const float v = Elem<T>::to_f32(src[j]); ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    if (lane == 0) o[r] = Elem<T>::from_f32(fmaxf(round_to<T>(sqrtf(ss)), eps_t));
  }
}

// In place: x = T(x / (temperature*divisor)); x = T(x - max); softmax over the row, rounded to T.
// One block per (layer, seq, head) row of N = NB*BS values.
template <typename T>
__global__ void redundancy_softmax_kernel(T* __restrict__ x, const int32_t* __restrict__ block_table,
                                          int B, int NB, int Hkv, int BS, float temperature,
                                          int per_sequence_len) {
  __shared__ float red[32];
  const int unit = blockIdx.x, b = (unit / Hkv) % B, N = NB * BS;
  T* row = x + (int64_t)unit * N;
  float divisor = temperature * (float)BS;
  if (per_sequence_len) {
    int valid = 0;
    for (int pg = 0; pg < NB; ++pg) valid += block_table[(int64_t)b * NB + pg] != -1;
    divisor = temperature * (float)(valid * BS);
  }
  float m = -INFINITY;
  for (int i = threadIdx.x; i < N; i += blockDim.x) {
    const float v = round_to<T>(Elem<T>::to_f32(row[i]) / divisor);
    row[i] = Elem<T>::from_f32(v);
    m = fmaxf(m, v);
  }
  m = block_max(m, red);
  float z = 0.f;
  for (int i = threadIdx.x; i < N; i += blockDim.x)
    z += expf(round_to<T>(Elem<T>::to_f32(row[i]) - m));
  z = block_sum(z, red);
  for (int i = threadIdx.x; i < N; i += blockDim.x) {
    const float e = expf(round_to<T>(Elem<T>::to_f32(row[i]) - m));
    row[i] = Elem<T>::from_f32(e / z);
  }
}

template <typename T, int D>
static int launch_rows(const RdParams& p, cudaStream_t st) {
  constexpr int LD = D + 4;
  const size_t smem = sizeof(float) * ((256 + RD_CT) * LD + 3 * 256);
  auto kern = redundancy_rows_kernel<T, D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_error("zp_redundancy: %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  kern<<<p.L * p.B * p.Hkv * p.NB, RD_THREADS, smem, st>>>(p);
  return check_launch("zp_redundancy rows kernel");
}

static int redundancy_simt(const RdParams& p, int D, int dtype, cudaStream_t st) {
  ZP_DISPATCH_DTYPE(dtype, T, {
    if (D == 128) return launch_rows<T, 128>(p, st);
    if (D == 64) return launch_rows<T, 64>(p, st);
  });
  set_error("zp_redundancy: head_dim %d not supported (64 or 128)", D);
  return ZP_ERR_UNSUPPORTED;
}

// tcgen05 path (zp_redundancy_tc.cu)
int redundancy_tc(const void* k_cache, const int32_t* block_table, void* logits_out, int L, int B,
                  int NB, int Hkv, int64_t k_stride_layer, int64_t k_stride_page, float threshold,
                  float eps, int dtype, cudaStream_t st);

// tcgen05 path of the exact form (zp_redundancy_exact_tc.cu)
int redundancy_exact_tc(const void* k_cache, const int32_t* block_table, float* rowsum, long long* sub,
                        float* stats, int L, int B, int NB, int Hkv, int64_t k_stride_layer,
                        int64_t k_stride_page, float threshold, float eps, int dtype, cudaStream_t st);

// which kernel family a call uses: 1 = tcgen05, 0 = SIMT, <0 = error already set
static int pick_tc(int impl, int dtype, int D, int BS, const char* who) {
  const bool can = (dtype == ZP_DTYPE_BF16 || dtype == ZP_DTYPE_F16) && D == 128 && BS == 256;
  if (impl == ZP_IMPL_SIMT) return 0;
  if (impl == ZP_IMPL_TCGEN05 && !can) {
    set_error("%s: the tcgen05 kernels need a 16-bit cache, head_dim 128 and page size 256", who);
    return ZP_ERR_UNSUPPORTED;
  }
  return can ? 1 : 0;
}

}  // namespace zp

extern "C" int zp_key_norm(const void* k_cache, const int32_t* block_table, void* norm_out, int L,
                           int B, int NB, int Hkv, int D, int BS, int64_t k_stride_layer,
                           int64_t k_stride_page, float eps, int dtype, void* stream) {
  if (L * B == 0) return ZP_OK;
  ZP_REQUIRE(k_cache && block_table && norm_out, "zp_key_norm: null pointer");
  ZP_REQUIRE(D == 64 || D == 128, "zp_key_norm: head_dim %d not supported (64 or 128)", D);
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = L * B * Hkv * NB;
  ZP_DISPATCH_DTYPE(dtype, T, {
    if (D == 128)
      zp::key_norm_kernel<T, 128><<<grid, 256, 0, st>>>((const T*)k_cache, block_table, (T*)norm_out,
                                                        B, NB, Hkv, BS, k_stride_layer,
                                                        k_stride_page, eps);
    else
      zp::key_norm_kernel<T, 64><<<grid, 256, 0, st>>>((const T*)k_cache, block_table, (T*)norm_out,
                                                       B, NB, Hkv, BS, k_stride_layer,
                                                       k_stride_page, eps);
  });
  return zp::check_launch("zp_key_norm");
}

extern "C" int zp_redundancy_lightning(const void* k_cache, const int32_t* block_table,
                                       void* logits_out, int L, int B, int NB, int Hkv, int D,
                                       int BS, int64_t k_stride_layer, int64_t k_stride_page,
                                       float threshold, int dtype, int impl, void* stream) {
  if (L * B == 0) return ZP_OK;
  ZP_REQUIRE(k_cache && block_table && logits_out, "zp_redundancy_lightning: null pointer");
  ZP_REQUIRE(BS == 256, "zp_redundancy_lightning: page size must be 256 (got %d)", BS);
  zp::RdParams p{};
  p.k_cache = k_cache; p.block_table = block_table; p.logits_out = logits_out;
  p.L = L; p.B = B; p.NB = NB; p.Hkv = Hkv; p.BS = BS;
  p.k_stride_layer = k_stride_layer; p.k_stride_page = k_stride_page;
  p.threshold = threshold; p.eps = 1e-6f; p.exact = 0;
  const int tc = zp::pick_tc(impl, dtype, D, BS, "zp_redundancy_lightning");
  if (tc < 0) return tc;
  if (tc)
    return zp::redundancy_tc(k_cache, block_table, logits_out, L, B, NB, Hkv, k_stride_layer,
                             k_stride_page, threshold, 1e-6f, dtype, (cudaStream_t)stream);
  return zp::redundancy_simt(p, D, dtype, (cudaStream_t)stream);
}

extern "C" size_t zp_redundancy_exact_workspace_bytes(int L, int B, int NB, int Hkv, int BS) {
  // fixed-point subtrahends + row sums; for the tcgen05 kernel also the latest-similar-key records
  // (64 bits per key, zeroed with the subtrahends) and the key statistics:
  // 1/|k| and self-similarity per key, the smallest norm per 32-key chunk, one 128-vector per unit
  const size_t units = (size_t)L * B * Hkv, n = units * NB * BS;
  return n * (sizeof(float) + 2 * sizeof(long long)) + (2 * n + units * ((size_t)NB * 8 + 128)) * sizeof(float) + 256;
}

extern "C" int zp_redundancy_exact(const void* k_cache, const int32_t* block_table, void* logits_out,
                                   int L, int B, int NB, int Hkv, int D, int BS,
                                   int64_t k_stride_layer, int64_t k_stride_page, float threshold,
                                   int dtype, int impl, void* workspace, size_t workspace_bytes,
                                   void* stream) {
  if (L * B == 0) return ZP_OK;
  ZP_REQUIRE(k_cache && block_table && logits_out && workspace, "zp_redundancy_exact: null pointer");
  ZP_REQUIRE(BS == 256, "zp_redundancy_exact: page size must be 256 (got %d)", BS);
  const size_t need = zp_redundancy_exact_workspace_bytes(L, B, NB, Hkv, BS);
  if (workspace_bytes < need) {
    zp::set_error("zp_redundancy_exact: workspace of %zu bytes, %zu needed", workspace_bytes, need);
    return ZP_ERR_WORKSPACE;
  }
  cudaStream_t st = (cudaStream_t)stream;
  const size_t n = (size_t)L * B * Hkv * NB * BS;
  uintptr_t w = ((uintptr_t)workspace + 255) & ~(uintptr_t)255;
  long long* sub = reinterpret_cast<long long*>(w);
  float* rowsum = reinterpret_cast<float*>(w + 2 * n * sizeof(long long));
  float* stats = rowsum + n;
  int tc = zp::pick_tc(impl, dtype, D, BS, "zp_redundancy_exact");
  if (tc < 0) return tc;
  // zeroed: the subtrahends and, for the tcgen05 kernel, the latest-similar-key records
  cudaError_t e = cudaMemsetAsync(sub, 0, (tc ? 2 : 1) * n * sizeof(long long), st);
  if (e != cudaSuccess) { zp::set_error("zp_redundancy_exact: %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  zp::RdParams p{};
  p.k_cache = k_cache; p.block_table = block_table; p.logits_out = logits_out;
  p.rowsum = rowsum; p.sub = sub;
  p.L = L; p.B = B; p.NB = NB; p.Hkv = Hkv; p.BS = BS;
  p.k_stride_layer = k_stride_layer; p.k_stride_page = k_stride_page;
  p.threshold = threshold; p.eps = 1e-6f; p.exact = 1;
  int rc = tc ? zp::redundancy_exact_tc(k_cache, block_table, rowsum, sub, stats, L, B, NB, Hkv,
                                        k_stride_layer, k_stride_page, threshold, 1e-6f, dtype, st)
              : zp::redundancy_simt(p, D, dtype, st);
  if (rc) return rc;
  const int64_t total = (int64_t)n;
  const int blocks = (int)((total + 255) / 256);
  ZP_DISPATCH_DTYPE(dtype, T, {
    zp::redundancy_finalize_kernel<T><<<blocks, 256, 0, st>>>(rowsum, sub, tc ? stats : nullptr,
                                                             block_table, (T*)logits_out, B, NB,
                                                             Hkv, BS, total);
  });
  return zp::check_launch("zp_redundancy_exact finalize");
}

extern "C" int zp_redundancy_softmax(void* logits_inout, const int32_t* block_table, int L, int B,
                                     int NB, int Hkv, int BS, float temperature,
                                     int per_sequence_len, int dtype, void* stream) {
  if (L * B == 0) return ZP_OK;
  ZP_REQUIRE(logits_inout && block_table, "zp_redundancy_softmax: null pointer");
  ZP_DISPATCH_DTYPE(dtype, T, {
    zp::redundancy_softmax_kernel<T><<<L * B * Hkv, 256, 0, (cudaStream_t)stream>>>(
        (T*)logits_inout, block_table, B, NB, Hkv, BS, temperature, per_sequence_len);
  });
  return zp::check_launch("zp_redundancy_softmax");
}
