// Paged decode attention: one query token per sequence over its paged K/V (GQA).
//
// HBM-bound: every step streams the whole KV budget once.  One block per (sequence, kv head,
// split); the G query heads of the group share every K/V load.  A key row (D elements) is read by
// D*sizeof(T)/16 adjacent lanes with one 16-byte load each, so a warp's load instruction covers
// whole 256/512-byte rows.  Each lane group walks 8 consecutive keys per iteration (all loads
// issued before use), keeps an online softmax per head and rescales its accumulators once per
// iteration.  Lane groups, then splits, are merged with the usual (max, sum, weighted out) rule.
#include "zp_common.cuh"

namespace zp {

constexpr int DEC_THREADS = 128;
constexpr int DEC_KPI = 8;  // keys per lane group per iteration

struct DecArgs {
  const void* q; const void* k; const void* v;
  const int32_t* seqlens; const int32_t* table;
  void* out; float* part;  // part: [B][Hkv][nsplit][GP][D+2] when nsplit > 1
  int B, NBmax, Hq, Hkv, BS, nsplit;
  int64_t kv_stride_page;
  float scale_log2e;
};

template <typename T> struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  static __device__ __forceinline__ void load(const T* p, float (&f)[N]) {
    const int4 raw = ld16(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int j = 0; j < N; ++j) f[j] = Elem<T>::to_f32(e[j]);
  }
};

// GP = group size padded to a power of two; heads g >= G are computed on zero queries and dropped.
template <typename T, int D, int GP>
__global__ void __launch_bounds__(DEC_THREADS) paged_decode_kernel(const DecArgs a) {
  constexpr int EPL = 16 / sizeof(T);        // elements per lane
  constexpr int LPK = D / EPL;               // lanes per key (16 for 16-bit, 32 for fp32 at D=128)
  constexpr int NGRP = DEC_THREADS / LPK;    // lane groups per block
  constexpr int TILE = NGRP * DEC_KPI;       // keys per block iteration
  extern __shared__ __align__(16) float smem[];  // [NGRP][GP][D+2]

  const int b = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
  const int G = a.Hq / a.Hkv;
  const int tid = threadIdx.x, grp = tid / LPK, gl = tid % LPK;
  const int n = a.seqlens[b];
  const int npages = (n + a.BS - 1) / a.BS;
  const int pages_per_split = (npages + a.nsplit - 1) / a.nsplit;
  const int k_begin = min(split * pages_per_split * a.BS, n);
  const int k_end = min((split + 1) * pages_per_split * a.BS, n);
  const int32_t* table = a.table + (int64_t)b * a.NBmax;
  const T* kc = reinterpret_cast<const T*>(a.k);
  const T* vc = reinterpret_cast<const T*>(a.v);

  float q[GP][EPL], o[GP][EPL], m[GP], l[GP];
#pragma unroll
  for (int g = 0; g < GP; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) { o[g][j] = 0.f; q[g][j] = 0.f; }
    if (g < G) {
      Vec16<T>::load(reinterpret_cast<const T*>(a.q) + ((int64_t)b * a.Hq + h * G + g) * D + gl * EPL, q[g]);
#pragma unroll
      for (int j = 0; j < EPL; ++j) q[g][j] *= a.scale_log2e;
    }
  }

  for (int base = k_begin; base < k_end; base += TILE) {
    const int k0 = base + grp * DEC_KPI;           // this group's 8 consecutive keys (same page)
    float kf[DEC_KPI][EPL], vf[DEC_KPI][EPL];
    const bool any = k0 < k_end;
    const int page = any ? table[k0 / a.BS] : 0;
#pragma unroll
    for (int t = 0; t < DEC_KPI; ++t) {
      const int key = min(k0 + t, k_end - 1);
      const int64_t off = (int64_t)page * a.kv_stride_page + ((int64_t)(key % a.BS) * a.Hkv + h) * D + gl * EPL;
      if (any) { Vec16<T>::load(kc + off, kf[t]); Vec16<T>::load(vc + off, vf[t]); }
    }
    // every lane of the warp takes part in the shuffles below, also lane groups that are past
    // the end of the range (their scores are masked and their update is skipped)
    float s[GP][DEC_KPI];
#pragma unroll
    for (int g = 0; g < GP; ++g)
#pragma unroll
      for (int t = 0; t < DEC_KPI; ++t) {
        float acc = 0.f;
        if (any) {
#pragma unroll
          for (int j = 0; j < EPL; ++j) acc = fmaf(q[g][j], kf[t][j], acc);
        }
        s[g][t] = acc;
      }
#pragma unroll
    for (int off = LPK / 2; off > 0; off >>= 1)
#pragma unroll
      for (int g = 0; g < GP; ++g)
#pragma unroll
        for (int t = 0; t < DEC_KPI; ++t) s[g][t] += __shfl_xor_sync(0xffffffffu, s[g][t], off);
    if (any) {
#pragma unroll
      for (int g = 0; g < GP; ++g) {
        float mx = m[g];
#pragma unroll
        for (int t = 0; t < DEC_KPI; ++t) {
          if (k0 + t >= k_end) s[g][t] = -INFINITY;
          mx = fmaxf(mx, s[g][t]);
        }
        // key k0 is in range, so mx is finite; m = -inf on the first tile gives corr = 0
        const float corr = exp2f(m[g] - mx);
        m[g] = mx;
        l[g] *= corr;
#pragma unroll
        for (int j = 0; j < EPL; ++j) o[g][j] *= corr;
#pragma unroll
        for (int t = 0; t < DEC_KPI; ++t) {
          const float p = exp2f(s[g][t] - mx);
          l[g] += p;
#pragma unroll
          for (int j = 0; j < EPL; ++j) o[g][j] = fmaf(p, vf[t][j], o[g][j]);
        }
      }
    }
  }

  // ---- merge the lane groups of the block ----
  float* mine = smem + (size_t)grp * GP * (D + 2);
#pragma unroll
  for (int g = 0; g < GP; ++g) {
#pragma unroll
    for (int j = 0; j < EPL; ++j) mine[g * (D + 2) + gl * EPL + j] = o[g][j];
    if (gl == 0) { mine[g * (D + 2) + D] = m[g]; mine[g * (D + 2) + D + 1] = l[g]; }
  }
  __syncthreads();
  for (int idx = tid; idx < G * D; idx += DEC_THREADS) {
    const int g = idx / D, d = idx % D;
    float M = -INFINITY;
    for (int r = 0; r < NGRP; ++r) M = fmaxf(M, smem[((size_t)r * GP + g) * (D + 2) + D]);
    float num = 0.f, den = 0.f;
    for (int r = 0; r < NGRP; ++r) {
      const float* rr = smem + ((size_t)r * GP + g) * (D + 2);
      const float w = rr[D] == -INFINITY ? 0.f : exp2f(rr[D] - M);
      num = fmaf(w, rr[d], num);
      den = fmaf(w, rr[D + 1], den);
    }
    if (a.nsplit == 1) {
      reinterpret_cast<T*>(a.out)[((int64_t)b * a.Hq + h * G + g) * D + d] =
          Elem<T>::from_f32(den > 0.f ? num / den : 0.f);
    } else {
      float* pp = a.part + ((((int64_t)b * a.Hkv + h) * a.nsplit + split) * GP + g) * (D + 2);
      pp[d] = num;
      if (d == 0) { pp[D] = M; pp[D + 1] = den; }
    }
  }
}

template <typename T, int D, int GP>
__global__ void decode_merge_kernel(const DecArgs a) {
  const int b = blockIdx.x, h = blockIdx.y;
  const int G = a.Hq / a.Hkv;
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    const float* base = a.part + (((int64_t)b * a.Hkv + h) * a.nsplit * GP + g) * (D + 2);
    const int64_t sstride = (int64_t)GP * (D + 2);
    float M = -INFINITY;
    for (int s = 0; s < a.nsplit; ++s) M = fmaxf(M, base[s * sstride + D]);
    float num = 0.f, den = 0.f;
    for (int s = 0; s < a.nsplit; ++s) {
      const float* rr = base + s * sstride;
      const float w = rr[D] == -INFINITY ? 0.f : exp2f(rr[D] - M);
      num = fmaf(w, rr[d], num);
      den = fmaf(w, rr[D + 1], den);
    }
    reinterpret_cast<T*>(a.out)[((int64_t)b * a.Hq + h * G + g) * D + d] =
        Elem<T>::from_f32(den > 0.f ? num / den : 0.f);
  }
}

static int pick_splits(int B, int Hkv, int NBmax) {
  const int target = 148 * 4;
  int s = (target + B * Hkv - 1) / (B * Hkv);
  if (s > NBmax) s = NBmax;
  if (s > 32) s = 32;
  return s < 1 ? 1 : s;
}

template <typename T, int D, int GP>
static int launch_decode(DecArgs a, cudaStream_t st) {
  constexpr int LPK = D / (16 / sizeof(T));
  constexpr int NGRP = DEC_THREADS / LPK;
  const size_t smem = sizeof(float) * NGRP * GP * (D + 2);
  auto kern = paged_decode_kernel<T, D, GP>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  kern<<<dim3(a.B, a.Hkv, a.nsplit), DEC_THREADS, smem, st>>>(a);
  int rc = check_launch("zp_paged_decode");
  if (rc || a.nsplit == 1) return rc;
  decode_merge_kernel<T, D, GP><<<dim3(a.B, a.Hkv), 128, 0, st>>>(a);
  return check_launch("zp_paged_decode merge");
}

template <typename T>
static int dispatch_decode(const DecArgs& a, int D, int G, cudaStream_t st) {
  if (D != 128) { set_error("zp_paged_decode: head_dim %d not supported (128)", D); return ZP_ERR_UNSUPPORTED; }
  if (G == 1) return launch_decode<T, 128, 1>(a, st);
  if (G == 2) return launch_decode<T, 128, 2>(a, st);
  if (G <= 4) return launch_decode<T, 128, 4>(a, st);
  if (G <= 8) return launch_decode<T, 128, 8>(a, st);
  set_error("zp_paged_decode: group size %d not supported (<= 8)", G);
  return ZP_ERR_UNSUPPORTED;
}

static int gp_of(int G) { return G == 1 ? 1 : G == 2 ? 2 : G <= 4 ? 4 : G <= 8 ? 8 : 16; }

// tensor-core path for 16-bit caches (zp_decode_mma.cu)
int paged_decode_mma(const void* q, const void* k, const void* v, const int32_t* seqlens,
                     const int32_t* table, void* out, float* part, int B, int NBmax, int Hq, int Hkv,
                     int BS, int nsplit, int gp, int64_t kv_stride_page, float scale_log2e, int dtype,
                     cudaStream_t st);

}  // namespace zp

extern "C" size_t zp_paged_decode_workspace_bytes(int B, int Hq, int D, int max_splits) {
  // upper bound: every (seq, q head) padded to 8 heads per group never exceeds 2x
  return (size_t)B * Hq * 2 * (size_t)(max_splits < 1 ? 1 : max_splits) * (D + 2) * sizeof(float) + 256;
}

extern "C" int zp_paged_decode(const void* q, const void* k_cache, const void* v_cache,
                               const int32_t* cache_seqlens, const int32_t* block_table, void* out,
                               int B, int NBmax, int Hq, int Hkv, int D, int BS,
                               int64_t kv_stride_page, float softmax_scale, int dtype,
                               void* workspace, size_t workspace_bytes, void* stream) {
  if (B == 0) return ZP_OK;
  ZP_REQUIRE(q && k_cache && v_cache && cache_seqlens && block_table && out, "zp_paged_decode: null pointer");
  ZP_REQUIRE(Hkv > 0 && Hq % Hkv == 0, "zp_paged_decode: Hq must be a multiple of Hkv");
  ZP_REQUIRE(BS % zp::DEC_KPI == 0, "zp_paged_decode: page size must be a multiple of 8");
  ZP_REQUIRE(((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) % 16 == 0,
             "zp_paged_decode: pointers must be 16-byte aligned");
  const int G = Hq / Hkv;
  zp::DecArgs a;
  a.q = q; a.k = k_cache; a.v = v_cache; a.seqlens = cache_seqlens; a.table = block_table; a.out = out;
  a.B = B; a.NBmax = NBmax; a.Hq = Hq; a.Hkv = Hkv; a.BS = BS;
  a.kv_stride_page = kv_stride_page;
  a.scale_log2e = softmax_scale * 1.4426950408889634f;
  a.nsplit = zp::pick_splits(B, Hkv, NBmax);
  a.part = nullptr;
  if (a.nsplit > 1) {
    const size_t need = (size_t)B * Hkv * a.nsplit * zp::gp_of(G) * (D + 2) * sizeof(float);
    if (!workspace || workspace_bytes < need) {
      // no scratch: run unsplit (correct, but one block per (sequence, kv head) leaves a small
      // batch on a few SMs); the call succeeds and the message says what happened
      zp::set_error("zp_paged_decode: workspace of %zu bytes, %zu needed for %d splits: running unsplit",
                    workspace_bytes, need, a.nsplit);
      a.nsplit = 1;
    }
    else a.part = reinterpret_cast<float*>(workspace);
  }
  cudaStream_t st = (cudaStream_t)stream;
  const bool mma = (dtype == ZP_DTYPE_BF16 || dtype == ZP_DTYPE_F16) && D == 128 && BS % 64 == 0 && G <= 16;
  if (mma)
    return zp::paged_decode_mma(q, k_cache, v_cache, cache_seqlens, block_table, out, a.part, B, NBmax,
                                Hq, Hkv, BS, a.nsplit, zp::gp_of(G), kv_stride_page, a.scale_log2e, dtype,
                                st);
  ZP_DISPATCH_DTYPE(dtype, T, { return zp::dispatch_decode<T>(a, D, G, st); });
  return ZP_OK;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of zp_paged_decode.
//
// Some hosts of this library must not allocate device memory at the moment they decode: a serving
// loop whose memory pool is fully handed out to the KV cache (the engine sizes the cache from all
// free memory at start-up), a real-time thread where cudaMalloc's implicit device synchronisation
// is unacceptable, or a caller running while a CUDA graph is being captured on another stream.
// For them the split-KV partial results live in the fixed device array below instead of in a
// caller-provided workspace.
namespace zp {
constexpr size_t DEC_STATIC_SCRATCH_BYTES = 4u << 20;  // 4 MiB per GPU that loads the library
static __device__ __align__(256) unsigned char g_decode_scratch[DEC_STATIC_SCRATCH_BYTES];

constexpr int DEC_MAX_DEVICES = 64;
static void* g_decode_scratch_ptr[DEC_MAX_DEVICES];  // device address of the array, per device
}  // namespace zp

extern "C" size_t zp_paged_decode_noalloc_max_scratch_bytes(void) { return zp::DEC_STATIC_SCRATCH_BYTES; }

extern "C" int zp_paged_decode_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                       const int32_t* cache_seqlens, const int32_t* block_table,
                                       void* out, int B, int NBmax, int Hq, int Hkv, int D, int BS,
                                       int64_t kv_stride_page, float softmax_scale, int dtype,
                                       void* stream) {
  if (B == 0) return ZP_OK;
  ZP_REQUIRE(Hkv > 0 && Hq % Hkv == 0, "zp_paged_decode_noalloc: Hq must be a multiple of Hkv");
  // the same split choice as zp_paged_decode makes when given scratch
  const int nsplit = zp::pick_splits(B, Hkv, NBmax);
  const size_t need = nsplit > 1
      ? (size_t)B * Hkv * nsplit * zp::gp_of(Hq / Hkv) * (D + 2) * sizeof(float) : 0;
  if (need > zp::DEC_STATIC_SCRATCH_BYTES) {
    zp::set_error("zp_paged_decode_noalloc: this batch needs %zu bytes of split scratch, the built-in "
                  "array holds %zu; use zp_paged_decode with a caller workspace",
                  need, zp::DEC_STATIC_SCRATCH_BYTES);
    return ZP_ERR_WORKSPACE;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= zp::DEC_MAX_DEVICES) {
    zp::set_error("zp_paged_decode_noalloc: cannot identify the current device");
    return ZP_ERR_CUDA;
  }
  // Set-up, once per device, with that device current: the array's name is a host-side handle,
  // the address a kernel can use has to be asked for.
  void* scratch = __atomic_load_n(&zp::g_decode_scratch_ptr[dev], __ATOMIC_ACQUIRE);
  if (!scratch) {
    e = cudaGetSymbolAddress(&scratch, zp::g_decode_scratch);
    if (e != cudaSuccess || !scratch) {
      zp::set_error("zp_paged_decode_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return ZP_ERR_CUDA;
    }
    __atomic_store_n(&zp::g_decode_scratch_ptr[dev], scratch, __ATOMIC_RELEASE);
  }
  return zp_paged_decode(q, k_cache, v_cache, cache_seqlens, block_table, out, B, NBmax, Hq, Hkv, D,
                         BS, kv_stride_page, softmax_scale, dtype, scratch,
                         zp::DEC_STATIC_SCRATCH_BYTES, stream);
}
