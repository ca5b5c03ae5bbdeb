// Variable-length causal prefill attention (bottom-right aligned), K/V dense or paged.
//
// Portable SIMT kernel with fp32 maths: one block per (64-query tile, query head, sequence);
// 64-key tiles of K and V stream through shared memory with an online softmax.
#include "zp_common.cuh"

namespace zp {

constexpr int PF_THREADS = 256;
constexpr int PF_TQ = 64, PF_TK = 64;

struct PfArgs {
  const void* q; const void* k; const void* v;
  const int32_t* cu_q; const int32_t* cu_k; const int32_t* table;
  void* out;
  int B, NBmax, Hq, Hkv, BS;
  int64_t kv_stride_page;
  float scale_log2e;
};

template <typename T, int D>
__device__ __forceinline__ void load_rows_f32(const T* __restrict__ base, int64_t row_stride, int nrows,
                                              int valid_rows, float* __restrict__ dst) {
  constexpr int LD = D + 4, EPV = 16 / sizeof(T), VPR = D / EPV;
  for (int v = threadIdx.x; v < nrows * VPR; v += PF_THREADS) {
    const int r = v / VPR, c = v % VPR;
    float* d = dst + r * LD + c * EPV;
    if (r < valid_rows) {
      const int4 raw = ld16(base + (int64_t)r * row_stride + c * EPV);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < EPV; ++j) d[j] = Elem<T>::to_f32(e[j]);
    } else {
#pragma unroll
      for (int j = 0; j < EPV; ++j) d[j] = 0.f;
    }
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(PF_THREADS, 1) varlen_prefill_kernel(const PfArgs a) {
  constexpr int LD = D + 4;
  constexpr int DPT = D / 16;  // output dims per thread
  extern __shared__ __align__(16) float smem[];
  float* sQ = smem;
  float* sK = sQ + PF_TQ * LD;
  float* sV = sK + PF_TK * LD;
  float* sP = sV + PF_TK * LD;  // [64][65]

  const int b = blockIdx.z, h = blockIdx.y, qt = blockIdx.x;
  const int q0 = a.cu_q[b], lq = a.cu_q[b + 1] - q0;
  const int k0 = a.cu_k[b], lk = a.cu_k[b + 1] - k0;
  const int qi0 = qt * PF_TQ;
  if (qi0 >= lq) return;
  const int G = a.Hq / a.Hkv, hk = h / G;
  const int rows = min(PF_TQ, lq - qi0);
  const int shift = lk - lq;  // query i sees keys j <= i + shift
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const T* qp = reinterpret_cast<const T*>(a.q) + ((int64_t)(q0 + qi0) * a.Hq + h) * D;
  load_rows_f32<T, D>(qp, (int64_t)a.Hq * D, PF_TQ, rows, sQ);

  float o[4][DPT], m[4], l[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    m[r] = -INFINITY; l[r] = 0.f;
#pragma unroll
    for (int j = 0; j < DPT; ++j) o[r][j] = 0.f;
  }
  const int kmax = min(lk, qi0 + rows + shift);  // keys any row of the tile can see
  for (int kj0 = 0; kj0 < kmax; kj0 += PF_TK) {
    const int kvalid = min(PF_TK, kmax - kj0);
    __syncthreads();
    if (a.table) {
      // a 64-key tile never straddles a page (BS is a multiple of 64)
      const int page = a.table[(int64_t)b * a.NBmax + kj0 / a.BS];
      const int64_t off = (int64_t)page * a.kv_stride_page + ((int64_t)(kj0 % a.BS) * a.Hkv + hk) * D;
      load_rows_f32<T, D>(reinterpret_cast<const T*>(a.k) + off, (int64_t)a.Hkv * D, PF_TK, kvalid, sK);
      load_rows_f32<T, D>(reinterpret_cast<const T*>(a.v) + off, (int64_t)a.Hkv * D, PF_TK, kvalid, sV);
    } else {
      const int64_t off = ((int64_t)(k0 + kj0) * a.Hkv + hk) * D;
      load_rows_f32<T, D>(reinterpret_cast<const T*>(a.k) + off, (int64_t)a.Hkv * D, PF_TK, kvalid, sK);
      load_rows_f32<T, D>(reinterpret_cast<const T*>(a.v) + off, (int64_t)a.Hkv * D, PF_TK, kvalid, sV);
    }
    __syncthreads();
    float s[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[r][c] = 0.f;
#pragma unroll 4
    for (int d = 0; d < D; d += 4) {
      float4 kv[4], qv[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) kv[c] = *reinterpret_cast<const float4*>(sK + (tx + 16 * c) * LD + d);
#pragma unroll
      for (int r = 0; r < 4; ++r) qv[r] = *reinterpret_cast<const float4*>(sQ + (ty * 4 + r) * LD + d);
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          s[r][c] = fmaf(qv[r].x, kv[c].x, s[r][c]);
          s[r][c] = fmaf(qv[r].y, kv[c].y, s[r][c]);
          s[r][c] = fmaf(qv[r].z, kv[c].z, s[r][c]);
          s[r][c] = fmaf(qv[r].w, kv[c].w, s[r][c]);
        }
    }
    float corr[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int qi = qi0 + ty * 4 + r;
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int kj = kj0 + tx + 16 * c;
        s[r][c] = (kj < lk && kj <= qi + shift) ? s[r][c] * a.scale_log2e : -INFINITY;
        mx = fmaxf(mx, s[r][c]);
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float mnew = fmaxf(m[r], mx);
      corr[r] = mnew == -INFINITY ? 1.f : exp2f(m[r] - mnew);
      float ps = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float p = mnew == -INFINITY ? 0.f : exp2f(s[r][c] - mnew);
        sP[(ty * 4 + r) * (PF_TK + 1) + tx + 16 * c] = p;
        ps += p;
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
      l[r] = l[r] * corr[r] + ps;
      m[r] = mnew;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int j = 0; j < DPT; ++j) o[r][j] *= corr[r];
    for (int n = 0; n < PF_TK; ++n) {
      float vv[DPT];
#pragma unroll
      for (int j = 0; j < DPT; j += 4)
        *reinterpret_cast<float4*>(&vv[j]) = *reinterpret_cast<const float4*>(sV + n * LD + tx * DPT + j);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float p = sP[(ty * 4 + r) * (PF_TK + 1) + n];
#pragma unroll
        for (int j = 0; j < DPT; ++j) o[r][j] = fmaf(p, vv[j], o[r][j]);
      }
    }
  }
  T* op = reinterpret_cast<T*>(a.out) + ((int64_t)(q0 + qi0) * a.Hq + h) * D;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int row = ty * 4 + r;
    if (row >= rows) continue;
    const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
#pragma unroll
    for (int j = 0; j < DPT; ++j)
      op[(int64_t)row * a.Hq * D + tx * DPT + j] = Elem<T>::from_f32(o[r][j] * inv);
  }
}

template <typename T, int D>
static int launch_prefill(const PfArgs& a, int max_seqlen_q, cudaStream_t st) {
  constexpr int LD = D + 4;
  const size_t smem = sizeof(float) * ((PF_TQ + 2 * PF_TK) * LD + PF_TQ * (PF_TK + 1));
  auto kern = varlen_prefill_kernel<T, D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_error("zp_varlen_prefill: %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  dim3 grid((max_seqlen_q + PF_TQ - 1) / PF_TQ, a.Hq, a.B);
  kern<<<grid, PF_THREADS, smem, st>>>(a);
  return check_launch("zp_varlen_prefill");
}

// tensor-core path for 16-bit tensors (zp_prefill_mma.cu)
int varlen_prefill_mma(const void* q, const void* k, const void* v, const int32_t* cu_q, const int32_t* cu_k,
                       const int32_t* table, void* out, int B, int max_seqlen_q, int NBmax, int Hq,
                       int Hkv, int BS, int64_t kv_stride_page, float scale_log2e, int dtype,
                       cudaStream_t st);

// tcgen05 path (zp_prefill_tc.cu)
int varlen_prefill_tc(const void* q, const void* k, const void* v, const int32_t* cu_q, const int32_t* cu_k,
                      const int32_t* table, void* out, int B, int max_seqlen_q, int NBmax, int Hq, int Hkv,
                      int BS, int64_t kv_stride_page, float scale_log2e, int total_q, int total_k, int dtype,
                      cudaStream_t st);

}  // namespace zp

extern "C" int zp_varlen_prefill_ex(const void* q, const void* k, const void* v,
                                    const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                    const int32_t* block_table, void* out, int B, int max_seqlen_q,
                                    int NBmax, int Hq, int Hkv, int D, int BS, int64_t kv_stride_page,
                                    float softmax_scale, int total_q, int total_k, int impl, int dtype,
                                    void* stream) {
  const bool can = (dtype == ZP_DTYPE_BF16 || dtype == ZP_DTYPE_F16) && D == 128 && Hkv > 0 &&
                   Hq % Hkv == 0 && total_q > 0 && (block_table ? BS % 128 == 0 : total_k > 0) &&
                   ((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) % 16 == 0 &&
                   (!block_table || (kv_stride_page * 2) % 16 == 0);
  if (impl == ZP_IMPL_TCGEN05 && !can) {
    zp::set_error("zp_varlen_prefill_ex: the tcgen05 kernel needs 16-bit tensors, head_dim 128, "
                  "16-byte aligned pointers, row counts, and pages of a multiple of 128 keys");
    return ZP_ERR_UNSUPPORTED;
  }
  if (impl == ZP_IMPL_SIMT || !can)
    return zp_varlen_prefill(q, k, v, cu_seqlens_q, cu_seqlens_k, block_table, out, B, max_seqlen_q, NBmax,
                             Hq, Hkv, D, BS, kv_stride_page, softmax_scale, dtype, stream);
  if (B == 0 || max_seqlen_q == 0) return ZP_OK;
  ZP_REQUIRE(q && k && v && cu_seqlens_q && cu_seqlens_k && out, "zp_varlen_prefill_ex: null pointer");
  return zp::varlen_prefill_tc(q, k, v, cu_seqlens_q, cu_seqlens_k, block_table, out, B, max_seqlen_q, NBmax,
                               Hq, Hkv, BS, kv_stride_page, softmax_scale * 1.4426950408889634f, total_q,
                               total_k, dtype, (cudaStream_t)stream);
}

extern "C" int zp_varlen_prefill(const void* q, const void* k, const void* v,
                                 const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                 const int32_t* block_table, void* out, int B, int max_seqlen_q,
                                 int NBmax, int Hq, int Hkv, int D, int BS, int64_t kv_stride_page,
                                 float softmax_scale, int dtype, void* stream) {
  if (B == 0 || max_seqlen_q == 0) return ZP_OK;
  ZP_REQUIRE(q && k && v && cu_seqlens_q && cu_seqlens_k && out, "zp_varlen_prefill: null pointer");
  ZP_REQUIRE(Hkv > 0 && Hq % Hkv == 0, "zp_varlen_prefill: Hq must be a multiple of Hkv");
  ZP_REQUIRE(!block_table || BS % zp::PF_TK == 0, "zp_varlen_prefill: page size must be a multiple of 64");
  ZP_REQUIRE(D == 128 || D == 64, "zp_varlen_prefill: head_dim %d not supported (64 or 128)", D);
  zp::PfArgs a;
  a.q = q; a.k = k; a.v = v; a.cu_q = cu_seqlens_q; a.cu_k = cu_seqlens_k; a.table = block_table;
  a.out = out; a.B = B; a.NBmax = NBmax; a.Hq = Hq; a.Hkv = Hkv; a.BS = BS;
  a.kv_stride_page = kv_stride_page;
  a.scale_log2e = softmax_scale * 1.4426950408889634f;
  cudaStream_t st = (cudaStream_t)stream;
  if ((dtype == ZP_DTYPE_BF16 || dtype == ZP_DTYPE_F16) && D == 128 &&
      ((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) % 16 == 0)
    return zp::varlen_prefill_mma(q, k, v, cu_seqlens_q, cu_seqlens_k, block_table, out, B, max_seqlen_q,
                                  NBmax, Hq, Hkv, BS, kv_stride_page, a.scale_log2e, dtype, st);
  ZP_DISPATCH_DTYPE(dtype, T, {
    if (D == 128) return zp::launch_prefill<T, 128>(a, max_seqlen_q, st);
    return zp::launch_prefill<T, 64>(a, max_seqlen_q, st);
  });
  return ZP_OK;
}
