// Variable-length causal prefill attention (bottom-right aligned) for 16-bit tensors, head_dim
// 128, K/V dense or paged: flash-attention style tiling on warp-level tensor-core MMAs.
//
// One block per (64-query tile, query head, sequence): 4 warps x 16 query rows.  The queries' A
// fragments stay in registers; 64-key tiles of K and V stream through two cp.async stages of
// XOR-swizzled shared memory.  Per tile and warp: S = Q K^T (64 MMAs m16n8k16), causal mask,
// online softmax in fp32, O += P V (64 MMAs, P rounded to the tensor dtype, V via ldmatrix.trans).
#include "zp_mma.cuh"

namespace zp {

constexpr int PM_THREADS = 128;
constexpr int PM_TQ = 64, PM_TK = 64;
constexpr int PM_TILE_BYTES = PM_TK * MMA_ROW_BYTES;

struct PmArgs {
  const void* q; const void* k; const void* v;
  const int32_t* cu_q; const int32_t* cu_k; const int32_t* table;
  void* out;
  int B, NBmax, Hq, Hkv, BS;
  int64_t kv_stride_page;
  float scale_log2e;
};

template <typename T>
__global__ void __launch_bounds__(PM_THREADS) varlen_prefill_mma_kernel(const PmArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];  // [2 stages][K tile | V tile]
  const int b = blockIdx.z, h = blockIdx.y, qt = blockIdx.x;
  const int q0 = a.cu_q[b], lq = a.cu_q[b + 1] - q0;
  const int k0 = a.cu_k[b], lk = a.cu_k[b + 1] - k0;
  const int qi0 = qt * PM_TQ;
  if (qi0 >= lq) return;
  const int G = a.Hq / a.Hkv, hk = h / G;
  const int shift = lk - lq;  // query i sees keys j <= i + shift
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int row0 = qi0 + warp * 16 + g, row1 = row0 + 8;  // this thread's two query rows
  const char* kc = reinterpret_cast<const char*>(a.k);
  const char* vc = reinterpret_cast<const char*>(a.v);
  const int64_t kv_row_stride = (int64_t)a.Hkv * 128 * sizeof(T);

  // ---- A fragments of this warp's 16 query rows ----
  uint32_t qa[8][4];
  {
    const T* qb = reinterpret_cast<const T*>(a.q) + ((int64_t)q0 * a.Hq + h) * 128;
    const int64_t qs = (int64_t)a.Hq * 128;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int d0 = ks * 16 + tq * 2;
      qa[ks][0] = row0 < lq ? *reinterpret_cast<const uint32_t*>(qb + row0 * qs + d0) : 0u;
      qa[ks][1] = row1 < lq ? *reinterpret_cast<const uint32_t*>(qb + row1 * qs + d0) : 0u;
      qa[ks][2] = row0 < lq ? *reinterpret_cast<const uint32_t*>(qb + row0 * qs + d0 + 8) : 0u;
      qa[ks][3] = row1 < lq ? *reinterpret_cast<const uint32_t*>(qb + row1 * qs + d0 + 8) : 0u;
    }
  }

  const int rows = min(PM_TQ, lq - qi0);
  const int kmax = min(lk, qi0 + rows + shift);  // keys any row of the tile can see
  const int ntiles = kmax > 0 ? (kmax + PM_TK - 1) / PM_TK : 0;

  auto load_tile = [&](int t, int stage) {
    const int key0 = t * PM_TK;
    int64_t base;
    if (a.table) {  // a 64-key tile never straddles a page (page size is a multiple of 64)
      const int page = a.table[(int64_t)b * a.NBmax + key0 / a.BS];
      base = ((int64_t)page * a.kv_stride_page + ((int64_t)(key0 % a.BS) * a.Hkv + hk) * 128) * (int64_t)sizeof(T);
    } else {
      base = ((int64_t)(k0 + key0) * a.Hkv + hk) * 128 * (int64_t)sizeof(T);
    }
    unsigned char* ks = smem + stage * 2 * PM_TILE_BYTES;
    unsigned char* vs = ks + PM_TILE_BYTES;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = tid + i * PM_THREADS;
      const int r = idx >> 4, c = idx & 15;
      const int ok = key0 + r < lk ? 16 : 0;  // rows past the sequence are zero-filled
      const int64_t off = base + (ok ? r : 0) * kv_row_stride + c * 16;
      cp_async16(ks + swz(r, c), kc + off, ok);
      cp_async16(vs + swz(r, c), vc + off, ok);
    }
  };

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  if (ntiles > 0) load_tile(0, 0);
  cp_async_commit();
  for (int t = 0; t < ntiles; ++t) {
    if (t + 1 < ntiles) load_tile(t + 1, (t + 1) & 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const unsigned char* ks = smem + (t & 1) * 2 * PM_TILE_BYTES;
    const unsigned char* vs = ks + PM_TILE_BYTES;
    const int key0 = t * PM_TK;
    // a warp whose rows all precede this tile's first visible key has nothing to do in it
    const bool warp_active = key0 <= qi0 + warp * 16 + 15 + shift;
    if (warp_active) {
      float s[8][4];
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
#pragma unroll
      for (int kp = 0; kp < 4; ++kp) {
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
          uint32_t bf[4];
          ldmatrix_x4(bf, ks + swz(nb * 8 + (lane & 7), kp * 4 + (lane >> 3)));
          mma16816<T>(s[nb], qa[2 * kp], bf[0], bf[1]);
          mma16816<T>(s[nb], qa[2 * kp + 1], bf[2], bf[3]);
        }
      }
      // causal + length mask, scale, row maxima
      float mx0 = m0, mx1 = m1;
      const int lim0 = min(lk - 1, row0 + shift), lim1 = min(lk - 1, row1 + shift);
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) {
        const int key = key0 + nb * 8 + 2 * tq;
        s[nb][0] = key <= lim0 ? s[nb][0] * a.scale_log2e : -INFINITY;
        s[nb][1] = key + 1 <= lim0 ? s[nb][1] * a.scale_log2e : -INFINITY;
        s[nb][2] = key <= lim1 ? s[nb][2] * a.scale_log2e : -INFINITY;
        s[nb][3] = key + 1 <= lim1 ? s[nb][3] * a.scale_log2e : -INFINITY;
        mx0 = fmaxf(mx0, fmaxf(s[nb][0], s[nb][1]));
        mx1 = fmaxf(mx1, fmaxf(s[nb][2], s[nb][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float c0 = mx0 == -INFINITY ? 1.f : exp2f(m0 - mx0);
      const float c1 = mx1 == -INFINITY ? 1.f : exp2f(m1 - mx1);
      const float e0 = mx0 == -INFINITY ? 0.f : mx0, e1 = mx1 == -INFINITY ? 0.f : mx1;
      m0 = mx0; m1 = mx1;
      float ps0 = 0.f, ps1 = 0.f;
      uint32_t pa[4][4];  // A fragments of P for the four 16-key steps
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const float p00 = exp2f(s[2 * kk][0] - e0), p01 = exp2f(s[2 * kk][1] - e0);
        const float p02 = exp2f(s[2 * kk][2] - e1), p03 = exp2f(s[2 * kk][3] - e1);
        const float p10 = exp2f(s[2 * kk + 1][0] - e0), p11 = exp2f(s[2 * kk + 1][1] - e0);
        const float p12 = exp2f(s[2 * kk + 1][2] - e1), p13 = exp2f(s[2 * kk + 1][3] - e1);
        ps0 += (p00 + p01) + (p10 + p11);
        ps1 += (p02 + p03) + (p12 + p13);
        pa[kk][0] = pack2<T>(p00, p01); pa[kk][1] = pack2<T>(p02, p03);
        pa[kk][2] = pack2<T>(p10, p11); pa[kk][3] = pack2<T>(p12, p13);
      }
      l0 = l0 * c0 + ps0;
      l1 = l1 * c1 + ps1;
#pragma unroll
      for (int i = 0; i < 16; ++i) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
        for (int np = 0; np < 8; ++np) {
          uint32_t bf[4];
          const int row = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          ldmatrix_x4_trans(bf, vs + swz(row, np * 2 + (lane >> 4)));
          mma16816<T>(o[2 * np], pa[kk], bf[0], bf[1]);
          mma16816<T>(o[2 * np + 1], pa[kk], bf[2], bf[3]);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
  T* ob = reinterpret_cast<T*>(a.out) + ((int64_t)q0 * a.Hq + h) * 128;
  const int64_t os = (int64_t)a.Hq * 128;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int d = i * 8 + 2 * tq;
    if (row0 < lq) *reinterpret_cast<uint32_t*>(ob + row0 * os + d) = pack2<T>(o[i][0] * i0, o[i][1] * i0);
    if (row1 < lq) *reinterpret_cast<uint32_t*>(ob + row1 * os + d) = pack2<T>(o[i][2] * i1, o[i][3] * i1);
  }
}

template <typename T>
static int launch_prefill_mma(const PmArgs& a, int max_seqlen_q, cudaStream_t st) {
  const size_t smem = 2 * 2 * PM_TILE_BYTES;
  auto kern = varlen_prefill_mma_kernel<T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_error("zp_varlen_prefill: %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  dim3 grid((max_seqlen_q + PM_TQ - 1) / PM_TQ, a.Hq, a.B);
  kern<<<grid, PM_THREADS, smem, st>>>(a);
  return check_launch("zp_varlen_prefill(mma)");
}

// Called by zp_varlen_prefill for 16-bit tensors with head_dim 128.
int varlen_prefill_mma(const void* q, const void* k, const void* v, const int32_t* cu_q, const int32_t* cu_k,
                       const int32_t* table, void* out, int B, int max_seqlen_q, int NBmax, int Hq,
                       int Hkv, int BS, int64_t kv_stride_page, float scale_log2e, int dtype,
                       cudaStream_t st) {
  PmArgs a;
  a.q = q; a.k = k; a.v = v; a.cu_q = cu_q; a.cu_k = cu_k; a.table = table; a.out = out;
  a.B = B; a.NBmax = NBmax; a.Hq = Hq; a.Hkv = Hkv; a.BS = BS; a.kv_stride_page = kv_stride_page;
  a.scale_log2e = scale_log2e;
  if (dtype == ZP_DTYPE_BF16) return launch_prefill_mma<__nv_bfloat16>(a, max_seqlen_q, st);
  return launch_prefill_mma<__half>(a, max_seqlen_q, st);
}

}  // namespace zp
