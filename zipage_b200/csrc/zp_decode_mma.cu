// Paged decode attention for 16-bit caches (head_dim 128): HBM-bound streaming of K/V pages with
// the dot products on warp-level tensor-core MMAs (mma.sync m16n8k16, fp32 accumulate).
//
// Decode is bound by the K/V stream (one query per sequence; the G query heads of a KV group reuse
// every loaded row), so the arithmetic only has to stay out of the way: the group's queries form
// the 16-row A operand (rows >= G are zero), 64-key tiles of K and V are brought into shared memory
// with 16-byte cp.async copies (two stages, XOR-swizzled 16-byte chunks so that ldmatrix is
// conflict-free), each of the four warps takes 16 keys of a tile: S = Q K^T (16 MMAs), online
// softmax in registers, O += P V (16 MMAs, V through ldmatrix.trans).  Warps, then key splits, are
// merged with the (max, sum, weighted output) rule.  One block per (sequence, kv head, split).
#include "zp_mma.cuh"

namespace zp {

constexpr int DM_THREADS = 128;
constexpr int DM_TILE = 64;                // keys per tile
constexpr int DM_TILE_BYTES = DM_TILE * MMA_ROW_BYTES;  // 16 KB per K or V tile

struct DmArgs {
  const void* q; const void* k; const void* v;
  const int32_t* seqlens; const int32_t* table;
  void* out; float* part;  // part: [B][Hkv][nsplit][gp][130] when nsplit > 1 (gp = padded group size)
  int B, NBmax, Hq, Hkv, BS, nsplit, gp;
  int64_t kv_stride_page;
  float scale_log2e;
};

template <typename T>
__global__ void __launch_bounds__(DM_THREADS) paged_decode_mma_kernel(const DmArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];  // [2 stages][K tile | V tile]
  const int b = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
  const int G = a.Hq / a.Hkv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;  // fragment row / column-pair index
  const int n = a.seqlens[b];
  const int npages = (n + a.BS - 1) / a.BS;
  const int pages_per_split = (npages + a.nsplit - 1) / a.nsplit;
  const int k_begin = min(split * pages_per_split * a.BS, n);
  const int k_end = min((split + 1) * pages_per_split * a.BS, n);
  const int32_t* table = a.table + (int64_t)b * a.NBmax;
  const char* kc = reinterpret_cast<const char*>(a.k);
  const char* vc = reinterpret_cast<const char*>(a.v);
  const int ntiles = (k_end - k_begin + DM_TILE - 1) / DM_TILE;

  // ---- A fragments of the queries: row g of the group (rows >= G and rows 8..15 are zero) ----
  uint32_t qa[8][4];
  {
    const T* qrow = reinterpret_cast<const T*>(a.q) + ((int64_t)b * a.Hq + h * G + g) * 128;
    const T* qrow8 = qrow + 8 * 128;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int d0 = ks * 16 + tq * 2;
      qa[ks][0] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + d0) : 0u;
      qa[ks][2] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + d0 + 8) : 0u;
      qa[ks][1] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qrow8 + d0) : 0u;
      qa[ks][3] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qrow8 + d0 + 8) : 0u;
    }
  }

  auto load_tile = [&](int t, int stage) {
    const int key0 = k_begin + t * DM_TILE;  // multiple of 64: a tile never straddles a page
    const int page = table[key0 / a.BS];
    const int64_t base = ((int64_t)page * a.kv_stride_page + ((int64_t)(key0 % a.BS) * a.Hkv + h) * 128) * (int64_t)sizeof(T);
    unsigned char* ks = smem + stage * 2 * DM_TILE_BYTES;
    unsigned char* vs = ks + DM_TILE_BYTES;
    const int64_t row_stride = (int64_t)a.Hkv * 128 * sizeof(T);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = tid + i * DM_THREADS;  // 1024 chunks of 16 bytes per tensor
      const int r = idx >> 4, c = idx & 15;
      const int ok = key0 + r < k_end ? 16 : 0;  // rows past the end are zero-filled
      const int64_t off = base + (ok ? r : 0) * row_stride + c * 16;
      cp_async16(ks + swz(r, c), kc + off, ok);
      cp_async16(vs + swz(r, c), vc + off, ok);
    }
  };

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // rows g and g + 8

  if (ntiles > 0) load_tile(0, 0);
  cp_async_commit();
  for (int t = 0; t < ntiles; ++t) {
    if (t + 1 < ntiles) load_tile(t + 1, (t + 1) & 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const unsigned char* ks = smem + (t & 1) * 2 * DM_TILE_BYTES;
    const unsigned char* vs = ks + DM_TILE_BYTES;
    const int kw = warp * 16;  // this warp's 16 keys of the tile

    // ---- S = Q K^T for 16 keys (two 8-key column blocks) ----
    float s[2][4];
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
#pragma unroll
    for (int kp = 0; kp < 4; ++kp) {  // 32 dims per step: two k-slices
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        uint32_t bf[4];
        const int row = kw + nb * 8 + (lane & 7);
        ldmatrix_x4(bf, ks + swz(row, kp * 4 + (lane >> 3)));
        mma16816<T>(s[nb], qa[2 * kp], bf[0], bf[1]);
        mma16816<T>(s[nb], qa[2 * kp + 1], bf[2], bf[3]);
      }
    }
    // ---- online softmax (rows g, g + 8; this thread's keys: kw + nb*8 + 2*tq, +1) ----
    const int key_base = k_begin + t * DM_TILE + kw;
    float mx0 = m0, mx1 = m1;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      const int key = key_base + nb * 8 + 2 * tq;
      s[nb][0] = key < k_end ? s[nb][0] * a.scale_log2e : -INFINITY;
      s[nb][1] = key + 1 < k_end ? s[nb][1] * a.scale_log2e : -INFINITY;
      s[nb][2] = key < k_end ? s[nb][2] * a.scale_log2e : -INFINITY;
      s[nb][3] = key + 1 < k_end ? s[nb][3] * a.scale_log2e : -INFINITY;
      mx0 = fmaxf(mx0, fmaxf(s[nb][0], s[nb][1]));
      mx1 = fmaxf(mx1, fmaxf(s[nb][2], s[nb][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    // a warp whose 16 keys are all past the end keeps m = -inf: guard the exponent
    const float c0 = mx0 == -INFINITY ? 1.f : exp2f(m0 - mx0);
    const float c1 = mx1 == -INFINITY ? 1.f : exp2f(m1 - mx1);
    const float e0 = mx0 == -INFINITY ? 0.f : mx0, e1 = mx1 == -INFINITY ? 0.f : mx1;
    m0 = mx0; m1 = mx1;
    uint32_t pa[4];
    float ps0 = 0.f, ps1 = 0.f;
    {
      const float p00 = exp2f(s[0][0] - e0), p01 = exp2f(s[0][1] - e0);
      const float p02 = exp2f(s[0][2] - e1), p03 = exp2f(s[0][3] - e1);
      const float p10 = exp2f(s[1][0] - e0), p11 = exp2f(s[1][1] - e0);
      const float p12 = exp2f(s[1][2] - e1), p13 = exp2f(s[1][3] - e1);
      ps0 = (p00 + p01) + (p10 + p11);
      ps1 = (p02 + p03) + (p12 + p13);
      pa[0] = pack2<T>(p00, p01); pa[1] = pack2<T>(p02, p03);
      pa[2] = pack2<T>(p10, p11); pa[3] = pack2<T>(p12, p13);
    }
    l0 = l0 * c0 + ps0;
    l1 = l1 * c1 + ps1;
#pragma unroll
    for (int i = 0; i < 16; ++i) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
    // ---- O += P V: 16 keys x 128 dims, two 8-dim column blocks per ldmatrix ----
#pragma unroll
    for (int np = 0; np < 8; ++np) {
      uint32_t bf[4];
      const int row = kw + (lane & 7) + ((lane >> 3) & 1) * 8;
      ldmatrix_x4_trans(bf, vs + swz(row, np * 2 + (lane >> 4)));
      mma16816<T>(o[2 * np], pa, bf[0], bf[1]);
      mma16816<T>(o[2 * np + 1], pa, bf[2], bf[3]);
    }
    __syncthreads();  // the stage is overwritten by the load issued in the next iteration
  }
  cp_async_wait<0>();

  // ---- merge the four warps (each saw a quarter of the keys) ----
  // l sums over the 4 lanes of a row are still partial: finish them
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  __syncthreads();
  float* mbuf = reinterpret_cast<float*>(smem);  // [4 warps][16 rows][130]: O(128), m, l
  {
    float* w0 = mbuf + ((size_t)warp * 16 + g) * 130;
    float* w1 = w0 + 8 * 130;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      w0[i * 8 + 2 * tq] = o[i][0]; w0[i * 8 + 2 * tq + 1] = o[i][1];
      w1[i * 8 + 2 * tq] = o[i][2]; w1[i * 8 + 2 * tq + 1] = o[i][3];
    }
    if (tq == 0) { w0[128] = m0; w0[129] = l0; w1[128] = m1; w1[129] = l1; }
  }
  __syncthreads();
  for (int idx = tid; idx < G * 128; idx += DM_THREADS) {
    const int row = idx >> 7, d = idx & 127;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, mbuf[((size_t)w * 16 + row) * 130 + 128]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float* rr = mbuf + ((size_t)w * 16 + row) * 130;
      const float wgt = rr[128] == -INFINITY ? 0.f : exp2f(rr[128] - M);
      num = fmaf(wgt, rr[d], num);
      den = fmaf(wgt, rr[129], den);
    }
    if (a.nsplit == 1) {
      reinterpret_cast<T*>(a.out)[((int64_t)b * a.Hq + h * G + row) * 128 + d] =
          Elem<T>::from_f32(den > 0.f ? num / den : 0.f);
    } else {
      float* pp = a.part + ((((int64_t)b * a.Hkv + h) * a.nsplit + split) * a.gp + row) * 130;
      pp[d] = num;
      if (d == 0) { pp[128] = M; pp[129] = den; }
    }
  }
}

template <typename T>
__global__ void decode_mma_merge_kernel(const DmArgs a) {
  const int b = blockIdx.x, h = blockIdx.y;
  const int G = a.Hq / a.Hkv;
  for (int idx = threadIdx.x; idx < G * 128; idx += blockDim.x) {
    const int row = idx >> 7, d = idx & 127;
    const float* base = a.part + ((((int64_t)b * a.Hkv + h) * a.nsplit) * a.gp + row) * 130;
    const int64_t sstride = (int64_t)a.gp * 130;
    float M = -INFINITY;
    for (int s = 0; s < a.nsplit; ++s) M = fmaxf(M, base[s * sstride + 128]);
    float num = 0.f, den = 0.f;
    for (int s = 0; s < a.nsplit; ++s) {
      const float* rr = base + s * sstride;
      const float w = rr[128] == -INFINITY ? 0.f : exp2f(rr[128] - M);
      num = fmaf(w, rr[d], num);
      den = fmaf(w, rr[129], den);
    }
    reinterpret_cast<T*>(a.out)[((int64_t)b * a.Hq + h * G + row) * 128 + d] =
        Elem<T>::from_f32(den > 0.f ? num / den : 0.f);
  }
}

template <typename T>
static int launch_decode_mma(const DmArgs& a, cudaStream_t st) {
  const size_t smem = 2 * 2 * DM_TILE_BYTES;  // 64 KB (also holds the 4 x 16 x 130 float merge buffer)
  auto kern = paged_decode_mma_kernel<T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_error("zp_paged_decode: %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  kern<<<dim3(a.B, a.Hkv, a.nsplit), DM_THREADS, smem, st>>>(a);
  int rc = check_launch("zp_paged_decode(mma)");
  if (rc || a.nsplit == 1) return rc;
  decode_mma_merge_kernel<T><<<dim3(a.B, a.Hkv), 128, 0, st>>>(a);
  return check_launch("zp_paged_decode(mma) merge");
}

// Called by zp_paged_decode for 16-bit caches with head_dim 128, page size % 64 == 0, G <= 16.
int paged_decode_mma(const void* q, const void* k, const void* v, const int32_t* seqlens,
                     const int32_t* table, void* out, float* part, int B, int NBmax, int Hq, int Hkv,
                     int BS, int nsplit, int gp, int64_t kv_stride_page, float scale_log2e, int dtype,
                     cudaStream_t st) {
  DmArgs a;
  a.q = q; a.k = k; a.v = v; a.seqlens = seqlens; a.table = table; a.out = out; a.part = part;
  a.B = B; a.NBmax = NBmax; a.Hq = Hq; a.Hkv = Hkv; a.BS = BS; a.nsplit = nsplit; a.gp = gp;
  a.kv_stride_page = kv_stride_page; a.scale_log2e = scale_log2e;
  if (dtype == ZP_DTYPE_BF16) return launch_decode_mma<__nv_bfloat16>(a, st);
  return launch_decode_mma<__half>(a, st);
}

}  // namespace zp
