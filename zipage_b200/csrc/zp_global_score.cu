// Global-score merge (and the optional max-normalisation that precedes it).
//
// The score tensor is [L,B,Hkv,NB,BS] (slot-minor) while the persisted score cache is
// [L,P,BS,Hkv] (head-minor); one block per (layer, sequence, page) stages the page's
// Hkv x BS scores through shared memory so that both sides are accessed coalesced.
#include "zp_common.cuh"

namespace zp {

template <typename T>
__global__ void max_norm_kernel(T* __restrict__ x, int N) {
  // one block per (layer, seq, head) row of N values: x /= max(x), rounded to T
  __shared__ float red[32];
  T* row = x + (int64_t)blockIdx.x * N;
  float m = -INFINITY;
  for (int i = threadIdx.x; i < N; i += blockDim.x) m = fmaxf(m, Elem<T>::to_f32(row[i]));
  m = block_max(m, red);
  for (int i = threadIdx.x; i < N; i += blockDim.x)
    row[i] = Elem<T>::from_f32(Elem<T>::to_f32(row[i]) / m);
}

template <typename T>
__global__ void global_score_kernel(T* __restrict__ scores, T* __restrict__ score_cache,
                                    const int32_t* __restrict__ block_table,
                                    const uint8_t* __restrict__ compressed, int B, int NB, int Hkv,
                                    int BS, int64_t sc_stride_layer, int64_t sc_stride_page,
                                    float decay, int activate) {
  extern __shared__ float tile[];  // [Hkv][BS+1]
  const int pg = blockIdx.x % NB, b = blockIdx.x / NB, l = blockIdx.y;
  const PageRef pr = decode_page(block_table[(int64_t)b * NB + pg]);
  if (!pr.valid) return;
  const bool merge = compressed[b] != 0 && !pr.last;
  T* srow = scores + ((int64_t)l * B + b) * Hkv * NB * BS + (int64_t)pg * BS;  // + h*NB*BS + slot
  T* crow = score_cache + (int64_t)l * sc_stride_layer + (int64_t)pr.id * sc_stride_page;
  const int n = Hkv * BS;
  for (int idx = threadIdx.x; idx < n; idx += blockDim.x) {
    const int h = idx / BS, s = idx % BS;
    tile[h * (BS + 1) + s] = Elem<T>::to_f32(srow[(int64_t)h * NB * BS + s]);
  }
  __syncthreads();
  const float decay_t = round_to<T>(decay);
  for (int idx = threadIdx.x; idx < n; idx += blockDim.x) {
    const int s = idx / Hkv, h = idx % Hkv;
    float v = tile[h * (BS + 1) + s];
    if (merge) {
      const float c = round_to<T>(Elem<T>::to_f32(crow[idx]) * decay_t);
      v = activate == 0 ? fmaxf(v, c) : round_to<T>(v + c);
      tile[h * (BS + 1) + s] = v;
    }
    crow[idx] = Elem<T>::from_f32(v);
  }
  if (!merge) return;
  __syncthreads();
  for (int idx = threadIdx.x; idx < n; idx += blockDim.x) {
    const int h = idx / BS, s = idx % BS;
    srow[(int64_t)h * NB * BS + s] = Elem<T>::from_f32(tile[h * (BS + 1) + s]);
  }
}

}  // namespace zp

extern "C" int zp_global_score(void* scores, void* score_cache, const int32_t* block_table,
                               const uint8_t* compressed, int L, int B, int NB, int Hkv, int BS,
                               int64_t sc_stride_layer, int64_t sc_stride_page, float decay,
                               int activate, int max_norm, int dtype, void* stream) {
  if (L * B == 0) return ZP_OK;
  ZP_REQUIRE(scores && score_cache && block_table && compressed, "zp_global_score: null pointer");
  ZP_REQUIRE(decay >= 0.f && decay <= 1.f, "zp_global_score: decay must be in [0,1]");
  ZP_REQUIRE(activate == 0 || activate == 1, "zp_global_score: activate must be 0 (max) or 1 (sum)");
  const size_t smem = sizeof(float) * (size_t)Hkv * (BS + 1);
  ZP_REQUIRE(smem <= 200 * 1024, "zp_global_score: Hkv*BS too large");
  cudaStream_t st = (cudaStream_t)stream;
  ZP_DISPATCH_DTYPE(dtype, T, {
    if (max_norm) {
      zp::max_norm_kernel<T><<<L * B * Hkv, 256, 0, st>>>((T*)scores, NB * BS);
      int rc = zp::check_launch("zp_global_score(max_norm)");
      if (rc) return rc;
    }
    auto kern = zp::global_score_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<dim3(B * NB, L), 256, smem, st>>>((T*)scores, (T*)score_cache, block_table, compressed, B,
                                            NB, Hkv, BS, sc_stride_layer, sc_stride_page, decay,
                                            activate);
  });
  return zp::check_launch("zp_global_score");
}
