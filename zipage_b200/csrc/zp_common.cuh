// Shared device/host helpers of libzipage_b200 (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/zipage_b200.h"

namespace zp {

// ---- error reporting (no exceptions cross the C boundary) -----------------
void set_error(const char* fmt, ...);
int check_launch(const char* what);

#define ZP_REQUIRE(cond, ...)            \
  do {                                   \
    if (!(cond)) {                       \
      zp::set_error(__VA_ARGS__);        \
      return ZP_ERR_INVALID_ARGUMENT;    \
    }                                    \
  } while (0)

// ---- element types ---------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Elem<__half> {
  static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};
template <> struct Elem<float> {
  static __device__ __forceinline__ float to_f32(float v) { return v; }
  static __device__ __forceinline__ float from_f32(float v) { return v; }
};

// Round an fp32 value to T and bring it back: the value a tensor of dtype T would hold.
template <typename T> __device__ __forceinline__ float round_to(float v) {
  return Elem<T>::to_f32(Elem<T>::from_f32(v));
}

static inline size_t dtype_size(int dtype) {
  return dtype == ZP_DTYPE_F32 ? 4 : 2;
}

// Dispatch a templated launcher on the dtype code.
#define ZP_DISPATCH_DTYPE(dtype, T, ...)                                  \
  do {                                                                    \
    if ((dtype) == ZP_DTYPE_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else if ((dtype) == ZP_DTYPE_F16) { using T = __half; __VA_ARGS__; }  \
    else if ((dtype) == ZP_DTYPE_F32) { using T = float; __VA_ARGS__; }   \
    else { zp::set_error("unknown dtype code %d", (int)(dtype)); return ZP_ERR_INVALID_ARGUMENT; } \
  } while (0)

// ---- block-table encoding ---------------------------------------------------
// -1 = padding, id >= 0 = ordinary page, -(id)-2 = the sequence's last page.
struct PageRef {
  int id;      // decoded page id (undefined when !valid)
  bool valid;
  bool last;
};
__device__ __forceinline__ PageRef decode_page(int entry) {
  PageRef r;
  r.valid = entry != -1;
  r.last = entry < -1;
  r.id = r.last ? (-entry - 2) : entry;
  return r;
}

// ---- reductions ---------------------------------------------------------------
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Block-wide reductions with a fixed combination order (deterministic).  `red` is
// shared scratch of at least 32 floats; all threads of the block must call.
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : 0.f;
  r = warp_sum(r);
  return r;
}

// 16-byte vector copy helpers
__device__ __forceinline__ int4 ld16(const void* p) { return *reinterpret_cast<const int4*>(p); }
__device__ __forceinline__ void st16(void* p, int4 v) { *reinterpret_cast<int4*>(p) = v; }

}  // namespace zp
