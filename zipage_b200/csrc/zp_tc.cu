// Host helpers of the tensor-core kernels: tensor-map encoding and the device error word.
#include "zp_tc.cuh"

namespace zp {
namespace tc {

__device__ int g_error_word = 0;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

int make_tensor_map_5d(CUtensorMap* out, CUtensorMapDataType dt, const void* base, const uint64_t dims[5],
                       const uint64_t strides_elems[4], const uint32_t box[5], size_t elem_size) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return ZP_ERR_CUDA; }
  cuuint64_t gdim[5], gstr[4];
  cuuint32_t bx[5], es[5] = {1, 1, 1, 1, 1};
  for (int i = 0; i < 5; ++i) { gdim[i] = dims[i]; bx[i] = box[i]; }
  for (int i = 0; i < 4; ++i) gstr[i] = strides_elems[i] * elem_size;
  CUresult r = fn(out, dt, 5, const_cast<void*>(base), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code %d (dims %llu %llu %llu %llu %llu)", (int)r,
              (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2],
              (unsigned long long)dims[3], (unsigned long long)dims[4]);
    return ZP_ERR_CUDA;
  }
  return ZP_OK;
}

int* device_error_word() {
  int* p = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_error_word) != cudaSuccess) return nullptr;
  return p;
}

}  // namespace tc
}  // namespace zp

// Reads (and optionally clears) the error word the tensor-core kernels raise when one of their
// bounded waits runs out.  Synchronises the device.  0 = no error.
extern "C" int zp_device_error(int* code_out, int reset) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, zp::tc::g_error_word, sizeof(int));
  if (e != cudaSuccess) { zp::set_error("zp_device_error: %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  if (code_out) *code_out = v;
  if (reset && v) {
    const int zero = 0;
    cudaMemcpyToSymbol(zp::tc::g_error_word, &zero, sizeof(int));
  }
  return ZP_OK;
}

extern "C" int zp_device_error_async(int* host_out, void* stream) {
  int* word = zp::tc::device_error_word();
  if (!word || !host_out) { zp::set_error("zp_device_error_async: no error word / null destination"); return ZP_ERR_CUDA; }
  cudaError_t e = cudaMemcpyAsync(host_out, word, sizeof(int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) { zp::set_error("zp_device_error_async: %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  return ZP_OK;
}
