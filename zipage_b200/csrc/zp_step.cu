// The small per-step ops around the attention path of one decoder layer, and the decode
// bookkeeping, as single launches:
//   * RMSNorm with optional residual add,
//   * SiLU(gate) * up,
//   * q/k head RMSNorm + rotary embedding + K/V cache write + observation-window write, fused,
//   * the sampler's exponential race,
//   * the decode step's positions / context lengths / slots / window triples, on the device.
// All are streams over HBM with fp32 maths and the reference's rounding points (the value is
// rounded to the tensor dtype T wherever the reference's eager code holds it in a T tensor).
// IEEE division and square root are used where the reference divides or takes rsqrt, and
// products that the reference rounds separately are kept apart (__fmul_rn), so that fp32 results
// agree with it to the last bits of the reductions' summation order.
#include "zp_common.cuh"

namespace zp {

template <typename T> struct Vec16 {   // one 16-byte vector of T
  static constexpr int N = 16 / sizeof(T);
  int4 raw;
  __device__ __forceinline__ float get(int i) const { return Elem<T>::to_f32(reinterpret_cast<const T*>(&raw)[i]); }
  __device__ __forceinline__ void set(int i, float v) { reinterpret_cast<T*>(&raw)[i] = Elem<T>::from_f32(v); }
};

// ---------------------------------------------------------------------------------------------
// RMSNorm (+ residual).  One block per row; the row stays in registers between the two passes.
//   s = x (+ residual) in fp32;  residual_out = T(s);  y = T(T(s * rsqrt(mean(s^2) + eps)) * w)
// ---------------------------------------------------------------------------------------------
template <typename T, int VPT>
__global__ void __launch_bounds__(256)
rms_norm_kernel(const T* x, const T* residual, const T* __restrict__ weight,
                T* out, T* residual_out, int H, int64_t x_stride, int64_t out_stride, float eps) {
  __shared__ float red[32];
  constexpr int EPV = Vec16<T>::N;
  const int64_t row = blockIdx.x;
  const T* xr = x + row * x_stride;
  const T* rr = residual ? residual + row * (int64_t)H : nullptr;
  const int nvec = H / EPV;
  float s[VPT][EPV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < nvec) {
      Vec16<T> a, b;
      a.raw = ld16(xr + v * EPV);
      if (rr) b.raw = ld16(rr + v * EPV);
#pragma unroll
      for (int j = 0; j < EPV; ++j) {
        s[i][j] = rr ? a.get(j) + b.get(j) : a.get(j);
        ss = fmaf(s[i][j], s[i][j], ss);
      }
      if (residual_out) {
        Vec16<T> o;
#pragma unroll
        for (int j = 0; j < EPV; ++j) o.set(j, s[i][j]);
        st16(residual_out + row * (int64_t)H + v * EPV, o.raw);
      }
    }
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)H + eps);
  T* orow = out + row * out_stride;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < nvec) {
      Vec16<T> w, o;
      w.raw = ld16(weight + v * EPV);
#pragma unroll
      for (int j = 0; j < EPV; ++j) o.set(j, __fmul_rn(round_to<T>(__fmul_rn(s[i][j], r)), w.get(j)));
      st16(orow + v * EPV, o.raw);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// out[n, i] = T( T(silu(x[n, i])) * x[n, I + i] ),  silu(a) = a / (1 + exp(-a)) in fp32
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void silu_and_mul_kernel(const T* __restrict__ x, T* __restrict__ out, int I, int64_t total_vec) {
  constexpr int EPV = Vec16<T>::N;
  const int vec_per_row = I / EPV;
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < total_vec;
       v += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = v / vec_per_row;
    const int c = (int)(v - row * vec_per_row) * EPV;
    Vec16<T> a, b, o;
    a.raw = ld16(x + row * 2 * I + c);
    b.raw = ld16(x + row * 2 * I + I + c);
#pragma unroll
    for (int j = 0; j < EPV; ++j) {
      const float g = a.get(j);
      const float sg = round_to<T>(g / (1.f + expf(-g)));
      o.set(j, __fmul_rn(sg, b.get(j)));
    }
    st16(out + row * I + c, o.raw);
  }
}

// ---------------------------------------------------------------------------------------------
// Fused q/k RMSNorm + rotary embedding + cache writes.  One warp per (token, head); a lane owns
// D/64 consecutive dims of each half of the head (the rotation pairs dim d with d + D/2).
// Blocks [0, n_tokens) handle a token each (q heads -> q_out; k heads -> k_out and the K cache; v
// heads -> the V cache); blocks [n_tokens, n_tokens + n_triples) redo the q heads of a window
// token and write them into the observation-window buffer.
// ---------------------------------------------------------------------------------------------
struct QkArgs {
  const void* qkv; const int64_t* positions; const float* cos_sin;
  const void* q_weight; const void* k_weight;
  void* q_out; void* k_out; void* k_cache; void* v_cache;
  const int32_t* slot_mapping; void* query_cache; const int32_t* triples;
  int n_tokens, n_triples, Hq, Hkv;
  int64_t qkv_stride, cache_stride_seq, cache_stride_slot;
  float eps;
};

template <typename T, int D>
__device__ __forceinline__ void norm_rope_head(const T* __restrict__ src, const T* __restrict__ w,
                                               const float* __restrict__ cs, float eps, int lane,
                                               float (&y1)[D / 64], float (&y2)[D / 64]) {
  constexpr int P = D / 64;
  float a[P], b[P];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < P; ++j) {
    a[j] = Elem<T>::to_f32(src[lane * P + j]);
    b[j] = Elem<T>::to_f32(src[D / 2 + lane * P + j]);
    ss = fmaf(a[j], a[j], ss);
    ss = fmaf(b[j], b[j], ss);
  }
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)D + eps);
#pragma unroll
  for (int j = 0; j < P; ++j) {
    const int d = lane * P + j;
    // RMSNorm: T(T(x * r) * w); rotation in fp32 with separately rounded products
    const float x1 = round_to<T>(__fmul_rn(round_to<T>(__fmul_rn(a[j], r)), Elem<T>::to_f32(w[d])));
    const float x2 = round_to<T>(__fmul_rn(round_to<T>(__fmul_rn(b[j], r)), Elem<T>::to_f32(w[D / 2 + d])));
    const float c = cs[d], s = cs[D / 2 + d];
    y1[j] = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));
    y2[j] = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(256) qk_norm_rope_store_kernel(const QkArgs a) {
  constexpr int P = D / 64;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const T* qkv = reinterpret_cast<const T*>(a.qkv);
  const T* qw = reinterpret_cast<const T*>(a.q_weight);
  const T* kw = reinterpret_cast<const T*>(a.k_weight);
  if ((int)blockIdx.x < a.n_tokens) {
    const int n = blockIdx.x;
    const T* row = qkv + (int64_t)n * a.qkv_stride;
    const float* cs = a.cos_sin + a.positions[n] * D;
    const int slot = a.slot_mapping ? a.slot_mapping[n] : -1;
    for (int h = wid; h < a.Hq + 2 * a.Hkv; h += nw) {
      if (h < a.Hq + a.Hkv) {
        const bool is_q = h < a.Hq;
        float y1[P], y2[P];
        norm_rope_head<T, D>(row + (int64_t)h * D, is_q ? qw : kw, cs, a.eps, lane, y1, y2);
        T* dst = is_q ? reinterpret_cast<T*>(a.q_out) + ((int64_t)n * a.Hq + h) * D
                      : (a.k_out ? reinterpret_cast<T*>(a.k_out) + ((int64_t)n * a.Hkv + (h - a.Hq)) * D : nullptr);
        T* cdst = (!is_q && slot != -1)
                      ? reinterpret_cast<T*>(a.k_cache) + ((int64_t)slot * a.Hkv + (h - a.Hq)) * D : nullptr;
#pragma unroll
        for (int j = 0; j < P; ++j) {
          const T o1 = Elem<T>::from_f32(y1[j]), o2 = Elem<T>::from_f32(y2[j]);
          if (dst) { dst[lane * P + j] = o1; dst[D / 2 + lane * P + j] = o2; }
          if (cdst) { cdst[lane * P + j] = o1; cdst[D / 2 + lane * P + j] = o2; }
        }
      } else if (slot != -1) {   // v head: plain copy into the cache
        const int hv = h - a.Hq - a.Hkv;
        const T* src = row + (int64_t)h * D;
        T* cdst = reinterpret_cast<T*>(a.v_cache) + ((int64_t)slot * a.Hkv + hv) * D;
#pragma unroll
        for (int j = 0; j < 2 * P; ++j) cdst[lane * 2 * P + j] = src[lane * 2 * P + j];
      }
    }
  } else {
    const int t = blockIdx.x - a.n_tokens;
    const int n = a.triples[3 * t], qid = a.triples[3 * t + 1], idx = a.triples[3 * t + 2];
    const T* row = qkv + (int64_t)n * a.qkv_stride;
    const float* cs = a.cos_sin + a.positions[n] * D;
    T* base = reinterpret_cast<T*>(a.query_cache) + (int64_t)qid * a.cache_stride_seq +
              (int64_t)idx * a.cache_stride_slot;
    for (int h = wid; h < a.Hq; h += nw) {
      float y1[P], y2[P];
      norm_rope_head<T, D>(row + (int64_t)h * D, qw, cs, a.eps, lane, y1, y2);
      T* dst = base + (int64_t)h * D;
#pragma unroll
      for (int j = 0; j < P; ++j) {
        dst[lane * P + j] = Elem<T>::from_f32(y1[j]);
        dst[D / 2 + lane * P + j] = Elem<T>::from_f32(y2[j]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Sampler: probs = softmax(fp32 logits / T); token = argmax(probs / max(noise, 1e-10)), lowest
// index on ties.  One block per row, three passes over the row (it stays in L2).  With
// noise == NULL the Exp(1) draws come from a counter-based generator keyed by (seed, row, index).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t mix32(uint32_t x) {   // a 32-bit finaliser (bijective)
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}
__device__ __forceinline__ float exp1_draw(uint64_t seed, uint32_t row, uint32_t i) {
  uint32_t h = mix32((uint32_t)seed ^ mix32(i + 0x9e3779b9u));
  h = mix32(h ^ (uint32_t)(seed >> 32) ^ mix32(row + 0x85ebca6bu));
  const float u = ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);   // (0, 1)
  return -logf(u);
}

template <typename T>
__global__ void __launch_bounds__(1024)
sample_kernel(const T* __restrict__ logits, const float* __restrict__ temperatures,
              const float* __restrict__ noise, int64_t* __restrict__ out, int V, uint64_t seed) {
  __shared__ float red[32];
  __shared__ float bval[32];
  __shared__ int bidx[32];
  const int row = blockIdx.x;
  const T* lr = logits + (int64_t)row * V;
  const float t = temperatures[row];
  float m = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) m = fmaxf(m, __fdiv_rn(Elem<T>::to_f32(lr[i]), t));
  m = block_max(m, red);
  float z = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) z += expf(__fdiv_rn(Elem<T>::to_f32(lr[i]), t) - m);
  z = block_sum(z, red);
  float best = -INFINITY;
  int besti = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float p = __fdiv_rn(expf(__fdiv_rn(Elem<T>::to_f32(lr[i]), t) - m), z);
    const float q = noise ? noise[(int64_t)row * V + i] : exp1_draw(seed, row, i);
    const float v = __fdiv_rn(p, fmaxf(q, 1e-10f));
    if (v > best) { best = v; besti = i; }   // ascending i per thread: the first maximum stays
  }
  // (value, index) arg-max: larger value wins, then the lower index
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
    if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) { bval[w] = best; bidx[w] = besti; }
  __syncthreads();
  if (w == 0) {
    best = lane < nw ? bval[lane] : -INFINITY;
    besti = lane < nw ? bidx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
      if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
    }
    if (lane == 0) out[row] = besti;
  }
}

// ---------------------------------------------------------------------------------------------
// Decode bookkeeping from device-resident state.  One block; the window triples keep the order
// of the sequences (block-wide exclusive scan of the "has a triple" flags).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
prepare_decode_kernel(const int32_t* __restrict__ num_tokens, const int32_t* __restrict__ block_tables,
                      const int32_t* __restrict__ query_ids, int B, int W, int qcl, int bs,
                      int64_t* __restrict__ positions, int32_t* __restrict__ context_lens,
                      int32_t* __restrict__ slot_mapping, int32_t* __restrict__ triples,
                      int32_t* __restrict__ n_triples) {
  __shared__ int wsum[32];
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int base = 0; base < B; base += blockDim.x) {
    const int i = base + threadIdx.x;
    int flag = 0, qid = -1, widx = 0;
    if (i < B) {
      const int n = num_tokens[i];
      const int nblocks = (n + bs - 1) / bs;
      const int last = n - (nblocks - 1) * bs;          // tokens in the last page, 1..bs
      int len = 0;
      while (len < W && block_tables[(int64_t)i * W + len] != -1) ++len;
      const int last_page = len > 0 ? block_tables[(int64_t)i * W + len - 1] : 0;
      positions[i] = n - 1;
      context_lens[i] = (len - 1) * bs + last;
      slot_mapping[i] = last_page * bs + last - 1;
      qid = query_ids[i];
      flag = qid != -1 && last > bs - qcl;
      widx = last - (bs - qcl) - 1;
    }
    // exclusive scan of `flag` over the block
    int incl = flag;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) wsum[w] = incl;
    __syncthreads();
    if (w == 0) {
      int s = lane < nw ? wsum[lane] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, s, o);
        if (lane >= o) s += v;
      }
      wsum[lane] = s;   // inclusive over warps
    }
    __syncthreads();
    const int before = carry + (w > 0 ? wsum[w - 1] : 0) + incl - flag;
    if (flag) {
      triples[3 * before] = i;
      triples[3 * before + 1] = qid;
      triples[3 * before + 2] = widx;
    }
    __syncthreads();
    if (threadIdx.x == 0) carry += wsum[nw - 1];
    __syncthreads();
  }
  if (threadIdx.x == 0) *n_triples = carry;
}

}  // namespace zp

extern "C" int zp_rms_norm(const void* x, const void* residual, const void* weight, void* out,
                           void* residual_out, int n_rows, int hidden, int64_t x_stride,
                           int64_t out_stride, float eps, int dtype, void* stream) {
  if (n_rows == 0) return ZP_OK;
  ZP_REQUIRE(x && weight && out, "zp_rms_norm: null pointer");
  ZP_REQUIRE(!residual_out || residual, "zp_rms_norm: residual_out without residual");
  const size_t es = zp::dtype_size(dtype);
  const int epv = (int)(16 / es);
  ZP_REQUIRE(hidden % epv == 0 && (x_stride * es) % 16 == 0 && (out_stride * es) % 16 == 0,
             "zp_rms_norm: rows must be multiples of 16 bytes");
  ZP_REQUIRE(((uintptr_t)x | (uintptr_t)residual | (uintptr_t)weight | (uintptr_t)out |
              (uintptr_t)residual_out) % 16 == 0, "zp_rms_norm: pointers must be 16-byte aligned");
  const int nvec = hidden / epv;
  ZP_REQUIRE(nvec <= 256 * 8, "zp_rms_norm: hidden size %d too large (at most %d)", hidden, 256 * 8 * epv);
  cudaStream_t st = (cudaStream_t)stream;
  ZP_DISPATCH_DTYPE(dtype, T, {
    const T* xp = (const T*)x; const T* rp = (const T*)residual; const T* wp = (const T*)weight;
    T* op = (T*)out; T* rop = (T*)residual_out;
    if (nvec <= 256) zp::rms_norm_kernel<T, 1><<<n_rows, 256, 0, st>>>(xp, rp, wp, op, rop, hidden, x_stride, out_stride, eps);
    else if (nvec <= 512) zp::rms_norm_kernel<T, 2><<<n_rows, 256, 0, st>>>(xp, rp, wp, op, rop, hidden, x_stride, out_stride, eps);
    else if (nvec <= 1024) zp::rms_norm_kernel<T, 4><<<n_rows, 256, 0, st>>>(xp, rp, wp, op, rop, hidden, x_stride, out_stride, eps);
    else zp::rms_norm_kernel<T, 8><<<n_rows, 256, 0, st>>>(xp, rp, wp, op, rop, hidden, x_stride, out_stride, eps);
  });
  return zp::check_launch("zp_rms_norm");
}

extern "C" int zp_silu_and_mul(const void* x, void* out, int n_rows, int inter, int dtype, void* stream) {
  if (n_rows == 0 || inter == 0) return ZP_OK;
  ZP_REQUIRE(x && out, "zp_silu_and_mul: null pointer");
  const size_t es = zp::dtype_size(dtype);
  const int epv = (int)(16 / es);
  ZP_REQUIRE(inter % epv == 0, "zp_silu_and_mul: the intermediate size must be a multiple of %d", epv);
  ZP_REQUIRE(((uintptr_t)x | (uintptr_t)out) % 16 == 0, "zp_silu_and_mul: pointers must be 16-byte aligned");
  const int64_t total_vec = (int64_t)n_rows * (inter / epv);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t want = (total_vec + 255) / 256;
  const int grid = (int)(want < (int64_t)sms * 16 ? want : (int64_t)sms * 16);
  ZP_DISPATCH_DTYPE(dtype, T, {
    zp::silu_and_mul_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>((const T*)x, (T*)out, inter, total_vec);
  });
  return zp::check_launch("zp_silu_and_mul");
}

extern "C" int zp_qk_norm_rope_store(const void* qkv, const int64_t* positions, const float* cos_sin,
                                     const void* q_weight, const void* k_weight, float eps,
                                     void* q_out, void* k_out, void* k_cache, void* v_cache,
                                     const int32_t* slot_mapping, void* query_cache,
                                     const int32_t* triples, int n_triples, int n_tokens, int Hq,
                                     int Hkv, int D, int64_t qkv_stride, int64_t cache_stride_seq,
                                     int64_t cache_stride_slot, int dtype, void* stream) {
  if (n_tokens == 0) return ZP_OK;
  ZP_REQUIRE(qkv && positions && cos_sin && q_weight && k_weight && q_out, "zp_qk_norm_rope_store: null pointer");
  ZP_REQUIRE(!slot_mapping || (k_cache && v_cache), "zp_qk_norm_rope_store: slot mapping without caches");
  ZP_REQUIRE(n_triples == 0 || (triples && query_cache), "zp_qk_norm_rope_store: window triples without a buffer");
  ZP_REQUIRE(D == 64 || D == 128, "zp_qk_norm_rope_store: head_dim %d not supported (64 or 128)", D);
  zp::QkArgs a;
  a.qkv = qkv; a.positions = positions; a.cos_sin = cos_sin; a.q_weight = q_weight; a.k_weight = k_weight;
  a.q_out = q_out; a.k_out = k_out; a.k_cache = k_cache; a.v_cache = v_cache;
  a.slot_mapping = slot_mapping; a.query_cache = query_cache; a.triples = triples;
  a.n_tokens = n_tokens; a.n_triples = n_triples; a.Hq = Hq; a.Hkv = Hkv;
  a.qkv_stride = qkv_stride; a.cache_stride_seq = cache_stride_seq; a.cache_stride_slot = cache_stride_slot;
  a.eps = eps;
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = n_tokens + n_triples;
  ZP_DISPATCH_DTYPE(dtype, T, {
    if (D == 128) zp::qk_norm_rope_store_kernel<T, 128><<<grid, 256, 0, st>>>(a);
    else zp::qk_norm_rope_store_kernel<T, 64><<<grid, 256, 0, st>>>(a);
  });
  return zp::check_launch("zp_qk_norm_rope_store");
}

extern "C" int zp_sample(const void* logits, const float* temperatures, const float* noise,
                         int64_t* tokens_out, int n_rows, int vocab, uint64_t seed, int dtype,
                         void* stream) {
  if (n_rows == 0) return ZP_OK;
  ZP_REQUIRE(logits && temperatures && tokens_out, "zp_sample: null pointer");
  ZP_REQUIRE(vocab > 0, "zp_sample: empty vocabulary");
  ZP_DISPATCH_DTYPE(dtype, T, {
    zp::sample_kernel<T><<<n_rows, 1024, 0, (cudaStream_t)stream>>>((const T*)logits, temperatures, noise,
                                                                   tokens_out, vocab, seed);
  });
  return zp::check_launch("zp_sample");
}

extern "C" int zp_prepare_decode(const int32_t* num_tokens, const int32_t* block_tables,
                                 const int32_t* query_ids, int B, int table_width,
                                 int query_cache_len, int block_size, int64_t* positions_out,
                                 int32_t* context_lens_out, int32_t* slot_mapping_out,
                                 int32_t* triples_out, int32_t* n_triples_out, void* stream) {
  ZP_REQUIRE(n_triples_out, "zp_prepare_decode: null pointer");
  if (B == 0) return cudaMemsetAsync(n_triples_out, 0, sizeof(int32_t), (cudaStream_t)stream) == cudaSuccess
                         ? ZP_OK : ZP_ERR_CUDA;
  ZP_REQUIRE(num_tokens && block_tables && query_ids && positions_out && context_lens_out &&
                 slot_mapping_out && triples_out, "zp_prepare_decode: null pointer");
  ZP_REQUIRE(table_width > 0 && block_size > 0 && query_cache_len >= 0 && query_cache_len <= block_size,
             "zp_prepare_decode: bad sizes");
  zp::prepare_decode_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(
      num_tokens, block_tables, query_ids, B, table_width, query_cache_len, block_size, positions_out,
      context_lens_out, slot_mapping_out, triples_out, n_triples_out);
  return zp::check_launch("zp_prepare_decode");
}
