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

// Two fp32 values rounded to T and back / stored as T, as one packed conversion where T is a
// 16-bit type (the scalar f32 -> 16-bit conversion issues at a quarter of the packed one's rate).
template <typename T> struct Two;
template <> struct Two<__nv_bfloat16> {
  static __device__ __forceinline__ void round(float& a, float& b) {
    const float2 f = __bfloat1622float2(__floats2bfloat162_rn(a, b));
    a = f.x; b = f.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    p[0] = v.x; p[1] = v.y;
  }
};
template <> struct Two<__half> {
  static __device__ __forceinline__ void round(float& a, float& b) {
    const float2 f = __half22float2(__floats2half2_rn(a, b));
    a = f.x; b = f.y;
  }
  static __device__ __forceinline__ void store(__half* p, float a, float b) {
    const __half2 v = __floats2half2_rn(a, b);
    p[0] = v.x; p[1] = v.y;
  }
};
template <> struct Two<float> {
  static __device__ __forceinline__ void round(float&, float&) {}
  static __device__ __forceinline__ void store(float* p, float a, float b) { p[0] = a; p[1] = b; }
};

template <typename T> struct Vec16 {   // one 16-byte vector of T
  static constexpr int N = 16 / sizeof(T);
  int4 raw;
  __device__ __forceinline__ float get(int i) const { return Elem<T>::to_f32(reinterpret_cast<const T*>(&raw)[i]); }
  __device__ __forceinline__ void set(int i, float v) { reinterpret_cast<T*>(&raw)[i] = Elem<T>::from_f32(v); }
  __device__ __forceinline__ void set2(int i, float a, float b) { Two<T>::store(reinterpret_cast<T*>(&raw) + i, a, b); }
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
        for (int j = 0; j < EPV; j += 2) o.set2(j, s[i][j], s[i][j + 1]);
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
      for (int j = 0; j < EPV; j += 2) {
        float a = __fmul_rn(s[i][j], r), b = __fmul_rn(s[i][j + 1], r);
        Two<T>::round(a, b);
        o.set2(j, __fmul_rn(a, w.get(j)), __fmul_rn(b, w.get(j + 1)));
      }
      st16(orow + v * EPV, o.raw);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// out[n, i] = T( T(silu(x[n, i])) * x[n, I + i] ),  silu(a) = a / (1 + exp(-a)) in fp32
// ---------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float silu_f32(float g) {
  // fp32 tensors: IEEE division and expf as the reference; 16-bit tensors: the fast forms' last-bit
  // errors disappear in the rounding to T (except at a rounding boundary, ~1 element in 10^4)
  if constexpr (sizeof(T) == 4) return g / (1.f + expf(-g));
  else return __fdividef(g, 1.f + __expf(-g));
}

template <typename T>
__global__ void __launch_bounds__(256)
silu_and_mul_kernel(const T* __restrict__ x, T* __restrict__ out, int I, int64_t total_vec) {
  constexpr int EPV = Vec16<T>::N;
  const int vec_per_row = I / EPV;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t v0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v0 < total_vec; v0 += 2 * stride) {
    Vec16<T> a[2], b[2];
    int64_t row[2];
    int c[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {   // both loads of both vectors in flight before any maths
      const int64_t v = v0 + u * stride;
      if (v < total_vec) {
        row[u] = v / vec_per_row;
        c[u] = (int)(v - row[u] * vec_per_row) * EPV;
        a[u].raw = ld16(x + row[u] * 2 * I + c[u]);
        b[u].raw = ld16(x + row[u] * 2 * I + I + c[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (v0 + u * stride < total_vec) {
        Vec16<T> o;
#pragma unroll
        for (int j = 0; j < EPV; j += 2) {
          float s0 = silu_f32<T>(a[u].get(j)), s1 = silu_f32<T>(a[u].get(j + 1));
          Two<T>::round(s0, s1);
          o.set2(j, __fmul_rn(s0, b[u].get(j)), __fmul_rn(s1, b[u].get(j + 1)));
        }
        st16(out + row[u] * I + c[u], o.raw);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Fused q/k RMSNorm + rotary embedding + cache writes.  One warp per token walks the token's heads
// four at a time (eight lanes per head; a lane owns D/16 consecutive dims of each half of the
// head — the rotation pairs dim d with d + D/2 — and moves them as one vector), with the next
// four heads' loads in flight: q heads -> q_out; k heads -> k_out and the K cache; v heads -> the
// V cache.  Warps past the tokens redo the q heads of a window token and write them into the
// observation-window buffer.
// ---------------------------------------------------------------------------------------------
struct QkArgs {
  const void* qkv; const int64_t* positions; const float* cos_sin;
  const void* q_weight; const void* k_weight;
  void* q_out; void* k_out; void* k_cache; void* v_cache;
  const int32_t* slot_mapping; void* query_cache; const int32_t* triples;
  const int32_t* n_triples_dev;   // NULL, or the device word that holds the number of valid triples
  int n_tokens, n_triples, Hq, Hkv;
  int64_t qkv_stride, cache_stride_seq, cache_stride_slot;
  float eps;
};

// N consecutive elements of T moved as one (or two) vector accesses
template <typename T, int N>
struct alignas((sizeof(T) * N > 16) ? 16 : sizeof(T) * N) Chunk { T v[N]; };
template <typename T, int N>
__device__ __forceinline__ Chunk<T, N> ld_chunk(const T* p) { return *reinterpret_cast<const Chunk<T, N>*>(p); }
template <typename T, int N>
__device__ __forceinline__ void st_chunk(T* p, const Chunk<T, N>& c) { *reinterpret_cast<Chunk<T, N>*>(p) = c; }

// One head on its eight lanes: RMSNorm over the D dims (T(T(x * r) * w)), then the rotation in
// fp32 with separately rounded products, rounded to T once.  ca/cb: this lane's elements of the
// two halves of the head; w1/w2, c/s: its slices of the weight and of the token's cos/sin row.
template <typename T, int D>
__device__ __forceinline__ void norm_rope_head(const Chunk<T, D / 16>& ca, const Chunk<T, D / 16>& cb,
                                               const Chunk<T, D / 16>& w1, const Chunk<T, D / 16>& w2,
                                               const float (&c)[D / 16], const float (&s)[D / 16],
                                               float eps, Chunk<T, D / 16>& o1, Chunk<T, D / 16>& o2) {
  constexpr int P = D / 16;
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < P; ++j) {
    const float av = Elem<T>::to_f32(ca.v[j]), bv = Elem<T>::to_f32(cb.v[j]);
    ss = fmaf(av, av, ss);
    ss = fmaf(bv, bv, ss);
  }
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // within the 8 lanes
  // fp32 tensors: IEEE square root and division as the reference's rsqrt; 16-bit tensors: the
  // fast reciprocal square root's last-bit error disappears in the rounding to T
  float r;
  if constexpr (sizeof(T) == 4) r = 1.f / sqrtf(ss / (float)D + eps);
  else r = rsqrtf(ss / (float)D + eps);
#pragma unroll
  for (int j = 0; j < P; j += 2) {
    // (the elements are unpacked again rather than kept in fp32 across the reduction: registers)
    float x1a = __fmul_rn(Elem<T>::to_f32(ca.v[j]), r), x1b = __fmul_rn(Elem<T>::to_f32(ca.v[j + 1]), r);
    float x2a = __fmul_rn(Elem<T>::to_f32(cb.v[j]), r), x2b = __fmul_rn(Elem<T>::to_f32(cb.v[j + 1]), r);
    Two<T>::round(x1a, x1b);
    Two<T>::round(x2a, x2b);
    x1a = __fmul_rn(x1a, Elem<T>::to_f32(w1.v[j])); x1b = __fmul_rn(x1b, Elem<T>::to_f32(w1.v[j + 1]));
    x2a = __fmul_rn(x2a, Elem<T>::to_f32(w2.v[j])); x2b = __fmul_rn(x2b, Elem<T>::to_f32(w2.v[j + 1]));
    Two<T>::round(x1a, x1b);
    Two<T>::round(x2a, x2b);
    Two<T>::store(o1.v + j, __fsub_rn(__fmul_rn(x1a, c[j]), __fmul_rn(x2a, s[j])),
                  __fsub_rn(__fmul_rn(x1b, c[j + 1]), __fmul_rn(x2b, s[j + 1])));
    Two<T>::store(o2.v + j, __fadd_rn(__fmul_rn(x2a, c[j]), __fmul_rn(x1a, s[j])),
                  __fadd_rn(__fmul_rn(x2b, c[j + 1]), __fmul_rn(x1b, s[j + 1])));
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(256) qk_norm_rope_store_kernel(const QkArgs a) {
  constexpr int P = D / 16;
  const int lane = threadIdx.x & 31, l8 = lane & 7, hg = lane >> 3;   // 4 heads per warp at a time
  // one warp per work item: a token, or (items >= n_tokens) a window triple
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= a.n_tokens + a.n_triples) return;
  const T* qkv = reinterpret_cast<const T*>(a.qkv);
  const bool window = item >= a.n_tokens;
  int n, qid = 0, idx = 0;
  if (!window) n = item;
  else {
    const int t = item - a.n_tokens;
    if (a.n_triples_dev && t >= *a.n_triples_dev) return;   // n_triples was only the upper bound
    n = a.triples[3 * t]; qid = a.triples[3 * t + 1]; idx = a.triples[3 * t + 2];
  }
  const T* row = qkv + (int64_t)n * a.qkv_stride;
  const int H = window ? a.Hq : a.Hq + 2 * a.Hkv;
  // the first heads' elements are requested before the (dependent) cos/sin loads
  auto load_head = [&](int h, Chunk<T, P>& ca, Chunk<T, P>& cb) {
    if (h < H) {
      ca = ld_chunk<T, P>(row + (int64_t)h * D + l8 * P);
      cb = ld_chunk<T, P>(row + (int64_t)h * D + D / 2 + l8 * P);
    } else {
#pragma unroll
      for (int j = 0; j < P; ++j) { ca.v[j] = Elem<T>::from_f32(0.f); cb.v[j] = Elem<T>::from_f32(0.f); }
    }
  };
  Chunk<T, P> ca, cb, na, nb;
  load_head(hg, ca, cb);
  // this lane's slices of the token's cos/sin row and of the two weights
  const float* cs = a.cos_sin + a.positions[n] * D;
  float c[P], sn[P];
  {
    const Chunk<float, P> cc = ld_chunk<float, P>(cs + l8 * P), sc = ld_chunk<float, P>(cs + D / 2 + l8 * P);
#pragma unroll
    for (int j = 0; j < P; ++j) { c[j] = cc.v[j]; sn[j] = sc.v[j]; }
  }
  const Chunk<T, P> qw1 = ld_chunk<T, P>(reinterpret_cast<const T*>(a.q_weight) + l8 * P);
  const Chunk<T, P> qw2 = ld_chunk<T, P>(reinterpret_cast<const T*>(a.q_weight) + D / 2 + l8 * P);
  const Chunk<T, P> kw1 = ld_chunk<T, P>(reinterpret_cast<const T*>(a.k_weight) + l8 * P);
  const Chunk<T, P> kw2 = ld_chunk<T, P>(reinterpret_cast<const T*>(a.k_weight) + D / 2 + l8 * P);
  const int slot = (!window && a.slot_mapping) ? a.slot_mapping[n] : -1;
  T* wbase = window ? reinterpret_cast<T*>(a.query_cache) + (int64_t)qid * a.cache_stride_seq +
                          (int64_t)idx * a.cache_stride_slot : nullptr;
  // every lane runs the same number of iterations (the shuffles need the whole warp)
  for (int h0 = 0; h0 < H; h0 += 4) {
    const int h = h0 + hg;
    load_head(h + 4, na, nb);   // the next four heads, in flight while these are computed
    const bool live = h < H;
    const bool is_q = h < a.Hq, is_k = !is_q && h < a.Hq + a.Hkv;
    Chunk<T, P> o1, o2;
    if (is_q) norm_rope_head<T, D>(ca, cb, qw1, qw2, c, sn, a.eps, o1, o2);
    else norm_rope_head<T, D>(ca, cb, kw1, kw2, c, sn, a.eps, o1, o2);   // (v heads: result unused)
    if (live) {
      T* d0 = nullptr; T* d1 = nullptr;
      if (window) d0 = wbase + (int64_t)h * D;
      else if (is_q) d0 = reinterpret_cast<T*>(a.q_out) + ((int64_t)n * a.Hq + h) * D;
      else if (is_k) {
        if (a.k_out) d0 = reinterpret_cast<T*>(a.k_out) + ((int64_t)n * a.Hkv + (h - a.Hq)) * D;
        if (slot != -1) d1 = reinterpret_cast<T*>(a.k_cache) + ((int64_t)slot * a.Hkv + (h - a.Hq)) * D;
      } else if (slot != -1) {   // v head: plain copy into the cache
        T* vd = reinterpret_cast<T*>(a.v_cache) + ((int64_t)slot * a.Hkv + (h - a.Hq - a.Hkv)) * D;
        st_chunk<T, P>(vd + l8 * P, ca);
        st_chunk<T, P>(vd + D / 2 + l8 * P, cb);
      }
      if (d0) { st_chunk<T, P>(d0 + l8 * P, o1); st_chunk<T, P>(d0 + D / 2 + l8 * P, o2); }
      if (d1) { st_chunk<T, P>(d1 + l8 * P, o1); st_chunk<T, P>(d1 + D / 2 + l8 * P, o2); }
    }
    ca = na; cb = nb;
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
  uint32_t h = mix32(((uint32_t)seed ^ (row * 0x9e3779b9u)) + i * 0x85ebca6bu);
  h = mix32(h ^ (uint32_t)(seed >> 32) ^ row);
  const float u = ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);   // (0, 1)
  return -__logf(u);
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
  // The row is read in 16-byte vectors where its start is aligned (two per thread in flight),
  // element by element otherwise; a thread sees its elements in ascending index order.
  constexpr int EPV = Vec16<T>::N;
  const int nvec = ((uintptr_t)lr % 16 == 0) ? V / EPV : 0;
  auto for_each = [&](auto&& fn) {
#pragma unroll 2
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      Vec16<T> a;
      a.raw = ld16(lr + v * EPV);
#pragma unroll
      for (int j = 0; j < EPV; ++j) fn(v * EPV + j, a.get(j));
    }
    for (int i = nvec * EPV + threadIdx.x; i < V; i += blockDim.x) fn(i, Elem<T>::to_f32(lr[i]));
  };
  // Pass 1: the row maximum of logits / t.  For t > 0 the correctly rounded quotient is monotonic
  // in the numerator, so the maximum of the quotients is the quotient of the maximum.
  float mx = -INFINITY;
  for_each([&](int, float x) { mx = fmaxf(mx, x); });
  mx = block_max(mx, red);
  float m = __fdiv_rn(mx, t);
  if (!(t > 0.f)) {   // a non-positive temperature: fall back to the literal maximum of the quotients
    m = -INFINITY;
    for_each([&](int, float x) { m = fmaxf(m, __fdiv_rn(x, t)); });
    m = block_max(m, red);
  }
  // Pass 2, with fast arithmetic: Z = sum of exp(x_i / t - m), and per thread the two best
  // candidates of the race e_i / q_i.  Dividing every e_i by Z (as the reference does) scales all
  // candidates alike, and the fast exp / reciprocal are off by a few units in the last place, so
  // only near-ties can be ordered differently by the reference's exact expression: the two best
  // per thread are re-evaluated with it below (correctly rounded divisions, expf), against the
  // same Z.
  const float inv_t = 1.f / t;
  float z = 0.f;
  float r0 = -INFINITY, r1 = -INFINITY, q0 = 1.f, q1 = 1.f;
  int i0 = 0x7fffffff, i1 = 0x7fffffff;
  for_each([&](int i, float x) {
    const float e = __expf(fmaf(x, inv_t, -m));
    z += e;
    const float q = fmaxf(noise ? noise[(int64_t)row * V + i] : exp1_draw(seed, row, i), 1e-10f);
    const float r = __fdividef(e, q);
    if (r > r1) {
      if (r > r0) { r1 = r0; q1 = q0; i1 = i0; r0 = r; q0 = q; i0 = i; }
      else { r1 = r; q1 = q; i1 = i; }
    }
  });
  z = block_sum(z, red);
  // the reference's value of a candidate: (exp(x / t - m) / Z) / q
  auto exact = [&](int i, float q) -> float {
    if (i == 0x7fffffff) return -INFINITY;
    const float e = expf(__fdiv_rn(Elem<T>::to_f32(lr[i]), t) - m);
    return __fdiv_rn(__fdiv_rn(e, z), q);
  };
  const float v0 = exact(i0, q0), v1 = exact(i1, q1);
  float best = v0;
  int besti = i0;
  if (v1 > best || (v1 == best && i1 < besti)) { best = v1; besti = i1; }
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
      if (n > 0 && len > 0) {
        positions[i] = n - 1;
        context_lens[i] = (len - 1) * bs + last;
        slot_mapping[i] = last_page * bs + last - 1;
        qid = query_ids[i];
        flag = qid != -1 && last > bs - qcl;
        widx = last - (bs - qcl) - 1;
      } else {  // a padding row of a fixed-size (graph) batch: nothing is stored, nothing attended
        positions[i] = 0;
        context_lens[i] = 0;
        slot_mapping[i] = -1;
      }
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
                                     const int32_t* triples, int n_triples,
                                     const int32_t* n_triples_device, int n_tokens, int Hq,
                                     int Hkv, int D, int64_t qkv_stride, int64_t cache_stride_seq,
                                     int64_t cache_stride_slot, int dtype, void* stream) {
  if (n_tokens == 0) return ZP_OK;
  ZP_REQUIRE(qkv && positions && cos_sin && q_weight && k_weight && q_out, "zp_qk_norm_rope_store: null pointer");
  ZP_REQUIRE(!slot_mapping || (k_cache && v_cache), "zp_qk_norm_rope_store: slot mapping without caches");
  ZP_REQUIRE(n_triples == 0 || (triples && query_cache), "zp_qk_norm_rope_store: window triples without a buffer");
  ZP_REQUIRE(D == 64 || D == 128, "zp_qk_norm_rope_store: head_dim %d not supported (64 or 128)", D);
  {
    const size_t es = zp::dtype_size(dtype);
    const size_t vec = (D / 16) * es > 16 ? 16 : (D / 16) * es;   // the widest vector access used
    ZP_REQUIRE(((uintptr_t)qkv | (uintptr_t)q_weight | (uintptr_t)k_weight | (uintptr_t)q_out |
                (uintptr_t)k_out | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)query_cache |
                (uintptr_t)cos_sin) % 16 == 0 && (qkv_stride * es) % vec == 0 &&
                   (cache_stride_seq * es) % vec == 0 && (cache_stride_slot * es) % vec == 0,
               "zp_qk_norm_rope_store: pointers must be 16-byte aligned and strides vector-aligned");
  }
  zp::QkArgs a;
  a.qkv = qkv; a.positions = positions; a.cos_sin = cos_sin; a.q_weight = q_weight; a.k_weight = k_weight;
  a.q_out = q_out; a.k_out = k_out; a.k_cache = k_cache; a.v_cache = v_cache;
  a.slot_mapping = slot_mapping; a.query_cache = query_cache; a.triples = triples;
  a.n_triples_dev = n_triples_device;
  a.n_tokens = n_tokens; a.n_triples = n_triples; a.Hq = Hq; a.Hkv = Hkv;
  a.qkv_stride = qkv_stride; a.cache_stride_seq = cache_stride_seq; a.cache_stride_slot = cache_stride_slot;
  a.eps = eps;
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = (n_tokens + n_triples + 7) / 8;   // eight warps per block, one work item each
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
