// Window-masked attention scoring (portable SIMT kernel, fp32 maths, any cache dtype).
//
// One block per unit (layer, sequence, kv head).  The unit's G*QCL window-query rows stay in
// shared memory; the unit's keys stream through in tiles of 64.  The logits buffer of the
// reference ([L,B,Hq,QCL,NB,BS]) is never materialised: three sweeps over the keys recompute the
// logits tile by tile — (1) row maximum, (2) row sum of exp, (3) probabilities, max over the
// query heads of the group, mean/max over the window rows.  Rounding follows the reference:
// logits are rounded to T when stored (attention_score.py:129-130); the shifted logits, the
// probabilities and the final mean are each rounded to T (torch ops on a T tensor, :220-243).
#include "zp_common.cuh"

namespace zp {

constexpr int WS_THREADS = 256;
constexpr int WS_KT = 64;         // keys per tile
constexpr int WS_RC_MAX = 128;    // rows per chunk (16 row groups x 8)

template <typename T, int D>
struct WsSmem {
  static constexpr int LD = D + 4;  // padded row of fp32, keeps float4 alignment
};

struct WsParams {
  const void* k_cache;
  const void* q_cache;
  const int32_t* seq_idx;
  const int32_t* block_table;
  void* scores_out;
  void* logits_out;
  int L, B, NB, Hq, Hkv, QCL, BS;
  int64_t k_stride_layer, k_stride_page, q_stride_layer, q_stride_seq;
  float scale;
  int reduce_mode;
};

// S[rows of chunk][64 keys] for one key tile; thread (ty,tx) owns rows ty+16a, keys tx+16c.
template <int D>
__device__ __forceinline__ void tile_dot(const float* __restrict__ sQ, const float* __restrict__ sK,
                                         int row0, int ty, int tx, float (&acc)[8][4]) {
  constexpr int LD = D + 4;
#pragma unroll
  for (int a = 0; a < 8; ++a)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[a][c] = 0.f;
#pragma unroll 4
  for (int d = 0; d < D; d += 4) {
    float4 kv[4];
#pragma unroll
    for (int c = 0; c < 4; ++c)
      kv[c] = *reinterpret_cast<const float4*>(sK + (tx + 16 * c) * LD + d);
#pragma unroll
    for (int a = 0; a < 8; ++a) {
      const float4 qv = *reinterpret_cast<const float4*>(sQ + (row0 + ty + 16 * a) * LD + d);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        acc[a][c] = fmaf(qv.x, kv[c].x, acc[a][c]);
        acc[a][c] = fmaf(qv.y, kv[c].y, acc[a][c]);
        acc[a][c] = fmaf(qv.z, kv[c].z, acc[a][c]);
        acc[a][c] = fmaf(qv.w, kv[c].w, acc[a][c]);
      }
    }
  }
}

template <typename T, int D>
__device__ __forceinline__ void load_key_tile(const T* __restrict__ kpage, int h, int Hkv, int slot0,
                                              float* __restrict__ sK) {
  constexpr int LD = D + 4;
  constexpr int EPV = 16 / sizeof(T);      // elements per 16-byte vector
  constexpr int VPR = D / EPV;             // vectors per row
  for (int v = threadIdx.x; v < WS_KT * VPR; v += WS_THREADS) {
    const int r = v / VPR, c = v % VPR;
    const T* src = kpage + ((int64_t)(slot0 + r) * Hkv + h) * D + c * EPV;
    const int4 raw = ld16(src);
    const T* e = reinterpret_cast<const T*>(&raw);
    float* dst = sK + r * LD + c * EPV;
#pragma unroll
    for (int j = 0; j < EPV; ++j) dst[j] = Elem<T>::to_f32(e[j]);
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(WS_THREADS, 1) window_score_kernel(const WsParams p) {
  constexpr int LD = D + 4;
  extern __shared__ __align__(16) float smem[];
  const int G = p.Hq / p.Hkv;
  const int ICH = min(p.QCL, WS_RC_MAX / G);     // window rows per chunk
  const int RC = ICH * G;                        // rows per chunk
  const int nchunk = (p.QCL + ICH - 1) / ICH;
  const int Rpad = nchunk * WS_RC_MAX;           // sQ rows incl. zero padding of the last chunk

  float* sQ = smem;                              // [nchunk*128][LD] (chunk c starts at row c*128)
  float* sK = sQ + (size_t)Rpad * LD;            // [64][LD]
  float* sP = sK + WS_KT * LD;                   // [128][65]
  float* sMax = sP + WS_RC_MAX * (WS_KT + 1);    // [Rpad]
  float* sZ = sMax + Rpad;                       // [Rpad]
  float* sPart = sZ + Rpad;                      // [4][64]
  float* sAcc = sPart + 4 * WS_KT;               // [64]

  const int unit = blockIdx.x;
  const int h = unit % p.Hkv;
  const int b = (unit / p.Hkv) % p.B;
  const int l = unit / (p.Hkv * p.B);
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;

  const T* kbase = reinterpret_cast<const T*>(p.k_cache) + (int64_t)l * p.k_stride_layer;
  const T* qbase = reinterpret_cast<const T*>(p.q_cache) + (int64_t)l * p.q_stride_layer +
                   (int64_t)p.seq_idx[b] * p.q_stride_seq;
  const int32_t* table = p.block_table + (int64_t)b * p.NB;
  T* out = reinterpret_cast<T*>(p.scores_out) + (((int64_t)l * p.B + b) * p.Hkv + h) * p.NB * p.BS;
  T* lout = p.logits_out ? reinterpret_cast<T*>(p.logits_out) : nullptr;

  // ---- stage the window queries: chunk c, local row (i_local*G + g) ----
  for (int idx = tid; idx < Rpad * (D / 4); idx += WS_THREADS) {
    const int row = idx / (D / 4), d4 = (idx % (D / 4)) * 4;
    const int c = row / WS_RC_MAX, lr = row % WS_RC_MAX;
    const int i = c * ICH + lr / G, g = lr % G;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (lr < RC && i < p.QCL) {
      const T* src = qbase + ((int64_t)i * p.Hq + (h * G + g)) * D + d4;
      v.x = Elem<T>::to_f32(src[0]); v.y = Elem<T>::to_f32(src[1]);
      v.z = Elem<T>::to_f32(src[2]); v.w = Elem<T>::to_f32(src[3]);
    }
    *reinterpret_cast<float4*>(sQ + (size_t)row * LD + d4) = v;
  }
  __syncthreads();

  // masked logit, rounded to T, for chunk-local row lr (window row i) and key slot in page
  auto logit_of = [&](float acc, int i, int slot, bool last) -> float {
    float v = round_to<T>(acc * p.scale);
    if (last && slot > p.BS - p.QCL + i) v = -INFINITY;
    return v;
  };

  // ---- sweeps 1 and 2: row maximum, then row sum of exp ----
  for (int c = 0; c < nchunk; ++c) {
    const int rows_here = min(ICH, p.QCL - c * ICH) * G;
    for (int sweep = 0; sweep < 2; ++sweep) {
      float st[8];
#pragma unroll
      for (int a = 0; a < 8; ++a) st[a] = sweep == 0 ? -INFINITY : 0.f;
      float mrow[8];
#pragma unroll
      for (int a = 0; a < 8; ++a) mrow[a] = sweep == 1 ? sMax[c * WS_RC_MAX + ty + 16 * a] : 0.f;
      for (int pg = 0; pg < p.NB; ++pg) {
        const PageRef pr = decode_page(table[pg]);
        if (!pr.valid) {
          if (lout && sweep == 0) {  // padded pages of the logits buffer hold -inf
            for (int idx = tid; idx < rows_here * p.BS; idx += WS_THREADS) {
              const int lr = idx / p.BS, s = idx % p.BS;
              const int i = c * ICH + lr / G, g = lr % G;
              lout[(((((int64_t)l * p.B + b) * p.Hq + (h * G + g)) * p.QCL + i) * p.NB + pg) * p.BS + s] =
                  Elem<T>::from_f32(-INFINITY);
            }
          }
          continue;
        }
        const T* kpage = kbase + (int64_t)pr.id * p.k_stride_page;
        for (int s0 = 0; s0 < p.BS; s0 += WS_KT) {
          __syncthreads();
          load_key_tile<T, D>(kpage, h, p.Hkv, s0, sK);
          __syncthreads();
          float acc[8][4];
          tile_dot<D>(sQ, sK, c * WS_RC_MAX, ty, tx, acc);
#pragma unroll
          for (int a = 0; a < 8; ++a) {
            const int lr = ty + 16 * a;
            if (lr >= rows_here) continue;
            const int i = c * ICH + lr / G;
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
              const int slot = s0 + tx + 16 * cc;
              const float lg = logit_of(acc[a][cc], i, slot, pr.last);
              if (sweep == 0) {
                st[a] = fmaxf(st[a], lg);
                if (lout) {
                  const int g = lr % G;
                  lout[(((((int64_t)l * p.B + b) * p.Hq + (h * G + g)) * p.QCL + i) * p.NB + pg) * p.BS + slot] =
                      Elem<T>::from_f32(lg);
                }
              } else {
                st[a] += expf(round_to<T>(lg - mrow[a]));
              }
            }
          }
        }
      }
      // combine the 16 key-groups of each row (lanes tx of one half-warp)
#pragma unroll
      for (int a = 0; a < 8; ++a) {
        float v = st[a];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
          const float w = __shfl_xor_sync(0xffffffffu, v, o);
          v = sweep == 0 ? fmaxf(v, w) : v + w;
        }
        if (tx == 0) (sweep == 0 ? sMax : sZ)[c * WS_RC_MAX + ty + 16 * a] = v;
      }
      __syncthreads();
    }
  }

  // ---- sweep 3: probabilities, group max, window mean/max ----
  const float inv_qcl_denominator = (float)p.QCL;
  for (int pg = 0; pg < p.NB; ++pg) {
    const PageRef pr = decode_page(table[pg]);
    if (!pr.valid) {  // softmax of -inf logits: exactly 0
      for (int s = tid; s < p.BS; s += WS_THREADS) out[(int64_t)pg * p.BS + s] = Elem<T>::from_f32(0.f);
      continue;
    }
    const T* kpage = kbase + (int64_t)pr.id * p.k_stride_page;
    for (int s0 = 0; s0 < p.BS; s0 += WS_KT) {
      __syncthreads();
      load_key_tile<T, D>(kpage, h, p.Hkv, s0, sK);
      if (tid < WS_KT) sAcc[tid] = p.reduce_mode == 0 ? 0.f : -INFINITY;
      __syncthreads();
      for (int c = 0; c < nchunk; ++c) {
        const int ich_here = min(ICH, p.QCL - c * ICH);
        const int rows_here = ich_here * G;
        float acc[8][4];
        tile_dot<D>(sQ, sK, c * WS_RC_MAX, ty, tx, acc);
#pragma unroll
        for (int a = 0; a < 8; ++a) {
          const int lr = ty + 16 * a;
          if (lr >= rows_here) continue;
          const int i = c * ICH + lr / G;
          const float m = sMax[c * WS_RC_MAX + lr], z = sZ[c * WS_RC_MAX + lr];
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            const int slot = s0 + tx + 16 * cc;
            const float lg = logit_of(acc[a][cc], i, slot, pr.last);
            const float e = expf(round_to<T>(lg - m));
            sP[lr * (WS_KT + 1) + tx + 16 * cc] = round_to<T>(e / z);
          }
        }
        __syncthreads();
        {  // thread (part, n): window rows i = part, part+4, ... of this chunk
          const int n = tid & 63, part = tid >> 6;
          float v = p.reduce_mode == 0 ? 0.f : -INFINITY;
          for (int il = part; il < ich_here; il += 4) {
            float mx = sP[(il * G) * (WS_KT + 1) + n];
            for (int g = 1; g < G; ++g) mx = fmaxf(mx, sP[(il * G + g) * (WS_KT + 1) + n]);
            v = p.reduce_mode == 0 ? v + mx : fmaxf(v, mx);
          }
          sPart[part * WS_KT + n] = v;
        }
        __syncthreads();
        if (tid < WS_KT) {
          float v = sAcc[tid];
          for (int part = 0; part < 4; ++part)
            v = p.reduce_mode == 0 ? v + sPart[part * WS_KT + tid] : fmaxf(v, sPart[part * WS_KT + tid]);
          sAcc[tid] = v;
        }
        __syncthreads();
      }
      if (tid < WS_KT) {
        const float v = p.reduce_mode == 0 ? sAcc[tid] / inv_qcl_denominator : sAcc[tid];
        out[(int64_t)pg * p.BS + s0 + tid] = Elem<T>::from_f32(v);
      }
    }
  }
}

template <typename T, int D>
static int launch_window_score(const WsParams& p, cudaStream_t stream) {
  constexpr int LD = D + 4;
  const int G = p.Hq / p.Hkv;
  const int ICH = p.QCL < WS_RC_MAX / G ? p.QCL : WS_RC_MAX / G;
  const int nchunk = (p.QCL + ICH - 1) / ICH;
  const int Rpad = nchunk * WS_RC_MAX;
  const size_t smem = sizeof(float) * ((size_t)Rpad * LD + WS_KT * LD + WS_RC_MAX * (WS_KT + 1) +
                                       2 * Rpad + 4 * WS_KT + WS_KT);
  if (smem > 227 * 1024) {
    set_error("zp_window_score: G*QCL=%d rows need %zu bytes of shared memory (max 232448)",
              G * p.QCL, smem);
    return ZP_ERR_UNSUPPORTED;
  }
  auto kern = window_score_kernel<T, D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_error("zp_window_score: %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  kern<<<p.L * p.B * p.Hkv, WS_THREADS, smem, stream>>>(p);
  return check_launch("zp_window_score");
}

int window_score_simt(const WsParams& p, int D, int dtype, cudaStream_t stream) {
  ZP_DISPATCH_DTYPE(dtype, T, {
    if (D == 128) return launch_window_score<T, 128>(p, stream);
    if (D == 64) return launch_window_score<T, 64>(p, stream);
  });
  set_error("zp_window_score: head_dim %d not supported (64 or 128)", D);
  return ZP_ERR_UNSUPPORTED;
}

// tcgen05 path (zp_window_score_tc.cu)
bool window_score_tc_supported(int dtype, int D, int BS, int Hq, int Hkv, int QCL, bool want_logits);
int window_score_tc(const void* k_cache, const void* q_cache, const int32_t* seq_idx,
                    const int32_t* block_table, void* scores_out, int L, int B, int NB, int Hq, int Hkv,
                    int QCL, int64_t k_stride_layer, int64_t k_stride_page, int64_t q_stride_layer,
                    int64_t q_stride_seq, float scale, int reduce_mode, int dtype, float* partial,
                    cudaStream_t st);
size_t window_score_tc_workspace_bytes(int L, int B, int NB, int Hq, int Hkv, int QCL);

}  // namespace zp

extern "C" size_t zp_window_score_workspace_bytes(int L, int B, int NB, int Hq, int Hkv, int QCL) {
  return Hkv > 0 && Hq % Hkv == 0 ? zp::window_score_tc_workspace_bytes(L, B, NB, Hq, Hkv, QCL) : 0;
}

extern "C" int zp_window_score(const void* k_cache, const void* query_cache, const int32_t* seq_idx,
                               const int32_t* block_table, void* scores_out, void* logits_out,
                               int L, int B, int NB, int Hq, int Hkv, int D, int QCL, int BS,
                               int64_t k_stride_layer, int64_t k_stride_page,
                               int64_t q_stride_layer, int64_t q_stride_seq, float softmax_scale,
                               int reduce_mode, int dtype, int impl, void* stream) {
  return zp_window_score_ws(k_cache, query_cache, seq_idx, block_table, scores_out, logits_out, L, B, NB,
                            Hq, Hkv, D, QCL, BS, k_stride_layer, k_stride_page, q_stride_layer,
                            q_stride_seq, softmax_scale, reduce_mode, dtype, impl, nullptr, 0, stream);
}

extern "C" int zp_window_score_ws(const void* k_cache, const void* query_cache, const int32_t* seq_idx,
                                  const int32_t* block_table, void* scores_out, void* logits_out,
                                  int L, int B, int NB, int Hq, int Hkv, int D, int QCL, int BS,
                                  int64_t k_stride_layer, int64_t k_stride_page,
                                  int64_t q_stride_layer, int64_t q_stride_seq, float softmax_scale,
                                  int reduce_mode, int dtype, int impl, void* workspace,
                                  size_t workspace_bytes, void* stream) {
  if (L * B == 0) return ZP_OK;
  ZP_REQUIRE(k_cache && query_cache && seq_idx && block_table && scores_out,
             "zp_window_score: null pointer");
  ZP_REQUIRE(Hkv > 0 && Hq % Hkv == 0, "zp_window_score: Hq=%d must be a multiple of Hkv=%d", Hq, Hkv);
  ZP_REQUIRE(BS % 64 == 0 && QCL >= 1 && QCL <= BS, "zp_window_score: bad BS=%d / QCL=%d", BS, QCL);
  ZP_REQUIRE(Hq / Hkv <= zp::WS_RC_MAX, "zp_window_score: group size %d too large", Hq / Hkv);
  ZP_REQUIRE(reduce_mode == 0 || reduce_mode == 1, "zp_window_score: reduce_mode must be 0 or 1");
  ZP_REQUIRE(((uintptr_t)k_cache % 16 == 0) && (k_stride_layer * zp::dtype_size(dtype)) % 16 == 0 &&
                 (k_stride_page * zp::dtype_size(dtype)) % 16 == 0,
             "zp_window_score: K cache must be 16-byte aligned");
  zp::WsParams p;
  p.k_cache = k_cache; p.q_cache = query_cache; p.seq_idx = seq_idx; p.block_table = block_table;
  p.scores_out = scores_out; p.logits_out = logits_out;
  p.L = L; p.B = B; p.NB = NB; p.Hq = Hq; p.Hkv = Hkv; p.QCL = QCL; p.BS = BS;
  p.k_stride_layer = k_stride_layer; p.k_stride_page = k_stride_page;
  p.q_stride_layer = q_stride_layer; p.q_stride_seq = q_stride_seq;
  p.scale = softmax_scale; p.reduce_mode = reduce_mode;
  ZP_REQUIRE(softmax_scale > 0.f, "zp_window_score: softmax_scale must be positive");
  const size_t ws_need = zp::window_score_tc_workspace_bytes(L, B, NB, Hq, Hkv, QCL);
  const bool ws_ok = ws_need == 0 || (workspace && workspace_bytes >= ws_need + 256);
  const bool can_tc = ws_ok && zp::window_score_tc_supported(dtype, D, BS, Hq, Hkv, QCL, logits_out != nullptr) &&
                      ((uintptr_t)query_cache % 16 == 0) &&
                      (q_stride_layer * zp::dtype_size(dtype)) % 16 == 0 &&
                      (q_stride_seq * zp::dtype_size(dtype)) % 16 == 0;
  if (impl == ZP_IMPL_TCGEN05 && !can_tc) {
    zp::set_error("zp_window_score: the tcgen05 kernel needs a 16-bit cache, head_dim 128, page size "
                  "256, a power-of-two group size, no logits output and, for more than 128 window rows, "
                  "a workspace of zp_window_score_workspace_bytes()");
    return ZP_ERR_UNSUPPORTED;
  }
  if (impl != ZP_IMPL_SIMT && can_tc)
    return zp::window_score_tc(k_cache, query_cache, seq_idx, block_table, scores_out, L, B, NB, Hq,
                               Hkv, QCL, k_stride_layer, k_stride_page, q_stride_layer, q_stride_seq,
                               softmax_scale, reduce_mode, dtype,
                               ws_need ? reinterpret_cast<float*>(((uintptr_t)workspace + 255) & ~(uintptr_t)255) : nullptr,
                               (cudaStream_t)stream);
  return zp::window_score_simt(p, D, dtype, (cudaStream_t)stream);
}
