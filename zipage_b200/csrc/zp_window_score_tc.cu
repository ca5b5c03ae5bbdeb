// Window-masked attention scoring on tcgen05 tensor cores (16-bit caches, head_dim 128, page
// size 256, G*QCL <= 128 window rows, G a power of two).
//
// One block per unit (layer, sequence, kv head).  The unit's window queries (row r = i*G + g) are
// loaded once by TMA; the unit's key pages stream through a 3-stage ring of 64 KB swizzled tiles.
// Three sweeps over the pages recompute the logits on the tensor cores instead of storing them:
//   sweep 0: D[row][key]  = Q K^T (M = 128 rows, N = 256 keys)   -> row maximum
//   sweep 1: same product                                         -> row sum of exp
//   sweep 2: D[key][row]  = K Q^T (2 x (M = 128 keys, N = 128 rows)) -> probabilities; each thread
//            owns one key and sees all window rows, so the max over the query heads of the group
//            and the mean/max over the window are register-local.
// Rounding points are the reference's: logits, shifted logits and probabilities are rounded to T
// (attention_score.py:129-130 and the torch ops at :220-243); exp uses ex2.approx.
// Roles: warp 0 = TMA producer + TMEM owner, warp 1 = MMA issuer, warps 2-5 = epilogue.
#include "zp_tc.cuh"

namespace zp {

using namespace tc;

constexpr int WT_THREADS = 192;
constexpr int WT_PAGE_BYTES = 65536;
constexpr int WT_BLOCK_BYTES = 32768;
constexpr int WT_QBLOCK_BYTES = 16384;  // 128 rows x 128 bytes
constexpr int WT_NS = 3;

struct WtParams {
  const int32_t* seq_idx;
  const int32_t* block_table;
  void* scores_out;
  int* error_word;
  int L, B, NB, Hq, Hkv, QCL;
  float scale;
  int reduce_mode;
};

struct __align__(16) WtShared {
  uint64_t full[WT_NS], empty[WT_NS], tfull[2], tempty[2], qfull, stats_ready;
  alignas(16) float2 stats[128];  // (row maximum in T, 1 / row sum of exp)
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// sum (or max) over window rows of the max over each group of G consecutive columns
template <int G>
__device__ __forceinline__ float group_reduce(const float (&p)[32], int ncols, bool use_max, float acc) {
#pragma unroll
  for (int j = 0; j < 32; j += G) {
    float mx = p[j];
#pragma unroll
    for (int g = 1; g < G; ++g) mx = fmaxf(mx, p[j + g]);
    if (j < ncols) acc = use_max ? fmaxf(acc, mx) : acc + mx;
  }
  return acc;
}

template <typename T>
__global__ void __launch_bounds__(WT_THREADS, 1)
window_score_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmQ,
                       const WtParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* bufs = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* qbuf = bufs + WT_NS * WT_PAGE_BYTES;
  WtShared& sh = *reinterpret_cast<WtShared*>(qbuf + 2 * WT_QBLOCK_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int unit = blockIdx.x;
  const int h = unit % p.Hkv, b = (unit / p.Hkv) % p.B, l = unit / (p.Hkv * p.B);
  const int G = p.Hq / p.Hkv, R = G * p.QCL;
  const int32_t* table = p.block_table + (int64_t)b * p.NB;
  int nvalid = 0;
  for (int pg = 0; pg < p.NB; ++pg) nvalid += table[pg] != -1;
  const int ntiles = 3 * nvalid;

  if (threadIdx.x == 0) {
    for (int i = 0; i < WT_NS; ++i) { mbar_init(&sh.full[i], 1); mbar_init(&sh.empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sh.tfull[i], 1); mbar_init(&sh.tempty[i], 4); }
    mbar_init(&sh.qfull, 1);
    mbar_init(&sh.stats_ready, 128);
    sh.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&sh.tmem_base, 512);
    tmem_relinquish();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = sh.tmem_base;
  volatile int* abortp = &sh.abort_flag;

  // tile tt -> (sweep, table position): sweeps 0 and 2 walk the table forwards, sweep 1 backwards
  // (the pages it starts with are the ones sweep 0 touched last, still in L2)
  auto tile_page = [&](int tt, int& sweep) -> int {
    sweep = tt / nvalid;
    int idx = tt % nvalid;
    if (sweep == 1) idx = nvalid - 1 - idx;
    int seen = 0;
    for (int pg = 0; pg < p.NB; ++pg)
      if (table[pg] != -1) { if (seen == idx) return pg; ++seen; }
    return 0;
  };

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tensormap(&tmK);
      prefetch_tensormap(&tmQ);
      mbar_arrive_expect_tx(&sh.qfull, (uint32_t)(2 * R * 128));
      const int qid = p.seq_idx[b];
      tma_load_5d(qbuf, &tmQ, &sh.qfull, 0, h * G, 0, qid, l);
      tma_load_5d(qbuf + WT_QBLOCK_BYTES, &tmQ, &sh.qfull, 64, h * G, 0, qid, l);
      for (int tt = 0; tt < ntiles; ++tt) {
        int sweep;
        const int pg = tile_page(tt, sweep);
        const int s = tt % WT_NS, k = tt / WT_NS;
        if (!mbar_wait(&sh.empty[s], (k & 1) ^ 1, abortp, p.error_word, 111)) break;
        const int id = decode_page(table[pg]).id;
        mbar_arrive_expect_tx(&sh.full[s], WT_PAGE_BYTES);
        tma_load_5d(bufs + s * WT_PAGE_BYTES, &tmK, &sh.full[s], 0, h, 0, id, l);
        tma_load_5d(bufs + s * WT_PAGE_BYTES + WT_BLOCK_BYTES, &tmK, &sh.full[s], 64, h, 0, id, l);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t IDESC_QK = idesc_f16(UmmaFmt<T>::fmt, 128, 256);
      constexpr uint32_t IDESC_KQ = idesc_f16(UmmaFmt<T>::fmt, 128, 128);
      bool ok = mbar_wait(&sh.qfull, 0, abortp, p.error_word, 211);
      const uint32_t q_addr = smem_u32(qbuf);
      for (int tt = 0; ok && tt < ntiles; ++tt) {
        const int sweep = tt / nvalid;
        const int s = tt % WT_NS, k = tt / WT_NS, buf = tt & 1, u = tt >> 1;
        if (!mbar_wait(&sh.full[s], k & 1, abortp, p.error_word, 212)) break;
        if (!mbar_wait(&sh.tempty[buf], (u & 1) ^ 1, abortp, p.error_word, 213)) break;
        fence_after_sync();
        const uint32_t k_addr = smem_u32(bufs + s * WT_PAGE_BYTES);
        const uint32_t d = tmem_base + buf * 256;
        if (sweep < 2) {
          umma_k128(d, q_addr, WT_QBLOCK_BYTES, k_addr, WT_BLOCK_BYTES, IDESC_QK);
        } else {
          umma_k128(d, k_addr, WT_BLOCK_BYTES, q_addr, WT_QBLOCK_BYTES, IDESC_KQ);
          umma_k128(d + 128, k_addr + 16384, WT_BLOCK_BYTES, q_addr, WT_QBLOCK_BYTES, IDESC_KQ);
        }
        umma_commit(&sh.tfull[buf]);
        umma_commit(&sh.empty[s]);
      }
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;  // sweeps 0/1: window row r; sweep 2: key slots r and r + 128
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const float LOG2E = 1.4426950408889634f;
    const int my_i = r / G;       // window index of row r
    float row_max = -INFINITY, row_m = 0.f, row_z = 0.f;
    T* out = reinterpret_cast<T*>(p.scores_out) + (int64_t)unit * p.NB * 256;
    // padded pages score exactly 0
    for (int pg = 0; pg < p.NB; ++pg)
      if (table[pg] == -1) { out[pg * 256 + r] = Elem<T>::from_f32(0.f); out[pg * 256 + 128 + r] = Elem<T>::from_f32(0.f); }
    for (int tt = 0; tt < ntiles; ++tt) {
      int sweep;
      const int pg = tile_page(tt, sweep);
      const bool last = table[pg] < -1;
      const int buf = tt & 1, u = tt >> 1;
      if (tt == nvalid) row_m = round_to<T>(row_max * p.scale);
      if (tt == 2 * nvalid) {
        sh.stats[r] = make_float2(row_m, 1.f / row_z);
        mbar_arrive(&sh.stats_ready);
        if (!mbar_wait(&sh.stats_ready, 0, abortp, p.error_word, 311)) break;
      }
      if (!mbar_wait(&sh.tfull[buf], u & 1, abortp, p.error_word, 312)) break;
      fence_after_sync();
      if (sweep < 2) {
        // columns = key slots; row r sees slot <= 256 - QCL + i inside the last page
        const int smax = last ? 256 - p.QCL + my_i : 256;
        for (int c = 0; c < 8; ++c) {
          float v[32];
          tmem_ld32(lane_base + buf * 256 + c * 32, v);
          const bool partial = c * 32 + 31 > smax;
          if (sweep == 0) {
            float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (partial) {
#pragma unroll
                for (int e = 0; e < 4; ++e) if (c * 32 + j + e > smax) v[j + e] = -INFINITY;
              }
              m0 = fmaxf(m0, v[j]); m1 = fmaxf(m1, v[j + 1]); m2 = fmaxf(m2, v[j + 2]); m3 = fmaxf(m3, v[j + 3]);
            }
            row_max = fmaxf(row_max, fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)));
          } else {
            float z0 = 0.f, z1 = 0.f, z2 = 0.f, z3 = 0.f;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float e4[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float lg = round_to<T>(v[j + e] * p.scale);
                e4[e] = ex2_approx(round_to<T>(lg - row_m) * LOG2E);
                if (partial && c * 32 + j + e > smax) e4[e] = 0.f;
              }
              z0 += e4[0]; z1 += e4[1]; z2 += e4[2]; z3 += e4[3];
            }
            row_z += (z0 + z1) + (z2 + z3);
          }
        }
      } else {
        // rows of D = key slots; columns = window rows j = i*G + g
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int slot = hh * 128 + r;
          const int jmask = last ? max(0, slot - (256 - p.QCL)) * G : 0;  // columns below are masked
          float acc = p.reduce_mode == 0 ? 0.f : -INFINITY;
          for (int c = 0; c * 32 < R; ++c) {
            float v[32];
            tmem_ld32(lane_base + buf * 256 + hh * 128 + c * 32, v);
            const float4* st4 = reinterpret_cast<const float4*>(&sh.stats[c * 32]);
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const float4 st = st4[j >> 1];
              const float l0 = round_to<T>(v[j] * p.scale), l1 = round_to<T>(v[j + 1] * p.scale);
              float p0 = round_to<T>(ex2_approx(round_to<T>(l0 - st.x) * LOG2E) * st.y);
              float p1 = round_to<T>(ex2_approx(round_to<T>(l1 - st.z) * LOG2E) * st.w);
              if (c * 32 + j < jmask) p0 = 0.f;
              if (c * 32 + j + 1 < jmask) p1 = 0.f;
              v[j] = p0; v[j + 1] = p1;
            }
            const int ncols = R - c * 32;
            const bool um = p.reduce_mode != 0;
            switch (G) {
              case 1: acc = group_reduce<1>(v, ncols, um, acc); break;
              case 2: acc = group_reduce<2>(v, ncols, um, acc); break;
              case 4: acc = group_reduce<4>(v, ncols, um, acc); break;
              case 8: acc = group_reduce<8>(v, ncols, um, acc); break;
              case 16: acc = group_reduce<16>(v, ncols, um, acc); break;
              default: acc = group_reduce<32>(v, ncols, um, acc); break;
            }
          }
          const float res = p.reduce_mode == 0 ? acc / (float)p.QCL : acc;
          out[pg * 256 + slot] = Elem<T>::from_f32(res);
        }
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.tempty[buf]);
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <typename T>
static int launch_window_tc(const void* k_cache, const void* q_cache, const WtParams& p,
                            int64_t k_stride_layer, int64_t k_stride_page, int64_t q_stride_layer,
                            int64_t q_stride_seq, cudaStream_t st) {
  CUtensorMap tmK, tmQ;
  const int G = p.Hq / p.Hkv;
  {
    const uint64_t pages = p.L > 1 ? (uint64_t)(k_stride_layer / k_stride_page) : (1ull << 30);
    const uint64_t dims[5] = {128, (uint64_t)p.Hkv, 256, pages, (uint64_t)p.L};
    const uint64_t strides[4] = {128, (uint64_t)p.Hkv * 128, (uint64_t)k_stride_page,
                                 (uint64_t)(p.L > 1 ? k_stride_layer : k_stride_page)};
    const uint32_t box[5] = {64, 1, 256, 1, 1};
    int rc = make_tensor_map_5d(&tmK, UmmaFmt<T>::tm, k_cache, dims, strides, box, sizeof(T));
    if (rc) return rc;
  }
  {
    const uint64_t seqs = p.L > 1 ? (uint64_t)(q_stride_layer / q_stride_seq) : (1ull << 30);
    const uint64_t dims[5] = {128, (uint64_t)p.Hq, (uint64_t)p.QCL, seqs, (uint64_t)p.L};
    const uint64_t strides[4] = {128, (uint64_t)p.Hq * 128, (uint64_t)q_stride_seq,
                                 (uint64_t)(p.L > 1 ? q_stride_layer : q_stride_seq)};
    const uint32_t box[5] = {64, (uint32_t)G, (uint32_t)p.QCL, 1, 1};
    int rc = make_tensor_map_5d(&tmQ, UmmaFmt<T>::tm, q_cache, dims, strides, box, sizeof(T));
    if (rc) return rc;
  }
  const size_t smem = WT_NS * WT_PAGE_BYTES + 2 * WT_QBLOCK_BYTES + sizeof(WtShared) + 1024;
  auto kern = window_score_tc_kernel<T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_error("zp_window_score(tcgen05): %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  kern<<<p.L * p.B * p.Hkv, WT_THREADS, smem, st>>>(tmK, tmQ, p);
  return check_launch("zp_window_score(tcgen05)");
}

// true when the tensor-core kernel covers these shapes
bool window_score_tc_supported(int dtype, int D, int BS, int Hq, int Hkv, int QCL, bool want_logits) {
  if (want_logits || !(dtype == ZP_DTYPE_BF16 || dtype == ZP_DTYPE_F16) || D != 128 || BS != 256) return false;
  const int G = Hq / Hkv;
  if (G < 1 || G > 32 || (G & (G - 1))) return false;
  const int R = G * QCL;
  return R <= 128 && R % 8 == 0 && QCL <= 256;
}

int window_score_tc(const void* k_cache, const void* q_cache, const int32_t* seq_idx,
                    const int32_t* block_table, void* scores_out, int L, int B, int NB, int Hq, int Hkv,
                    int QCL, int64_t k_stride_layer, int64_t k_stride_page, int64_t q_stride_layer,
                    int64_t q_stride_seq, float scale, int reduce_mode, int dtype, cudaStream_t st) {
  WtParams p;
  p.seq_idx = seq_idx; p.block_table = block_table; p.scores_out = scores_out;
  p.error_word = device_error_word();
  p.L = L; p.B = B; p.NB = NB; p.Hq = Hq; p.Hkv = Hkv; p.QCL = QCL; p.scale = scale;
  p.reduce_mode = reduce_mode;
  if (!p.error_word) { set_error("zp_window_score(tcgen05): no device error word"); return ZP_ERR_CUDA; }
  if (dtype == ZP_DTYPE_BF16)
    return launch_window_tc<__nv_bfloat16>(k_cache, q_cache, p, k_stride_layer, k_stride_page,
                                           q_stride_layer, q_stride_seq, st);
  return launch_window_tc<__half>(k_cache, q_cache, p, k_stride_layer, k_stride_page, q_stride_layer,
                                  q_stride_seq, st);
}

}  // namespace zp
