// Key-similarity redundancy on tcgen05 tensor cores (16-bit caches, head_dim 128, page size 256).
//
// S = K K^T is a dense contraction: the RAW key tiles (not normalised copies) are staged by TMA
// (128-byte swizzle, one 64 KB page = 256 keys x 128 dims per stage), multiplied with
// tcgen05.mma (M = 128 rows, N = 256 columns, K = 128) into fp32 accumulators in TMEM, and the
// cosine normalisation is applied in the epilogue: S[m,n] = acc[m,n] / (|k_m| |k_n|), with the
// norms computed from the same shared-memory tile and rounded to T as key_norm does.
//
// Roles (576 threads, persistent blocks, one per SM): warp 0 = TMA producer and TMEM owner,
// warp 1 = MMA issuer, warps 2-17 = epilogue (thread <-> TMEM lane <-> similarity row; the four
// warps of a lane quadrant split the 256 columns of an item in groups of 64).  A work item is
// (column page, row half h): 128 rows x 256 columns = 256 TMEM columns; the two halves alternate
// between the two halves of TMEM, so the MMA of one item overlaps the epilogue of the previous one.
//   lightning: a job is a unit; rows and columns are the same page (A = B tile).
//   exact:     a job is (unit, row page); the row page stays resident, every page streams by.
// Blocks walk over the jobs with a fixed stride, so the pipeline never drains between jobs.
// The epilogue keeps row-wise state only (row sum, last column above the threshold and its value);
// see zp_redundancy.cu for why that is enough.  The "subtract the exempted entries" step uses
// 64-bit fixed-point atomics (2^-32 units), so the result does not depend on execution order.
#include "zp_tc.cuh"

namespace zp {

using namespace tc;

constexpr int RT_THREADS = 576;
constexpr int RT_PAGE_BYTES = 65536;   // 256 keys x 128 dims x 2 bytes
constexpr int RT_BLOCK_BYTES = 32768;  // one 64-column block of a page
constexpr int RT_NBUF = 3;

struct RtParams {
  const int32_t* block_table;
  void* logits_out;
  float* rowsum;
  long long* sub;
  int* error_word;
  int L, B, NB, Hkv;
  float threshold, eps;
  int total_jobs;
};

struct __align__(16) RtShared {
  uint64_t full[RT_NBUF], empty[RT_NBUF], tfull[2], tempty[2], afull, aempty, sync_bar;
  alignas(16) float rn[2][256];     // 1 / |k| of the column page (double-buffered over pages)
  float nmin[2][8];                 // smallest |k| of each 32-column chunk of that page
  float s_sum[256];                 // combined row sums of a page (lightning)
  float pb_sum[4][256], pb_val[4][256];  // per column group partials of rows 0..255
  int pb_col[4][256];
  unsigned long long s_sub[256];    // fixed-point sums of exempted entries (lightning)
  uint32_t tmem_base;
  int abort_flag;
};

// sum of squares of one 128-element row of a swizzled [256][128] tile (two 64-column blocks)
template <typename T>
__device__ __forceinline__ float row_sumsq(const unsigned char* tile, int row) {
  float2 a0 = make_float2(0.f, 0.f), a1 = a0, a2 = a0, a3 = a0;
#pragma unroll
  for (int blk = 0; blk < 2; ++blk) {
    const unsigned char* base = tile + blk * RT_BLOCK_BYTES + row * 128;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int4 raw = *reinterpret_cast<const int4*>(base + ((c ^ (row & 7)) << 4));
      const typename Pair<T>::V* e = reinterpret_cast<const typename Pair<T>::V*>(&raw);
      const float2 f0 = Pair<T>::unpack(e[0]), f1 = Pair<T>::unpack(e[1]);
      const float2 f2 = Pair<T>::unpack(e[2]), f3 = Pair<T>::unpack(e[3]);
      ffma2(a0, f0, f0); ffma2(a1, f1, f1); ffma2(a2, f2, f2); ffma2(a3, f3, f3);
    }
  }
  return ((a0.x + a0.y) + (a1.x + a1.y)) + ((a2.x + a2.y) + (a3.x + a3.y));
}

template <typename T, bool EXACT>
__global__ void __launch_bounds__(RT_THREADS, 1)
redundancy_tc_kernel(const __grid_constant__ CUtensorMap tmK, const RtParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* bufs = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  RtShared& sh = *reinterpret_cast<RtShared*>(bufs + RT_NBUF * RT_PAGE_BYTES);
  constexpr int NS = EXACT ? 2 : 3;      // ring of streaming stages
  constexpr int RING0 = EXACT ? 1 : 0;   // buffer 0 holds the resident row page in the exact form
  auto stage_ptr = [&](int s) { return bufs + (RING0 + s) * RT_PAGE_BYTES; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < RT_NBUF; ++i) { mbar_init(&sh.full[i], 1); mbar_init(&sh.empty[i], 2); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sh.tfull[i], 1); mbar_init(&sh.tempty[i], 16); }
    mbar_init(&sh.afull, 1);
    mbar_init(&sh.aempty, 1);
    mbar_init(&sh.sync_bar, 16);  // one arrival per epilogue warp
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
  constexpr uint32_t IDESC = idesc_f16(UmmaFmt<T>::fmt, 128, 256);

  // job -> (unit, row page).  All roles walk the same job sequence; `t` counts column pages since
  // kernel start (stage and TMEM-buffer parity), `nj` counts the jobs that had work.
  struct Job {
    int unit, mp, h, b, l; const int32_t* table; bool valid;
    __device__ __forceinline__ Job(const RtParams& p, int job) {
      unit = EXACT ? job / p.NB : job;
      mp = EXACT ? job % p.NB : 0;
      h = unit % p.Hkv; b = (unit / p.Hkv) % p.B; l = unit / (p.Hkv * p.B);
      table = p.block_table + (int64_t)b * p.NB;
      valid = EXACT ? table[mp] != -1 : true;
    }
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      prefetch_tensormap(&tmK);
      int t = 0, nj = 0;
      bool ok = true;
      for (int job = blockIdx.x; ok && job < p.total_jobs; job += gridDim.x) {
        const Job jb(p, job);
        if (!jb.valid) continue;
        if (EXACT) {
          if (!mbar_wait<true>(&sh.aempty, (nj & 1) ^ 1, abortp, p.error_word, 100)) break;
          const int id = decode_page(jb.table[jb.mp]).id;
          mbar_arrive_expect_tx(&sh.afull, RT_PAGE_BYTES);
          tma_load_5d(bufs, &tmK, &sh.afull, 0, jb.h, 0, id, jb.l);
          tma_load_5d(bufs + RT_BLOCK_BYTES, &tmK, &sh.afull, 64, jb.h, 0, id, jb.l);
        }
        for (int pg = 0; pg < p.NB; ++pg) {
          const PageRef cp = decode_page(jb.table[pg]);
          if (!cp.valid) continue;
          const int s = t % NS, k = t / NS;
          if (!mbar_wait<true>(&sh.empty[s], (k & 1) ^ 1, abortp, p.error_word, 101)) { ok = false; break; }
          mbar_arrive_expect_tx(&sh.full[s], RT_PAGE_BYTES);
          tma_load_5d(stage_ptr(s), &tmK, &sh.full[s], 0, jb.h, 0, cp.id, jb.l);
          tma_load_5d(stage_ptr(s) + RT_BLOCK_BYTES, &tmK, &sh.full[s], 64, jb.h, 0, cp.id, jb.l);
          ++t;
        }
        ++nj;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int t = 0, nj = 0;
      bool ok = true;
      for (int job = blockIdx.x; ok && job < p.total_jobs; job += gridDim.x) {
        const Job jb(p, job);
        if (!jb.valid) continue;
        if (EXACT && !mbar_wait<true>(&sh.afull, nj & 1, abortp, p.error_word, 201)) break;
        for (int pg = 0; pg < p.NB; ++pg) {
          if (jb.table[pg] == -1) continue;
          const int s = t % NS, k = t / NS;
          if (!mbar_wait<true>(&sh.full[s], k & 1, abortp, p.error_word, 202)) { ok = false; break; }
          const uint32_t b_addr = smem_u32(stage_ptr(s));
          const uint32_t a_base = EXACT ? smem_u32(bufs) : b_addr;
          for (int hh = 0; hh < 2; ++hh) {
            if (!mbar_wait<true>(&sh.tempty[hh], (t & 1) ^ 1, abortp, p.error_word, 203)) { ok = false; break; }
            fence_after_sync();
            umma_k128(tmem_base + hh * 256, a_base + hh * 16384, RT_BLOCK_BYTES, b_addr, RT_BLOCK_BYTES, IDESC);
            umma_commit(&sh.tfull[hh]);
          }
          if (!ok) break;
          umma_commit(&sh.empty[s]);
          ++t;
        }
        if (EXACT && ok) umma_commit(&sh.aempty);  // the resident row page is no longer read
        ++nj;
      }
    }
  } else {
    // ---------------- epilogue ----------------
    // thread (grp, r): rows r (half 0) and r + 128 (half 1) of every item, columns grp*64 .. +63
    const int q = warp & 3;            // TMEM lane quadrant this warp may read
    const int grp = (warp - 2) >> 2;   // column group 0..3
    const int r = q * 32 + lane;
    const int myrow = (grp & 1) * 128 + r;   // row this thread normalises (groups 0,1) / writes
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + grp * 64;
    const float eps_t = round_to<T>(p.eps);
    uint32_t ph = 0;                   // phase of sync_bar (all epilogue warps in lock step)
    auto sync_epilogue = [&](int where) -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.sync_bar);
      const bool ok_ = mbar_wait(&sh.sync_bar, ph & 1, abortp, p.error_word, where);
      ++ph;
      return ok_;
    };
    int t = 0, nj = 0;
    bool ok = true;
    for (int job = blockIdx.x; ok && job < p.total_jobs; job += gridDim.x) {
      const Job jb(p, job);
      if (!jb.valid) continue;
      const int32_t* table = jb.table;
      float rsum[2] = {0.f, 0.f}, bval[2] = {0.f, 0.f}, rn_m[2] = {0.f, 0.f}, thr_m[2] = {0.f, 0.f};
      int bcol[2] = {-1, -1};
      if (EXACT) {
        if (!mbar_wait(&sh.afull, nj & 1, abortp, p.error_word, 301)) break;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const float nrm = fmaxf(round_to<T>(sqrtf(row_sumsq<T>(bufs, r + 128 * hh))), eps_t);
          rn_m[hh] = 1.f / nrm;
          thr_m[hh] = p.threshold * nrm;
        }
      }
      for (int pg = 0; pg < p.NB; ++pg) {
        if (table[pg] == -1) {
          if (!EXACT && grp < 2)  // padded page: logits -inf
            reinterpret_cast<T*>(p.logits_out)[((int64_t)jb.unit * p.NB + pg) * 256 + myrow] = Elem<T>::from_f32(-INFINITY);
          continue;
        }
        const int s = t % NS, k = t / NS;
        if (!mbar_wait(&sh.full[s], k & 1, abortp, p.error_word, 302)) { ok = false; break; }
        float* rn = sh.rn[t & 1];
        if (grp < 2) {   // a warp covers exactly one 32-column chunk of the page
          const float nrm = fmaxf(round_to<T>(sqrtf(row_sumsq<T>(stage_ptr(s), myrow))), eps_t);
          rn[myrow] = 1.f / nrm;
          float mn = nrm;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
          if (lane == 0) sh.nmin[t & 1][(grp & 1) * 4 + q] = mn;
          if (!EXACT) sh.s_sub[myrow] = 0ull;
        }
        if (!sync_epilogue(303)) { ok = false; break; }
        if (warp == 2 && lane == 0) mbar_arrive(&sh.empty[s]);  // the epilogue is done reading the stage
        if (!EXACT) {
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            rn_m[hh] = rn[r + 128 * hh]; thr_m[hh] = p.threshold / rn_m[hh];
            rsum[hh] = 0.f; bcol[hh] = -1; bval[hh] = 0.f;
          }
        }
        const bool diag_page = EXACT ? (pg == jb.mp) : true;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          if (!mbar_wait(&sh.tfull[hh], t & 1, abortp, p.error_word, 304)) { ok = false; break; }
          fence_after_sync();
          const uint32_t tbase = lane_base + hh * 256;
          float2 sa = make_float2(0.f, 0.f), sb = sa;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t raw[32];
            tmem_ld32_issue(tbase + c * 32, raw);
            tmem_ld32_wait(raw);
            if (c == 1) {  // every TMEM read of this item has landed in registers
              fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&sh.tempty[hh]);
            }
            const int cg = grp * 2 + c;  // chunk index within the 256 columns
            if (diag_page && cg == hh * 4 + q) {  // warp-uniform: the chunk that holds this warp's diagonal
#pragma unroll
              for (int j = 0; j < 32; ++j) raw[j] = (j == lane) ? 0u : raw[j];
            }
            // row sum: acc * (1/|k_n|) accumulated two columns at a time; threshold filter on the raw
            // accumulators: S > thr needs acc > thr * |k_m| * |k_n| >= thr * |k_m| * min|k_n|
            const float4* rn4 = reinterpret_cast<const float4*>(rn + cg * 32);
            float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 f = rn4[j];
              const float a0 = __uint_as_float(raw[4 * j]), a1 = __uint_as_float(raw[4 * j + 1]);
              const float a2 = __uint_as_float(raw[4 * j + 2]), a3 = __uint_as_float(raw[4 * j + 3]);
              ffma2(sa, make_float2(a0, a1), make_float2(f.x, f.y));
              ffma2(sb, make_float2(a2, a3), make_float2(f.z, f.w));
              m0 = fmax3(m0, a0, a1);
              m1 = fmax3(m1, a2, a3);
            }
            if (fmaxf(m0, m1) > thr_m[hh] * sh.nmin[t & 1][cg]) {  // rare: look at the normalised values
              const float* rnc = rn + cg * 32;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float v = __uint_as_float(raw[j]) * rnc[j];
                if (v > thr_m[hh]) { bcol[hh] = pg * 256 + cg * 32 + j; bval[hh] = v; }
              }
            }
          }
          const float s0 = sa.x, s1 = sa.y, s2 = sb.x, s3 = sb.y;
          rsum[hh] += (s0 + s1) + (s2 + s3);
        }
        if (!ok) break;
        if (!EXACT) {
          // page done: merge the four column groups, subtract the exempted entries, write the logits
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            sh.pb_sum[grp][r + 128 * hh] = rsum[hh]; sh.pb_col[grp][r + 128 * hh] = bcol[hh];
            sh.pb_val[grp][r + 128 * hh] = bval[hh];
          }
          if (!sync_epilogue(305)) { ok = false; break; }
          if (grp < 2) {
            const int row = myrow;
            float total = 0.f, bv = 0.f;
            int bc = -1;
#pragma unroll
            for (int g = 0; g < 4; ++g) {   // fixed order; higher column groups win
              total += sh.pb_sum[g][row];
              if (sh.pb_col[g][row] >= 0) { bc = sh.pb_col[g][row]; bv = sh.pb_val[g][row]; }
            }
            const float rnm = rn[row];
            sh.s_sum[row] = total * rnm;
            if (bc >= 0) {
              const long long fx = __float2ll_rn(bv * rnm * 4294967296.f);
              atomicAdd(&sh.s_sub[bc - pg * 256], (unsigned long long)fx);
            }
          }
          if (!sync_epilogue(306)) { ok = false; break; }
          if (grp < 2) {
            const float sub = (float)((double)(long long)sh.s_sub[myrow] * (1.0 / 4294967296.0));
            reinterpret_cast<T*>(p.logits_out)[((int64_t)jb.unit * p.NB + pg) * 256 + myrow] =
                Elem<T>::from_f32(sh.s_sum[myrow] - sub);
          }
        }
        ++t;
      }
      if (!ok) break;
      if (EXACT) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          sh.pb_sum[grp][r + 128 * hh] = rsum[hh]; sh.pb_col[grp][r + 128 * hh] = bcol[hh];
          sh.pb_val[grp][r + 128 * hh] = bval[hh];
        }
        if (!sync_epilogue(307)) break;
        if (grp < 2) {
          const int row = myrow;
          const int64_t base = (int64_t)jb.unit * p.NB * 256;
          float total = 0.f, bv = 0.f;
          int bc = -1;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            total += sh.pb_sum[g][row];
            if (sh.pb_col[g][row] >= 0) { bc = sh.pb_col[g][row]; bv = sh.pb_val[g][row]; }
          }
          const float rnm = grp == 0 ? rn_m[0] : rn_m[1];
          p.rowsum[base + jb.mp * 256 + row] = total * rnm;
          if (bc >= 0) {
            const long long fx = __float2ll_rn(bv * rnm * 4294967296.f);
            atomicAdd(reinterpret_cast<unsigned long long*>(p.sub + base + bc), (unsigned long long)fx);
          }
        }
        if (!sync_epilogue(308)) break;  // pb_* are free again
      }
      ++nj;
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
static int launch_redundancy_tc(const void* k_cache, const RtParams& p, int64_t k_stride_layer,
                                int64_t k_stride_page, bool exact, cudaStream_t st) {
  CUtensorMap tm;
  const uint64_t pages = p.L > 1 ? (uint64_t)(k_stride_layer / k_stride_page) : (1ull << 30);
  const uint64_t dims[5] = {128, (uint64_t)p.Hkv, 256, pages, (uint64_t)p.L};
  const uint64_t strides[4] = {128, (uint64_t)p.Hkv * 128, (uint64_t)k_stride_page,
                               (uint64_t)(p.L > 1 ? k_stride_layer : k_stride_page)};
  const uint32_t box[5] = {64, 1, 256, 1, 1};
  int rc = make_tensor_map_5d(&tm, UmmaFmt<T>::tm, k_cache, dims, strides, box, sizeof(T));
  if (rc) return rc;
  const size_t smem = RT_NBUF * RT_PAGE_BYTES + sizeof(RtShared) + 1024;
  const int units = p.L * p.B * p.Hkv;
  RtParams pp = p;
  pp.total_jobs = exact ? units * p.NB : units;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = pp.total_jobs < sms ? pp.total_jobs : sms;
  cudaError_t e;
  if (exact) {
    auto kern = redundancy_tc_kernel<T, true>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) kern<<<grid, RT_THREADS, smem, st>>>(tm, pp);
  } else {
    auto kern = redundancy_tc_kernel<T, false>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) kern<<<grid, RT_THREADS, smem, st>>>(tm, pp);
  }
  if (e != cudaSuccess) { set_error("zp_redundancy(tcgen05): %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  return check_launch("zp_redundancy(tcgen05)");
}

// Called by the C entry points in zp_redundancy.cu.
int redundancy_tc(const void* k_cache, const int32_t* block_table, void* logits_out, float* rowsum,
                  long long* sub, int L, int B, int NB, int Hkv, int64_t k_stride_layer,
                  int64_t k_stride_page, float threshold, float eps, int dtype, bool exact,
                  cudaStream_t st) {
  RtParams p;
  p.block_table = block_table; p.logits_out = logits_out; p.rowsum = rowsum; p.sub = sub;
  p.error_word = device_error_word();
  p.L = L; p.B = B; p.NB = NB; p.Hkv = Hkv; p.threshold = threshold; p.eps = eps;
  if (!p.error_word) { set_error("zp_redundancy(tcgen05): no device error word"); return ZP_ERR_CUDA; }
  if (dtype == ZP_DTYPE_BF16)
    return launch_redundancy_tc<__nv_bfloat16>(k_cache, p, k_stride_layer, k_stride_page, exact, st);
  if (dtype == ZP_DTYPE_F16)
    return launch_redundancy_tc<__half>(k_cache, p, k_stride_layer, k_stride_page, exact, st);
  set_error("zp_redundancy(tcgen05): 16-bit caches only");
  return ZP_ERR_UNSUPPORTED;
}

}  // namespace zp
