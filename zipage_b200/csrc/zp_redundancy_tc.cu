// Lightning (page-local) key-similarity redundancy on tcgen05 tensor cores
// (16-bit caches, head_dim 128, page size 256).
//
// S = K K^T is a dense contraction: the RAW key tiles (not normalised copies) are staged by TMA
// (128-byte swizzle, one 64 KB page = 256 keys x 128 dims per stage), multiplied with
// tcgen05.mma (M = 128 rows, N = 256 columns, K = 128) into fp32 accumulators in TMEM, and the
// cosine normalisation is applied in the epilogue: S[m,n] = acc[m,n] / (|k_m| |k_n|), with the
// norms computed from the same shared-memory tile and rounded to T as key_norm does.
//
// Roles (576 threads, persistent blocks, one per SM): warp 0 = TMA producer and TMEM owner,
// warp 1 = MMA issuer, warps 2-17 = two epilogue TEAMS of 8 warps.  Column pages alternate between
// the teams; a team owns one half of TMEM (256 columns).  A work item is (column page, row half h):
// 128 rows x 256 columns; thread <-> TMEM lane <-> similarity row, the two warps of a lane quadrant
// split the 256 columns.  While one team normalises / merges / writes a page, the other is in the
// middle of its items, so the phases of consecutive pages overlap and the tensor pipe is fed by
// whichever team has a free accumulator.
// A job is a unit; rows and columns are the same page (A = B tile).  Blocks walk over the jobs with
// a fixed stride, so the pipeline never drains between jobs.
// Per key the op needs the row sum and the LAST other key above the threshold with its similarity
// (see zp_redundancy.cu for why that is enough); both are per-thread row state here.  The
// "subtract the exempted entries" step uses 64-bit fixed-point atomics in shared memory (2^-32
// units), so the result does not depend on execution order.  The whole-sequence (exact) form has
// its own kernel in zp_redundancy_exact_tc.cu.
#include "zp_tc.cuh"

namespace zp {

using namespace tc;

constexpr int RT_THREADS = 576;
constexpr int RT_PAGE_BYTES = 65536;   // 256 keys x 128 dims x 2 bytes
constexpr int RT_BLOCK_BYTES = 32768;  // one 64-column block of a page
constexpr int RT_NS = 3;               // ring of page stages

struct RtParams {
  const int32_t* block_table;
  void* logits_out;
  int* error_word;
  int L, B, NB, Hkv;
  float threshold, eps;
  int total_jobs;
};

struct __align__(16) RtTeam {        // per epilogue team
  alignas(16) float rn[256];         // 1 / |k| of the team's current page
  float nmin[8];                     // smallest |k| of each 32-column chunk of that page
  float s_sum[256];                  // combined row sums of the page
  float pb_sum[2][256], pb_val[2][256];  // per column group partials of rows 0..255
  int pb_col[2][256];
  unsigned long long s_sub[256];     // fixed-point sums of exempted entries
};

struct __align__(16) RtShared {
  uint64_t full[RT_NS], empty[RT_NS], tfull[2], tempty[2], team_bar[2];
  RtTeam team[2];
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

template <typename T>
__global__ void __launch_bounds__(RT_THREADS, 1)
redundancy_tc_kernel(const __grid_constant__ CUtensorMap tmK, const RtParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* bufs = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  RtShared& sh = *reinterpret_cast<RtShared*>(bufs + RT_NS * RT_PAGE_BYTES);
  constexpr int NS = RT_NS;
  auto stage_ptr = [&](int s) { return bufs + s * RT_PAGE_BYTES; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    // a stage is released by the MMA commit and by the team that read it for the norms
    for (int i = 0; i < NS; ++i) { mbar_init(&sh.full[i], 1); mbar_init(&sh.empty[i], 2); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh.tfull[i], 1); mbar_init(&sh.tempty[i], 8);
      mbar_init(&sh.team_bar[i], 8);   // one arrival per warp of the team
    }
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

  // All roles walk the same job sequence; `t` counts pages since kernel start (stage ring
  // position; page t belongs to team t & 1).
  struct Job {
    int unit, h, l; const int32_t* table;
    __device__ __forceinline__ Job(const RtParams& p, int job) {
      unit = job;
      h = unit % p.Hkv;
      const int b = (unit / p.Hkv) % p.B;
      l = unit / (p.Hkv * p.B);
      table = p.block_table + (int64_t)b * p.NB;
    }
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      prefetch_tensormap(&tmK);
      int t = 0;
      bool ok = true;
      for (int job = blockIdx.x; ok && job < p.total_jobs; job += gridDim.x) {
        const Job jb(p, job);
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
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // Pages of a job are issued in pairs (one per team): both first halves, then both second
    // halves, so that each team's accumulator is refilled while the other team's is being read.
    if (lane == 0) {
      int t = 0;
      bool ok = true;
      auto issue = [&](int tt, int hh) -> bool {   // item (page tt, row half hh) into team tt & 1
        const int team = tt & 1, s = tt % NS;
        const int use = (tt >> 1) * 2 + hh;         // how often this team's accumulator was used before
        if (!mbar_wait<true>(&sh.tempty[team], (use & 1) ^ 1, abortp, p.error_word, 203)) return false;
        fence_after_sync();
        const uint32_t b_addr = smem_u32(stage_ptr(s));
        umma_k128(tmem_base + team * 256, b_addr + hh * 16384, RT_BLOCK_BYTES, b_addr, RT_BLOCK_BYTES, IDESC);
        umma_commit(&sh.tfull[team]);
        return true;
      };
      for (int job = blockIdx.x; ok && job < p.total_jobs; job += gridDim.x) {
        const Job jb(p, job);
        int nvalid = 0;
        for (int pg = 0; pg < p.NB; ++pg) nvalid += jb.table[pg] != -1;
        for (int i = 0; ok && i < nvalid; i += 2) {
          const int npair = min(2, nvalid - i);
          for (int j = 0; ok && j < npair; ++j) {
            const int tt = t + i + j, s = tt % NS, k = tt / NS;
            ok = mbar_wait<true>(&sh.full[s], k & 1, abortp, p.error_word, 202);
          }
          for (int hh = 0; ok && hh < 2; ++hh)
            for (int j = 0; ok && j < npair; ++j) {
              ok = issue(t + i + j, hh);
              // a stage is free as soon as the MMAs of its second half are done
              if (ok && hh == 1) umma_commit(&sh.empty[(t + i + j) % NS]);
            }
        }
        t += nvalid;
      }
    }
  } else {
    // ---------------- epilogue teams ----------------
    // thread (team, grp, r): rows r (half 0) and r + 128 (half 1) of the team's items, columns
    // grp*128 .. +127; during the norm / merge phases it owns row `myrow` of the page
    const int ew = warp - 2;
    const int team = ew >> 3;
    const int q = warp & 3;            // TMEM lane quadrant this warp may read
    const int grp = (ew >> 2) & 1;     // column group 0..1
    const int r = q * 32 + lane;
    const int myrow = grp * 128 + r;
    RtTeam& tm = sh.team[team];
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + team * 256 + grp * 128;
    const float eps_t = round_to<T>(p.eps);
    uint32_t ph_team = 0;
    auto sync_team = [&](int where) -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.team_bar[team]);
      const bool ok_ = mbar_wait<0>(&sh.team_bar[team], ph_team & 1, abortp, p.error_word, where);
      ++ph_team;
      return ok_;
    };
    int t = 0;
    bool ok = true;
    for (int job = blockIdx.x; ok && job < p.total_jobs; job += gridDim.x) {
      const Job jb(p, job);
      const int32_t* table = jb.table;
      for (int pg = 0; pg < p.NB; ++pg) {
        if (table[pg] == -1) {
          if (team == 0)  // padded page: logits -inf
            reinterpret_cast<T*>(p.logits_out)[((int64_t)jb.unit * p.NB + pg) * 256 + myrow] = Elem<T>::from_f32(-INFINITY);
          continue;
        }
        const int tt = t++;
        if ((tt & 1) != team) continue;   // the other team's page
        const int s = tt % NS, k = tt / NS;
        if (!mbar_wait<32>(&sh.full[s], k & 1, abortp, p.error_word, 302)) { ok = false; break; }
        {   // a warp covers exactly one 32-column chunk of the page
          const float nrm = fmaxf(round_to<T>(sqrtf(row_sumsq<T>(stage_ptr(s), myrow))), eps_t);
          tm.rn[myrow] = 1.f / nrm;
          float mn = nrm;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
          if (lane == 0) tm.nmin[grp * 4 + q] = mn;
          tm.s_sub[myrow] = 0ull;
        }
        if (!sync_team(303)) { ok = false; break; }
        if ((ew & 7) == 0 && lane == 0) mbar_arrive(&sh.empty[s]);  // the team is done reading the stage
        float rsum[2], bval[2], rn_m[2], thr_m[2];
        int bcol[2];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          rn_m[hh] = tm.rn[r + 128 * hh]; thr_m[hh] = p.threshold / rn_m[hh];
          rsum[hh] = 0.f; bcol[hh] = -1; bval[hh] = 0.f;
        }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int use = (tt >> 1) * 2 + hh;
          if (!mbar_wait<32>(&sh.tfull[team], use & 1, abortp, p.error_word, 304)) { ok = false; break; }
          fence_after_sync();
          float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t raw[32];
            tmem_ld32_issue(lane_base + c * 32, raw);
            tmem_ld32_wait(raw);
            if (c == 3) {  // every TMEM read of this item has landed in registers
              fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&sh.tempty[team]);
            }
            const int cg = grp * 4 + c;  // chunk index within the 256 columns
            if (cg == hh * 4 + q) {      // warp-uniform: the chunk that holds this warp's diagonal
#pragma unroll
              for (int j = 0; j < 32; ++j) raw[j] = (j == lane) ? 0u : raw[j];
            }
            // row sum: acc * (1/|k_n|) accumulated in four chains; and the threshold filter on the
            // raw accumulators: S > thr needs acc > thr * |k_m| * |k_n| >= thr * |k_m| * min|k_n|
            // (the bound is positive, and positive floats order like their bit patterns read as
            // signed integers while every negative float reads as a negative integer: the largest
            // positive accumulator, if there is one, is found with 3-input integer maxima)
            int m0 = 0, m1 = 0;
            const float4* rn4 = reinterpret_cast<const float4*>(tm.rn + cg * 32);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 f = rn4[j];
              const float a0 = __uint_as_float(raw[4 * j]), a1 = __uint_as_float(raw[4 * j + 1]);
              const float a2 = __uint_as_float(raw[4 * j + 2]), a3 = __uint_as_float(raw[4 * j + 3]);
              s0 = fmaf(a0, f.x, s0); s1 = fmaf(a1, f.y, s1);
              s2 = fmaf(a2, f.z, s2); s3 = fmaf(a3, f.w, s3);
              m0 = __vimax3_s32(m0, (int)raw[4 * j], (int)raw[4 * j + 1]);
              m1 = __vimax3_s32(m1, (int)raw[4 * j + 2], (int)raw[4 * j + 3]);
            }
            if (__int_as_float(max(m0, m1)) > thr_m[hh] * tm.nmin[cg]) {  // rare: look at the normalised values
              const float* rnc = tm.rn + cg * 32;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float v = __uint_as_float(raw[j]) * rnc[j];
                if (v > thr_m[hh]) { bcol[hh] = pg * 256 + cg * 32 + j; bval[hh] = v; }
              }
            }
          }
          rsum[hh] += (s0 + s1) + (s2 + s3);
        }
        if (!ok) break;
        // page done: merge the two column groups, subtract the exempted entries, write the logits
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          tm.pb_sum[grp][r + 128 * hh] = rsum[hh]; tm.pb_col[grp][r + 128 * hh] = bcol[hh];
          tm.pb_val[grp][r + 128 * hh] = bval[hh];
        }
        if (!sync_team(305)) { ok = false; break; }
        {
          const int row = myrow;
          const float total = tm.pb_sum[0][row] + tm.pb_sum[1][row];
          const int bc = tm.pb_col[1][row] >= 0 ? tm.pb_col[1][row] : tm.pb_col[0][row];  // upper columns win
          const float bv = tm.pb_col[1][row] >= 0 ? tm.pb_val[1][row] : tm.pb_val[0][row];
          const float rnm = tm.rn[row];
          tm.s_sum[row] = total * rnm;
          if (bc >= 0) {
            const long long fx = __float2ll_rn(bv * rnm * 4294967296.f);
            atomicAdd(&tm.s_sub[bc - pg * 256], (unsigned long long)fx);
          }
        }
        if (!sync_team(306)) { ok = false; break; }
        const float sub = (float)((double)(long long)tm.s_sub[myrow] * (1.0 / 4294967296.0));
        reinterpret_cast<T*>(p.logits_out)[((int64_t)jb.unit * p.NB + pg) * 256 + myrow] =
            Elem<T>::from_f32(tm.s_sum[myrow] - sub);
      }
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
                                int64_t k_stride_page, cudaStream_t st) {
  CUtensorMap tm;
  const uint64_t pages = p.L > 1 ? (uint64_t)(k_stride_layer / k_stride_page) : (1ull << 30);
  const uint64_t dims[5] = {128, (uint64_t)p.Hkv, 256, pages, (uint64_t)p.L};
  const uint64_t strides[4] = {128, (uint64_t)p.Hkv * 128, (uint64_t)k_stride_page,
                               (uint64_t)(p.L > 1 ? k_stride_layer : k_stride_page)};
  const uint32_t box[5] = {64, 1, 256, 1, 1};
  int rc = make_tensor_map_5d(&tm, UmmaFmt<T>::tm, k_cache, dims, strides, box, sizeof(T));
  if (rc) return rc;
  const size_t smem = RT_NS * RT_PAGE_BYTES + sizeof(RtShared) + 1024;
  RtParams pp = p;
  pp.total_jobs = p.L * p.B * p.Hkv;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = pp.total_jobs < sms ? pp.total_jobs : sms;
  auto kern = redundancy_tc_kernel<T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_error("zp_redundancy_lightning(tcgen05): %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  kern<<<grid, RT_THREADS, smem, st>>>(tm, pp);
  return check_launch("zp_redundancy_lightning(tcgen05)");
}

// Called by zp_redundancy_lightning (zp_redundancy.cu).
int redundancy_tc(const void* k_cache, const int32_t* block_table, void* logits_out, int L, int B,
                  int NB, int Hkv, int64_t k_stride_layer, int64_t k_stride_page, float threshold,
                  float eps, int dtype, cudaStream_t st) {
  RtParams p{};
  p.block_table = block_table; p.logits_out = logits_out;
  p.error_word = device_error_word();
  p.L = L; p.B = B; p.NB = NB; p.Hkv = Hkv; p.threshold = threshold; p.eps = eps;
  if (!p.error_word) { set_error("zp_redundancy_lightning(tcgen05): no device error word"); return ZP_ERR_CUDA; }
  if (dtype == ZP_DTYPE_BF16)
    return launch_redundancy_tc<__nv_bfloat16>(k_cache, p, k_stride_layer, k_stride_page, st);
  if (dtype == ZP_DTYPE_F16)
    return launch_redundancy_tc<__half>(k_cache, p, k_stride_layer, k_stride_page, st);
  set_error("zp_redundancy_lightning(tcgen05): 16-bit caches only");
  return ZP_ERR_UNSUPPORTED;
}

}  // namespace zp
