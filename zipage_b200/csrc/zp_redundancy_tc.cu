// Key-similarity redundancy on tcgen05 tensor cores (16-bit caches, head_dim 128, page size 256).
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
//   lightning: a job is a unit; rows and columns are the same page (A = B tile).
//   exact:     a job is (unit, row page I); the row page stays resident and the column pages
//              J >= I stream by.  S is symmetric, so the tiles below the diagonal are never
//              computed: an entry (m, n) above the threshold found in tile (I, J) is recorded for
//              key m and, when J > I, for key n as well.
// Blocks walk over the jobs with a fixed stride, so the pipeline never drains between jobs.
// Exact form, row sums without touching every element: sum_n S[m,n] = (k_m / |k_m|) . w with
// w = sum_n k_n / |k_n|, a vector a small pre-pass (key_stats_kernel) computes once per unit together
// with the norms.  The epilogue then only has to FIND entries above the threshold: a 3-input max
// over the raw accumulators against the bound thr * |k_m| * min|k_n| of the 32-column chunk, and a
// look at the normalised values only where that bound is exceeded.  That leaves the kernel bound
// by the tensor pipe instead of by epilogue instruction issue.
// Per key the op needs the row sum and the LAST other key above the threshold with its similarity
// (see zp_redundancy.cu for why that is enough).  The lightning form keeps both as per-thread row
// state; the exact form records the latter with a 64-bit atomicMax on (index + 1) << 32 | value
// bits, which a small kernel afterwards turns into the "subtract the exempted entries" sums.  Those
// sums use 64-bit fixed-point atomics (2^-32 units), so the result does not depend on execution
// order.
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
  // exact form: per-key statistics from key_stats_kernel
  const float* rn;     // [units][NB*256]  1 / |k|
  const float* dself;  // [units][NB*256]  the key's similarity with itself (the zeroed diagonal)
  const float* nmin;   // [units][NB*8]    smallest |k| of each 32-key chunk
  const float* wvec;   // [units][128]     sum over the sequence of k / |k|
  unsigned long long* best;  // [units][NB*256] exact form: latest similar key, packed; zeroed
};

struct __align__(16) RtTeam {        // per epilogue team
  alignas(16) float rn[256];         // 1 / |k| of the team's current column page
  float nmin[8];                     // smallest |k| of each 32-column chunk of that page
  float s_sum[256];                  // combined row sums of the page (lightning)
  float pb_sum[2][256], pb_val[2][256];  // per column group partials of rows 0..255
  int pb_col[2][256];
  unsigned long long s_sub[256];     // fixed-point sums of exempted entries (lightning)
};

struct __align__(16) RtShared {
  uint64_t full[RT_NBUF], empty[RT_NBUF], tfull[2], tempty[2], afull, aempty, team_bar[2];
  RtTeam team[2];
  alignas(16) float wv[128];         // exact form: the unit's sum of normalised keys
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
    // a stage is released by the MMA commit and, in the lightning form, by the team that read it
    for (int i = 0; i < RT_NBUF; ++i) { mbar_init(&sh.full[i], 1); mbar_init(&sh.empty[i], EXACT ? 1 : 2); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh.tfull[i], 1); mbar_init(&sh.tempty[i], 8);
      mbar_init(&sh.team_bar[i], 8);   // one arrival per warp of the team
    }
    mbar_init(&sh.afull, 1);
    mbar_init(&sh.aempty, 2);  // MMA commit + the epilogue's row-sum pass over the resident page
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
  // kernel start (stage ring position; page t belongs to team t & 1), `nj` counts jobs with work.
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
        for (int pg = EXACT ? jb.mp : 0; pg < p.NB; ++pg) {
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
    // Pages of a job are issued in pairs (one per team): both first halves, then both second
    // halves, so that each team's accumulator is refilled while the other team's is being read.
    if (lane == 0) {
      int t = 0, nj = 0;
      bool ok = true;
      auto issue = [&](int tt, int hh) -> bool {   // item (page tt, row half hh) into team tt & 1
        const int team = tt & 1, s = tt % NS;
        const int use = (tt >> 1) * 2 + hh;         // how often this team's accumulator was used before
        if (!mbar_wait<true>(&sh.tempty[team], (use & 1) ^ 1, abortp, p.error_word, 203)) return false;
        fence_after_sync();
        const uint32_t b_addr = smem_u32(stage_ptr(s));
        const uint32_t a_base = EXACT ? smem_u32(bufs) : b_addr;
        umma_k128(tmem_base + team * 256, a_base + hh * 16384, RT_BLOCK_BYTES, b_addr, RT_BLOCK_BYTES, IDESC);
        umma_commit(&sh.tfull[team]);
        return true;
      };
      for (int job = blockIdx.x; ok && job < p.total_jobs; job += gridDim.x) {
        const Job jb(p, job);
        if (!jb.valid) continue;
        if (EXACT && !mbar_wait<true>(&sh.afull, nj & 1, abortp, p.error_word, 201)) break;
        int nvalid = 0;
        for (int pg = EXACT ? jb.mp : 0; pg < p.NB; ++pg) nvalid += jb.table[pg] != -1;
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
        if (EXACT && ok) umma_commit(&sh.aempty);  // the resident row page is no longer read
        ++nj;
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
      const bool ok_ = mbar_wait(&sh.team_bar[team], ph_team & 1, abortp, p.error_word, where);
      ++ph_team;
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
      const int64_t ubase = (int64_t)jb.unit * p.NB * 256;
      if (EXACT) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          rn_m[hh] = p.rn[ubase + jb.mp * 256 + r + 128 * hh];
          thr_m[hh] = p.threshold / rn_m[hh];
        }
      }
      for (int pg = EXACT ? jb.mp : 0; pg < p.NB; ++pg) {
        if (table[pg] == -1) {
          if (!EXACT && team == 0)  // padded page: logits -inf
            reinterpret_cast<T*>(p.logits_out)[((int64_t)jb.unit * p.NB + pg) * 256 + myrow] = Elem<T>::from_f32(-INFINITY);
          continue;
        }
        const int tt = t++;
        if ((tt & 1) != team) continue;   // the other team's page
        const int s = tt % NS, k = tt / NS;
        float nm[4] = {0.f, 0.f, 0.f, 0.f};   // exact form: smallest |k| of this thread's four chunks
        if (EXACT) {
#pragma unroll
          for (int c = 0; c < 4; ++c) nm[c] = p.nmin[(int64_t)jb.unit * p.NB * 8 + pg * 8 + grp * 4 + c];
        } else {
          if (!mbar_wait(&sh.full[s], k & 1, abortp, p.error_word, 302)) { ok = false; break; }
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
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            rn_m[hh] = tm.rn[r + 128 * hh]; thr_m[hh] = p.threshold / rn_m[hh];
            rsum[hh] = 0.f; bcol[hh] = -1; bval[hh] = 0.f;
          }
        }
        const bool diag_page = EXACT ? (pg == jb.mp) : true;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int use = (tt >> 1) * 2 + hh;
          if (!mbar_wait(&sh.tfull[team], use & 1, abortp, p.error_word, 304)) { ok = false; break; }
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
            if (diag_page && cg == hh * 4 + q) {  // warp-uniform: the chunk that holds this warp's diagonal
#pragma unroll
              for (int j = 0; j < 32; ++j) raw[j] = (j == lane) ? 0u : raw[j];
            }
            // threshold filter on the raw accumulators: S > thr needs
            // acc > thr * |k_m| * |k_n| >= thr * |k_m| * min|k_n|
            float m0 = -INFINITY, m1 = -INFINITY;
            if (EXACT) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                m0 = fmax3(m0, __uint_as_float(raw[4 * j]), __uint_as_float(raw[4 * j + 1]));
                m1 = fmax3(m1, __uint_as_float(raw[4 * j + 2]), __uint_as_float(raw[4 * j + 3]));
              }
              if (fmaxf(m0, m1) > thr_m[hh] * nm[c]) {  // look at the normalised values
                const float* rnc = p.rn + ubase + pg * 256 + cg * 32;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  const float v = __uint_as_float(raw[j]) * rnc[j];
                  if (v > thr_m[hh]) {
                    const unsigned m_key = jb.mp * 256 + r + 128 * hh, n_key = pg * 256 + cg * 32 + j;
                    const unsigned long long bits = __float_as_uint(v * rn_m[hh]);
                    atomicMax(p.best + ubase + m_key, ((unsigned long long)(n_key + 1) << 32) | bits);
                    if (!diag_page)  // the mirrored entry of the tile that is not computed
                      atomicMax(p.best + ubase + n_key, ((unsigned long long)(m_key + 1) << 32) | bits);
                  }
                }
              }
            } else {
              // row sum: acc * (1/|k_n|) accumulated in four chains
              const float4* rn4 = reinterpret_cast<const float4*>(tm.rn + cg * 32);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 f = rn4[j];
                const float a0 = __uint_as_float(raw[4 * j]), a1 = __uint_as_float(raw[4 * j + 1]);
                const float a2 = __uint_as_float(raw[4 * j + 2]), a3 = __uint_as_float(raw[4 * j + 3]);
                s0 = fmaf(a0, f.x, s0); s1 = fmaf(a1, f.y, s1);
                s2 = fmaf(a2, f.z, s2); s3 = fmaf(a3, f.w, s3);
                m0 = fmax3(m0, a0, a1);
                m1 = fmax3(m1, a2, a3);
              }
              if (fmaxf(m0, m1) > thr_m[hh] * tm.nmin[cg]) {  // rare: look at the normalised values
                const float* rnc = tm.rn + cg * 32;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  const float v = __uint_as_float(raw[j]) * rnc[j];
                  if (v > thr_m[hh]) { bcol[hh] = pg * 256 + cg * 32 + j; bval[hh] = v; }
                }
              }
            }
          }
          rsum[hh] += (s0 + s1) + (s2 + s3);
        }
        if (!ok) break;
        if (!EXACT) {
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
      if (!ok) break;
      if (EXACT && team == 0) {
        // job done: the row sums from the linear form  sum_n S[m,n] = rn_m * (k_m . w) - S[m,m]
        if (myrow < 128) sh.wv[myrow] = p.wvec[(int64_t)jb.unit * 128 + myrow];
        if (!mbar_wait(&sh.afull, nj & 1, abortp, p.error_word, 301)) break;  // (long since complete)
        if (!sync_team(307)) break;
        {
          const int row = myrow;
          float d0 = 0.f, d1 = 0.f;   // k_m . w over the resident (swizzled) row page
#pragma unroll
          for (int blk = 0; blk < 2; ++blk) {
            const unsigned char* base = bufs + blk * RT_BLOCK_BYTES + row * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const int4 rawk = *reinterpret_cast<const int4*>(base + ((c ^ (row & 7)) << 4));
              const typename Pair<T>::V* e = reinterpret_cast<const typename Pair<T>::V*>(&rawk);
              const float4 wa = *reinterpret_cast<const float4*>(&sh.wv[blk * 64 + c * 8]);
              const float4 wb = *reinterpret_cast<const float4*>(&sh.wv[blk * 64 + c * 8 + 4]);
              const float2 f0 = Pair<T>::unpack(e[0]), f1 = Pair<T>::unpack(e[1]);
              const float2 f2 = Pair<T>::unpack(e[2]), f3 = Pair<T>::unpack(e[3]);
              d0 = fmaf(f0.x, wa.x, d0); d1 = fmaf(f0.y, wa.y, d1);
              d0 = fmaf(f1.x, wa.z, d0); d1 = fmaf(f1.y, wa.w, d1);
              d0 = fmaf(f2.x, wb.x, d0); d1 = fmaf(f2.y, wb.y, d1);
              d0 = fmaf(f3.x, wb.z, d0); d1 = fmaf(f3.y, wb.w, d1);
            }
          }
          const float rnm = grp == 0 ? rn_m[0] : rn_m[1];
          p.rowsum[ubase + jb.mp * 256 + row] = rnm * (d0 + d1) - p.dself[ubase + jb.mp * 256 + row];
        }
        if (!sync_team(308)) break;  // wv and the resident page are free again
        if (ew == 0 && lane == 0) mbar_arrive(&sh.aempty);
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

// Pre-pass of the exact form: per key 1/|k| (the norm rounded to T as key_norm does) and the key's
// similarity with itself, per 32-key chunk the smallest norm, per unit w = sum_n k_n / |k_n| in
// fp32.  One block per unit walks the unit's pages in order (a fixed summation order); a warp owns
// one 32-key chunk of each page, a lane four of the 128 dims.
template <typename T>
__global__ void __launch_bounds__(256)
key_stats_kernel(const T* __restrict__ k_cache, const int32_t* __restrict__ block_table,
                 float* __restrict__ rn, float* __restrict__ dself, float* __restrict__ nmin,
                 float* __restrict__ wvec, int B, int NB, int Hkv, int64_t k_stride_layer,
                 int64_t k_stride_page, float eps) {
  __shared__ float part[8][128];
  const int unit = blockIdx.x;
  const int h = unit % Hkv, b = (unit / Hkv) % B, l = unit / (Hkv * B);
  const int lane = threadIdx.x & 31, wv = threadIdx.x >> 5;
  const float eps_t = round_to<T>(eps);
  float w0 = 0.f, w1 = 0.f, w2 = 0.f, w3 = 0.f;
  for (int pg = 0; pg < NB; ++pg) {
    const PageRef pr = decode_page(block_table[(int64_t)b * NB + pg]);
    if (!pr.valid) continue;
    const T* kp = k_cache + (int64_t)l * k_stride_layer + (int64_t)pr.id * k_stride_page +
                  ((int64_t)(wv * 32) * Hkv + h) * 128 + lane * 4;
    float my_rn = 0.f, my_ds = 0.f, mn = INFINITY;
#pragma unroll 1
    for (int r0 = 0; r0 < 32; r0 += 8) {
      uint2 raw[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        raw[j] = *reinterpret_cast<const uint2*>(kp + (int64_t)(r0 + j) * Hkv * 128);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 a = Pair<T>::unpack(*reinterpret_cast<const typename Pair<T>::V*>(&raw[j].x));
        const float2 c = Pair<T>::unpack(*reinterpret_cast<const typename Pair<T>::V*>(&raw[j].y));
        const float ss = warp_sum(fmaf(a.x, a.x, a.y * a.y) + fmaf(c.x, c.x, c.y * c.y));
        const float nrm = fmaxf(round_to<T>(sqrtf(ss)), eps_t);
        const float rnv = 1.f / nrm;
        w0 = fmaf(rnv, a.x, w0); w1 = fmaf(rnv, a.y, w1);
        w2 = fmaf(rnv, c.x, w2); w3 = fmaf(rnv, c.y, w3);
        if (lane == r0 + j) { my_rn = rnv; my_ds = rnv * rnv * ss; }
        mn = fminf(mn, nrm);
      }
    }
    const int64_t idx = ((int64_t)unit * NB + pg) * 256 + wv * 32 + lane;
    rn[idx] = my_rn;
    dself[idx] = my_ds;
    if (lane == 0) nmin[((int64_t)unit * NB + pg) * 8 + wv] = mn;
  }
  *reinterpret_cast<float4*>(&part[wv][lane * 4]) = make_float4(w0, w1, w2, w3);
  __syncthreads();
  if (threadIdx.x < 128) {
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += part[i][threadIdx.x];
    wvec[(int64_t)unit * 128 + threadIdx.x] = acc;
  }
}

// exact form: key i's latest similar key y = c(i) loses S[i, y] from its row sum
__global__ void exempt_scatter_kernel(const unsigned long long* __restrict__ best,
                                      long long* __restrict__ sub, int N, int64_t total) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const unsigned long long bq = best[i];
  if (!bq) return;
  const int64_t y = (int64_t)(bq >> 32) - 1;
  const long long fx = __float2ll_rn(__uint_as_float((unsigned)bq) * 4294967296.f);
  atomicAdd(reinterpret_cast<unsigned long long*>(sub + (i / N) * N + y), (unsigned long long)fx);
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
    key_stats_kernel<T><<<units, 256, 0, st>>>(
        reinterpret_cast<const T*>(k_cache), p.block_table, const_cast<float*>(p.rn),
        const_cast<float*>(p.dself), const_cast<float*>(p.nmin), const_cast<float*>(p.wvec), p.B, p.NB,
        p.Hkv, k_stride_layer, k_stride_page, p.eps);
    auto kern = redundancy_tc_kernel<T, true>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) {
      kern<<<grid, RT_THREADS, smem, st>>>(tm, pp);
      const int64_t total = (int64_t)units * p.NB * 256;
      exempt_scatter_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(p.best, p.sub, p.NB * 256, total);
    }
  } else {
    auto kern = redundancy_tc_kernel<T, false>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) kern<<<grid, RT_THREADS, smem, st>>>(tm, pp);
  }
  if (e != cudaSuccess) { set_error("zp_redundancy(tcgen05): %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  return check_launch("zp_redundancy(tcgen05)");
}

// Called by the C entry points in zp_redundancy.cu.
// Exact form: `sub` holds 2*n zeroed 64-bit words (the subtrahends, then the latest-similar-key
// records), `stats` 2*n + units*(NB*8 + 128) floats of scratch, n = units*NB*256.
int redundancy_tc(const void* k_cache, const int32_t* block_table, void* logits_out, float* rowsum,
                  long long* sub, float* stats, int L, int B, int NB, int Hkv, int64_t k_stride_layer,
                  int64_t k_stride_page, float threshold, float eps, int dtype, bool exact,
                  cudaStream_t st) {
  RtParams p;
  const size_t units_ = (size_t)L * B * Hkv, n_ = units_ * NB * 256;
  p.best = reinterpret_cast<unsigned long long*>(sub) + n_;  // zeroed together with `sub`
  p.rn = stats; p.dself = stats + n_; p.nmin = stats + 2 * n_; p.wvec = stats + 2 * n_ + units_ * NB * 8;
  if (exact && !stats) { set_error("zp_redundancy(tcgen05): no scratch for the key statistics"); return ZP_ERR_WORKSPACE; }
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
