// Exact (whole-sequence) key-similarity redundancy on tcgen05 tensor cores
// (16-bit caches, head_dim 128, page size 256).
//
// S = K K^T over the N = NB*256 keys of a unit is symmetric, so only the page tiles (I, J) with
// J >= I are computed.  What the op needs per key m is
//   * the row sum  sum_n S[m,n]  (diagonal excluded), and
//   * the LAST other key n with S[m,n] above the threshold, with that similarity.
// The row sum is linear in the normalised keys:  sum_n S[m,n] = (k_m / |k_m|) . w - S[m,m]  with
// w = sum_n k_n / |k_n|; a pre-pass (key_stats_kernel) computes the norms (rounded to T as key_norm
// does), w and S[m,m] once per unit.  The tensor-core pass then only has to FIND entries above the
// threshold: a 3-input max over the raw fp32 accumulators against the bound
// thr * |k_m| * min|k_n| of a 32-column chunk, and a look at the normalised values only where that
// bound is exceeded.  A hit (m, n) is recorded for key m and, off the diagonal page, for key n
// (the mirrored entry that is never computed) with a 64-bit atomicMax on (index + 1) << 32 | value
// bits; a small kernel afterwards turns the records into the "subtract the exempted entries" sums
// (64-bit fixed point, 2^-32 units, so the result does not depend on execution order).
//
// Tiling: a job is (unit, row page I).  The row page (256 keys, 64 KB) is the A operand of two
// row groups of 128; the column pages J >= I stream by as B operands (M = 128, N = 256, K = 128
// per item, the shape that keeps the tensor pipe at its full rate).  Shared memory holds three
// page slots that rotate between the two uses: the slots are handed out in the order in which
// they are released (a column page once its products are issued, the row page at the end of its
// job), so the next job's row page is fetched while the current job's last column pages are
// still being multiplied and the pipe never waits for an operand at a job boundary.  Every role
// replays the same hand-out order from the job sequence alone (SlotFifo).
// Roles (640 threads, persistent blocks, one per SM): warp 0 = TMA producer and TMEM owner,
// warp 1 = MMA issuer, warps 18-19 = row sums (the k_m . w products, read from the resident row
// page while the tensor pipe works on it), warps 2-17 = two epilogue teams of eight warps.  Team g owns
// row group g and its 256-column accumulator in TMEM (thread <-> TMEM lane <-> similarity row,
// the two warps of a lane quadrant split the 256 columns), so one team reads its accumulator
// while the tensor pipe fills the other's.
#include "zp_tc.cuh"

namespace zp {

using namespace tc;

constexpr int XT_THREADS = 640;
constexpr int XT_PAGE_BYTES = 65536;    // 256 keys x 128 dims x 2 bytes
constexpr int XT_BLOCK_BYTES = 32768;   // one 64-dim block of a page
constexpr int XT_NSLOT = 3;

struct XtParams {
  const int32_t* block_table;
  float* rowsum;               // [units][NB*256]  k_m . w (the caller's finalize kernel scales it)
  unsigned long long* best;    // [units][NB*256] latest similar key, packed; zeroed before the launch
  int* error_word;
  int L, B, NB, Hkv;
  float threshold;
  int total_jobs;
  const float* rn;             // [units][NB*256]  1 / |k|
  const float* dself;          // [units][NB*256]  the key's similarity with itself
  const float* nmin;           // [units][NB*8]    smallest |k| of each 32-key chunk
  const float* wvec;           // [units][128]     sum over the sequence of k / |k|
};

struct __align__(16) XtShared {
  uint64_t full[XT_NSLOT], empty[XT_NSLOT], tfull[2], tempty[2], adone[2], aready[2];
  uint32_t tmem_base;
  int abort_flag;
};

// The three page slots in the order in which they become free.  pop() = the slot the next load
// goes to; a column page's slot is pushed back at once (it is released as soon as its products are
// issued), a row page's slot at the end of its job.  use() keeps the parity of the number of loads
// into each slot (the mbarrier phase).  One register: bits 0-5 the queue (2 bits per entry), bits
// 6-7 its length, bits 8-10 the parities.
struct SlotFifo {
  uint32_t st = 0u | (1u << 2) | (2u << 4) | (3u << 6);
  __device__ __forceinline__ int pop() {
    const int s = st & 3u;
    const uint32_t n = (st >> 6) & 3u;
    st = (st & ~0xFFu) | ((st >> 2) & 0xFu) | ((n - 1) << 6);
    return s;
  }
  __device__ __forceinline__ void push(int s) {
    const uint32_t n = (st >> 6) & 3u;
    st = (st & ~(0xC0u | (3u << (2 * n)))) | (static_cast<uint32_t>(s) << (2 * n)) | ((n + 1) << 6);
  }
  // call once per load into slot s; returns the parity of the number of earlier loads into it
  __device__ __forceinline__ uint32_t use(int s) {
    const uint32_t u = (st >> (8 + s)) & 1u;
    st ^= 1u << (8 + s);
    return u;
  }
};

// Pre-pass: per key 1/|k| and the key's similarity with itself, per 32-key chunk the smallest norm,
// per unit w = sum_n k_n / |k_n| in fp32.  One block per unit walks the unit's pages in order (a
// fixed summation order); a warp owns one 32-key chunk of each page, a lane four of the 128 dims.
template <typename T>
__global__ void __launch_bounds__(256, 4)
key_stats_kernel(const T* __restrict__ k_cache, const int32_t* __restrict__ block_table,
                 float* __restrict__ rn, float* __restrict__ dself, float* __restrict__ nmin,
                 float* __restrict__ wvec, int B, int NB, int Hkv, int64_t k_stride_layer,
                 int64_t k_stride_page, float eps) {
  __shared__ float part[8][128];
  const int unit = blockIdx.x;
  const int h = unit % Hkv, b = (unit / Hkv) % B, l = unit / (Hkv * B);
  const int lane = threadIdx.x & 31, wv = threadIdx.x >> 5;
  const float eps_t = round_to<T>(eps);
  // after the folding below a lane holds the sum of squares of row `myr` of each group of 8 rows
  const int myr = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
  float w0 = 0.f, w1 = 0.f, w2 = 0.f, w3 = 0.f;
  for (int pg = 0; pg < NB; ++pg) {
    const PageRef pr = decode_page(block_table[(int64_t)b * NB + pg]);
    if (!pr.valid) continue;
    const T* kp = k_cache + (int64_t)l * k_stride_layer + (int64_t)pr.id * k_stride_page +
                  ((int64_t)(wv * 32) * Hkv + h) * 128 + lane * 4;
    float mn = INFINITY;
    const int64_t kbase = ((int64_t)unit * NB + pg) * 256 + wv * 32;
#pragma unroll 1
    for (int r0 = 0; r0 < 32; r0 += 8) {
      uint2 raw[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        raw[j] = *reinterpret_cast<const uint2*>(kp + (int64_t)(r0 + j) * Hkv * 128);
      float2 a[8], c[8];
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        a[j] = Pair<T>::unpack(*reinterpret_cast<const typename Pair<T>::V*>(&raw[j].x));
        c[j] = Pair<T>::unpack(*reinterpret_cast<const typename Pair<T>::V*>(&raw[j].y));
        v[j] = fmaf(a[j].x, a[j].x, a[j].y * a[j].y) + fmaf(c[j].x, c[j].x, c[j].y * c[j].y);
      }
      // transposed reduction: 8 values x 32 lanes -> one row total per lane (9 shuffles)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float send = b4 ? v[i] : v[i + 4], keep = b4 ? v[i + 4] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float send = b3 ? v[i] : v[i + 2], keep = b3 ? v[i + 2] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
      }
      {
        const float send = b2 ? v[0] : v[1], keep = b2 ? v[1] : v[0];
        v[0] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
      }
      float ss = v[0];
      ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      const float nrm = fmaxf(round_to<T>(sqrtf(ss)), eps_t);
      const float rnv = 1.f / nrm;
      mn = fminf(mn, nrm);
      if ((lane & 3) == 0) {
        rn[kbase + r0 + myr] = rnv;
        dself[kbase + r0 + myr] = rnv * rnv * ss;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float rj = __shfl_sync(0xffffffffu, rnv, ((j >> 2) & 1) * 16 + ((j >> 1) & 1) * 8 + (j & 1) * 4);
        w0 = fmaf(rj, a[j].x, w0); w1 = fmaf(rj, a[j].y, w1);
        w2 = fmaf(rj, c[j].x, w2); w3 = fmaf(rj, c[j].y, w3);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
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

// key i's latest similar key y = c(i) loses S[i, y] from its row sum
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
__global__ void __launch_bounds__(XT_THREADS, 1)
redundancy_exact_tc_kernel(const __grid_constant__ CUtensorMap tmK, const XtParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* bufs = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  XtShared& sh = *reinterpret_cast<XtShared*>(bufs + XT_NSLOT * XT_PAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < XT_NSLOT; ++i) { mbar_init(&sh.full[i], 1); mbar_init(&sh.empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sh.tfull[i], 1); mbar_init(&sh.tempty[i], 8); }
    // the two row-sum warps are done reading the row page; by job parity (two barriers, so that a waiter
    // one job behind can never see the phase it waits for wrap around)
    mbar_init(&sh.adone[0], 2);
    mbar_init(&sh.adone[1], 2);
    // the job's row page has landed (MMA issuer -> row-sum warp), by job parity as well.  The
    // row-sum warp cannot use full[] itself: it does not wait for the column pages, so it could
    // be more than one phase away from a slot's barrier, which a parity wait cannot tell apart.
    mbar_init(&sh.aready[0], 1);
    mbar_init(&sh.aready[1], 1);
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

  // job -> (unit, row page mp); all roles walk the same sequence of jobs and column pages
  struct Job {
    int unit, mp, h, l; const int32_t* table; bool valid;
    __device__ __forceinline__ Job(const XtParams& p, int job) {
      unit = job / p.NB;
      mp = job % p.NB;
      h = unit % p.Hkv;
      const int b = (unit / p.Hkv) % p.B;
      l = unit / (p.Hkv * p.B);
      table = p.block_table + (int64_t)b * p.NB;
      valid = table[mp] != -1;
    }
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      prefetch_tensormap(&tmK);
      SlotFifo fifo;
      bool ok = true;
      // Per slot: 1 + the running number of the job whose row page it held last, until it is
      // loaded again (0 = none).  The epilogue reads that page for the row sums after the job's
      // products are done, so the MMA commit alone does not free it.
      int pend0 = 0, pend1 = 0, pend2 = 0;
      uint32_t jobs_done = 0;
      auto load_page = [&](int slot, int id, int h, int l, int where) -> bool {
        const uint32_t u = fifo.use(slot);
        if (!mbar_wait<true>(&sh.empty[slot], (u & 1) ^ 1, abortp, p.error_word, where)) return false;
        const int pend = slot == 0 ? pend0 : (slot == 1 ? pend1 : pend2);
        if (pend) {
          const uint32_t k = pend - 1;
          if (!mbar_wait<true>(&sh.adone[k & 1], (k >> 1) & 1, abortp, p.error_word, 102)) return false;
          if (slot == 0) pend0 = 0; else if (slot == 1) pend1 = 0; else pend2 = 0;
        }
        unsigned char* dst = bufs + slot * XT_PAGE_BYTES;
        mbar_arrive_expect_tx(&sh.full[slot], XT_PAGE_BYTES);
        tma_load_5d(dst, &tmK, &sh.full[slot], 0, h, 0, id, l);
        tma_load_5d(dst + XT_BLOCK_BYTES, &tmK, &sh.full[slot], 64, h, 0, id, l);
        return true;
      };
      for (int job = blockIdx.x; ok && job < p.total_jobs; job += gridDim.x) {
        const Job jb(p, job);
        if (!jb.valid) continue;
        const int sa = fifo.pop();
        ok = load_page(sa, decode_page(jb.table[jb.mp]).id, jb.h, jb.l, 100);
        for (int pg = jb.mp; ok && pg < p.NB; ++pg) {
          const PageRef cp = decode_page(jb.table[pg]);
          if (!cp.valid) continue;
          const int sb = fifo.pop();
          fifo.push(sb);
          ok = load_page(sb, cp.id, jb.h, jb.l, 101);
        }
        fifo.push(sa);
        ++jobs_done;
        if (sa == 0) pend0 = jobs_done; else if (sa == 1) pend1 = jobs_done; else pend2 = jobs_done;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      SlotFifo fifo;
      int nj = 0;
      uint32_t use = 0;   // items issued per row group so far (both groups take part in every page)
      bool ok = true;
      for (int job = blockIdx.x; ok && job < p.total_jobs; job += gridDim.x) {
        const Job jb(p, job);
        if (!jb.valid) continue;
        const int sa = fifo.pop();
        if (!mbar_wait<true>(&sh.full[sa], fifo.use(sa) & 1, abortp, p.error_word, 201)) break;
        mbar_arrive(&sh.aready[nj & 1]);
        const uint32_t a_addr = smem_u32(bufs + sa * XT_PAGE_BYTES);
        for (int pg = jb.mp; ok && pg < p.NB; ++pg) {
          if (jb.table[pg] == -1) continue;
          const int sb = fifo.pop();
          fifo.push(sb);
          if (!mbar_wait<true>(&sh.full[sb], fifo.use(sb) & 1, abortp, p.error_word, 202)) { ok = false; break; }
          const uint32_t b_addr = smem_u32(bufs + sb * XT_PAGE_BYTES);
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            if (!mbar_wait<true>(&sh.tempty[g], (use & 1) ^ 1, abortp, p.error_word, 203)) { ok = false; break; }
            fence_after_sync();
            umma_k128(tmem_base + g * 256, a_addr + g * 16384, XT_BLOCK_BYTES, b_addr, XT_BLOCK_BYTES, IDESC);
            umma_commit(&sh.tfull[g]);
          }
          ++use;
          if (ok) umma_commit(&sh.empty[sb]);   // the slot is free once these products are done
        }
        if (ok) umma_commit(&sh.empty[sa]);   // (the epilogue still reads it: see `adone`)
        fifo.push(sa);
        ++nj;
      }
    }
  } else if (warp >= 18) {
    // ---------------- row sums ----------------
    // k_m . w for the 256 rows of the job's row page (128 per warp), read from the resident
    // (swizzled) page; sum_n S[m,n] = rn_m * (k_m . w) - S[m,m] is finished by the caller's
    // finalize kernel.  A lane owns four of the 128 dims (its slice of w stays in registers) and
    // eight rows are reduced across the warp at a time.  Off the tensor pipe's critical path: the
    // page slot is only reloaded after the arrival on `adone` (the producer waits for it), which
    // comes early in the job.
    const int blk = lane >> 4, cc = (lane >> 1) & 7, half = lane & 1;
    const int myr = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
    const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
    SlotFifo fifo;
    uint32_t nj = 0;
    for (int job = blockIdx.x; job < p.total_jobs; job += gridDim.x) {
      const Job jb(p, job);
      if (!jb.valid) continue;
      const float4 w4 = *reinterpret_cast<const float4*>(p.wvec + (int64_t)jb.unit * 128 + blk * 64 + cc * 8 + half * 4);
      const int sa = fifo.pop();
      for (int pg = jb.mp; pg < p.NB; ++pg) {   // replay the column pages' slots
        if (jb.table[pg] == -1) continue;
        fifo.push(fifo.pop());
      }
      fifo.push(sa);
      if (!mbar_wait(&sh.aready[nj & 1], (nj >> 1) & 1, abortp, p.error_word, 401)) break;
      const unsigned char* page = bufs + sa * XT_PAGE_BYTES + blk * XT_BLOCK_BYTES + half * 8;
      float* out = p.rowsum + (int64_t)job * 256;   // = (unit * NB + row page) * 256
#pragma unroll 2
      for (int r0 = (warp - 18) * 128; r0 < (warp - 18) * 128 + 128; r0 += 8) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int row = r0 + j;
          const uint2 rawk = *reinterpret_cast<const uint2*>(page + row * 128 + ((cc ^ (row & 7)) << 4));
          const float2 a = Pair<T>::unpack(*reinterpret_cast<const typename Pair<T>::V*>(&rawk.x));
          const float2 c = Pair<T>::unpack(*reinterpret_cast<const typename Pair<T>::V*>(&rawk.y));
          v[j] = fmaf(a.x, w4.x, a.y * w4.y) + fmaf(c.x, w4.z, c.y * w4.w);
        }
        // transposed reduction: 8 values x 32 lanes -> one row total per lane
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float send = b4 ? v[i] : v[i + 4], keep = b4 ? v[i + 4] : v[i];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float send = b3 ? v[i] : v[i + 2], keep = b3 ? v[i + 2] : v[i];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
        }
        {
          const float send = b2 ? v[0] : v[1], keep = b2 ? v[1] : v[0];
          v[0] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
        }
        float tot = v[0];
        tot += __shfl_xor_sync(0xffffffffu, tot, 2);
        tot += __shfl_xor_sync(0xffffffffu, tot, 1);
        if ((lane & 3) == 0) out[r0 + myr] = tot;
      }
      __syncwarp();   // every lane is done with the row page
      if (lane == 0) mbar_arrive(&sh.adone[nj & 1]);
      ++nj;
    }
  } else {
    // ---------------- epilogue teams ----------------
    // thread (g, ch, r): row r of row group g, columns ch*128 .. +127 of every column page, in
    // four 32-column chunks
    const int ew = warp - 2;
    const int g = ew >> 3;             // team = row group
    const int q = warp & 3;            // TMEM lane quadrant this warp may read
    const int ch = (ew >> 2) & 1;      // column half
    const int r = q * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + g * 256 + ch * 128;
    uint32_t use = 0;
    // fetched during the previous job where possible: 1/|k_m| of this thread's row and the chunk
    // minima of the first column page
    int pref_job = -1;
    float pref_rn = 0.f;
    float4 pref_nm = make_float4(0.f, 0.f, 0.f, 0.f);
    bool ok = true;
    for (int job = blockIdx.x; ok && job < p.total_jobs; job += gridDim.x) {
      const int unit = job / p.NB, mp = job - unit * p.NB;
      const int32_t* table = p.block_table + (int64_t)((unit / p.Hkv) % p.B) * p.NB;
      if (table[mp] == -1) continue;
      const int64_t rbase = (int64_t)job * 256;   // = (unit * NB + row page) * 256
      // smallest |k| of this thread's four 32-column chunks, fetched one page ahead
      const float4* nmp = reinterpret_cast<const float4*>(p.nmin + ((int64_t)unit * p.NB) * 8) + ch;
      float rn_m;
      float4 nm_next;
      if (pref_job == job) { rn_m = pref_rn; nm_next = pref_nm; }
      else { rn_m = p.rn[rbase + g * 128 + r]; nm_next = __ldg(nmp + mp * 2); }
      pref_job = job + (int)gridDim.x;
      if (pref_job < p.total_jobs) {
        pref_rn = p.rn[(int64_t)pref_job * 256 + g * 128 + r];
        pref_nm = __ldg(reinterpret_cast<const float4*>(p.nmin) + (int64_t)pref_job * 2 + ch);
      }
      const float thr_m = p.threshold / rn_m;
      const unsigned m_key = mp * 256 + g * 128 + r;
      for (int pg = mp; ok && pg < p.NB; ++pg) {
        if (table[pg] == -1) continue;   // padding (the entry is in L1: every role walks this row)
        const float4 nm4 = nm_next;
        nm_next = __ldg(nmp + min(pg + 1, p.NB - 1) * 2);
        const bool diag_page = pg == mp;
        // one 32-column chunk: the threshold filter on the raw accumulators (S > thr needs
        // acc > thr * |k_m| * |k_n| >= thr * |k_m| * min|k_n|), then, rarely, the values
        auto scan = [&](uint32_t (&raw)[32], int c, float nmc) {
          if (diag_page && ch == g && c == q) {  // warp-uniform: the chunk with this warp's diagonal
#pragma unroll
            for (int j = 0; j < 32; ++j) raw[j] = (j == lane) ? 0u : raw[j];
          }
          // Largest positive accumulator of the 32 as a tree of 3-input INTEGER maxima (depth 4):
          // the bound is positive, positive floats order like their bit patterns read as signed
          // integers, and every negative float reads as a negative integer.
          int t[11];
#pragma unroll
          for (int j = 0; j < 10; ++j)
            t[j] = __vimax3_s32((int)raw[3 * j], (int)raw[3 * j + 1], (int)raw[3 * j + 2]);
          t[10] = max((int)raw[30], (int)raw[31]);
          const int u0 = __vimax3_s32(t[0], t[1], t[2]), u1 = __vimax3_s32(t[3], t[4], t[5]);
          const int u2 = __vimax3_s32(t[6], t[7], t[8]), u3 = max(t[9], t[10]);
          if (__int_as_float(max(__vimax3_s32(u0, u1, u2), max(u3, 0))) > thr_m * nmc) {
            const int64_t ubase = rbase - (int64_t)mp * 256;
            const unsigned n0 = pg * 256 + ch * 128 + c * 32;
            const float* rnc = p.rn + ubase + n0;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float v = __uint_as_float(raw[j]) * rnc[j];
              if (v > thr_m) {
                const unsigned long long bits = __float_as_uint(v * rn_m);
                atomicMax(p.best + ubase + m_key, ((unsigned long long)(n0 + j + 1) << 32) | bits);
                if (!diag_page)  // the mirrored entry of the tile that is not computed
                  atomicMax(p.best + ubase + n0 + j, ((unsigned long long)(m_key + 1) << 32) | bits);
              }
            }
          }
        };
        if (!mbar_wait<32>(&sh.tfull[g], use & 1, abortp, p.error_word, 304)) { ok = false; break; }
        ++use;
        fence_after_sync();
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t raw[32];
          tmem_ld32_issue(lane_base + c * 32, raw);
          tmem_ld32_wait(raw);
          if (c == 3) {  // every TMEM read of this item has landed in registers
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.tempty[g]);
          }
          scan(raw, c, c == 0 ? nm4.x : (c == 1 ? nm4.y : (c == 2 ? nm4.z : nm4.w)));
        }
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
static int launch_exact_tc(const void* k_cache, XtParams p, int64_t k_stride_layer, int64_t k_stride_page,
                           long long* sub, float eps, cudaStream_t st) {
  CUtensorMap tm;
  const uint64_t pages = p.L > 1 ? (uint64_t)(k_stride_layer / k_stride_page) : (1ull << 30);
  const uint64_t dims[5] = {128, (uint64_t)p.Hkv, 256, pages, (uint64_t)p.L};
  const uint64_t strides[4] = {128, (uint64_t)p.Hkv * 128, (uint64_t)k_stride_page,
                               (uint64_t)(p.L > 1 ? k_stride_layer : k_stride_page)};
  const uint32_t box[5] = {64, 1, 256, 1, 1};
  int rc = make_tensor_map_5d(&tm, UmmaFmt<T>::tm, k_cache, dims, strides, box, sizeof(T));
  if (rc) return rc;
  const int units = p.L * p.B * p.Hkv;
  p.total_jobs = units * p.NB;
  key_stats_kernel<T><<<units, 256, 0, st>>>(
      reinterpret_cast<const T*>(k_cache), p.block_table, const_cast<float*>(p.rn),
      const_cast<float*>(p.dself), const_cast<float*>(p.nmin), const_cast<float*>(p.wvec), p.B, p.NB,
      p.Hkv, k_stride_layer, k_stride_page, eps);
  const size_t smem = XT_NSLOT * XT_PAGE_BYTES + sizeof(XtShared) + 1024;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = p.total_jobs < sms ? p.total_jobs : sms;
  auto kern = redundancy_exact_tc_kernel<T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_error("zp_redundancy_exact(tcgen05): %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  kern<<<grid, XT_THREADS, smem, st>>>(tm, p);
  const int64_t total = (int64_t)units * p.NB * 256;
  exempt_scatter_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(p.best, sub, p.NB * 256, total);
  return check_launch("zp_redundancy_exact(tcgen05)");
}

// Called by zp_redundancy_exact (zp_redundancy.cu).  `sub` holds 2*n zeroed 64-bit words (the
// fixed-point subtrahends, then the latest-similar-key records), `stats` 2*n + units*(NB*8 + 128)
// floats of scratch, n = units*NB*256.  Fills rowsum and sub; the caller's finalize kernel makes
// the logits from them.
int redundancy_exact_tc(const void* k_cache, const int32_t* block_table, float* rowsum, long long* sub,
                        float* stats, int L, int B, int NB, int Hkv, int64_t k_stride_layer,
                        int64_t k_stride_page, float threshold, float eps, int dtype, cudaStream_t st) {
  XtParams p{};
  const size_t units = (size_t)L * B * Hkv, n = units * NB * 256;
  p.block_table = block_table; p.rowsum = rowsum;
  p.best = reinterpret_cast<unsigned long long*>(sub) + n;
  p.rn = stats; p.dself = stats + n; p.nmin = stats + 2 * n; p.wvec = stats + 2 * n + units * NB * 8;
  p.error_word = device_error_word();
  p.L = L; p.B = B; p.NB = NB; p.Hkv = Hkv; p.threshold = threshold;
  if (!p.error_word) { set_error("zp_redundancy_exact(tcgen05): no device error word"); return ZP_ERR_CUDA; }
  if (dtype == ZP_DTYPE_BF16)
    return launch_exact_tc<__nv_bfloat16>(k_cache, p, k_stride_layer, k_stride_page, sub, eps, st);
  if (dtype == ZP_DTYPE_F16)
    return launch_exact_tc<__half>(k_cache, p, k_stride_layer, k_stride_page, sub, eps, st);
  set_error("zp_redundancy_exact(tcgen05): 16-bit caches only");
  return ZP_ERR_UNSUPPORTED;
}

}  // namespace zp
