// Window-masked attention scoring on tcgen05 tensor cores (16-bit caches, head_dim 128, page
// size 256, G*QCL <= 128 window rows, G a power of two).
//
// Persistent blocks (one per SM) walk over the units (layer, sequence, kv head) with a fixed
// stride, so the TMA/MMA pipeline never drains between units.  A unit's window queries (row
// r = i*G + g) are loaded once by TMA (double-buffered across units); its key pages stream through
// a ring of 64 KB swizzled tiles.
// Three sweeps over the pages recompute the logits on the tensor cores instead of storing them:
//   sweep 0: D[row][key]  = Q K^T (M = 128 rows, N = 256 keys)   -> row maximum
//   sweep 1: same product                                         -> row sum of exp
//   sweep 2: D[key][row]  = K Q^T (2 x (M = 128 keys, N = 128 rows)) -> probabilities; each thread
//            owns one key and sees all window rows, so the max over the query heads of the group
//            and the mean/max over the window are register-local.
// Rounding points are the reference's: logits, shifted logits and probabilities are rounded to T
// (attention_score.py:129-130 and the torch ops at :220-243) — done two at a time with packed
// 16-bit instructions; exp uses ex2.approx.
// Roles (576 threads): warp 0 = TMA producer + TMEM owner, warp 1 = MMA issuer, warps 2-17 =
// epilogue.  The four epilogue warps of a TMEM lane quadrant split the 256 columns of a tile in
// four groups of 64 (sweeps 0/1: key slots; sweep 2: group g owns keys (g/2)*128.. and window-row
// columns (g%2)*64.., the two partial sums of a key meet in shared memory).  Four warps per
// scheduler hide the latency of the TMEM loads and of the dependent maths.
#include "zp_tc.cuh"

namespace zp {

using namespace tc;

constexpr int WT_THREADS = 576;
constexpr int WT_PAGE_BYTES = 65536;
constexpr int WT_BLOCK_BYTES = 32768;
constexpr int WT_QBLOCK_BYTES = 16384;  // 128 rows x 128 bytes
constexpr int WT_NS = 2;

struct WtParams {
  const int32_t* seq_idx;
  const int32_t* block_table;
  void* scores_out;
  int* error_word;
  int L, B, NB, Hq, Hkv, QCL;
  float scale;
  int reduce_mode;
  int total_units;
  // Window rows are processed in passes of at most 128 rows (G * qcl_pass): this launch covers
  // window indices [i0, i0 + qcl_pass).  With more than one pass the per-key sums go to `partial`
  // ([pass][unit][NB*256] fp32) and a small kernel adds the passes and rounds.
  int i0, qcl_pass, pass;
  float* partial;
};

struct __align__(16) WtShared {
  uint64_t full[WT_NS], empty[WT_NS], tfull[2], tempty[2], qfull[2], qempty[2], stats_bar;
  alignas(16) uint32_t colm[64];   // sweep 2, per pair of window rows: packed row maxima (T)
  alignas(16) float colrz[128];    // sweep 2, per window row: 1 / row sum of exp
  float part[4][128];              // per column-group partial row maximum / row sum
  float acc[2][256];               // sweep 2: per key, sum (or max) over window rows; by tile parity
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Reduce 32 columns held as 16 packed pairs: max over each group of G adjacent columns, then
// sum (or max) over the groups.  Columns >= ncols are ignored.
// FULL: all 32 columns are window rows (no per-column test).
template <typename T, int G, bool FULL>
__device__ __forceinline__ float group_reduce(const typename Pair<T>::V (&pp)[16], int ncols, bool use_max,
                                              float acc) {
  using V = typename Pair<T>::V;
  constexpr int PG = G >= 2 ? G / 2 : 1;  // packed pairs per group
  constexpr int NG = 32 / G;
  float part[NG];
  if constexpr (G == 1) {
#pragma unroll
    for (int jp = 0; jp < 16; ++jp) {
      const float2 f = Pair<T>::unpack(pp[jp]);
      part[2 * jp] = f.x; part[2 * jp + 1] = f.y;
    }
  } else {
#pragma unroll
    for (int jp = 0; jp < 16; jp += PG) {
      V m = pp[jp];
#pragma unroll
      for (int k = 1; k < PG; ++k) m = __hmax2(m, pp[jp + k]);
      const float2 f = Pair<T>::unpack(m);
      part[jp / PG] = fmaxf(f.x, f.y);
    }
  }
  if (use_max) {
#pragma unroll
    for (int g = 0; g < NG; ++g) if (FULL || g * G < ncols) acc = fmaxf(acc, part[g]);
  } else {
#pragma unroll
    for (int g = 0; g < NG; ++g) if (FULL || g * G < ncols) acc += part[g];
  }
  return acc;
}

template <typename T, int G>
__global__ void __launch_bounds__(WT_THREADS, 1)
window_score_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmQ,
                       const WtParams p) {
  using V = typename Pair<T>::V;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* bufs = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* qbufs = bufs + WT_NS * WT_PAGE_BYTES;   // two query buffers of 2 x 16 KB
  WtShared& sh = *reinterpret_cast<WtShared*>(qbufs + 4 * WT_QBLOCK_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = G * p.qcl_pass;

  if (threadIdx.x == 0) {
    for (int i = 0; i < WT_NS; ++i) { mbar_init(&sh.full[i], 1); mbar_init(&sh.empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh.tfull[i], 1); mbar_init(&sh.tempty[i], 16);
      mbar_init(&sh.qfull[i], 1); mbar_init(&sh.qempty[i], 1);
    }
    mbar_init(&sh.stats_bar, 16);  // one arrival per epilogue warp
    sh.abort_flag = 0;
    fence_mbar_init();
  }
  if (threadIdx.x < 512) (&sh.acc[0][0])[threadIdx.x] = 0.f;
  if (warp == 0) {
    tmem_alloc(&sh.tmem_base, 512);
    tmem_relinquish();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = sh.tmem_base;
  volatile int* abortp = &sh.abort_flag;

  // Tile order within a unit: sweeps 0 and 2 walk the table forwards, sweep 1 backwards (the pages
  // it starts with are the ones sweep 0 touched last, still in L2).  Each role keeps a cursor, so
  // finding the next valid table position costs one (cached) load instead of a scan of the table.
  struct TileCursor {
    // The table entry of the tile after the current one is loaded one call ahead, so its latency
    // is hidden behind the current tile's work.
    const int32_t* table; int NB, nvalid, pg, nxt_pg, nxt_entry;
    __device__ __forceinline__ void probe(int from, int step) {   // next valid position from `from`
      int q = from;
      int e = table[q];
      while (e == -1) { q += step; e = table[q]; }
      nxt_pg = q; nxt_entry = e;
    }
    __device__ __forceinline__ void start() { probe(0, 1); }
    // returns the table position of tile tt and its (encoded) entry
    __device__ __forceinline__ int next(int tt, int ntiles, int& entry) {
      pg = nxt_pg; entry = nxt_entry;
      const int t2 = tt + 1;
      if (t2 < ntiles) {
        const int sweep = t2 / nvalid;
        if (t2 % nvalid == 0) { if (sweep == 1) probe(NB - 1, -1); else probe(0, 1); }
        else if (sweep == 1) probe(pg - 1, -1);
        else probe(pg + 1, 1);
      }
      return pg;
    }
  };
  // Every role walks the same sequence of units and tiles; `gt` counts tiles since kernel start
  // (it selects the shared-memory stage and the TMEM buffer), `n` counts this block's units.
  struct Unit {
    int h, b, l, nvalid, ntiles; const int32_t* table;
    __device__ __forceinline__ Unit(const WtParams& p, int unit) {
      h = unit % p.Hkv; b = (unit / p.Hkv) % p.B; l = unit / (p.Hkv * p.B);
      table = p.block_table + (int64_t)b * p.NB;
      nvalid = 0;
      for (int pg = 0; pg < p.NB; ++pg) nvalid += table[pg] != -1;
      ntiles = 3 * nvalid;
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tensormap(&tmK);
      prefetch_tensormap(&tmQ);
      int gt = 0, n = 0;  // n counts the units that have tiles (query buffer n & 1)
      bool ok = true;
      for (int unit = blockIdx.x; ok && unit < p.total_units; unit += gridDim.x) {
        const Unit un(p, unit);
        if (un.ntiles == 0) continue;
        const int qb = n & 1;
        if (!mbar_wait<true>(&sh.qempty[qb], ((n >> 1) & 1) ^ 1, abortp, p.error_word, 110)) break;
        mbar_arrive_expect_tx(&sh.qfull[qb], (uint32_t)(2 * R * 128));
        const int qid = p.seq_idx[un.b];
        unsigned char* qbuf = qbufs + qb * 2 * WT_QBLOCK_BYTES;
        tma_load_5d(qbuf, &tmQ, &sh.qfull[qb], 0, un.h * G, p.i0, qid, un.l);
        tma_load_5d(qbuf + WT_QBLOCK_BYTES, &tmQ, &sh.qfull[qb], 64, un.h * G, p.i0, qid, un.l);
        TileCursor cur{un.table, p.NB, un.nvalid, 0, 0, 0};
        cur.start();
        for (int tt = 0; tt < un.ntiles; ++tt, ++gt) {
          int entry;
          cur.next(tt, un.ntiles, entry);
          const int s = gt % WT_NS, k = gt / WT_NS;
          if (!mbar_wait<true>(&sh.empty[s], (k & 1) ^ 1, abortp, p.error_word, 111)) { ok = false; break; }
          const int id = decode_page(entry).id;
          mbar_arrive_expect_tx(&sh.full[s], WT_PAGE_BYTES);
          tma_load_5d(bufs + s * WT_PAGE_BYTES, &tmK, &sh.full[s], 0, un.h, 0, id, un.l);
          tma_load_5d(bufs + s * WT_PAGE_BYTES + WT_BLOCK_BYTES, &tmK, &sh.full[s], 64, un.h, 0, id, un.l);
        }
        ++n;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t IDESC_QK = idesc_f16(UmmaFmt<T>::fmt, 128, 256);
      constexpr uint32_t IDESC_KQ = idesc_f16(UmmaFmt<T>::fmt, 128, 128);
      int gt = 0, n = 0;
      bool ok = true;
      for (int unit = blockIdx.x; ok && unit < p.total_units; unit += gridDim.x) {
        const Unit un(p, unit);
        if (un.ntiles == 0) continue;
        const int qb = n & 1;
        if (!mbar_wait<true>(&sh.qfull[qb], (n >> 1) & 1, abortp, p.error_word, 211)) break;
        const uint32_t q_addr = smem_u32(qbufs + qb * 2 * WT_QBLOCK_BYTES);
        for (int tt = 0; tt < un.ntiles; ++tt, ++gt) {
          const int sweep = tt / un.nvalid;
          const int s = gt % WT_NS, k = gt / WT_NS, buf = gt & 1, u = gt >> 1;
          if (!mbar_wait<true>(&sh.full[s], k & 1, abortp, p.error_word, 212)) { ok = false; break; }
          if (!mbar_wait<true>(&sh.tempty[buf], (u & 1) ^ 1, abortp, p.error_word, 213)) { ok = false; break; }
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
        if (ok) umma_commit(&sh.qempty[qb]);  // the unit's queries are no longer read
        ++n;
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int q = warp & 3;               // TMEM lane quadrant
    const int grp = (warp - 2) >> 2;      // column group 0..3 (64 columns each)
    const int r = q * 32 + lane;          // TMEM lane: window row (sweeps 0/1) or key (sweep 2)
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + grp * 64;
    const float2 log2e2 = make_float2(1.4426950408889634f, 1.4426950408889634f);
    const float2 scale2 = make_float2(p.scale, p.scale);
    const int my_i = r / G;
    const bool use_max = p.reduce_mode != 0;
    uint32_t ph = 0;                      // phase of stats_bar (all 512 epilogue threads in lock step)
    auto sync_epilogue = [&](int where) -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.stats_bar);
      const bool ok_ = mbar_wait(&sh.stats_bar, ph & 1, abortp, p.error_word, where);
      ++ph;
      return ok_;
    };
    // sweep 2: this thread's key and the window-row columns it covers
    const int hh = grp >> 1, cbase = (grp & 1) * 64;
    const int slot = hh * 128 + r;

    int gt = 0;
    bool ok = true;
    for (int unit = blockIdx.x; ok && unit < p.total_units; unit += gridDim.x) {
    const Unit un(p, unit);
    const int32_t* table = un.table;
    const int nvalid = un.nvalid, ntiles = un.ntiles;
    float row_max = -INFINITY, row_z = 0.f;
    V m2 = Pair<T>::pack(0.f, 0.f);       // this row's maximum, twice
    T* out = reinterpret_cast<T*>(p.scores_out) + (int64_t)unit * p.NB * 256;
    if (grp < 2)
      for (int pg = 0; pg < p.NB; ++pg)   // padded pages score exactly 0
        if (table[pg] == -1) {
          if (p.partial) p.partial[((int64_t)p.pass * p.total_units + unit) * p.NB * 256 + pg * 256 + grp * 128 + r] = 0.f;
          else out[pg * 256 + grp * 128 + r] = Elem<T>::from_f32(0.f);
        }
    TileCursor cur{table, p.NB, nvalid, 0, 0, 0};
    if (ntiles > 0) cur.start();
    for (int tt = 0; tt < ntiles; ++tt, ++gt) {
      int entry;
      const int pg = cur.next(tt, ntiles, entry);
      const int sweep = tt / nvalid;
      const bool last = entry < -1;
      const int buf = gt & 1, u = gt >> 1;
      if (tt == nvalid) {  // row maximum: combine the four column groups
        sh.part[grp][r] = row_max;
        if (!sync_epilogue(311)) { ok = false; break; }
        const float m = fmaxf(fmaxf(sh.part[0][r], sh.part[1][r]), fmaxf(sh.part[2][r], sh.part[3][r])) * p.scale;
        m2 = Pair<T>::pack(m, m);
        if (!sync_epilogue(312)) { ok = false; break; }  // everyone has read `part` before it is reused
      }
      if (tt == 2 * nvalid) {  // row sum: combine, publish per-column statistics for sweep 2
        sh.part[grp][r] = row_z;
        if (!sync_epilogue(313)) { ok = false; break; }
        if (grp == 0) {
          const float z = (sh.part[0][r] + sh.part[1][r]) + (sh.part[2][r] + sh.part[3][r]);
          reinterpret_cast<T*>(sh.colm)[r] = reinterpret_cast<const T*>(&m2)[0];
          sh.colrz[r] = 1.f / z;
        }
        if (!sync_epilogue(314)) { ok = false; break; }
      }
      if (!mbar_wait(&sh.tfull[buf], u & 1, abortp, p.error_word, 315)) { ok = false; break; }
      fence_after_sync();

      if (sweep < 2) {
        // columns = key slots grp*64 ..; row r sees slot <= smax inside the last page
        const uint32_t tbase = lane_base + buf * 256;
        const int smax = last ? 256 - p.QCL + p.i0 + my_i : 256;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t raw[32];
          tmem_ld32_issue(tbase + c * 32, raw);
          tmem_ld32_wait(raw);
          if (c == 1) {  // all TMEM reads of this tile have landed in registers
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.tempty[buf]);
          }
          const int s0 = grp * 64 + c * 32;
          if (s0 + 31 > smax) {  // masked key slots (last page only)
#pragma unroll
            for (int j = 0; j < 32; ++j) if (s0 + j > smax) raw[j] = 0xff800000u;  // -inf
          }
          if (sweep == 0) {
            float m0 = -INFINITY, m1 = -INFINITY, m2_ = -INFINITY, m3 = -INFINITY;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              m0 = fmaxf(m0, __uint_as_float(raw[j])); m1 = fmaxf(m1, __uint_as_float(raw[j + 1]));
              m2_ = fmaxf(m2_, __uint_as_float(raw[j + 2])); m3 = fmaxf(m3, __uint_as_float(raw[j + 3]));
            }
            row_max = fmaxf(row_max, fmaxf(fmaxf(m0, m1), fmaxf(m2_, m3)));
          } else {
            float z0 = 0.f, z1 = 0.f, z2 = 0.f, z3 = 0.f;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const float2 xa = fmul2(make_float2(__uint_as_float(raw[j]), __uint_as_float(raw[j + 1])), scale2);
              const float2 xb = fmul2(make_float2(__uint_as_float(raw[j + 2]), __uint_as_float(raw[j + 3])), scale2);
              const V la = Pair<T>::pack(xa.x, xa.y), lb = Pair<T>::pack(xb.x, xb.y);
              const float2 da = fmul2(Pair<T>::unpack(__hsub2(la, m2)), log2e2);
              const float2 db = fmul2(Pair<T>::unpack(__hsub2(lb, m2)), log2e2);
              z0 += ex2_approx(da.x); z1 += ex2_approx(da.y);
              z2 += ex2_approx(db.x); z3 += ex2_approx(db.y);
            }
            row_z += (z0 + z1) + (z2 + z3);
          }
        }
      } else {
        // rows of D = keys; columns = window rows j = i*G + g; key `slot` is hidden from columns < jmask
        const uint32_t tbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * 256 + hh * 128 + cbase;
        const int jmask = last ? max(0, slot - (256 - p.QCL) - p.i0) * G : 0;
        float acc2 = use_max ? -INFINITY : 0.f;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          const int col0 = cbase + c * 32;
          if (col0 >= R) {  // no window rows in this chunk (R < 128)
            if (c == 1) { fence_before_sync(); __syncwarp(); if (lane == 0) mbar_arrive(&sh.tempty[buf]); }
            continue;
          }
          uint32_t raw[32];
          tmem_ld32_issue(tbase + c * 32, raw);
          tmem_ld32_wait(raw);
          if (c == 1) {
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.tempty[buf]);
          }
          V pp[16];
          const uint4* cm4 = reinterpret_cast<const uint4*>(&sh.colm[col0 >> 1]);
          const float4* rz4 = reinterpret_cast<const float4*>(&sh.colrz[col0]);
#pragma unroll
          for (int j4 = 0; j4 < 4; ++j4) {   // 4 pairs (8 columns) per step
            const uint4 cm = cm4[j4];
            const uint32_t cmv[4] = {cm.x, cm.y, cm.z, cm.w};
            const float4 rza = rz4[2 * j4], rzb = rz4[2 * j4 + 1];
            const float rzv[8] = {rza.x, rza.y, rza.z, rza.w, rzb.x, rzb.y, rzb.z, rzb.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int jp = 4 * j4 + k;
              const float2 x = fmul2(make_float2(__uint_as_float(raw[2 * jp]), __uint_as_float(raw[2 * jp + 1])), scale2);
              const V lg = Pair<T>::pack(x.x, x.y);
              const float2 d = fmul2(Pair<T>::unpack(__hsub2(lg, *reinterpret_cast<const V*>(&cmv[k]))), log2e2);
              const float2 e = fmul2(make_float2(ex2_approx(d.x), ex2_approx(d.y)),
                                     make_float2(rzv[2 * k], rzv[2 * k + 1]));
              pp[jp] = Pair<T>::pack(e.x, e.y);
            }
          }
          if (jmask > col0) {  // some of this chunk's window rows cannot see this key (last page only)
            const T zero = Elem<T>::from_f32(0.f);
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < jmask) reinterpret_cast<T*>(pp)[j] = zero;
          }
          const int ncols = R - col0;
          acc2 = ncols >= 32 ? group_reduce<T, G, true>(pp, ncols, use_max, acc2)
                             : group_reduce<T, G, false>(pp, ncols, use_max, acc2);
        }
        // the two column halves of a key meet in shared memory (two addends: order cannot matter)
        float* accbuf = sh.acc[tt & 1];
        if (cbase < R) {
          if (use_max) atomicMax(reinterpret_cast<int*>(&accbuf[slot]), __float_as_int(fmaxf(acc2, 0.f)));
          else atomicAdd(&accbuf[slot], acc2);
        }
        if (!sync_epilogue(316)) { ok = false; break; }
        if ((grp & 1) == 0) {
          const float a = accbuf[slot];
          accbuf[slot] = 0.f;
          if (p.partial)
            p.partial[((int64_t)p.pass * p.total_units + unit) * p.NB * 256 + pg * 256 + slot] = a;
          else
            out[pg * 256 + slot] = Elem<T>::from_f32(use_max ? a : a / (float)p.QCL);
        }
      }
    }
    }  // units
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
    const uint32_t box[5] = {64, (uint32_t)G, (uint32_t)p.qcl_pass, 1, 1};
    int rc = make_tensor_map_5d(&tmQ, UmmaFmt<T>::tm, q_cache, dims, strides, box, sizeof(T));
    if (rc) return rc;
  }
  const size_t smem = WT_NS * WT_PAGE_BYTES + 4 * WT_QBLOCK_BYTES + sizeof(WtShared) + 1024;
  void (*kern)(const CUtensorMap, const CUtensorMap, const WtParams) = nullptr;
  switch (G) {
    case 1: kern = window_score_tc_kernel<T, 1>; break;
    case 2: kern = window_score_tc_kernel<T, 2>; break;
    case 4: kern = window_score_tc_kernel<T, 4>; break;
    case 8: kern = window_score_tc_kernel<T, 8>; break;
    case 16: kern = window_score_tc_kernel<T, 16>; break;
    default: kern = window_score_tc_kernel<T, 32>; break;
  }
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_error("zp_window_score(tcgen05): %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = p.total_units < sms ? p.total_units : sms;
  kern<<<grid, WT_THREADS, smem, st>>>(tmK, tmQ, p);
  return check_launch("zp_window_score(tcgen05)");
}

// adds the passes' per-key sums (or takes their max) and rounds: out = T(sum / QCL)
template <typename T>
__global__ void window_score_combine_kernel(const float* __restrict__ partial, T* __restrict__ out,
                                            int64_t n, int npass, float qcl, int use_max) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float a = partial[i];
  for (int ps = 1; ps < npass; ++ps) a = use_max ? fmaxf(a, partial[ps * n + i]) : a + partial[ps * n + i];
  out[i] = Elem<T>::from_f32(use_max ? a : a / qcl);
}

// number of passes over the window rows (0 = shapes not covered)
int window_score_tc_passes(int Hq, int Hkv, int QCL) {
  const int G = Hq / Hkv;
  if (G < 1 || G > 32 || (G & (G - 1))) return 0;
  for (int np = 1; np <= 8; np *= 2) {
    if (QCL % np) return 0;
    const int R = G * (QCL / np);
    if (R <= 128) return (R % 8 == 0) ? np : 0;
  }
  return 0;
}
size_t window_score_tc_workspace_bytes(int L, int B, int NB, int Hq, int Hkv, int QCL) {
  const int np = window_score_tc_passes(Hq, Hkv, QCL);
  return np > 1 ? (size_t)np * L * B * Hkv * NB * 256 * sizeof(float) : 0;
}

// true when the tensor-core kernel covers these shapes
bool window_score_tc_supported(int dtype, int D, int BS, int Hq, int Hkv, int QCL, bool want_logits) {
  if (want_logits || !(dtype == ZP_DTYPE_BF16 || dtype == ZP_DTYPE_F16) || D != 128 || BS != 256) return false;
  return QCL <= 256 && window_score_tc_passes(Hq, Hkv, QCL) > 0;
}

int window_score_tc(const void* k_cache, const void* q_cache, const int32_t* seq_idx,
                    const int32_t* block_table, void* scores_out, int L, int B, int NB, int Hq, int Hkv,
                    int QCL, int64_t k_stride_layer, int64_t k_stride_page, int64_t q_stride_layer,
                    int64_t q_stride_seq, float scale, int reduce_mode, int dtype, float* partial,
                    cudaStream_t st) {
  const int npass = window_score_tc_passes(Hq, Hkv, QCL);
  if (npass > 1 && !partial) {
    set_error("zp_window_score(tcgen05): %d window rows need %d passes and a workspace", (Hq / Hkv) * QCL, npass);
    return ZP_ERR_WORKSPACE;
  }
  WtParams p;
  p.qcl_pass = QCL / npass; p.partial = npass > 1 ? partial : nullptr;
  p.seq_idx = seq_idx; p.block_table = block_table; p.scores_out = scores_out;
  p.error_word = device_error_word();
  p.L = L; p.B = B; p.NB = NB; p.Hq = Hq; p.Hkv = Hkv; p.QCL = QCL; p.scale = scale;
  p.reduce_mode = reduce_mode;
  p.total_units = L * B * Hkv;
  if (!p.error_word) { set_error("zp_window_score(tcgen05): no device error word"); return ZP_ERR_CUDA; }
  for (int ps = 0; ps < npass; ++ps) {
    p.pass = ps; p.i0 = ps * p.qcl_pass;
    const int rc = dtype == ZP_DTYPE_BF16
        ? launch_window_tc<__nv_bfloat16>(k_cache, q_cache, p, k_stride_layer, k_stride_page, q_stride_layer, q_stride_seq, st)
        : launch_window_tc<__half>(k_cache, q_cache, p, k_stride_layer, k_stride_page, q_stride_layer, q_stride_seq, st);
    if (rc) return rc;
  }
  if (npass > 1) {
    const int64_t n = (int64_t)L * B * Hkv * NB * 256;
    const int blocks = (int)((n + 255) / 256);
    if (dtype == ZP_DTYPE_BF16)
      window_score_combine_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(partial, (__nv_bfloat16*)scores_out, n, npass, (float)QCL, reduce_mode);
    else
      window_score_combine_kernel<__half><<<blocks, 256, 0, st>>>(partial, (__half*)scores_out, n, npass, (float)QCL, reduce_mode);
    return check_launch("zp_window_score(tcgen05) combine");
  }
  return ZP_OK;
}

}  // namespace zp
