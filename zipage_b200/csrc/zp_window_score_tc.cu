// Window-masked attention scoring on tcgen05 tensor cores (16-bit caches, head_dim 128, page
// size 256, G*QCL <= 128 window rows per pass, G a power of two).
//
// Persistent blocks (one per SM) walk over the units (layer, sequence, kv head) with a fixed
// stride, so the TMA/MMA pipeline never drains between units.  A unit's window queries (row
// r = i*G + g) are loaded once by TMA; its key pages stream through a ring of three 64 KB
// swizzled tiles.
// Three sweeps over the pages recompute the logits on the tensor cores instead of storing them:
//   sweep 0: D[row][key]  = Q K^T (M = 128 rows, N = 256 keys)   -> row maximum
//   sweep 1: same product                                         -> row sum of exp
//   sweep 2: D[key][row]  = K Q^T (2 x (M = 128 keys, N = 128 rows)) -> probabilities; each thread
//            owns one key and sees all window rows, so the max over the query heads of the group
//            and the mean/max over the window are register-local.
// Rounding points are the reference's: logits and shifted logits are rounded to T
// (attention_score.py:129-130 and the torch ops at :220-243) two at a time with packed 16-bit
// instructions; exp uses ex2.approx.  In sweep 2 the probability of a (key, window row) pair is
// needed only for the query head of the group that maximises it; rounding to T and exp are both
// monotonic, so max_g T(exp(x_g) / Z_g) = T(exp(max_g (x_g - ln Z_g))): one exp and one rounding
// per group instead of one per query head.
// Roles (576 threads): warp 0 = TMA producer + TMEM owner, warp 1 = MMA issuer, warps 2-17 =
// epilogue.  Sweeps 0/1: the four epilogue warps of a TMEM lane quadrant split the 256 key
// columns of a tile in four groups of 64.  Sweep 2: the epilogue warps form two teams of eight,
// team b takes the tiles that land in accumulator buffer b; inside a team a warp owns 32 keys
// and all window rows, so no partial sums cross warps and a key's score is written straight
// from registers.
#include "zp_tc.cuh"

namespace zp {

using namespace tc;

constexpr int WT_THREADS = 576;
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
  int total_units;
  // Window rows are processed in passes of at most 128 rows (G * qcl_pass): this launch covers
  // window indices [i0, i0 + qcl_pass).  With more than one pass the per-key sums go to `partial`
  // ([pass][unit][NB*256] fp32) and a small kernel adds the passes and rounds.
  int i0, qcl_pass, pass;
  float* partial;
  int smem_bytes;
};

struct __align__(16) WtShared {
  uint64_t full[WT_NS], empty[WT_NS], tfull[2], tempty[2], qfull, qempty, stats_bar;
  alignas(16) uint32_t colm[64];   // sweep 2, per pair of window rows: packed row maxima (T)
  alignas(16) float collz[128];    // sweep 2, per window row: ln(row sum of exp)
  float part[4][128];              // per column-group partial row maximum / row sum
  uint32_t tmem_base;
  int abort_flag;
};
constexpr size_t WT_SMEM_BYTES = WT_NS * WT_PAGE_BYTES + 2 * WT_QBLOCK_BYTES + sizeof(WtShared);
static_assert(WT_SMEM_BYTES <= 232448, "window-score kernel: shared memory budget");

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// a - c in fp32 with a a 16-bit value: one instruction, no separate widening of a (sm_100)
template <typename T> struct MixedSub;
template <> struct MixedSub<__nv_bfloat16> {
  static __device__ __forceinline__ float sub(__nv_bfloat16 a, float c) {
    float d;
    asm("sub.rn.f32.bf16 %0, %1, %2;" : "=f"(d) : "h"(__bfloat16_as_ushort(a)), "f"(c));
    return d;
  }
};
template <> struct MixedSub<__half> {
  static __device__ __forceinline__ float sub(__half a, float c) {
    float d;
    asm("sub.rn.f32.f16 %0, %1, %2;" : "=f"(d) : "h"(__half_as_ushort(a)), "f"(c));
    return d;
  }
};

// two 32-column TMEM loads in flight, one wait: uses of `b` are ordered after the wait by the
// empty statement that names its registers
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t (&a)[32], uint32_t (&b)[32]) {
  tmem_ld32_issue(taddr, a);
  tmem_ld32_issue(taddr + 32, b);
  tmem_ld32_wait(a);
  asm volatile(""
      : "+r"(b[0]), "+r"(b[1]), "+r"(b[2]), "+r"(b[3]), "+r"(b[4]), "+r"(b[5]), "+r"(b[6]), "+r"(b[7]),
        "+r"(b[8]), "+r"(b[9]), "+r"(b[10]), "+r"(b[11]), "+r"(b[12]), "+r"(b[13]), "+r"(b[14]), "+r"(b[15]),
        "+r"(b[16]), "+r"(b[17]), "+r"(b[18]), "+r"(b[19]), "+r"(b[20]), "+r"(b[21]), "+r"(b[22]), "+r"(b[23]),
        "+r"(b[24]), "+r"(b[25]), "+r"(b[26]), "+r"(b[27]), "+r"(b[28]), "+r"(b[29]), "+r"(b[30]), "+r"(b[31])
      :
      : "memory");
}

// Sweep 0 on 32 raw logits: running maximum (four independent chains).
__device__ __forceinline__ float s0_chunk(const uint32_t (&raw)[32], float m) {
  float m0 = m, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    m0 = fmaxf(m0, __uint_as_float(raw[j]));
    m1 = fmaxf(m1, __uint_as_float(raw[j + 1]));
    m2 = fmaxf(m2, __uint_as_float(raw[j + 2]));
    m3 = fmaxf(m3, __uint_as_float(raw[j + 3]));
  }
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// Sweep 1 on 32 raw logits: sum of exp(T(T(raw * scale) - m)).
template <typename T>
__device__ __forceinline__ float2 s1_chunk(const uint32_t (&raw)[32], typename Pair<T>::V m2, float2 scale2,
                                           float2 z) {
  using V = typename Pair<T>::V;
  const float2 log2e2 = make_float2(1.4426950408889634f, 1.4426950408889634f);
  float2 z1 = make_float2(0.f, 0.f);
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    const float2 xa = __fmul2_rn(make_float2(__uint_as_float(raw[j]), __uint_as_float(raw[j + 1])), scale2);
    const float2 xb = __fmul2_rn(make_float2(__uint_as_float(raw[j + 2]), __uint_as_float(raw[j + 3])), scale2);
    const V la = Pair<T>::pack(xa.x, xa.y), lb = Pair<T>::pack(xb.x, xb.y);
    const float2 da = __fmul2_rn(Pair<T>::unpack(__hsub2(la, m2)), log2e2);
    const float2 db = __fmul2_rn(Pair<T>::unpack(__hsub2(lb, m2)), log2e2);
    z = __fadd2_rn(z, make_float2(ex2_approx(da.x), ex2_approx(da.y)));
    z1 = __fadd2_rn(z1, make_float2(ex2_approx(db.x), ex2_approx(db.y)));
  }
  return __fadd2_rn(z, z1);
}

// Sweep 2 on 32 columns (window rows col0 .. col0+31 of this thread's key): per group of G
// columns max_g (x_g - ln Z_g), one exp, rounded to T, then summed (or maximised) over the groups.
// Groups starting at a column >= nvalid_cols are not window rows; groups starting below `jmask`
// cannot see this key (last page) and count as probability 0.
template <typename T, int G>
__device__ __forceinline__ float s2_chunk(const uint32_t (&raw)[32], const uint32_t* colm_pairs,
                                          const float* collz, int nvalid_cols, int jmask_rel, float2 scale2,
                                          bool use_max, float acc) {
  using V = typename Pair<T>::V;
  float b[32];
  const uint4* cm4 = reinterpret_cast<const uint4*>(colm_pairs);
  const float4* lz4 = reinterpret_cast<const float4*>(collz);
#pragma unroll
  for (int j4 = 0; j4 < 4; ++j4) {   // 8 columns per step
    const uint4 cm = cm4[j4];
    const uint32_t cmv[4] = {cm.x, cm.y, cm.z, cm.w};
    const float4 lza = lz4[2 * j4], lzb = lz4[2 * j4 + 1];
    const float lzv[8] = {lza.x, lza.y, lza.z, lza.w, lzb.x, lzb.y, lzb.z, lzb.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int j = 8 * j4 + 2 * k;
      const float2 x = __fmul2_rn(make_float2(__uint_as_float(raw[j]), __uint_as_float(raw[j + 1])), scale2);
      const V xs = __hsub2(Pair<T>::pack(x.x, x.y), *reinterpret_cast<const V*>(&cmv[k]));
      b[j] = MixedSub<T>::sub(xs.x, lzv[2 * k]);
      b[j + 1] = MixedSub<T>::sub(xs.y, lzv[2 * k + 1]);
    }
  }
  constexpr int NG = 32 / G;
  float e[NG];
#pragma unroll
  for (int g = 0; g < NG; ++g) {
    float m;
    if constexpr (G == 1) m = b[g];
    else if constexpr (G == 2) m = fmaxf(b[2 * g], b[2 * g + 1]);
    else {
      m = fmaxf(fmaxf(b[g * G], b[g * G + 1]), fmaxf(b[g * G + 2], b[g * G + 3]));
#pragma unroll
      for (int k = 4; k < G; k += 4)
        m = fmaxf(fmaxf(m, b[g * G + k]), fmaxf(fmaxf(b[g * G + k + 1], b[g * G + k + 2]), b[g * G + k + 3]));
    }
    e[g] = ex2_approx(m * 1.4426950408889634f);
    if (g * G >= nvalid_cols || g * G < jmask_rel) e[g] = 0.f;
  }
  if constexpr (NG == 1) {
    const float f = Elem<T>::to_f32(Elem<T>::from_f32(e[0]));
    return use_max ? fmaxf(acc, f) : acc + f;
  } else {
    float2 a2 = make_float2(acc, use_max ? acc : 0.f);
#pragma unroll
    for (int g = 0; g < NG; g += 2) {
      const float2 f = Pair<T>::unpack(Pair<T>::pack(e[g], e[g + 1]));
      if (use_max) { a2.x = fmaxf(a2.x, f.x); a2.y = fmaxf(a2.y, f.y); }
      else a2 = __fadd2_rn(a2, f);
    }
    return use_max ? fmaxf(a2.x, a2.y) : a2.x + a2.y;
  }
}

template <typename T, int G>
__global__ void __launch_bounds__(WT_THREADS, 1)
window_score_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmQ,
                       const WtParams p) {
  using V = typename Pair<T>::V;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* bufs = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* qbuf = bufs + WT_NS * WT_PAGE_BYTES;    // the unit's queries: 2 x 16 KB
  WtShared& sh = *reinterpret_cast<WtShared*>(qbuf + 2 * WT_QBLOCK_BYTES);
  if (reinterpret_cast<unsigned char*>(&sh + 1) > smem_raw + p.smem_bytes) {
    // the tiles need 1024-byte alignment and the budget has no room for a misaligned base
    if (threadIdx.x == 0) atomicCAS(p.error_word, 0, 100);
    return;
  }

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = G * p.qcl_pass;

  if (threadIdx.x == 0) {
    for (int i = 0; i < WT_NS; ++i) { mbar_init(&sh.full[i], 1); mbar_init(&sh.empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sh.tfull[i], 1); mbar_init(&sh.tempty[i], 16); }
    mbar_init(&sh.qfull, 1); mbar_init(&sh.qempty, 1);
    mbar_init(&sh.stats_bar, 16);  // one arrival per epilogue warp
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

  // Tile order within a unit: sweeps 0 and 2 walk the table forwards, sweep 1 backwards (the pages
  // it starts with are the ones sweep 0 touched last, still in L2).  Every role walks the same
  // sequence of units, sweeps and tiles with counters only (no division in a per-tile path);
  // `gt` counts tiles since kernel start (it selects the TMEM buffer), `n` counts the block's units.
  struct Unit {
    int h, b, l, nvalid; const int32_t* table;
    __device__ __forceinline__ Unit(const WtParams& p, int unit) {
      h = unit % p.Hkv; b = (unit / p.Hkv) % p.B; l = unit / (p.Hkv * p.B);
      table = p.block_table + (int64_t)b * p.NB;
      nvalid = 0;
      for (int pg = 0; pg < p.NB; ++pg) nvalid += table[pg] != -1;
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tensormap(&tmK);
      prefetch_tensormap(&tmQ);
      int s = 0, sph = 0, n = 0;  // ring stage and its phase; n counts the units that have tiles
      bool ok = true;
      for (int unit = blockIdx.x; ok && unit < p.total_units; unit += gridDim.x) {
        const Unit un(p, unit);
        if (un.nvalid == 0) continue;
        for (int sweep = 0; ok && sweep < 3; ++sweep) {
          const int dir = sweep == 1 ? -1 : 1;
          int pos = sweep == 1 ? p.NB - 1 : 0;
          for (int j = 0; j < un.nvalid; ++j) {
            int entry = un.table[pos];
            while (entry == -1) { pos += dir; entry = un.table[pos]; }
            pos += dir;
            if (!mbar_wait<64>(&sh.empty[s], sph ^ 1, abortp, p.error_word, 111)) { ok = false; break; }
            const int id = decode_page(entry).id;
            mbar_arrive_expect_tx(&sh.full[s], WT_PAGE_BYTES);
            tma_load_5d(bufs + s * WT_PAGE_BYTES, &tmK, &sh.full[s], 0, un.h, 0, id, un.l);
            tma_load_5d(bufs + s * WT_PAGE_BYTES + WT_BLOCK_BYTES, &tmK, &sh.full[s], 64, un.h, 0, id, un.l);
            if (++s == WT_NS) { s = 0; sph ^= 1; }
            if (sweep == 0 && j == 0) {
              // The single query buffer is free once the previous unit's last product has been
              // read; the first key page of this unit is already on its way.
              if (!mbar_wait<64>(&sh.qempty, (n & 1) ^ 1, abortp, p.error_word, 110)) { ok = false; break; }
              mbar_arrive_expect_tx(&sh.qfull, (uint32_t)(2 * R * 128));
              const int qid = p.seq_idx[un.b];
              tma_load_5d(qbuf, &tmQ, &sh.qfull, 0, un.h * G, p.i0, qid, un.l);
              tma_load_5d(qbuf + WT_QBLOCK_BYTES, &tmQ, &sh.qfull, 64, un.h * G, p.i0, qid, un.l);
            }
          }
        }
        ++n;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t IDESC_QK = idesc_f16(UmmaFmt<T>::fmt, 128, 256);
      constexpr uint32_t IDESC_KQ = idesc_f16(UmmaFmt<T>::fmt, 128, 128);
      int gt = 0, n = 0, s = 0, sph = 0;
      bool ok = true;
      const uint32_t q_addr = smem_u32(qbuf);
      for (int unit = blockIdx.x; ok && unit < p.total_units; unit += gridDim.x) {
        const Unit un(p, unit);
        if (un.nvalid == 0) continue;
        if (!mbar_wait<64>(&sh.qfull, n & 1, abortp, p.error_word, 211)) break;
        for (int sweep = 0; ok && sweep < 3; ++sweep) {
          for (int j = 0; j < un.nvalid; ++j, ++gt) {
            const int buf = gt & 1, u = gt >> 1;
            if (!mbar_wait<64>(&sh.full[s], sph, abortp, p.error_word, 212)) { ok = false; break; }
            if (!mbar_wait<64>(&sh.tempty[buf], (u & 1) ^ 1, abortp, p.error_word, 213)) { ok = false; break; }
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
            if (++s == WT_NS) { s = 0; sph ^= 1; }
          }
        }
        if (ok) umma_commit(&sh.qempty);  // the unit's queries are no longer read
        ++n;
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int q = warp & 3;               // TMEM lane quadrant
    const int grp = (warp - 2) >> 2;      // sweeps 0/1: column group 0..3 (64 key columns each)
    const int r = q * 32 + lane;          // TMEM lane: window row (sweeps 0/1) or key (sweep 2)
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const float2 scale2 = make_float2(p.scale, p.scale);
    const int my_i = r / G;
    const bool use_max = p.reduce_mode != 0;
    uint32_t ph = 0;                      // phase of stats_bar (all 512 epilogue threads in lock step)
    auto sync_epilogue = [&](int where) -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.stats_bar);
      const bool ok_ = mbar_wait<0>(&sh.stats_bar, ph & 1, abortp, p.error_word, where);
      ++ph;
      return ok_;
    };
    auto release_tmem = [&](int buf) {    // this warp has read what it needs of the accumulator
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.tempty[buf]);
    };
    // sweep 2: team = accumulator buffer, hh = key half of the page, slot = this thread's key
    const int team = grp >> 1, hh = grp & 1;
    const int slot = hh * 128 + r;

    int gt = 0;
    bool ok = true;
    for (int unit = blockIdx.x; ok && unit < p.total_units; unit += gridDim.x) {
      const int b = (unit / p.Hkv) % p.B;
      const int32_t* table = p.block_table + (int64_t)b * p.NB;
      float row_max = -INFINITY;
      float2 row_z = make_float2(0.f, 0.f);
      V m2 = Pair<T>::pack(0.f, 0.f);       // this row's maximum, twice
      T* out = reinterpret_cast<T*>(p.scores_out) + (int64_t)unit * p.NB * 256;
      float* pout = p.partial ? p.partial + ((int64_t)p.pass * p.total_units + unit) * p.NB * 256 : nullptr;
      bool any = false;
      for (int sweep = 0; ok && sweep < 3; ++sweep) {
        if (sweep == 1 && any) {  // row maximum: combine the four column groups
          sh.part[grp][r] = row_max;
          if (!sync_epilogue(311)) { ok = false; break; }
          const float m = fmaxf(fmaxf(sh.part[0][r], sh.part[1][r]), fmaxf(sh.part[2][r], sh.part[3][r])) * p.scale;
          m2 = Pair<T>::pack(m, m);
          if (!sync_epilogue(312)) { ok = false; break; }  // everyone has read `part` before it is reused
        }
        if (sweep == 2 && any) {  // row sum: combine, publish per-column statistics for sweep 2
          sh.part[grp][r] = row_z.x + row_z.y;
          if (!sync_epilogue(313)) { ok = false; break; }
          if (grp == 0) {
            const float z = (sh.part[0][r] + sh.part[1][r]) + (sh.part[2][r] + sh.part[3][r]);
            reinterpret_cast<T*>(sh.colm)[r] = reinterpret_cast<const T*>(&m2)[0];
            sh.collz[r] = logf(z);
          }
          if (!sync_epilogue(314)) { ok = false; break; }
        }
        // The table is read 32 entries at a time (one per lane); ballots give the positions of
        // the real pages and of the page that holds the window.
        const int nwords = (p.NB + 31) >> 5;
        for (int wi = 0; ok && wi < nwords; ++wi) {
          const int w = sweep == 1 ? nwords - 1 - wi : wi;
          const int idx = w * 32 + lane;
          const int e = idx < p.NB ? table[idx] : -1;
          uint32_t vmask = __ballot_sync(0xffffffffu, e != -1);
          const uint32_t lmask = __ballot_sync(0xffffffffu, e < -1);
          if (sweep == 0 && grp < 2 && q == 0 && idx < p.NB && e == -1) {   // padded pages score exactly 0
            for (int k = 0; k < 128; ++k) {
              if (pout) pout[idx * 256 + grp * 128 + k] = 0.f;
              else out[idx * 256 + grp * 128 + k] = Elem<T>::from_f32(0.f);
            }
          }
          while (vmask) {
            const int bit = sweep == 1 ? 31 - __clz(vmask) : __ffs(vmask) - 1;
            vmask &= ~(1u << bit);
            const int pg = w * 32 + bit;
            const bool last = (lmask >> bit) & 1u;
            const int buf = gt & 1, u = gt >> 1;
            ++gt;
            any = true;
            if (!mbar_wait<32>(&sh.tfull[buf], u & 1, abortp, p.error_word, 315)) { ok = false; break; }
            fence_after_sync();

            if (sweep < 2) {
              // columns = key slots grp*64 ..; row r sees slot <= smax inside the last page
              uint32_t ra[32], rb[32];
              tmem_ld64(lane_addr + buf * 256 + grp * 64, ra, rb);
              release_tmem(buf);
              const int smax = last ? 256 - p.QCL + p.i0 + my_i : 256;
              const int s0 = grp * 64;
              if (s0 + 63 > smax) {  // masked key slots (last page only)
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  if (s0 + j > smax) ra[j] = 0xff800000u;  // -inf
                  if (s0 + 32 + j > smax) rb[j] = 0xff800000u;
                }
              }
              if (sweep == 0) {
                row_max = s0_chunk(rb, s0_chunk(ra, row_max));
              } else {
                row_z = s1_chunk<T>(ra, m2, scale2, row_z);
                row_z = s1_chunk<T>(rb, m2, scale2, row_z);
              }
            } else if (team != buf) {
              release_tmem(buf);   // the other team's tile (the barrier counts every epilogue warp)
            } else {
              // rows of D = keys; columns = window rows j = i*G + g; key `slot` is hidden from columns < jmask
              const uint32_t tb = lane_addr + buf * 256 + hh * 128;
              const int jmask = last ? max(0, slot - (256 - p.QCL) - p.i0) * G : 0;
              float acc2 = 0.f;   // probabilities are >= 0: the neutral element of both reductions
              uint32_t ra[32], rb[32];
              if (R > 64) {
                tmem_ld64(tb, ra, rb);
                acc2 = s2_chunk<T, G>(ra, &sh.colm[0], &sh.collz[0], R, jmask, scale2, use_max, acc2);
                acc2 = s2_chunk<T, G>(rb, &sh.colm[16], &sh.collz[32], R - 32, jmask - 32, scale2, use_max, acc2);
                if (R > 96) {
                  tmem_ld64(tb + 64, ra, rb);
                  release_tmem(buf);
                  acc2 = s2_chunk<T, G>(ra, &sh.colm[32], &sh.collz[64], R - 64, jmask - 64, scale2, use_max, acc2);
                  acc2 = s2_chunk<T, G>(rb, &sh.colm[48], &sh.collz[96], R - 96, jmask - 96, scale2, use_max, acc2);
                } else {
                  tmem_ld32(tb + 64, reinterpret_cast<float(&)[32]>(ra));
                  release_tmem(buf);
                  acc2 = s2_chunk<T, G>(ra, &sh.colm[32], &sh.collz[64], R - 64, jmask - 64, scale2, use_max, acc2);
                }
              } else if (R > 32) {
                tmem_ld64(tb, ra, rb);
                release_tmem(buf);
                acc2 = s2_chunk<T, G>(ra, &sh.colm[0], &sh.collz[0], R, jmask, scale2, use_max, acc2);
                acc2 = s2_chunk<T, G>(rb, &sh.colm[16], &sh.collz[32], R - 32, jmask - 32, scale2, use_max, acc2);
              } else {
                tmem_ld32(tb, reinterpret_cast<float(&)[32]>(ra));
                release_tmem(buf);
                acc2 = s2_chunk<T, G>(ra, &sh.colm[0], &sh.collz[0], R, jmask, scale2, use_max, acc2);
              }
              if (pout) pout[pg * 256 + slot] = acc2;
              else out[pg * 256 + slot] = Elem<T>::from_f32(use_max ? acc2 : acc2 / (float)p.QCL);
            }
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
  const size_t smem = 232448;  // all of it: the tiles take 224 KB, the rest is barriers and statistics
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
  WtParams pl = p;
  pl.smem_bytes = (int)smem;
  kern<<<grid, WT_THREADS, smem, st>>>(tmK, tmQ, pl);
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

