// Variable-length causal prefill attention (bottom-right aligned) on tcgen05 tensor cores:
// 16-bit tensors, head_dim 128, K/V dense or paged (page size a multiple of 128).
//
// One block per (128-query tile, query head, sequence).  Two passes over the key tiles the query
// tile can see.  This is the kernel for pages of an odd multiple of 128 keys, 128 keys at a time;
// dense K/V and pages of a multiple of 256 keys take the 256-key-tile kernel further down:
//   pass 1:  S = Q K^T (M = 128 queries, N = 128 keys, K = 128 dims)   -> row maxima
//   pass 2:  S again, P = exp2(S * scale*log2e - max) (masked entries 0), row sums of P in fp32,
//            P rounded to the tensor dtype and stored to TMEM as the A operand of
//            O += P V (M = 128 queries, N = 128 dims, K = 128 keys; V is the B operand as it lies in
//            memory: dims contiguous, i.e. MN-major), accumulated in TMEM over all tiles
// and out = O / row sum.  Recomputing S costs half as many tensor-core flops again but needs no
// rescaling of the output accumulator when a row maximum grows, so O never leaves TMEM and the
// softmax warps only stream S.
// Roles (576 threads, one block per SM): warp 0 = TMA producer and TMEM owner, warp 1 = MMA
// issuer, warps 2-17 = softmax (thread <-> TMEM lane <-> query row; the four warps of a lane
// quadrant split a tile's 128 columns).  Shared memory: the Q tile and a ring of four 32 KB K/V
// stages; TMEM: two S accumulators, O and two P tiles (all 512 columns).
// Keys past the end of a sequence: their S columns are masked by index; in the V tile their rows
// are overwritten with zeros before the product (their P is 0, but 0 * garbage may be NaN).
#include "zp_tc.cuh"

namespace zp {

using namespace tc;

constexpr int PT_THREADS = 576;
constexpr int PT_TILE_BYTES = 32768;   // 128 rows x 128 elements x 2 bytes
constexpr int PT_BLK_BYTES = 16384;    // one 64-element block of a tile
constexpr int PT_NRING = 4;
constexpr int PT_PCOL = 384;           // TMEM columns of the two P tiles (64 each), after S0, S1 and O

struct PtParams {
  const int32_t* cu_q; const int32_t* cu_k; const int32_t* table;
  void* out;
  int* error_word;
  int B, NBmax, Hq, Hkv, BS;
  int total_q, total_k;   // rows of q and of dense k/v (tensor-map extents: rows past them read as 0)
  float scale_log2e;
};

struct __align__(16) PtShared {
  uint64_t qfull, full[PT_NRING], empty[PT_NRING], sfull[2], sempty[2], pfull[2], pempty[2], ofull, sbar;
  float stat[4][128];   // row statistics exchanged between the four column quarters
  uint32_t tmem_base;
  int abort_flag;
};

// MN-major operand tile, 128-byte swizzle: 64 contiguous elements (128 bytes) per K row, 8-row
// groups `sbo` bytes apart along K, the next 64 elements along MN `lbo` bytes away.
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | ((lbo >> 4) << 16);
  const uint32_t hi = (sbo >> 4) | (1u << 14) | (2u << 29);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// A operand taken from TMEM (one row per lane, two 16-bit elements per 32-bit column)
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 16 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T>
__global__ void __launch_bounds__(PT_THREADS, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const PtParams p) {
  // tile geometry (identical in every role)
  const int b = blockIdx.z, h = blockIdx.y;
  const int q0 = p.cu_q[b], lq = p.cu_q[b + 1] - q0;
  const int k0 = p.cu_k[b], lk = p.cu_k[b + 1] - k0;
  const int nqt = (lq + 127) >> 7;
  if ((int)blockIdx.x >= nqt) return;
  const int qt = nqt - 1 - blockIdx.x;          // the tiles with the most keys start first
  const int qi0 = qt * 128;
  const int hk = h / (p.Hq / p.Hkv);
  const int shift = lk - lq;                    // query i sees keys j <= i + shift
  const int rows = min(128, lq - qi0);
  const int kmax = min(lk, qi0 + rows + shift); // keys any row of the tile can see
  const int n = kmax > 0 ? (kmax + 127) >> 7 : 0;
  const int n1 = n;                             // tiles of pass 1
  const int base2 = n;                          // ring position of pass 2's first load
  // S tile bookkeeping: pass-1 tile jj -> TMEM buffer jj & 1, its (jj >> 1)-th use; pass-2 tile j ->
  // buffer j & 1, use u1[j & 1] + (j >> 1) with u1[b] = pass-1 uses of buffer b
  const int u1_0 = (n1 + 1) >> 1, u1_1 = n1 >> 1;

  extern __shared__ unsigned char smem_raw[];
  unsigned char* bufs = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* qbuf = bufs;
  unsigned char* ring = bufs + PT_TILE_BYTES;
  PtShared& sh = *reinterpret_cast<PtShared*>(ring + PT_NRING * PT_TILE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (n == 0) {   // nothing visible: zeros
    if (warp >= 2) {
      const int t = threadIdx.x - 64;           // 512 threads: row t >> 2, quarter t & 3
      const int r = t >> 2;
      if (r < rows) {
        T* o = reinterpret_cast<T*>(p.out) + ((int64_t)(q0 + qi0 + r) * p.Hq + h) * 128 + (t & 3) * 32;
        for (int i = 0; i < 32; i += 8) *reinterpret_cast<int4*>(o + i) = make_int4(0, 0, 0, 0);
      }
    }
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(&sh.qfull, 1);
    for (int i = 0; i < PT_NRING; ++i) { mbar_init(&sh.full[i], 1); mbar_init(&sh.empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh.sfull[i], 1); mbar_init(&sh.sempty[i], 16);
      mbar_init(&sh.pfull[i], 16); mbar_init(&sh.pempty[i], 1);
    }
    mbar_init(&sh.ofull, 1);
    mbar_init(&sh.sbar, 16);  // the sixteen softmax warps (a bounded wait, unlike bar.sync)
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
  constexpr uint32_t IDESC_QK = idesc_f16(UmmaFmt<T>::fmt, 128, 128);
  constexpr uint32_t IDESC_PV = IDESC_QK | (1u << 16);   // B operand MN-major

  // ring position of a load: pass 1: K_j -> j; pass 2: K_j -> base2 + 2j, V_j -> base2 + 2j + 1
  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      prefetch_tensormap(&tmQ);
      prefetch_tensormap(&tmK);
      prefetch_tensormap(&tmV);
      mbar_arrive_expect_tx(&sh.qfull, PT_TILE_BYTES);
      tma_load_5d(qbuf, &tmQ, &sh.qfull, 0, h, q0 + qi0, 0, 0);
      tma_load_5d(qbuf + PT_BLK_BYTES, &tmQ, &sh.qfull, 64, h, q0 + qi0, 0, 0);
      bool ok = true;
      auto load = [&](int t, const CUtensorMap* tm, int j) -> bool {
        const int s = t % PT_NRING, k = t / PT_NRING;
        if (!mbar_wait<true>(&sh.empty[s], (k & 1) ^ 1, abortp, p.error_word, 501)) return false;
        unsigned char* dst = ring + s * PT_TILE_BYTES;
        int c2, c3;
        if (p.table) {   // a 128-key tile never straddles a page
          c2 = (j * 128) % p.BS;
          c3 = p.table[(int64_t)b * p.NBmax + (j * 128) / p.BS];
        } else {
          c2 = k0 + j * 128;
          c3 = 0;
        }
        mbar_arrive_expect_tx(&sh.full[s], PT_TILE_BYTES);
        tma_load_5d(dst, tm, &sh.full[s], 0, hk, c2, c3, 0);
        tma_load_5d(dst + PT_BLK_BYTES, tm, &sh.full[s], 64, hk, c2, c3, 0);
        return true;
      };
      for (int j = 0; ok && j < n; ++j) ok = load(j, &tmK, j);
      for (int j = 0; ok && j < n; ++j) {
        ok = load(base2 + 2 * j, &tmK, j);
        if (ok) ok = load(base2 + 2 * j + 1, &tmV, j);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      bool ok = mbar_wait(&sh.qfull, 0, abortp, p.error_word, 601);
      const uint32_t q_addr = smem_u32(qbuf);
      // one S tile: TMEM buffer sb (its `use`-th use), key tile at ring position t
      auto issue_s = [&](int sb, int use, int t) -> bool {
        const int s = t % PT_NRING, k = t / PT_NRING;
        if (!mbar_wait(&sh.full[s], k & 1, abortp, p.error_word, 602)) return false;
        if (!mbar_wait(&sh.sempty[sb], (use & 1) ^ 1, abortp, p.error_word, 603)) return false;
        fence_after_sync();
        umma_k128(tmem_base + sb * 128, q_addr, PT_BLK_BYTES, smem_u32(ring + s * PT_TILE_BYTES), PT_BLK_BYTES,
                  IDESC_QK);
        umma_commit(&sh.sfull[sb]);
        umma_commit(&sh.empty[s]);
        return true;
      };
      for (int jj = 0; ok && jj < n1; ++jj) ok = issue_s(jj & 1, jj >> 1, jj);
      auto issue_s2 = [&](int j) -> bool {
        return issue_s(j & 1, ((j & 1) ? u1_1 : u1_0) + (j >> 1), base2 + 2 * j);
      };
      if (ok) ok = issue_s2(0);
      for (int j = 0; ok && j < n; ++j) {
        if (j + 1 < n) ok = issue_s2(j + 1);   // S of the next tile first
        if (!ok) break;
        const int t = base2 + 2 * j + 1, s = t % PT_NRING, k = t / PT_NRING, pb = j & 1;
        if (!mbar_wait(&sh.full[s], k & 1, abortp, p.error_word, 604)) { ok = false; break; }
        if (!mbar_wait(&sh.pfull[pb], (j >> 1) & 1, abortp, p.error_word, 605)) { ok = false; break; }
        fence_after_sync();
        const uint32_t v_addr = smem_u32(ring + s * PT_TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {   // 16 keys per step: 8 columns of P
          const uint64_t bd = smem_desc_sw128_mn(v_addr + ks * 2048, PT_BLK_BYTES, 1024);
          umma_f16_ts(tmem_base + 256, tmem_base + PT_PCOL + pb * 64 + ks * 8, bd, IDESC_PV, (j | ks) ? 1u : 0u);
        }
        umma_commit(&sh.pempty[pb]);
        umma_commit(&sh.empty[s]);
      }
      if (ok) umma_commit(&sh.ofull);
    }
  } else {
    // ---------------- softmax ----------------
    const int q = warp & 3;               // TMEM lane quadrant
    const int cq = (warp - 2) >> 2;       // column quarter: keys / dims cq*32 .. +31 of a tile
    const int r = q * 32 + lane;          // query row of the tile
    const int lim = r < rows ? min(lk - 1, qi0 + r + shift) : -1;   // last visible key (-1: none)
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + cq * 32;
    bool ok = true;
    uint32_t sph = 0;
    auto softmax_sync = [&](int where) -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.sbar);
      const bool ok_ = mbar_wait(&sh.sbar, sph & 1, abortp, p.error_word, where);
      ++sph;
      return ok_;
    };
    uint32_t ra[32];
    // ---- pass 1: row maxima of the raw products ----
    float rmax = -INFINITY;
    auto row_max32 = [&](const uint32_t (&v)[32], int key0) {   // 32 keys from key0 on
      if (key0 + 31 <= lim) {
        float m0 = rmax, m1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          m0 = fmax3(m0, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
          m1 = fmax3(m1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
        }
        rmax = fmaxf(m0, m1);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (key0 + i <= lim) rmax = fmaxf(rmax, __uint_as_float(v[i]));
      }
    };
    for (int jj = 0; ok && jj < n1; ++jj) {
      const int sb = jj & 1, use = jj >> 1;
      if (!mbar_wait(&sh.sfull[sb], use & 1, abortp, p.error_word, 701)) { ok = false; break; }
      fence_after_sync();
      tmem_ld32_issue(lane_base + sb * 128, ra);
      tmem_ld32_wait(ra);
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.sempty[sb]);
      row_max32(ra, jj * 128 + cq * 32);
    }
    if (ok) {
      sh.stat[cq][r] = rmax;
      ok = softmax_sync(711);
      if (ok) {
        rmax = fmaxf(fmaxf(sh.stat[0][r], sh.stat[1][r]), fmaxf(sh.stat[2][r], sh.stat[3][r]));
        ok = softmax_sync(712);   // everyone has read before `stat` is reused
      }
    }
    const float m_s = rmax == -INFINITY ? 0.f : rmax * p.scale_log2e;
    // ---- pass 2: P = exp2(S * scale_log2e - max), row sums, P to shared memory ----
    float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
    for (int j = 0; ok && j < n; ++j) {
      const int sb = j & 1, use = ((j & 1) ? u1_1 : u1_0) + (j >> 1), pb = j & 1;
      if (!mbar_wait(&sh.sfull[sb], use & 1, abortp, p.error_word, 702)) { ok = false; break; }
      fence_after_sync();
      tmem_ld32_issue(lane_base + sb * 128, ra);
      tmem_ld32_wait(ra);
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.sempty[sb]);
      const int key0 = j * 128 + cq * 32;
      const bool full_vis = key0 + 31 <= lim;
      uint32_t pk[16];   // 32 values of P, packed in pairs
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        float a0 = ex2f(fmaf(__uint_as_float(ra[i]), p.scale_log2e, -m_s));
        float a1 = ex2f(fmaf(__uint_as_float(ra[i + 1]), p.scale_log2e, -m_s));
        float a2 = ex2f(fmaf(__uint_as_float(ra[i + 2]), p.scale_log2e, -m_s));
        float a3 = ex2f(fmaf(__uint_as_float(ra[i + 3]), p.scale_log2e, -m_s));
        if (!full_vis) {
          if (key0 + i > lim) a0 = 0.f;
          if (key0 + i + 1 > lim) a1 = 0.f;
          if (key0 + i + 2 > lim) a2 = 0.f;
          if (key0 + i + 3 > lim) a3 = 0.f;
        }
        l0 += a0; l1 += a1; l2 += a2; l3 += a3;
        const typename Pair<T>::V pa = Pair<T>::pack(a0, a1), pq = Pair<T>::pack(a2, a3);
        pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&pa);
        pk[(i >> 1) + 1] = *reinterpret_cast<const uint32_t*>(&pq);
      }
      // the V tile's rows past the end of the sequence become zeros (0 * garbage could be NaN)
      if ((j + 1) * 128 > lk) {
        const int t = base2 + 2 * j + 1, s = t % PT_NRING, k = t / PT_NRING;
        if (!mbar_wait(&sh.full[s], k & 1, abortp, p.error_word, 703)) { ok = false; break; }
        unsigned char* vt = ring + s * PT_TILE_BYTES;
        const int first = lk - j * 128;   // first row to clear
        // 512 threads: row (first + i), 16-byte chunk c of both blocks
        for (int idx = threadIdx.x - 64; idx < (128 - first) * 16; idx += 512) {
          const int row = first + (idx >> 4), c = idx & 15;
          *reinterpret_cast<int4*>(vt + (c >> 3) * PT_BLK_BYTES + row * 128 + ((c & 7) << 4)) = make_int4(0, 0, 0, 0);
        }
      }
      if (!mbar_wait(&sh.pempty[pb], ((j >> 1) & 1) ^ 1, abortp, p.error_word, 704)) { ok = false; break; }
      // keys cq*32 .. +31 of the row -> 16 columns of the P tile in TMEM (the A operand of P.V)
      fence_after_sync();
      tmem_st16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + PT_PCOL + pb * 64 + cq * 16, pk);
      tmem_st_wait();
      if ((j + 1) * 128 > lk) fence_proxy_async();   // the zeros written into the V tile above
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.pfull[pb]);
    }
    // ---- output ----
    float l = (l0 + l1) + (l2 + l3);
    if (ok) {
      sh.stat[cq][r] = l;
      ok = softmax_sync(713);
      if (ok) {
        l = (sh.stat[0][r] + sh.stat[1][r]) + (sh.stat[2][r] + sh.stat[3][r]);
        ok = mbar_wait(&sh.ofull, 0, abortp, p.error_word, 705);
      }
    }
    if (ok) {
      fence_after_sync();
      tmem_ld32_issue(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + 256 + cq * 32, ra);
      tmem_ld32_wait(ra);
      if (r < rows) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        T* o = reinterpret_cast<T*>(p.out) + ((int64_t)(q0 + qi0 + r) * p.Hq + h) * 128 + cq * 32;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t w0[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const typename Pair<T>::V x = Pair<T>::pack(__uint_as_float(ra[8 * c + 2 * i]) * inv,
                                                        __uint_as_float(ra[8 * c + 2 * i + 1]) * inv);
            w0[i] = *reinterpret_cast<const uint32_t*>(&x);
          }
          *reinterpret_cast<int4*>(o + 8 * c) = make_int4((int)w0[0], (int)w0[1], (int)w0[2], (int)w0[3]);
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

// ------------------------------------------------------------------------------------------------
// The same algorithm on 256-key tiles in BOTH passes (dense K/V, or pages of a multiple of 256
// keys): S = Q K^T as M128 N256 products (the shape that runs at the tensor pipe's full rate),
// P.V as sixteen K = 16 steps over 256 keys, half as many hand-offs per key.  A 256-key tile is two
// adjacent ring stages (one 64-dim block of the 256 keys each); the ring has six stages.
// TMEM, pass 1: two S tiles of 256 columns; pass 2: S (256 columns), O (128), P (128).  In pass 2
// S and P are single tiles: S is free again as soon as the softmax warps hold it in registers,
// P once its product is done, so S of tile J+1 is computed while the softmax works on tile J.
// ------------------------------------------------------------------------------------------------
constexpr int PW_NRING = 6;
constexpr int PW_SLACK = 128;   // alignment padding the launch provides for

struct __align__(16) PwShared {
  uint64_t qfull, full[PW_NRING], empty[PW_NRING], sfull[2], sempty[2], pfull, pempty, ofull, sbar;
  float stat[4][128];
  uint32_t tmem_base;
  int abort_flag;
};

template <typename T>
__global__ void __launch_bounds__(PT_THREADS, 1)
prefill_tc_wide_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK2,
                       const __grid_constant__ CUtensorMap tmV2, const PtParams p) {
  const int b = blockIdx.z, h = blockIdx.y;
  const int q0 = p.cu_q[b], lq = p.cu_q[b + 1] - q0;
  const int k0 = p.cu_k[b], lk = p.cu_k[b + 1] - k0;
  const int nqt = (lq + 127) >> 7;
  if ((int)blockIdx.x >= nqt) return;
  const int qt = nqt - 1 - blockIdx.x;          // the tiles with the most keys start first
  const int qi0 = qt * 128;
  const int hk = h / (p.Hq / p.Hkv);
  const int shift = lk - lq;                    // query i sees keys j <= i + shift
  const int rows = min(128, lq - qi0);
  const int kmax = min(lk, qi0 + rows + shift); // keys any row of the tile can see
  const int n = kmax > 0 ? (kmax + 255) >> 8 : 0;   // 256-key tiles
  // S tile bookkeeping: pass-1 tile J -> TMEM tile J & 1, its (J >> 1)-th use; pass 2 uses tile 0
  // only, J-th use after the u1_0 of pass 1
  const int u1_0 = (n + 1) >> 1, u1_1 = n >> 1;

  // The tiles need 1024-byte alignment and all but ~3 KB of the SM's shared memory, so there is no
  // room for a full kilobyte of alignment slack: the declaration asks for the alignment, and a base
  // that is not aligned after all (more than PW_SLACK bytes of padding) is reported, not used.
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* bufs = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if (bufs - smem_raw > PW_SLACK) {
    if (threadIdx.x == 0) atomicCAS(p.error_word, 0, 500);
    return;
  }
  unsigned char* qbuf = bufs;
  unsigned char* ring = bufs + PT_TILE_BYTES;
  PwShared& sh = *reinterpret_cast<PwShared*>(ring + PW_NRING * PT_TILE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (n == 0) {   // nothing visible: zeros
    if (warp >= 2) {
      const int t = threadIdx.x - 64;           // 512 threads: row t >> 2, quarter t & 3
      const int r = t >> 2;
      if (r < rows) {
        T* o = reinterpret_cast<T*>(p.out) + ((int64_t)(q0 + qi0 + r) * p.Hq + h) * 128 + (t & 3) * 32;
        for (int i = 0; i < 32; i += 8) *reinterpret_cast<int4*>(o + i) = make_int4(0, 0, 0, 0);
      }
    }
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(&sh.qfull, 1);
    for (int i = 0; i < PW_NRING; ++i) { mbar_init(&sh.full[i], 1); mbar_init(&sh.empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sh.sfull[i], 1); mbar_init(&sh.sempty[i], 16); }
    mbar_init(&sh.pfull, 16);
    mbar_init(&sh.pempty, 1);
    mbar_init(&sh.ofull, 1);
    mbar_init(&sh.sbar, 16);
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
  constexpr uint32_t IDESC_S = idesc_f16(UmmaFmt<T>::fmt, 128, 256);
  constexpr uint32_t IDESC_PV = idesc_f16(UmmaFmt<T>::fmt, 128, 128) | (1u << 16);   // B operand MN-major
  constexpr uint32_t O_COL = 256, P_COL = 384;

  // ring positions (pairs of stages): pass 1: K_J -> 2J; pass 2: K_J -> 2n + 4J, V_J -> 2n + 4J + 2
  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      prefetch_tensormap(&tmQ);
      prefetch_tensormap(&tmK2);
      prefetch_tensormap(&tmV2);
      mbar_arrive_expect_tx(&sh.qfull, PT_TILE_BYTES);
      tma_load_5d(qbuf, &tmQ, &sh.qfull, 0, h, q0 + qi0, 0, 0);
      tma_load_5d(qbuf + PT_BLK_BYTES, &tmQ, &sh.qfull, 64, h, q0 + qi0, 0, 0);
      bool ok = true;
      auto load = [&](int t, const CUtensorMap* tm, int J) -> bool {   // t even: stages s and s + 1
        const int s = t % PW_NRING, k = t / PW_NRING;
        if (!mbar_wait<true>(&sh.empty[s], (k & 1) ^ 1, abortp, p.error_word, 501) ||
            !mbar_wait<true>(&sh.empty[s + 1], (k & 1) ^ 1, abortp, p.error_word, 502)) return false;
        int c2, c3;
        if (p.table) {   // the page size is a multiple of 256
          c2 = (J * 256) % p.BS;
          c3 = p.table[(int64_t)b * p.NBmax + (J * 256) / p.BS];
        } else {
          c2 = k0 + J * 256;
          c3 = 0;
        }
        // one 64-dim block of the 256 keys per stage, each on its own stage barrier
        mbar_arrive_expect_tx(&sh.full[s], PT_TILE_BYTES);
        tma_load_5d(ring + s * PT_TILE_BYTES, tm, &sh.full[s], 0, hk, c2, c3, 0);
        mbar_arrive_expect_tx(&sh.full[s + 1], PT_TILE_BYTES);
        tma_load_5d(ring + (s + 1) * PT_TILE_BYTES, tm, &sh.full[s + 1], 64, hk, c2, c3, 0);
        return true;
      };
      for (int J = 0; ok && J < n; ++J) ok = load(2 * J, &tmK2, J);
      for (int J = 0; ok && J < n; ++J) {
        ok = load(2 * n + 4 * J, &tmK2, J);
        if (ok) ok = load(2 * n + 4 * J + 2, &tmV2, J);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      bool ok = mbar_wait(&sh.qfull, 0, abortp, p.error_word, 601);
      const uint32_t q_addr = smem_u32(qbuf);
      auto wait_pair = [&](int t, int where) -> bool {
        const int s = t % PW_NRING, k = t / PW_NRING;
        return mbar_wait(&sh.full[s], k & 1, abortp, p.error_word, where) &&
               mbar_wait(&sh.full[s + 1], k & 1, abortp, p.error_word, where + 1);
      };
      auto issue_s = [&](int sb, int use, int t) -> bool {   // S into TMEM tile sb (its `use`-th use)
        if (!wait_pair(t, 602)) return false;
        if (!mbar_wait(&sh.sempty[sb], (use & 1) ^ 1, abortp, p.error_word, 604)) return false;
        fence_after_sync();
        const int s = t % PW_NRING;
        umma_k128(tmem_base + sb * 256, q_addr, PT_BLK_BYTES, smem_u32(ring + s * PT_TILE_BYTES), PT_TILE_BYTES,
                  IDESC_S);
        umma_commit(&sh.sfull[sb]);
        umma_commit(&sh.empty[s]);
        umma_commit(&sh.empty[s + 1]);
        return true;
      };
      for (int J = 0; ok && J < n; ++J) ok = issue_s(J & 1, J >> 1, 2 * J);
      // pass 2 lays O and P over the second S tile of pass 1: it must have been read to the end
      if (ok && u1_1 > 0) ok = mbar_wait(&sh.sempty[1], (u1_1 - 1) & 1, abortp, p.error_word, 608);
      if (ok) ok = issue_s(0, u1_0, 2 * n);
      for (int J = 0; ok && J < n; ++J) {
        if (J + 1 < n) ok = issue_s(0, u1_0 + J + 1, 2 * n + 4 * (J + 1));   // S of the next tile first
        if (!ok) break;
        const int t = 2 * n + 4 * J + 2, s = t % PW_NRING;
        if (!wait_pair(t, 605)) { ok = false; break; }
        if (!mbar_wait(&sh.pfull, J & 1, abortp, p.error_word, 607)) { ok = false; break; }
        fence_after_sync();
        const uint32_t v_addr = smem_u32(ring + s * PT_TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < 16; ++ks) {   // 16 keys per step: 8 columns of P
          const uint64_t bd = smem_desc_sw128_mn(v_addr + ks * 2048, PT_TILE_BYTES, 1024);
          umma_f16_ts(tmem_base + O_COL, tmem_base + P_COL + ks * 8, bd, IDESC_PV, (J | ks) ? 1u : 0u);
        }
        umma_commit(&sh.pempty);
        umma_commit(&sh.empty[s]);
        umma_commit(&sh.empty[s + 1]);
      }
      if (ok) umma_commit(&sh.ofull);
    }
  } else {
    // ---------------- softmax ----------------
    const int q = warp & 3;               // TMEM lane quadrant
    const int cq = (warp - 2) >> 2;       // column quarter: keys cq*64 .. +63 of a tile; dims cq*32 .. of O
    const int r = q * 32 + lane;          // query row of the tile
    const int lim = r < rows ? min(lk - 1, qi0 + r + shift) : -1;   // last visible key (-1: none)
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    bool ok = true;
    uint32_t sph = 0;
    auto softmax_sync = [&](int where) -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.sbar);
      const bool ok_ = mbar_wait(&sh.sbar, sph & 1, abortp, p.error_word, where);
      ++sph;
      return ok_;
    };
    uint32_t ra[32];
    // ---- pass 1: row maxima of the raw products ----
    float rmax = -INFINITY;
    auto row_max32 = [&](const uint32_t (&v)[32], int key0) {   // 32 keys from key0 on
      if (key0 + 31 <= lim) {
        float m0 = rmax, m1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          m0 = fmax3(m0, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
          m1 = fmax3(m1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
        }
        rmax = fmaxf(m0, m1);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (key0 + i <= lim) rmax = fmaxf(rmax, __uint_as_float(v[i]));
      }
    };
    for (int J = 0; ok && J < n; ++J) {
      const int sb = J & 1, use = J >> 1;
      if (!mbar_wait(&sh.sfull[sb], use & 1, abortp, p.error_word, 701)) { ok = false; break; }
      fence_after_sync();
      uint32_t rb[32];
      const uint32_t tb = lane_addr + sb * 256 + cq * 64;
      tmem_ld32_issue(tb, ra);
      tmem_ld32_issue(tb + 32, rb);
      tmem_ld32_wait(ra);
      tmem_ld32_wait(rb);
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.sempty[sb]);
      row_max32(ra, J * 256 + cq * 64);
      row_max32(rb, J * 256 + cq * 64 + 32);
    }
    if (ok) {
      sh.stat[cq][r] = rmax;
      ok = softmax_sync(711);
      if (ok) {
        rmax = fmaxf(fmaxf(sh.stat[0][r], sh.stat[1][r]), fmaxf(sh.stat[2][r], sh.stat[3][r]));
        ok = softmax_sync(712);   // everyone has read before `stat` is reused
      }
    }
    const float m_s = rmax == -INFINITY ? 0.f : rmax * p.scale_log2e;
    // ---- pass 2: P = exp2(S * scale_log2e - max), row sums, P to TMEM ----
    float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
    auto exp32 = [&](const uint32_t (&v)[32], int key0, uint32_t (&pk)[16]) {   // 32 keys -> 16 packed pairs
      const bool full_vis = key0 + 31 <= lim;
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        float a0 = ex2f(fmaf(__uint_as_float(v[i]), p.scale_log2e, -m_s));
        float a1 = ex2f(fmaf(__uint_as_float(v[i + 1]), p.scale_log2e, -m_s));
        float a2 = ex2f(fmaf(__uint_as_float(v[i + 2]), p.scale_log2e, -m_s));
        float a3 = ex2f(fmaf(__uint_as_float(v[i + 3]), p.scale_log2e, -m_s));
        if (!full_vis) {
          if (key0 + i > lim) a0 = 0.f;
          if (key0 + i + 1 > lim) a1 = 0.f;
          if (key0 + i + 2 > lim) a2 = 0.f;
          if (key0 + i + 3 > lim) a3 = 0.f;
        }
        l0 += a0; l1 += a1; l2 += a2; l3 += a3;
        const typename Pair<T>::V pa = Pair<T>::pack(a0, a1), pq = Pair<T>::pack(a2, a3);
        pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&pa);
        pk[(i >> 1) + 1] = *reinterpret_cast<const uint32_t*>(&pq);
      }
    };
    for (int J = 0; ok && J < n; ++J) {
      if (!mbar_wait(&sh.sfull[0], (u1_0 + J) & 1, abortp, p.error_word, 702)) { ok = false; break; }
      fence_after_sync();
      const uint32_t tb = lane_addr + cq * 64;
      const int key0 = J * 256 + cq * 64;
      uint32_t pka[16], pkb[16];
      tmem_ld32_issue(tb, ra);
      tmem_ld32_wait(ra);
      exp32(ra, key0, pka);
      tmem_ld32_issue(tb + 32, ra);
      tmem_ld32_wait(ra);
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.sempty[0]);   // S is in registers: the next S may be computed
      exp32(ra, key0 + 32, pkb);
      // the V tile's rows past the end of the sequence become zeros (0 * garbage could be NaN)
      if ((J + 1) * 256 > lk) {
        const int t = 2 * n + 4 * J + 2, s = t % PW_NRING, k = t / PW_NRING;
        if (!mbar_wait(&sh.full[s], k & 1, abortp, p.error_word, 703) ||
            !mbar_wait(&sh.full[s + 1], k & 1, abortp, p.error_word, 704)) { ok = false; break; }
        unsigned char* vt = ring + s * PT_TILE_BYTES;   // stage s: dims 0-63, stage s + 1: dims 64-127
        const int first = lk - J * 256;   // first row to clear
        for (int idx = threadIdx.x - 64; idx < (256 - first) * 16; idx += 512) {
          const int row = first + (idx >> 4), c = idx & 15;
          *reinterpret_cast<int4*>(vt + (c >> 3) * PT_TILE_BYTES + row * 128 + ((c & 7) << 4)) = make_int4(0, 0, 0, 0);
        }
      }
      if (!mbar_wait(&sh.pempty, (J & 1) ^ 1, abortp, p.error_word, 705)) { ok = false; break; }
      // keys cq*64 .. +63 of the row -> 32 columns of the P tile (the A operand of P.V)
      fence_after_sync();
      tmem_st16(lane_addr + P_COL + cq * 32, pka);
      tmem_st16(lane_addr + P_COL + cq * 32 + 16, pkb);
      tmem_st_wait();
      if ((J + 1) * 256 > lk) fence_proxy_async();   // the zeros written into the V tile above
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.pfull);
    }
    // ---- output ----
    float l = (l0 + l1) + (l2 + l3);
    if (ok) {
      sh.stat[cq][r] = l;
      ok = softmax_sync(713);
      if (ok) {
        l = (sh.stat[0][r] + sh.stat[1][r]) + (sh.stat[2][r] + sh.stat[3][r]);
        ok = mbar_wait(&sh.ofull, 0, abortp, p.error_word, 706);
      }
    }
    if (ok) {
      fence_after_sync();
      tmem_ld32_issue(lane_addr + O_COL + cq * 32, ra);
      tmem_ld32_wait(ra);
      if (r < rows) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        T* o = reinterpret_cast<T*>(p.out) + ((int64_t)(q0 + qi0 + r) * p.Hq + h) * 128 + cq * 32;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t w0[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const typename Pair<T>::V x = Pair<T>::pack(__uint_as_float(ra[8 * c + 2 * i]) * inv,
                                                        __uint_as_float(ra[8 * c + 2 * i + 1]) * inv);
            w0[i] = *reinterpret_cast<const uint32_t*>(&x);
          }
          *reinterpret_cast<int4*>(o + 8 * c) = make_int4((int)w0[0], (int)w0[1], (int)w0[2], (int)w0[3]);
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
static int launch_prefill_tc(const void* q, const void* k, const void* v, const PtParams& p,
                             int max_seqlen_q, int64_t kv_stride_page, cudaStream_t st) {
  CUtensorMap tmQ, tmK, tmK2, tmV, tmV2;
  const uint32_t box[5] = {64, 1, 128, 1, 1}, box2[5] = {64, 1, 256, 1, 1};
  const bool wide = !p.table || p.BS % 256 == 0;   // a 256-key tile never straddles a page
  {
    const uint64_t dims[5] = {128, (uint64_t)p.Hq, (uint64_t)p.total_q, 1, 1};
    const uint64_t strides[4] = {128, (uint64_t)p.Hq * 128, (uint64_t)p.Hq * 128, (uint64_t)p.Hq * 128};
    int rc = make_tensor_map_5d(&tmQ, UmmaFmt<T>::tm, q, dims, strides, box, sizeof(T));
    if (rc) return rc;
  }
  for (int which = 0; which < 4; ++which) {   // K (128-key box), K (256-key box), V, V (256-key box)
    const void* base = which >= 2 ? v : k;
    CUtensorMap* tm = which == 0 ? &tmK : (which == 1 ? &tmK2 : (which == 2 ? &tmV : &tmV2));
    const uint32_t* bx = (which & 1) ? box2 : box;
    int rc;
    if (p.table) {
      const uint64_t dims[5] = {128, (uint64_t)p.Hkv, (uint64_t)p.BS, 1ull << 30, 1};
      const uint64_t strides[4] = {128, (uint64_t)p.Hkv * 128, (uint64_t)kv_stride_page, (uint64_t)kv_stride_page};
      rc = make_tensor_map_5d(tm, UmmaFmt<T>::tm, base, dims, strides, (which & 1) && !wide ? box : bx, sizeof(T));
    } else {
      const uint64_t dims[5] = {128, (uint64_t)p.Hkv, (uint64_t)p.total_k, 1, 1};
      const uint64_t strides[4] = {128, (uint64_t)p.Hkv * 128, (uint64_t)p.Hkv * 128, (uint64_t)p.Hkv * 128};
      rc = make_tensor_map_5d(tm, UmmaFmt<T>::tm, base, dims, strides, bx, sizeof(T));
    }
    if (rc) return rc;
  }
  const size_t smem = (1 + PT_NRING) * PT_TILE_BYTES + sizeof(PtShared) + 1024;
  dim3 grid((max_seqlen_q + 127) / 128, p.Hq, p.B);
  if (wide) {
    const size_t smem2 = (1 + PW_NRING) * PT_TILE_BYTES + sizeof(PwShared) + PW_SLACK;
    auto kern2 = prefill_tc_wide_kernel<T>;
    cudaError_t e2 = cudaFuncSetAttribute(kern2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
    if (e2 != cudaSuccess) { set_error("zp_varlen_prefill(tcgen05): %s", cudaGetErrorString(e2)); return ZP_ERR_CUDA; }
    kern2<<<grid, PT_THREADS, smem2, st>>>(tmQ, tmK2, tmV2, p);
    return check_launch("zp_varlen_prefill(tcgen05, 256-key tiles)");
  }
  auto kern = prefill_tc_kernel<T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_error("zp_varlen_prefill(tcgen05): %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  kern<<<grid, PT_THREADS, smem, st>>>(tmQ, tmK, tmV, p);
  return check_launch("zp_varlen_prefill(tcgen05)");
}

// Called by zp_varlen_prefill_ex (zp_prefill.cu).
// total_q / total_k: rows of q and (dense case) of k and v.
int varlen_prefill_tc(const void* q, const void* k, const void* v, const int32_t* cu_q, const int32_t* cu_k,
                      const int32_t* table, void* out, int B, int max_seqlen_q, int NBmax, int Hq, int Hkv,
                      int BS, int64_t kv_stride_page, float scale_log2e, int total_q, int total_k, int dtype,
                      cudaStream_t st) {
  PtParams p{};
  p.total_q = total_q; p.total_k = total_k;
  p.cu_q = cu_q; p.cu_k = cu_k; p.table = table; p.out = out;
  p.error_word = device_error_word();
  p.B = B; p.NBmax = NBmax; p.Hq = Hq; p.Hkv = Hkv; p.BS = BS; p.scale_log2e = scale_log2e;
  if (!p.error_word) { set_error("zp_varlen_prefill(tcgen05): no device error word"); return ZP_ERR_CUDA; }
  if (dtype == ZP_DTYPE_BF16)
    return launch_prefill_tc<__nv_bfloat16>(q, k, v, p, max_seqlen_q, kv_stride_page, st);
  if (dtype == ZP_DTYPE_F16)
    return launch_prefill_tc<__half>(q, k, v, p, max_seqlen_q, kv_stride_page, st);
  set_error("zp_varlen_prefill(tcgen05): 16-bit tensors only");
  return ZP_ERR_UNSUPPORTED;
}

}  // namespace zp
