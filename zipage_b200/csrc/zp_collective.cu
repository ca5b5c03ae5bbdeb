// Tensor-parallel all-reduce over NVLink peer memory, with the residual add + RMSNorm that follows
// it in a decoder block fused into the same kernel.
//
// Replaces, for the row-parallel projections of a decode step, `dist.all_reduce(y)` of
// RowParallelLinear.forward (third_party/nanovllm/layers/linear.py:149-153) and, fused, the
// `RMSNorm.add_rms_forward` that consumes its result (third_party/nanovllm/layers/layernorm.py:
// 28-40; call sites third_party/nanovllm/models/qwen3.py:146-152).
//
// Every rank owns one segment of device memory that all ranks of the node map (CUDA IPC, or any
// mapping the caller attaches): [flags | 2 parities x (one input slot per source rank, a result
// area)].  One launch:
//   1. each block stores its rows of the input into slot `rank` of every rank's segment (one-shot)
//      or of the segment of the rank that owns each 512-byte chunk (two-shot): posted writes over
//      the link, no round trip,
//   2. meets the same block of every peer (a flag per (phase, source rank, block) written into
//      the peer's segment with release/system scope, polled locally, then an acquire fence),
//   3. one-shot: sums its rows over the local slots in fp32 in rank order (so every rank gets the
//      same bits), rounding to T once;
//      two-shot: each rank sums only the chunks it owns and stores the result into every rank's
//      result area, the blocks meet again, and each reads its rows from its own result area,
//   4. writes the sum, or (fused) adds the residual, writes the new residual, and writes the
//      RMS-normalised, weighted row — the same arithmetic as the stand-alone RMSNorm kernel.
// The two parities alternate between calls, so a rank may start the next call while a peer still
// reads this call's areas; a rank reaches the call after that only after meeting every peer in the
// call between, by which time the peer's earlier kernel has ended.
//
// Every wait is bounded (wall-clock limit given at creation): when it runs out the kernel records
// ZP_COMM_TIMEOUT in the communicator's status word and finishes without waiting further.  The
// failure is sticky: every wait looks at the status word first and from time to time while it
// polls, so the other waits of that launch and all waits of later launches return at once (a lost
// peer costs about one time limit in total, not one per wait).  The
// result of that call is undefined and the communicator must be destroyed and built again, but
// the context stays usable.  Blocks only ever wait for the block of the same index on the peers,
// and a launch has at most one block per SM, so on a GPU otherwise free of spinning kernels every
// waiting block's partner gets to run.
#include "zp_common.cuh"

#include <algorithm>
#include <cstring>
#include <new>

namespace zp { namespace coll {

constexpr int MAX_WORLD = 8;
constexpr int MAX_BLOCKS = 256;
constexpr int THREADS = 512;
constexpr int VPT = 2;                                   // 16-byte vectors of a row per thread
constexpr size_t FLAG_BYTES = 2 * MAX_WORLD * MAX_BLOCKS * sizeof(uint32_t);
constexpr int STATUS_TIMEOUT = 1;

struct Dev {
  char* seg[MAX_WORLD];     // every rank's segment as mapped here (seg[rank] is the local one)
  uint32_t* state;          // local only: [0] epoch, [1] blocks done, [2] status
  size_t area_bytes;
  size_t ll_bytes;          // payload capacity of one flagged-line slot (0: none)
  long long timeout_ns;
  int rank, world;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ long long now_ns() {
  long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// The communicator's status word, read past the caches.  Once a wait has run out it stays non-zero
// until the communicator is destroyed: every later wait, in this launch and in every launch that
// follows (a replayed decode graph issues dozens), gives up at its first look instead of spending
// its own time limit, so a lost peer costs about one limit in total.
__device__ __forceinline__ bool comm_failed(const uint32_t* state) {
  return *reinterpret_cast<const volatile uint32_t*>(state + 2) != 0u;
}
__device__ __forceinline__ int4 ld16_l2(const void* p) {   // L2 only: the line may be a peer's write
  return __ldcg(reinterpret_cast<const int4*>(p));
}
// `seg`: the segment pointers in shared memory (a kernel parameter array indexed by a run-time
// value would be copied to the stack)
__device__ __forceinline__ uint32_t* flag_of(char* const* seg, int owner, int phase, int src, int blk) {
  return reinterpret_cast<uint32_t*>(seg[owner]) + (phase * MAX_WORLD + src) * MAX_BLOCKS + blk;
}
// Area `which` of `owner`'s segment: 0..world-1 = the input slot written by that source rank,
// world = the result area of the two-shot form.
__device__ __forceinline__ char* area_of(char* const* seg, size_t area_bytes, int world, int owner,
                                         uint32_t parity, int which) {
  return seg[owner] + FLAG_BYTES + (size_t)(parity * (world + 1) + which) * area_bytes;
}

// Flagged lines (mode 2): a 16-byte store carries two 4-byte payload words, each followed by the
// call's epoch, so the data announces itself — no fence, no separate flag, no meeting; it relies on
// 8-byte stores arriving whole.  A payload vector of 16 bytes becomes two such lines.  Slot
// (parity, source rank) of `owner`'s segment, after the areas:
__device__ __forceinline__ char* ll_of(char* const* seg, size_t area_bytes, size_t ll_bytes, int world, int owner,
                                       uint32_t parity, int src) {
  return seg[owner] + FLAG_BYTES + 2 * (size_t)(world + 1) * area_bytes +
         (size_t)(parity * world + src) * 2 * ll_bytes;
}
__device__ __forceinline__ uint4 ld_volatile16(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// Wait (bounded) for the two lines of payload vector `v` of a slot; returns the 16 payload bytes.
__device__ __forceinline__ int4 ll_read(const Dev& c, const char* slot, int64_t v, uint32_t epoch) {
  const char* p = slot + v * 32;
  uint4 a = ld_volatile16(p), b = ld_volatile16(p + 16);
  if (a.y != epoch || a.w != epoch || b.y != epoch || b.w != epoch) {
    if (comm_failed(c.state)) return make_int4((int)a.x, (int)a.z, (int)b.x, (int)b.z);
    const long long t0 = now_ns();
    uint32_t spins = 0;
    do {
      a = ld_volatile16(p); b = ld_volatile16(p + 16);
      if ((++spins & 255u) == 0) {
        if (comm_failed(c.state)) break;
        if (now_ns() - t0 > c.timeout_ns) {
          atomicCAS(c.state + 2, 0u, (uint32_t)STATUS_TIMEOUT);
          break;
        }
      }
    } while (a.y != epoch || a.w != epoch || b.y != epoch || b.w != epoch);
  }
  return make_int4((int)a.x, (int)a.z, (int)b.x, (int)b.z);
}

// Wait (bounded) for one line {a, epoch, b, epoch}; returns (a, b).
__device__ __forceinline__ uint2 ll_read_line(const Dev& c, const char* p, uint32_t epoch) {
  uint4 a = ld_volatile16(p);
  if (a.y != epoch || a.w != epoch) {
    if (comm_failed(c.state)) return make_uint2(a.x, a.z);
    const long long t0 = now_ns();
    uint32_t spins = 0;
    do {
      a = ld_volatile16(p);
      if ((++spins & 255u) == 0) {
        if (comm_failed(c.state)) break;
        if (now_ns() - t0 > c.timeout_ns) {
          atomicCAS(c.state + 2, 0u, (uint32_t)STATUS_TIMEOUT);
          break;
        }
      }
    } while (a.y != epoch || a.w != epoch);
  }
  return make_uint2(a.x, a.z);
}

__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// All threads of the block have issued their stores; meet the same block of every peer.  The
// block barrier orders every thread's stores before the signalling thread's release (which is
// cumulative), and the signalling thread's acquire fence before every thread's later loads, so
// only the threads that signal pay for system-scope fences; the poll itself is a relaxed load.
__device__ __forceinline__ void meet_peers(const Dev& c, char* const* seg, int phase, uint32_t epoch, int blk) {
  __syncthreads();
  const int t = threadIdx.x;
  if (t < c.world && t != c.rank) {
    st_release_sys(flag_of(seg, t, phase, c.rank, blk), epoch);
    const uint32_t* mine = flag_of(seg, c.rank, phase, t, blk);
    const long long t0 = now_ns();
    uint32_t spins = 0;
    while ((int32_t)(ld_relaxed_sys(mine) - epoch) < 0) {
      if ((++spins & 1023u) == 1u && comm_failed(c.state)) break;   // first look, then every 1024th
      if (spins > 4096u) {
        __nanosleep(64);
        if ((spins & 63u) == 0 && now_ns() - t0 > c.timeout_ns) {
          atomicCAS(c.state + 2, 0u, (uint32_t)STATUS_TIMEOUT);
          break;
        }
      }
    }
    asm volatile("fence.acq_rel.sys;" ::: "memory");
  }
  __syncthreads();
}

template <typename T> struct Pack {
  static constexpr int N = 16 / sizeof(T);
  int4 raw;
  __device__ __forceinline__ float get(int i) const { return Elem<T>::to_f32(reinterpret_cast<const T*>(&raw)[i]); }
  __device__ __forceinline__ void set(int i, float v) { reinterpret_cast<T*>(&raw)[i] = Elem<T>::from_f32(v); }
};

// Rows of `row_vecs` 16-byte vectors (<= THREADS * VPT); row r belongs to block r % gridDim.x.
// `blk` of `nblk`: this block's index among the rank's blocks (the x dimension of the grid).
// MODE 0: one-shot, 1: two-shot, 2: flagged lines (one-shot without a meeting).
template <typename T, int WORLD, int MODE, bool FUSED>
__device__ __forceinline__ void
all_reduce_body(const Dev& c, const int blk, const int nblk, const T* in, T* out, int64_t nvec, int row_vecs,
                int64_t nrows, const T* residual, const T* __restrict__ weight, T* residual_out, float eps) {
  constexpr int EPV = Pack<T>::N;
  constexpr bool TWO_SHOT = MODE == 1, LL = MODE == 2;
  __shared__ uint32_t s_epoch;
  __shared__ float red[32];
  __shared__ char* seg[MAX_WORLD];
  if (threadIdx.x == 0) {
    s_epoch = *reinterpret_cast<volatile uint32_t*>(c.state) + 1u;
#pragma unroll
    for (int r = 0; r < MAX_WORLD; ++r) seg[r] = c.seg[r];
  }
  __syncthreads();
  const uint32_t epoch = s_epoch, parity = epoch & 1u;
  // Push: the input goes straight into slot `rank` of the ranks that will sum it (one-shot: all of
  // them; two-shot: the owner of each 512-byte chunk), so that after the meeting every load of the
  // reduction is local and no round trip over the link is left on the critical path.
  for (int64_t row = blk; row < nrows; row += nblk) {
    const int64_t v0 = row * row_vecs, v1 = min(v0 + row_vecs, nvec);
    for (int64_t v = v0 + threadIdx.x; v < v1; v += THREADS) {
      const int4 x = ld16(reinterpret_cast<const char*>(in) + v * 16);
      if constexpr (LL) {
        const int4 la = make_int4(x.x, (int)epoch, x.y, (int)epoch), lb = make_int4(x.z, (int)epoch, x.w, (int)epoch);
#pragma unroll
        for (int r = 0; r < WORLD; ++r) {
          char* dst = ll_of(seg, c.area_bytes, c.ll_bytes, WORLD, r, parity, c.rank) + v * 32;
          st16(dst, la);
          st16(dst + 16, lb);
        }
      } else if constexpr (TWO_SHOT) {
        st16(area_of(seg, c.area_bytes, WORLD, (int)((v >> 5) % WORLD), parity, c.rank) + v * 16, x);
      } else {
#pragma unroll
        for (int r = 0; r < WORLD; ++r) st16(area_of(seg, c.area_bytes, WORLD, r, parity, c.rank) + v * 16, x);
      }
    }
  }
  if constexpr (!LL) meet_peers(c, seg, 0, epoch, blk);

  if constexpr (TWO_SHOT) {
    for (int64_t row = blk; row < nrows; row += nblk) {
      const int64_t v0 = row * row_vecs, v1 = min(v0 + row_vecs, nvec);
      for (int64_t v = v0 + threadIdx.x; v < v1; v += THREADS) {
        if ((int)((v >> 5) % WORLD) != c.rank) continue;   // 512-byte chunks, dealt round-robin
        Pack<T> x[WORLD], o;
#pragma unroll
        for (int r = 0; r < WORLD; ++r) x[r].raw = ld16_l2(area_of(seg, c.area_bytes, WORLD, c.rank, parity, r) + v * 16);
#pragma unroll
        for (int j = 0; j < EPV; ++j) {   // fp32 sum in rank order, one rounding
          float acc = x[0].get(j);
#pragma unroll
          for (int r = 1; r < WORLD; ++r) acc += x[r].get(j);
          o.set(j, acc);
        }
#pragma unroll
        for (int r = 0; r < WORLD; ++r) st16(area_of(seg, c.area_bytes, WORLD, r, parity, WORLD) + v * 16, o.raw);
      }
    }
    meet_peers(c, seg, 1, epoch, blk);
  }

  // The raw vectors of the block's next row are requested before the current row is summed and
  // normalised.
  constexpr int NSRC = TWO_SHOT ? 1 : WORLD;
  const char* src[NSRC];
#pragma unroll
  for (int r = 0; r < NSRC; ++r)
    src[r] = LL ? ll_of(seg, c.area_bytes, c.ll_bytes, WORLD, c.rank, parity, r)
                : area_of(seg, c.area_bytes, WORLD, c.rank, parity, TWO_SHOT ? WORLD : r);
  Pack<T> raw[VPT][NSRC];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int r = 0; r < NSRC; ++r) raw[i][r].raw = make_int4(0, 0, 0, 0);
  auto request = [&](int64_t row) {
    const int64_t v0 = row * row_vecs, v1 = min(v0 + row_vecs, nvec);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int64_t v = v0 + threadIdx.x + i * THREADS;
      if (v < v1) {
#pragma unroll
        for (int r = 0; r < NSRC; ++r)
          raw[i][r].raw = LL ? ll_read(c, src[r], v, epoch) : ld16_l2(src[r] + v * 16);
      }
    }
  };
  if ((int64_t)blk < nrows) request(blk);
  for (int64_t row = blk; row < nrows; row += nblk) {
    const int64_t v0 = row * row_vecs, v1 = min(v0 + row_vecs, nvec);
    Pack<T> x[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      if constexpr (TWO_SHOT) {
        x[i] = raw[i][0];
      } else {   // fp32 sum in rank order, one rounding
#pragma unroll
        for (int j = 0; j < EPV; ++j) {
          float acc = raw[i][0].get(j);
#pragma unroll
          for (int r = 1; r < WORLD; ++r) acc += raw[i][r].get(j);
          x[i].set(j, acc);
        }
      }
    }
    if (row + nblk < nrows) request(row + nblk);
    if constexpr (!FUSED) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int64_t v = v0 + threadIdx.x + i * THREADS;
        if (v < v1) st16(reinterpret_cast<char*>(out) + v * 16, x[i].raw);
      }
    } else {
      // s = x + residual (fp32); residual_out = T(s); y = T(T(s * rsqrt(mean(s^2) + eps)) * w)
      const int H = row_vecs * EPV;
      float s[VPT][EPV];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int64_t v = v0 + threadIdx.x + i * THREADS;
        if (v < v1) {
          Pack<T> b, o;
          b.raw = ld16(reinterpret_cast<const char*>(residual) + v * 16);
#pragma unroll
          for (int j = 0; j < EPV; ++j) {
            s[i][j] = x[i].get(j) + b.get(j);
            ss = fmaf(s[i][j], s[i][j], ss);
            o.set(j, s[i][j]);
          }
          st16(reinterpret_cast<char*>(residual_out) + v * 16, o.raw);
        }
      }
      ss = block_sum(ss, red);
      const float rinv = 1.f / sqrtf(ss / (float)H + eps);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int64_t v = v0 + threadIdx.x + i * THREADS;
        if (v < v1) {
          Pack<T> w, o;
          w.raw = ld16(reinterpret_cast<const char*>(weight) + (v - v0) * 16);
#pragma unroll
          for (int j = 0; j < EPV; ++j)
            o.set(j, __fmul_rn(round_to<T>(__fmul_rn(s[i][j], rinv)), w.get(j)));
          st16(reinterpret_cast<char*>(out) + v * 16, o.raw);
        }
      }
      __syncthreads();   // `red` is reused by the next row
    }
  }

  // the last block to finish advances the epoch for the next launch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(c.state + 1, 1u) == (uint32_t)nblk - 1) {
      c.state[1] = 0;
      c.state[0] = epoch;
      __threadfence();
    }
  }
}

// MODE 0: one-shot, 1: two-shot, 2: flagged lines (one-shot without a meeting).
template <typename T, int WORLD, int MODE, bool FUSED>
__global__ void __launch_bounds__(THREADS)
all_reduce_kernel(const Dev c, const T* in, T* out, int64_t nvec, int row_vecs, int64_t nrows,
                  const T* residual, const T* __restrict__ weight, T* residual_out, float eps) {
  all_reduce_body<T, WORLD, MODE, FUSED>(c, blockIdx.x, gridDim.x, in, out, nvec, row_vecs, nrows, residual,
                                             weight, residual_out, eps);
}

// Every rank of a world as one cooperative launch on ONE GPU: blockIdx.y is the rank, all blocks
// are resident at once, so the ranks' blocks can wait for one another.  Test support for world
// sizes for which no multi-GPU machine is at hand; the per-rank code is the body above, unchanged.
struct EmulatedWorld {
  Dev dev[MAX_WORLD];
  const void* in[MAX_WORLD];
  void* out[MAX_WORLD];
  void* residual_out[MAX_WORLD];
};

template <typename T, int WORLD, int MODE, bool FUSED>
__global__ void __launch_bounds__(THREADS)
all_reduce_emulated_kernel(const EmulatedWorld w, int64_t nvec, int row_vecs, int64_t nrows, const T* residual,
                           const T* __restrict__ weight, float eps) {
  __shared__ Dev c;
  if (threadIdx.x == 0) {
#pragma unroll
    for (int r = 0; r < WORLD; ++r)
      if (r == (int)blockIdx.y) c = w.dev[r];
  }
  __shared__ const void* in;
  __shared__ void* out;
  __shared__ void* res_out;
  if (threadIdx.x == 0) {
#pragma unroll
    for (int r = 0; r < WORLD; ++r)
      if (r == (int)blockIdx.y) { in = w.in[r]; out = w.out[r]; res_out = w.residual_out[r]; }
  }
  __syncthreads();
  all_reduce_body<T, WORLD, MODE, FUSED>(c, blockIdx.x, gridDim.x, (const T*)in, (T*)out, nvec, row_vecs, nrows,
                                             residual, weight, (T*)res_out, eps);
}

// ---------------------------------------------------------------------------------------------
// Sampler over a vocabulary sharded across the ranks, without gathering the logits.
// Every rank holds logits[:, rank * Vs : (rank + 1) * Vs].  One launch on every rank:
//   A. per row: the shard's maximum m_r of logits / t, then in one pass z_r = sum exp(x / t - m_r)
//      and the race e_i / q_i with fast arithmetic (the two best candidates per thread are kept in
//      shared memory); (m_r, z_r) pushed into every rank's segment as a flagged line;
//   B. per row: M = max m_r, Z = sum z_r exp(m_r - M) (rank order: the same bits everywhere); the
//      kept candidates re-evaluated with the reference's expression (exp(x / t - M) / Z) / q, the
//      shard's winner (value, global index) pushed into every rank's segment as a flagged line;
//   C. per row: the best of the ranks' winners (larger value, then lower index) -> tokens_out.
// All ranks end with the same tokens.  The draws of the built-in generator are keyed by the
// global index, so they do not depend on the sharding.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}
__device__ __forceinline__ float exp1_draw(uint64_t seed, uint32_t row, uint32_t i) {   // as zp_sample
  uint32_t h = mix32(((uint32_t)seed ^ (row * 0x9e3779b9u)) + i * 0x85ebca6bu);
  h = mix32(h ^ (uint32_t)(seed >> 32) ^ row);
  const float u = ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);
  return -__logf(u);
}

constexpr int SAMPLE_THREADS = 1024;
constexpr int SAMPLE_ROWS_PER_BLOCK = 4;
constexpr int SAMPLE_SMEM = SAMPLE_ROWS_PER_BLOCK * 2 * SAMPLE_THREADS * (int)sizeof(int2);   // 64 KB

template <typename T, int WORLD>
__device__ __forceinline__ void
sample_sharded_body(const Dev& c, const int blk, const int nblk, const T* __restrict__ logits,
                    const float* __restrict__ temperatures, const float* __restrict__ noise,
                    int64_t* __restrict__ out, int rows, int Vs, uint64_t seed, uint32_t row0) {
  // (index, draw) of the two best candidates per thread for each of the block's rows
  // (at most SAMPLE_ROWS_PER_BLOCK; `row0`: the first row's index in the caller's batch, which
  // keys the generator)
  extern __shared__ __align__(16) unsigned char sample_smem[];
  int2* cand = reinterpret_cast<int2*>(sample_smem);
  constexpr int EPV = Pack<T>::N;
  __shared__ uint32_t s_epoch;
  __shared__ char* seg[MAX_WORLD];
  __shared__ float red[32];
  __shared__ float bval[32];
  __shared__ int bidx[32];
  if (threadIdx.x == 0) {
    s_epoch = *reinterpret_cast<volatile uint32_t*>(c.state) + 1u;
#pragma unroll
    for (int r = 0; r < MAX_WORLD; ++r) seg[r] = c.seg[r];
  }
  __syncthreads();
  const uint32_t epoch = s_epoch, parity = epoch & 1u;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;

  auto for_each = [&](const T* lr, auto&& fn) {   // a thread sees its elements in ascending order
    const int nvec = ((uintptr_t)lr % 16 == 0) ? Vs / EPV : 0;
#pragma unroll 2
    for (int v = threadIdx.x; v < nvec; v += SAMPLE_THREADS) {
      Pack<T> a;
      a.raw = ld16(lr + v * EPV);
#pragma unroll
      for (int j = 0; j < EPV; ++j) fn(v * EPV + j, a.get(j));
    }
    for (int i = nvec * EPV + threadIdx.x; i < Vs; i += SAMPLE_THREADS) fn(i, Elem<T>::to_f32(lr[i]));
  };

  // ---- A: shard statistics, and the race against the shard's own maximum ----
  // (the order of the candidates does not depend on which maximum is subtracted; the two best per
  // thread wait in shared memory for the global statistics)
  int slot = 0;
  for (int row = blk; row < rows; row += nblk, ++slot) {
    const T* lr = logits + (int64_t)row * Vs;
    const float t = temperatures[row];
    float mx = -INFINITY;
    if (t > 0.f) {   // the correctly rounded quotient is monotonic in the numerator
      for_each(lr, [&](int, float x) { mx = fmaxf(mx, x); });
      mx = __fdiv_rn(block_max(mx, red), t);
    } else {
      for_each(lr, [&](int, float x) { mx = fmaxf(mx, __fdiv_rn(x, t)); });
      mx = block_max(mx, red);
    }
    const float inv_t = 1.f / t;
    const int64_t nbase = (int64_t)row * Vs;
    const uint32_t gbase = (uint32_t)c.rank * (uint32_t)Vs;
    float z = 0.f;
    float r0 = -INFINITY, r1 = -INFINITY, q0 = 1.f, q1 = 1.f;
    int i0 = 0x7fffffff, i1 = 0x7fffffff;
    for_each(lr, [&](int i, float x) {
      const float e = __expf(fmaf(x, inv_t, -mx));
      z += e;
      const float q = fmaxf(noise ? noise[nbase + i] : exp1_draw(seed, row0 + row, gbase + i), 1e-10f);
      const float r = __fdividef(e, q);
      if (r > r1) {
        if (r > r0) { r1 = r0; q1 = q0; i1 = i0; r0 = r; q0 = q; i0 = i; }
        else { r1 = r; q1 = q; i1 = i; }
      }
    });
    z = block_sum(z, red);
    cand[(slot * 2 + 0) * SAMPLE_THREADS + threadIdx.x] = make_int2(i0, __float_as_int(q0));
    cand[(slot * 2 + 1) * SAMPLE_THREADS + threadIdx.x] = make_int2(i1, __float_as_int(q1));
    if (threadIdx.x < WORLD)   // one flagged line per row and peer: {m, epoch, z, epoch}
      st16(ll_of(seg, c.area_bytes, c.ll_bytes, WORLD, threadIdx.x, parity, c.rank) + (size_t)row * 16,
           make_int4(__float_as_int(mx), (int)epoch, __float_as_int(z), (int)epoch));
    __syncthreads();
  }

  // ---- B: the candidates' exact values against the global maximum and sum ----
  slot = 0;
  for (int row = blk; row < rows; row += nblk, ++slot) {
    const T* lr = logits + (int64_t)row * Vs;
    const float t = temperatures[row];
    float ms[WORLD], zs[WORLD];
    float m = -INFINITY;
#pragma unroll
    for (int r = 0; r < WORLD; ++r) {   // every thread polls the same lines (broadcast loads)
      const uint2 st = ll_read_line(c, ll_of(seg, c.area_bytes, c.ll_bytes, WORLD, c.rank, parity, r) + (size_t)row * 16,
                                    epoch);
      ms[r] = __uint_as_float(st.x); zs[r] = __uint_as_float(st.y);
      m = fmaxf(m, ms[r]);
    }
    float zsum = 0.f;
#pragma unroll
    for (int r = 0; r < WORLD; ++r) zsum += zs[r] * expf(ms[r] - m);
    const uint32_t gbase = (uint32_t)c.rank * (uint32_t)Vs;
    auto exact = [&](int2 cd) -> float {   // the reference's value of a candidate
      if (cd.x == 0x7fffffff) return -INFINITY;
      const float e = expf(__fdiv_rn(Elem<T>::to_f32(lr[cd.x]), t) - m);
      return __fdiv_rn(__fdiv_rn(e, zsum), __int_as_float(cd.y));
    };
    const int2 c0 = cand[(slot * 2 + 0) * SAMPLE_THREADS + threadIdx.x];
    const int2 c1 = cand[(slot * 2 + 1) * SAMPLE_THREADS + threadIdx.x];
    const float v0 = exact(c0), v1 = exact(c1);
    float best = v0;
    int besti = c0.x;
    if (v1 > best || (v1 == best && c1.x < besti)) { best = v1; besti = c1.x; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
      if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
    }
    if (lane == 0) { bval[w] = best; bidx[w] = besti; }
    __syncthreads();
    if (w == 0) {
      best = bval[lane]; besti = bidx[lane];   // SAMPLE_THREADS / 32 == 32 warps
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
        if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
      }
      if (lane < WORLD) {
        const int gi = besti == 0x7fffffff ? 0x7fffffff : (int)gbase + besti;
        st16(ll_of(seg, c.area_bytes, c.ll_bytes, WORLD, lane, parity, c.rank) + ((size_t)rows + row) * 16,
             make_int4(__float_as_int(best), (int)epoch, gi, (int)epoch));
      }
    }
    __syncthreads();
  }

  // ---- C: the best of the shards' winners ----
  for (int row = blk; row < rows; row += nblk) {
    if (threadIdx.x == 0) {
      float best = -INFINITY;
      int besti = 0x7fffffff;
#pragma unroll
      for (int r = 0; r < WORLD; ++r) {
        const uint2 cnd = ll_read_line(c, ll_of(seg, c.area_bytes, c.ll_bytes, WORLD, c.rank, parity, r) +
                                              ((size_t)rows + row) * 16, epoch);
        const float cv = __uint_as_float(cnd.x);
        const int ci = (int)cnd.y;
        if (cv > best || (cv == best && ci < besti)) { best = cv; besti = ci; }
      }
      out[row] = besti;
    }
  }

  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(c.state + 1, 1u) == (uint32_t)nblk - 1) {
      c.state[1] = 0;
      c.state[0] = epoch;
      __threadfence();
    }
  }
}

template <typename T, int WORLD>
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_sharded_kernel(const Dev c, const T* __restrict__ logits, const float* __restrict__ temperatures,
                      const float* __restrict__ noise, int64_t* __restrict__ out, int rows, int Vs,
                      uint64_t seed, uint32_t row0) {
  sample_sharded_body<T, WORLD>(c, blockIdx.x, gridDim.x, logits, temperatures, noise, out, rows, Vs, seed, row0);
}

// Every rank as blocks of one cooperative launch on one GPU (test support, as above): rank r reads
// columns [r * Vs, (r + 1) * Vs) of the full [rows, WORLD * Vs] logits (row stride = full width is
// not supported by the body, so the shards are separate contiguous tensors).
template <typename T, int WORLD>
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_sharded_emulated_kernel(const EmulatedWorld w, const float* __restrict__ temperatures, int rows, int Vs,
                               uint64_t seed) {
  __shared__ Dev c;
  __shared__ const void* logits;
  __shared__ const void* noise;
  __shared__ void* out;
  if (threadIdx.x == 0) {
#pragma unroll
    for (int r = 0; r < WORLD; ++r)
      if (r == (int)blockIdx.y) { c = w.dev[r]; logits = w.in[r]; out = w.out[r]; noise = w.residual_out[r]; }
  }
  __syncthreads();
  sample_sharded_body<T, WORLD>(c, blockIdx.x, gridDim.x, (const T*)logits, temperatures, (const float*)noise,
                                (int64_t*)out, rows, Vs, seed, 0u);
}

}}  // namespace zp::coll

struct zp_comm {
  int rank = 0, world = 0, device = 0, sms = 0;
  size_t area_bytes = 0;
  size_t ll_bytes = 0;
  char* seg[zp::coll::MAX_WORLD] = {};
  bool ipc_opened[zp::coll::MAX_WORLD] = {};
  uint32_t* state = nullptr;
  long long timeout_ns = 0;
};

namespace {

constexpr size_t LL_MAX_BYTES = 2u << 20;   // largest message sent as flagged lines
// ... and the largest for which they are the default: measured on 2 GPUs, 64 KiB 7 us against
// 10.4 us for the one-shot form with a meeting, 2 MiB 17.5 us against 15.7 us
constexpr size_t LL_AUTO_BYTES = 512u << 10;

size_t ll_bytes_for(size_t area_bytes) { return std::min(area_bytes, LL_MAX_BYTES); }
size_t segment_bytes(size_t area_bytes, int world) {
  return zp::coll::FLAG_BYTES + 2 * (size_t)(world + 1) * area_bytes +
         2 * (size_t)world * 2 * ll_bytes_for(area_bytes);
}

template <typename T, int WORLD>
void launch(const zp_comm* c, int mode, bool fused, const void* in, void* out, int64_t nvec,
            int row_vecs, int64_t nrows, const void* residual, const void* weight, void* residual_out,
            float eps, cudaStream_t st) {
  using namespace zp::coll;
  Dev d;
  for (int r = 0; r < MAX_WORLD; ++r) d.seg[r] = c->seg[r];
  d.state = c->state; d.area_bytes = c->area_bytes; d.ll_bytes = c->ll_bytes; d.timeout_ns = c->timeout_ns;
  d.rank = c->rank; d.world = c->world;
  auto go = [&](auto kernel) {
    // one block per SM: every block of the launch is resident at once (blocks wait for their
    // peers' blocks), and more blocks only add flags to exchange (256 blocks measured slower)
    const int grid = (int)std::min<int64_t>(nrows, std::min(c->sms, MAX_BLOCKS));
    kernel<<<grid, THREADS, 0, st>>>(d, (const T*)in, (T*)out, nvec, row_vecs, nrows, (const T*)residual,
                                     (const T*)weight, (T*)residual_out, eps);
  };
  if (mode == 2)      { if (fused) go(all_reduce_kernel<T, WORLD, 2, true>); else go(all_reduce_kernel<T, WORLD, 2, false>); }
  else if (mode == 1) { if (fused) go(all_reduce_kernel<T, WORLD, 1, true>); else go(all_reduce_kernel<T, WORLD, 1, false>); }
  else                { if (fused) go(all_reduce_kernel<T, WORLD, 0, true>); else go(all_reduce_kernel<T, WORLD, 0, false>); }
}

int run(zp_comm* c, int algo, bool fused, const void* in, void* out, int64_t nvec, int row_vecs,
        int64_t nrows, const void* residual, const void* weight, void* residual_out, float eps, int dtype,
        void* stream, const char* what) {
  using namespace zp::coll;
  ZP_REQUIRE(c && c->state, "%s: null communicator", what);
  for (int r = 0; r < c->world; ++r) ZP_REQUIRE(c->seg[r], "%s: the segment of rank %d is not attached", what, r);
  ZP_REQUIRE(algo >= 0 && algo <= 3, "%s: algorithm %d (0 auto, 1 one-shot, 2 two-shot, 3 flagged lines)", what, algo);
  ZP_REQUIRE(algo != 3 || (size_t)nvec * 16 <= c->ll_bytes, "%s: flagged lines carry at most %zu bytes", what, c->ll_bytes);
  ZP_REQUIRE((size_t)nvec * 16 <= c->area_bytes, "%s: %lld bytes exceed the communicator's %zu", what,
             (long long)nvec * 16, c->area_bytes);
  ZP_REQUIRE(((uintptr_t)in | (uintptr_t)out | (uintptr_t)residual | (uintptr_t)weight | (uintptr_t)residual_out) % 16 == 0,
             "%s: pointers must be 16-byte aligned", what);
  if (nvec == 0) return ZP_OK;
  // one-shot moves (world-1) x the message into every GPU, two-shot 2 x (world-1)/world of it
  // small messages go as flagged lines (twice the bytes on the link, but no fence and no
  // meeting: a decode step's messages are latency-bound); above that one-shot moves (world-1) x
  // the message into every GPU, two-shot 2 x (world-1)/world of it
  int mode;
  if (algo == 0) {
    // flagged lines by default only up to 4 ranks: with 8, the 64 KiB message measured 23 us
    // against 16 us for the one-shot form (seven peers' worth of doubled stores and polls)
    const bool lines = c->world <= 4 && (size_t)nvec * 16 <= std::min(c->ll_bytes, LL_AUTO_BYTES);
    mode = lines ? 2 : (c->world > 2 && (size_t)nvec * 16 >= (512u << 10) ? 1 : 0);
  }
  else mode = algo - 1;
  cudaStream_t st = (cudaStream_t)stream;
#define ZP_COLL_WORLD(W) \
  ZP_DISPATCH_DTYPE(dtype, T, (launch<T, W>(c, mode, fused, in, out, nvec, row_vecs, nrows, residual, weight, residual_out, eps, st)))
  switch (c->world) {
    case 2: ZP_COLL_WORLD(2); break;
    case 4: ZP_COLL_WORLD(4); break;
    case 8: ZP_COLL_WORLD(8); break;
    default: zp::set_error("%s: world size %d (2, 4 or 8)", what, c->world); return ZP_ERR_INVALID_ARGUMENT;
  }
#undef ZP_COLL_WORLD
  return zp::check_launch(what);
}

}  // namespace

extern "C" int zp_comm_create(int rank, int world, size_t max_bytes, int timeout_ms, zp_comm** out) {
  using namespace zp::coll;
  ZP_REQUIRE(out, "zp_comm_create: null output");
  ZP_REQUIRE(world == 2 || world == 4 || world == 8, "zp_comm_create: world size %d (2, 4 or 8)", world);
  ZP_REQUIRE(rank >= 0 && rank < world, "zp_comm_create: rank %d of %d", rank, world);
  ZP_REQUIRE(max_bytes > 0 && timeout_ms > 0, "zp_comm_create: max_bytes and timeout_ms must be positive");
  zp_comm* c = new (std::nothrow) zp_comm();
  ZP_REQUIRE(c, "zp_comm_create: out of host memory");
  c->rank = rank; c->world = world;
  c->area_bytes = (max_bytes + 255) / 256 * 256;
  c->ll_bytes = ll_bytes_for(c->area_bytes);
  c->timeout_ns = (long long)timeout_ms * 1000000ll;
  cudaError_t e = cudaGetDevice(&c->device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&c->sms, cudaDevAttrMultiProcessorCount, c->device);
  void* seg = nullptr; void* state = nullptr;
  if (e == cudaSuccess) e = cudaMalloc(&seg, segment_bytes(c->area_bytes, world));
  if (e == cudaSuccess) e = cudaMemset(seg, 0, FLAG_BYTES);
  if (e == cudaSuccess)   // no line of the flagged-line slots may carry a future epoch
    e = cudaMemset((char*)seg + FLAG_BYTES + 2 * (size_t)(world + 1) * c->area_bytes, 0,
                   2 * (size_t)world * 2 * c->ll_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&state, 256);
  if (e == cudaSuccess) e = cudaMemset(state, 0, 256);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    zp::set_error("zp_comm_create: %s", cudaGetErrorString(e));
    if (seg) cudaFree(seg);
    if (state) cudaFree(state);
    delete c;
    return ZP_ERR_CUDA;
  }
  c->seg[rank] = (char*)seg;
  c->state = (uint32_t*)state;
  *out = c;
  return ZP_OK;
}

extern "C" int zp_comm_segment(zp_comm* c, void** ptr_out, size_t* bytes_out) {
  ZP_REQUIRE(c && ptr_out && bytes_out, "zp_comm_segment: null pointer");
  *ptr_out = c->seg[c->rank];
  *bytes_out = segment_bytes(c->area_bytes, c->world);
  return ZP_OK;
}

extern "C" int zp_comm_ipc_handle(zp_comm* c, void* handle64) {
  ZP_REQUIRE(c && handle64, "zp_comm_ipc_handle: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, c->seg[c->rank]);
  if (e != cudaSuccess) { zp::set_error("zp_comm_ipc_handle: %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  memcpy(handle64, &h, 64);
  return ZP_OK;
}

extern "C" int zp_comm_open_peer(zp_comm* c, int peer, const void* handle64) {
  ZP_REQUIRE(c && handle64, "zp_comm_open_peer: null pointer");
  ZP_REQUIRE(peer >= 0 && peer < c->world && peer != c->rank, "zp_comm_open_peer: peer %d", peer);
  ZP_REQUIRE(!c->seg[peer], "zp_comm_open_peer: peer %d is attached already", peer);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) { zp::set_error("zp_comm_open_peer: %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  c->seg[peer] = (char*)p;
  c->ipc_opened[peer] = true;
  return ZP_OK;
}

extern "C" int zp_comm_attach_peer(zp_comm* c, int peer, void* segment) {
  ZP_REQUIRE(c && segment, "zp_comm_attach_peer: null pointer");
  ZP_REQUIRE(peer >= 0 && peer < c->world && peer != c->rank, "zp_comm_attach_peer: peer %d", peer);
  ZP_REQUIRE(!c->seg[peer], "zp_comm_attach_peer: peer %d is attached already", peer);
  c->seg[peer] = (char*)segment;
  return ZP_OK;
}

extern "C" int zp_comm_status(zp_comm* c, int* status_out) {
  ZP_REQUIRE(c && status_out, "zp_comm_status: null pointer");
  uint32_t v = 0;
  cudaError_t e = cudaMemcpy(&v, c->state + 2, sizeof(v), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) { zp::set_error("zp_comm_status: %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  *status_out = (int)v;
  return ZP_OK;
}

extern "C" int zp_comm_destroy(zp_comm* c) {
  if (!c) return ZP_OK;
  cudaDeviceSynchronize();
  for (int r = 0; r < c->world; ++r)
    if (c->ipc_opened[r]) cudaIpcCloseMemHandle(c->seg[r]);
  if (c->seg[c->rank]) cudaFree(c->seg[c->rank]);
  if (c->state) cudaFree(c->state);
  delete c;
  return ZP_OK;
}

extern "C" int zp_all_reduce(zp_comm* c, const void* in, void* out, int64_t count, int dtype, int algo,
                             void* stream) {
  ZP_REQUIRE(in && out, "zp_all_reduce: null pointer");
  ZP_REQUIRE(count >= 0 && (count * (int64_t)zp::dtype_size(dtype)) % 16 == 0,
             "zp_all_reduce: the message must be a multiple of 16 bytes");
  const int64_t nvec = count * (int64_t)zp::dtype_size(dtype) / 16;
  const int row_vecs = zp::coll::THREADS * zp::coll::VPT;
  return run(c, algo, false, in, out, nvec, row_vecs, (nvec + row_vecs - 1) / row_vecs, nullptr, nullptr,
             nullptr, 0.f, dtype, stream, "zp_all_reduce");
}

extern "C" int zp_all_reduce_add_rms_norm(zp_comm* c, const void* in, const void* residual, const void* weight,
                                          void* out, void* residual_out, int64_t rows, int hidden, float eps,
                                          int dtype, int algo, void* stream) {
  ZP_REQUIRE(in && residual && weight && out && residual_out, "zp_all_reduce_add_rms_norm: null pointer");
  const int64_t row_bytes = (int64_t)hidden * (int64_t)zp::dtype_size(dtype);
  ZP_REQUIRE(rows >= 0 && hidden > 0 && row_bytes % 16 == 0 &&
                 row_bytes / 16 <= zp::coll::THREADS * zp::coll::VPT,
             "zp_all_reduce_add_rms_norm: a row must be a multiple of 16 bytes and at most %d bytes",
             zp::coll::THREADS * zp::coll::VPT * 16);
  return run(c, algo, true, in, out, rows * (row_bytes / 16), (int)(row_bytes / 16), rows, residual, weight,
             residual_out, eps, dtype, stream, "zp_all_reduce_add_rms_norm");
}

extern "C" int zp_sample_sharded(zp_comm* c, const void* logits, const float* temperatures, const float* noise,
                                 int64_t* tokens_out, int n_rows, int vocab_shard, uint64_t seed, int dtype,
                                 void* stream) {
  using namespace zp::coll;
  ZP_REQUIRE(c && c->state, "zp_sample_sharded: null communicator");
  for (int r = 0; r < c->world; ++r) ZP_REQUIRE(c->seg[r], "zp_sample_sharded: the segment of rank %d is not attached", r);
  if (n_rows == 0) return ZP_OK;
  ZP_REQUIRE(logits && temperatures && tokens_out, "zp_sample_sharded: null pointer");
  ZP_REQUIRE(n_rows > 0 && vocab_shard > 0 && (int64_t)vocab_shard * c->world < 0x7fffffff,
             "zp_sample_sharded: bad sizes");
  ZP_REQUIRE((size_t)std::min(n_rows, SAMPLE_ROWS_PER_BLOCK * std::min(c->sms, MAX_BLOCKS)) * 16 <= c->ll_bytes,
             "zp_sample_sharded: the communicator's message area (%zu bytes) is too small for %d rows",
             c->area_bytes, n_rows);
  Dev d;
  for (int r = 0; r < MAX_WORLD; ++r) d.seg[r] = c->seg[r];
  d.state = c->state; d.area_bytes = c->area_bytes; d.ll_bytes = c->ll_bytes; d.timeout_ns = c->timeout_ns;
  d.rank = c->rank; d.world = c->world;
  cudaStream_t st = (cudaStream_t)stream;
  const int es = (int)zp::dtype_size(dtype);
  const int max_grid = std::min(c->sms, MAX_BLOCKS);
  // a block keeps the candidates of at most SAMPLE_ROWS_PER_BLOCK rows: larger batches take
  // several launches (each a complete exchange)
  for (int row0 = 0; row0 < n_rows; row0 += SAMPLE_ROWS_PER_BLOCK * max_grid) {
    const int rows = std::min(n_rows - row0, SAMPLE_ROWS_PER_BLOCK * max_grid);
    const int grid = std::min(rows, max_grid);
    const char* lg = (const char*)logits + (size_t)row0 * vocab_shard * es;
    const float* nz = noise ? noise + (size_t)row0 * vocab_shard : nullptr;
#define ZP_SAMPLE_WORLD(W)                                                                               \
  ZP_DISPATCH_DTYPE(dtype, T, {                                                                          \
    cudaFuncSetAttribute(sample_sharded_kernel<T, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, SAMPLE_SMEM); \
    sample_sharded_kernel<T, W><<<grid, SAMPLE_THREADS, SAMPLE_SMEM, st>>>(                              \
        d, (const T*)lg, temperatures + row0, nz, tokens_out + row0, rows, vocab_shard, seed, (uint32_t)row0); \
  })
    switch (c->world) {
      case 2: ZP_SAMPLE_WORLD(2); break;
      case 4: ZP_SAMPLE_WORLD(4); break;
      case 8: ZP_SAMPLE_WORLD(8); break;
      default: zp::set_error("zp_sample_sharded: world size %d", c->world); return ZP_ERR_INVALID_ARGUMENT;
    }
#undef ZP_SAMPLE_WORLD
  }
  return zp::check_launch("zp_sample_sharded");
}

// Test support (see all_reduce_emulated_kernel): `comms[r]` is rank r's communicator, all created
// in this process on the current device with each other's segments attached by pointer.
extern "C" int zp_all_reduce_emulated(zp_comm* const* comms, int world, const void* const* ins, void* const* outs,
                                      const void* residual, const void* weight, void* const* residual_outs,
                                      int64_t rows, int row_elems, float eps, int dtype, int algo, int fused,
                                      void* stream) {
  using namespace zp::coll;
  ZP_REQUIRE(comms && ins && outs, "zp_all_reduce_emulated: null pointer");
  ZP_REQUIRE(world == 2 || world == 4 || world == 8, "zp_all_reduce_emulated: world size %d", world);
  ZP_REQUIRE(algo >= 1 && algo <= 3, "zp_all_reduce_emulated: algorithm %d (1 one-shot, 2 two-shot, 3 flagged lines)", algo);
  const int64_t row_bytes = (int64_t)row_elems * (int64_t)zp::dtype_size(dtype);
  ZP_REQUIRE(rows > 0 && row_elems > 0 && row_bytes % 16 == 0 && row_bytes / 16 <= THREADS * VPT,
             "zp_all_reduce_emulated: bad row size");
  ZP_REQUIRE(!fused || (residual && weight && residual_outs), "zp_all_reduce_emulated: fused form needs residual and weight");
  EmulatedWorld w{};
  for (int r = 0; r < world; ++r) {
    const zp_comm* c = comms[r];
    ZP_REQUIRE(c && c->world == world && c->rank == r, "zp_all_reduce_emulated: communicator %d", r);
    ZP_REQUIRE((size_t)(rows * row_bytes) <= (algo == 3 ? c->ll_bytes : c->area_bytes),
               "zp_all_reduce_emulated: message exceeds the areas");
    for (int q = 0; q < world; ++q) ZP_REQUIRE(c->seg[q], "zp_all_reduce_emulated: rank %d lacks segment %d", r, q);
    for (int q = 0; q < MAX_WORLD; ++q) w.dev[r].seg[q] = c->seg[q];
    w.dev[r].state = c->state; w.dev[r].area_bytes = c->area_bytes; w.dev[r].ll_bytes = c->ll_bytes;
    w.dev[r].timeout_ns = c->timeout_ns;
    w.dev[r].rank = r; w.dev[r].world = world;
    w.in[r] = ins[r]; w.out[r] = outs[r]; w.residual_out[r] = fused ? residual_outs[r] : nullptr;
  }
  int64_t nvec = rows * (row_bytes / 16);
  int row_vecs = (int)(row_bytes / 16);
  int64_t nrows = rows;
  const int nblk = (int)std::min<int64_t>(nrows, std::max(1, comms[0]->sms / world));
  void* args[] = {&w, &nvec, &row_vecs, &nrows, (void*)&residual, (void*)&weight, &eps};
  const dim3 grid(nblk, world);
  cudaError_t e = cudaSuccess;
  auto go = [&](auto kernel) {
    e = cudaLaunchCooperativeKernel((const void*)kernel, grid, dim3(THREADS), args, 0, (cudaStream_t)stream);
  };
#define ZP_EMU(W)                                                                                     \
  ZP_DISPATCH_DTYPE(dtype, T, {                                                                       \
    if (algo == 3)      { if (fused) go(all_reduce_emulated_kernel<T, W, 2, true>); else go(all_reduce_emulated_kernel<T, W, 2, false>); } \
    else if (algo == 2) { if (fused) go(all_reduce_emulated_kernel<T, W, 1, true>); else go(all_reduce_emulated_kernel<T, W, 1, false>); } \
    else                { if (fused) go(all_reduce_emulated_kernel<T, W, 0, true>); else go(all_reduce_emulated_kernel<T, W, 0, false>); } \
  })
  switch (world) {
    case 2: ZP_EMU(2); break;
    case 4: ZP_EMU(4); break;
    default: ZP_EMU(8); break;
  }
#undef ZP_EMU
  if (e != cudaSuccess) { zp::set_error("zp_all_reduce_emulated: %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  return zp::check_launch("zp_all_reduce_emulated");
}

// Test support: zp_sample_sharded for every rank of a world as one cooperative launch on one GPU.
// logits_shards / noise_shards (or NULL) / tokens_outs: one pointer per rank.
extern "C" int zp_sample_sharded_emulated(zp_comm* const* comms, int world, const void* const* logits_shards,
                                          const float* temperatures, const float* const* noise_shards,
                                          int64_t* const* tokens_outs, int n_rows, int vocab_shard, uint64_t seed,
                                          int dtype, void* stream) {
  using namespace zp::coll;
  ZP_REQUIRE(comms && logits_shards && temperatures && tokens_outs, "zp_sample_sharded_emulated: null pointer");
  ZP_REQUIRE(world == 2 || world == 4 || world == 8, "zp_sample_sharded_emulated: world size %d", world);
  ZP_REQUIRE(n_rows > 0 && vocab_shard > 0, "zp_sample_sharded_emulated: bad sizes");
  EmulatedWorld w{};
  for (int r = 0; r < world; ++r) {
    const zp_comm* c = comms[r];
    ZP_REQUIRE(c && c->world == world && c->rank == r, "zp_sample_sharded_emulated: communicator %d", r);
    ZP_REQUIRE((size_t)n_rows * 16 <= c->ll_bytes, "zp_sample_sharded_emulated: too many rows for the areas");
    for (int q = 0; q < world; ++q) ZP_REQUIRE(c->seg[q], "zp_sample_sharded_emulated: rank %d lacks segment %d", r, q);
    for (int q = 0; q < MAX_WORLD; ++q) w.dev[r].seg[q] = c->seg[q];
    w.dev[r].state = c->state; w.dev[r].area_bytes = c->area_bytes; w.dev[r].ll_bytes = c->ll_bytes;
    w.dev[r].timeout_ns = c->timeout_ns;
    w.dev[r].rank = r; w.dev[r].world = world;
    w.in[r] = logits_shards[r]; w.out[r] = tokens_outs[r];
    w.residual_out[r] = noise_shards ? (void*)noise_shards[r] : nullptr;
  }
  // 1024-thread blocks: one per SM; the ranks share the SMs
  const int nblk = std::min(n_rows, std::max(1, comms[0]->sms / world));
  ZP_REQUIRE(n_rows <= SAMPLE_ROWS_PER_BLOCK * nblk, "zp_sample_sharded_emulated: at most %d rows at this world size",
             SAMPLE_ROWS_PER_BLOCK * nblk);
  void* args[] = {&w, (void*)&temperatures, &n_rows, &vocab_shard, &seed};
  const dim3 grid(nblk, world);
  cudaError_t e = cudaSuccess;
  auto go = [&](auto kernel) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SAMPLE_SMEM);
    e = cudaLaunchCooperativeKernel((const void*)kernel, grid, dim3(SAMPLE_THREADS), args, SAMPLE_SMEM,
                                    (cudaStream_t)stream);
  };
  switch (world) {
    case 2: ZP_DISPATCH_DTYPE(dtype, T, go(sample_sharded_emulated_kernel<T, 2>)); break;
    case 4: ZP_DISPATCH_DTYPE(dtype, T, go(sample_sharded_emulated_kernel<T, 4>)); break;
    default: ZP_DISPATCH_DTYPE(dtype, T, go(sample_sharded_emulated_kernel<T, 8>)); break;
  }
  if (e != cudaSuccess) { zp::set_error("zp_sample_sharded_emulated: %s", cudaGetErrorString(e)); return ZP_ERR_CUDA; }
  return zp::check_launch("zp_sample_sharded_emulated");
}
