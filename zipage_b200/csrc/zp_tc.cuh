// Blackwell (sm_100a) building blocks used by the tensor-core kernels: mbarriers with bounded
// waits, TMA tiled loads through tensor maps, tcgen05 MMA / commit / TMEM load, UMMA descriptors.
//
// Conventions used by every kernel built on this header
//   * operands are K-major bf16/fp16 tiles of [rows][64 elements] (128-byte rows) written by TMA
//     with the 128-byte swizzle, 8-row groups 1024 bytes apart, every tile 1024-byte aligned;
//   * accumulators are fp32 in TMEM, one row per lane (M = 128), read back with 32x32b loads;
//   * no thread-block clusters and no multicast anywhere;
//   * every wait is bounded: after WAIT_LIMIT unsuccessful polls a role raises the block's abort
//     flag and the device error word, and every role leaves its loop; TMEM is freed at the end.
#pragma once
#include <cuda.h>

#include "zp_common.cuh"

namespace zp {
namespace tc {

constexpr uint32_t WAIT_LIMIT = 1u << 22;  // polls (each poll may itself block for a short while)

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ---------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the block is aborting (this wait ran out, or another role's did).
// SLEEP_NS > 0: sleep that long between polls, so that a waiting warp leaves the issue slots of
// its scheduler to the warps that have work (a poll is several instructions).  `true` = 64 ns.
template <int SLEEP_NS = 0>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* error_word, int where) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (SLEEP_NS > 0) __nanosleep(SLEEP_NS == 1 ? 64 : SLEEP_NS);
  }
  *abort_flag = 1;
  atomicCAS(error_word, 0, where);
  return false;
}

// ---- TMA ----------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_5d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0,
                                            int c1, int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1),
      "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}

// Hint: bring a tile into L2 ahead of the load that will ask for it (no shared memory, no barrier).
__device__ __forceinline__ void tma_prefetch_l2_5d(const CUtensorMap* m, int c0, int c1, int c2, int c3, int c4) {
  asm volatile("cp.async.bulk.prefetch.tensor.5d.L2.global.tile [%0, {%1, %2, %3, %4, %5}];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
               : "memory");
}

// ---- tcgen05 ------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, one thread issues
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// mbarrier arrives once all tcgen05 operations issued so far by this thread have completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// Split form for software pipelining: issue the load of the next chunk, then wait.  The wait names
// the destination registers as read-write operands so that no use of them can be scheduled
// before it.  (tcgen05.wait::ld waits for every load the thread has issued so far.)
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32_wait(uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
        "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
        "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
        "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
      :
      : "memory");
}

// 32 consecutive fp32 columns of this thread's TMEM lane (load and wait)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  tmem_ld32_issue(taddr, r);
  tmem_ld32_wait(r);
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// ---- packed fp32 pairs and 3-input max (sm_100) ----
__device__ __forceinline__ void ffma2(float2& d, float2 a, float2 b) {  // d += a * b, both lanes
  asm("{\n\t.reg .b64 ra, rb, rc;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mov.b64 rc, {%0, %1};\n\tfma.rn.f32x2 rc, ra, rb, rc;\n\tmov.b64 {%0, %1}, rc;\n\t}"
      : "+f"(d.x), "+f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {  // a * b, both lanes
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 rc, ra, rb;\n\tmov.b64 {%0, %1}, rc;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// ---- packed 16-bit pairs (two values per 32-bit register, element 0 in the low half) ----
template <typename T> struct Pair;
template <> struct Pair<__nv_bfloat16> {
  using V = __nv_bfloat162;
  static __device__ __forceinline__ V pack(float lo, float hi) { return __floats2bfloat162_rn(lo, hi); }
  static __device__ __forceinline__ float2 unpack(V v) { return __bfloat1622float2(v); }
};
template <> struct Pair<__half> {
  using V = __half2;
  static __device__ __forceinline__ V pack(float lo, float hi) { return __floats2half2_rn(lo, hi); }
  static __device__ __forceinline__ float2 unpack(V v) { return __half22float2(v); }
};

// ---- descriptors ----------------------------------------------------------------------------------
// K-major operand tile in shared memory, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024
// bytes apart (stride byte offset 1024), leading byte offset unused (1), descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | (1u << 16);
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}
// Instruction descriptor: fp32 accumulate, A and B both K-major, both of `fmt` (0 = f16, 1 = bf16).
__host__ __device__ constexpr uint32_t idesc_f16(int fmt, int M, int N) {
  return (1u << 4) | (static_cast<uint32_t>(fmt) << 7) | (static_cast<uint32_t>(fmt) << 10) |
         (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}
template <typename T> struct UmmaFmt;
template <> struct UmmaFmt<__nv_bfloat16> { static constexpr int fmt = 1; static constexpr CUtensorMapDataType tm = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; };
template <> struct UmmaFmt<__half> { static constexpr int fmt = 0; static constexpr CUtensorMapDataType tm = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; };

// One [rows x 128] bf16/fp16 operand = two 64-column blocks of rows*128 bytes each.
// Issues the 8 k-steps (K = 16 each) of D[128 x N] (+)= A[128 x 128] * B[N x 128]^T.
__device__ __forceinline__ void umma_k128(uint32_t d_tmem, uint32_t a_addr, uint32_t a_block_bytes,
                                          uint32_t b_addr, uint32_t b_block_bytes, uint32_t idesc) {
#pragma unroll
  for (int kb = 0; kb < 2; ++kb) {
    const uint64_t ad = smem_desc_sw128(a_addr + kb * a_block_bytes);
    const uint64_t bd = smem_desc_sw128(b_addr + kb * b_block_bytes);
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)  // 32 bytes (16 elements) further along K: +2 in the address field
      umma_f16(d_tmem, ad + 2u * ks, bd + 2u * ks, idesc, (kb | ks) ? 1u : 0u);
  }
}

// ---- host: tensor maps ------------------------------------------------------------------------------
// 5-D tiled map over a cache laid out [.., .., .., .., inner] with the given element strides of
// dims 1..4; box = {64, b1, b2, 1, 1}, 128-byte swizzle.  Returns 0 on success.
int make_tensor_map_5d(CUtensorMap* out, CUtensorMapDataType dt, const void* base, const uint64_t dims[5],
                       const uint64_t strides_elems[4], const uint32_t box[5], size_t elem_size);

// Device error word shared by the tensor-core kernels (0 = no error).
int* device_error_word();

}  // namespace tc
}  // namespace zp
