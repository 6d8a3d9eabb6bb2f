// PTX building blocks shared by the tcgen05 GEMM kernels: mbarriers with bounded waits, TMA loads and stores,
// UMMA descriptors, TMEM loads.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace molt {

constexpr int kStatusTimeout = MOLT_E_TIMEOUT;   // code in the top byte of the device status word

// ---- PTX wrappers ------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// try_wait that lets the hardware park the thread for up to hint_ns before it answers
__device__ __forceinline__ bool mbar_try_parked(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return done != 0;
}

// Bounded wait: gives up after limit_cycles SM clock cycles.  Returns false when the wait expired or another role
// of the CTA already gave up; the first to give up records (code, where, block) in the device status word.
// Waiting warps share issue slots with the working ones, so the loop is kept short: the thread is parked inside
// try_wait, and the abort flag and the clock are looked at once in sixteen rounds.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status,
                                          int where, long long limit_cycles) {
  if (mbar_try(bar, parity)) return true;
  const long long start = clock64();
#ifdef MOLT_SPIN_OLD
  for (uint32_t spin = 0;; ++spin) {
    if (mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if ((spin & 63u) == 63u && clock64() - start > limit_cycles) {
      *abort_flag = 1;
      atomicCAS(status, 0, (kStatusTimeout << 24) | (where << 16) | (int)(blockIdx.x & 0xffff));
      return false;
    }
  }
#else
  for (;;) {
#pragma unroll 1
    for (int spin = 0; spin < 16; ++spin)
      if (mbar_try_parked(bar, parity, 4000u)) return true;
    if (*abort_flag) return false;
    if (clock64() - start > limit_cycles) {
      *abort_flag = 1;
      atomicCAS(status, 0, (kStatusTimeout << 24) | (where << 16) | (int)(blockIdx.x & 0xffff));
      return false;
    }
  }
#endif
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(src),
               "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1 (Blackwell).
//   K-major  (forward operands, activations): 8-row groups 1024 bytes apart  -> SBO = 1024, LBO unused (1)
//   MN-major (backward weight operand): 64-column atoms 8192 bytes apart     -> LBO = 8192; 8 contraction rows
//                                        are 1024 bytes apart                -> SBO = 1024
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= (uint64_t)1 << 46;   // version
  d |= (uint64_t)2 << 61;   // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16: bf16 x bf16 -> fp32, A K-major, B K-major or MN-major.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ uint64_t desc64(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// ---- NF4 decode in registers ---------------------------------------------------------------------------------
// The sixteen bf16 values of one segment, split into byte planes: lo[i] / hi[i] hold the low / high bytes of entries
// 4 i .. 4 i + 3.
struct SegmentTable {
  uint32_t lo[4], hi[4];
};
__device__ __forceinline__ SegmentTable make_segment_table(const float (&codebook)[16], float absmax) {
  uint32_t pairs[8];   // (entry 2 i, entry 2 i + 1) as bf16x2; one fp32 multiply and one rounding per entry
#pragma unroll
  for (int i = 0; i < 8; ++i)
    pairs[i] = pack_bf16x2(__fmul_rn(codebook[2 * i], absmax), __fmul_rn(codebook[2 * i + 1], absmax));
  SegmentTable t;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    t.lo[i] = __byte_perm(pairs[2 * i], pairs[2 * i + 1], 0x6420u);
    t.hi[i] = __byte_perm(pairs[2 * i], pairs[2 * i + 1], 0x7531u);
  }
  return t;
}
// Eight codes (one 32-bit word, code i in bits 4 i .. 4 i + 3) -> eight bf16 values.  A byte permute indexes eight
// bytes with the low three bits of a selector nibble (bit 3 would ask for sign replication, so it is masked off);
// the code's top bit chooses between the two halves of the table through a byte mask.  pick01 / pick23 order the
// result for the weight's nibble order.
__device__ __forceinline__ void decode_word(uint32_t w, const SegmentTable& t, uint32_t pick01, uint32_t pick23,
                                            uint32_t (&out)[4]) {
  const uint32_t low3 = w & 0x77777777u;
  const uint32_t top = (w >> 3) & 0x11111111u;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const uint32_t sel = c == 0 ? low3 : (low3 >> 16);   // prmt reads the low 16 bits of its selector
    const uint32_t upper = __byte_perm(0x0000ff00u, 0u, c == 0 ? top : (top >> 16));   // 0xff where the code is >= 8
    const uint32_t lo = (__byte_perm(t.lo[0], t.lo[1], sel) & ~upper) | (__byte_perm(t.lo[2], t.lo[3], sel) & upper);
    const uint32_t hi = (__byte_perm(t.hi[0], t.hi[1], sel) & ~upper) | (__byte_perm(t.hi[2], t.hi[3], sel) & upper);
    out[2 * c] = __byte_perm(lo, hi, pick01);
    out[2 * c + 1] = __byte_perm(lo, hi, pick23);
  }
}


// Tiled tensor map (2-D) through the driver entry point; defined next to the CTA-pair GEMM.
int make_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, const void* ptr, uint64_t inner, uint64_t outer,
                    uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle,
                    const char* what);

}  // namespace molt
