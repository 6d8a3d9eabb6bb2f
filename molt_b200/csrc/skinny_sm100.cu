// Few-token forward of the NF4-LoRA linear on the tensor cores with the operands swapped:
//
//   y[tok, row] = sum_k deq(W)[row, k] x[tok, k]  +  sum_j bf16(s B[row, j]) bf16(T[tok, j]),   T = x . A^T,   tok < m <= 128
//
// The weight rows fill the UMMA M dimension (128 decoded rows per tile), the tokens are the N dimension (16 .. 128), so
// no tensor work is spent on padding tokens up to a 256-row tile and every weight element is decoded exactly once.  The
// bound is the decode of the weight stream, so the work is cut to balance it: the contraction blocks (64 columns) of
// all row tiles, laid end to end, are dealt out in equal contiguous ranges to one CTA per SM.  A CTA therefore
// holds the tail of one row tile, whole tiles, and the head of another; every part leaves the kernel as an fp32
// accumulator [token][row] in a scratch slot, and a small second kernel adds the parts of each tile in CTA order
// (deterministic), adds the low-rank term and rounds once to bf16.  Nothing in the kernel waits for another CTA.
//
// Per CTA: a TMA ring of packed-code tiles (128 rows x 32 bytes), a TMA ring of token tiles (NT rows x 128 bytes, rows
// >= m zero-filled by the copy), and a ring of decoded weight tiles written by groups of four decode warps that take the
// blocks in turn (one thread = one 64-element segment).  Two decodes:
//   * table decode (default): one lookup per packed byte in a table of bf16 codebook pairs (replicated per lane, so the
//     lookups never conflict), times the segment's absmax as one bf16x2 multiply.  The weight value is then
//     bf16(bf16(code) * bf16(absmax)) instead of the dequantiser's bf16(code * absmax): a relative deviation of at most
//     2^-8 per element, far inside the 1e-2 gate on the output, for a third of the instructions;
//   * exact decode: the sixteen values bf16(codebook x absmax) are formed once per segment and selected with byte
//     permutes -- the bits of the standalone dequantiser.
// A nested (double-quantised) absmax is resolved by the decoder itself from the uint8 codes, so no resolved copy is
// written first.  Two threads (of two warps) issue the MMAs, taking the blocks of a part in turn, each into its own
// TMEM accumulator (the issue of one block's four tcgen05.mma is a dependent chain of several hundred cycles); four
// epilogue warps add the two accumulators of a finished part and store it while the next part accumulates in the other
// pair.  All waits are bounded (status word + clean exit).
#include <cuda.h>
#include <cudaTypedefs.h>
#ifdef MOLT_SKINNY_TRACE
#include <stdlib.h>
#endif

#include "internal.h"
#include "sm100_ptx.cuh"

namespace molt {
namespace skinny {

constexpr int BR = 128;   // weight rows per tile (UMMA M)
constexpr int BK = 64;    // contraction block
#ifndef MOLT_SKINNY_GROUPS
#define MOLT_SKINNY_GROUPS 3
#endif
constexpr int kGroups = MOLT_SKINNY_GROUPS;   // decode groups of four warps
constexpr int kBStages = 6;                   // decoded weight tiles, 16 KB each
constexpr int kCodeStages = 8;                // packed-code tiles, 4 KB each
constexpr int kXRingBytes = 32768;            // token tiles: as many stages as fit, at most eight
constexpr int kEpilogueWarps = 4;
// Warp roles.  An SM issues from four schedulers and warp w belongs to scheduler w % 4.  The single-thread loops that
// pace the pipeline (two MMA issuers, two TMA producers) are long dependent instruction chains, so they get
// scheduler 1 to themselves (next to one epilogue warp, which sleeps in its wait most of the time); the decode warps
// are the warps >= 4 on the other three schedulers, four consecutive ones forming a group.
constexpr int kMmaWarp = 5, kCodeWarp = 9, kXWarp = 13, kMmaWarp2 = 17;
#ifndef MOLT_SKINNY_MMA_WARPS
#define MOLT_SKINNY_MMA_WARPS 2
#endif
constexpr int kMmaWarps = MOLT_SKINNY_MMA_WARPS;   // 1 or 2 issuers
__host__ __device__ constexpr bool is_decode_warp(int warp) { return warp >= 4 && (warp & 3) != 1; }
__host__ __device__ constexpr int decode_warp_index(int warp) {
  return ((warp >> 2) - 1) * 3 + ((warp & 3) == 0 ? 0 : (warp & 3) - 1);
}
constexpr int count_warps(int groups) {
  int warp = 4, found = 0;
  while (found < 4 * groups) {
    if (is_decode_warp(warp)) ++found;
    ++warp;
  }
  return warp > kMmaWarp2 + 1 ? warp : kMmaWarp2 + 1;
}
constexpr int kWarps = count_warps(kGroups);
constexpr int kThreads = kWarps * 32;
constexpr uint32_t kTileBytes = BR * BK * 2;      // 16384
constexpr uint32_t kPackedBytes = BR * BK / 2;    // 4096
constexpr uint32_t kPairLutBytes = 256 * 32 * 4;  // table decode: [byte][lane] bf16x2
constexpr int kConsumedSlots = 16;
constexpr int kLowrankSlices = 8;                 // K slices of the low-rank input's first stage
constexpr int kLowrankThreads = 128;
// A decode group starts block g once block g - kBStages has been consumed; its parity wait on the code ring is only
// meaningful if the slot's previous use lies behind that front.
static_assert(kBStages <= kCodeStages && kCodeStages < kConsumedSlots, "ring depths");

constexpr int x_stages(int nt) { return kXRingBytes / (nt * 128) > 8 ? 8 : kXRingBytes / (nt * 128); }
constexpr uint32_t smem_bytes(int nt, bool table) {
  return kBStages * kTileBytes + x_stages(nt) * nt * 128 + kCodeStages * kPackedBytes + 1024 /*code2*/ +
         (table ? kPairLutBytes : 0) + 512 /*barriers*/ + 1024 /*alignment*/;
}

// The contiguous range of (tile, block) units of CTA c starts at floor(units * c / ctas), written with the quotient and
// remainder of units / ctas so that it needs no 64-bit division on the device (rem * c < ctas^2).
struct Ranges {
  int quot, rem, ctas;
};
__host__ __device__ __forceinline__ int range_begin(const Ranges& r, int cta) {
  return r.quot * cta + (int)((unsigned)(r.rem * cta) / (unsigned)r.ctas);
}

struct Params {
  const void* absmax;      // fp32 [n * k / 64], or uint8 codes of the nested form
  const float* absmax2;    // nested: second-level scales
  const float* code2;      // nested: 256-entry table
  float offset;
  int block2_shift;
  int32_t* status;
  long long n, k;
  int m;
  int num_kb;              // contraction blocks per row tile
  int tiles;               // row tiles of 128
  Ranges ranges;           // how the units are dealt out to the CTAs
  int max_parts;           // scratch slots per CTA
  float* partial;          // [ctas][max_parts][NT tokens][128 rows] fp32
  int nibble_high_first;
  long long wait_cycles;
  int withhold;            // failure injection (tests): the code producer issues this many blocks fewer than expected
#ifdef MOLT_SKINNY_TRACE
  unsigned long long* trace;   // optional [16 roles][128 events] cycle stamps of CTA 0
#endif
  float codebook[16];
};

#ifdef MOLT_SKINNY_TRACE
#define MOLT_CTRACE(role, index)                                                                   \
  do {                                                                                             \
    if (p.trace != nullptr && blockIdx.x == 0 && (index) < 128) p.trace[(role) * 128 + (index)] = (unsigned long long)clock64(); \
  } while (0)
#else
#define MOLT_CTRACE(role, index) do {} while (0)
#endif

// 88 registers per thread leave room on the SM for the blocks of the low-rank side kernel, which runs beside this one.
template <int NT, bool kNested, bool kTable>
__global__ void __maxnreg__(88)
nf4_skinny_sm100_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_packed,
                        const __grid_constant__ Params p) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag_s;
  constexpr int XS = x_stages(NT);
  constexpr uint32_t kXBytes = NT * 128;
  constexpr uint32_t kAccStride = NT < 32 ? 32 : NT;   // TMEM columns per accumulator (loads come 32 columns at a time)
  // two parts in flight x one accumulator per MMA issuer: 128 .. 512 columns, a power of two
  constexpr uint32_t kTmemCols = 2 * kMmaWarps * kAccStride < 64 ? 64 : 2 * kMmaWarps * kAccStride;
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t wtile0 = base;                                   // decoded weight tiles: the A operand
  const uint32_t x0 = wtile0 + kBStages * kTileBytes;             // token tiles: the B operand
  const uint32_t codes0 = x0 + XS * kXBytes;
  const uint32_t code2_0 = codes0 + kCodeStages * kPackedBytes;   // nested absmax: the 256-entry table
  const uint32_t lut0 = code2_0 + 1024u;                          // table decode: byte -> bf16 pair, per lane
  const uint32_t bar0 = lut0 + (kTable ? kPairLutBytes : 0u);
  auto bar_xfull = [&](int s) { return bar0 + 8u * s; };
  auto bar_pkfull = [&](int s) { return bar0 + 8u * (XS + s); };
  auto bar_consumed = [&](int g) { return bar0 + 8u * (XS + kCodeStages + (g & (kConsumedSlots - 1))); };
  auto consumed_parity = [&](int g) { return (uint32_t)((g / kConsumedSlots) & 1); };
  auto bar_bfull = [&](int s) { return bar0 + 8u * (XS + kCodeStages + kConsumedSlots + s); };
  auto bar_accfull = [&](int b) { return bar0 + 8u * (XS + kCodeStages + kConsumedSlots + kBStages + b); };
  auto bar_accempty = [&](int b) { return bar0 + 8u * (XS + kCodeStages + kConsumedSlots + kBStages + 2 + b); };
  static_assert(XS + kCodeStages + kConsumedSlots + kBStages + 4 <= 64, "barrier area");
  static_assert(XS >= 2, "token ring");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) MOLT_CTRACE(15, 0);
  volatile int* abort_flag = &abort_flag_s;
  auto wait_on = [&](uint32_t bar, uint32_t parity, int where) {
    return mbar_wait(bar, parity, abort_flag, p.status, where, p.wait_cycles);
  };

  if (threadIdx.x == 0) {
    abort_flag_s = 0;
    for (int s = 0; s < XS; ++s) mbar_init(bar_xfull(s), 1);
    for (int s = 0; s < kCodeStages; ++s) mbar_init(bar_pkfull(s), 1);
    for (int g = 0; g < kConsumedSlots; ++g) mbar_init(bar_consumed(g), 1);
    for (int s = 0; s < kBStages; ++s) mbar_init(bar_bfull(s), 4);   // the four warps of one decode group
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_accfull(b), kMmaWarps);                          // every issuer reports its last block of the part
      mbar_init(bar_accempty(b), kEpilogueWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // Launched as a programmatic dependent of the kernel before it in the stream: the set-up above touches no global
  // memory; nothing below runs before that kernel has completed and its writes are visible.  Then the kernel behind
  // (the low-rank side kernel, which needs nothing from this one) may start beside this grid.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (kNested) {
    float* table = reinterpret_cast<float*>(smem_dyn + (code2_0 - raw));
    for (int i = threadIdx.x; i < 256; i += blockDim.x) table[i] = __ldg(p.code2 + i);
  }
  if (kTable) {
    uint32_t* lut = reinterpret_cast<uint32_t*>(smem_dyn + (lut0 - raw));
    for (int i = threadIdx.x; i < 256 * 32; i += blockDim.x) {
      const int byte = i >> 5;   // the same for all lanes of a warp: the codebook reads below are broadcasts
      const int first = p.nibble_high_first ? byte >> 4 : byte & 15, second = p.nibble_high_first ? byte & 15 : byte >> 4;
      lut[i] = pack_bf16x2(p.codebook[first], p.codebook[second]);
    }
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  if (threadIdx.x == 0) MOLT_CTRACE(15, 1);

  const int nb = p.num_kb;
  const int u_begin = range_begin(p.ranges, (int)blockIdx.x);
  const int u_end = range_begin(p.ranges, (int)blockIdx.x + 1);
  const int first_tile = u_begin / nb;
  const int first_kb = u_begin - first_tile * nb;
  // Every role walks the same parts: (tile, kb0, kb1), u advancing by the part's length.
#define MOLT_SKINNY_PARTS(TILE, KB0, KB1)                                                          \
  for (int u_ = u_begin, TILE = first_tile, KB0 = first_kb,                                        \
           KB1 = (nb - KB0 < u_end - u_begin ? nb : KB0 + (u_end - u_begin));                      \
       u_ < u_end;                                                                                 \
       u_ += KB1 - KB0, ++TILE, KB0 = 0, KB1 = (nb < u_end - u_ ? nb : u_end - u_))

  if (warp == kCodeWarp || warp == kXWarp) {
    // ================= TMA producers: packed codes of the tile's rows, and the token tile of the same block =========
    const bool codes = warp == kCodeWarp;
    const int depth = codes ? kCodeStages : XS;
    if (lane == 0) {
      int total_blocks = u_end - u_begin;
      if (codes && p.withhold > 0) total_blocks -= p.withhold;
      int t = 0, stage = 0;
      bool ok = true;
      MOLT_SKINNY_PARTS(tile, kb0, kb1) {
        for (int kb = kb0; kb < kb1 && t < total_blocks; ++kb, ++t) {
          if (t >= depth) ok = wait_on(bar_consumed(t - depth), consumed_parity(t - depth), 1);
          if (!ok) break;
          if (codes) {
            MOLT_CTRACE(0, t);
            mbar_expect_tx(bar_pkfull(stage), kPackedBytes);
            tma_load_2d(codes0 + (uint32_t)stage * kPackedBytes, &map_packed, kb * (BK / 2), tile * BR, bar_pkfull(stage));
          } else {
            MOLT_CTRACE(1, t);
            mbar_expect_tx(bar_xfull(stage), kXBytes);
            tma_load_2d(x0 + (uint32_t)stage * kXBytes, &map_x, kb * BK, 0, bar_xfull(stage));
          }
          if (++stage == depth) stage = 0;
        }
        if (!ok || t >= total_blocks) break;
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp || (kMmaWarps == 2 && warp == kMmaWarp2)) {
    // ================= MMA issuers =================
    // Issuer i takes the blocks of a part whose position in the part is congruent to i, into accumulator
    // (part parity, i).  A commit covers the issuing thread's own MMAs, so every block is committed by its issuer.
    if (lane == 0) {
      const int me = kMmaWarps == 2 && warp == kMmaWarp2 ? 1 : 0;
      constexpr uint32_t idesc = make_idesc(BR, NT, 0);
      // K-major operands, 128-byte swizzle: 8-row groups 1024 bytes apart (SBO), LBO unused.  The start-address field
      // (bits 0..13, in 16-byte units) never carries into the next field: shared memory ends below 256 KB.
      constexpr uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
      const uint64_t a_desc0 = desc64(((wtile0 >> 4) & 0x3fffu) | (1u << 16), desc_hi);
      const uint64_t b_desc0 = desc64(((x0 >> 4) & 0x3fffu) | (1u << 16), desc_hi);
      int g_part = 0, parts_done = 0;
      uint32_t acc_phase[2] = {0u, 0u};   // flips every time an accumulator pair has been handed to the epilogue
      bool ok = true;
      MOLT_SKINNY_PARTS(tile, kb0, kb1) {
        const int acc = parts_done & 1;
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * kMmaWarps + me) * kAccStride;
        ok = wait_on(bar_accempty(acc), acc_phase[acc] ^ 1u, 2);   // the epilogue has drained this pair
        if (!ok) break;
        uint32_t accumulate = 0u;
        for (int kb = kb0 + me; kb < kb1; kb += kMmaWarps) {
          const int g = g_part + (kb - kb0);
          const uint32_t bstage = (uint32_t)g % kBStages, xstage = (uint32_t)g % XS;
          MOLT_CTRACE(2, g);
          ok = wait_on(bar_bfull(bstage), (uint32_t)((g / kBStages) & 1), 4);
          if (ok) ok = wait_on(bar_xfull(xstage), (uint32_t)((g / XS) & 1), 3);
          if (!ok) break;
          MOLT_CTRACE(3, g);
          tc_fence_after();
          const uint64_t a_desc = a_desc0 + (uint64_t)(bstage * (kTileBytes >> 4));
          const uint64_t b_desc = b_desc0 + (uint64_t)(xstage * (kXBytes >> 4));
          umma_bf16(d_tmem, a_desc, b_desc, idesc, accumulate);
#pragma unroll
          for (int ks = 1; ks < BK / 16; ++ks) umma_bf16(d_tmem, a_desc + 2u * ks, b_desc + 2u * ks, idesc, 1u);
          accumulate = 1u;
          MOLT_CTRACE(5, g);
          umma_commit(bar_consumed(g));   // releases the code stage, the token stage and the decoded tile of this block
        }
        if (!ok) break;
        // this issuer's share of the part is complete once its MMAs are; with no block of its own it just reports
        if (accumulate) umma_commit(bar_accfull(acc));
        else mbar_arrive(bar_accfull(acc));
        acc_phase[acc] ^= 1u;
        g_part += kb1 - kb0;
        ++parts_done;
      }
    }
    __syncwarp();
  } else if (is_decode_warp(warp) && decode_warp_index(warp) < 4 * kGroups) {
    // ================= decode groups: packed codes -> bf16 weight tile (K-major, 128-byte swizzle) =================
    const int dwarp = decode_warp_index(warp);
    const int grp = dwarp >> 2;
    const int u = (dwarp & 3) * 32 + lane;   // the weight row of the tile this thread decodes
    const uint32_t pick01 = p.nibble_high_first ? 0x4051u : 0x5140u;
    const uint32_t pick23 = p.nibble_high_first ? 0x6273u : 0x7362u;
    const long long kpr = p.k / 64;
    // 32-byte code rows loaded with the 32-byte TMA swizzle: the halves of rows 4..7 (mod 8) are exchanged
    const uint32_t flip = ((uint32_t)u >> 2) & 1u;
    const uint32_t src_off0 = (uint32_t)u * 32u + flip * 16u;
    const uint32_t src_off1 = (uint32_t)u * 32u + (flip ^ 1u) * 16u;
    const uint32_t dst_off = (uint32_t)u * 128u;
    const uint32_t swz = (uint32_t)u & 7u;
    const uint32_t lut_lane = lut0 + (uint32_t)lane * 4u;
    const float* table2 = reinterpret_cast<const float*>(smem_dyn + (code2_0 - raw));
    constexpr int kPrefetch = 4;   // absmax values are fetched this many of the group's blocks ahead of their use
    bool ok = true;
    int g_part = 0;                // running block number of the part's first block
    MOLT_SKINNY_PARTS(tile, kb0, kb1) {
      const long long row = (long long)tile * BR + u;
      const bool row_ok = row < p.n;
      const long long seg0 = (row_ok ? row : 0) * kpr;   // first absmax block of this row
      // raw absmax of block kb: the fp32 value, or (nested) the uint8 code and the second-level scale
      auto load_raw = [&](int kb, float& second) -> float {
        second = 0.f;
        if (kb >= kb1 || !row_ok) return 0.f;
        if (!kNested) return __ldg(reinterpret_cast<const float*>(p.absmax) + seg0 + kb);
        second = __ldg(p.absmax2 + ((seg0 + kb) >> p.block2_shift));
        return __uint_as_float((uint32_t)__ldg(reinterpret_cast<const uint8_t*>(p.absmax) + seg0 + kb));
      };
      const int kb_first = kb0 + ((grp - g_part) % kGroups + kGroups) % kGroups;
      float cur[kPrefetch], cur2[kPrefetch];
#pragma unroll
      for (int q = 0; q < kPrefetch; ++q) cur[q] = load_raw(kb_first + kGroups * q, cur2[q]);
      for (int kbq = kb_first; kbq < kb1 && ok; kbq += kGroups * kPrefetch) {
        float nxt[kPrefetch], nxt2[kPrefetch];
#pragma unroll
        for (int q = 0; q < kPrefetch; ++q) nxt[q] = load_raw(kbq + kGroups * (kPrefetch + q), nxt2[q]);
#pragma unroll
        for (int q = 0; q < kPrefetch; ++q) {
          const int kb = kbq + kGroups * q;
          if (kb >= kb1 || !ok) continue;
          float scale = cur[q];
          if (kNested)   // code2[u8] * absmax2 + offset with a separate multiply and add: the dequantiser's bits
            scale = row_ok ? __fadd_rn(__fmul_rn(table2[__float_as_uint(cur[q])], cur2[q]), p.offset) : 0.f;
          const int g = g_part + (kb - kb0);
          const int bs = g % kBStages, cs = g % kCodeStages;
          if (u == 0) MOLT_CTRACE(6, g);
          ok = wait_on(bar_pkfull(cs), (uint32_t)((g / kCodeStages) & 1), 5);
          if (ok && g >= kBStages) ok = wait_on(bar_consumed(g - kBStages), consumed_parity(g - kBStages), 6);
          if (!ok) continue;
          if (u == 0) MOLT_CTRACE(8, g);
          const uint32_t wt = wtile0 + (uint32_t)bs * kTileBytes;
          const uint32_t pk = codes0 + (uint32_t)cs * kPackedBytes;
#ifndef MOLT_SKINNY_EXP_NO_DECODE   // (timing experiment: waits and arrivals only; results are wrong)
          uint32_t words[8];
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(words[0]), "=r"(words[1]), "=r"(words[2]), "=r"(words[3])
                       : "r"(pk + src_off0)
                       : "memory");
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(words[4]), "=r"(words[5]), "=r"(words[6]), "=r"(words[7])
                       : "r"(pk + src_off1)
                       : "memory");
          if (kTable) {
            // The table never changes after start-up, so its loads are plain (not volatile) asm: the compiler may
            // issue the lookups of several words ahead of the stores and hide their latency.
            const uint32_t scale2 = pack_bf16x2(scale, scale);
#pragma unroll
            for (int c = 0; c < 8; ++c) {   // one word = 8 codes = 16 bytes of bf16 = one swizzled chunk of the row
              uint32_t out[4];
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                const uint32_t byte = __byte_perm(words[c], 0u, 0x4440u + (uint32_t)b);
                uint32_t pair;
                asm("ld.shared.b32 %0, [%1];" : "=r"(pair) : "r"(lut_lane + byte * 128u));
                asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(out[b]) : "r"(pair), "r"(scale2));
              }
              asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(wt + dst_off + (((uint32_t)c ^ swz) << 4)),
                           "r"(out[0]), "r"(out[1]), "r"(out[2]), "r"(out[3])
                           : "memory");
            }
          } else {
            const SegmentTable table = make_segment_table(p.codebook, scale);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              uint32_t out[4];
              decode_word(words[c], table, pick01, pick23, out);
              asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(wt + dst_off + (((uint32_t)c ^ swz) << 4)),
                           "r"(out[0]), "r"(out[1]), "r"(out[2]), "r"(out[3])
                           : "memory");
            }
          }
#endif
          fence_proxy_async();
          if (u == 0) MOLT_CTRACE(9, g);
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_bfull(bs));
        }
#pragma unroll
        for (int q = 0; q < kPrefetch; ++q) { cur[q] = nxt[q]; cur2[q] = nxt2[q]; }
      }
      if (!ok) break;
      g_part += kb1 - kb0;
    }
  } else if (warp < kEpilogueWarps) {
    // ================= epilogue: TMEM -> fp32 part [token][row] in the CTA's scratch slot =================
    const int row = warp * 32 + lane;
    uint32_t full_phase[2] = {0u, 0u};
    int parts_done = 0;
    bool ok = true;
    MOLT_SKINNY_PARTS(tile, kb0, kb1) {
      const int acc = parts_done & 1;
      ok = wait_on(bar_accfull(acc), full_phase[acc], 8);
      if (!ok) break;
      if (threadIdx.x == 0) MOLT_CTRACE(10, parts_done);
      full_phase[acc] ^= 1u;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(acc * kMmaWarps) * kAccStride;
      const bool both = kMmaWarps == 2 && kb1 - kb0 >= 2;   // the second issuer had blocks of this part
      float* part = p.partial + ((size_t)blockIdx.x * p.max_parts + (size_t)(tile - first_tile)) * (size_t)(NT * BR) + row;
#pragma unroll 1
      for (int cg = 0; cg < (NT + 31) / 32; ++cg) {
        uint32_t v[32], w[32];
        tmem_ld32(t_row + (uint32_t)cg * 32u, v);
        if (both) tmem_ld32(t_row + kAccStride + (uint32_t)cg * 32u, w);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int tok = cg * 32 + c;
          const float value = __uint_as_float(v[c]) + (both ? __uint_as_float(w[c]) : 0.f);
          if (tok < p.m) __stcg(part + (size_t)tok * BR, value);   // a warp writes 128 contiguous bytes
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_accempty(acc));
      if (threadIdx.x == 0) MOLT_CTRACE(11, parts_done);
      ++parts_done;
    }
  }
#undef MOLT_SKINNY_PARTS

  // ---- teardown ----
  if (threadIdx.x == 0) MOLT_CTRACE(15, 2);
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);   // copies in flight land before the CTA gives up its memory
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
  if (threadIdx.x == 0) MOLT_CTRACE(15, 3);
}

// Low-rank input, first stage: part[ks][tok][j] = sum over the ks-th slice of K of x[tok][k] * bf16(A[j][k]).
// Grid (adapter rows, K slices, groups of 16 tokens); the slices are added in a fixed order by the reader.  Launched
// behind the streaming kernel as its programmatic dependent and without waiting for it (it reads only x and A), so its
// blocks run beside that grid on the registers and shared memory it leaves free.
__global__ void __maxnreg__(64) skinny_lowrank_kernel(const __nv_bfloat16* __restrict__ x,
                                                                         const float* __restrict__ a, int m, int m_pad,
                                                                         long long k, float* __restrict__ part) {
  __shared__ float red[kLowrankThreads / 32][16];
  const int j = blockIdx.x, ks = blockIdx.y, tok0 = blockIdx.z * 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long slice = (k / 8 + kLowrankSlices - 1) / kLowrankSlices * 8;   // columns per slice, a multiple of 8
  const long long c_begin = ks * slice, c_end = c_begin + slice < k ? c_begin + slice : k;
  float sums[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) sums[i] = 0.f;
  for (long long c = c_begin + threadIdx.x * 8LL; c < c_end; c += kLowrankThreads * 8) {
    const float4 a0 = __ldg(reinterpret_cast<const float4*>(a + j * k + c));
    const float4 a1 = __ldg(reinterpret_cast<const float4*>(a + j * k + c + 4));
    const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    float ab[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) ab[i] = __bfloat162float(__float2bfloat16_rn(av[i]));
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      if (tok0 + t >= m) continue;
      const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x + (long long)(tok0 + t) * k + c));
      const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        sums[t] = fmaf(bf16_lo(xw[i]), ab[2 * i], sums[t]);
        sums[t] = fmaf(bf16_hi(xw[i]), ab[2 * i + 1], sums[t]);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < 16; ++t) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sums[t] += __shfl_xor_sync(0xffffffffu, sums[t], o);
    if (lane == 0) red[warp][t] = sums[t];
  }
  __syncthreads();
  if (threadIdx.x < 16) {
    const int t = threadIdx.x;
    float total = 0.f;
#pragma unroll
    for (int wv = 0; wv < kLowrankThreads / 32; ++wv) total += red[wv][t];
    part[((size_t)ks * m_pad + tok0 + t) * 64 + j] = total;
  }
  // This grid must not be seen as complete before the streaming kernel in front of it is: the kernel behind is an
  // ordinary launch that orders itself after this one only.
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// y[tok, row] = bf16(sum of the parts of the row's tile, in CTA order, + sum_j bf16(s B[row, j]) bf16(T[tok, j])),
// T = sum of its K slices, rounded to bf16.  Grid (row tiles, groups of 16 tokens); a block has one thread per (row,
// group of kTok tokens), i.e. 128 * 16 / kTok threads.  The kernel is nothing but round trips to memory with a little
// arithmetic behind them, so everything it reads is asked for up front and together: the slices of T, the tile's
// adapter rows (contiguous in memory: read coalesced and staged in shared memory, rounded once) and the parts of the
// tile (addresses of up to four parts are formed before any of them is read).  The blocks of tile 0 also write T
// (bf16, [m, 64], zero padded) when the caller wants it.
template <int kTok>
__global__ void __launch_bounds__(BR * 16 / kTok) skinny_finish_kernel(const float* __restrict__ partial, int nt, int max_parts,
                                                                      Ranges ranges, int nb, long long units,
                                                                      const float* __restrict__ low_part, int m, int m_pad,
                                                                      const float* __restrict__ lora_b, float scaling,
                                                                      int rank, long long n, __nv_bfloat16* __restrict__ y,
                                                                      __nv_bfloat16* __restrict__ t_out) {
  constexpr int kThreadsF = BR * 16 / kTok;
  constexpr int kPartsAtOnce = 4;
  __shared__ float t_s[16][64];
  __shared__ float b_s[BR][64 + 1];   // bf16(s B) of the tile's rows, as fp32 (row pitch 65: no bank conflicts by row)
  const int tile = blockIdx.x;
  const int r = threadIdx.x & (BR - 1);
  const int tok0 = blockIdx.y * 16, tokq = tok0 + (threadIdx.x / BR) * kTok;   // first token of the block / of this thread
  const long long row = (long long)tile * BR + r;
  const bool row_ok = row < n;
  // The CTAs whose ranges hold units of this tile: range c starts at floor(units c / ctas), so the last range that
  // starts at or before unit u is floor(((u + 1) ctas - 1) / units).
  const long long unit0 = (long long)tile * nb, unit1 = unit0 + nb;
  const int first = (int)(((unit0 + 1) * ranges.ctas - 1) / units);
  const int last = (int)((unit1 * ranges.ctas - 1) / units);

  // ---- requests: the first parts of the tile ----
  float acc[kTok];
#pragma unroll
  for (int t = 0; t < kTok; ++t) acc[t] = 0.f;
  float got[kPartsAtOnce][kTok];
  auto request_parts = [&](int c0) {
#pragma unroll
    for (int q = 0; q < kPartsAtOnce; ++q) {
      const int c = c0 + q;
      const bool live = row_ok && c <= last;
      const int slot = live ? tile - range_begin(ranges, c) / nb : 0;
      const float* src = partial + ((size_t)(live ? c : 0) * max_parts + slot) * (size_t)(nt * BR) + r;
#pragma unroll
      for (int t = 0; t < kTok; ++t) got[q][t] = (live && tokq + t < m) ? __ldcg(src + (size_t)(tokq + t) * BR) : 0.f;
    }
  };
  request_parts(first);
  // ---- requests: T's slices and the tile's adapter rows, then into shared memory ----
  for (int i = threadIdx.x; i < 16 * rank; i += kThreadsF) {
    const int t = i / rank, j = i - t * rank;
    float total = 0.f;
    if (tok0 + t < m) {
      float slice[kLowrankSlices];
#pragma unroll
      for (int ks = 0; ks < kLowrankSlices; ++ks) slice[ks] = __ldcg(low_part + ((size_t)ks * m_pad + tok0 + t) * 64 + j);
#pragma unroll
      for (int ks = 0; ks < kLowrankSlices; ++ks) total += slice[ks];
    }
    t_s[t][j] = __bfloat162float(__float2bfloat16_rn(total));
  }
  {
    const long long rows_here = n - (long long)tile * BR < BR ? n - (long long)tile * BR : BR;
    const float* b0 = lora_b + (long long)tile * BR * rank;        // rows_here * rank contiguous floats
    const int count = (int)rows_here * rank;
    if ((rank & 3) == 0 && (reinterpret_cast<uintptr_t>(b0) & 15) == 0) {
      for (int i = threadIdx.x * 4; i < count; i += kThreadsF * 4) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(b0 + i));
        const int br = i / rank, bj = i - br * rank;                 // four consecutive columns of one row
        b_s[br][bj] = __bfloat162float(__float2bfloat16_rn(scaling * v.x));
        b_s[br][bj + 1] = __bfloat162float(__float2bfloat16_rn(scaling * v.y));
        b_s[br][bj + 2] = __bfloat162float(__float2bfloat16_rn(scaling * v.z));
        b_s[br][bj + 3] = __bfloat162float(__float2bfloat16_rn(scaling * v.w));
      }
    } else {
      for (int i = threadIdx.x; i < count; i += kThreadsF) {
        const int br = i / rank, bj = i - br * rank;
        b_s[br][bj] = __bfloat162float(__float2bfloat16_rn(scaling * __ldg(b0 + i)));
      }
    }
  }
  // ---- the parts, in CTA order ----
  for (int c0 = first; c0 <= last; c0 += kPartsAtOnce) {
    if (c0 != first) request_parts(c0);
#pragma unroll
    for (int q = 0; q < kPartsAtOnce; ++q)
#pragma unroll
      for (int t = 0; t < kTok; ++t) acc[t] += got[q][t];          // absent parts and tokens were read as zero
  }
  __syncthreads();
  if (t_out != nullptr && tile == 0) {   // T itself, zero padded to 64 columns
    for (int i = threadIdx.x; i < 16 * 64; i += kThreadsF) {
      const int t = i >> 6, j = i & 63;
      if (tok0 + t < m) t_out[(size_t)(tok0 + t) * 64 + j] = __float2bfloat16_rn(j < rank ? t_s[t][j] : 0.f);
    }
  }
  if (!row_ok || tokq >= m) return;
  const int tl = tokq - tok0;
  for (int j0 = 0; j0 < rank; j0 += 16) {
    float b[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) b[j] = j0 + j < rank ? b_s[r][j0 + j] : 0.f;
#pragma unroll
    for (int t = 0; t < kTok; ++t) {
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) sum = fmaf(b[j], j0 + j < rank ? t_s[tl + t][j0 + j] : 0.f, sum);
      acc[t] += sum;
    }
  }
#pragma unroll
  for (int t = 0; t < kTok; ++t)
    if (tokq + t < m) y[(size_t)(tokq + t) * n + row] = __float2bfloat16_rn(acc[t]);
}

// The same for more than 16 tokens, with a thread owning four neighbouring rows and four tokens (a warp = the tile's
// 128 rows x four tokens; block = four warps = the 16 tokens of its group): a part is read with one 16-byte load per
// lane and token (512 contiguous bytes per warp), an output row segment is written 8 bytes per lane, and a value of T
// read from shared memory serves four rows.  Sums are formed in the same order as in the kernel above.
__global__ void __launch_bounds__(BR) skinny_finish_quad_kernel(const float* __restrict__ partial, int nt, int max_parts,
                                                                Ranges ranges, int nb, long long units,
                                                                const float* __restrict__ low_part, int m, int m_pad,
                                                                const float* __restrict__ lora_b, float scaling, int rank,
                                                                long long n, __nv_bfloat16* __restrict__ y,
                                                                __nv_bfloat16* __restrict__ t_out) {
  constexpr int kThreadsF = BR;
  constexpr int kPartsAtOnce = 4;
  __shared__ __align__(16) float t_s[16][64];
  __shared__ __align__(16) float b_t[64][BR];   // bf16(s B) of the tile's rows, as fp32, transposed: [column][row]
  const int tile = blockIdx.x;
  const int rq = threadIdx.x & 31, tq = threadIdx.x >> 5;
  const int tok0 = blockIdx.y * 16, tokq = tok0 + tq * 4;
  const long long row = (long long)tile * BR + rq * 4;              // first of this thread's four rows
  const bool row_ok = row < n;                                      // n is a multiple of 64: a quad is all in or all out
  const long long unit0 = (long long)tile * nb, unit1 = unit0 + nb;
  const int first = (int)(((unit0 + 1) * ranges.ctas - 1) / units);
  const int last = (int)((unit1 * ranges.ctas - 1) / units);

  float acc[4][4];   // [token][row]
#pragma unroll
  for (int t = 0; t < 4; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[t][i] = 0.f;
  float4 got[kPartsAtOnce][4];
  auto request_parts = [&](int c0) {
#pragma unroll
    for (int q = 0; q < kPartsAtOnce; ++q) {
      const int c = c0 + q;
      const bool live = row_ok && c <= last;
      const int slot = live ? tile - range_begin(ranges, c) / nb : 0;
      const float* src = partial + ((size_t)(live ? c : 0) * max_parts + slot) * (size_t)(nt * BR) + rq * 4;
#pragma unroll
      for (int t = 0; t < 4; ++t)
        got[q][t] = (live && tokq + t < m) ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)(tokq + t) * BR))
                                           : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  request_parts(first);
  for (int i = threadIdx.x; i < 16 * rank; i += kThreadsF) {
    const int t = i / rank, j = i - t * rank;
    float total = 0.f;
    if (tok0 + t < m) {
      float slice[kLowrankSlices];
#pragma unroll
      for (int ks = 0; ks < kLowrankSlices; ++ks) slice[ks] = __ldcg(low_part + ((size_t)ks * m_pad + tok0 + t) * 64 + j);
#pragma unroll
      for (int ks = 0; ks < kLowrankSlices; ++ks) total += slice[ks];
    }
    t_s[t][j] = __bfloat162float(__float2bfloat16_rn(total));
  }
  {
    const long long rows_here = n - (long long)tile * BR < BR ? n - (long long)tile * BR : BR;
    const float* b0 = lora_b + (long long)tile * BR * rank;        // rows_here * rank contiguous floats
    const int count = (int)rows_here * rank;
    if ((rank & 3) == 0 && (reinterpret_cast<uintptr_t>(b0) & 15) == 0) {
      for (int i = threadIdx.x * 4; i < count; i += kThreadsF * 4) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(b0 + i));
        const int br = i / rank, bj = i - br * rank;
        b_t[bj][br] = __bfloat162float(__float2bfloat16_rn(scaling * v.x));
        b_t[bj + 1][br] = __bfloat162float(__float2bfloat16_rn(scaling * v.y));
        b_t[bj + 2][br] = __bfloat162float(__float2bfloat16_rn(scaling * v.z));
        b_t[bj + 3][br] = __bfloat162float(__float2bfloat16_rn(scaling * v.w));
      }
    } else {
      for (int i = threadIdx.x; i < count; i += kThreadsF) {
        const int br = i / rank, bj = i - br * rank;
        b_t[bj][br] = __bfloat162float(__float2bfloat16_rn(scaling * __ldg(b0 + i)));
      }
    }
  }
  for (int c0 = first; c0 <= last; c0 += kPartsAtOnce) {
    if (c0 != first) request_parts(c0);
#pragma unroll
    for (int q = 0; q < kPartsAtOnce; ++q)
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        acc[t][0] += got[q][t].x; acc[t][1] += got[q][t].y; acc[t][2] += got[q][t].z; acc[t][3] += got[q][t].w;
      }
  }
  __syncthreads();
  if (t_out != nullptr && tile == 0) {   // T itself, zero padded to 64 columns
    for (int i = threadIdx.x; i < 16 * 64; i += kThreadsF) {
      const int t = i >> 6, j = i & 63;
      if (tok0 + t < m) t_out[(size_t)(tok0 + t) * 64 + j] = __float2bfloat16_rn(j < rank ? t_s[t][j] : 0.f);
    }
  }
  if (!row_ok || tokq >= m) return;
  for (int j0 = 0; j0 < rank; j0 += 16) {
    float sum[4][4];
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) sum[t][i] = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      if (j0 + j < rank) {   // (uniform) columns past the rank add nothing, as multiplying by zero would
        float tv[4];
        const float4 b4 = *reinterpret_cast<const float4*>(&b_t[j0 + j][rq * 4]);   // this thread's four rows
        const float b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) tv[t] = t_s[tq * 4 + t][j0 + j];
#pragma unroll
        for (int t = 0; t < 4; ++t)
#pragma unroll
          for (int i = 0; i < 4; ++i) sum[t][i] = fmaf(b[i], tv[t], sum[t][i]);
      }
    }
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[t][i] += sum[t][i];
  }
#pragma unroll
  for (int t = 0; t < 4; ++t)
    if (tokq + t < m) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(acc[t][0], acc[t][1]), hi = __floats2bfloat162_rn(acc[t][2], acc[t][3]);
      uint2 out;
      out.x = *reinterpret_cast<uint32_t*>(&lo);
      out.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(y + (size_t)(tokq + t) * n + row) = out;
    }
}

struct Plan {
  int nt, ctas, max_parts, m_pad;
  Ranges ranges;
  size_t low_bytes, partial_bytes;
};

static Plan make_plan(long long n, long long k, long long m) {
  Plan pl;
  pl.nt = m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128;
  const long long tiles = (n + BR - 1) / BR, nb = k / BK, units = tiles * nb;
  long long ctas = sm_count();
  if (ctas > units / 8) ctas = units / 8 > 0 ? units / 8 : 1;   // at least eight blocks per CTA
  pl.ctas = (int)ctas;
  pl.ranges.quot = (int)(units / ctas);
  pl.ranges.rem = (int)(units % ctas);
  pl.ranges.ctas = (int)ctas;
  const long long range = (units + ctas - 1) / ctas;
  pl.max_parts = (int)((range + nb - 1) / nb) + 1;
  pl.m_pad = (int)((m + 15) / 16 * 16);
  pl.low_bytes = ((size_t)kLowrankSlices * pl.m_pad * 64 * sizeof(float) + 255) / 256 * 256;
  pl.partial_bytes = (size_t)pl.ctas * pl.max_parts * pl.nt * BR * sizeof(float);
  return pl;
}

}  // namespace skinny

bool sm100_skinny_supported(const WeightView& w, int rank, long long m) {
  return w.blocksize == 64 && w.k % 64 == 0 && w.n % 64 == 0 && rank >= 1 && rank <= 64 && m >= 1 && m <= 128 &&
         (w.absmax_kind != MOLT_ABSMAX_NESTED || w.block2_shift >= 0) && w.k / 64 * ((w.n + 127) / 128) < (1LL << 30);
}

size_t sm100_skinny_bytes(long long n, long long k, long long m) {
  const skinny::Plan pl = skinny::make_plan(n, k, m);
  return pl.low_bytes + pl.partial_bytes + 256;
}

int sm100_skinny_forward(const WeightView& w, const __nv_bfloat16* x, const float* lora_a, const float* lora_b,
                         float scaling, int rank, __nv_bfloat16* y, int m, __nv_bfloat16* t_out, void* workspace,
                         size_t workspace_bytes, int flags, cudaStream_t s) {
  using namespace skinny;
  if (!sm100_skinny_supported(w, rank, m)) return fail(MOLT_E_CAPABILITY, "few-token tcgen05 forward: unsupported shape");
  MOLT_REQUIRE((reinterpret_cast<uintptr_t>(lora_a) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0, MOLT_E_CAPABILITY,
               "few-token tcgen05 forward: x and lora_a must start on 16-byte boundaries");
  const Plan pl = make_plan(w.n, w.k, m);
  const uintptr_t ws0 = (reinterpret_cast<uintptr_t>(workspace) + 255) & ~(uintptr_t)255;
  MOLT_REQUIRE(workspace != nullptr && ws0 + pl.low_bytes + pl.partial_bytes <= reinterpret_cast<uintptr_t>(workspace) + workspace_bytes,
               MOLT_E_VALUE, "few-token tcgen05 forward: workspace too small");
  float* low_part = reinterpret_cast<float*>(ws0);
  float* partial = reinterpret_cast<float*>(ws0 + pl.low_bytes);

  CUtensorMap map_x, map_packed;
  if (int rc = make_tensor_map(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, w.k, m, w.k * 2, BK, pl.nt,
                               CU_TENSOR_MAP_SWIZZLE_128B, "tokens"))
    return rc;
  if (int rc = make_tensor_map(&map_packed, CU_TENSOR_MAP_DATA_TYPE_UINT8, w.packed, w.k / 2, w.n, w.k / 2, BK / 2, BR,
                               CU_TENSOR_MAP_SWIZZLE_32B, "packed weight"))
    return rc;
  Params p;
  p.absmax = w.absmax;
  p.absmax2 = w.absmax2;
  p.code2 = w.code2;
  p.offset = w.offset;
  p.block2_shift = w.block2_shift;
  p.status = device_status_word();
  if (p.status == nullptr) return fail(MOLT_E_RUNTIME, "few-token tcgen05 forward: no device status word");
  p.n = w.n;
  p.k = w.k;
  p.m = m;
  p.num_kb = (int)(w.k / BK);
  p.tiles = (int)((w.n + BR - 1) / BR);
  p.max_parts = pl.max_parts;
  p.ranges = pl.ranges;
  p.partial = partial;
  p.nibble_high_first = w.nibble_order == MOLT_NIBBLE_HIGH_FIRST ? 1 : 0;
  p.wait_cycles = wait_limit_cycles();
  p.withhold = take_withheld_blocks();
  for (int i = 0; i < 16; ++i) p.codebook[i] = w.codebook[i];
#ifdef MOLT_SKINNY_TRACE
  {
    const char* tr = getenv("MOLT_B200_TRACE_PTR");   // device pointer (decimal) of a 16 KB trace buffer
    p.trace = tr != nullptr ? reinterpret_cast<unsigned long long*>(strtoull(tr, nullptr, 10)) : nullptr;
  }
#endif

  const bool nested = w.absmax_kind == MOLT_ABSMAX_NESTED;
  const bool table = !(flags & kGemmExactDecode);   // table decode unless the caller asks for the dequantiser's bits
  static thread_local bool configured[64][4][2][2] = {};
  int dev = 0;
  MOLT_CUDA(cudaGetDevice(&dev));
  const int nt_index = pl.nt == 16 ? 0 : pl.nt == 32 ? 1 : pl.nt == 64 ? 2 : 3;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)pl.ctas);
  cfg.blockDim = dim3((unsigned)kThreads);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
#define MOLT_SKINNY_LAUNCH(NTOK, NESTED, TABLE)                                                                   \
  do {                                                                                                            \
    auto kernel = nf4_skinny_sm100_kernel<NTOK, NESTED, TABLE>;                                                   \
    cfg.dynamicSmemBytes = smem_bytes(NTOK, TABLE);                                                               \
    const bool need_config = dev >= 0 && dev < 64 && !configured[dev][nt_index][NESTED ? 1 : 0][TABLE ? 1 : 0];   \
    if (need_config) {                                                                                            \
      MOLT_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,                         \
                                     (int)smem_bytes(NTOK, TABLE)));                                              \
      configured[dev][nt_index][NESTED ? 1 : 0][TABLE ? 1 : 0] = true;                                            \
    }                                                                                                             \
    MOLT_CUDA(cudaLaunchKernelEx(&cfg, kernel, map_x, map_packed, p));                                            \
  } while (0)
#define MOLT_SKINNY_BY_NT(NESTED, TABLE)                            \
  do {                                                              \
    if (pl.nt == 16) MOLT_SKINNY_LAUNCH(16, NESTED, TABLE);         \
    else if (pl.nt == 32) MOLT_SKINNY_LAUNCH(32, NESTED, TABLE);    \
    else if (pl.nt == 64) MOLT_SKINNY_LAUNCH(64, NESTED, TABLE);    \
    else MOLT_SKINNY_LAUNCH(128, NESTED, TABLE);                    \
  } while (0)
  if (table) {
    if (nested) MOLT_SKINNY_BY_NT(true, true);
    else MOLT_SKINNY_BY_NT(false, true);
  } else {
    if (nested) MOLT_SKINNY_BY_NT(true, false);
    else MOLT_SKINNY_BY_NT(false, false);
  }
#undef MOLT_SKINNY_BY_NT
#undef MOLT_SKINNY_LAUNCH
  if (int rc = launch_status("nf4_skinny_sm100_kernel")) return rc;

  {   // the low-rank input, beside the streaming kernel (the second stage behind both is an ordinary launch)
    cudaLaunchConfig_t lcfg = {};
    lcfg.gridDim = dim3((unsigned)rank, kLowrankSlices, (unsigned)(pl.m_pad / 16));
    lcfg.blockDim = dim3(kLowrankThreads);
    lcfg.stream = s;
    lcfg.attrs = attr;
    lcfg.numAttrs = 1;
    MOLT_CUDA(cudaLaunchKernelEx(&lcfg, skinny_lowrank_kernel, x, lora_a, m, pl.m_pad, (long long)w.k, low_part));
    if (int rc = launch_status("skinny_lowrank_kernel")) return rc;
  }

  // an ordinary launch: placing its blocks early, as a programmatic dependent, was measured to be slower.
  // Up to 16 tokens: one thread per row and four tokens (512 threads per tile).  More tokens: four rows x four tokens
  // per thread (16-byte loads and 8-byte stores; 6.0 us against 10.4 us at 64 tokens for one row x sixteen tokens).
  const dim3 fgrid((unsigned)p.tiles, (unsigned)((m + 15) / 16));
  if (m <= 16)
    skinny_finish_kernel<4><<<fgrid, BR * 4, 0, s>>>(partial, pl.nt, pl.max_parts, pl.ranges, p.num_kb,
                                                      (long long)p.tiles * p.num_kb, low_part, m, pl.m_pad, lora_b,
                                                      scaling, rank, w.n, y, t_out);
#ifdef MOLT_SKINNY_EXP_FINISH_ROWS   // comparison build: a thread owns one row and sixteen tokens
  else
    skinny_finish_kernel<16><<<fgrid, BR, 0, s>>>(partial, pl.nt, pl.max_parts, pl.ranges, p.num_kb,
                                                   (long long)p.tiles * p.num_kb, low_part, m, pl.m_pad, lora_b, scaling,
                                                   rank, w.n, y, t_out);
#else
  else
    skinny_finish_quad_kernel<<<fgrid, BR, 0, s>>>(partial, pl.nt, pl.max_parts, pl.ranges, p.num_kb,
                                                    (long long)p.tiles * p.num_kb, low_part, m, pl.m_pad, lora_b, scaling,
                                                    rank, w.n, y, t_out);
#endif
  return launch_status("skinny_finish_kernel");
}

}  // namespace molt
