// Small-token (M <= 16) NF4 + LoRA forward: y = x . deq(W)^T + s (x A^T) B^T with the packed weight streamed from
// HBM exactly once, straight into registers.
//
// One kernel does the whole product.  A CTA owns a contiguous range of 8-row groups of W with their FULL rows, so
// nothing leaves the SM as a partial sum.  Inside the CTA the warps split the contraction: a warp owns a K-slice of
// up to four absmax blocks (64 columns each) per pass, keeps the matching X fragments in registers, and walks over
// the CTA's row groups two at a time (16 weight rows = the M dimension of mma.sync m16n8k16; the tokens are the N
// dimension, eight per MMA).  Per 16 x 64 tile a lane issues two 8-byte loads of packed codes (the four lanes of a
// quad cover the 32 contiguous bytes of one row's block, so every 32-byte sector fetched is used in full) a few
// tiles ahead of their use (the absmax of the CTA's rows is staged in shared memory once per pass, resolved to fp32), expands every byte into a bf16 pair of codebook values with one byte-permute (table
// offset) and one shared-memory lookup (table replicated per lane, conflict-free), and runs four MMAs on the UNSCALED
// values; the fp32 absmax of the row's block scales the block's partial sum afterwards (one FMA per accumulator), so
// no per-element multiply is needed.  The accumulators of all row groups stay in registers for the whole kernel;
// the warps' K-slice sums meet once, at the end, through shared memory (the table's space is reused), in warp order
// (deterministic).  The summing threads add the low-rank term s T B^T and round once to bf16.
//
// T = bf16(x . bf16(A)^T) is produced by a small companion kernel launched in front.  The streaming kernel is launched
// as its programmatic dependent: it starts at once and only waits for T (griddepcontrol.wait) after its own stream
// is done, so the two run concurrently and the caller sees one kernel's latency.
//
// No thread waits on another except at __syncthreads, so there is no bounded-wait machinery here.
#ifdef MOLT_GEMV_TRACE
#include <stdlib.h>
#endif

#include "internal.h"

namespace molt {

constexpr int kGemvLowrankSlices = 8;    // K slices of the low-rank input's first stage
constexpr int kGemvLowrankThreads = 128;
constexpr int kGemvMaxPairs = 7;            // row-group pairs (16 weight rows) per CTA whose sums stay in registers
constexpr int kGemvLutStride = 256;         // bytes per table entry: 32 lanes x 4 bytes used, so that (byte << 8) | (lane * 4)
constexpr int kGemvLutBytes = 256 * kGemvLutStride;   // is the offset and one byte-permute builds it

struct GemvParams {
  WeightView w;
  const __nv_bfloat16* x;    // [m, k]
  const float* lora_b;       // [n, rank] fp32
  const float* t;            // [slices][16][64] fp32: the K slices of x . bf16(A)^T (written by the companion kernel)
  __nv_bfloat16* y;          // [m, n]
  float scaling;
  int rank;
  int m;
  int nblk;                  // k / 64
  int warps;                 // streaming warps that own a K-slice (<= the kernel's warp count)
  int passes;                // K passes: pass p covers blocks [p * warps * BPW, (p + 1) * warps * BPW)
  int groups_total;          // n / 8
  int ctas;
#ifdef MOLT_GEMV_TRACE
  unsigned long long* trace;   // [8 stamps][2 CTAs] globaltimer values of the first and the last CTA
#endif
};

#ifdef MOLT_GEMV_TRACE
#define GEMV_STAMP(i)                                                                                  \
  do {                                                                                                 \
    if (threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1)) {                        \
      unsigned long long now;                                                                          \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));                                          \
      p.trace[(i) * 2 + (blockIdx.x == 0 ? 0 : 1)] = now;                                              \
    }                                                                                                  \
  } while (0)
#else
#define GEMV_STAMP(i) do {} while (0)
#endif

__device__ __forceinline__ void gemv_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1, const float (&c)[4]) {
#if defined(MOLT_GEMV_EXP) && (MOLT_GEMV_EXP & 2)   // instruction-count experiment: no MMAs (results are wrong)
  d[0] = c[0] + __uint_as_float(a0 ^ b0); d[1] = c[1] + __uint_as_float(a1 ^ b1);
  d[2] = c[2] + __uint_as_float(a2); d[3] = c[3] + __uint_as_float(a3);
  return;
#endif
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

__device__ __forceinline__ uint2 ldg_stream8(const void* p) {
  uint2 v;
  // L2::128B: a miss brings the whole 128-byte line into L2, so DRAM sees full-line requests although a lane asks for 8
  // bytes and a quad for one 32-byte sector; the line's other sectors are this warp's next blocks or its neighbours'.
  asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

// Ring of tiles in flight per warp: R = BPW * U tiles (U row-group pairs), refilled as tiles are consumed.
#ifndef MOLT_GEMV_RING
#define MOLT_GEMV_RING 4
#endif
constexpr int gemv_unroll_pairs(int bpw) { return bpw == 3 ? 2 : (MOLT_GEMV_RING / bpw > 0 ? MOLT_GEMV_RING / bpw : 1); }
constexpr int kGemvMaxRows = 2 * kGemvMaxPairs * 8;                       // weight rows a CTA owns at most
constexpr int kGemvScaleStride = 64 + 1;                                  // floats per row of the staged absmax (+1: no bank conflicts)
constexpr int kGemvScaleBytes = kGemvMaxRows * kGemvScaleStride * 4;

constexpr size_t gemv_smem_bytes(int warps, int tt) {
  return (size_t)kGemvLutBytes + (size_t)warps * kGemvMaxPairs * tt * 32 * sizeof(float4) + kGemvScaleBytes;
}

// WARPS: warps per CTA.  BPW: absmax blocks per warp per pass
// (WARPS x BPW <= 64).  TT: token tiles of eight (1 for m <= 8, 2 for m <= 16).
template <int WARPS, int BPW, int TT>
__global__ void __launch_bounds__(WARPS * 32, 1) nf4_gemv_kernel(const __grid_constant__ GemvParams p) {
  constexpr int kGemvWarps = WARPS;
  static_assert(WARPS * BPW <= 64, "a pass covers at most 64 absmax blocks (staged absmax rows)");
  constexpr int U = gemv_unroll_pairs(BPW);
  constexpr int R = BPW * U;
  extern __shared__ __align__(256) unsigned char smem_raw[];
  unsigned char* lut_bytes = smem_raw;                                          // [256 entries][256 bytes]
  float4* sums = reinterpret_cast<float4*>(smem_raw + kGemvLutBytes);           // [warp][pair][tt][lane]
  float* scales_s = reinterpret_cast<float*>(smem_raw + kGemvLutBytes +
                                             kGemvWarps * kGemvMaxPairs * TT * 32 * sizeof(float4));   // [row][block of the pass]
  __shared__ float t_s[16 * 64];

  GEMV_STAMP(0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const bool nested = p.w.absmax_kind == MOLT_ABSMAX_NESTED;

  // ---- this CTA's row groups: [group0, group1), walked in pairs ----
  const int group0 = (int)(((long long)p.groups_total * blockIdx.x) / p.ctas);
  const int group1 = (int)(((long long)p.groups_total * (blockIdx.x + 1)) / p.ctas);
  const int ngroups = group1 - group0;
  const int npairs = (ngroups + 1) >> 1;
  const long long row_bytes = p.w.k / 2;

  // ---- table: byte -> bf16 pair (first element, second element) of codebook values, one copy per lane ----
  for (int i = threadIdx.x; i < 256 * 8; i += kGemvWarps * 32) {
    const int byte = i >> 3;
    const int first = p.w.nibble_order == MOLT_NIBBLE_LOW_FIRST ? (byte & 15) : (byte >> 4);
    const int second = p.w.nibble_order == MOLT_NIBBLE_LOW_FIRST ? (byte >> 4) : (byte & 15);
    const uint32_t pair = pack_bf16x2(p.w.codebook[first], p.w.codebook[second]);
    *reinterpret_cast<uint4*>(lut_bytes + byte * kGemvLutStride + (i & 7) * 16) = make_uint4(pair, pair, pair, pair);
  }

  const uint32_t lane4 = (uint32_t)lane * 4u;
  auto lookup = [&](uint32_t q, uint32_t selector) -> uint32_t {   // table entry of one code byte of q
#if defined(MOLT_GEMV_EXP) && (MOLT_GEMV_EXP & 1)   // instruction-count experiment: no table lookups (results are wrong)
    return q ^ selector ^ lane4;
#else
    return *reinterpret_cast<const uint32_t*>(lut_bytes + __byte_perm(q, lane4, selector));
#endif
  };
  const float zero[4] = {0.f, 0.f, 0.f, 0.f};
  const long long pair_stride = 16 * row_bytes;                   // bytes between the first rows of two pairs
  const int blocks_per_pass = p.warps * BPW;

  for (int pass = 0; pass < p.passes; ++pass) {
    const int pass_blk0 = pass * blocks_per_pass;
    int pass_blocks = p.nblk - pass_blk0;
    if (pass_blocks > blocks_per_pass) pass_blocks = blocks_per_pass;
    const int blk0 = pass_blk0 + warp * BPW;                      // first absmax block of this warp's K-slice
    int nb = p.nblk - blk0;
    if (nb > BPW) nb = BPW;
    const bool streaming = warp < p.warps && nb > 0;

    // ---- first requests of the codes: before anything else, so that the stream from HBM starts at once ----
    // Ring slot = (pair within the unrolled group) * BPW + b.  Lane (g, t) reads bytes 8 t .. 8 t + 7 of the block's 32
    // in rows g of both groups of the pair; a missing block (b >= nb) re-reads block blk0 and meets zero X fragments,
    // a missing second group (odd group count) re-reads the first.
    const uint8_t* cp = p.w.packed + ((long long)group0 * 8 + g) * row_bytes + (long long)blk0 * 32 + 8 * t;
    uint2 q0[R], q1[R];
    auto request_pair = [&](int u, const uint8_t* src, int pr) {
      const long long second = (2 * pr + 1 < ngroups) ? 8 * row_bytes : 0;
#pragma unroll
      for (int b = 0; b < BPW; ++b) {
        const int off = b < nb ? b * 32 : 0;
        q0[u * BPW + b] = ldg_stream8(src + off);
        q1[u * BPW + b] = ldg_stream8(src + second + off);
      }
    };
    if (streaming) {
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (u < npairs) request_pair(u, cp + (long long)u * pair_stride, u);
    }

    // ---- absmax of this CTA's rows for the blocks of this pass, resolved to fp32, into shared memory ----
    if (pass > 0) __syncthreads();                                // the previous pass no longer reads the staged values
    {
      // all loads first (they are independent), then the arithmetic: one round trip to memory instead of one per value.
      // A warp takes rows warp, warp + WARPS, ...; a lane takes blocks lane and lane + 32 of the pass (at most 64).
      constexpr int kRowsPerWarp = (kGemvMaxRows + kGemvWarps - 1) / kGemvWarps;
      const int nrows = ngroups * 8;
      float first[kRowsPerWarp][2], second[kRowsPerWarp][2];
#pragma unroll
      for (int j = 0; j < kRowsPerWarp; ++j) {
        const int row = warp + j * kGemvWarps;
        const long long blk_row = ((long long)group0 * 8 + row) * p.nblk + pass_blk0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int b = lane + 32 * h;
          first[j][h] = second[j][h] = 0.f;
          if (row < nrows && b < pass_blocks) {
            if (!nested) {
              first[j][h] = __ldg(reinterpret_cast<const float*>(p.w.absmax) + blk_row + b);
            } else {
              first[j][h] = __ldg(p.w.code2 + __ldg(reinterpret_cast<const uint8_t*>(p.w.absmax) + blk_row + b));
              second[j][h] = __ldg(p.w.absmax2 + ((blk_row + b) >> p.w.block2_shift));
            }
          }
        }
      }
#pragma unroll
      for (int j = 0; j < kRowsPerWarp; ++j) {
        const int row = warp + j * kGemvWarps;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int b = lane + 32 * h;
          // nested: code2[u8] * absmax2 + offset with a separate multiply and add, the dequantiser's bits
          if (row < nrows && b < pass_blocks)
            scales_s[row * kGemvScaleStride + b] =
                nested ? __fadd_rn(__fmul_rn(first[j][h], second[j][h]), p.w.offset) : first[j][h];
        }
      }
    }

    // ---- X fragments of the K-slice: lane (g, t) holds token g's (and g + 8's) columns 64 b + 16 t .. + 15 ----
    uint32_t xf[BPW][TT][8];
#pragma unroll
    for (int b = 0; b < BPW; ++b)
#pragma unroll
      for (int tt = 0; tt < TT; ++tt) {
        uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
        const int tok = tt * 8 + g;
        if (streaming && b < nb && tok < p.m) {
          const uint4* src = reinterpret_cast<const uint4*>(p.x + (long long)tok * p.w.k + (long long)(blk0 + b) * 64 + 16 * t);
          lo = __ldg(src);
          hi = __ldg(src + 1);
        }
        xf[b][tt][0] = lo.x; xf[b][tt][1] = lo.y; xf[b][tt][2] = lo.z; xf[b][tt][3] = lo.w;
        xf[b][tt][4] = hi.x; xf[b][tt][5] = hi.y; xf[b][tt][6] = hi.z; xf[b][tt][7] = hi.w;
      }
    __syncthreads();                                              // table (first pass) and staged absmax are in place
    if (pass == 0) GEMV_STAMP(1);
    if (!streaming) continue;

    const float* sp = scales_s + g * kGemvScaleStride + warp * BPW;   // row g of the first group of pair 0
    float4* mine = sums + (warp * kGemvMaxPairs * TT) * 32 + lane;
    for (int pr0 = 0; pr0 < npairs; pr0 += U) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int pr = pr0 + u;
        if (pr < npairs) {                                          // warp-uniform
          float acc[TT][4];
#pragma unroll
          for (int tt = 0; tt < TT; ++tt) {
            if (pass == 0) {
              acc[tt][0] = acc[tt][1] = acc[tt][2] = acc[tt][3] = 0.f;
            } else {
              const float4 v = mine[(pr * TT + tt) * 32];
              acc[tt][0] = v.x; acc[tt][1] = v.y; acc[tt][2] = v.z; acc[tt][3] = v.w;
            }
          }
          uint2 c0[BPW], c1[BPW];
#pragma unroll
          for (int b = 0; b < BPW; ++b) {
            c0[b] = q0[u * BPW + b];
            c1[b] = q1[u * BPW + b];
          }
          if (pr + U < npairs) request_pair(u, cp + (long long)(pr + U) * pair_stride, pr + U);   // refill, U pairs ahead
          const float* sp0 = sp + pr * 16 * kGemvScaleStride;
          const float* sp1 = sp0 + 8 * kGemvScaleStride;          // (an absent second group reads rows that are never stored)
#pragma unroll
          for (int b = 0; b < BPW; ++b) {
            const float sc0 = b < nb ? sp0[b] : 0.f, sc1 = b < nb ? sp1[b] : 0.f;
            // eight table lookups per row: bytes 2 s, 2 s + 1 of the lane's eight feed k-step s
            uint32_t a_lo[8], a_hi[8];
            a_lo[0] = lookup(c0[b].x, 0x5504); a_lo[1] = lookup(c0[b].x, 0x5514); a_lo[2] = lookup(c0[b].x, 0x5524); a_lo[3] = lookup(c0[b].x, 0x5534);
            a_lo[4] = lookup(c0[b].y, 0x5504); a_lo[5] = lookup(c0[b].y, 0x5514); a_lo[6] = lookup(c0[b].y, 0x5524); a_lo[7] = lookup(c0[b].y, 0x5534);
            a_hi[0] = lookup(c1[b].x, 0x5504); a_hi[1] = lookup(c1[b].x, 0x5514); a_hi[2] = lookup(c1[b].x, 0x5524); a_hi[3] = lookup(c1[b].x, 0x5534);
            a_hi[4] = lookup(c1[b].y, 0x5504); a_hi[5] = lookup(c1[b].y, 0x5514); a_hi[6] = lookup(c1[b].y, 0x5524); a_hi[7] = lookup(c1[b].y, 0x5534);
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) {
              float part[4];
              gemv_mma(part, a_lo[0], a_hi[0], a_lo[1], a_hi[1], xf[b][tt][0], xf[b][tt][1], zero);
#pragma unroll
              for (int s = 1; s < 4; ++s)
                gemv_mma(part, a_lo[2 * s], a_hi[2 * s], a_lo[2 * s + 1], a_hi[2 * s + 1], xf[b][tt][2 * s],
                         xf[b][tt][2 * s + 1], part);
              // accumulator rows: c0, c1 belong to weight row g of the first group, c2, c3 to row g of the second
              acc[tt][0] = fmaf(part[0], sc0, acc[tt][0]);
              acc[tt][1] = fmaf(part[1], sc0, acc[tt][1]);
              acc[tt][2] = fmaf(part[2], sc1, acc[tt][2]);
              acc[tt][3] = fmaf(part[3], sc1, acc[tt][3]);
            }
          }
#pragma unroll
          for (int tt = 0; tt < TT; ++tt)
            mine[(pr * TT + tt) * 32] = make_float4(acc[tt][0], acc[tt][1], acc[tt][2], acc[tt][3]);
        }
      }
    }
  }

  // the low-rank input comes from the companion kernel: wait for it only now
  GEMV_STAMP(2);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  GEMV_STAMP(3);
  for (int i = threadIdx.x; i < 16 * 64; i += kGemvWarps * 32) {
    float total = 0.f;
#pragma unroll
    for (int ks = 0; ks < kGemvLowrankSlices; ++ks) total += __ldcg(p.t + ks * 16 * 64 + i);   // fixed order
    t_s[i] = __bfloat162float(__float2bfloat16_rn(total));   // T is a bf16 tensor in the reference's dataflow
  }
  __syncthreads();   // all K-slice sums and the low-rank input are in shared memory
  GEMV_STAMP(4);

  // ---- one thread per (pair, token tile, lane slot): add the K-slices in warp order, the low-rank term, round ----
  const int active = p.nblk < p.warps * BPW ? (p.nblk + BPW - 1) / BPW : p.warps;   // warps that own at least one block
  for (int item = threadIdx.x; item < npairs * TT * 32; item += kGemvWarps * 32) {
    const int slot = item & 31, tt = (item >> 5) % TT, pr = (item >> 5) / TT;
    float4 sum = sums[((0 * kGemvMaxPairs + pr) * TT + tt) * 32 + slot];
    for (int wv = 1; wv < active; ++wv) {
      const float4 v = sums[((wv * kGemvMaxPairs + pr) * TT + tt) * 32 + slot];
      sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
    }
    const int sg = slot >> 2, st = slot & 3;
    const int tok0 = tt * 8 + 2 * st;
    const float base[2][2] = {{sum.x, sum.y}, {sum.z, sum.w}};   // [group of the pair][token]
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int grp = group0 + 2 * pr + half;
      if (grp >= group1) continue;
      const long long row = (long long)grp * 8 + sg;
      float lora[2] = {0.f, 0.f};
      const float* brow = p.lora_b + row * p.rank;
      if ((p.rank & 3) == 0 && (reinterpret_cast<uintptr_t>(brow) & 15) == 0) {
        for (int q0 = 0; 4 * q0 < p.rank; q0 += 4) {     // 16 adapter columns per round: four independent loads
          float4 bv[4];
#pragma unroll
          for (int q = 0; q < 4; ++q)
            bv[q] = 4 * (q0 + q) < p.rank ? __ldg(reinterpret_cast<const float4*>(brow) + q0 + q) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float bs[4] = {bv[q].x, bv[q].y, bv[q].z, bv[q].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int r = 4 * (q0 + q) + e;              // columns past the rank meet zeros in t_s and in bv
              const float v = __bfloat162float(__float2bfloat16_rn(p.scaling * bs[e]));
              lora[0] = fmaf(t_s[tok0 * 64 + r], v, lora[0]);
              lora[1] = fmaf(t_s[(tok0 + 1) * 64 + r], v, lora[1]);
            }
          }
        }
      } else {
        for (int r = 0; r < p.rank; ++r) {
          const float bs = __bfloat162float(__float2bfloat16_rn(p.scaling * __ldg(brow + r)));
          lora[0] = fmaf(t_s[tok0 * 64 + r], bs, lora[0]);
          lora[1] = fmaf(t_s[(tok0 + 1) * 64 + r], bs, lora[1]);
        }
      }
      if (tok0 < p.m) p.y[(long long)tok0 * p.w.n + row] = __float2bfloat16_rn(base[half][0] + lora[0]);
      if (tok0 + 1 < p.m) p.y[(long long)(tok0 + 1) * p.w.n + row] = __float2bfloat16_rn(base[half][1] + lora[1]);
    }
  }
  GEMV_STAMP(5);
}

// Low-rank input, first stage: part[ks][tok][r] = sum over the ks-th slice of K of x[tok][k] * bf16(A[r][k]) for tok < m,
// r < rank (zero elsewhere).  Grid (64 adapter rows, K slices): one short round of loads per CTA, so the kernel is over
// before the streaming kernel needs its result.  The slices are added in a fixed order by the reader (deterministic).
__global__ void __launch_bounds__(kGemvLowrankThreads) gemv_lowrank_kernel(const __nv_bfloat16* __restrict__ x,
                                                                           const float* __restrict__ a, int m, long long k,
                                                                           int rank, float* __restrict__ part
#ifdef MOLT_GEMV_TRACE
                                                                           , unsigned long long* trace
#endif
                                                                           ) {
  // the streaming kernel behind this one may start now; it waits for this grid only before it reads the result
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#ifdef MOLT_GEMV_TRACE
  if (trace != nullptr && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0)
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(trace[12]));
#endif
  __shared__ float red[kGemvLowrankThreads / 32][16];
  const int r = blockIdx.x, ks = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long slice = (k / 8 + kGemvLowrankSlices - 1) / kGemvLowrankSlices * 8;   // columns per slice, multiple of 8
  const long long c_begin = ks * slice, c_end = c_begin + slice < k ? c_begin + slice : k;
  float sums[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) sums[i] = 0.f;
  if (r < rank) {
    for (long long c = c_begin + threadIdx.x * 8LL; c < c_end; c += kGemvLowrankThreads * 8) {
      const float4 a0 = __ldg(reinterpret_cast<const float4*>(a + r * k + c));
      const float4 a1 = __ldg(reinterpret_cast<const float4*>(a + r * k + c + 4));
      uint4 xv[16];
#pragma unroll
      for (int tok = 0; tok < 16; ++tok)
        xv[tok] = tok < m ? __ldg(reinterpret_cast<const uint4*>(x + (long long)tok * k + c)) : make_uint4(0, 0, 0, 0);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      float ab[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) ab[j] = __bfloat162float(__float2bfloat16_rn(av[j]));
#pragma unroll
      for (int tok = 0; tok < 16; ++tok) {
        const uint32_t xw[4] = {xv[tok].x, xv[tok].y, xv[tok].z, xv[tok].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          sums[tok] = fmaf(bf16_lo(xw[j]), ab[2 * j], sums[tok]);
          sums[tok] = fmaf(bf16_hi(xw[j]), ab[2 * j + 1], sums[tok]);
        }
      }
    }
  }
#pragma unroll
  for (int tok = 0; tok < 16; ++tok) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sums[tok] += __shfl_xor_sync(0xffffffffu, sums[tok], o);
    if (lane == 0) red[warp][tok] = sums[tok];
  }
  __syncthreads();
  if (threadIdx.x < 16) {
    const int tok = threadIdx.x;
    float total = 0.f;
#pragma unroll
    for (int wv = 0; wv < kGemvLowrankThreads / 32; ++wv) total += red[wv][tok];
    part[(ks * 16 + tok) * 64 + r] = (r < rank && tok < m) ? total : 0.f;
  }
#ifdef MOLT_GEMV_TRACE
  if (trace != nullptr && threadIdx.x == 0 && blockIdx.x == gridDim.x - 1 && blockIdx.y == gridDim.y - 1)
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(trace[13]));
#endif
}

// Second stage for callers that want the low-rank input itself: t_out[tok][0..64) = bf16(sum of the slices), zero padded.
__global__ void gemv_lowrank_finish_kernel(const float* __restrict__ part, int m, __nv_bfloat16* __restrict__ t_out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= m * 64) return;
  float total = 0.f;
#pragma unroll
  for (int ks = 0; ks < kGemvLowrankSlices; ++ks) total += part[ks * 16 * 64 + i];
  t_out[i] = __float2bfloat16_rn(total);
}

namespace {

struct GemvPlan {
  int nblk, cta_warps, warps, bpw, passes, ctas, tt;
  size_t smem_bytes;
};

// K-slices: `warps` warps x `bpw` blocks per pass; chosen to waste as few warp-passes as possible.
GemvPlan gemv_plan(long long n, long long k, int m) {
  GemvPlan g;
  g.nblk = (int)(k / 64);
  g.tt = m > 8 ? 2 : 1;
#ifdef MOLT_GEMV_WIDE
  g.cta_warps = g.tt == 1 ? 32 : 16;
  const int max_bpw = 2;
#else
  g.cta_warps = 16;
  const int max_bpw = g.tt == 1 ? 4 : 2;   // X fragments in registers: 8 per block and token tile
#endif
  long long best_cost = -1;
  g.warps = g.cta_warps; g.bpw = 1; g.passes = (g.nblk + g.cta_warps - 1) / g.cta_warps;
  for (int bpw = 1; bpw <= max_bpw; ++bpw)
    for (int warps = g.cta_warps; warps >= g.cta_warps / 2; --warps) {
      const int per_pass = warps * bpw;
      if (per_pass > 64) continue;
      const int passes = (g.nblk + per_pass - 1) / per_pass;
      // time ~ passes x bpw tile-rows per warp, plus a fixed cost per pass (X fragments, staging) and idle warps
      const long long cost = (long long)passes * bpw * 16 * (32 / g.cta_warps) + passes * 6 + (g.cta_warps - warps);
      if (best_cost < 0 || cost < best_cost) {
        best_cost = cost;
        g.warps = warps; g.bpw = bpw; g.passes = passes;
      }
    }
  const long long groups = n / 8;
  const int sms = sm_count();
  const long long per_wave = (long long)sms * 2 * kGemvMaxPairs;   // row groups one wave of CTAs can hold
  const long long waves = (groups + per_wave - 1) / per_wave;
  long long ctas = waves * sms;
  if (ctas > groups) ctas = groups;
  g.ctas = (int)ctas;
  g.smem_bytes = gemv_smem_bytes(g.cta_warps, g.tt);
  return g;
}

}  // namespace

// The kernel resolves a nested absmax itself (per CTA, into shared memory) when the second-level block size is a power
// of two; otherwise the caller resolves the absmax to fp32 first.
bool gemv_reads_nested(const WeightView& w) { return w.block2_shift >= 0; }

// Workspace layout: [slices][16][64] fp32 parts of the low-rank input | n * k / 64 fp32 resolved absmax (used by the caller for nested forms
// the kernel cannot read), each region starting on a 256-byte boundary.
static size_t gemv_resolved_offset() { return (size_t)kGemvLowrankSlices * 16 * 64 * sizeof(float); }

size_t gemv_workspace_bytes(long long n, long long k) {
  return gemv_resolved_offset() + (size_t)n * (k / 64) * sizeof(float) + 256;
}

float* gemv_resolved_absmax_slot(void* workspace, long long, long long) {
  return reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + gemv_resolved_offset());
}

template <int WARPS, int BPW, int TT>
static int gemv_launch(const GemvParams& p, const GemvPlan& g, cudaStream_t s) {
  static thread_local bool configured[64] = {};
  int dev = 0;
  MOLT_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    MOLT_CUDA(cudaFuncSetAttribute(nf4_gemv_kernel<WARPS, BPW, TT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)gemv_smem_bytes(WARPS, TT)));
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)g.ctas);
  cfg.blockDim = dim3(WARPS * 32);
  cfg.dynamicSmemBytes = g.smem_bytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  MOLT_CUDA(cudaLaunchKernelEx(&cfg, nf4_gemv_kernel<WARPS, BPW, TT>, p));
  return launch_status("nf4_gemv_kernel");
}

int gemv_forward(const WeightView& w, const __nv_bfloat16* x, const float* lora_a, const float* lora_b, float scaling,
                 int rank, __nv_bfloat16* y, int m, __nv_bfloat16* t_out, void* workspace, size_t workspace_bytes,
                 cudaStream_t s) {
  if (workspace_bytes < gemv_resolved_offset())
    return fail(MOLT_E_VALUE, "molt_nf4_gemv: workspace too small (%zu < %zu bytes)", workspace_bytes,
                gemv_resolved_offset());
  const bool nested = w.absmax_kind == MOLT_ABSMAX_NESTED;
  if (nested && !gemv_reads_nested(w))
    return fail(MOLT_E_RUNTIME, "molt_nf4_gemv: this nested absmax layout must be resolved to fp32 before the call");
  if ((reinterpret_cast<uintptr_t>(w.packed) & 15) != 0 || (reinterpret_cast<uintptr_t>(lora_a) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(x) & 15) != 0)
    return fail(MOLT_E_CAPABILITY, "molt_nf4_gemv: the packed weight, lora_a and x must start on 16-byte boundaries");
  if (m < 1 || m > 16) return fail(MOLT_E_CAPABILITY, "molt_nf4_gemv: 1 to 16 tokens");
  const GemvPlan g = gemv_plan(w.n, w.k, m);
  GemvParams p;
  p.w = w;
  p.x = x;
  p.lora_b = lora_b;
  p.t = reinterpret_cast<const float*>(workspace);
  p.y = y;
  p.scaling = scaling;
  p.rank = rank;
  p.m = m;
  p.nblk = g.nblk;
  p.warps = g.warps;
  p.passes = g.passes;
  p.groups_total = (int)(w.n / 8);
  p.ctas = g.ctas;
#ifdef MOLT_GEMV_TRACE
  {
    const char* tr = getenv("MOLT_B200_TRACE_PTR");   // device pointer (decimal) of a trace buffer of 16 x 8 bytes
    if (tr == nullptr) return fail(MOLT_E_VALUE, "trace build: MOLT_B200_TRACE_PTR is not set");
    p.trace = reinterpret_cast<unsigned long long*>(strtoull(tr, nullptr, 10));
  }
#endif
  gemv_lowrank_kernel<<<dim3(64, kGemvLowrankSlices), kGemvLowrankThreads, 0, s>>>(x, lora_a, m, w.k, rank,
                                                                                    reinterpret_cast<float*>(workspace)
#ifdef MOLT_GEMV_TRACE
                                                                                    , p.trace
#endif
                                                                                    );
  if (int rc = launch_status("gemv_lowrank_kernel")) return rc;
  int rc = MOLT_E_RUNTIME;
  bool found = false;
#define MOLT_GEMV_CASE(WP, BP, T)                                            \
  if (!found && g.cta_warps == WP && g.bpw == BP && g.tt == T) {             \
    found = true;                                                            \
    rc = gemv_launch<WP, BP, T>(p, g, s);                                    \
  }
#ifdef MOLT_GEMV_WIDE
  MOLT_GEMV_CASE(32, 1, 1); MOLT_GEMV_CASE(32, 2, 1);
#else
  MOLT_GEMV_CASE(16, 1, 1); MOLT_GEMV_CASE(16, 2, 1); MOLT_GEMV_CASE(16, 3, 1); MOLT_GEMV_CASE(16, 4, 1);
#endif
  MOLT_GEMV_CASE(16, 1, 2); MOLT_GEMV_CASE(16, 2, 2);
#undef MOLT_GEMV_CASE
  if (!found) return fail(MOLT_E_RUNTIME, "molt_nf4_gemv: no kernel for this plan");
  if (rc != MOLT_OK) return rc;
  if (t_out != nullptr) {   // behind the streaming kernel, so that kernel stays the programmatic dependent of the first stage
    gemv_lowrank_finish_kernel<<<(m * 64 + 255) / 256, 256, 0, s>>>(reinterpret_cast<const float*>(workspace), m, t_out);
    return launch_status("gemv_lowrank_finish_kernel");
  }
  return MOLT_OK;
}

}  // namespace molt
