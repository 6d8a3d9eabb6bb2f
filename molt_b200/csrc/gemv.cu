// Small-token (M <= 16) NF4 + LoRA forward: y = x . deq(W)^T + s (x A^T) B^T with the packed weight streamed from
// HBM exactly once, straight into registers.
//
// One kernel does the whole product.  A CTA owns a contiguous range of 8-row groups of W with their FULL rows, so
// nothing leaves the SM as a partial sum.  Inside the CTA the warps split the contraction: a warp owns a K-slice of
// up to four absmax blocks (64 columns each) per pass, keeps the matching X fragments in registers, and walks over
// the CTA's row groups two at a time (16 weight rows = the M dimension of mma.sync m16n8k16; the tokens are the N
// dimension, eight per MMA).  Per 16 x 64 tile a lane issues two 8-byte loads of packed codes (the four lanes of a
// quad cover the 32 contiguous bytes of one row's block, so every 32-byte sector fetched is used in full) a few
// tiles ahead of their use, expands every byte into a bf16 pair of codebook values with one byte-permute (table
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
#include "internal.h"

namespace molt {

constexpr int kGemvWarps = 16;
constexpr int kGemvMaxPairs = 7;            // row-group pairs (16 weight rows) per CTA whose sums stay in registers
constexpr int kGemvLutStride = 256;         // bytes per table entry: 32 lanes x 4 bytes used, so that (byte << 8) | (lane * 4)
constexpr int kGemvLutBytes = 256 * kGemvLutStride;   // is the offset and one byte-permute builds it

struct GemvParams {
  WeightView w;
  const __nv_bfloat16* x;    // [m, k]
  const float* lora_b;       // [n, rank] fp32
  const float* t;            // [16][64] fp32: x . A^T rounded to bf16 values (written by the companion kernel)
  __nv_bfloat16* y;          // [m, n]
  float scaling;
  int rank;
  int m;
  int nblk;                  // k / 64
  int warps;                 // streaming warps that own a K-slice (<= kGemvWarps)
  int passes;                // K passes: pass p covers blocks [p * warps * BPW, (p + 1) * warps * BPW)
  int groups_total;          // n / 8
  int ctas;
};

__device__ __forceinline__ void gemv_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1, const float (&c)[4]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

__device__ __forceinline__ uint2 ldg_stream8(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

// Ring of tiles in flight per warp: R = BPW * U tiles (U row-group pairs), refilled as tiles are consumed.
constexpr int gemv_unroll_pairs(int bpw) { return bpw == 1 ? 4 : bpw == 2 ? 2 : 1; }

// BPW: absmax blocks per warp per pass.  TT: token tiles of eight (1 for m <= 8, 2 for m <= 16).
template <bool NESTED, int BPW, int TT>
__global__ void __launch_bounds__(kGemvWarps * 32, 1) nf4_gemv_kernel(const __grid_constant__ GemvParams p) {
  constexpr int U = gemv_unroll_pairs(BPW);
  constexpr int R = BPW * U;
  extern __shared__ __align__(256) unsigned char smem_raw[];
  unsigned char* lut_bytes = smem_raw;                                          // [256 entries][256 bytes]
  float4* sums = reinterpret_cast<float4*>(smem_raw + kGemvLutBytes);           // [warp][pair][tt][lane]
  __shared__ float code2_s[NESTED ? 256 : 1];
  __shared__ float t_s[16 * 64];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

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
  if (NESTED)
    for (int i = threadIdx.x; i < 256; i += kGemvWarps * 32) code2_s[i] = p.w.code2[i];
  __syncthreads();

  const uint32_t lane4 = (uint32_t)lane * 4u;
  auto lookup = [&](uint32_t q, uint32_t selector) -> uint32_t {   // table entry of one code byte of q
    return *reinterpret_cast<const uint32_t*>(lut_bytes + __byte_perm(q, lane4, selector));
  };
  const float zero[4] = {0.f, 0.f, 0.f, 0.f};

  if (warp < p.warps) {
    for (int pass = 0; pass < p.passes; ++pass) {
      const int blk0 = (pass * p.warps + warp) * BPW;         // first absmax block of this warp's K-slice
      int nb = p.nblk - blk0;
      if (nb > BPW) nb = BPW;
      if (nb <= 0) continue;                                  // (its sums from earlier passes stay as they are)
      // ---- X fragments of the K-slice: lane (g, t) holds token g's (and g + 8's) columns 64 b + 16 t .. + 15 ----
      // A missing block (b >= nb) keeps zero fragments; its codes are read from block blk0 instead.
      uint32_t xf[BPW][TT][8];
#pragma unroll
      for (int b = 0; b < BPW; ++b)
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
          uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
          const int tok = tt * 8 + g;
          if (b < nb && tok < p.m) {
            const uint4* src = reinterpret_cast<const uint4*>(p.x + (long long)tok * p.w.k + (long long)(blk0 + b) * 64 + 16 * t);
            lo = __ldg(src);
            hi = __ldg(src + 1);
          }
          xf[b][tt][0] = lo.x; xf[b][tt][1] = lo.y; xf[b][tt][2] = lo.z; xf[b][tt][3] = lo.w;
          xf[b][tt][4] = hi.x; xf[b][tt][5] = hi.y; xf[b][tt][6] = hi.z; xf[b][tt][7] = hi.w;
        }
      // ---- the ring of tiles in flight: codes of rows g (first group of the pair) and g (second group), and the
      // two absmax values (nested form: the 8-bit code and its second-level absmax), R tiles ahead of their use ----
      const uint8_t* code_base = p.w.packed + ((long long)group0 * 8 + g) * row_bytes + (long long)blk0 * 32 + 8 * t;
      const long long scale_base = ((long long)group0 * 8 + g) * p.nblk + blk0;
      uint2 q0[R], q1[R];
      float s0[R], s1[R];
      uint32_t n0[NESTED ? R : 1], n1[NESTED ? R : 1];   // nested: raw 8-bit codes (s0/s1 then hold the second level)
      auto request = [&](int slot, int pr, int b) {
        if (pr >= npairs) pr = npairs - 1;                     // past the end: re-read the last tile (never used)
        const int bb = b < nb ? b : 0;
        const long long second_group = (2 * pr + 1 < ngroups) ? 8 : 0;   // odd group count: the last pair reads its first group twice
        const uint8_t* src = code_base + (long long)pr * 16 * row_bytes + bb * 32;
        q0[slot] = ldg_stream8(src);
        q1[slot] = ldg_stream8(src + second_group * row_bytes);
        const long long blk = scale_base + (long long)pr * 16 * p.nblk + bb;
        const long long blk_second = blk + second_group * p.nblk;
        if (!NESTED) {
          s0[slot] = __ldg(reinterpret_cast<const float*>(p.w.absmax) + blk);
          s1[slot] = __ldg(reinterpret_cast<const float*>(p.w.absmax) + blk_second);
        } else {
          n0[NESTED ? slot : 0] = __ldg(reinterpret_cast<const uint8_t*>(p.w.absmax) + blk);
          n1[NESTED ? slot : 0] = __ldg(reinterpret_cast<const uint8_t*>(p.w.absmax) + blk_second);
          s0[slot] = __ldg(p.w.absmax2 + (blk >> p.w.block2_shift));
          s1[slot] = __ldg(p.w.absmax2 + (blk_second >> p.w.block2_shift));
        }
      };
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int b = 0; b < BPW; ++b) request(u * BPW + b, u, b);

      for (int pr0 = 0; pr0 < npairs; pr0 += U) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int pr = pr0 + u;
          if (pr < npairs) {                                   // warp-uniform
            float acc[TT][4];
            float4* mine = sums + ((warp * kGemvMaxPairs + pr) * TT) * 32 + lane;
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) {
              if (pass == 0) {
                acc[tt][0] = acc[tt][1] = acc[tt][2] = acc[tt][3] = 0.f;
              } else {
                const float4 v = mine[tt * 32];
                acc[tt][0] = v.x; acc[tt][1] = v.y; acc[tt][2] = v.z; acc[tt][3] = v.w;
              }
            }
#pragma unroll
            for (int b = 0; b < BPW; ++b) {
              constexpr int kNone = 0;
              const int slot = u * BPW + b;                      // compile-time
              const uint2 c0 = q0[slot], c1 = q1[slot];
              float sc0, sc1;
              if (!NESTED) {
                sc0 = s0[slot];
                sc1 = s1[slot];
              } else {
                // code2[u8] * absmax2 + offset with a separate multiply and add: the dequantiser's bits
                sc0 = __fadd_rn(__fmul_rn(code2_s[n0[NESTED ? slot : kNone]], s0[slot]), p.w.offset);
                sc1 = __fadd_rn(__fmul_rn(code2_s[n1[NESTED ? slot : kNone]], s1[slot]), p.w.offset);
              }
              if (b >= nb) sc0 = sc1 = 0.f;
              request(slot, pr + U, b);                          // refill the slot, U pairs ahead
              // eight table lookups per row: bytes 2 s, 2 s + 1 of the lane's eight feed k-step s
              uint32_t a_lo[8], a_hi[8];
              a_lo[0] = lookup(c0.x, 0x5504); a_lo[1] = lookup(c0.x, 0x5514); a_lo[2] = lookup(c0.x, 0x5524); a_lo[3] = lookup(c0.x, 0x5534);
              a_lo[4] = lookup(c0.y, 0x5504); a_lo[5] = lookup(c0.y, 0x5514); a_lo[6] = lookup(c0.y, 0x5524); a_lo[7] = lookup(c0.y, 0x5534);
              a_hi[0] = lookup(c1.x, 0x5504); a_hi[1] = lookup(c1.x, 0x5514); a_hi[2] = lookup(c1.x, 0x5524); a_hi[3] = lookup(c1.x, 0x5534);
              a_hi[4] = lookup(c1.y, 0x5504); a_hi[5] = lookup(c1.y, 0x5514); a_hi[6] = lookup(c1.y, 0x5524); a_hi[7] = lookup(c1.y, 0x5534);
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
            for (int tt = 0; tt < TT; ++tt) mine[tt * 32] = make_float4(acc[tt][0], acc[tt][1], acc[tt][2], acc[tt][3]);
          }
        }
      }
    }
  }

  // the low-rank input comes from the companion kernel: wait for it only now
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int i = threadIdx.x; i < 16 * 64; i += kGemvWarps * 32) t_s[i] = __ldcg(p.t + i);
  __syncthreads();   // all K-slice sums and the low-rank input are in shared memory

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
      for (int r = 0; r < p.rank; ++r) {
        const float bs = __bfloat162float(__float2bfloat16_rn(p.scaling * __ldg(p.lora_b + row * p.rank + r)));
        lora[0] = fmaf(t_s[tok0 * 64 + r], bs, lora[0]);
        lora[1] = fmaf(t_s[(tok0 + 1) * 64 + r], bs, lora[1]);
      }
      if (tok0 < p.m) p.y[(long long)tok0 * p.w.n + row] = __float2bfloat16_rn(base[half][0] + lora[0]);
      if (tok0 + 1 < p.m) p.y[(long long)(tok0 + 1) * p.w.n + row] = __float2bfloat16_rn(base[half][1] + lora[1]);
    }
  }
}

// T[tok][r] = bf16(sum_k x[tok][k] * bf16(A[r][k])) for tok < m, r < rank, as fp32 values in t [16][64] (zero elsewhere)
// and, when t_out is given, as bf16 in t_out [m][64].  One CTA per adapter row.
__global__ void __launch_bounds__(256) gemv_lowrank_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ a,
                                                           int m, long long k, int rank, float* __restrict__ t,
                                                           __nv_bfloat16* __restrict__ t_out) {
  // the streaming kernel behind this one may start now; it waits for this grid only before it reads t
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ float red[8][16];
  const int r = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float sums[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) sums[i] = 0.f;
  if (r < rank) {
    for (long long c = threadIdx.x * 8LL; c < k; c += 256 * 8) {
      const float4 a0 = __ldg(reinterpret_cast<const float4*>(a + r * k + c));
      const float4 a1 = __ldg(reinterpret_cast<const float4*>(a + r * k + c + 4));
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      float ab[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) ab[j] = __bfloat162float(__float2bfloat16_rn(av[j]));
#pragma unroll
      for (int tok = 0; tok < 16; ++tok) {
        if (tok < m) {
          const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x + (long long)tok * k + c));
          const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            sums[tok] = fmaf(bf16_lo(xw[j]), ab[2 * j], sums[tok]);
            sums[tok] = fmaf(bf16_hi(xw[j]), ab[2 * j + 1], sums[tok]);
          }
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
    for (int wv = 0; wv < 8; ++wv) total += red[wv][tok];
    const __nv_bfloat16 rounded = __float2bfloat16_rn((r < rank && tok < m) ? total : 0.f);
    t[tok * 64 + r] = __bfloat162float(rounded);
    if (t_out != nullptr && tok < m) t_out[(long long)tok * 64 + r] = rounded;
  }
}

namespace {

struct GemvPlan {
  int nblk, warps, bpw, passes, ctas, tt;
  size_t smem_bytes;
};

// K-slices: `warps` warps x `bpw` blocks per pass; chosen to waste as few warp-passes as possible.
GemvPlan gemv_plan(long long n, long long k, int m) {
  GemvPlan g;
  g.nblk = (int)(k / 64);
  g.tt = m > 8 ? 2 : 1;
  const int max_bpw = g.tt == 2 ? 2 : 4;   // X fragments in registers: 8 per block and token tile
  long long best_cost = -1;
  g.warps = kGemvWarps; g.bpw = 1; g.passes = g.nblk;
  for (int bpw = 1; bpw <= max_bpw; ++bpw)
    for (int warps = kGemvWarps; warps >= 8; --warps) {
      const int per_pass = warps * bpw;
      const int passes = (g.nblk + per_pass - 1) / per_pass;
      // time ~ passes x bpw tile-rows per warp, plus a fixed cost per pass (X fragments) and idle warps
      const long long cost = (long long)passes * bpw * 16 + passes * 4 + (kGemvWarps - warps);
      if (best_cost < 0 || cost < best_cost) {
        best_cost = cost;
        g.warps = warps; g.bpw = bpw; g.passes = passes;
      }
    }
  const long long groups = n / 8;
  const int sms = sm_count();
  const long long per_wave = (long long)sms * 2 * kGemvMaxPairs;   // row groups one wave of CTAs can hold in registers
  const long long waves = (groups + per_wave - 1) / per_wave;
  long long ctas = waves * sms;
  if (ctas > groups) ctas = groups;
  g.ctas = (int)ctas;
  g.smem_bytes = (size_t)kGemvLutBytes + (size_t)kGemvWarps * kGemvMaxPairs * g.tt * 32 * sizeof(float4);
  return g;
}

}  // namespace

// The kernel reads a nested absmax itself when the second-level block size is a power of two and rows hold whole
// second-level... (a K-slice never crosses a row, and rows of k / 64 codes must not straddle a second-level block inside
// a slice: guaranteed when block2 is a multiple of the slice or k / 64 divides block2).  Otherwise the caller resolves
// the absmax to fp32 first.
bool gemv_reads_nested(const WeightView& w) {
  if (w.block2_shift < 0) return false;
  const long long nblk = w.k / 64;
  return nblk > 0 && (w.block2 % nblk == 0 || nblk % w.block2 == 0) && (w.block2 % 4 == 0);
}

// Workspace layout: [16][64] fp32 low-rank input | n * k / 64 fp32 resolved absmax (used by the caller for nested forms
// the kernel cannot read), each region starting on a 256-byte boundary.
static size_t gemv_resolved_offset() { return 16 * 64 * sizeof(float); }

size_t gemv_workspace_bytes(long long n, long long k) {
  return gemv_resolved_offset() + (size_t)n * (k / 64) * sizeof(float) + 256;
}

float* gemv_resolved_absmax_slot(void* workspace, long long, long long) {
  return reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + gemv_resolved_offset());
}

template <bool NESTED, int BPW, int TT>
static int gemv_launch(const GemvParams& p, const GemvPlan& g, cudaStream_t s) {
  static thread_local bool configured[64] = {};
  int dev = 0;
  MOLT_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    MOLT_CUDA(cudaFuncSetAttribute(nf4_gemv_kernel<NESTED, BPW, TT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)(kGemvLutBytes + kGemvWarps * kGemvMaxPairs * TT * 32 * sizeof(float4))));
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)g.ctas);
  cfg.blockDim = dim3(kGemvWarps * 32);
  cfg.dynamicSmemBytes = g.smem_bytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  MOLT_CUDA(cudaLaunchKernelEx(&cfg, nf4_gemv_kernel<NESTED, BPW, TT>, p));
  return launch_status("nf4_gemv_kernel");
}

int gemv_forward(const WeightView& w, const __nv_bfloat16* x, const float* lora_a, const float* lora_b, float scaling,
                 int rank, __nv_bfloat16* y, int m, __nv_bfloat16* t_out, void* workspace, size_t workspace_bytes,
                 cudaStream_t s) {
  if (workspace_bytes < 16 * 64 * sizeof(float))
    return fail(MOLT_E_VALUE, "molt_nf4_gemv: workspace too small (%zu < %zu bytes)", workspace_bytes,
                16 * 64 * sizeof(float));
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
  gemv_lowrank_kernel<<<64, 256, 0, s>>>(x, lora_a, m, w.k, rank, reinterpret_cast<float*>(workspace), t_out);
  if (int rc = launch_status("gemv_lowrank_kernel")) return rc;
#define MOLT_GEMV_CASE(NE, BP, T)                                            \
  if (nested == NE && g.bpw == BP && g.tt == T) return gemv_launch<NE, BP, T>(p, g, s)
  MOLT_GEMV_CASE(false, 1, 1); MOLT_GEMV_CASE(false, 2, 1); MOLT_GEMV_CASE(false, 3, 1); MOLT_GEMV_CASE(false, 4, 1);
  MOLT_GEMV_CASE(false, 1, 2); MOLT_GEMV_CASE(false, 2, 2);
  MOLT_GEMV_CASE(true, 1, 1); MOLT_GEMV_CASE(true, 2, 1); MOLT_GEMV_CASE(true, 3, 1); MOLT_GEMV_CASE(true, 4, 1);
  MOLT_GEMV_CASE(true, 1, 2); MOLT_GEMV_CASE(true, 2, 2);
#undef MOLT_GEMV_CASE
  return fail(MOLT_E_RUNTIME, "molt_nf4_gemv: no kernel for this plan");
}

}  // namespace molt
