// CTA-pair (cta_group::2) tcgen05 GEMM with the NF4 decode fused in front of the tensor core.
//
//   forward : out[m, n] = in[m, k] . deq(W)[n, k]^T + low[m, r] . ext[n, r]^T        contraction over k
//   backward: out[m, k] = in[m, n] . deq(W)[n, k]   + low[m, r] . ext[r, k]          contraction over n
//
// Two CTAs on neighbouring SMs form a cluster and share one UMMA of shape 256 x 256 x 16: each CTA owns 128 token
// rows (its A operand and its 128 x 256 fp32 accumulator in TMEM) and supplies one half of the B operand, i.e. it
// decodes only 128 weight segments per 64-wide contraction block while the tensor cores of both SMs consume the
// whole 256-wide tile.  Compared with a single-CTA tile this halves the decode work and the shared-memory operand
// traffic per FLOP.
//
// Per CTA: two TMA rings (16 KB activation tiles; 4 KB packed-code tiles, deeper) run several blocks ahead of a
// separate ring of decoded B half-tiles, so the global-memory latency is not serialised with the decode.
// Decode: one 8-byte shared-memory lookup per packed byte returns both fp32 codebook values (table replicated
// per bank pair, conflict free), multiplied by the fp32 absmax and rounded once to bf16 -- the bits of the
// standalone dequantiser.  The leader CTA's MMA warp issues the pair MMA and signals both CTAs with
// tcgen05.commit; decoders and epilogue warps of the second CTA signal the leader with remote mbarrier arrives.
// All waits are bounded (status word + clean exit), and TMEM is released after a cluster barrier.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <stdlib.h>

#include "internal.h"
#include "sm100_ptx.cuh"

namespace molt {
namespace pair {

constexpr int BM = 128;            // token rows per CTA (256 per pair)
constexpr int BN = 256;            // output columns per pair tile
constexpr int BNH = 128;           // B rows decoded per CTA
constexpr int BK = 64;
constexpr int kEpilogueWarps = 4;
// Decode groups: groups of four warps that take the contraction blocks in turn.  Measured on the 14336 x 4096 weight at
// 4096 tokens with the (6, 3) rings, same box, forward / backward: 2 groups 451-457 / 439-444 us, 3 groups 478-482 /
// 459-471 us, 4 groups 476 / 479-485 us.  Two groups also leave 128 registers per thread (no spills).
constexpr int decode_groups(bool) { return 2; }
constexpr int kProducerWarp = 4;
constexpr int kMmaWarp = 5;
constexpr int kFirstDecodeWarp = 6;
constexpr int pair_threads(int groups) { return (kFirstDecodeWarp + 4 * groups) * 32; }

constexpr uint32_t kTileABytes = BM * BK * 2;          // 16384
constexpr uint32_t kPackedBytes = BNH * BK / 2;        // 4096
constexpr uint32_t kLoadStageBytes = kTileABytes;      // activation ring stage
constexpr int kCodeStages = 8;                         // ring of packed-code tiles; runs further ahead than the activations
constexpr uint32_t kTileBBytes = BNH * BK * 2;         // 16384
constexpr uint32_t kStoreBytes = BM * 64 * 2;          // 16384
constexpr uint32_t kLutBytes = 256 * 16 * 8;           // 32768: [byte][16 copies] of float2
constexpr uint32_t smem_bytes(int load_stages, int b_stages, int store_bufs) {
  return load_stages * kLoadStageBytes + kCodeStages * kPackedBytes + b_stages * kTileBBytes +
         store_bufs * kStoreBytes + kLutBytes + 512 /*barriers*/ + 1024 /*alignment*/;
}

struct Params {
  const uint8_t* packed; // [n, k / 2] packed codes
  const float* absmax;   // fp32 [n * k / 64]
  int32_t* status;
  long long m, n, k;
  int num_kb;
  int ext_steps;         // rp / 16, 0 = no low-rank block
  int tiles_m, tiles_n;  // pair tiles: 256 tokens x 256 columns
  int full_tiles;        // tiles on the static schedule (whole waves); the tiles after them are split along the contraction
  float* split_partial;  // [pairs][2 parts][2 CTAs][128 rows][256 columns] fp32 partial accumulators of the split tiles
  int nibble_high_first;
  unsigned long long* trace;   // optional [2 CTAs][4 roles][256 events] timestamps (ns) for pipeline analysis
  int debug;             // timing experiments only: 1 = skip decode, 2 = skip MMA issue, 4 = skip epilogue stores,
                         // 16 = skip writing split partials
  float codebook[16];
};

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// role: 0 producer (TMA issued), 1 MMA (issued), 2 decoder warp 0 (waits done), 3 decoder warp 0 (arrived)
#define MOLT_TRACE(role, index)                                                                       \
  do {                                                                                                \
    if (p.trace != nullptr && blockIdx.x < 2 && (index) < 256)                                        \
      p.trace[(blockIdx.x * 4 + (role)) * 256 + (index)] = global_ns();                               \
  } while (0)

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(local_smem_addr), "r"(rank));
  return out;
}
// Remote arrive with the default (CTA-scope release) semantics.  A cluster-scope release here was measured to
// cost several hundred nanoseconds per arrive; the data handed over is made visible to its only reader, the
// tensor core, by the fence.proxy.async each writer executes before arriving.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Barriers completed from the other CTA (remote arrives, tcgen05.commit of the leader) are waited on with the
// ordinary CTA-scope try_wait.
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  int32_t* status, int where) {
  return mbar_wait(bar, parity, abort_flag, status, where);
}
__device__ __forceinline__ uint64_t desc64(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on one mbarrier (given by its shared::cluster address) when all MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_bar_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar_addr)
               : "memory");
}
// One commit that arrives on the barrier at the same shared-memory offset in both CTAs of the pair (a
// tcgen05.commit multicast: it signals barriers only, it does not move data).
__device__ __forceinline__ void umma_commit_both(uint32_t local_bar_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(local_bar_addr), "h"((unsigned short)3)
               : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int kBand = 8;  // 8 pair tiles = 2048 tokens share the L2 while the weight columns stream by
  const int band_tiles = kBand * tiles_n;
  const int band = tile / band_tiles;
  const int first_m = band * kBand;
  int rows = tiles_m - first_m;
  if (rows > kBand) rows = kBand;
  const int inside = tile - band * band_tiles;
  tn = inside / rows;
  tm = first_m + inside % rows;
}

// Work of one CTA pair.  Whole waves of tiles follow the static schedule (tile = pair, pair + pairs, ...).  The tiles
// of the last, partial wave are cut along the contraction instead: their blocks, laid end to end, are dealt out in
// equal contiguous ranges, so every pair gets at most the tail of one tile and the head of the next.  Every part of
// a split tile leaves the kernel as an fp32 partial accumulator in global memory; a small second kernel adds the
// parts of each tile in pair order (deterministic) and writes the bf16 output.  Nothing inside the GEMM kernel waits
// for another pair.
struct WorkPlan {
  int num_pairs, pair_id, blocks;   // blocks per tile, the low-rank block included
  int full_tiles, num_tiles;
  int tail_units;                   // blocks of all split tiles (at most pairs x blocks: fits easily)
  int tail_begin, tail_end;         // this pair's range of them
};
struct WorkItem {
  int tile, kb0, kb1;
  int u;                            // position in the tail (split tiles only)
  bool valid;
};
__host__ __device__ __forceinline__ int tail_range_begin(const WorkPlan& w, int pair) {
  return w.tail_units * pair / w.num_pairs;   // at most pairs^2 x blocks < 2^31 (the host checks)
}
__device__ __forceinline__ void tail_item(const WorkPlan& w, WorkItem& it) {
  if (it.u >= w.tail_end) {
    it.valid = false;
    return;
  }
  it.tile = w.full_tiles + it.u / w.blocks;
  it.kb0 = it.u % w.blocks;
  const int left = w.tail_end - it.u;
  it.kb1 = left < w.blocks - it.kb0 ? it.kb0 + left : w.blocks;
  it.valid = true;
}
__device__ __forceinline__ WorkItem first_item(const WorkPlan& w) {
  WorkItem it;
  it.tile = w.pair_id;
  it.kb0 = 0;
  it.kb1 = w.blocks;
  it.u = w.tail_begin;
  it.valid = true;
  if (it.tile >= w.full_tiles) tail_item(w, it);
  return it;
}
__device__ __forceinline__ void next_item(const WorkPlan& w, WorkItem& it) {
  if (it.tile < w.full_tiles) {
    it.tile += w.num_pairs;
    if (it.tile < w.full_tiles) return;
    it.u = w.tail_begin;
  } else {
    it.u += it.kb1 - it.kb0;
  }
  tail_item(w, it);
}
// Slot of a pair's partial accumulator: two per pair, [0] for the part that ends a tile, [1] for the part that starts one.
__host__ __device__ __forceinline__ size_t split_slot_offset(int pair, int starts_tile, int rank) {
  return ((size_t)(pair * 2 + starts_tile) * 2 + rank) * BM * BN;
}

template <bool BACKWARD, int kLoadStages, int kBStages, int kStoreBufs, int kDecodeGroups>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(pair_threads(kDecodeGroups), 1)
nf4_gemm_sm100_pair_kernel(const __grid_constant__ CUtensorMap map_in, const __grid_constant__ CUtensorMap map_packed,
                           const __grid_constant__ CUtensorMap map_low, const __grid_constant__ CUtensorMap map_ext,
                           const __grid_constant__ CUtensorMap map_out, const __grid_constant__ Params p) {
  constexpr int kThreads = pair_threads(kDecodeGroups);
  extern __shared__ unsigned char smem_dyn[];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag_s;
  __shared__ WorkPlan plan_s;
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_dyn + (base - raw);
  const uint32_t load0 = base;
  const uint32_t codes0 = load0 + kLoadStages * kLoadStageBytes;
  const uint32_t btile0 = codes0 + kCodeStages * kPackedBytes;
  const uint32_t store0 = btile0 + kBStages * kTileBBytes;
  const uint32_t lut0 = store0 + kStoreBufs * kStoreBytes;
  const uint32_t bar0 = lut0 + kLutBytes;
  float2* lut_ptr = reinterpret_cast<float2*>(base_ptr + (lut0 - base));
  auto bar_ldfull = [&](int s) { return bar0 + 8u * s; };
  // consumed[g % 8] completes when the MMAs of contraction block number g (counted per CTA across tiles) have
  // finished reading their operands; ONE commit per block releases both the load stage and the B stage, in both
  // CTAs.  Sixteen slots exceed every ring depth, so a waiter can never be lapped.
  constexpr int kConsumedSlots = 16;
  static_assert(kLoadStages < kCodeStages && kCodeStages < kConsumedSlots && kBStages < kConsumedSlots,
                "ring deeper than the consumed slots");
  auto bar_consumed = [&](int g) { return bar0 + 8u * (kLoadStages + (g & (kConsumedSlots - 1))); };
  auto bar_bfull = [&](int s) { return bar0 + 8u * (kLoadStages + kConsumedSlots + s); };          // used in the leader
  auto bar_accfull = [&](int b) { return bar0 + 8u * (kLoadStages + kConsumedSlots + kBStages + b); };
  auto bar_accempty = [&](int b) { return bar0 + 8u * (kLoadStages + kConsumedSlots + kBStages + 2 + b); };  // leader
  const uint32_t bar_ext = bar0 + 8u * (kLoadStages + kConsumedSlots + kBStages + 4);
  auto bar_pkfull = [&](int s) { return bar_ext + 8u * (1 + s); };
  auto consumed_parity = [&](int g) { return (uint32_t)((g / kConsumedSlots) & 1); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  volatile int* abort_flag = &abort_flag_s;

  if (threadIdx.x == 0) {
    abort_flag_s = 0;
    plan_s.num_pairs = (int)(gridDim.x >> 1);
    plan_s.pair_id = (int)(blockIdx.x >> 1);
    plan_s.blocks = p.num_kb + (p.ext_steps > 0 ? 1 : 0);
    plan_s.full_tiles = p.full_tiles;
    plan_s.num_tiles = p.tiles_m * p.tiles_n;
    plan_s.tail_units = (plan_s.num_tiles - p.full_tiles) * plan_s.blocks;
    plan_s.tail_begin = tail_range_begin(plan_s, plan_s.pair_id);
    plan_s.tail_end = tail_range_begin(plan_s, plan_s.pair_id + 1);
    for (int s = 0; s < kLoadStages; ++s) mbar_init(bar_ldfull(s), 1);
    for (int s = 0; s < kCodeStages; ++s) mbar_init(bar_pkfull(s), 1);
    for (int g = 0; g < kConsumedSlots; ++g) mbar_init(bar_consumed(g), 1);
    for (int s = 0; s < kBStages; ++s) mbar_init(bar_bfull(s), 8);   // 4 warps of one group x 2 CTAs
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_accfull(b), 1);
      mbar_init(bar_accempty(b), 2 * kEpilogueWarps);
    }
    mbar_init(bar_ext, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // byte -> (first element, second element) fp32 codebook values; 16 copies so that lane l reads bank pair l % 16
  for (int i = threadIdx.x; i < 256 * 16; i += kThreads) {
    const int byte = i >> 4;
    const int lo = byte & 15, hi = byte >> 4;
    lut_ptr[i] = p.nibble_high_first ? make_float2(p.codebook[hi], p.codebook[lo])
                                     : make_float2(p.codebook[lo], p.codebook[hi]);
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // barriers of both CTAs are initialised before anyone signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  // Launched as a programmatic dependent of the kernel before it in the stream: everything above (barriers, the lookup
  // table, TMEM) touches no global memory and may overlap that kernel's tail; nothing below runs before that kernel
  // has completed and its writes are visible.  (Same-box A/B at 4096 tokens: +0.4 % per fwd+bwd step.  Launching the
  // small side kernels the same way was measured too and is slower, -0.7 %, so only the GEMM does it.)
  asm volatile("griddepcontrol.wait;" ::: "memory");

  const int pair_id = blockIdx.x >> 1;
  const int blocks_per_tile = p.num_kb + (p.ext_steps > 0 ? 1 : 0);
  const WorkPlan& plan = plan_s;   // in shared memory: read at item boundaries only, so it does not occupy registers

  if (warp == kProducerWarp) {
    // ================= TMA producer (each CTA loads its own token rows and its own half of the codes) ==========
    // Two streams with the same block order: packed codes (small, kCodeStages deep, needed first by the decoders)
    // and activation tiles (large, kLoadStages deep, needed last by the MMA).  Step t issues the codes of block t
    // and the activations of block t - kLag; both ring slots are free once block t - kCodeStages is consumed.
    constexpr int kLag = kCodeStages - kLoadStages;
    struct Cursor {
      WorkItem item;
      int kb, tm, tn;
      bool valid;
    };
    auto start_cursor = [&]() {
      Cursor c;
      c.item = first_item(plan);
      c.valid = c.item.valid;
      c.kb = c.item.kb0;
      c.tm = c.tn = 0;
      if (c.valid) pair_tile_coords(c.item.tile, p.tiles_m, p.tiles_n, c.tm, c.tn);
      return c;
    };
    auto advance = [&](Cursor& c) {
      if (++c.kb == c.item.kb1) {
        next_item(plan, c.item);
        c.valid = c.item.valid;
        c.kb = c.item.kb0;
        if (c.valid) pair_tile_coords(c.item.tile, p.tiles_m, p.tiles_n, c.tm, c.tn);
      }
    };
    Cursor pc = start_cursor(), ac = start_cursor();
    bool ok = true;
    for (int t = 0; ok; ++t) {
      if (!pc.valid && !ac.valid) break;
      const bool do_codes = pc.valid;
      const bool do_act = t >= kLag && ac.valid;
      if (t >= kCodeStages)
        ok = mbar_wait_cluster(bar_consumed(t - kCodeStages), consumed_parity(t - kCodeStages), abort_flag, p.status, 1);
      if (!ok) break;
      if (lane == 0) {
        if (do_codes) {
          const int s = t % kCodeStages;
          if (pc.kb < p.num_kb) {
            const uint32_t pk_dst = codes0 + (uint32_t)s * kPackedBytes;
            mbar_expect_tx(bar_pkfull(s), kPackedBytes);
            if (!BACKWARD) tma_load_2d(pk_dst, &map_packed, pc.kb * (BK / 2), pc.tn * BN + (int)rank * BNH, bar_pkfull(s));
            else tma_load_2d(pk_dst, &map_packed, (pc.tn * BN + (int)rank * BNH) / 2, pc.kb * BK, bar_pkfull(s));
          } else {
            mbar_arrive(bar_pkfull(s));   // the low-rank block has no codes; keep the ring's phases in step
          }
        }
        if (do_act) {
          const int s = (t - kLag) % kLoadStages;
          const uint32_t a_dst = load0 + (uint32_t)s * kLoadStageBytes;
          const int row0 = ac.tm * 2 * BM + (int)rank * BM;
          mbar_expect_tx(bar_ldfull(s), kTileABytes);
          if (ac.kb < p.num_kb) tma_load_2d(a_dst, &map_in, ac.kb * BK, row0, bar_ldfull(s));
          else tma_load_2d(a_dst, &map_low, 0, row0, bar_ldfull(s));
        }
#ifdef MOLT_PAIR_TRACE
        MOLT_TRACE(0, t);
#endif
      }
      __syncwarp();
      if (do_codes) advance(pc);
      if (do_act) advance(ac);
    }
  } else if (warp == kMmaWarp) {
    // ================= MMA issuer (leader CTA only) =================
    if (leader) {
      constexpr uint32_t idesc = make_idesc(2 * BM, BN, BACKWARD ? 1 : 0);
      // low descriptor words of stage 0: start address and leading byte offset (K-major: unused, 16; MN-major: 8192)
      const uint32_t a_lo0 = ((load0 >> 4) & 0x3fffu) | (1u << 16);
      const uint32_t b_lo0 = ((btile0 >> 4) & 0x3fffu) | ((BACKWARD ? (8192u >> 4) : 1u) << 16);
      // high word: stride byte offset 1024, descriptor version 1, 128-byte swizzle
      constexpr uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t kBStep = BACKWARD ? 128u : 2u;   // 16 contraction elements: 2048 bytes MN-major, 32 bytes K-major
      // One thread runs this loop: it is the serial heart of the kernel (it feeds the tensor cores of two SMs),
      // so it holds nothing but the wait, the four MMAs and the commit.
      if (lane == 0) {
        int ls = 0, bs = 0, acc = 0, g = 0;
        uint32_t bphase = 0, acc_phase = 0;
        bool ok = true;
        for (WorkItem item = first_item(plan); item.valid && ok; next_item(plan, item)) {
          ok = mbar_wait_cluster(bar_accempty(acc), acc_phase ^ 1u, abort_flag, p.status, 2);
          if (!ok) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)acc * BN;
          uint32_t accumulate = 0u;
          for (int kb = item.kb0; kb < item.kb1; ++kb) {
            // The decoders of both CTAs arrive on b_full only after their own activation tile has landed, so
            // this one wait covers both operands in both CTAs.
            ok = mbar_wait_cluster(bar_bfull(bs), bphase, abort_flag, p.status, 4);
            if (!ok) break;
            tc_fence_after();
            const uint32_t a_lo = a_lo0 + (uint32_t)ls * (kLoadStageBytes >> 4);
            const uint32_t b_lo = b_lo0 + (uint32_t)bs * (kTileBBytes >> 4);
            if (kb < p.num_kb) {
              umma_bf16_pair(d_tmem, desc64(a_lo, desc_hi), desc64(b_lo, desc_hi), idesc, accumulate);
#pragma unroll
              for (int ks = 1; ks < BK / 16; ++ks)
                umma_bf16_pair(d_tmem, desc64(a_lo + ks * 2, desc_hi), desc64(b_lo + ks * kBStep, desc_hi), idesc, 1u);
            } else {   // the low-rank block
              for (int ks = 0; ks < p.ext_steps; ++ks)
                umma_bf16_pair(d_tmem, desc64(a_lo + ks * 2, desc_hi), desc64(b_lo + ks * kBStep, desc_hi), idesc,
                               (accumulate | (uint32_t)(ks > 0)));
            }
            accumulate = 1u;
            // one commit releases this block's load stage and B stage in both CTAs once the MMAs have read them
            umma_commit_both(bar_consumed(g));
            if (kb == item.kb1 - 1) umma_commit_both(bar_accfull(acc));
#ifdef MOLT_PAIR_TRACE
            MOLT_TRACE(1, g);
#endif
            ++g;
            if (++ls == kLoadStages) ls = 0;
            if (++bs == kBStages) { bs = 0; bphase ^= 1u; }
          }
          if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
      }
      __syncwarp();
    }
  } else if (warp >= kFirstDecodeWarp) {
    // ================= NF4 decoders =================
    // Groups of four warps take the contraction blocks in turn (running block number modulo the group count),
    // so the decode latency of one block overlaps the following blocks'.  Inside a group every thread expands one whole
    // 64-element segment (one absmax) per block.
    const int dt = threadIdx.x - kFirstDecodeWarp * 32;
    const int dwarp = dt >> 5;
    const int grp = dwarp % kDecodeGroups;
    const int u = (dwarp / kDecodeGroups) * 32 + lane;   // 0..127 inside the group
    const uint32_t lut_lane = lut0 + (uint32_t)(lane & 15) * 8u;
    const long long kblocks_per_row = p.k / 64;
    const uint32_t bfull_remote_base = map_to_cta(bar_bfull(0), 0);
    uint32_t ext_phase = 0;
    bool ok = true;
    // Segment geometry of this thread (the same for every contraction block).
    const int seg_j = u & 63, seg_a = u >> 6;        // backward: contraction row, 64-column atom
    uint32_t src_off0, src_off1;                     // the two 16-byte halves of the segment's packed codes
    if (!BACKWARD) {
      // 32-byte rows loaded with the 32-byte TMA swizzle: the halves of rows 4..7 (mod 8) are exchanged, so the eight
      // lanes of a quarter-warp, all reading the same logical half, touch eight different 16-byte bank groups
      const uint32_t flip = ((uint32_t)u >> 2) & 1u;
      src_off0 = (uint32_t)u * 32u + flip * 16u;
      src_off1 = (uint32_t)u * 32u + (flip ^ 1u) * 16u;
    } else {
      const uint32_t x = ((uint32_t)seg_j >> 1) & 3u;   // 64-byte swizzle of the packed tile
      src_off0 = (uint32_t)seg_j * 64u + ((((uint32_t)(2 * seg_a)) ^ x) << 4);
      src_off1 = (uint32_t)seg_j * 64u + ((((uint32_t)(2 * seg_a + 1)) ^ x) << 4);
    }
    const uint32_t dst_off = !BACKWARD ? (uint32_t)u * 128u : (uint32_t)seg_a * 8192u + (uint32_t)seg_j * 128u;
    const uint32_t swz = (dst_off >> 7) & 7u;
    constexpr int kPrefetch = 4;   // absmax values are fetched this many of the group's blocks ahead of their use
    int g_tile = 0;                // running block number of the item's first block
    for (WorkItem item = first_item(plan); item.valid && ok; g_tile += item.kb1 - item.kb0, next_item(plan, item)) {
      int tm, tn;
      pair_tile_coords(item.tile, p.tiles_m, p.tiles_n, tm, tn);
      const int col0 = tn * BN + (int)rank * BNH;   // first B row (forward: weight row; backward: weight column)
      // forward : absmax[(col0 + i) * kpr + kb]            backward: absmax[(kb * 64 + j) * kpr + col0 / 64 + a]
      const float* scale_ptr;
      long long scale_step;
      bool scale_ok;
      if (!BACKWARD) {
        const long long row = (long long)col0 + u;
        scale_ok = row < p.n;
        scale_ptr = p.absmax + (scale_ok ? row : 0) * kblocks_per_row;
        scale_step = 1;
      } else {
        const long long colblk = (long long)(col0 >> 6) + seg_a;
        scale_ok = colblk < kblocks_per_row;
        scale_ptr = p.absmax + (long long)seg_j * kblocks_per_row + (scale_ok ? colblk : 0);
        scale_step = (long long)BK * kblocks_per_row;
      }
      auto load_scale = [&](int kb) -> float {
        return (kb < p.num_kb && scale_ok) ? __ldg(scale_ptr + (long long)kb * scale_step) : 0.f;
      };
      // the group's first block of this item: running block number g_tile + (kb - kb0) is congruent to grp
      const int kb_first = item.kb0 + ((grp - g_tile) % kDecodeGroups + kDecodeGroups) % kDecodeGroups;
      float cur[kPrefetch];
#pragma unroll
      for (int q = 0; q < kPrefetch; ++q) cur[q] = load_scale(kb_first + kDecodeGroups * q);
      for (int kb0 = kb_first; kb0 < item.kb1 && ok; kb0 += kDecodeGroups * kPrefetch) {
        float nxt[kPrefetch];
#pragma unroll
        for (int q = 0; q < kPrefetch; ++q) nxt[q] = load_scale(kb0 + kDecodeGroups * (kPrefetch + q));
#pragma unroll
        for (int q = 0; q < kPrefetch; ++q) {
          const int kb = kb0 + kDecodeGroups * q;
          if (kb >= item.kb1 || !ok) continue;
          const float scale = cur[q];
          unsigned long long scale2;   // (scale, scale)
          asm("mov.b64 %0, {%1, %1};" : "=l"(scale2) : "f"(scale));
          const int g = g_tile + (kb - item.kb0);
          const int ls = g % kLoadStages, bs = g % kBStages, cs = g % kCodeStages;
          ok = mbar_wait(bar_pkfull(cs), (uint32_t)((g / kCodeStages) & 1), abort_flag, p.status, 5);
          if (ok && g >= kBStages)   // the block that used this B stage must have been consumed
            ok = mbar_wait_cluster(bar_consumed(g - kBStages), consumed_parity(g - kBStages), abort_flag, p.status, 6);
          if (!ok) continue;
#ifdef MOLT_PAIR_TRACE
          if (dt == 0 && !(p.debug & 64)) MOLT_TRACE(2, g);
#endif
          const uint32_t bt = btile0 + bs * kTileBBytes;
          if (kb < p.num_kb && (p.debug & 1)) {
          } else if (kb < p.num_kb) {
            const uint32_t pk = codes0 + (uint32_t)cs * kPackedBytes;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              uint32_t words[4];
              asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(words[0]), "=r"(words[1]), "=r"(words[2]), "=r"(words[3])
                           : "r"(pk + (half == 0 ? src_off0 : src_off1))
                           : "memory");
              // 16 table lookups (independent, issued back to back), then 16 two-wide multiplies (mul.rn.f32x2 rounds
              // each lane like a scalar multiply), 16 roundings, 4 stores
              unsigned long long codes[16];
#pragma unroll
              for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                  const uint32_t byte = __byte_perm(words[c], 0u, 0x4440u + (uint32_t)b);
                  asm("ld.shared.b64 %0, [%1];" : "=l"(codes[c * 4 + b]) : "r"(lut_lane + byte * 128u));
                }
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                uint32_t out[4];
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                  unsigned long long prod;
                  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(prod) : "l"(codes[c * 4 + b]), "l"(scale2));
                  asm("{\n\t.reg .f32 lo, hi;\n\tmov.b64 {lo, hi}, %1;\n\tcvt.rn.bf16x2.f32 %0, hi, lo;\n\t}" : "=r"(out[b]) : "l"(prod));
                }
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(bt + dst_off + ((((uint32_t)(4 * half + c)) ^ swz) << 4)),
                             "r"(out[0]), "r"(out[1]), "r"(out[2]), "r"(out[3])
                             : "memory");
              }
            }
            fence_proxy_async();
          } else {
            // low-rank block: this CTA's half of the ready-made B operand comes by TMA into the B stage
            if (u == 0) {
              if (!BACKWARD) {
                mbar_expect_tx(bar_ext, kTileBBytes);
                tma_load_2d(bt, &map_ext, 0, col0, bar_ext);
              } else {
                mbar_expect_tx(bar_ext, 2u * (uint32_t)p.ext_steps * 16u * 128u);
                tma_load_2d(bt, &map_ext, col0, 0, bar_ext);
                tma_load_2d(bt + 8192u, &map_ext, col0 + 64, 0, bar_ext);
              }
            }
            ok = mbar_wait(bar_ext, ext_phase, abort_flag, p.status, 7);
            if (!ok) continue;
          }
          // this CTA's activation tile must have landed before the block is announced to the MMA thread
          ok = mbar_wait(bar_ldfull(ls), (uint32_t)((g / kLoadStages) & 1), abort_flag, p.status, 9);
          if (!ok) continue;
          __syncwarp();
          if (lane == 0) mbar_arrive_remote(bfull_remote_base + 8u * (uint32_t)bs);
#ifdef MOLT_PAIR_TRACE
          if (dt == 0 && !(p.debug & 64)) MOLT_TRACE(3, g);
#endif
        }
#pragma unroll
        for (int q = 0; q < kPrefetch; ++q) cur[q] = nxt[q];
      }
      // the low-rank barrier completes once per item that holds the low-rank block, whichever group handled it
      if (p.ext_steps > 0 && item.kb1 == blocks_per_tile) ext_phase ^= 1u;
    }
  } else {
    // ================= epilogue: TMEM -> bf16 -> shared -> TMA store (own 128 token rows) =================
    const int row = warp * 32 + lane;
    const uint32_t accempty_remote_base = map_to_cta(bar_accempty(0), 0);
    int acc = 0;
    uint32_t acc_phase = 0;
    int store_buf = 0;
    bool ok = true;
    for (WorkItem item = first_item(plan); item.valid && ok; next_item(plan, item)) {
      int tm, tn;
      pair_tile_coords(item.tile, p.tiles_m, p.tiles_n, tm, tn);
      const int row0 = tm * 2 * BM + (int)rank * BM;
      ok = mbar_wait_cluster(bar_accfull(acc), acc_phase, abort_flag, p.status, 8);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)acc * BN;
      if (item.tile >= plan.full_tiles) {
        // ---- part of a split tile: the fp32 accumulator goes to this pair's slot, row-major ----
        float* part = p.split_partial + split_slot_offset(pair_id, item.kb0 == 0 ? 1 : 0, (int)rank) + (size_t)row * BN;
        const bool row_valid = (long long)row0 + row < p.m;   // the fix-up kernel never reads rows past the end
        for (int cg = 0; cg < BN / 32 && !(p.debug & 16); ++cg) {
          uint32_t v[32];
          tmem_ld32(t_row + (uint32_t)cg * 32u, v);
          tmem_ld_wait();
          if (!row_valid) continue;
#pragma unroll
          for (int c = 0; c < 8; ++c)
            __stcg(reinterpret_cast<float4*>(part + cg * 32 + c * 4),
                   make_float4(__uint_as_float(v[4 * c]), __uint_as_float(v[4 * c + 1]), __uint_as_float(v[4 * c + 2]),
                               __uint_as_float(v[4 * c + 3])));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(accempty_remote_base + 8u * (uint32_t)acc);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        continue;
      }
      for (int cg = 0; cg < BN / 64 && !(p.debug & 4); ++cg) {
        const uint32_t stage_addr = store0 + (uint32_t)store_buf * kStoreBytes;
        // the store that last read this staging buffer must have finished reading it
        if (threadIdx.x == 0) {
          if (kStoreBufs == 2) tma_store_wait_read<1>();
          else tma_store_wait_read<0>();
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        uint32_t v0[32], v1[32];
        tmem_ld32(t_row + (uint32_t)cg * 64u, v0);
        tmem_ld32(t_row + (uint32_t)cg * 64u + 32u, v1);
        tmem_ld_wait();
        const uint32_t dst_row = stage_addr + (uint32_t)row * 128u;
        const uint32_t swz = (uint32_t)row & 7u;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t o0 = pack_bf16x2(__uint_as_float(v0[c * 8 + 0]), __uint_as_float(v0[c * 8 + 1]));
          const uint32_t o1 = pack_bf16x2(__uint_as_float(v0[c * 8 + 2]), __uint_as_float(v0[c * 8 + 3]));
          const uint32_t o2 = pack_bf16x2(__uint_as_float(v0[c * 8 + 4]), __uint_as_float(v0[c * 8 + 5]));
          const uint32_t o3 = pack_bf16x2(__uint_as_float(v0[c * 8 + 6]), __uint_as_float(v0[c * 8 + 7]));
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst_row + (((uint32_t)c ^ swz) << 4)), "r"(o0),
                       "r"(o1), "r"(o2), "r"(o3)
                       : "memory");
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t o0 = pack_bf16x2(__uint_as_float(v1[c * 8 + 0]), __uint_as_float(v1[c * 8 + 1]));
          const uint32_t o1 = pack_bf16x2(__uint_as_float(v1[c * 8 + 2]), __uint_as_float(v1[c * 8 + 3]));
          const uint32_t o2 = pack_bf16x2(__uint_as_float(v1[c * 8 + 4]), __uint_as_float(v1[c * 8 + 5]));
          const uint32_t o3 = pack_bf16x2(__uint_as_float(v1[c * 8 + 6]), __uint_as_float(v1[c * 8 + 7]));
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst_row + (((uint32_t)(c + 4) ^ swz) << 4)),
                       "r"(o0), "r"(o1), "r"(o2), "r"(o3)
                       : "memory");
        }
        fence_proxy_async();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 0) {
          if (row0 < p.m) tma_store_2d(&map_out, stage_addr, tn * BN + cg * 64, row0);
          tma_store_commit();
        }
        if (kStoreBufs == 2) store_buf ^= 1;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(accempty_remote_base + 8u * (uint32_t)acc);
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if (threadIdx.x == 0) tma_store_wait_all();
  }

  // ---- teardown ----
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // neither CTA releases TMEM or exits while the other may still signal it or use its operands
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// out[row, col] = bf16(sum over the parts of a split tile), parts added in pair order.  One thread per 8 columns.
__global__ void __launch_bounds__(256) split_fixup_kernel(const float* __restrict__ partial, WorkPlan plan, int tiles_m,
                                                          int tiles_n, long long m, long long out_cols,
                                                          __nv_bfloat16* __restrict__ out) {
  const int tail_tile = blockIdx.y;
  const int tile = plan.full_tiles + tail_tile;
  int tm, tn;
  pair_tile_coords(tile, tiles_m, tiles_n, tm, tn);
  const int idx = blockIdx.x * 256 + threadIdx.x;          // 2 * BM rows x BN / 8 column groups
  const int r = idx / (BN / 8), cgroup = idx % (BN / 8);
  const long long row = (long long)tm * 2 * BM + r, col = (long long)tn * BN + cgroup * 8;
  if (row >= m || col >= out_cols) return;
  const int unit0 = tail_tile * plan.blocks, unit1 = unit0 + plan.blocks;
  int first = (int)(((long long)unit0 * plan.num_pairs) / plan.tail_units);   // the pair whose range holds unit0
  while (first + 1 < plan.num_pairs && tail_range_begin(plan, first + 1) <= unit0) ++first;
  while (first > 0 && tail_range_begin(plan, first) > unit0) --first;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int c = first; c < plan.num_pairs && tail_range_begin(plan, c) < unit1; ++c) {
    const int start = tail_range_begin(plan, c) > unit0 ? tail_range_begin(plan, c) : unit0;
    const float* src = partial + split_slot_offset(c, start == unit0 ? 1 : 0, r / BM) + (size_t)(r % BM) * BN + cgroup * 8;
    const float4 lo = __ldcg(reinterpret_cast<const float4*>(src)), hi = __ldcg(reinterpret_cast<const float4*>(src + 4));
    acc[0] += lo.x; acc[1] += lo.y; acc[2] += lo.z; acc[3] += lo.w;
    acc[4] += hi.x; acc[5] += hi.y; acc[6] += hi.z; acc[7] += hi.w;
  }
  const uint4 packed = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                                  pack_bf16x2(acc[6], acc[7]));
  *reinterpret_cast<uint4*>(out + row * out_cols + col) = packed;
}

}  // namespace pair

// ---- host side -----------------------------------------------------------------------------------------
int make_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, const void* ptr, uint64_t inner, uint64_t outer,
                    uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle,
                    const char* what);

// Scratch for splitting the last wave: two fp32 partial tiles per CTA pair.
size_t sm100_split_bytes() {
  return pair::split_slot_offset(sm_count() / 2, 0, 0) * sizeof(float);
}

int sm100_gemm_pair(bool backward, const WeightView& w, const float* absmax_f32, const __nv_bfloat16* in,
                    const __nv_bfloat16* low, const __nv_bfloat16* ext, int rp, __nv_bfloat16* out, long long m,
                    void* split_ws, cudaStream_t s) {
  using namespace pair;
  if (!sm100_gemm_supported(w, rp)) return fail(MOLT_E_CAPABILITY, "tcgen05 GEMM: unsupported shape");
  const long long contraction = backward ? w.n : w.k;
  const long long out_cols = backward ? w.k : w.n;
  CUtensorMap map_in, map_packed, map_low, map_ext, map_out;
  if (int rc = make_tensor_map(&map_in, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, in, contraction, m, contraction * 2, BK, BM,
                               CU_TENSOR_MAP_SWIZZLE_128B, "activations"))
    return rc;
  if (!backward) {
    if (int rc = make_tensor_map(&map_packed, CU_TENSOR_MAP_DATA_TYPE_UINT8, w.packed, w.k / 2, w.n, w.k / 2, BK / 2,
                                 BNH, CU_TENSOR_MAP_SWIZZLE_32B, "packed weight"))
      return rc;
  } else {
    if (int rc = make_tensor_map(&map_packed, CU_TENSOR_MAP_DATA_TYPE_UINT8, w.packed, w.k / 2, w.n, w.k / 2, BNH / 2,
                                 BK, CU_TENSOR_MAP_SWIZZLE_64B, "packed weight"))
      return rc;
  }
  const bool has_low = low != nullptr && ext != nullptr && rp > 0;
  if (has_low) {
    if (int rc = make_tensor_map(&map_low, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, low, 64, m, 128, 64, BM,
                                 CU_TENSOR_MAP_SWIZZLE_128B, "low-rank input"))
      return rc;
    if (!backward) {
      if (int rc = make_tensor_map(&map_ext, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, ext, 64, w.n, 128, 64, BNH,
                                   CU_TENSOR_MAP_SWIZZLE_128B, "scaled LoRA B"))
        return rc;
    } else {
      if (int rc = make_tensor_map(&map_ext, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, ext, w.k, rp, w.k * 2, 64, rp,
                                   CU_TENSOR_MAP_SWIZZLE_128B, "LoRA A"))
        return rc;
    }
  } else {
    map_low = map_in;
    map_ext = map_in;
  }
  if (int rc = make_tensor_map(&map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, out, out_cols, m, out_cols * 2, 64, BM,
                               CU_TENSOR_MAP_SWIZZLE_128B, "output"))
    return rc;

  Params p;
  p.packed = w.packed;
  p.absmax = absmax_f32;
  p.status = device_status_word();
  if (p.status == nullptr) return fail(MOLT_E_RUNTIME, "tcgen05 GEMM: no device status word");
  p.m = m;
  p.n = w.n;
  p.k = w.k;
  p.num_kb = (int)(contraction / BK);
  p.ext_steps = has_low ? rp / 16 : 0;
  p.tiles_m = (int)((m + 2 * BM - 1) / (2 * BM));
  p.tiles_n = (int)((out_cols + BN - 1) / BN);
  p.nibble_high_first = w.nibble_order == MOLT_NIBBLE_HIGH_FIRST ? 1 : 0;
  {
    const char* dbg = getenv("MOLT_B200_DEBUG");
    p.debug = dbg != nullptr ? atoi(dbg) : 0;
    const char* tr = getenv("MOLT_B200_TRACE_PTR");   // device pointer (decimal) of a 16 KB trace buffer
    p.trace = tr != nullptr ? reinterpret_cast<unsigned long long*>(strtoull(tr, nullptr, 10)) : nullptr;
  }
  for (int i = 0; i < 16; ++i) p.codebook[i] = w.codebook[i];

  int variant = 0;
  {
    const char* env = getenv("MOLT_B200_PAIR_STAGES");   // timing experiments: 0 = activation/B stages (6,3), the default; 1 = (4,4), 2 = (4,5), 3 = (3,6), 4 = (5,4); 5, 6, 7, 8 = (6,3) with 2, 3, 4, 1 decode groups; 9 = (5,3) with two store buffers
    variant = env != nullptr ? atoi(env) : 0;
    if (variant < 0 || variant > 9) variant = 0;
  }
  const long long tiles = (long long)p.tiles_m * p.tiles_n;
  const long long all_pairs = sm_count() / 2;
  long long pairs = all_pairs;
  if (tiles < pairs) pairs = tiles;
  // Whole waves run the static schedule; a last partial wave is split along the contraction when scratch was given.
  p.full_tiles = (int)tiles;
  p.split_partial = nullptr;
  {
    const char* env = getenv("MOLT_B200_NO_SPLIT");   // tests and timing experiments: 1 = keep the plain schedule
    const char* force = getenv("MOLT_B200_FORCE_SPLIT");   // 1 = split whenever the shape allows it
    const bool allowed = split_ws != nullptr && !(env != nullptr && atoi(env) != 0);
    const bool forced = force != nullptr && atoi(force) != 0;
    const long long blocks = p.num_kb + (p.ext_steps > 0 ? 1 : 0);
    if (tiles < all_pairs) {
      // Fewer tiles than CTA pairs (few tokens): cutting all tiles along the contraction so that every pair of the device
      // gets an equal run of blocks was measured and is slower (14336 x 4096 weight, 32..256 tokens: 55-69 us against
      // 52-54 us) -- the fp32 partial tiles and the fix-up launch cost more than the shorter runs save.
    } else {
      const long long rem = tiles % pairs;
      // Splitting costs about 40 us (fp32 partial tiles out and in again, one more launch).  It pays when the last wave
      // is at most half full and every pair still gets a run of blocks long enough to fill its pipeline (measured on
      // the 14336 x 4096 weight: backward at 4096 tokens -8 %, forward with its 65-block tiles no gain).
      const bool worth_it = (rem * 2 <= pairs && rem * blocks / pairs >= 32) || forced;
      if (allowed && rem != 0 && tiles > pairs && worth_it && rem * blocks >= pairs && rem * blocks * pairs < (1LL << 30)) {
        p.full_tiles = (int)(tiles - rem);
        p.split_partial = reinterpret_cast<float*>(split_ws);
      }
    }
  }
  const int grid = (int)pairs * 2;
  static thread_local bool configured[64][2][10] = {};
  int dev = 0;
  MOLT_CUDA(cudaGetDevice(&dev));
  const bool need_config = dev >= 0 && dev < 64 && !configured[dev][backward ? 1 : 0][variant];
#define MOLT_PAIR_LAUNCH(BWD, LS, BS, SB, GR)                                                              \
  do {                                                                                                     \
    if (need_config)                                                                                       \
      MOLT_CUDA(cudaFuncSetAttribute(nf4_gemm_sm100_pair_kernel<BWD, LS, BS, SB, GR>,                      \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize,                          \
                                     (int)smem_bytes(LS, BS, SB)));                                        \
    cudaLaunchConfig_t cfg = {};                                                                           \
    cfg.gridDim = dim3((unsigned)grid);                                                                    \
    cfg.blockDim = dim3((unsigned)pair_threads(GR));                                                       \
    cfg.dynamicSmemBytes = smem_bytes(LS, BS, SB);                                                         \
    cfg.stream = s;                                                                                        \
    cudaLaunchAttribute attr[1];                                                                           \
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                                       \
    attr[0].val.programmaticStreamSerializationAllowed = 1;                                                \
    cfg.attrs = attr;                                                                                      \
    cfg.numAttrs = 1;                                                                                      \
    MOLT_CUDA(cudaLaunchKernelEx(&cfg, nf4_gemm_sm100_pair_kernel<BWD, LS, BS, SB, GR>, map_in, map_packed, map_low, \
                                 map_ext, map_out, p));                                                    \
  } while (0)
#define MOLT_PAIR_DISPATCH(BWD)                                                  \
  do {                                                                           \
    if (variant == 1) MOLT_PAIR_LAUNCH(BWD, 4, 4, 2, decode_groups(BWD));        \
    else if (variant == 2) MOLT_PAIR_LAUNCH(BWD, 4, 5, 1, decode_groups(BWD));   \
    else if (variant == 3) MOLT_PAIR_LAUNCH(BWD, 3, 6, 1, decode_groups(BWD));   \
    else if (variant == 4) MOLT_PAIR_LAUNCH(BWD, 5, 4, 1, decode_groups(BWD));   \
    else if (variant == 5) MOLT_PAIR_LAUNCH(BWD, 6, 3, 1, 2);                    \
    else if (variant == 6) MOLT_PAIR_LAUNCH(BWD, 6, 3, 1, 3);                    \
    else if (variant == 7) MOLT_PAIR_LAUNCH(BWD, 6, 3, 1, 4);                    \
    else if (variant == 8) MOLT_PAIR_LAUNCH(BWD, 6, 3, 1, 1);                    \
    else if (variant == 9) MOLT_PAIR_LAUNCH(BWD, 5, 3, 2, 2);                    \
    else MOLT_PAIR_LAUNCH(BWD, 6, 3, 1, decode_groups(BWD));                     \
  } while (0)
  if (backward) MOLT_PAIR_DISPATCH(true);
  else MOLT_PAIR_DISPATCH(false);
#undef MOLT_PAIR_DISPATCH
#undef MOLT_PAIR_LAUNCH
  if (need_config) configured[dev][backward ? 1 : 0][variant] = true;
  if (int rc = launch_status("nf4_gemm_sm100_pair_kernel")) return rc;
  if (p.full_tiles < tiles) {
    WorkPlan plan;
    plan.num_pairs = (int)pairs;
    plan.pair_id = 0;
    plan.blocks = p.num_kb + (p.ext_steps > 0 ? 1 : 0);
    plan.full_tiles = p.full_tiles;
    plan.num_tiles = (int)tiles;
    plan.tail_units = (int)(tiles - p.full_tiles) * plan.blocks;
    plan.tail_begin = plan.tail_end = 0;
    dim3 fgrid((unsigned)(2 * BM * (BN / 8) / 256), (unsigned)(tiles - p.full_tiles));
    split_fixup_kernel<<<fgrid, 256, 0, s>>>(p.split_partial, plan, p.tiles_m, p.tiles_n, m, out_cols, out);
    return launch_status("split_fixup_kernel");
  }
  return MOLT_OK;
}

}  // namespace molt
