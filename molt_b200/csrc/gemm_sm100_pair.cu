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
// Tall tiles (kSub = 2): a pair tile covers 512 token rows, i.e. every CTA holds TWO 128-row activation tiles per
// contraction block and two accumulators (all 512 TMEM columns), and multiplies both by the SAME decoded B tile.  The
// decode, the packed-code traffic and every handshake are then paid once per two MMAs, which is what bounds the kernel;
// the price is that the epilogue of a tile no longer overlaps the whole next tile (the first accumulator is handed back
// as soon as it is drained, so the next tile's first MMAs start early).  Short tiles (kSub = 1: 256 rows, two
// accumulators used in turn) remain for small token counts and for shapes whose tall tiles quantise badly.
//
// Dense variant (kDense): the same pipeline for a frozen bf16 weight (the LM head): the second producer warp loads the
// B half-tiles ready-made by TMA into the B ring, one decode warp merely relays "both operands of this CTA have landed"
// to the leader, everything else (tall tiles, MMA issue, epilogue, split schedule) is shared.
//
// Per CTA: two TMA rings (16 KB activation tiles; 4 KB packed-code tiles, deeper) run several blocks ahead of a
// separate ring of decoded B half-tiles, so the global-memory latency is not serialised with the decode.
// Decode: a decoder thread owns one 64-element segment (one absmax) per block.  It first forms the sixteen values
// the segment can take, bf16(fp32 codebook value x fp32 absmax) -- one fp32 multiply and one rounding each, the bits
// of the standalone dequantiser -- and keeps them in registers as two byte planes (low and high bytes of the sixteen
// bf16 values).  Every 4-bit code then selects its value with byte permutes (prmt): the code's low three bits index
// eight table bytes, its top bit picks between the two table halves.  No lookup table in shared memory: the L1 /
// shared-memory data path, the busiest unit of this kernel, carries only the TMA writes, the packed codes, the
// decoded tile and the tensor core's operand reads.  The leader CTA's MMA warp issues the pair MMA and signals
// both CTAs with tcgen05.commit; decoders and epilogue warps of the second CTA signal the leader with remote
// mbarrier arrives.  All waits are bounded (status word + clean exit), and TMEM is released after a cluster barrier.
#include <cuda.h>
#include <cudaTypedefs.h>
#ifdef MOLT_PAIR_TRACE
#include <stdlib.h>
#endif
#include "internal.h"
#include "sm100_ptx.cuh"

namespace molt {
namespace pair {

constexpr int BM = 128;            // token rows per CTA (256 per pair)
constexpr int BN = 256;            // output columns per pair tile
constexpr int BNH = 128;           // B rows decoded per CTA
constexpr int BK = 64;
constexpr int kEpilogueWarps = 4;
// Decode groups: groups of four warps that take the contraction blocks in turn.
#ifndef MOLT_PAIR_GROUPS
#define MOLT_PAIR_GROUPS 3
#endif
#ifndef MOLT_PAIR_LOAD_STAGES
#define MOLT_PAIR_LOAD_STAGES 6
#endif
// How many of the eight code words of a segment are decoded through the lookup table in shared memory (load/store
// pipe) instead of byte permutes in registers (integer pipe): the two pipes work side by side.
#ifndef MOLT_PAIR_LUT_WORDS
#define MOLT_PAIR_LUT_WORDS 0
#endif
#ifndef MOLT_PAIR_B_STAGES
#define MOLT_PAIR_B_STAGES (MOLT_PAIR_LUT_WORDS > 0 ? 3 : 5)
#endif
constexpr int kDecodeGroupsDefault = MOLT_PAIR_GROUPS;
constexpr int kLoadStagesDefault = MOLT_PAIR_LOAD_STAGES;   // ring of activation tiles
constexpr int kBStagesDefault = MOLT_PAIR_B_STAGES;         // ring of decoded B half-tiles
// Warp roles.  An SM issues from four schedulers and warp w belongs to scheduler w % 4.  The three single-thread loops
// that pace the pipeline (MMA issue, the two TMA producers) are long dependent instruction chains, so they get
// scheduler 1 to themselves (next to one epilogue warp, which is idle most of the time); the decoder warps, which
// issue thousands of instructions per block, are the warps >= 4 on the other three schedulers.
constexpr int kMmaWarp = 5;
constexpr int kActivationWarp = 9;    // TMA producer of the activation tiles
constexpr int kCodeWarp = 13;         // TMA producer of the packed-code tiles
__host__ __device__ constexpr bool is_decode_warp(int warp) { return warp >= 4 && (warp & 3) != 1; }
// position of a decode warp among the decode warps (warps 4, 6, 7, 8, 10, 11, 12, 14, ...)
__host__ __device__ constexpr int decode_warp_index(int warp) {
  return ((warp >> 2) - 1) * 3 + ((warp & 3) == 0 ? 0 : (warp & 3) - 1);
}
constexpr int pair_warps(int groups) {
  int warp = 4, found = 0;
  while (found < 4 * groups) {
    if (is_decode_warp(warp)) ++found;
    ++warp;
  }
  return warp > kCodeWarp + 1 ? warp : kCodeWarp + 1;
}
constexpr int pair_threads(int groups) { return pair_warps(groups) * 32; }

constexpr uint32_t kTileABytes = BM * BK * 2;          // 16384
constexpr uint32_t kPackedBytes = BNH * BK / 2;        // 4096
constexpr uint32_t kLoadStageBytes = kTileABytes;      // activation ring stage
#ifndef MOLT_PAIR_CODE_STAGES
#define MOLT_PAIR_CODE_STAGES 8
#endif
constexpr int kCodeStages = MOLT_PAIR_CODE_STAGES;                         // ring of packed-code tiles; runs further ahead than the activations
constexpr uint32_t kTileBBytes = BNH * BK * 2;         // 16384
constexpr uint32_t kStoreBytes = BM * 64 * 2;          // 16384
constexpr int kLutWords = MOLT_PAIR_LUT_WORDS;
constexpr uint32_t kLutBytes = kLutWords > 0 ? 256 * 16 * 8 : 0;   // [byte][16 copies] of float2 (both codebook values of a byte)
constexpr uint32_t smem_bytes(int load_stages, int b_stages, int store_bufs, bool dense = false) {
  return load_stages * kLoadStageBytes + (dense ? 0 : kCodeStages * kPackedBytes) + b_stages * kTileBBytes +
         store_bufs * kStoreBytes + (dense ? 0 : kLutBytes) + 512 /*barriers*/ + 1024 /*alignment*/;
}

struct Params {
  const uint8_t* packed; // [n, k / 2] packed codes
  const float* absmax;   // fp32 [n * k / 64], or NULL when the decoders read the double-quantised form themselves:
  const uint8_t* absmax_u8;   //   8-bit codes [n * k / 64]
  const float* absmax2;       //   fp32 absmax of every 2^block2_shift of them
  const float* code2;         //   256-entry table
  float offset;
  int block2_shift;
  int32_t* status;
  long long m, n, k;
  int num_kb;
  int ext_steps;         // rp / 16, 0 = no low-rank block
  int tiles_m, tiles_n;  // pair tiles: 256 tokens x 256 columns
  int full_tiles;        // tiles on the static schedule (whole waves); the tiles after them are split along the contraction
  int tail_pairs;        // pairs that share the split tiles (>= 1)
  float* split_partial;  // [pairs][2 parts][2 CTAs][128 rows][256 columns] fp32 partial accumulators of the split tiles
  int nibble_high_first;
  long long wait_cycles; // limit of every bounded wait, in SM clock cycles
  int withhold;          // failure injection (tests): the producers issue this many contraction blocks fewer than the
                         // consumers expect, so that a bounded wait runs out; 0 in normal use
#ifdef MOLT_PAIR_TRACE
  unsigned long long* trace;   // optional [2 CTAs][12 roles][256 events] timestamps (ns) for pipeline analysis
#endif
  float codebook[16];
};

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// role: 0 producer (TMA issued), 1 MMA (issued), 2 decoder warp 0 (waits done), 3 decoder warp 0 (arrived),
//       4 decoder warp 0 (block decoded, before the wait for the activation tile), 5 decoder warp 0 (loop entry)
#ifdef MOLT_PAIR_TRACE
#define MOLT_TRACE(role, index)                                                                       \
  do {                                                                                                \
    if (p.trace != nullptr && blockIdx.x < 2 && (index) < 256)                                        \
      p.trace[(blockIdx.x * 12 + (role)) * 256 + (index)] = global_ns();                               \
  } while (0)
#else
#define MOLT_TRACE(role, index) do {} while (0)
#endif

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

template <int kSub>
__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int kBand = 8 / kSub;  // 2048 tokens share the L2 while the weight columns stream by
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
  int tail_pairs;                   // the first tail_pairs pairs share them (every part costs a partial tile of traffic)
  int tail_begin, tail_end;         // this pair's range of them
};
struct WorkItem {
  int tile, kb0, kb1;
  int u;                            // position in the tail (split tiles only)
  bool valid;
};
__host__ __device__ __forceinline__ int tail_range_begin(const WorkPlan& w, int pair) {
  const int q = pair < w.tail_pairs ? pair : w.tail_pairs;
  return w.tail_units * q / w.tail_pairs;   // at most pairs^2 x blocks < 2^31 (the host checks)
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
__host__ __device__ __forceinline__ size_t split_slot_offset(int pair, int starts_tile, int sub, int rank, int subs) {
  return ((size_t)((pair * 2 + starts_tile) * subs + sub) * 2 + rank) * BM * BN;
}

template <bool BACKWARD, bool kDense, int kSub, int kLoadStages, int kBStages, int kStoreBufs, int kDecodeGroups>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(pair_threads(kDecodeGroups), 1)
nf4_gemm_sm100_pair_kernel(const __grid_constant__ CUtensorMap map_in, const __grid_constant__ CUtensorMap map_packed,
                           const __grid_constant__ CUtensorMap map_low, const __grid_constant__ CUtensorMap map_ext,
                           const __grid_constant__ CUtensorMap map_out, const __grid_constant__ Params p) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag_s;
  __shared__ WorkPlan plan_s;
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t load0 = base;
  const uint32_t codes0 = load0 + kLoadStages * kLoadStageBytes;
  const uint32_t btile0 = codes0 + (kDense ? 0 : kCodeStages * kPackedBytes);
  const uint32_t store0 = btile0 + kBStages * kTileBBytes;
  const uint32_t lut0 = store0 + kStoreBufs * kStoreBytes;
  const uint32_t bar0 = lut0 + (kDense ? 0 : kLutBytes);
  auto bar_ldfull = [&](int s) { return bar0 + 8u * s; };
  // consumed[g % 8] completes when the MMAs of contraction block number g (counted per CTA across tiles) have
  // finished reading their operands; ONE commit per block releases both the load stage and the B stage, in both
  // CTAs.  Sixteen slots exceed every ring depth, so a waiter can never be lapped.
  constexpr int kConsumedSlots = 16;
  constexpr int kPkBarriers = kDense ? kBStages : kCodeStages;   // the dense variant uses these barriers for its B stages
  static_assert(kLoadStages < kConsumedSlots && kCodeStages < kConsumedSlots && kBStages < kConsumedSlots,
                "ring deeper than the consumed slots");
  // A decode group starts block g once block g - kBStages has been consumed, so it runs at most kBStages blocks ahead
  // of the consumed front.  Its parity waits on the code and activation rings are only meaningful if the previous use
  // of the slot (block g - depth) lies behind that front: both rings must be at least kBStages blocks deep.  (The dense
  // variant has one relay warp that takes the blocks in order, so it cannot run ahead.)
  static_assert(kDense || (kBStages <= kCodeStages && kBStages <= kLoadStages / kSub),
                "B ring deeper than the code ring or the activation ring: a decode group could pass a stale phase");
  auto bar_consumed = [&](int g) { return bar0 + 8u * (kLoadStages + (g & (kConsumedSlots - 1))); };
  auto bar_bfull = [&](int s) { return bar0 + 8u * (kLoadStages + kConsumedSlots + s); };          // used in the leader
  auto bar_accfull = [&](int b) { return bar0 + 8u * (kLoadStages + kConsumedSlots + kBStages + b); };
  auto bar_accempty = [&](int b) { return bar0 + 8u * (kLoadStages + kConsumedSlots + kBStages + 2 + b); };  // leader
  // one low-rank barrier per decode group: a group waits for its own load before it moves on, so a barrier never sees
  // the expect_tx of a second load while the first is still pending (groups run several blocks apart)
  auto bar_ext = [&](int grp) { return bar0 + 8u * (kLoadStages + kConsumedSlots + kBStages + 4 + grp); };
  auto bar_pkfull = [&](int s) { return bar0 + 8u * (kLoadStages + kConsumedSlots + kBStages + 4 + kDecodeGroups + s); };
  auto consumed_parity = [&](int g) { return (uint32_t)((g / kConsumedSlots) & 1); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  volatile int* abort_flag = &abort_flag_s;
  auto wait_on = [&](uint32_t bar, uint32_t parity, int where) {
    return mbar_wait(bar, parity, abort_flag, p.status, where, p.wait_cycles);
  };

  if (threadIdx.x == 0) {
    abort_flag_s = 0;
    plan_s.num_pairs = (int)(gridDim.x >> 1);
    plan_s.pair_id = (int)(blockIdx.x >> 1);
    plan_s.blocks = p.num_kb + (p.ext_steps > 0 ? 1 : 0);
    plan_s.full_tiles = p.full_tiles;
    plan_s.num_tiles = p.tiles_m * p.tiles_n;
    plan_s.tail_units = (plan_s.num_tiles - p.full_tiles) * plan_s.blocks;
    plan_s.tail_pairs = p.tail_pairs;
    plan_s.tail_begin = tail_range_begin(plan_s, plan_s.pair_id);
    plan_s.tail_end = tail_range_begin(plan_s, plan_s.pair_id + 1);
    for (int s = 0; s < kLoadStages; ++s) mbar_init(bar_ldfull(s), 1);
    for (int s = 0; s < kPkBarriers; ++s) mbar_init(bar_pkfull(s), 1);
    for (int g = 0; g < kConsumedSlots; ++g) mbar_init(bar_consumed(g), 1);
    for (int s = 0; s < kBStages; ++s) mbar_init(bar_bfull(s), kDense ? 2 : 8);   // 4 warps of one group (dense: one relay) x 2 CTAs
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_accfull(b), 1);
      mbar_init(bar_accempty(b), 2 * kEpilogueWarps);
    }
    for (int gr = 0; gr < kDecodeGroups; ++gr) mbar_init(bar_ext(gr), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (kLutWords > 0 && !kDense) {
    // byte -> (first element, second element) fp32 codebook values; 16 copies so that lane l reads bank pair l % 16
    float2* lut_ptr = reinterpret_cast<float2*>(smem_dyn + (lut0 - raw));
    for (int i = threadIdx.x; i < 256 * 16; i += blockDim.x) {
      const int byte = i >> 4;
      const int lo = byte & 15, hi = byte >> 4;
      lut_ptr[i] = p.nibble_high_first ? make_float2(p.codebook[hi], p.codebook[lo])
                                       : make_float2(p.codebook[lo], p.codebook[hi]);
    }
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
  // Launched as a programmatic dependent of the kernel before it in the stream: everything above (barriers, TMEM)
  // touches no global memory and may overlap that kernel's tail; nothing below runs before that kernel
  // has completed and its writes are visible.  (Same-box A/B at 4096 tokens: +0.4 % per fwd+bwd step.  Launching the
  // small side kernels the same way was measured too and is slower, -0.7 %, so only the GEMM does it.)
  asm volatile("griddepcontrol.wait;" ::: "memory");

  const int pair_id = blockIdx.x >> 1;
  const WorkPlan& plan = plan_s;   // in shared memory: read at item boundaries only, so it does not occupy registers

  if (warp == kActivationWarp || warp == kCodeWarp) {
    // ================= TMA producers (each CTA loads its own token rows and its own half of the codes) ==========
    // Two warps, one stream each, same block order: packed codes (small, kCodeStages deep, needed first by the
    // decoders) and activation tiles (large, kLoadStages deep, needed last by the MMA).  The slot of block t is free
    // once block t - depth has been consumed.  One thread per warp runs the loop; it is kept short because its
    // iteration time bounds the whole pipeline.
    const bool codes = warp == kCodeWarp;
    static_assert(kLoadStages % kSub == 0, "the activation ring holds whole blocks");
    const int depth = codes ? (kDense ? kBStages : kCodeStages) : kLoadStages / kSub;   // in contraction blocks
    if (lane == 0) {
      // Failure injection for tests: with p.withhold = w the last w blocks of this CTA are never requested, so the
      // consumers' bounded waits run out.  total_blocks is only computed when the injection is on.
      int total_blocks = 0x7fffffff;
      if (p.withhold > 0) {
        total_blocks = 0;
        for (WorkItem it = first_item(plan); it.valid; next_item(plan, it)) total_blocks += it.kb1 - it.kb0;
        total_blocks -= p.withhold;
      }
      int t = 0, stage = 0;                                     // stage: code stage, or first activation stage of the block
      for (WorkItem item = first_item(plan); item.valid && t < total_blocks; next_item(plan, item)) {
        int tm, tn;
        pair_tile_coords<kSub>(item.tile, p.tiles_m, p.tiles_n, tm, tn);
        const int row0 = tm * (2 * BM * kSub) + (int)rank * BM;  // first token row of this CTA (sub-tile s: + s * 2 * BM)
        const int col0 = tn * BN + (int)rank * BNH;             // first B row of this CTA
        bool ok = true;
        for (int kb = item.kb0; kb < item.kb1 && t < total_blocks; ++kb, ++t) {
          if (t >= depth) ok = wait_on(bar_consumed(t - depth), consumed_parity(t - depth), 1);
          if (!ok) break;
          if (codes && kDense) {
            // the B half-tile itself, straight into the B ring (bar_pkfull doubles as "B stage has landed")
            const uint32_t bt = btile0 + (uint32_t)stage * kTileBBytes;
            mbar_expect_tx(bar_pkfull(stage), kTileBBytes);
            if (!BACKWARD) {
              tma_load_2d(bt, &map_packed, kb * BK, col0, bar_pkfull(stage));
            } else {
              tma_load_2d(bt, &map_packed, col0, kb * BK, bar_pkfull(stage));
              tma_load_2d(bt + 8192u, &map_packed, col0 + 64, kb * BK, bar_pkfull(stage));
            }
            if (++stage == kBStages) stage = 0;
          } else if (codes) {
            MOLT_TRACE(8, t);
            if (kb < p.num_kb) {
              const uint32_t pk_dst = codes0 + (uint32_t)stage * kPackedBytes;
              mbar_expect_tx(bar_pkfull(stage), kPackedBytes);
              if (!BACKWARD) tma_load_2d(pk_dst, &map_packed, kb * (BK / 2), col0, bar_pkfull(stage));
              else tma_load_2d(pk_dst, &map_packed, col0 / 2, kb * BK, bar_pkfull(stage));
            } else {
              mbar_arrive(bar_pkfull(stage));   // the low-rank block has no codes; keep the ring's phases in step
            }
            MOLT_TRACE(9, t);
            if (++stage == kCodeStages) stage = 0;
          } else {
#pragma unroll
            for (int sub = 0; sub < kSub; ++sub) {
              const uint32_t a_dst = load0 + (uint32_t)(stage + sub) * kLoadStageBytes;
#ifdef MOLT_PAIR_EXP_HALF_A      // timing experiment: the second activation tile of a block is not loaded (results are wrong)
              if (sub == 1) { mbar_arrive(bar_ldfull(stage + sub)); continue; }
#endif
              mbar_expect_tx(bar_ldfull(stage + sub), kTileABytes);
              if (kb < p.num_kb) tma_load_2d(a_dst, &map_in, kb * BK, row0 + sub * 2 * BM, bar_ldfull(stage + sub));
              else tma_load_2d(a_dst, &map_low, 0, row0 + sub * 2 * BM, bar_ldfull(stage + sub));
            }
            MOLT_TRACE(0, t);
            stage += kSub;
            if (stage == kLoadStages) stage = 0;
          }
        }
        if (!ok) break;
      }
    }
    __syncwarp();
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
        int ls = 0, bs = 0, g = 0, tiles_done = 0;
        uint32_t bphase = 0;
        uint32_t slot_phase[2] = {0u, 0u};     // flips every time an accumulator has been handed to the epilogue
        bool ok = true;
        for (WorkItem item = first_item(plan); item.valid && ok; next_item(plan, item), ++tiles_done) {
          uint32_t accumulate = 0u;
          for (int kb = item.kb0; kb < item.kb1; ++kb) {
            // The decoders of both CTAs arrive on b_full only after their own activation tiles have landed, so
            // this one wait covers both operands in both CTAs.
            ok = wait_on(bar_bfull(bs), bphase, 4);
            if (!ok) break;
            MOLT_TRACE(6, g);
            tc_fence_after();
            const uint32_t b_lo = b_lo0 + (uint32_t)bs * (kTileBBytes >> 4);
#pragma unroll
            for (int sub = 0; sub < kSub; ++sub) {
              // short tiles use the two accumulators in turn, tall tiles use both at once (one per sub-tile)
              const int slot = kSub == 1 ? (tiles_done & 1) : sub;
              if (kb == item.kb0) {   // first use in this tile: the epilogue must have drained the accumulator
                ok = wait_on(bar_accempty(slot), slot_phase[slot] ^ 1u, 2);
                if (!ok) break;
                tc_fence_after();
              }
              const uint32_t d_tmem = tmem_base + (uint32_t)slot * BN;
              const uint32_t a_lo = a_lo0 + (uint32_t)(ls + sub) * (kLoadStageBytes >> 4);
#ifdef MOLT_PAIR_EXP_NO_MMA      // timing experiment: no tensor work, only the commits (results are wrong)
              if (false) {
#else
              if (kb < p.num_kb) {
#endif
                umma_bf16_pair(d_tmem, desc64(a_lo, desc_hi), desc64(b_lo, desc_hi), idesc, accumulate);
#pragma unroll
                for (int ks = 1; ks < BK / 16; ++ks)
                  umma_bf16_pair(d_tmem, desc64(a_lo + ks * 2, desc_hi), desc64(b_lo + ks * kBStep, desc_hi), idesc, 1u);
              } else {   // the low-rank block
                for (int ks = 0; ks < p.ext_steps; ++ks)
                  umma_bf16_pair(d_tmem, desc64(a_lo + ks * 2, desc_hi), desc64(b_lo + ks * kBStep, desc_hi), idesc,
                                 (accumulate | (uint32_t)(ks > 0)));
              }
            }
            if (!ok) break;
            accumulate = 1u;
            MOLT_TRACE(7, g);
            // one commit releases this block's load stages and B stage in both CTAs once the MMAs have read them
            umma_commit_both(bar_consumed(g));
            if (kb == item.kb1 - 1) {
#pragma unroll
              for (int sub = 0; sub < kSub; ++sub) {
                const int slot = kSub == 1 ? (tiles_done & 1) : sub;
                umma_commit_both(bar_accfull(slot));
                slot_phase[slot] ^= 1u;
              }
            }
            MOLT_TRACE(1, g);
            ++g;
            ls += kSub;
            if (ls == kLoadStages) ls = 0;
            if (++bs == kBStages) { bs = 0; bphase ^= 1u; }
          }
        }
      }
      __syncwarp();
    }
  } else if (kDense && is_decode_warp(warp)) {
    // ================= dense variant: one warp relays "this CTA's operands of block g have landed" =================
    if (decode_warp_index(warp) == 0) {
      const uint32_t bfull_remote_base = map_to_cta(bar_bfull(0), 0);
      int g = 0, bs = 0;
      uint32_t bphase = 0;
      bool ok = true;
      for (WorkItem item = first_item(plan); item.valid && ok; next_item(plan, item)) {
        for (int kb = item.kb0; kb < item.kb1 && ok; ++kb, ++g) {
          ok = wait_on(bar_pkfull(bs), bphase, 5);
#pragma unroll
          for (int sub = 0; sub < kSub; ++sub) {
            const int a = g * kSub + sub;
            ok = ok && wait_on(bar_ldfull(a % kLoadStages), (uint32_t)((a / kLoadStages) & 1), 9);
          }
          if (!ok) break;
          __syncwarp();
          if (lane == 0) mbar_arrive_remote(bfull_remote_base + 8u * (uint32_t)bs);
          if (++bs == kBStages) { bs = 0; bphase ^= 1u; }
        }
      }
    }
  } else if (is_decode_warp(warp) && decode_warp_index(warp) < 4 * kDecodeGroups) {
    // ================= NF4 decoders =================
    // Groups of four warps take the contraction blocks in turn (running block number modulo the group count),
    // so the decode latency of one block overlaps the following blocks'.  Inside a group every thread expands one whole
    // 64-element segment (one absmax) per block.
    const int dwarp = decode_warp_index(warp);
    const int dt = dwarp * 32 + lane;                    // 0 for the thread that writes the trace
    const int grp = dwarp >> 2;                          // four consecutive decode warps form a group
    const int u = (dwarp & 3) * 32 + lane;               // 0..127 inside the group
    const uint32_t lut_lane = lut0 + (uint32_t)(lane & 15) * 8u;
    // which table bytes make the bf16 pairs (element 0, element 1) and (element 2, element 3) of four decoded codes
    const uint32_t pick01 = p.nibble_high_first ? 0x4051u : 0x5140u;
    const uint32_t pick23 = p.nibble_high_first ? 0x6273u : 0x7362u;
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
      pair_tile_coords<kSub>(item.tile, p.tiles_m, p.tiles_n, tm, tn);
      const int col0 = tn * BN + (int)rank * BNH;   // first B row (forward: weight row; backward: weight column)
      // forward : absmax[(col0 + i) * kpr + kb]            backward: absmax[(kb * 64 + j) * kpr + col0 / 64 + a]
      long long scale_at, scale_step;   // index of the segment's absmax in block 0, and its step per block
      bool scale_ok;
      if (!BACKWARD) {
        const long long row = (long long)col0 + u;
        scale_ok = row < p.n;
        scale_at = (scale_ok ? row : 0) * kblocks_per_row;
        scale_step = 1;
      } else {
        const long long colblk = (long long)(col0 >> 6) + seg_a;
        scale_ok = colblk < kblocks_per_row;
        scale_at = (long long)seg_j * kblocks_per_row + (scale_ok ? colblk : 0);
        scale_step = (long long)BK * kblocks_per_row;
      }
      // fp32 absmax: one load.  Double-quantised absmax: code2[u8] * absmax2 + offset with a separate multiply and
      // add (the dequantiser's bits); the 8-bit code and the second-level absmax are fetched one round of the
      // prefetch earlier than the table entry, so that no load waits for another.
      const bool nested = p.absmax == nullptr;
      auto load_raw = [&](int kb, uint32_t& code, float& second) {
        code = 0u;
        second = 0.f;
        if (kb < p.num_kb && scale_ok) {
          const long long at = scale_at + (long long)kb * scale_step;
          code = __ldg(p.absmax_u8 + at);
          second = __ldg(p.absmax2 + (at >> p.block2_shift));
        }
      };
      auto resolve = [&](int kb, uint32_t code, float second) -> float {
        return (kb < p.num_kb && scale_ok) ? __fadd_rn(__fmul_rn(__ldg(p.code2 + code), second), p.offset) : 0.f;
      };
      auto load_scale = [&](int kb) -> float {
        if (nested) {
          uint32_t code;
          float second;
          load_raw(kb, code, second);
          return resolve(kb, code, second);
        }
        return (kb < p.num_kb && scale_ok) ? __ldg(p.absmax + scale_at + (long long)kb * scale_step) : 0.f;
      };
      // the group's first block of this item: running block number g_tile + (kb - kb0) is congruent to grp
      const int kb_first = item.kb0 + ((grp - g_tile) % kDecodeGroups + kDecodeGroups) % kDecodeGroups;
      float cur[kPrefetch];
      uint32_t raw_code[kPrefetch];     // nested only: the round after `cur`
      float raw_second[kPrefetch];
#pragma unroll
      for (int q = 0; q < kPrefetch; ++q) {
        cur[q] = load_scale(kb_first + kDecodeGroups * q);
        raw_code[q] = 0u;
        raw_second[q] = 0.f;
        if (nested) load_raw(kb_first + kDecodeGroups * (kPrefetch + q), raw_code[q], raw_second[q]);
      }
      for (int kb0 = kb_first; kb0 < item.kb1 && ok; kb0 += kDecodeGroups * kPrefetch) {
        float nxt[kPrefetch];
#pragma unroll
        for (int q = 0; q < kPrefetch; ++q) {
          const int kb_next = kb0 + kDecodeGroups * (kPrefetch + q);
          if (nested) {
            nxt[q] = resolve(kb_next, raw_code[q], raw_second[q]);
            load_raw(kb_next + kDecodeGroups * kPrefetch, raw_code[q], raw_second[q]);
          } else {
            nxt[q] = load_scale(kb_next);
          }
        }
#pragma unroll
        for (int q = 0; q < kPrefetch; ++q) {
          const int kb = kb0 + kDecodeGroups * q;
          if (kb >= item.kb1 || !ok) continue;
          const float scale = cur[q];
          const int g = g_tile + (kb - item.kb0);
          const int bs = g % kBStages, cs = g % kCodeStages;
          // The sixteen values this segment can take, as byte planes (needs only the absmax: done before the waits).
          SegmentTable table;
          if (kLutWords < 8 && kb < p.num_kb) table = make_segment_table(p.codebook, scale);
          unsigned long long scale2;   // (scale, scale)
          asm("mov.b64 %0, {%1, %1};" : "=l"(scale2) : "f"(scale));
          if (dt == 0) MOLT_TRACE(5, g);
          ok = wait_on(bar_pkfull(cs), (uint32_t)((g / kCodeStages) & 1), 5);
          if (ok && g >= kBStages)   // the block that used this B stage must have been consumed
            ok = wait_on(bar_consumed(g - kBStages), consumed_parity(g - kBStages), 6);
          if (!ok) continue;
          if (dt == 0) MOLT_TRACE(2, g);
          const uint32_t bt = btile0 + bs * kTileBBytes;
          if (kb < p.num_kb) {
#ifndef MOLT_PAIR_EXP_NO_DECODE   // (timing experiment: the decoders only do their waits and arrivals; results are wrong)
            const uint32_t pk = codes0 + (uint32_t)cs * kPackedBytes;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              uint32_t words[4];
              asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(words[0]), "=r"(words[1]), "=r"(words[2]), "=r"(words[3])
                           : "r"(pk + (half == 0 ? src_off0 : src_off1))
                           : "memory");
#pragma unroll
              for (int c = 0; c < 4; ++c) {   // one word = 8 codes = 16 bytes of bf16 = one swizzled chunk of the row
                uint32_t out[4];
                if (4 * half + c < kLutWords) {
                  // table path: one 8-byte lookup per byte gives both fp32 codebook values; two-wide multiply
                  // (mul.rn.f32x2 rounds each lane like a scalar multiply) and one rounding to bf16
#pragma unroll
                  for (int b = 0; b < 4; ++b) {
                    const uint32_t byte = __byte_perm(words[c], 0u, 0x4440u + (uint32_t)b);
                    unsigned long long pair, prod;
                    asm("ld.shared.b64 %0, [%1];" : "=l"(pair) : "r"(lut_lane + byte * 128u));
                    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(prod) : "l"(pair), "l"(scale2));
                    asm("{\n\t.reg .f32 lo, hi;\n\tmov.b64 {lo, hi}, %1;\n\tcvt.rn.bf16x2.f32 %0, hi, lo;\n\t}" : "=r"(out[b]) : "l"(prod));
                  }
                } else {
#ifdef MOLT_PAIR_EXP_NO_ALU      // timing experiment: loads and stores as usual, no decode arithmetic (results are wrong)
                  out[0] = words[c]; out[1] = words[c] ^ 1u; out[2] = words[c] ^ 2u; out[3] = words[c] ^ 3u;
#else
                  decode_word(words[c], table, pick01, pick23, out);
#endif
                }
#ifdef MOLT_PAIR_EXP_NO_STS      // timing experiment: decode, but store only when a value that never occurs shows up
                if (out[0] == 0x12345678u)
#endif
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(bt + dst_off + ((((uint32_t)(4 * half + c)) ^ swz) << 4)),
                             "r"(out[0]), "r"(out[1]), "r"(out[2]), "r"(out[3])
                             : "memory");
              }
            }
#endif
            fence_proxy_async();
            if (dt == 0) MOLT_TRACE(4, g);
          } else {
            // low-rank block: this CTA's half of the ready-made B operand comes by TMA into the B stage
            if (u == 0) {
              if (!BACKWARD) {
                mbar_expect_tx(bar_ext(grp), kTileBBytes);
                tma_load_2d(bt, &map_ext, 0, col0, bar_ext(grp));
              } else {
                mbar_expect_tx(bar_ext(grp), 2u * (uint32_t)p.ext_steps * 16u * 128u);
                tma_load_2d(bt, &map_ext, col0, 0, bar_ext(grp));
                tma_load_2d(bt + 8192u, &map_ext, col0 + 64, 0, bar_ext(grp));
              }
            }
            ok = wait_on(bar_ext(grp), ext_phase, 7);
            if (!ok) continue;
            ext_phase ^= 1u;   // this group's barrier has completed once more
          }
          // this CTA's activation tile must have landed before the block is announced to the MMA thread
#pragma unroll
          for (int sub = 0; sub < kSub; ++sub) {
            const int a = g * kSub + sub;   // running number of the activation tile
            ok = ok && wait_on(bar_ldfull(a % kLoadStages), (uint32_t)((a / kLoadStages) & 1), 9);
          }
          if (!ok) continue;
          __syncwarp();
          if (lane == 0) mbar_arrive_remote(bfull_remote_base + 8u * (uint32_t)bs);
          if (dt == 0) MOLT_TRACE(3, g);
        }
#pragma unroll
        for (int q = 0; q < kPrefetch; ++q) cur[q] = nxt[q];
      }
    }
  } else if (warp < kEpilogueWarps) {
    // ================= epilogue: TMEM -> bf16 -> shared -> TMA store (own 128 token rows) =================
    const int row = warp * 32 + lane;
    const uint32_t accempty_remote_base = map_to_cta(bar_accempty(0), 0);
    uint32_t full_phase[2] = {0u, 0u};     // flips every time an accumulator has been drained
    int store_buf = 0, tiles_done = 0;
    bool ok = true;
    for (WorkItem item = first_item(plan); item.valid && ok; next_item(plan, item), ++tiles_done) {
      int tm, tn;
      pair_tile_coords<kSub>(item.tile, p.tiles_m, p.tiles_n, tm, tn);
#pragma unroll
      for (int sub = 0; sub < kSub; ++sub) {
      const int acc = kSub == 1 ? (tiles_done & 1) : sub;   // accumulator of this sub-tile
      const int row0 = tm * (2 * BM * kSub) + sub * 2 * BM + (int)rank * BM;
      ok = wait_on(bar_accfull(acc), full_phase[acc], 8);
      if (!ok) break;
      full_phase[acc] ^= 1u;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)acc * BN;
      if (item.tile >= plan.full_tiles) {
        // ---- part of a split tile: the fp32 accumulator goes to this pair's slot, row-major ----
        float* part = p.split_partial + split_slot_offset(pair_id, item.kb0 == 0 ? 1 : 0, sub, (int)rank, kSub) + (size_t)row * BN;
        const bool row_valid = (long long)row0 + row < p.m;   // the fix-up kernel never reads rows past the end
        for (int cg = 0; cg < BN / 32; ++cg) {
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
        continue;
      }
      for (int cg = 0; cg < BN / 64; ++cg) {
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
#ifndef MOLT_PAIR_EXP_NO_STORE   // (timing experiment: the result never leaves the SM)
          if (row0 < p.m) tma_store_2d(&map_out, stage_addr, tn * BN + cg * 64, row0);
#endif
          tma_store_commit();
        }
        if (kStoreBufs == 2) store_buf ^= 1;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(accempty_remote_base + 8u * (uint32_t)acc);
      }   // sub-tiles
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
                                                          int tiles_n, int subs, long long m, long long out_cols,
                                                          __nv_bfloat16* __restrict__ out) {
  const int tail_tile = blockIdx.y;
  const int tile = plan.full_tiles + tail_tile;
  int tm, tn;
  if (subs == 2) pair_tile_coords<2>(tile, tiles_m, tiles_n, tm, tn);
  else pair_tile_coords<1>(tile, tiles_m, tiles_n, tm, tn);
  const int idx = blockIdx.x * 256 + threadIdx.x;          // 2 * BM * subs rows x BN / 8 column groups
  const int r = idx / (BN / 8), cgroup = idx % (BN / 8);   // row inside the tile: sub-tile, CTA, row of the CTA
  const long long row = (long long)tm * (2 * BM * subs) + r, col = (long long)tn * BN + cgroup * 8;
  if (row >= m || col >= out_cols) return;
  const int sub = r / (2 * BM), cta = (r % (2 * BM)) / BM, local = r % BM;
  const int unit0 = tail_tile * plan.blocks, unit1 = unit0 + plan.blocks;
  int first = (int)(((long long)unit0 * plan.tail_pairs) / plan.tail_units);   // the pair whose range holds unit0
  while (first + 1 < plan.tail_pairs && tail_range_begin(plan, first + 1) <= unit0) ++first;
  while (first > 0 && tail_range_begin(plan, first) > unit0) --first;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int c = first; c < plan.tail_pairs && tail_range_begin(plan, c) < unit1; ++c) {
    const int start = tail_range_begin(plan, c) > unit0 ? tail_range_begin(plan, c) : unit0;
    const float* src = partial + split_slot_offset(c, start == unit0 ? 1 : 0, sub, cta, subs) + (size_t)local * BN + cgroup * 8;
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
static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  }
  return fn;
}

int make_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, const void* ptr, uint64_t inner, uint64_t outer,
                    uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle,
                    const char* what) {
  auto fn = encode_fn();
  if (fn == nullptr) return fail(MOLT_E_RUNTIME, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult rc = fn(map, dtype, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return fail(MOLT_E_RUNTIME, "cuTensorMapEncodeTiled(%s) failed with code %d", what, (int)rc);
  return MOLT_OK;
}

bool sm100_gemm_supported(const WeightView& w, int rank) {
  return w.blocksize == 64 && w.k % 64 == 0 && w.n % 64 == 0 && rank <= 64;
}

// Scratch for splitting the last wave: two fp32 partial tiles (of the tall kind) per CTA pair.
size_t sm100_split_bytes() {
  return pair::split_slot_offset(sm_count() / 2, 0, 0, 0, 2) * sizeof(float);
}

int run_pair_gemm(bool backward, bool dense, pair::Params& p, const CUtensorMap& map_in, const CUtensorMap& map_packed,
                  const CUtensorMap& map_low, const CUtensorMap& map_ext, const CUtensorMap& map_out,
                  __nv_bfloat16* out, long long m, long long out_cols, void* split_ws, int flags, cudaStream_t s);

int sm100_gemm(bool backward, const WeightView& w, const float* absmax_f32, const __nv_bfloat16* in,
               const __nv_bfloat16* low, const __nv_bfloat16* ext, int rp, __nv_bfloat16* out, long long m,
               void* split_ws, int flags, cudaStream_t s) {
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
  p.absmax_u8 = nullptr;
  p.absmax2 = nullptr;
  p.code2 = nullptr;
  p.offset = 0.f;
  p.block2_shift = 0;
  if (absmax_f32 == nullptr) {   // the decoders read the double-quantised absmax themselves
    if (w.absmax_kind != MOLT_ABSMAX_NESTED || w.block2_shift < 0)
      return fail(MOLT_E_RUNTIME, "tcgen05 GEMM: no fp32 absmax given and the weight's own cannot be read in the kernel");
    p.absmax_u8 = reinterpret_cast<const uint8_t*>(w.absmax);
    p.absmax2 = w.absmax2;
    p.code2 = w.code2;
    p.offset = w.offset;
    p.block2_shift = w.block2_shift;
  }
  p.m = m;
  p.n = w.n;
  p.k = w.k;
  p.num_kb = (int)(contraction / BK);
  p.ext_steps = has_low ? rp / 16 : 0;
  p.nibble_high_first = w.nibble_order == MOLT_NIBBLE_HIGH_FIRST ? 1 : 0;
  for (int i = 0; i < 16; ++i) p.codebook[i] = w.codebook[i];
  return run_pair_gemm(backward, false, p, map_in, map_packed, map_low, map_ext, map_out, out, m, out_cols, split_ws,
                       flags, s);
}

// out[m, n] = in[m, k] . weight[n, k]^T (forward) or out[m, k] = in[m, n] . weight[n, k] (backward) for a dense bf16
// weight: the same kernel with its B tiles loaded ready-made (n, k multiples of 64).
int sm100_dense_gemm(bool backward, const __nv_bfloat16* weight, long long n, long long k, const __nv_bfloat16* in,
                     __nv_bfloat16* out, long long m, void* split_ws, int flags, cudaStream_t s) {
  using namespace pair;
  if (n % 64 != 0 || k % 64 != 0 || (reinterpret_cast<uintptr_t>(weight) & 15) != 0)
    return fail(MOLT_E_CAPABILITY, "dense tcgen05 GEMM: n and k must be multiples of 64 and the weight 16-byte aligned");
  const long long contraction = backward ? n : k;
  const long long out_cols = backward ? k : n;
  CUtensorMap map_in, map_weight, map_out;
  if (int rc = make_tensor_map(&map_in, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, in, contraction, m, contraction * 2, BK, BM,
                               CU_TENSOR_MAP_SWIZZLE_128B, "activations"))
    return rc;
  // forward: K-major half-tiles of 128 weight rows x 64 columns; backward: MN-major, two boxes of 64 rows x 64 columns
  if (int rc = make_tensor_map(&map_weight, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, weight, k, n, k * 2, 64,
                               backward ? 64 : BNH, CU_TENSOR_MAP_SWIZZLE_128B, "dense weight"))
    return rc;
  if (int rc = make_tensor_map(&map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, out, out_cols, m, out_cols * 2, 64, BM,
                               CU_TENSOR_MAP_SWIZZLE_128B, "output"))
    return rc;
  Params p;
  p.packed = nullptr;
  p.absmax = nullptr;
  p.absmax_u8 = nullptr;
  p.absmax2 = nullptr;
  p.code2 = nullptr;
  p.offset = 0.f;
  p.block2_shift = 0;
  p.m = m;
  p.n = n;
  p.k = k;
  p.num_kb = (int)(contraction / BK);
  p.ext_steps = 0;
  p.nibble_high_first = 0;
  for (int i = 0; i < 16; ++i) p.codebook[i] = 0.f;
  return run_pair_gemm(backward, true, p, map_in, map_weight, map_in, map_in, map_out, out, m, out_cols, split_ws, flags, s);
}

// Schedule and launch, shared by the NF4 and the dense variant.
int run_pair_gemm(bool backward, bool dense, pair::Params& p, const CUtensorMap& map_in, const CUtensorMap& map_packed,
                  const CUtensorMap& map_low, const CUtensorMap& map_ext, const CUtensorMap& map_out,
                  __nv_bfloat16* out, long long m, long long out_cols, void* split_ws, int flags, cudaStream_t s) {
  using namespace pair;
  p.status = device_status_word();
  if (p.status == nullptr) return fail(MOLT_E_RUNTIME, "tcgen05 GEMM: no device status word");
  p.tiles_n = (int)((out_cols + BN - 1) / BN);
  p.wait_cycles = wait_limit_cycles();
  p.withhold = take_withheld_blocks();
#ifdef MOLT_PAIR_TRACE
  {
    const char* tr = getenv("MOLT_B200_TRACE_PTR");   // device pointer (decimal) of a 24 KB trace buffer
    p.trace = tr != nullptr ? reinterpret_cast<unsigned long long*>(strtoull(tr, nullptr, 10)) : nullptr;
  }
#endif

  const long long all_pairs = sm_count() / 2;
  const long long blocks = p.num_kb + (p.ext_steps > 0 ? 1 : 0);
  // Schedule: tile height (short = 256 tokens per pair, tall = 512: two MMAs per decoded B tile) and whether the tiles
  // of a last, partial wave are split along the contraction.  Every admissible combination is costed with figures
  // measured on B200 (14336 x 4096 and 8960 x 1536 weights): a tile takes 0.58 us (short) or 0.80 us (tall) per
  // contraction block, a tall tile 4 us more for its partly exposed epilogue; splitting costs 38 us (short) or 50 us
  // (tall) for the fp32 partial tiles and the extra launch.  The cheapest estimate wins.
  int subs = 1;
  bool split = false;
  {
    const bool may_split = split_ws != nullptr && !(flags & kGemmNoSplit);
    const bool forced_split = (flags & kGemmForceSplit) != 0;
    double best = -1.0;
    for (int cand = 1; cand <= 2; ++cand) {
      if (cand == 2 && ((flags & kGemmShortTiles) || m <= 2 * BM)) continue;
      if (cand == 1 && (flags & kGemmTallTiles) && m > 0) continue;
      const long long tiles_c = ((m + 2 * BM * cand - 1) / (2 * BM * cand)) * p.tiles_n;
      const double tile_us = blocks * (cand == 2 ? 0.80 : 0.58) + (cand == 2 ? 4.0 : 0.0);
      const long long full = tiles_c / all_pairs, rem = tiles_c % all_pairs;
      const double plain_us = (double)(full + (rem != 0 ? 1 : 0)) * tile_us;
      // a split needs whole waves in front of it, at least one block per pair, and indices that fit 32 bits
      const bool can_split = may_split && full >= 1 && rem != 0 && rem * blocks >= all_pairs &&
                             rem * blocks * all_pairs < (1LL << 30);
      const double split_us = (double)full * tile_us + (double)rem / (double)all_pairs * tile_us + (cand == 2 ? 50.0 : 38.0);
      const bool take_split = can_split && (forced_split || split_us < plain_us);
      const double est = take_split ? split_us : plain_us;
      if (best < 0.0 || est < best) {
        best = est;
        subs = cand;
        split = take_split;
      }
    }
  }
  p.tiles_m = (int)((m + 2 * BM * subs - 1) / (2 * BM * subs));
  const long long tiles = (long long)p.tiles_m * p.tiles_n;
  long long pairs = all_pairs;
  if (tiles < pairs) pairs = tiles;
  // Whole waves run the static schedule; the tiles of a split last wave leave the kernel as fp32 partial tiles.
  p.full_tiles = (int)tiles;
  p.split_partial = nullptr;
  p.tail_pairs = (int)pairs;
  if (split) {
    p.full_tiles = (int)(tiles - tiles % pairs);
    p.split_partial = reinterpret_cast<float*>(split_ws);
#ifndef MOLT_PAIR_EXP_ALL_TAIL_PAIRS
    // How many pairs share the split tiles: every part of a tile is written and read back as a whole fp32 tile
    // (512 KB tall, 256 KB short: about 0.19 / 0.10 us of HBM time), so a few blocks more per pair can be cheaper than
    // a part more.  A pair's range may span at most two tiles, hence at least `rem` pairs.
    const long long rem = tiles % pairs, units = rem * blocks;
    const double block_us = subs == 2 ? 0.80 : 0.58, part_us = subs == 2 ? 0.19 : 0.10;
    double best_us = -1.0;
    for (long long tp = rem; tp <= pairs; ++tp) {
      const double us = (double)((units + tp - 1) / tp) * block_us + (double)(tp + rem) * part_us;
      if (best_us < 0.0 || us < best_us) {
        best_us = us;
        p.tail_pairs = (int)tp;
      }
    }
#endif
  }
  const int grid = (int)pairs * 2;
  constexpr int BS = kBStagesDefault, SB = 1, GR = kDecodeGroupsDefault;
  constexpr int LS1 = kLoadStagesDefault;                 // short tiles: one activation tile per block
  #ifndef MOLT_PAIR_TALL_LS
#define MOLT_PAIR_TALL_LS (kLutWords > 0 ? 6 : 8)
#define MOLT_PAIR_TALL_BS 3
#endif
  constexpr int LS2 = MOLT_PAIR_TALL_LS, BS2 = MOLT_PAIR_TALL_BS;     // tall tiles: two per block (four blocks deep; three beside a table), B ring of three
  constexpr int DLS1 = 6, DBS1 = 7, DLS2 = 8, DBS2 = 5;   // dense variant: no code ring and no table, deeper B rings
  static_assert(smem_bytes(LS2, BS2, SB) <= 232448 && smem_bytes(LS1, BS, SB) <= 232448 &&
                smem_bytes(DLS1, DBS1, SB, true) <= 232448 && smem_bytes(DLS2, DBS2, SB, true) <= 232448,
                "shared memory budget");
  static thread_local bool configured[64][2][2][2] = {};
  int dev = 0;
  MOLT_CUDA(cudaGetDevice(&dev));
  const bool need_config = dev >= 0 && dev < 64 && !configured[dev][dense ? 1 : 0][backward ? 1 : 0][subs - 1];
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)pair_threads(GR));
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
#define MOLT_PAIR_LAUNCH(BWD, DENSE, SUB, LS, BSTAGES)                                                       \
  do {                                                                                                       \
    cfg.dynamicSmemBytes = smem_bytes(LS, BSTAGES, SB, DENSE);                                               \
    if (need_config)                                                                                         \
      MOLT_CUDA(cudaFuncSetAttribute(nf4_gemm_sm100_pair_kernel<BWD, DENSE, SUB, LS, BSTAGES, SB, GR>,       \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize,                            \
                                     (int)smem_bytes(LS, BSTAGES, SB, DENSE)));                              \
    MOLT_CUDA(cudaLaunchKernelEx(&cfg, nf4_gemm_sm100_pair_kernel<BWD, DENSE, SUB, LS, BSTAGES, SB, GR>,     \
                                 map_in, map_packed, map_low, map_ext, map_out, p));                         \
  } while (0)
  if (!dense) {
    if (backward && subs == 2) MOLT_PAIR_LAUNCH(true, false, 2, LS2, BS2);
    else if (backward) MOLT_PAIR_LAUNCH(true, false, 1, LS1, BS);
    else if (subs == 2) MOLT_PAIR_LAUNCH(false, false, 2, LS2, BS2);
    else MOLT_PAIR_LAUNCH(false, false, 1, LS1, BS);
  } else {
    if (backward && subs == 2) MOLT_PAIR_LAUNCH(true, true, 2, DLS2, DBS2);
    else if (backward) MOLT_PAIR_LAUNCH(true, true, 1, DLS1, DBS1);
    else if (subs == 2) MOLT_PAIR_LAUNCH(false, true, 2, DLS2, DBS2);
    else MOLT_PAIR_LAUNCH(false, true, 1, DLS1, DBS1);
  }
#undef MOLT_PAIR_LAUNCH
  if (need_config) configured[dev][dense ? 1 : 0][backward ? 1 : 0][subs - 1] = true;
  if (int rc = launch_status("nf4_gemm_sm100_pair_kernel")) return rc;
  if (p.full_tiles < tiles) {
    WorkPlan plan;
    plan.num_pairs = (int)pairs;
    plan.pair_id = 0;
    plan.blocks = p.num_kb + (p.ext_steps > 0 ? 1 : 0);
    plan.full_tiles = p.full_tiles;
    plan.num_tiles = (int)tiles;
    plan.tail_units = (int)(tiles - p.full_tiles) * plan.blocks;
    plan.tail_pairs = p.tail_pairs;
    plan.tail_begin = plan.tail_end = 0;
    dim3 fgrid((unsigned)(2 * BM * subs * (BN / 8) / 256), (unsigned)(tiles - p.full_tiles));
    split_fixup_kernel<<<fgrid, 256, 0, s>>>(p.split_partial, plan, p.tiles_m, p.tiles_n, subs, m, out_cols, out);
    return launch_status("split_fixup_kernel");
  }
  return MOLT_OK;
}

}  // namespace molt
