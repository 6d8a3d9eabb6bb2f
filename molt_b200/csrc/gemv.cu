// Small-token (M <= 16) NF4 + LoRA forward.  The packed weight is streamed from HBM exactly once.
//
// Work split: the grid is (CTAs per K-group, K-groups); a K-group is up to 32 absmax blocks (2048 columns) and
// a CTA walks over 16-row chunks of W inside its K-group.  Up to sixteen streaming warps each own a fixed K-slice
// of 2 absmax blocks (128 columns) and keep the matching X fragments in registers for their whole life.  Every
// streaming warp runs its own load pipeline: per chunk it copies its 16 x 64 bytes of packed codes and its 32
// absmax values into a private ring of shared-memory stages with cp.async (several chunks ahead, completion by
// cp.async groups), so the load path needs no barrier between warps and the warps drift apart instead of
// alternating between a load phase and a compute phase in lockstep.  Codes are expanded two at a time through a
// byte-indexed table of bf16 pairs that is replicated once per lane (256 bytes per entry, bank = lane, so
// lookups never conflict; one byte-permute builds the table offset from a code byte and the lane) and fed to
// mma.sync m16n8k16 with the tokens as the M dimension.  The MMA runs on the unscaled code values; each absmax
// block's partial sum is multiplied by its fp32 absmax afterwards (nested absmax: each lane resolves one value
// per chunk and the quads fetch theirs by shuffle), so no per-element multiply is needed.  The streaming warps
// drop their K-slice sums into a ring of buffers and two reducing warps add them in warp order (deterministic)
// and write an fp32 partial per K-group.  The low-rank input T = X . A^T rides along: the X fragments are
// already in registers, so the first CTAs of every K-group run a few more MMAs against bf16(A) and write their
// K-group's part of T.  A small second kernel adds the K-groups, rounds T to bf16, adds the low-rank term and
// rounds to bf16.  The only waits between warps are mbarrier waits of the sum ring; they have a time limit that
// reports to the device status word.
#include <cstdlib>

#include "sm100_ptx.cuh"

namespace molt {

constexpr int kGemvMaxWarps = 16;
constexpr int kGemvBlocksPerWarp = 2;   // absmax blocks (of 64 columns) per warp
constexpr int kGemvChunkRows = 16;
constexpr int kGemvRing = 2;            // buffers between the streaming warps and the reducing warps
constexpr int kGemvLutBytes = 256 * 256;   // [256 entries][64 lane positions, 32 used] bf16x2
constexpr int kGemvStageBytes = 1024 + 128 + 64;   // codes [16 rows][64 B] | 32 absmax words | 16 raw words (nested)
constexpr int kGemvStages = 6;   // depth of every warp's private ring (chunks in flight + the one being read)
constexpr int kGemvSmemLimit = 227 * 1024;

struct GemvParams {
  WeightView w;
  const __nv_bfloat16* x;   // [m, k]
  const float* lora_a;      // [rank, k] fp32
  float* t_partial;         // [kgroups][16][64] fp32: every K-group's part of x . bf16(A)^T
  int rank;
  int m;
  int nblk;                 // k / 64
  int kgroups;
  int warps_per_cta;        // streaming warps
  int32_t* status;
  float* partial;           // [kgroups][16][n] fp32
  int debug;                // with -DMOLT_GEMV_TRACE: bit 0 skips the decode + MMA work
  long long* trace;         // optional [8 roles][64] clock64 stamps of one CTA; only with -DMOLT_GEMV_TRACE
};

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// d = a . b + c with c given separately (used with c = 0 for the first MMA of an absmax block)
__device__ __forceinline__ void mma_16816_c(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                            const float (&c)[4]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

#ifdef MOLT_GEMV_TRACE
#define GEMV_TRACE(role, index)                                                                  \
  do {                                                                                           \
    if (p.trace != nullptr && blockIdx.x == 3 && blockIdx.y == 0 && (threadIdx.x & 31) == 0 && (index) < 64) \
      p.trace[(role) * 64 + (index)] = clock64();                                                \
  } while (0)
#else
#define GEMV_TRACE(role, index) do {} while (0)
#endif

__device__ __forceinline__ void named_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's most recent cp.async groups are still in flight.
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <bool NESTED>
__global__ void __launch_bounds__((kGemvMaxWarps + 2) * 32, 1) nf4_gemv_kernel(const __grid_constant__ GemvParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  // pair table | [ring][warps][2 n-tiles][32 lanes][4] K-slice sums | [warps][32 lanes][4] low-rank sums | code2 |
  // barriers | [warps][stages] private load stages
  const int warps = p.warps_per_cta;   // streaming warps; the two warps after them reduce
  unsigned char* lut_bytes = smem_raw;
  float* red = reinterpret_cast<float*>(smem_raw + kGemvLutBytes);
  float* t_red = red + kGemvRing * warps * 256;     // [warps][32][4]
  float* code2_s = t_red + warps * 128;             // [256]
  uint64_t* bars = reinterpret_cast<uint64_t*>(code2_s + 256);
  const uint32_t bar0 = smem_u32(bars);
  auto red_full_bar = [&](int s) { return bar0 + 8u * s; };
  auto red_empty_bar = [&](int s) { return bar0 + 8u * (kGemvRing + s); };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * kGemvRing);
  unsigned char* stage_mem = reinterpret_cast<unsigned char*>(bars + 8);   // 64 bytes hold the barriers and the flag

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int kgroup = blockIdx.y;
  const int blk_first = kgroup * warps * kGemvBlocksPerWarp;                      // first absmax block of this K-group
  const long long row_bytes = p.w.k / 2;
  const int chunks = (int)(p.w.n / kGemvChunkRows);
  const int stride = gridDim.x;
  const int total = (chunks - (int)blockIdx.x + stride - 1) / stride;             // chunks of this CTA

  if (warp == 0) GEMV_TRACE(7, 0);
  if (threadIdx.x == 0) {
    for (int s = 0; s < kGemvRing; ++s) {
      mbar_init(red_full_bar(s), warps);
      mbar_init(red_empty_bar(s), 2);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }

  // ---- this warp's K-slice ----
  const int blk0 = blk_first + warp * kGemvBlocksPerWarp;
  int nb = p.nblk - blk0;
  if (nb < 0 || warp >= warps) nb = 0;
  if (nb > kGemvBlocksPerWarp) nb = kGemvBlocksPerWarp;
  // A warp whose K-slice has fewer than two blocks reads a valid block in place of the missing one; its X fragments
  // for the missing block are zero, so that block adds zero.  Nothing is predicated inside the loop.
  const int blkc = nb > 0 ? blk0 : 0;               // first block actually read
  const int b1 = nb == kGemvBlocksPerWarp ? 1 : 0;  // offset of the second block, in blocks

  // ---- private load pipeline (streaming warps) ----
  // codes: lane copies 16-byte granule c = lane % 4 of rows lane / 4 and lane / 4 + 8; a granule of row r sits at
  // position c ^ (2 * ((r / 2) % 2)) of the row's 64 bytes, which makes the 8-byte fragment reads conflict-free
  const uint32_t my_stages = smem_u32(stage_mem) + (uint32_t)(warp * kGemvStages) * kGemvStageBytes;
  const int cp_row = lane >> 2, cp_gran = lane & 3;
  const bool cp_on = warp < warps && cp_gran < 2 * (b1 + 1);    // granules of blocks this warp really reads
  const uint32_t cp_dst = (uint32_t)(cp_row * 64 + ((cp_gran ^ (((cp_row >> 1) & 1) << 1)) * 16));
  const long long chunk_bytes = (long long)kGemvChunkRows * row_bytes;
  const uint8_t* code_src = p.w.packed + ((long long)blockIdx.x * kGemvChunkRows + cp_row) * row_bytes +
                            (long long)blkc * 32 + cp_gran * 16;
  // absmax: lane copies the value of (row lane / 2, block lane % 2)
  const int sc_row = lane >> 1, sc_b = (lane & 1) * b1;
  const long long sc_index0 = ((long long)blockIdx.x * kGemvChunkRows + sc_row) * p.nblk + blkc + sc_b;
  const long long sc_chunk = (long long)kGemvChunkRows * p.nblk;
  const long long code_step = (long long)stride * chunk_bytes, sc_step = (long long)stride * sc_chunk;
  const uint8_t* code_next = code_src;   // this lane's sources for the next chunk to request
  long long sc_next = sc_index0;
  // for the nested form, lanes 0..15 also copy the aligned word that holds row `lane`'s two codes; the rows' segments
  // start on 2-byte boundaries of words because nblk % 4 == 0 (host-checked)
  long long raw_next = (((long long)blockIdx.x * kGemvChunkRows + (lane & 15)) * p.nblk + blkc) & ~3LL;
  int requested = 0;
  auto issue = [&](int stage) {   // requests this CTA's next chunk into `stage`
    if (requested < total) {
      const uint32_t base = my_stages + (uint32_t)stage * kGemvStageBytes;
      if (cp_on) {
        cp_async_16(base + cp_dst, code_next);
        cp_async_16(base + cp_dst + 512, code_next + 8 * row_bytes);
      }
      if (!NESTED) {
        cp_async_4(base + 1024 + lane * 4, reinterpret_cast<const float*>(p.w.absmax) + sc_next);
      } else {
        cp_async_4(base + 1024 + lane * 4, p.w.absmax2 + (sc_next >> p.w.block2_shift));
        if (lane < kGemvChunkRows)
          cp_async_4(base + 1024 + 128 + lane * 4, reinterpret_cast<const uint8_t*>(p.w.absmax) + raw_next);
      }
      code_next += code_step;
      sc_next += sc_step;
      raw_next += sc_step;
      ++requested;
    }
    cp_async_commit();
  };

  // ---- X fragments ----
  uint32_t xa[kGemvBlocksPerWarp][4][4];
#pragma unroll
  for (int b = 0; b < kGemvBlocksPerWarp; ++b)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long col = (long long)(blk0 + b) * 64 + 16 * t + 4 * j;
      uint2 lo = make_uint2(0, 0), hi = make_uint2(0, 0);
      if (b < nb) {
        if (g < p.m) lo = __ldg(reinterpret_cast<const uint2*>(p.x + (long long)g * p.w.k + col));
        if (g + 8 < p.m) hi = __ldg(reinterpret_cast<const uint2*>(p.x + (long long)(g + 8) * p.w.k + col));
      }
      xa[b][j][0] = lo.x; xa[b][j][1] = hi.x; xa[b][j][2] = lo.y; xa[b][j][3] = hi.y;
    }

  // the first chunks are requested behind the X loads, so that X (L2 hits) does not queue behind them
  if (warp < warps)
    for (int j = 0; j < kGemvStages - 1; ++j) issue(j);

  // ---- tables: one (byte, 8 lanes) item per step ----
  {
    const int builders = (warps + 2) * 32;
    for (int i = threadIdx.x; i < 256 * 4; i += builders) {
      const int byte = i >> 2;
      const int first = p.w.nibble_order == MOLT_NIBBLE_LOW_FIRST ? (byte & 15) : (byte >> 4);
      const int second = p.w.nibble_order == MOLT_NIBBLE_LOW_FIRST ? (byte >> 4) : (byte & 15);
      const uint32_t pair = pack_bf16x2(p.w.codebook[first], p.w.codebook[second]);
      uint4* dst = reinterpret_cast<uint4*>(lut_bytes + byte * 256 + (i & 3) * 32);
      dst[0] = make_uint4(pair, pair, pair, pair);
      dst[1] = make_uint4(pair, pair, pair, pair);
    }
    if (NESTED)
      for (int i = threadIdx.x; i < 256; i += builders) code2_s[i] = p.w.code2[i];
  }

  // ---- low-rank input: CTA x of a K-group computes rows 8x .. 8x+7 of A against this K-group's columns ----
  const int t_tile = blockIdx.x;                      // 8-row tile of A handled by this CTA (if any)
  const bool t_owner = t_tile * 8 < p.rank;
  if (t_owner && warp < warps) {
    float tacc[4] = {0.f, 0.f, 0.f, 0.f};
    const int r = t_tile * 8 + g;
#pragma unroll
    for (int b = 0; b < kGemvBlocksPerWarp; ++b)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float4 av = make_float4(0.f, 0.f, 0.f, 0.f);
        if (b < nb && r < p.rank)
          av = __ldg(reinterpret_cast<const float4*>(p.lora_a + (long long)r * p.w.k + (long long)(blk0 + b) * 64 + 16 * t + 4 * j));
        mma_16816(tacc, xa[b][j], pack_bf16x2(av.x, av.y), pack_bf16x2(av.z, av.w));
      }
    *reinterpret_cast<float4*>(t_red + (warp * 32 + lane) * 4) = make_float4(tacc[0], tacc[1], tacc[2], tacc[3]);
  }
  __syncthreads();   // tables, barriers and the low-rank sums are in place

  if (warp >= warps) {
    // ---- reducing warps (one per 8-row tile): add the K-slices of each chunk in warp order, write the fp32 partial ----
    const int nt = warp - warps;
    if (t_owner && nt == 0) {
      // lane (g, t) holds tokens g, g + 8 and rows 2t, 2t + 1 of the tile: add the warps' K-slices in warp order
      float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int wv = 0; wv < warps; ++wv) {
        const float4 v = *reinterpret_cast<const float4*>(t_red + (wv * 32 + lane) * 4);
        sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
      }
      float* dst = p.t_partial + (long long)kgroup * 16 * 64 + t_tile * 8 + 2 * t;
      *reinterpret_cast<float2*>(dst + g * 64) = make_float2(sum.x, sum.y);
      *reinterpret_cast<float2*>(dst + (g + 8) * 64) = make_float2(sum.z, sum.w);
    }
    int buf = 0, phase = 0, tr_it = 0;
    for (int chunk = blockIdx.x; chunk < chunks; chunk += stride) {
      if (!mbar_wait(red_full_bar(buf), phase, abort_flag, p.status, 42)) return;
      if (nt == 0) GEMV_TRACE(5, tr_it + 1);
      const float* src = red + (size_t)buf * warps * 256 + (nt * 32 + lane) * 4;
      float4 v[kGemvMaxWarps];
#pragma unroll
      for (int wv = 0; wv < kGemvMaxWarps; ++wv)
        v[wv] = wv < warps ? *reinterpret_cast<const float4*>(src + wv * 256) : make_float4(0.f, 0.f, 0.f, 0.f);
      float4 sum = v[0];
#pragma unroll
      for (int wv = 1; wv < kGemvMaxWarps; ++wv) {
        sum.x += v[wv].x; sum.y += v[wv].y; sum.z += v[wv].z; sum.w += v[wv].w;
      }
      __syncwarp();                                     // every lane's loads have been consumed by its sums
      if (lane == 0) mbar_arrive(red_empty_bar(buf));   // the buffer may be overwritten
      // lane (g, t) holds tokens g and g + 8, rows 2t and 2t + 1 of the 8-row tile
      float* dst = p.partial + (long long)kgroup * 16 * p.w.n + (long long)chunk * kGemvChunkRows + 2 * t + nt * 8;
      *reinterpret_cast<float2*>(dst + (long long)g * p.w.n) = make_float2(sum.x, sum.y);
      *reinterpret_cast<float2*>(dst + (long long)(g + 8) * p.w.n) = make_float2(sum.z, sum.w);
      if (nt == 0) GEMV_TRACE(6, tr_it + 1);
      ++tr_it;
      if (++buf == kGemvRing) { buf = 0; phase ^= 1; }
    }
    return;
  }

  // ---- streaming warps ----
  // fragment reads: lane (g, t) takes bytes 8 * (t % 2) .. + 7 of granule 2b + t / 2 of rows g and g + 8
  uint32_t frag_off[kGemvBlocksPerWarp];
#pragma unroll
  for (int b = 0; b < kGemvBlocksPerWarp; ++b)
    frag_off[b] = (uint32_t)(g * 64 + (((2 * b * b1 + (t >> 1)) ^ (((g >> 1) & 1) << 1)) * 16) + (t & 1) * 8);
  const uint32_t lane4 = (uint32_t)lane * 4u;
  const int raw_off = 1024 + 128 + sc_row * 4 + (blkc & 3) + sc_b;   // this lane's code in the raw words (nested)
  // table offset of code byte `which` of q: (byte << 8) | (lane * 4), built by one byte permute
  auto lookup = [&](uint32_t q, uint32_t selector) -> uint32_t {
    return *reinterpret_cast<const uint32_t*>(lut_bytes + __byte_perm(q, lane4, selector));
  };
  const float zero[4] = {0.f, 0.f, 0.f, 0.f};
  const unsigned char* my_stage_ptr = stage_mem + (size_t)(warp * kGemvStages) * kGemvStageBytes;
  int stage = 0, fill = kGemvStages - 1, buf = 0, red_phase = 0, red_wrapped = 0;
  if (warp == 0) GEMV_TRACE(2, 0);
  for (int it = 0; it < total; ++it) {
    issue(fill);                          // into the stage the previous iteration read
    if (++fill == kGemvStages) fill = 0;
    cp_async_wait<kGemvStages - 1>();     // this lane's copies of chunk `it` have landed ...
    __syncwarp();                         // ... and so have the other lanes'
    if (warp == 0) GEMV_TRACE(2, it + 1);
    const unsigned char* base = my_stage_ptr + stage * kGemvStageBytes;
    uint2 cq[2][kGemvBlocksPerWarp];
    float sc[2][2][kGemvBlocksPerWarp];   // absmax of (n-tile, row 2t + r, block)
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int b = 0; b < kGemvBlocksPerWarp; ++b)
        cq[nt][b] = *reinterpret_cast<const uint2*>(base + frag_off[b] + nt * 512);
    if (!NESTED) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const float2 v = *reinterpret_cast<const float2*>(base + 1024 + (nt * 8 + 2 * t + r) * 8);
          sc[nt][r][0] = v.x;
          sc[nt][r][1] = v.y;
        }
    } else {
      // lane L resolves the absmax of (row L / 2, block L % 2) of this warp's K-slice -- code2[u8] * absmax2 + offset
      // with a separate multiply and add, the bits the dequantiser produces -- and the quads fetch theirs by shuffle
      const float second = *reinterpret_cast<const float*>(base + 1024 + lane * 4);
      const float mine = __fadd_rn(__fmul_rn(code2_s[base[raw_off]], second), p.w.offset);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int b = 0; b < kGemvBlocksPerWarp; ++b)
            sc[nt][r][b] = __shfl_sync(0xffffffffu, mine, ((nt * 8 + 2 * t + r) << 1) | b);
    }
    float acc[2][4];
#ifdef MOLT_GEMV_TRACE
    if (p.debug & 1) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = __uint_as_float(cq[nt][0].x + cq[nt][1].y) * sc[nt][i & 1][i >> 1];
    } else
#endif
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      float part[kGemvBlocksPerWarp][4];
      uint32_t pr[kGemvBlocksPerWarp][8];
#pragma unroll
      for (int b = 0; b < kGemvBlocksPerWarp; ++b) {
        const uint2 q = cq[nt][b];
        pr[b][0] = lookup(q.x, 0x5504); pr[b][1] = lookup(q.x, 0x5514); pr[b][2] = lookup(q.x, 0x5524); pr[b][3] = lookup(q.x, 0x5534);
        pr[b][4] = lookup(q.y, 0x5504); pr[b][5] = lookup(q.y, 0x5514); pr[b][6] = lookup(q.y, 0x5524); pr[b][7] = lookup(q.y, 0x5534);
      }
#pragma unroll
      for (int b = 0; b < kGemvBlocksPerWarp; ++b) mma_16816_c(part[b], xa[b][0], pr[b][0], pr[b][1], zero);
#pragma unroll
      for (int j = 1; j < 4; ++j)
#pragma unroll
        for (int b = 0; b < kGemvBlocksPerWarp; ++b) mma_16816(part[b], xa[b][j], pr[b][2 * j], pr[b][2 * j + 1]);
      // accumulator columns: c0, c2 belong to row 2t (r = 0), c1, c3 to row 2t + 1 (r = 1)
      acc[nt][0] = part[0][0] * sc[nt][0][0];
      acc[nt][1] = part[0][1] * sc[nt][1][0];
      acc[nt][2] = part[0][2] * sc[nt][0][0];
      acc[nt][3] = part[0][3] * sc[nt][1][0];
#pragma unroll
      for (int b = 1; b < kGemvBlocksPerWarp; ++b) {
        acc[nt][0] = fmaf(part[b][0], sc[nt][0][b], acc[nt][0]);
        acc[nt][1] = fmaf(part[b][1], sc[nt][1][b], acc[nt][1]);
        acc[nt][2] = fmaf(part[b][2], sc[nt][0][b], acc[nt][2]);
        acc[nt][3] = fmaf(part[b][3], sc[nt][1][b], acc[nt][3]);
      }
    }
    if (warp == 0) GEMV_TRACE(3, it + 1);
    if (++stage == kGemvStages) stage = 0;
    // hand the K-slice sums to the reducing warps through a ring of buffers
    if (red_wrapped && !mbar_wait(red_empty_bar(buf), red_phase ^ 1, abort_flag, p.status, 44)) return;
    if (warp == 0) GEMV_TRACE(4, it + 1);
    float* my_red = red + ((size_t)buf * warps + warp) * 256;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
      *reinterpret_cast<float4*>(my_red + (nt * 32 + lane) * 4) =
          make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
    __syncwarp();   // also orders this iteration's stage reads before the next iteration's copies into that stage
    if (lane == 0) mbar_arrive(red_full_bar(buf));
    if (++buf == kGemvRing) { buf = 0; red_wrapped = 1; red_phase ^= 1; }
  }
  cp_async_wait<0>();
}

// y[tok, n] = bf16(sum over K-groups of partial + low-rank term).  One thread per output column: it keeps its row of
// bf16(scaling * B) in registers and handles all tokens; T = bf16(sum over K-groups of its parts) sits in shared memory.
constexpr int kGemvFinishThreads = 128;
constexpr int kGemvMaxKGroups = 8;   // K up to 16384 columns
template <int RP>   // rank rounded up to a multiple of 16
__global__ void __launch_bounds__(kGemvFinishThreads) gemv_finish_kernel(const float* __restrict__ partial, int kgroups,
                                                                         const float* __restrict__ t_partial,
                                                                         const float* __restrict__ lora_b, float scaling,
                                                                         int rank, int m, long long n,
                                                                         __nv_bfloat16* __restrict__ y) {
  __shared__ float t_s[16 * 64];
  float tv[16 * 64 / kGemvFinishThreads];
#pragma unroll
  for (int j = 0; j < 16 * 64 / kGemvFinishThreads; ++j) {   // all requested before any is used
    const int i = threadIdx.x + j * kGemvFinishThreads;
    tv[j] = 0.f;
    if ((i & 63) < rank && (i >> 6) < m) {
#pragma unroll
      for (int kg = 0; kg < kGemvMaxKGroups; ++kg)
        if (kg < kgroups) tv[j] += __ldg(t_partial + kg * 16 * 64 + i);
    }
  }
#pragma unroll
  for (int j = 0; j < 16 * 64 / kGemvFinishThreads; ++j)
    t_s[threadIdx.x + j * kGemvFinishThreads] = __bfloat162float(__float2bfloat16_rn(tv[j]));
  __syncthreads();
  const long long col = blockIdx.x * (long long)kGemvFinishThreads + threadIdx.x;
  if (col >= n) return;
  float bs[RP];
#pragma unroll
  for (int rk = 0; rk < RP; ++rk)
    bs[rk] = rk < rank ? __bfloat162float(__float2bfloat16_rn(scaling * __ldg(lora_b + col * rank + rk))) : 0.f;
  // eight tokens at a time; all loads of a batch are requested before any is used (kgroups and m only predicate them)
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    float part[8][kGemvMaxKGroups];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int kg = 0; kg < kGemvMaxKGroups; ++kg)
        part[i][kg] = (half * 8 + i < m && kg < kgroups) ? __ldg(partial + ((long long)kg * 16 + half * 8 + i) * n + col) : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int tok = half * 8 + i;
      if (tok < m) {
        float lora = 0.f;
#pragma unroll
        for (int rk = 0; rk < RP; ++rk) lora += t_s[tok * 64 + rk] * bs[rk];   // entries past the rank are zero
        float base = part[i][0];
#pragma unroll
        for (int kg = 1; kg < kGemvMaxKGroups; ++kg) base += part[i][kg];
        y[(long long)tok * n + col] = __float2bfloat16_rn(base + lora);
      }
    }
  }
}

namespace {

struct GemvPlan {
  int nblk, warps_needed, kgroups, warps;
  size_t smem_bytes;
};

GemvPlan gemv_plan(long long k) {
  GemvPlan g;
  g.nblk = (int)(k / 64);
  g.warps_needed = (g.nblk + kGemvBlocksPerWarp - 1) / kGemvBlocksPerWarp;
  g.kgroups = (g.warps_needed + kGemvMaxWarps - 1) / kGemvMaxWarps;
  g.warps = (g.warps_needed + g.kgroups - 1) / g.kgroups;
  // pair table, sum ring, low-rank sums, code2, barriers; the rest goes to the warps' private load stages
  const size_t fixed = kGemvLutBytes + (size_t)kGemvRing * g.warps * 1024 + (size_t)g.warps * 512 + 1024 + 64;
  g.smem_bytes = fixed + (size_t)kGemvStages * g.warps * kGemvStageBytes;
  return g;
}

}  // namespace

// Whether the kernel can read this weight's nested absmax itself; otherwise the caller resolves it to fp32 first.
// It copies the u8 codes as aligned 4-byte words, which needs K / 64 to be a multiple of 4 and an aligned array.
bool gemv_reads_nested(const WeightView& w) {
  if (w.block2_shift < 0) return false;
  if ((w.k / 64) % 4 != 0) return false;
  return (reinterpret_cast<uintptr_t>(w.absmax) & 3) == 0;
}

// Workspace layout: [kgroups][16][64] fp32 parts of T | [kgroups][16][n] fp32 partial outputs | n * k / 64 fp32 resolved
// absmax (used by the caller for nested forms the kernel cannot read), each region starting on a 256-byte boundary.
static size_t gemv_partial_offset(const GemvPlan& g) { return ((size_t)g.kgroups * 16 * 64 * sizeof(float) + 255) & ~size_t(255); }
static size_t gemv_resolved_offset(const GemvPlan& g, long long n) {
  return (gemv_partial_offset(g) + (size_t)g.kgroups * 16 * n * sizeof(float) + 255) & ~size_t(255);
}

size_t gemv_workspace_bytes(long long n, long long k) {
  const GemvPlan g = gemv_plan(k);
  return gemv_resolved_offset(g, n) + (size_t)n * g.nblk * sizeof(float) + 256;
}

// Where in the workspace a caller puts the resolved absmax.
float* gemv_resolved_absmax_slot(void* workspace, long long n, long long k) {
  return reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + gemv_resolved_offset(gemv_plan(k), n));
}

int gemv_forward(const WeightView& w, const __nv_bfloat16* x, const float* lora_a, const float* lora_b, float scaling,
                 int rank, __nv_bfloat16* y, int m, void* workspace, size_t workspace_bytes, cudaStream_t s) {
  if (workspace_bytes < gemv_workspace_bytes(w.n, w.k))
    return fail(MOLT_E_VALUE, "molt_nf4_gemv: workspace too small (%zu < %zu bytes)", workspace_bytes,
                gemv_workspace_bytes(w.n, w.k));
  const bool nested = w.absmax_kind == MOLT_ABSMAX_NESTED;
  if (nested && !gemv_reads_nested(w))
    return fail(MOLT_E_RUNTIME, "molt_nf4_gemv: this nested absmax layout must be resolved to fp32 before the call");
  if ((reinterpret_cast<uintptr_t>(w.packed) & 15) != 0 || (reinterpret_cast<uintptr_t>(lora_a) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(x) & 7) != 0)
    return fail(MOLT_E_CAPABILITY, "molt_nf4_gemv: the packed weight and lora_a must start on 16-byte boundaries, x on 8");
  const GemvPlan g = gemv_plan(w.k);
  if (g.kgroups > kGemvMaxKGroups) return fail(MOLT_E_CAPABILITY, "molt_nf4_gemv: K is limited to %d columns", kGemvMaxKGroups * 2048);
  if (g.smem_bytes > (size_t)kGemvSmemLimit) return fail(MOLT_E_CAPABILITY, "molt_nf4_gemv: no room for the load stages");
  GemvParams p;
  p.w = w;
  p.x = x;
  p.lora_a = lora_a;
  p.rank = rank;
  p.m = m;
  p.nblk = g.nblk;
  p.kgroups = g.kgroups;
  p.warps_per_cta = g.warps;
  p.status = device_status_word();
  if (p.status == nullptr) return fail(MOLT_E_RUNTIME, "molt_nf4_gemv: no device status word");
  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  p.t_partial = reinterpret_cast<float*>(ws);
  p.partial = reinterpret_cast<float*>(ws + gemv_partial_offset(g));
  p.trace = nullptr;
  p.debug = 0;
#ifdef MOLT_GEMV_TRACE
  if (const char* dbg = getenv("MOLT_B200_DEBUG")) p.debug = atoi(dbg);
  if (const char* tr = getenv("MOLT_B200_TRACE_PTR")) p.trace = reinterpret_cast<long long*>(strtoull(tr, nullptr, 10));
#endif

  static thread_local bool configured[64][2] = {};
  int dev = 0;
  MOLT_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev][nested ? 1 : 0]) {
    if (nested) MOLT_CUDA(cudaFuncSetAttribute(nf4_gemv_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvSmemLimit));
    else MOLT_CUDA(cudaFuncSetAttribute(nf4_gemv_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvSmemLimit));
    configured[dev][nested ? 1 : 0] = true;
  }
  const int chunks = (int)(w.n / kGemvChunkRows);
  int gx = sm_count() / p.kgroups;
  if (gx < 1) gx = 1;
  if (gx > chunks) gx = chunks;
  if (gx * 8 < rank) return fail(MOLT_E_CAPABILITY, "molt_nf4_gemv: too few row chunks for this rank");
  dim3 grid((unsigned)gx, (unsigned)p.kgroups);
  const int threads = (p.warps_per_cta + 2) * 32;   // streaming warps + two reducing warps
  if (nested) nf4_gemv_kernel<true><<<grid, threads, g.smem_bytes, s>>>(p);
  else nf4_gemv_kernel<false><<<grid, threads, g.smem_bytes, s>>>(p);
  if (int rc = launch_status("nf4_gemv_kernel")) return rc;
  const unsigned fgrid = (unsigned)((w.n + kGemvFinishThreads - 1) / kGemvFinishThreads);
  switch ((rank + 15) / 16) {
    case 1: gemv_finish_kernel<16><<<fgrid, kGemvFinishThreads, 0, s>>>(p.partial, p.kgroups, p.t_partial, lora_b, scaling, rank, m, w.n, y); break;
    case 2: gemv_finish_kernel<32><<<fgrid, kGemvFinishThreads, 0, s>>>(p.partial, p.kgroups, p.t_partial, lora_b, scaling, rank, m, w.n, y); break;
    case 3: gemv_finish_kernel<48><<<fgrid, kGemvFinishThreads, 0, s>>>(p.partial, p.kgroups, p.t_partial, lora_b, scaling, rank, m, w.n, y); break;
    default: gemv_finish_kernel<64><<<fgrid, kGemvFinishThreads, 0, s>>>(p.partial, p.kgroups, p.t_partial, lora_b, scaling, rank, m, w.n, y); break;
  }
  return launch_status("gemv_finish_kernel");
}

}  // namespace molt
