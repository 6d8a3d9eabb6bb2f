// Small-token (M <= 16) NF4 + LoRA forward.  The packed weight is streamed from HBM exactly once.
//
// Work split: a warp owns a fixed K-slice of 2 absmax blocks (128 columns) and keeps the matching
// X fragments in registers for its whole life; a CTA's warps cover consecutive slices and walk over
// 16-row chunks of W.  Per chunk every thread issues four 8-byte loads (a quad reads 32 contiguous bytes
// of one weight row).  Codes are expanded two at a time through a byte-indexed table of bf16 pairs that
// is replicated once per lane (bank = lane, so lookups never conflict) and fed to mma.sync m16n8k16
// with the tokens as the M dimension.  The MMA runs on the unscaled code values; each absmax block's
// partial sum is multiplied by its fp32 absmax afterwards, so no per-element multiply is needed.
// K-slices are summed in warp order through shared memory (deterministic).  When K needs more warps
// than a CTA holds, CTAs of different K-groups exchange fp32 partials through the workspace and the
// last CTA to arrive at a chunk finishes it (an atomic ticket, nobody waits).
#include "common.cuh"

namespace molt {

constexpr int kGemvMaxWarps = 16;
constexpr int kGemvBlocksPerWarp = 2;   // absmax blocks (of 64 columns) per warp
constexpr int kGemvChunkRows = 16;

struct GemvParams {
  WeightView w;
  const __nv_bfloat16* x;   // [m, k]
  const float* t;           // [16, 64] fp32 (bf16-rounded values), x . A^T
  const float* lora_b;      // [n, rank]
  float scaling;
  int rank;
  int m;
  int nblk;                 // k / 64
  int warps_needed;         // ceil(nblk / 2)
  int kgroups;
  int warps_per_cta;
  float* partial;           // [kgroups][16][n] fp32 (kgroups > 1)
  unsigned* tickets;        // [n / 16] zero-initialised (kgroups > 1)
  __nv_bfloat16* y;         // [m, n]
};

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float resolve_absmax(const GemvParams& p, long long blk) { return load_absmax(p.w, blk); }

__global__ void __launch_bounds__(kGemvMaxWarps * 32, 1) nf4_gemv_kernel(GemvParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // [256 entries][32 lanes] bf16x2 pair table, then [2 buffers][warps][2 ntiles][32 lanes][4] partials, then T
  uint32_t* pair_lut = reinterpret_cast<uint32_t*>(smem_raw);
  float* red = reinterpret_cast<float*>(smem_raw + 256 * 32 * 4);
  const int warps = p.warps_per_cta;
  float* t_s = red + 2 * warps * 256;  // [16][64]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int kgroup = blockIdx.y;

  // ---- tables ----
  for (int i = threadIdx.x; i < 256 * 32; i += blockDim.x) {
    const int byte = i >> 5;
    const int first = p.w.nibble_order == MOLT_NIBBLE_LOW_FIRST ? (byte & 15) : (byte >> 4);
    const int second = p.w.nibble_order == MOLT_NIBBLE_LOW_FIRST ? (byte >> 4) : (byte & 15);
    pair_lut[i] = pack_bf16x2(p.w.codebook[first], p.w.codebook[second]);
  }
  for (int i = threadIdx.x; i < 16 * 64; i += blockDim.x) t_s[i] = p.t != nullptr ? p.t[i] : 0.f;

  // ---- this warp's K-slice and its X fragments ----
  const int slice = kgroup * warps + warp;             // global warp-slice index
  const int blk0 = slice * kGemvBlocksPerWarp;
  int nb = p.nblk - blk0;                              // blocks owned by this warp (0, 1 or 2)
  if (slice >= p.warps_needed || nb < 0) nb = 0;
  if (nb > kGemvBlocksPerWarp) nb = kGemvBlocksPerWarp;
  uint32_t xa[kGemvBlocksPerWarp][4][4];
#pragma unroll
  for (int b = 0; b < kGemvBlocksPerWarp; ++b)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long col = (long long)(blk0 + b) * 64 + 16 * t + 4 * j;
      uint2 lo = make_uint2(0, 0), hi = make_uint2(0, 0);
      if (b < nb) {
        if (g < p.m) lo = *reinterpret_cast<const uint2*>(p.x + (long long)g * p.w.k + col);
        if (g + 8 < p.m) hi = *reinterpret_cast<const uint2*>(p.x + (long long)(g + 8) * p.w.k + col);
      }
      xa[b][j][0] = lo.x; xa[b][j][1] = hi.x; xa[b][j][2] = lo.y; xa[b][j][3] = hi.y;
    }
  __syncthreads();

  const uint32_t* my_lut = pair_lut + lane;
  const long long row_bytes = p.w.k / 2;
  const int chunks = (int)(p.w.n / kGemvChunkRows);
  const uint8_t* wbase = p.w.packed + (long long)blk0 * 32 + t * 8;

  auto load_chunk = [&](int chunk, uint2 (&dst)[2][kGemvBlocksPerWarp]) {
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const long long row = (long long)chunk * kGemvChunkRows + nt * 8 + g;
#pragma unroll
      for (int b = 0; b < kGemvBlocksPerWarp; ++b)
        dst[nt][b] = (b < nb) ? __ldcs(reinterpret_cast<const uint2*>(wbase + row * row_bytes + b * 32))
                              : make_uint2(0, 0);
    }
  };

  uint2 cur[2][kGemvBlocksPerWarp], nxt[2][kGemvBlocksPerWarp];
  int chunk = blockIdx.x;
  if (chunk < chunks) load_chunk(chunk, cur);
  int buf = 0;
  for (; chunk < chunks; chunk += gridDim.x) {
    const int next = chunk + gridDim.x;
    if (next < chunks) load_chunk(next, nxt);
    float acc[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[nt][c] = 0.f;
      const long long n_lo = (long long)chunk * kGemvChunkRows + nt * 8 + 2 * t;  // rows of c0/c2 ; +1 for c1/c3
#pragma unroll
      for (int b = 0; b < kGemvBlocksPerWarp; ++b) {
        if (b < nb) {
          float part[4] = {0.f, 0.f, 0.f, 0.f};
          const uint32_t words[2] = {cur[nt][b].x, cur[nt][b].y};
#pragma unroll
          for (int wi = 0; wi < 2; ++wi) {
            const uint32_t wd = words[wi];
            const uint32_t p0 = my_lut[(wd & 0xffu) << 5];
            const uint32_t p1 = my_lut[((wd >> 8) & 0xffu) << 5];
            const uint32_t p2 = my_lut[((wd >> 16) & 0xffu) << 5];
            const uint32_t p3 = my_lut[(wd >> 24) << 5];
            mma_16816(part, xa[b][wi * 2], p0, p1);
            mma_16816(part, xa[b][wi * 2 + 1], p2, p3);
          }
          const float s0 = resolve_absmax(p, n_lo * p.nblk + blk0 + b);
          const float s1 = resolve_absmax(p, (n_lo + 1) * p.nblk + blk0 + b);
          acc[nt][0] = fmaf(part[0], s0, acc[nt][0]);
          acc[nt][1] = fmaf(part[1], s1, acc[nt][1]);
          acc[nt][2] = fmaf(part[2], s0, acc[nt][2]);
          acc[nt][3] = fmaf(part[3], s1, acc[nt][3]);
        }
      }
    }
    // ---- sum the K-slices of this CTA (warp order) ----
    float* my_red = red + (buf * warps + warp) * 256;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
      *reinterpret_cast<float4*>(my_red + (nt * 32 + lane) * 4) =
          make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
    __syncthreads();
    if (threadIdx.x < 256) {
      // output element: row r (0..15) of the chunk, token tok (0..15)
      const int r = threadIdx.x & 15, tok = threadIdx.x >> 4;
      const int nt = r >> 3, rr = r & 7;
      const int src_lane = (tok & 7) * 4 + (rr >> 1);
      const int src_c = (rr & 1) + (tok >> 3) * 2;
      float sum = 0.f;
      for (int wv = 0; wv < warps; ++wv) sum += red[((buf * warps + wv) * 64 + nt * 32 + src_lane) * 4 + src_c];
      const long long n = (long long)chunk * kGemvChunkRows + r;
      bool finish = true;
      if (p.kgroups > 1) {
        p.partial[((long long)kgroup * 16 + tok) * p.w.n + n] = sum;
        __threadfence();
        __shared__ unsigned last_flag[2];
        __syncwarp();
        // 256 finishing threads = 8 full warps; one ticket per chunk taken by thread 0 after a CTA-local barrier
        asm volatile("bar.sync 1, 256;\n" ::);
        if (threadIdx.x == 0) {
          const unsigned old = atomicAdd(p.tickets + chunk, 1u);
          last_flag[buf] = (old == (unsigned)(p.kgroups - 1));
          if (old == (unsigned)(p.kgroups - 1)) p.tickets[chunk] = 0;  // leave the tickets clean for the next call
        }
        asm volatile("bar.sync 1, 256;\n" ::);
        finish = last_flag[buf] != 0;
        if (finish) {
          __threadfence();
          sum = 0.f;
          for (int kg = 0; kg < p.kgroups; ++kg)
            sum += __ldcg(p.partial + ((long long)kg * 16 + tok) * p.w.n + n);
        }
      }
      if (finish && tok < p.m) {
        float lora = 0.f;
        for (int rk = 0; rk < p.rank; ++rk)
          lora += t_s[tok * 64 + rk] * __bfloat162float(__float2bfloat16_rn(p.scaling * p.lora_b[n * p.rank + rk]));
        p.y[(long long)tok * p.w.n + n] = __float2bfloat16_rn(sum + lora);
      }
    }
    buf ^= 1;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int b = 0; b < kGemvBlocksPerWarp; ++b) cur[nt][b] = nxt[nt][b];
  }
}

// t[tok, r] = bf16(sum_k x[tok, k] * bf16(A[r, k])) as fp32, zero elsewhere in the [16, 64] tile.
// One warp per (token, r).  Also clears the chunk tickets.
__global__ void gemv_lowrank_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ a, int m, int rank,
                                    long long k, float* __restrict__ t, unsigned* tickets, int ticket_count) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < ticket_count; i += gridDim.x * blockDim.x) tickets[i] = 0;
  if (warp >= 16 * 64) return;
  const int tok = warp >> 6, r = warp & 63;
  float sum = 0.f;
  if (tok < m && r < rank) {
    for (long long c = lane; c < k; c += 32)
      sum += __bfloat162float(x[(long long)tok * k + c]) *
             __bfloat162float(__float2bfloat16_rn(a[(long long)r * k + c]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  }
  if (lane == 0) t[warp] = __bfloat162float(__float2bfloat16_rn(sum));
}

size_t gemv_workspace_bytes(long long n, long long k) {
  const int nblk = (int)(k / 64);
  const int warps_needed = (nblk + kGemvBlocksPerWarp - 1) / kGemvBlocksPerWarp;
  const int kgroups = (warps_needed + kGemvMaxWarps - 1) / kGemvMaxWarps;
  size_t bytes = 16 * 64 * sizeof(float);                         // T
  bytes += (size_t)(n / kGemvChunkRows + 1) * sizeof(unsigned);   // tickets
  bytes = (bytes + 255) & ~size_t(255);
  if (kgroups > 1) bytes += (size_t)kgroups * 16 * n * sizeof(float);
  return bytes;
}

int gemv_forward(const WeightView& w, const __nv_bfloat16* x, const float* lora_a, const float* lora_b, float scaling,
                 int rank, __nv_bfloat16* y, int m, void* workspace, size_t workspace_bytes, cudaStream_t s) {
  if (workspace_bytes < gemv_workspace_bytes(w.n, w.k))
    return fail(MOLT_E_VALUE, "molt_nf4_gemv: workspace too small (%zu < %zu bytes)", workspace_bytes,
                gemv_workspace_bytes(w.n, w.k));
  GemvParams p;
  p.w = w;
  p.x = x;
  p.lora_b = lora_b;
  p.scaling = scaling;
  p.rank = rank;
  p.m = m;
  p.nblk = (int)(w.k / 64);
  p.warps_needed = (p.nblk + kGemvBlocksPerWarp - 1) / kGemvBlocksPerWarp;
  p.kgroups = (p.warps_needed + kGemvMaxWarps - 1) / kGemvMaxWarps;
  p.warps_per_cta = (p.warps_needed + p.kgroups - 1) / p.kgroups;
  if (p.warps_per_cta < 8) p.warps_per_cta = 8;  // the finishing step uses 256 threads
  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  float* t = reinterpret_cast<float*>(ws);
  unsigned* tickets = reinterpret_cast<unsigned*>(ws + 16 * 64 * sizeof(float));
  const int ticket_count = (int)(w.n / kGemvChunkRows);
  size_t head = 16 * 64 * sizeof(float) + (size_t)(ticket_count + 1) * sizeof(unsigned);
  head = (head + 255) & ~size_t(255);
  p.t = t;
  p.tickets = tickets;
  p.partial = reinterpret_cast<float*>(ws + head);
  p.y = y;
  gemv_lowrank_kernel<<<(16 * 64 * 32 + 255) / 256, 256, 0, s>>>(x, lora_a, m, rank, w.k, t, tickets, ticket_count);
  if (int rc = launch_status("gemv_lowrank_kernel")) return rc;

  const size_t smem = 256 * 32 * 4 + (size_t)2 * p.warps_per_cta * 256 * 4 + 16 * 64 * 4;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(nf4_gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (err != cudaSuccess) return fail(MOLT_E_RUNTIME, "cudaFuncSetAttribute(gemv): %s", cudaGetErrorString(err));
    configured = true;
  }
  int gx = sm_count() / p.kgroups;
  if (gx < 1) gx = 1;
  if (gx > ticket_count) gx = ticket_count;
  dim3 grid((unsigned)gx, (unsigned)p.kgroups);
  nf4_gemv_kernel<<<grid, p.warps_per_cta * 32, smem, s>>>(p);
  return launch_status("nf4_gemv_kernel");
}

}  // namespace molt
