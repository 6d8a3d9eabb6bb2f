// Small-token (M <= 16) NF4 + LoRA forward.  The packed weight is streamed from HBM exactly once.
//
// Work split: a warp owns a fixed K-slice of 2 absmax blocks (128 columns) and keeps the matching
// X fragments in registers for its whole life; a CTA's warps cover consecutive slices and walk over
// 16-row chunks of W.  Per chunk every thread issues four 8-byte loads (a quad reads 32 contiguous bytes
// of one weight row).  Codes are expanded two at a time through a byte-indexed table of bf16 pairs that
// is replicated once per lane (bank = lane, so lookups never conflict) and fed to mma.sync m16n8k16
// with the tokens as the M dimension.  The MMA runs on the unscaled code values; each absmax block's
// partial sum is multiplied by its fp32 absmax afterwards, so no per-element multiply is needed.
// Packed codes are fetched two chunks ahead and the absmax data one chunk ahead of their use.
// K-slices are summed in warp order through shared memory (deterministic).  When K needs more warps
// than a CTA holds, CTAs of different K-groups write fp32 partials to the workspace and a small second
// kernel adds them, adds the low-rank term and rounds to bf16.
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
  __nv_bfloat16* y;         // [m, n]
};

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Raw absmax data of one weight row for this warp's two blocks, fetched ahead of use.
template <bool NESTED>
struct RowScales;
template <>
struct RowScales<false> {
  float2 v;
  __device__ __forceinline__ void load(const GemvParams& p, long long row, int blk0, int nb) {
    const long long blk = row * p.nblk + blk0;
    const float* src = reinterpret_cast<const float*>(p.w.absmax) + blk;
    if (nb == 2 && (blk & 1) == 0) v = __ldg(reinterpret_cast<const float2*>(src));
    else v = make_float2(nb >= 1 ? __ldg(src) : 0.f, nb == 2 ? __ldg(src + 1) : 0.f);
  }
  __device__ __forceinline__ float get(const GemvParams&, const float*, int b) const { return b == 0 ? v.x : v.y; }
};
template <>
struct RowScales<true> {
  unsigned codes;   // two uint8 codes
  float2 second;    // absmax2 of the two blocks
  __device__ __forceinline__ void load(const GemvParams& p, long long row, int blk0, int nb) {
    const long long blk = row * p.nblk + blk0;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(p.w.absmax) + blk;
    if (nb == 2 && (blk & 1) == 0) codes = (unsigned)__ldg(reinterpret_cast<const unsigned short*>(src));
    else codes = (nb >= 1 ? (unsigned)__ldg(src) : 0u) | (nb == 2 ? (unsigned)__ldg(src + 1) << 8 : 0u);
    second.x = nb >= 1 ? __ldg(p.w.absmax2 + blk / p.w.block2) : 0.f;
    second.y = nb == 2 ? __ldg(p.w.absmax2 + (blk + 1) / p.w.block2) : 0.f;
  }
  // code2[u8] * absmax2 + offset with separate multiply and add: the bits the dequantiser produces
  __device__ __forceinline__ float get(const GemvParams& p, const float* code2_s, int b) const {
    const unsigned c = b == 0 ? (codes & 0xffu) : (codes >> 8);
    return __fadd_rn(__fmul_rn(code2_s[c], b == 0 ? second.x : second.y), p.w.offset);
  }
};

template <bool NESTED>
__global__ void __launch_bounds__(kGemvMaxWarps * 32, 1) nf4_gemv_kernel(const __grid_constant__ GemvParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // [256 entries][32 lanes] bf16x2 pair table, [2 buffers][warps][2 ntiles][32 lanes][4] partials, T, code2
  uint32_t* pair_lut = reinterpret_cast<uint32_t*>(smem_raw);
  float* red = reinterpret_cast<float*>(smem_raw + 256 * 32 * 4);
  const int warps = p.warps_per_cta;
  float* t_s = red + 2 * warps * 256;  // [16][64]
  float* code2_s = t_s + 16 * 64;      // [256]
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
  if (NESTED)
    for (int i = threadIdx.x; i < 256; i += blockDim.x) code2_s[i] = p.w.code2[i];

  // ---- this warp's K-slice and its X fragments ----
  const int slice = kgroup * warps + warp;
  const int blk0 = slice * kGemvBlocksPerWarp;
  int nb = p.nblk - blk0;
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

  struct Chunk {
    uint2 wq[2][kGemvBlocksPerWarp];   // packed codes: [n-tile][block]
  };
  auto load_codes = [&](int chunk, Chunk& dst) {
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const long long row = (long long)chunk * kGemvChunkRows + nt * 8 + g;
#pragma unroll
      for (int b = 0; b < kGemvBlocksPerWarp; ++b)
        dst.wq[nt][b] = (b < nb && chunk < chunks)
                            ? __ldcs(reinterpret_cast<const uint2*>(wbase + row * row_bytes + b * 32))
                            : make_uint2(0, 0);
    }
  };
  auto load_scales = [&](int chunk, RowScales<NESTED> (&dst)[2][2]) {
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const long long row = (long long)chunk * kGemvChunkRows + nt * 8 + 2 * t + r;
        dst[nt][r].load(p, chunk < chunks ? row : 0, blk0, chunk < chunks ? nb : 0);
      }
  };

  // software pipeline: codes two chunks ahead, scales one chunk ahead
  Chunk c0, c1, c2;
  RowScales<NESTED> s0[2][2], s1[2][2];
  int chunk = blockIdx.x;
  const int stride = gridDim.x;
  load_codes(chunk, c0);
  load_codes(chunk + stride, c1);
  load_scales(chunk, s0);
  int buf = 0;
  for (; chunk < chunks; chunk += stride) {
    load_codes(chunk + 2 * stride, c2);
    load_scales(chunk + stride, s1);
    float acc[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[nt][c] = 0.f;
#pragma unroll
      for (int b = 0; b < kGemvBlocksPerWarp; ++b) {
        if (b < nb) {
          float part[4] = {0.f, 0.f, 0.f, 0.f};
          const uint32_t words[2] = {c0.wq[nt][b].x, c0.wq[nt][b].y};
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
          const float sc0 = s0[nt][0].get(p, code2_s, b);   // row 2t   : accumulator columns c0, c2
          const float sc1 = s0[nt][1].get(p, code2_s, b);   // row 2t+1 : accumulator columns c1, c3
          acc[nt][0] = fmaf(part[0], sc0, acc[nt][0]);
          acc[nt][1] = fmaf(part[1], sc1, acc[nt][1]);
          acc[nt][2] = fmaf(part[2], sc0, acc[nt][2]);
          acc[nt][3] = fmaf(part[3], sc1, acc[nt][3]);
        }
      }
    }
    // ---- sum the K-slices of this CTA in warp order (double-buffered, one barrier per chunk) ----
    float* my_red = red + (buf * warps + warp) * 256;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
      *reinterpret_cast<float4*>(my_red + (nt * 32 + lane) * 4) =
          make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
    __syncthreads();
    if (threadIdx.x < 256) {
      const int r = threadIdx.x & 15, tok = threadIdx.x >> 4;   // row inside the chunk, token
      const int nt = r >> 3, rr = r & 7;
      const int src_lane = (tok & 7) * 4 + (rr >> 1);
      const int src_c = (rr & 1) + (tok >> 3) * 2;
      float sum = 0.f;
      for (int wv = 0; wv < warps; ++wv) sum += red[((buf * warps + wv) * 64 + nt * 32 + src_lane) * 4 + src_c];
      const long long n = (long long)chunk * kGemvChunkRows + r;
      if (p.kgroups > 1) {
        p.partial[((long long)kgroup * 16 + tok) * p.w.n + n] = sum;
      } else if (tok < p.m) {
        float lora = 0.f;
        for (int rk = 0; rk < p.rank; ++rk)
          lora += t_s[tok * 64 + rk] * __bfloat162float(__float2bfloat16_rn(p.scaling * p.lora_b[n * p.rank + rk]));
        p.y[(long long)tok * p.w.n + n] = __float2bfloat16_rn(sum + lora);
      }
    }
    buf ^= 1;
    c0 = c1;
    c1 = c2;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int r = 0; r < 2; ++r) s0[nt][r] = s1[nt][r];
  }
}

// y[tok, n] = bf16(sum over K-groups of partial + low-rank term); only launched when K needed several CTAs.
__global__ void gemv_finish_kernel(const float* __restrict__ partial, int kgroups, const float* __restrict__ t,
                                   const float* __restrict__ lora_b, float scaling, int rank, int m, long long n,
                                   __nv_bfloat16* __restrict__ y) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)m * n) return;
  const int tok = (int)(idx / n);
  const long long col = idx % n;
  float sum = 0.f;
  for (int kg = 0; kg < kgroups; ++kg) sum += partial[((long long)kg * 16 + tok) * n + col];
  float lora = 0.f;
  for (int rk = 0; rk < rank; ++rk)
    lora += t[tok * 64 + rk] * __bfloat162float(__float2bfloat16_rn(scaling * lora_b[col * rank + rk]));
  y[idx] = __float2bfloat16_rn(sum + lora);
}

// t[tok, r] = bf16(sum_k x[tok, k] * bf16(A[r, k])) as fp32, zero elsewhere in the [16, 64] tile.
// One 128-thread CTA per (token, r): every thread sums a strided share of K, then the shares are added in a fixed
// order (warp shuffles, then the four warp sums), so the result is deterministic.
__global__ void __launch_bounds__(128) gemv_lowrank_kernel(const __nv_bfloat16* __restrict__ x,
                                                           const float* __restrict__ a, int m, int rank, long long k,
                                                           float* __restrict__ t) {
  __shared__ float warp_sums[4];
  const int tok = blockIdx.x >> 6, r = blockIdx.x & 63;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float sum = 0.f;
  if (tok < m && r < rank) {
    const __nv_bfloat16* xr = x + (long long)tok * k;
    const float* ar = a + (long long)r * k;
    for (long long c = threadIdx.x * 2; c < k; c += 256) {
      const __nv_bfloat162 xv = *reinterpret_cast<const __nv_bfloat162*>(xr + c);
      const float2 av = *reinterpret_cast<const float2*>(ar + c);
      sum += __bfloat162float(xv.x) * __bfloat162float(__float2bfloat16_rn(av.x));
      sum += __bfloat162float(xv.y) * __bfloat162float(__float2bfloat16_rn(av.y));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) warp_sums[warp] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    const float total = (warp_sums[0] + warp_sums[1]) + (warp_sums[2] + warp_sums[3]);
    t[blockIdx.x] = __bfloat162float(__float2bfloat16_rn(total));
  }
}

size_t gemv_workspace_bytes(long long n, long long k) {
  const int nblk = (int)(k / 64);
  const int warps_needed = (nblk + kGemvBlocksPerWarp - 1) / kGemvBlocksPerWarp;
  const int kgroups = (warps_needed + kGemvMaxWarps - 1) / kGemvMaxWarps;
  size_t bytes = 16 * 64 * sizeof(float);  // T
  if (kgroups > 1) bytes += (size_t)kgroups * 16 * n * sizeof(float);
  return bytes + 256;
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
  if (p.warps_per_cta < 8) p.warps_per_cta = 8;  // the chunk reduction uses 256 threads
  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  float* t = reinterpret_cast<float*>(ws);
  p.t = t;
  p.partial = reinterpret_cast<float*>(ws + 16 * 64 * sizeof(float) + 256 - (16 * 64 * sizeof(float)) % 256);
  p.y = y;
  gemv_lowrank_kernel<<<16 * 64, 128, 0, s>>>(x, lora_a, m, rank, w.k, t);
  if (int rc = launch_status("gemv_lowrank_kernel")) return rc;

  const size_t smem = 256 * 32 * 4 + (size_t)2 * p.warps_per_cta * 256 * 4 + 16 * 64 * 4 + 256 * 4;
  const bool nested = w.absmax_kind == MOLT_ABSMAX_NESTED;
  static thread_local bool configured[64][2] = {};
  int dev = 0;
  MOLT_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev][nested ? 1 : 0]) {
    if (nested) MOLT_CUDA(cudaFuncSetAttribute(nf4_gemv_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    else MOLT_CUDA(cudaFuncSetAttribute(nf4_gemv_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    configured[dev][nested ? 1 : 0] = true;
  }
  const int chunks = (int)(w.n / kGemvChunkRows);
  int gx = sm_count() / p.kgroups;
  if (gx < 1) gx = 1;
  if (gx > chunks) gx = chunks;
  dim3 grid((unsigned)gx, (unsigned)p.kgroups);
  if (nested) nf4_gemv_kernel<true><<<grid, p.warps_per_cta * 32, smem, s>>>(p);
  else nf4_gemv_kernel<false><<<grid, p.warps_per_cta * 32, smem, s>>>(p);
  if (int rc = launch_status("nf4_gemv_kernel")) return rc;
  if (p.kgroups > 1) {
    const long long total = (long long)m * w.n;
    gemv_finish_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(p.partial, p.kgroups, t, lora_b, scaling, rank, m,
                                                                       w.n, y);
    return launch_status("gemv_finish_kernel");
  }
  return MOLT_OK;
}

}  // namespace molt
