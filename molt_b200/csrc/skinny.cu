// Low-rank (LoRA) side kernels for aligned shapes.  All are HBM-bound passes over X or dY:
//   lora_prep      fp32 adapter masters -> bf16 operand layouts
//   rowsum_mma     T = X . A^T        and   U = dY . (s B)        ([M, C] x [rp, C]^T -> [M, 64] bf16)
//   colsum_mma     dA = U^T . X       and   dB^T = T^T . dY       ([M, 64]^T x [M, C] -> [rp, C] fp32 partials)
//   colsum_reduce  deterministic sum of the split-M partials into the fp32 gradient
// Tensor-core work uses mma.sync m16n8k16 (these passes are bandwidth-bound; the tcgen05 kernels carry the FLOPs).
#include "common.cuh"

namespace molt {

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ------------------------------------------------------------------------------------------------
// Adapter operand preparation.
//   a16  [rp, k]  bf16(A), rows >= rank zero
//   bs   [n, 64]  bf16(scaling * B), columns >= rank zero      (forward low-rank k-block, K-major)
//   bt   [rp, n]  bf16(scaling * B)^T, rows >= rank zero       (U = dY . (sB))
// Any of the three outputs may be NULL.  The same launch also resolves a nested absmax to fp32 when `resolved` is given
// (one launch instead of two in front of every GEMM).
// ------------------------------------------------------------------------------------------------
// One item of the preparation lists of one adapter (a16: 8 elements, bs: one row of 64, bt: one column); returns the
// index left over when i lies past the three lists, or -1 when the item was handled.
__device__ __forceinline__ long long lora_prep_item(long long i, const float* __restrict__ a, const float* __restrict__ b,
                                                    float scaling, int rank, int rp, long long n, long long k,
                                                    __nv_bfloat16* __restrict__ a16, __nv_bfloat16* __restrict__ bs,
                                                    __nv_bfloat16* __restrict__ bt) {
  const long long items_a = a16 != nullptr ? (long long)rp * k / 8 : 0;
  const long long items_bs = bs != nullptr ? n : 0;
  const long long items_bt = bt != nullptr ? n : 0;
  if (i < items_a) {
    const long long e = i * 8;
    const int r = (int)(e / k);
    uint32_t out[4] = {0u, 0u, 0u, 0u};
    if (r < rank) {
      const float4 lo = __ldg(reinterpret_cast<const float4*>(a + e)), hi = __ldg(reinterpret_cast<const float4*>(a + e + 4));
      out[0] = pack_bf16x2(lo.x, lo.y); out[1] = pack_bf16x2(lo.z, lo.w);
      out[2] = pack_bf16x2(hi.x, hi.y); out[3] = pack_bf16x2(hi.z, hi.w);
    }
    *reinterpret_cast<uint4*>(a16 + e) = make_uint4(out[0], out[1], out[2], out[3]);
    return -1;
  }
  i -= items_a;
  if (i < items_bs) {   // one row of B -> one 64-wide row of bs (128 bytes)
    uint32_t out[32];
#pragma unroll
    for (int q = 0; q < 32; ++q) {
      const float v0 = 2 * q < rank ? scaling * __ldg(b + i * rank + 2 * q) : 0.f;
      const float v1 = 2 * q + 1 < rank ? scaling * __ldg(b + i * rank + 2 * q + 1) : 0.f;
      out[q] = pack_bf16x2(v0, v1);
    }
    uint4* dst = reinterpret_cast<uint4*>(bs + i * 64);
#pragma unroll
    for (int q = 0; q < 8; ++q) dst[q] = make_uint4(out[4 * q], out[4 * q + 1], out[4 * q + 2], out[4 * q + 3]);
    return -1;
  }
  i -= items_bs;
  if (i < items_bt) {   // one row of B -> one column of bt: neighbouring threads write neighbouring elements of every row
    for (int r = 0; r < rp; ++r)
      bt[(long long)r * n + i] = __float2bfloat16_rn(r < rank ? scaling * __ldg(b + i * rank + r) : 0.f);
    return -1;
  }
  return i - items_bt;
}

__global__ void lora_prep_kernel(const float* __restrict__ a, const float* __restrict__ b, float scaling, int rank,
                                 int rp, long long n, long long k, __nv_bfloat16* __restrict__ a16,
                                 __nv_bfloat16* __restrict__ bs, __nv_bfloat16* __restrict__ bt, WeightView w,
                                 float* __restrict__ resolved, long long absmax_blocks) {
  // One item per thread out of the four lists laid end to end, so that all of them are in flight together:
  // a16 (8 elements), bs (one row of 64), bt (one column), resolved absmax (4 blocks).
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  i = lora_prep_item(i, a, b, scaling, rank, rp, n, k, a16, bs, bt);
  if (i < 0) return;
  if (resolved != nullptr) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const long long blk = i * 4 + q;
      if (blk < absmax_blocks) resolved[blk] = load_absmax(w, blk);
    }
  }
}

// The shadows of many adapters in one launch: blockIdx.y = adapter, the blocks of a row walk its item lists.
__global__ void __launch_bounds__(256) lora_shadow_refresh_kernel(const molt_lora_shadow_item* __restrict__ items) {
  const molt_lora_shadow_item it = items[blockIdx.y];
  const int rp = (it.rank + 15) / 16 * 16;
  const long long total = (long long)rp * it.k / 8 + 2 * it.n;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
    lora_prep_item(i, it.lora_a, it.lora_b, it.scaling, it.rank, rp, it.n, it.k, reinterpret_cast<__nv_bfloat16*>(it.a16),
                   reinterpret_cast<__nv_bfloat16*>(it.bs), reinterpret_cast<__nv_bfloat16*>(it.bt));
}

// ------------------------------------------------------------------------------------------------
// rowsum: out[m, 0..63] = bf16(sum_c in[m, c] * wt[r, c]), zero for r >= RP.
// One CTA = 16 rows; its warps split the contraction in 32-column chunks and are summed in warp order.
// The k index inside each MMA is permuted (thread t owns 8 consecutive columns) so that both operands are
// fetched with 16-byte loads; the permutation is applied to both operands, so the sum is unchanged.
// ------------------------------------------------------------------------------------------------
// warps per CTA of 16 rows: they split the contraction; 16 where the partial sums still fit in 48 KB of shared memory
constexpr int rowsum_warps(int rp) { return rp <= 32 ? 16 : 8; }   // 32 warps measured slower than 16
template <int RP, int kRowsumWarps, int kUnroll>
__global__ void __launch_bounds__(kRowsumWarps * 32) rowsum_mma_kernel(const __nv_bfloat16* __restrict__ in,
                                                         const __nv_bfloat16* __restrict__ wt, long long m_total,
                                                         long long cols, __nv_bfloat16* __restrict__ out) {
  constexpr int NT = RP / 8;
  static_assert(kRowsumWarps <= rowsum_warps(RP), "the partial sums of all warps must fit in 48 KB");
  // the GEMM that follows in the stream may begin its set-up (it waits for this grid before it touches global memory)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ float partial[kRowsumWarps][16][RP + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const long long row0 = blockIdx.x * 16LL;
  const long long r_lo = row0 + g, r_hi = row0 + g + 8;
  const bool lo_ok = r_lo < m_total, hi_ok = r_hi < m_total;
  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
  const long long chunks = cols / 32;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  // kUnroll NEIGHBOURING chunks per trip, so that a warp asks for whole 128-byte lines of its rows (64 bytes per
  // chunk); the activation loads of a trip (the HBM stream) are requested before anything is used.
#ifdef MOLT_ROWSUM_FAR_CHUNKS   // the previous assignment: chunks c and c + W to a warp (a line is shared by two warps)
  constexpr int kFirst = 1, kNext = kRowsumWarps;
#else
  constexpr int kFirst = kUnroll, kNext = 1;
#endif
  for (long long c0 = warp * kFirst; c0 < chunks; c0 += kRowsumWarps * kUnroll) {
    uint4 lo[kUnroll], hi[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long col = (c0 + kNext * u) * 32 + t * 8;
      const bool in_range = c0 + kNext * u < chunks;
      lo[u] = (lo_ok && in_range) ? __ldg(reinterpret_cast<const uint4*>(in + r_lo * cols + col)) : zero;
      hi[u] = (hi_ok && in_range) ? __ldg(reinterpret_cast<const uint4*>(in + r_hi * cols + col)) : zero;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (c0 + kNext * u < chunks) {
        const long long col = (c0 + kNext * u) * 32 + t * 8;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          const uint4 b = __ldg(reinterpret_cast<const uint4*>(wt + (long long)(j * 8 + g) * cols + col));
          mma_bf16_16816(acc[j], lo[u].x, hi[u].x, lo[u].y, hi[u].y, b.x, b.y);
          mma_bf16_16816(acc[j], lo[u].z, hi[u].z, lo[u].w, hi[u].w, b.z, b.w);
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    partial[warp][g][j * 8 + 2 * t] = acc[j][0];
    partial[warp][g][j * 8 + 2 * t + 1] = acc[j][1];
    partial[warp][g + 8][j * 8 + 2 * t] = acc[j][2];
    partial[warp][g + 8][j * 8 + 2 * t + 1] = acc[j][3];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < 16 * 64; idx += kRowsumWarps * 32) {
    const int row = idx >> 6, r = idx & 63;
    if (row0 + row >= m_total) continue;
    float sum = 0.f;
    if (r < RP) {
#pragma unroll
      for (int wv = 0; wv < kRowsumWarps; ++wv) sum += partial[wv][row][r];
    }
    out[(row0 + row) * 64 + r] = __float2bfloat16_rn(sum);
  }
}

// ------------------------------------------------------------------------------------------------
// colsum: partial[split][r][c] = sum_{m in split} low[m, r] * in[m, c].
// CTA = 4 warps on a 64-column slab; rows are streamed in 64-row tiles through a 2-stage cp.async ring
// and both operands are read transposed with ldmatrix.trans.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

constexpr int kColsumRowBytes = 144;  // 128 data bytes + 16 pad: conflict-free ldmatrix rows
constexpr int kColsumTileBytes = 64 * kColsumRowBytes;

struct ColsumProblem {
  const __nv_bfloat16* low;   // [m, 64]
  const __nv_bfloat16* in;    // [m, cols]
  long long cols;
  int tiles_per_split, splits;
  float* partial;             // [splits][RP][cols]
  unsigned blocks;            // slabs * splits
};

// One launch serves up to two problems (dA and dB of one backward): the first `first.blocks` CTAs work on the first.
template <int RP>
__global__ void __launch_bounds__(128) colsum_mma_kernel(ColsumProblem first, ColsumProblem second, long long m_total) {
  constexpr int MT = RP / 16;
  __shared__ __align__(16) unsigned char smem[2][2][kColsumTileBytes];  // [stage][0 = in, 1 = low]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool use_second = blockIdx.x >= first.blocks;
  const ColsumProblem& pr = use_second ? second : first;
  const unsigned local = use_second ? blockIdx.x - first.blocks : blockIdx.x;
  const __nv_bfloat16* __restrict__ low = pr.low;
  const __nv_bfloat16* __restrict__ in = pr.in;
  const long long cols = pr.cols;
  const int tiles_per_split = pr.tiles_per_split;
  float* __restrict__ partial = pr.partial;
  const unsigned slabs = (unsigned)(cols / 64);
  const long long col0 = (local % slabs) * 64LL;
  const int split = (int)(local / slabs);
  const long long tiles_total = (m_total + 63) / 64;
  const long long tile_begin = (long long)split * tiles_per_split;
  long long tile_end = tile_begin + tiles_per_split;
  if (tile_end > tiles_total) tile_end = tiles_total;
  const int ntiles = (int)(tile_end > tile_begin ? tile_end - tile_begin : 0);

  float acc[MT][2][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[i][j][q] = 0.f;

  const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(&smem[0][0][0]);
  auto issue = [&](int tile_idx, int stage) {
    const long long m0 = (tile_begin + tile_idx) * 64;
    const uint32_t in_s = smem_base + (stage * 2 + 0) * kColsumTileBytes;
    const uint32_t low_s = smem_base + (stage * 2 + 1) * kColsumTileBytes;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int chunk = threadIdx.x + i * 128;  // 512 chunks: 64 rows x 8
      const int row = chunk >> 3, c16 = chunk & 7;
      const bool ok = (m0 + row) < m_total;
      const __nv_bfloat16* src = in + (ok ? (m0 + row) : 0) * cols + col0 + c16 * 8;
      cp_async16(in_s + row * kColsumRowBytes + c16 * 16, src, ok);
    }
    constexpr int LOW_CHUNKS = 64 * (RP / 8);
    for (int chunk = threadIdx.x; chunk < LOW_CHUNKS; chunk += 128) {
      const int row = chunk / (RP / 8), c16 = chunk % (RP / 8);
      const bool ok = (m0 + row) < m_total;
      const __nv_bfloat16* src = low + (ok ? (m0 + row) : 0) * 64 + c16 * 8;
      cp_async16(low_s + row * kColsumRowBytes + c16 * 16, src, ok);
    }
    cp_async_commit();
  };

  if (ntiles > 0) issue(0, 0);
  for (int it = 0; it < ntiles; ++it) {
    const int stage = it & 1;
    if (it + 1 < ntiles) {
      issue(it + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t in_s = smem_base + (stage * 2 + 0) * kColsumTileBytes;
    const uint32_t low_s = smem_base + (stage * 2 + 1) * kColsumTileBytes;
    const int q = lane >> 3, rr = lane & 7;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, in_s + (ks * 16 + (q & 1) * 8 + rr) * kColsumRowBytes + (warp * 16 + (q >> 1) * 8) * 2);
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        uint32_t a[4];
        ldmatrix_x4_trans(a, low_s + (ks * 16 + (q >> 1) * 8 + rr) * kColsumRowBytes + (i * 16 + (q & 1) * 8) * 2);
        mma_bf16_16816(acc[i][0], a[0], a[1], a[2], a[3], b[0], b[1]);
        mma_bf16_16816(acc[i][1], a[0], a[1], a[2], a[3], b[2], b[3]);
      }
    }
    __syncthreads();
  }
  const int g = lane >> 2, t = lane & 3;
  float* dst = partial + (long long)split * RP * cols;
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const long long c = col0 + warp * 16 + j * 8 + 2 * t;
      *reinterpret_cast<float2*>(dst + (long long)(i * 16 + g) * cols + c) = make_float2(acc[i][j][0], acc[i][j][1]);
      *reinterpret_cast<float2*>(dst + (long long)(i * 16 + g + 8) * cols + c) =
          make_float2(acc[i][j][2], acc[i][j][3]);
    }
}

// grad (+)= scale * sum_split partial[split][r][c];  transpose writes grad[c, r] (dB), else grad[r, c] (dA).
struct ReduceProblem {
  const float* partial;
  int splits, transpose;
  long long cols;
  float scale;
  float* grad;
  long long total;   // cols * rank
};
__global__ void colsum_reduce_kernel(ReduceProblem first, ReduceProblem second, int rp, int rank, int accumulate) {
  long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const bool use_second = idx >= first.total;
  const ReduceProblem& pr = use_second ? second : first;
  if (use_second) idx -= first.total;
  if (idx >= pr.total) return;
  const int r = pr.transpose ? (int)(idx % rank) : (int)(idx / pr.cols);
  const long long c = pr.transpose ? idx / rank : idx % pr.cols;
  float sum = 0.f;
  for (int s = 0; s < pr.splits; ++s) sum += pr.partial[((long long)s * rp + r) * pr.cols + c];
  sum *= pr.scale;
  pr.grad[idx] = accumulate ? pr.grad[idx] + sum : sum;
}

// Operands of the low-rank block of the standalone input-gradient op: one thread per 8 output elements of either list.
__global__ void dx_lora_prep_kernel(const __nv_bfloat16* __restrict__ lora_grad, int rank, long long m,
                                    const void* __restrict__ lora_a, int a_is_f32, float scaling, int rp, long long k,
                                    __nv_bfloat16* __restrict__ low, __nv_bfloat16* __restrict__ a16) {
  const long long items_low = m * 8;            // [m, 64] in groups of 8
  const long long items_a = (long long)rp * k / 8;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  uint32_t out[4] = {0u, 0u, 0u, 0u};
  if (i < items_low) {
    const long long row = i >> 3;
    const int c0 = (int)(i & 7) * 8;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = c0 + j < rank ? __bfloat162float(lora_grad[row * rank + c0 + j]) : 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) out[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
    *reinterpret_cast<uint4*>(low + row * 64 + c0) = make_uint4(out[0], out[1], out[2], out[3]);
    return;
  }
  i -= items_low;
  if (i < items_a) {
    const long long e = i * 8;
    const int r = (int)(e / k);
    if (r < rank) {
      float v[8];
      if (a_is_f32) {
        const float* a = reinterpret_cast<const float*>(lora_a);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = scaling * __ldg(a + e + j);
      } else {
        const __nv_bfloat16* a = reinterpret_cast<const __nv_bfloat16*>(lora_a);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = scaling * __bfloat162float(a[e + j]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) out[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
    }
    *reinterpret_cast<uint4*>(a16 + e) = make_uint4(out[0], out[1], out[2], out[3]);
  }
}

// ---- host wrappers --------------------------------------------------------------------------------
int lora_prep(const float* a, const float* b, float scaling, int rank, int rp, long long n, long long k,
              __nv_bfloat16* a16, __nv_bfloat16* bs, __nv_bfloat16* bt, const WeightView* w, float* resolved,
              cudaStream_t s) {
  // k and n are multiples of 64 on this path, so the 8-element items never straddle a row
  const long long absmax_blocks = (w != nullptr && resolved != nullptr) ? (w->n * w->k + w->blocksize - 1) / w->blocksize : 0;
  const long long items = (a16 ? (long long)rp * k / 8 : 0) + (bs ? n : 0) + (bt ? n : 0) +
                          (absmax_blocks + 3) / 4;
  if (items == 0) return MOLT_OK;
  WeightView view{};
  if (absmax_blocks > 0) view = *w;
  lora_prep_kernel<<<(unsigned)((items + 255) / 256), 256, 0, s>>>(a, b, scaling, rank, rp, n, k, a16, bs, bt, view,
                                                                    absmax_blocks > 0 ? resolved : nullptr, absmax_blocks);
  return launch_status("lora_prep_kernel");
}

int lora_shadow_refresh(const molt_lora_shadow_item* items, int count, long long max_n, long long max_k, cudaStream_t s) {
  if (count == 0) return MOLT_OK;
  const long long most = 64 * max_k / 8 + 2 * max_n;   // items of the largest adapter (rank <= 64)
  long long blocks = (most + 255) / 256;
  if (blocks > 64) blocks = 64;                        // grid-stride: 64 x count blocks fill the device
  lora_shadow_refresh_kernel<<<dim3((unsigned)blocks, (unsigned)count), 256, 0, s>>>(items);
  return launch_status("lora_shadow_refresh_kernel");
}

int dx_lora_prep(const __nv_bfloat16* lora_grad, int rank, long long m, const void* lora_a, int lora_a_dtype,
                 float scaling, int rp, long long k, __nv_bfloat16* low, __nv_bfloat16* a16, cudaStream_t s) {
  const long long items = m * 8 + (long long)rp * k / 8;   // k is a multiple of 64 on this path
  if (items == 0) return MOLT_OK;
  dx_lora_prep_kernel<<<(unsigned)((items + 255) / 256), 256, 0, s>>>(lora_grad, rank, m, lora_a,
                                                                      lora_a_dtype == MOLT_DTYPE_F32 ? 1 : 0, scaling, rp, k,
                                                                      low, a16);
  return launch_status("dx_lora_prep_kernel");
}

int rowsum_mma(const __nv_bfloat16* in, const __nv_bfloat16* wt, int rp, long long m, long long cols,
               __nv_bfloat16* out, cudaStream_t s) {
  if (m == 0) return MOLT_OK;
  const unsigned grid = (unsigned)((m + 15) / 16);
  // Warps per CTA of 16 rows.  A warp takes every W-th 32-column chunk, two per trip: with few columns a CTA of 16
  // warps is over after one or two trips and is all set-up and final sum, so narrow inputs get smaller CTAs (more of
  // them per SM, more trips each).
#ifdef MOLT_ROWSUM_W
  const int want = MOLT_ROWSUM_W;
#else
  const int want = cols <= 2048 ? 8 : 16;
#endif
  const int cap = rowsum_warps(rp);
  const int warps = want < cap ? want : cap;
#ifdef MOLT_ROWSUM_U
  const bool deep = MOLT_ROWSUM_U == 4;
#else
  const bool deep = cols <= 2048;   // four chunks per trip measured faster for narrow inputs, two for wide ones
#endif
#define MOLT_ROWSUM_CASE(RP, W)                                                        \
  if (rp == RP && warps == W) {                                                        \
    if (deep) rowsum_mma_kernel<RP, W, 4><<<grid, W * 32, 0, s>>>(in, wt, m, cols, out); \
    else rowsum_mma_kernel<RP, W, 2><<<grid, W * 32, 0, s>>>(in, wt, m, cols, out);    \
    return launch_status("rowsum_mma_kernel");                                         \
  }
  MOLT_ROWSUM_CASE(16, 4) MOLT_ROWSUM_CASE(16, 8) MOLT_ROWSUM_CASE(16, 16)
  MOLT_ROWSUM_CASE(32, 4) MOLT_ROWSUM_CASE(32, 8) MOLT_ROWSUM_CASE(32, 16)
  MOLT_ROWSUM_CASE(48, 4) MOLT_ROWSUM_CASE(48, 8)
  MOLT_ROWSUM_CASE(64, 4) MOLT_ROWSUM_CASE(64, 8)
#undef MOLT_ROWSUM_CASE
  return fail(MOLT_E_CAPABILITY, "rowsum_mma: padded rank %d unsupported", rp);
}

int colsum_splits(long long m, long long cols) {
  const long long tiles = (m + 63) / 64;
  const long long slabs = cols / 64;
  long long want = ((long long)sm_count() * 4 + slabs - 1) / slabs;
  if (want > tiles) want = tiles;
  if (want > 64) want = 64;
  if (want < 1) want = 1;
  // make every split non-empty
  const long long per = (tiles + want - 1) / want;
  return (int)((tiles + per - 1) / per);
}

size_t colsum_partial_bytes(long long m, long long cols, int rp) {
  return (size_t)colsum_splits(m, cols) * rp * cols * sizeof(float);
}

// dA = U^T . X ([rp, k]) and dB = scale_b * (T^T . dY)^T ([n, rank]) of one backward: one launch for the split-M
// partial sums of both and one for the two reductions.  partial_a / partial_b: colsum_partial_bytes each.
int colsum_pair(const __nv_bfloat16* u, const __nv_bfloat16* x, long long k, float* partial_a, float* grad_a,
                const __nv_bfloat16* t, const __nv_bfloat16* dy, long long n, float scale_b, float* partial_b,
                float* grad_b, int rp, int rank, long long m, int accumulate, cudaStream_t s) {
  if (rank == 0 || m == 0) return MOLT_OK;
  const long long tiles = (m + 63) / 64;
  ColsumProblem pa{}, pb{};
  ReduceProblem ra{}, rb{};
  auto fill = [&](ColsumProblem& pr, ReduceProblem& rr, const __nv_bfloat16* low, const __nv_bfloat16* in, long long cols,
                  float* partial, float* grad, float scale, int transpose) {
    pr.low = low; pr.in = in; pr.cols = cols; pr.partial = partial;
    pr.splits = colsum_splits(m, cols);
    pr.tiles_per_split = (int)((tiles + pr.splits - 1) / pr.splits);
    pr.blocks = (unsigned)(cols / 64) * (unsigned)pr.splits;
    rr.partial = partial; rr.splits = pr.splits; rr.transpose = transpose; rr.cols = cols; rr.scale = scale;
    rr.grad = grad; rr.total = cols * rank;
  };
  fill(pa, ra, u, x, k, partial_a, grad_a, 1.0f, 0);
  fill(pb, rb, t, dy, n, partial_b, grad_b, scale_b, 1);
  const unsigned grid = pa.blocks + pb.blocks;
  switch (rp) {
    case 16: colsum_mma_kernel<16><<<grid, 128, 0, s>>>(pa, pb, m); break;
    case 32: colsum_mma_kernel<32><<<grid, 128, 0, s>>>(pa, pb, m); break;
    case 48: colsum_mma_kernel<48><<<grid, 128, 0, s>>>(pa, pb, m); break;
    case 64: colsum_mma_kernel<64><<<grid, 128, 0, s>>>(pa, pb, m); break;
    default: return fail(MOLT_E_CAPABILITY, "colsum_mma: padded rank %d unsupported", rp);
  }
  if (int rc = launch_status("colsum_mma_kernel")) return rc;
  const long long total = ra.total + rb.total;
  colsum_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(ra, rb, rp, rank, accumulate);
  return launch_status("colsum_reduce_kernel");
}

}  // namespace molt
