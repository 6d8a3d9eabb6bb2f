// General-shape kernels: any N, K, blocksize and rank (tails such as W[70, 65], rank 7).
// They exist for coverage, not speed: one output element per thread with a 16x16 shared tile over the
// contraction.  The aligned shapes every real projection has take the tcgen05 path instead.
#include "common.cuh"

namespace molt {

__device__ __forceinline__ float decode_weight(const WeightView& w, const float* lut, long long row, long long col) {
  const long long flat = row * w.k + col;
  const uint32_t byte = w.packed[flat >> 1];
  const bool second = flat & 1;
  const bool high = (w.nibble_order == MOLT_NIBBLE_LOW_FIRST) ? second : !second;
  const uint32_t code = high ? (byte >> 4) : (byte & 15u);
  // the dense weight is bf16 on the device path, exactly as the reference's dequantise-to-bf16 makes it
  return __bfloat162float(__float2bfloat16_rn(__fmul_rn(lut[code], load_absmax(w, flat / w.blocksize))));
}

// out[m, j] = sum_c in[m, c] * Wd(c, j)   (+ sum_r low[m, r] * right(r, j))
//   TRANSPOSED_W = false: forward,  c = k, j = n, Wd(c, j) = W[j, c]
//   TRANSPOSED_W = true : backward, c = n, j = k, Wd(c, j) = W[c, j]
// low: bf16 [m, low_ld]; right(r, j): forward scale * B[j, r] (fp32 [n, rank]); backward A[r, j] (fp32/bf16 [rank, k]).
template <bool TRANSPOSED_W, typename RightT>
__global__ void __launch_bounds__(256) general_gemm_kernel(WeightView w, const __nv_bfloat16* __restrict__ in,
                                                           const __nv_bfloat16* __restrict__ low, int low_ld,
                                                           const RightT* __restrict__ right, float scale, int rank,
                                                           __nv_bfloat16* __restrict__ out, long long m_total) {
  __shared__ float lut[16];
  __shared__ float tile_in[16][17];
  __shared__ float tile_w[16][17];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  if (threadIdx.x < 16) lut[threadIdx.x] = w.codebook[threadIdx.x];
  __syncthreads();
  const long long contraction = TRANSPOSED_W ? w.n : w.k;
  const long long out_cols = TRANSPOSED_W ? w.k : w.n;
  const long long row = blockIdx.y * 16LL + ty;
  const long long col = blockIdx.x * 16LL + tx;
  float acc = 0.f;
  for (long long c0 = 0; c0 < contraction; c0 += 16) {
    const long long cin = c0 + tx;
    tile_in[ty][tx] = (row < m_total && cin < contraction) ? __bfloat162float(in[row * contraction + cin]) : 0.f;
    // tile_w[c_local = ty][j_local = tx]
    const long long cw = c0 + ty;
    float wv = 0.f;
    if (cw < contraction && col < out_cols) wv = TRANSPOSED_W ? decode_weight(w, lut, cw, col) : decode_weight(w, lut, col, cw);
    tile_w[ty][tx] = wv;
    __syncthreads();
#pragma unroll
    for (int c = 0; c < 16; ++c) acc += tile_in[ty][c] * tile_w[c][tx];
    __syncthreads();
  }
  if (row < m_total && col < out_cols) {
    if (low != nullptr) {
      // The base result is rounded to bf16 before the adapter term is added (reference nf4_backward.py:127-136).
      float base = __bfloat162float(__float2bfloat16_rn(acc));
      float extra = 0.f;
      for (int r = 0; r < rank; ++r) {
        const float rv = TRANSPOSED_W ? (float)right[(long long)r * out_cols + col] : (float)right[col * rank + r];
        extra += __bfloat162float(low[row * low_ld + r]) * __bfloat162float(__float2bfloat16_rn(rv));
      }
      acc = base + __bfloat162float(__float2bfloat16_rn(extra * scale));
    }
    out[row * out_cols + col] = __float2bfloat16_rn(acc);
  }
}

// low[m, r] = bf16(scale * sum_c in[m, c] * right(c, r)) for r < rank, zero for rank <= r < low_ld.
//   BY_ROWS = true : right(c, r) = mat[r, c]   (mat = A [rank, cols], T = X . A^T)
//   BY_ROWS = false: right(c, r) = mat[c, r]   (mat = B [cols, rank], U = dY . B)
template <bool BY_ROWS>
__global__ void general_rowsum_kernel(const __nv_bfloat16* __restrict__ in, const float* __restrict__ mat,
                                      float scale, long long m_total, long long cols, int rank,
                                      __nv_bfloat16* __restrict__ low, int low_ld) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= m_total * low_ld) return;
  const long long row = idx / low_ld;
  const int r = (int)(idx % low_ld);
  float acc = 0.f;
  if (r < rank) {
    for (long long c = 0; c < cols; ++c) {
      const float mv = BY_ROWS ? mat[(long long)r * cols + c] : mat[c * rank + r];
      acc += __bfloat162float(in[row * cols + c]) * __bfloat162float(__float2bfloat16_rn(mv));
    }
  }
  low[idx] = __float2bfloat16_rn(acc * scale);
}

// grad[...] (+)= scale * sum_m low[m, r] * in[m, c]
//   OUT_BY_ROWS = true : grad is [rank, cols]  (dA = U^T . X)
//   OUT_BY_ROWS = false: grad is [cols, rank]  (dB = dY^T . T)
template <bool OUT_BY_ROWS>
__global__ void general_colsum_kernel(const __nv_bfloat16* __restrict__ low, int low_ld,
                                      const __nv_bfloat16* __restrict__ in, float scale, long long m_total,
                                      long long cols, int rank, float* __restrict__ grad, int accumulate) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= cols * rank) return;
  const int r = OUT_BY_ROWS ? (int)(idx / cols) : (int)(idx % rank);
  const long long c = OUT_BY_ROWS ? idx % cols : idx / rank;
  float acc = 0.f;
  for (long long mrow = 0; mrow < m_total; ++mrow)
    acc += __bfloat162float(low[mrow * low_ld + r]) * __bfloat162float(in[mrow * cols + c]);
  acc *= scale;
  grad[idx] = accumulate ? grad[idx] + acc : acc;
}

// ---- host wrappers used by api.cu ----------------------------------------------------------------
int general_forward(const WeightView& w, const __nv_bfloat16* x, const __nv_bfloat16* t, int t_ld, const float* lora_b,
                    float scaling, int rank, __nv_bfloat16* y, long long m, cudaStream_t s) {
  dim3 grid((unsigned)((w.n + 15) / 16), (unsigned)((m + 15) / 16));
  general_gemm_kernel<false, float><<<grid, 256, 0, s>>>(w, x, t, t_ld, lora_b, scaling, rank, y, m);
  return launch_status("general_gemm_kernel<forward>");
}

int general_backward_input(const WeightView& w, const __nv_bfloat16* dy, const __nv_bfloat16* u, int u_ld,
                           const void* lora_a, int lora_a_dtype, float scaling, int rank, __nv_bfloat16* dx,
                           long long m, cudaStream_t s) {
  dim3 grid((unsigned)((w.k + 15) / 16), (unsigned)((m + 15) / 16));
  if (lora_a_dtype == MOLT_DTYPE_BF16)
    general_gemm_kernel<true, __nv_bfloat16><<<grid, 256, 0, s>>>(w, dy, u, u_ld, (const __nv_bfloat16*)lora_a,
                                                                  scaling, rank, dx, m);
  else
    general_gemm_kernel<true, float><<<grid, 256, 0, s>>>(w, dy, u, u_ld, (const float*)lora_a, scaling, rank, dx, m);
  return launch_status("general_gemm_kernel<backward>");
}

int general_rowsum(bool by_rows, const __nv_bfloat16* in, const float* mat, float scale, long long m, long long cols,
                   int rank, __nv_bfloat16* low, int low_ld, cudaStream_t s) {
  const long long total = m * low_ld;
  if (total == 0) return MOLT_OK;
  const unsigned grid = (unsigned)((total + 127) / 128);
  if (by_rows) general_rowsum_kernel<true><<<grid, 128, 0, s>>>(in, mat, scale, m, cols, rank, low, low_ld);
  else general_rowsum_kernel<false><<<grid, 128, 0, s>>>(in, mat, scale, m, cols, rank, low, low_ld);
  return launch_status("general_rowsum_kernel");
}

int general_colsum(bool out_by_rows, const __nv_bfloat16* low, int low_ld, const __nv_bfloat16* in, float scale,
                   long long m, long long cols, int rank, float* grad, int accumulate, cudaStream_t s) {
  const long long total = cols * rank;
  if (total == 0) return MOLT_OK;
  const unsigned grid = (unsigned)((total + 127) / 128);
  if (out_by_rows) general_colsum_kernel<true><<<grid, 128, 0, s>>>(low, low_ld, in, scale, m, cols, rank, grad, accumulate);
  else general_colsum_kernel<false><<<grid, 128, 0, s>>>(low, low_ld, in, scale, m, cols, rank, grad, accumulate);
  return launch_status("general_colsum_kernel");
}

}  // namespace molt
