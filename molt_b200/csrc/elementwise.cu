// HBM-bound kernels: NF4 dequantisation, absmax resolution, SwiGLU forward/backward, RMSNorm replay.
// Each thread moves 16-byte vectors; grids are sized in multiples of the SM count.
#include <math.h>

#include "common.cuh"

namespace molt {

// ------------------------------------------------------------------------------------------------
// NF4 dequantisation.  One thread expands 16 packed bytes (32 codes).  Bit-exact contract:
// value = fp32(codebook[code]) * fp32(absmax) with one IEEE multiply, then one round-to-nearest cast.
// ------------------------------------------------------------------------------------------------
template <typename OutT>
__device__ __forceinline__ void store_pair(OutT* out, long long idx, float a, float b, long long elements);

template <>
__device__ __forceinline__ void store_pair<float>(float* out, long long idx, float a, float b, long long elements) {
  if (idx < elements) out[idx] = a;
  if (idx + 1 < elements) out[idx + 1] = b;
}
template <>
__device__ __forceinline__ void store_pair<__nv_bfloat16>(__nv_bfloat16* out, long long idx, float a, float b,
                                                          long long elements) {
  if (idx < elements) out[idx] = __float2bfloat16_rn(a);
  if (idx + 1 < elements) out[idx + 1] = __float2bfloat16_rn(b);
}

template <typename OutT, bool ALIGNED>
__global__ void __launch_bounds__(256) nf4_dequant_kernel(WeightView w, OutT* __restrict__ out, long long elements,
                                                          long long packed_bytes) {
  __shared__ float lut[16];
  if (threadIdx.x < 16) lut[threadIdx.x] = w.codebook[threadIdx.x];
  __syncthreads();
  const int lo_shift = w.nibble_order == MOLT_NIBBLE_LOW_FIRST ? 0 : 4;
  const int hi_shift = 4 - lo_shift;
  const long long vectors = (packed_bytes + 15) / 16;
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < vectors;
       v += (long long)gridDim.x * blockDim.x) {
    const long long byte0 = v * 16;
    const long long elem0 = byte0 * 2;
    if (ALIGNED) {
      // 32 elements, all inside one absmax block (blocksize % 32 == 0) and inside the tensor.
      uint4 raw = __ldcs(reinterpret_cast<const uint4*>(w.packed + byte0));
      const float scale = load_absmax(w, elem0 / w.blocksize);
      uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
      float vals[32];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          uint32_t byte = (words[i] >> (8 * b)) & 0xffu;
          vals[i * 8 + b * 2] = __fmul_rn(lut[(byte >> lo_shift) & 15u], scale);
          vals[i * 8 + b * 2 + 1] = __fmul_rn(lut[(byte >> hi_shift) & 15u], scale);
        }
      }
      if (sizeof(OutT) == 2) {
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out) + elem0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 o;
          o.x = pack_bf16x2(vals[q * 8 + 0], vals[q * 8 + 1]);
          o.y = pack_bf16x2(vals[q * 8 + 2], vals[q * 8 + 3]);
          o.z = pack_bf16x2(vals[q * 8 + 4], vals[q * 8 + 5]);
          o.w = pack_bf16x2(vals[q * 8 + 6], vals[q * 8 + 7]);
          __stcs(dst + q, o);
        }
      } else {
        float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + elem0);
#pragma unroll
        for (int q = 0; q < 8; ++q)
          __stcs(dst + q, make_float4(vals[q * 4], vals[q * 4 + 1], vals[q * 4 + 2], vals[q * 4 + 3]));
      }
    } else {
      for (int b = 0; b < 16; ++b) {
        const long long byte_idx = byte0 + b;
        if (byte_idx >= packed_bytes) break;
        const long long e = byte_idx * 2;
        if (e >= elements) break;
        const uint32_t byte = w.packed[byte_idx];
        const float s0 = load_absmax(w, e / w.blocksize);
        const float s1 = (e + 1 < elements) ? load_absmax(w, (e + 1) / w.blocksize) : 0.f;
        store_pair<OutT>(out, e, __fmul_rn(lut[(byte >> lo_shift) & 15u], s0),
                         __fmul_rn(lut[(byte >> hi_shift) & 15u], s1), elements);
      }
    }
  }
}

__global__ void resolve_absmax_kernel(WeightView w, float* __restrict__ out, long long blocks) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < blocks;
       i += (long long)gridDim.x * blockDim.x)
    out[i] = load_absmax(w, i);
}

// ------------------------------------------------------------------------------------------------
// SwiGLU.  fp32 arithmetic from the stored dtype, a single rounding on store.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float sigmoidf_(float g) { return 1.0f / (1.0f + expf(-g)); }

template <bool WRITE_H>
__global__ void __launch_bounds__(256) swiglu_bf16_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up,
                                                          const uint4* __restrict__ grad, uint4* __restrict__ out_h,
                                                          uint4* __restrict__ dgate, uint4* __restrict__ dup,
                                                          long long vectors, bool backward) {
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < vectors;
       v += (long long)gridDim.x * blockDim.x) {
    const uint4 g4 = __ldcs(gate + v);
    const uint4 u4 = __ldcs(up + v);
    const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w};
    const uint32_t uw[4] = {u4.x, u4.y, u4.z, u4.w};
    if (!backward) {
      uint32_t hw[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float g0 = bf16_lo(gw[i]), g1 = bf16_hi(gw[i]);
        const float u0 = bf16_lo(uw[i]), u1 = bf16_hi(uw[i]);
        hw[i] = pack_bf16x2(g0 * sigmoidf_(g0) * u0, g1 * sigmoidf_(g1) * u1);
      }
      __stcs(out_h + v, make_uint4(hw[0], hw[1], hw[2], hw[3]));
    } else {
      const uint4 d4 = __ldcs(grad + v);
      const uint32_t dw[4] = {d4.x, d4.y, d4.z, d4.w};
      uint32_t og[4], ou[4], oh[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float g[2] = {bf16_lo(gw[i]), bf16_hi(gw[i])};
        float u[2] = {bf16_lo(uw[i]), bf16_hi(uw[i])};
        float d[2] = {bf16_lo(dw[i]), bf16_hi(dw[i])};
        float rg[2], ru[2], rh[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const float sig = sigmoidf_(g[j]);
          const float silu = g[j] * sig;
          rg[j] = d[j] * u[j] * (sig * (1.0f + g[j] * (1.0f - sig)));
          ru[j] = d[j] * silu;
          rh[j] = silu * u[j];
        }
        og[i] = pack_bf16x2(rg[0], rg[1]);
        ou[i] = pack_bf16x2(ru[0], ru[1]);
        oh[i] = pack_bf16x2(rh[0], rh[1]);
      }
      __stcs(dgate + v, make_uint4(og[0], og[1], og[2], og[3]));
      __stcs(dup + v, make_uint4(ou[0], ou[1], ou[2], ou[3]));
      if (WRITE_H) __stcs(out_h + v, make_uint4(oh[0], oh[1], oh[2], oh[3]));
    }
  }
}

// Scalar kernel: fp32 tensors, and the unaligned head/tail of bf16 tensors.
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__global__ void swiglu_scalar_kernel(const T* __restrict__ gate, const T* __restrict__ up, const T* __restrict__ grad,
                                     T* __restrict__ out_h, T* __restrict__ dgate, T* __restrict__ dup,
                                     long long begin, long long count, bool backward) {
  for (long long i = begin + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
       i += (long long)gridDim.x * blockDim.x) {
    const float g = to_f32<T>(gate[i]);
    const float u = to_f32<T>(up[i]);
    const float sig = sigmoidf_(g);
    const float silu = g * sig;
    if (!backward) {
      out_h[i] = from_f32<T>(silu * u);
    } else {
      const float d = to_f32<T>(grad[i]);
      dgate[i] = from_f32<T>(d * u * (sig * (1.0f + g * (1.0f - sig))));
      dup[i] = from_f32<T>(d * silu);
      if (out_h != nullptr) out_h[i] = from_f32<T>(silu * u);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Frozen RMSNorm, forward and backward: one warp per row, 16-byte loads, fp32 reduction, bf16 in and out.
//   forward : out = bf16(x * rsqrt(mean(x^2) + eps) * (w + offset))
//   backward: dx  = bf16(inv * (dy (w + offset) - x inv * mean(dy (w + offset) * x inv)))   (weight frozen: no dw)
// The row is read twice; the second pass finds it in L1.  Rows whose width is not a multiple of 8 (or unaligned
// tensors) take the scalar loops.
// ------------------------------------------------------------------------------------------------
template <typename WT>
__device__ __forceinline__ void load_weight8(const WT* w, long long c, float offset, float (&out)[8]);
template <>
__device__ __forceinline__ void load_weight8<float>(const float* w, long long c, float offset, float (&out)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(w + c)), b = __ldg(reinterpret_cast<const float4*>(w + c + 4));
  out[0] = a.x + offset; out[1] = a.y + offset; out[2] = a.z + offset; out[3] = a.w + offset;
  out[4] = b.x + offset; out[5] = b.y + offset; out[6] = b.z + offset; out[7] = b.w + offset;
}
template <>
__device__ __forceinline__ void load_weight8<__nv_bfloat16>(const __nv_bfloat16* w, long long c, float offset,
                                                            float (&out)[8]) {
  const uint4 a = __ldg(reinterpret_cast<const uint4*>(w + c));
  const uint32_t v[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = bf16_lo(v[i]) + offset;
    out[2 * i + 1] = bf16_hi(v[i]) + offset;
  }
}
__device__ __forceinline__ void unpack8(const uint4& raw, float (&out)[8]) {
  const uint32_t v[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = bf16_lo(v[i]);
    out[2 * i + 1] = bf16_hi(v[i]);
  }
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename WT, bool VEC, bool BACKWARD>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const WT* __restrict__ weight,
                                                      const __nv_bfloat16* __restrict__ grad, float eps,
                                                      float weight_offset, __nv_bfloat16* __restrict__ out,
                                                      long long rows, long long width) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp; row < rows; row += warps) {
    const __nv_bfloat16* src = x + row * width;
    const __nv_bfloat16* gsrc = BACKWARD ? grad + row * width : nullptr;
    __nv_bfloat16* dst = out + row * width;
    float sum = 0.f, dot = 0.f;   // sum of x^2; backward: sum of dy (w + offset) x
    if (VEC) {
      for (long long c = lane * 8LL; c < width; c += 256) {
        float xv[8];
        unpack8(*reinterpret_cast<const uint4*>(src + c), xv);
#pragma unroll
        for (int i = 0; i < 8; ++i) sum += xv[i] * xv[i];
        if (BACKWARD) {
          float gv[8], wv[8];
          unpack8(__ldcs(reinterpret_cast<const uint4*>(gsrc + c)), gv);
          load_weight8<WT>(weight, c, weight_offset, wv);
#pragma unroll
          for (int i = 0; i < 8; ++i) dot += gv[i] * wv[i] * xv[i];
        }
      }
    } else {
      for (long long c = lane; c < width; c += 32) {
        const float v = __bfloat162float(src[c]);
        sum += v * v;
        if (BACKWARD) dot += __bfloat162float(gsrc[c]) * (to_f32<WT>(weight[c]) + weight_offset) * v;
      }
    }
    sum = warp_sum(sum);
    const float inv = rsqrtf(sum / (float)width + eps);
    float correction = 0.f;
    if (BACKWARD) correction = warp_sum(dot) * inv / (float)width;   // mean(weighted * normalized)
    if (VEC) {
      for (long long c = lane * 8LL; c < width; c += 256) {
        float xv[8], wv[8], res[8];
        unpack8(*reinterpret_cast<const uint4*>(src + c), xv);
        load_weight8<WT>(weight, c, weight_offset, wv);
        if (!BACKWARD) {
#pragma unroll
          for (int i = 0; i < 8; ++i) res[i] = xv[i] * inv * wv[i];
        } else {
          float gv[8];
          unpack8(*reinterpret_cast<const uint4*>(gsrc + c), gv);
#pragma unroll
          for (int i = 0; i < 8; ++i) res[i] = inv * (gv[i] * wv[i] - xv[i] * inv * correction);
        }
        __stcs(reinterpret_cast<uint4*>(dst + c), make_uint4(pack_bf16x2(res[0], res[1]), pack_bf16x2(res[2], res[3]),
                                                              pack_bf16x2(res[4], res[5]), pack_bf16x2(res[6], res[7])));
      }
    } else {
      for (long long c = lane; c < width; c += 32) {
        const float v = __bfloat162float(src[c]);
        const float w = to_f32<WT>(weight[c]) + weight_offset;
        dst[c] = __float2bfloat16_rn(!BACKWARD ? v * inv * w
                                               : inv * (__bfloat162float(gsrc[c]) * w - v * inv * correction));
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Residual add fused with the RMSNorm that follows it (one pass over the hidden states instead of two):
//   forward : sum = bf16(x + delta);  out = bf16(sum * rsqrt(mean(sum^2) + eps) * (w + offset))
//   backward: grad_x = bf16(grad_sum + inv * (dy (w + offset) - sum inv * mean(dy (w + offset) * sum inv)))
// The norm is taken from the ROUNDED sum, the tensor the backward sees.  One warp per row, width a multiple of 8.
// ------------------------------------------------------------------------------------------------
template <typename WT, bool BACKWARD>
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ a,      // fwd: x;     bwd: sum
                                                          const __nv_bfloat16* __restrict__ b,      // fwd: delta; bwd: dy
                                                          const __nv_bfloat16* __restrict__ c_in,   // bwd: grad_sum
                                                          const WT* __restrict__ weight, float eps, float weight_offset,
                                                          __nv_bfloat16* __restrict__ sum_out,      // fwd only
                                                          __nv_bfloat16* __restrict__ out, long long rows,
                                                          long long width) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp; row < rows; row += warps) {
    const long long base = row * width;
    float sq = 0.f, dot = 0.f;
    for (long long c = lane * 8LL; c < width; c += 256) {
      float av[8], bv[8];
      unpack8(__ldcs(reinterpret_cast<const uint4*>(a + base + c)), av);
      unpack8(__ldcs(reinterpret_cast<const uint4*>(b + base + c)), bv);
      if (!BACKWARD) {
        uint32_t packed[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) packed[i] = pack_bf16x2(av[2 * i] + bv[2 * i], av[2 * i + 1] + bv[2 * i + 1]);
        const uint4 stored = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        *reinterpret_cast<uint4*>(sum_out + base + c) = stored;   // re-read below, from L1/L2
        float sv[8];
        unpack8(stored, sv);
#pragma unroll
        for (int i = 0; i < 8; ++i) sq += sv[i] * sv[i];
      } else {
        float wv[8];
        load_weight8<WT>(weight, c, weight_offset, wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          sq += av[i] * av[i];
          dot += bv[i] * wv[i] * av[i];
        }
      }
    }
    sq = warp_sum(sq);
    const float inv = rsqrtf(sq / (float)width + eps);
    float correction = 0.f;
    if (BACKWARD) correction = warp_sum(dot) * inv / (float)width;
    __syncwarp();
    for (long long c = lane * 8LL; c < width; c += 256) {
      float wv[8], res[8];
      load_weight8<WT>(weight, c, weight_offset, wv);
      if (!BACKWARD) {
        float sv[8];
        unpack8(*reinterpret_cast<const uint4*>(sum_out + base + c), sv);   // this lane's own store
#pragma unroll
        for (int i = 0; i < 8; ++i) res[i] = sv[i] * inv * wv[i];
      } else {
        float sv[8], gv[8], rv[8];
        unpack8(*reinterpret_cast<const uint4*>(a + base + c), sv);
        unpack8(*reinterpret_cast<const uint4*>(b + base + c), gv);
        unpack8(__ldcs(reinterpret_cast<const uint4*>(c_in + base + c)), rv);
#pragma unroll
        for (int i = 0; i < 8; ++i) res[i] = rv[i] + inv * (gv[i] * wv[i] - sv[i] * inv * correction);
      }
      __stcs(reinterpret_cast<uint4*>(out + base + c), make_uint4(pack_bf16x2(res[0], res[1]), pack_bf16x2(res[2], res[3]),
                                                                  pack_bf16x2(res[4], res[5]), pack_bf16x2(res[6], res[7])));
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Rotary position embedding (in place or into other buffers) on the query and key projections of a whole batch:
//   (x1, x2) -> (x1 cos - x2 sin, x2 cos + x1 sin),   x1 / x2 = first / second half of a head's vector;
// inverse = 1 applies the transposed rotation (the gradient).  fp32 arithmetic, one rounding.
// q [batch, seq, heads, d], k [batch, seq, kv_heads, d], cos / sin [seq, d] (both halves equal), all bf16.
// One thread rotates 8 elements of the first half with their partners in the second half.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rope_kernel(const __nv_bfloat16* q, const __nv_bfloat16* k, __nv_bfloat16* q_out,
                                                   __nv_bfloat16* k_out, const __nv_bfloat16* __restrict__ cos_t,
                                                   const __nv_bfloat16* __restrict__ sin_t, long long tokens, int seq,
                                                   int heads, int kv_heads, int d, float sign) {
  const int per_vec = d / 16;                       // threads per head vector
  const long long vectors = tokens * (heads + kv_heads);
  const long long total = vectors * per_vec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long vec = i / per_vec;
    const int part = (int)(i - vec * per_vec);
    const long long token = vec / (heads + kv_heads);
    const int head = (int)(vec - token * (heads + kv_heads));
    const long long offset = head < heads ? (token * heads + head) * (long long)d
                                          : (token * kv_heads + (head - heads)) * (long long)d;
    const __nv_bfloat16* x = (head < heads ? q : k) + offset;
    __nv_bfloat16* y = (head < heads ? q_out : k_out) + offset;   // may be x itself: a thread reads before it writes
    const int pos = (int)(token % seq);
    float x1[8], x2[8], cv[8], sv[8];
    unpack8(*reinterpret_cast<const uint4*>(x + part * 8), x1);
    unpack8(*reinterpret_cast<const uint4*>(x + d / 2 + part * 8), x2);
    unpack8(__ldg(reinterpret_cast<const uint4*>(cos_t + (long long)pos * d + part * 8)), cv);
    unpack8(__ldg(reinterpret_cast<const uint4*>(sin_t + (long long)pos * d + part * 8)), sv);
    float o1[8], o2[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      o1[j] = x1[j] * cv[j] - sign * x2[j] * sv[j];
      o2[j] = x2[j] * cv[j] + sign * x1[j] * sv[j];
    }
    *reinterpret_cast<uint4*>(y + part * 8) = make_uint4(pack_bf16x2(o1[0], o1[1]), pack_bf16x2(o1[2], o1[3]),
                                                         pack_bf16x2(o1[4], o1[5]), pack_bf16x2(o1[6], o1[7]));
    *reinterpret_cast<uint4*>(y + d / 2 + part * 8) = make_uint4(pack_bf16x2(o2[0], o2[1]), pack_bf16x2(o2[2], o2[3]),
                                                                 pack_bf16x2(o2[4], o2[5]), pack_bf16x2(o2[6], o2[7]));
  }
}

// ------------------------------------------------------------------------------------------------
// AdamW over flat fp32 arrays (decoupled weight decay, bias correction as torch.optim.AdamW computes it).
// All adapter parameters, their gradients and both moments live in flat arenas, so one launch steps every adapter.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) adamw_kernel(float4* __restrict__ param, const float4* __restrict__ grad,
                                                    float4* __restrict__ exp_avg, float4* __restrict__ exp_avg_sq,
                                                    long long vectors, float lr, float beta1, float beta2, float eps,
                                                    float weight_decay, float bias1, float bias2_sqrt, float grad_scale) {
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < vectors;
       v += (long long)gridDim.x * blockDim.x) {
    const float4 g4 = __ldcs(grad + v);
    float4 p4 = param[v], m4 = exp_avg[v], s4 = exp_avg_sq[v];
    float g[4] = {g4.x, g4.y, g4.z, g4.w};
    float p[4] = {p4.x, p4.y, p4.z, p4.w}, m[4] = {m4.x, m4.y, m4.z, m4.w}, s[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float gi = g[i] * grad_scale;
      p[i] *= 1.0f - lr * weight_decay;
      m[i] = beta1 * m[i] + (1.0f - beta1) * gi;
      s[i] = beta2 * s[i] + (1.0f - beta2) * gi * gi;
      const float denom = sqrtf(s[i]) / bias2_sqrt + eps;
      p[i] -= (lr / bias1) * (m[i] / denom);
    }
    param[v] = make_float4(p[0], p[1], p[2], p[3]);
    exp_avg[v] = make_float4(m[0], m[1], m[2], m[3]);
    exp_avg_sq[v] = make_float4(s[0], s[1], s[2], s[3]);
  }
}

static int grid_for(long long work_items, int threads, int waves_cap = 8) {
  long long blocks = (work_items + threads - 1) / threads;
  long long cap = (long long)sm_count() * waves_cap;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace molt

using namespace molt;

extern "C" int molt_nf4_dequant(const molt_nf4_desc* w, void* out, int out_dtype, uintptr_t stream) {
  int64_t blocks = 0;
  if (int rc = check_desc(w, &blocks)) return rc;
  MOLT_REQUIRE(out != nullptr, MOLT_E_VALUE, "molt_nf4_dequant: out is NULL");
  MOLT_REQUIRE(out_dtype == MOLT_DTYPE_BF16 || out_dtype == MOLT_DTYPE_F32, MOLT_E_CAPABILITY,
               "molt_nf4_dequant: output dtype must be bf16 or fp32");
  const long long elements = w->n * w->k;
  const long long packed_bytes = blocks * w->blocksize / 2;
  const bool aligned = (w->blocksize % 32 == 0) && (elements % 32 == 0) && aligned16(w->packed) && aligned16(out);
  WeightView view = make_view(w);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long vectors = (packed_bytes + 15) / 16;
  const int grid = grid_for(vectors, 256, 16);
  if (out_dtype == MOLT_DTYPE_BF16) {
    auto* o = reinterpret_cast<__nv_bfloat16*>(out);
    if (aligned) nf4_dequant_kernel<__nv_bfloat16, true><<<grid, 256, 0, s>>>(view, o, elements, packed_bytes);
    else nf4_dequant_kernel<__nv_bfloat16, false><<<grid, 256, 0, s>>>(view, o, elements, packed_bytes);
  } else {
    auto* o = reinterpret_cast<float*>(out);
    if (aligned) nf4_dequant_kernel<float, true><<<grid, 256, 0, s>>>(view, o, elements, packed_bytes);
    else nf4_dequant_kernel<float, false><<<grid, 256, 0, s>>>(view, o, elements, packed_bytes);
  }
  return launch_status("nf4_dequant_kernel");
}

extern "C" int molt_nf4_resolve_absmax(const molt_nf4_desc* w, float* out, uintptr_t stream) {
  int64_t blocks = 0;
  if (int rc = check_desc(w, &blocks)) return rc;
  MOLT_REQUIRE(out != nullptr, MOLT_E_VALUE, "molt_nf4_resolve_absmax: out is NULL");
  resolve_absmax_kernel<<<grid_for(blocks, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(make_view(w), out,
                                                                                                  blocks);
  return launch_status("resolve_absmax_kernel");
}

static int swiglu_launch(const void* gate, const void* up, const void* grad, void* out_h, void* dgate, void* dup,
                         int64_t count, int dtype, bool backward, uintptr_t stream) {
  MOLT_REQUIRE(count >= 0, MOLT_E_VALUE, "swiglu: negative element count");
  MOLT_REQUIRE(dtype == MOLT_DTYPE_BF16 || dtype == MOLT_DTYPE_F32, MOLT_E_CAPABILITY,
               "swiglu: dtype must be bf16 or fp32");
  MOLT_REQUIRE(gate && up && (backward ? (grad && dgate && dup) : out_h != nullptr), MOLT_E_VALUE,
               "swiglu: NULL tensor pointer");
  if (count == 0) return MOLT_OK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == MOLT_DTYPE_F32) {
    swiglu_scalar_kernel<float><<<grid_for(count, 256, 16), 256, 0, s>>>(
        (const float*)gate, (const float*)up, (const float*)grad, (float*)out_h, (float*)dgate, (float*)dup, 0, count,
        backward);
    return launch_status("swiglu_scalar_kernel<float>");
  }
  const bool vec_ok = aligned16(gate) && aligned16(up) && (!backward || (aligned16(grad) && aligned16(dgate) &&
                                                                         aligned16(dup))) &&
                      (out_h == nullptr || aligned16(out_h));
  long long vectors = vec_ok ? count / 8 : 0;
  if (vectors > 0) {
    const int grid = grid_for(vectors, 256, 16);
    if (backward && out_h != nullptr)
      swiglu_bf16_kernel<true><<<grid, 256, 0, s>>>((const uint4*)gate, (const uint4*)up, (const uint4*)grad,
                                                    (uint4*)out_h, (uint4*)dgate, (uint4*)dup, vectors, true);
    else
      swiglu_bf16_kernel<false><<<grid, 256, 0, s>>>((const uint4*)gate, (const uint4*)up, (const uint4*)grad,
                                                     (uint4*)out_h, (uint4*)dgate, (uint4*)dup, vectors, backward);
    if (int rc = launch_status("swiglu_bf16_kernel")) return rc;
  }
  if (vectors * 8 < count) {
    swiglu_scalar_kernel<__nv_bfloat16><<<grid_for(count - vectors * 8, 256), 256, 0, s>>>(
        (const __nv_bfloat16*)gate, (const __nv_bfloat16*)up, (const __nv_bfloat16*)grad, (__nv_bfloat16*)out_h,
        (__nv_bfloat16*)dgate, (__nv_bfloat16*)dup, vectors * 8, count, backward);
    if (int rc = launch_status("swiglu_scalar_kernel<bf16>")) return rc;
  }
  return MOLT_OK;
}

extern "C" int molt_swiglu_fwd(const void* gate, const void* up, void* out, int64_t count, int dtype,
                               uintptr_t stream) {
  return swiglu_launch(gate, up, nullptr, out, nullptr, nullptr, count, dtype, false, stream);
}

extern "C" int molt_swiglu_bwd(const void* grad_out, const void* gate, const void* up, void* dgate, void* dup,
                               void* h_out, int64_t count, int dtype, uintptr_t stream) {
  return swiglu_launch(gate, up, grad_out, h_out, dgate, dup, count, dtype, true, stream);
}

static int rmsnorm_launch(const char* who, const void* x, const void* weight, int weight_dtype, const void* grad, float eps,
                          float weight_offset, void* out, int64_t rows, int64_t width, uintptr_t stream) {
  MOLT_REQUIRE(x && weight && out, MOLT_E_VALUE, "%s: NULL tensor pointer", who);
  MOLT_REQUIRE(rows >= 0 && width > 0, MOLT_E_VALUE, "%s: bad shape", who);
  MOLT_REQUIRE(weight_dtype == MOLT_DTYPE_BF16 || weight_dtype == MOLT_DTYPE_F32, MOLT_E_CAPABILITY,
               "%s: weight dtype must be bf16 or fp32", who);
  if (rows == 0) return MOLT_OK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = grid_for(rows * 32, 256, 8);
  const bool vec = width % 8 == 0 && aligned16(x) && aligned16(out) && aligned16(weight) && (grad == nullptr || aligned16(grad));
  auto* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  auto* gb = reinterpret_cast<const __nv_bfloat16*>(grad);
  auto* ob = reinterpret_cast<__nv_bfloat16*>(out);
#define MOLT_RMS_LAUNCH(WT, VEC, BWD)                                                                       \
  rmsnorm_kernel<WT, VEC, BWD><<<grid, 256, 0, s>>>(xb, reinterpret_cast<const WT*>(weight), gb, eps, weight_offset, ob, \
                                                    rows, width)
  const bool f32 = weight_dtype == MOLT_DTYPE_F32, bwd = grad != nullptr;
  if (f32 && vec && !bwd) MOLT_RMS_LAUNCH(float, true, false);
  else if (f32 && vec && bwd) MOLT_RMS_LAUNCH(float, true, true);
  else if (f32 && !vec && !bwd) MOLT_RMS_LAUNCH(float, false, false);
  else if (f32 && !vec && bwd) MOLT_RMS_LAUNCH(float, false, true);
  else if (!f32 && vec && !bwd) MOLT_RMS_LAUNCH(__nv_bfloat16, true, false);
  else if (!f32 && vec && bwd) MOLT_RMS_LAUNCH(__nv_bfloat16, true, true);
  else if (!f32 && !vec && !bwd) MOLT_RMS_LAUNCH(__nv_bfloat16, false, false);
  else MOLT_RMS_LAUNCH(__nv_bfloat16, false, true);
#undef MOLT_RMS_LAUNCH
  return launch_status("rmsnorm_kernel");
}

extern "C" int molt_rmsnorm_fwd(const void* x, const void* weight, int weight_dtype, float eps, float weight_offset,
                                void* out, int64_t rows, int64_t width, uintptr_t stream) {
  return rmsnorm_launch("molt_rmsnorm_fwd", x, weight, weight_dtype, nullptr, eps, weight_offset, out, rows, width, stream);
}

extern "C" int molt_rmsnorm_bwd(const void* grad_out, const void* x, const void* weight, int weight_dtype, float eps,
                                float weight_offset, void* grad_x, int64_t rows, int64_t width, uintptr_t stream) {
  MOLT_REQUIRE(grad_out != nullptr, MOLT_E_VALUE, "molt_rmsnorm_bwd: NULL tensor pointer");
  return rmsnorm_launch("molt_rmsnorm_bwd", x, weight, weight_dtype, grad_out, eps, weight_offset, grad_x, rows, width,
                        stream);
}

static int add_rmsnorm_launch(const char* who, const void* a, const void* b, const void* c, const void* weight,
                              int weight_dtype, float eps, float weight_offset, void* sum_out, void* out, int64_t rows,
                              int64_t width, bool backward, uintptr_t stream) {
  MOLT_REQUIRE(a && b && weight && out && (backward ? c != nullptr : sum_out != nullptr), MOLT_E_VALUE,
               "%s: NULL tensor pointer", who);
  MOLT_REQUIRE(rows >= 0 && width > 0 && width % 8 == 0, MOLT_E_VALUE, "%s: width must be a positive multiple of 8", who);
  MOLT_REQUIRE(weight_dtype == MOLT_DTYPE_F32 || weight_dtype == MOLT_DTYPE_BF16, MOLT_E_CAPABILITY,
               "%s: weight dtype must be bf16 or fp32", who);
  MOLT_REQUIRE(aligned16(a) && aligned16(b) && aligned16(out) && aligned16(weight) && (c == nullptr || aligned16(c)) &&
                   (sum_out == nullptr || aligned16(sum_out)),
               MOLT_E_VALUE, "%s: tensors must be 16-byte aligned", who);
  if (rows == 0) return MOLT_OK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long blocks = (rows + 7) / 8;   // eight warps (rows) per block
  const unsigned grid = (unsigned)(blocks < (long long)sm_count() * 8 ? blocks : (long long)sm_count() * 8);
  auto* ab = reinterpret_cast<const __nv_bfloat16*>(a);
  auto* bb = reinterpret_cast<const __nv_bfloat16*>(b);
  auto* cb = reinterpret_cast<const __nv_bfloat16*>(c);
  auto* sb = reinterpret_cast<__nv_bfloat16*>(sum_out);
  auto* ob = reinterpret_cast<__nv_bfloat16*>(out);
  if (weight_dtype == MOLT_DTYPE_F32) {
    auto* w = reinterpret_cast<const float*>(weight);
    if (backward) add_rmsnorm_kernel<float, true><<<grid, 256, 0, s>>>(ab, bb, cb, w, eps, weight_offset, sb, ob, rows, width);
    else add_rmsnorm_kernel<float, false><<<grid, 256, 0, s>>>(ab, bb, cb, w, eps, weight_offset, sb, ob, rows, width);
  } else {
    auto* w = reinterpret_cast<const __nv_bfloat16*>(weight);
    if (backward) add_rmsnorm_kernel<__nv_bfloat16, true><<<grid, 256, 0, s>>>(ab, bb, cb, w, eps, weight_offset, sb, ob, rows, width);
    else add_rmsnorm_kernel<__nv_bfloat16, false><<<grid, 256, 0, s>>>(ab, bb, cb, w, eps, weight_offset, sb, ob, rows, width);
  }
  return launch_status("add_rmsnorm_kernel");
}

extern "C" int molt_add_rmsnorm_fwd(const void* x, const void* delta, const void* weight, int weight_dtype, float eps,
                                    float weight_offset, void* sum_out, void* out, int64_t rows, int64_t width,
                                    uintptr_t stream) {
  return add_rmsnorm_launch("molt_add_rmsnorm_fwd", x, delta, nullptr, weight, weight_dtype, eps, weight_offset, sum_out,
                            out, rows, width, false, stream);
}

extern "C" int molt_add_rmsnorm_bwd(const void* grad_out, const void* grad_sum, const void* sum, const void* weight,
                                    int weight_dtype, float eps, float weight_offset, void* grad_x, int64_t rows,
                                    int64_t width, uintptr_t stream) {
  return add_rmsnorm_launch("molt_add_rmsnorm_bwd", sum, grad_out, grad_sum, weight, weight_dtype, eps, weight_offset,
                            nullptr, grad_x, rows, width, true, stream);
}

extern "C" int molt_rope(const void* q, const void* k, void* q_out, void* k_out, const void* cos_table,
                         const void* sin_table, int64_t batch, int64_t seq, int heads, int kv_heads, int head_dim,
                         int inverse, uintptr_t stream) {
  MOLT_REQUIRE(q && k && q_out && k_out && cos_table && sin_table, MOLT_E_VALUE, "molt_rope: NULL tensor pointer");
  MOLT_REQUIRE(batch >= 0 && seq > 0 && heads > 0 && kv_heads >= 0, MOLT_E_VALUE, "molt_rope: bad sizes");
  MOLT_REQUIRE(head_dim > 0 && head_dim % 16 == 0, MOLT_E_CAPABILITY, "molt_rope: head_dim must be a multiple of 16");
  MOLT_REQUIRE(aligned16(q) && aligned16(k) && aligned16(q_out) && aligned16(k_out) && aligned16(cos_table) &&
                   aligned16(sin_table),
               MOLT_E_VALUE, "molt_rope: tensors must be 16-byte aligned");
  if (batch == 0) return MOLT_OK;
  const long long total = batch * seq * (long long)(heads + kv_heads) * (head_dim / 16);
  rope_kernel<<<grid_for(total, 256, 4), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(q), reinterpret_cast<const __nv_bfloat16*>(k),
      reinterpret_cast<__nv_bfloat16*>(q_out), reinterpret_cast<__nv_bfloat16*>(k_out),
      reinterpret_cast<const __nv_bfloat16*>(cos_table), reinterpret_cast<const __nv_bfloat16*>(sin_table), batch * seq,
      (int)seq, heads, kv_heads, head_dim, inverse ? -1.0f : 1.0f);
  return launch_status("rope_kernel");
}

extern "C" int molt_adamw_step(float* param, const float* grad, float* exp_avg, float* exp_avg_sq, int64_t count,
                               float lr, float beta1, float beta2, float eps, float weight_decay, int64_t step,
                               float grad_scale, uintptr_t stream) {
  MOLT_REQUIRE(param && grad && exp_avg && exp_avg_sq, MOLT_E_VALUE, "molt_adamw_step: NULL tensor pointer");
  MOLT_REQUIRE(count >= 0 && count % 4 == 0, MOLT_E_VALUE, "molt_adamw_step: the element count must be a multiple of 4");
  MOLT_REQUIRE(aligned16(param) && aligned16(grad) && aligned16(exp_avg) && aligned16(exp_avg_sq), MOLT_E_VALUE,
               "molt_adamw_step: arrays must be 16-byte aligned");
  MOLT_REQUIRE(step >= 1, MOLT_E_VALUE, "molt_adamw_step: step counts from 1");
  if (count == 0) return MOLT_OK;
  const double bias1 = 1.0 - pow((double)beta1, (double)step);
  const double bias2 = 1.0 - pow((double)beta2, (double)step);
  const long long vectors = count / 4;
  adamw_kernel<<<grid_for(vectors, 256, 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<float4*>(param), reinterpret_cast<const float4*>(grad), reinterpret_cast<float4*>(exp_avg),
      reinterpret_cast<float4*>(exp_avg_sq), vectors, lr, beta1, beta2, eps, weight_decay, (float)bias1,
      (float)sqrt(bias2), grad_scale);
  return launch_status("adamw_kernel");
}

// ------------------------------------------------------------------------------------------------
// Frozen-head cross-entropy: per row, loss = logsumexp(logits) - logits[target] and, in place,
// logits <- (softmax(logits) - onehot(target)) * grad_scale, both from bf16 logits with fp32 arithmetic.
// One CTA per row: an online max/sum pass, then the gradient pass (the row stays in L2 in between).
// Replaces the two Triton kernels of reference kernels/frozen_linear_cross_entropy.py:27-139.
// ------------------------------------------------------------------------------------------------
namespace molt {

__global__ void __launch_bounds__(512) ce_softmax_grad_kernel(__nv_bfloat16* __restrict__ logits,
                                                              const long long* __restrict__ targets,
                                                              float* __restrict__ row_loss, long long vocab,
                                                              float grad_scale) {
  __shared__ float red_max[16], red_sum[16];
  __shared__ float row_stats[2];
  const long long row = blockIdx.x;
  __nv_bfloat16* x = logits + row * vocab;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long vectors = vocab / 8;
  float m = -INFINITY, s = 0.f;
  for (long long v = threadIdx.x; v < vectors; v += blockDim.x) {
    const uint4 raw = *reinterpret_cast<const uint4*>(x + v * 8);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    float vals[8];
    float local = -INFINITY;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      vals[2 * i] = bf16_lo(w[i]);
      vals[2 * i + 1] = bf16_hi(w[i]);
      local = fmaxf(local, fmaxf(vals[2 * i], vals[2 * i + 1]));
    }
    const float nm = fmaxf(m, local);
    float add = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) add += __expf(vals[i] - nm);
    s = s * __expf(m - nm) + add;
    m = nm;
  }
  for (long long c = vectors * 8 + threadIdx.x; c < vocab; c += blockDim.x) {
    const float val = __bfloat162float(x[c]);
    const float nm = fmaxf(m, val);
    s = s * __expf(m - nm) + __expf(val - nm);
    m = nm;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
    m = nm;
  }
  if (lane == 0) { red_max[warp] = m; red_sum[warp] = s; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float gm = -INFINITY, gs = 0.f;
    const int warps = blockDim.x >> 5;
    for (int i = 0; i < warps; ++i) gm = fmaxf(gm, red_max[i]);
    for (int i = 0; i < warps; ++i) gs += red_max[i] == -INFINITY ? 0.f : red_sum[i] * __expf(red_max[i] - gm);
    row_stats[0] = gm;
    row_stats[1] = gs;
    // labels outside [0, vocab) (an ignore index such as -100) contribute no loss and no one-hot term, as at
    // reference kernels/frozen_linear_cross_entropy.py:42-43, 63
    const long long t = targets[row];
    row_loss[row] = (t >= 0 && t < vocab) ? logf(gs) + gm - __bfloat162float(x[t]) : 0.f;
  }
  __syncthreads();
  const float gm = row_stats[0];
  const float inv = grad_scale / row_stats[1];
  // an out-of-range label matches no column below, so nothing is subtracted (reference :94-95, 133)
  const long long t = targets[row];
  for (long long v = threadIdx.x; v < vectors; v += blockDim.x) {
    const uint4 raw = *reinterpret_cast<const uint4*>(x + v * 8);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t out[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float a = __expf(bf16_lo(w[i]) - gm) * inv, b = __expf(bf16_hi(w[i]) - gm) * inv;
      const long long c = v * 8 + 2 * i;
      if (c == t) a -= grad_scale;
      if (c + 1 == t) b -= grad_scale;
      out[i] = pack_bf16x2(a, b);
    }
    *reinterpret_cast<uint4*>(x + v * 8) = make_uint4(out[0], out[1], out[2], out[3]);
  }
  for (long long c = vectors * 8 + threadIdx.x; c < vocab; c += blockDim.x) {
    float a = __expf(__bfloat162float(x[c]) - gm) * inv;
    if (c == t) a -= grad_scale;
    x[c] = __float2bfloat16_rn(a);
  }
}

}  // namespace molt

extern "C" int molt_ce_softmax_grad(void* logits, const int64_t* targets, float* row_loss, int64_t rows, int64_t vocab,
                                    float grad_scale, uintptr_t stream) {
  MOLT_REQUIRE(logits && targets && row_loss, MOLT_E_VALUE, "molt_ce_softmax_grad: NULL tensor pointer");
  MOLT_REQUIRE(rows >= 0 && vocab > 0, MOLT_E_VALUE, "molt_ce_softmax_grad: bad shape");
  MOLT_REQUIRE(aligned16(logits) && vocab % 8 == 0, MOLT_E_VALUE,
               "molt_ce_softmax_grad: logits must be 16-byte aligned with a vocabulary that is a multiple of 8");
  if (rows == 0) return MOLT_OK;
  ce_softmax_grad_kernel<<<(unsigned)rows, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(logits), reinterpret_cast<const long long*>(targets), row_loss, vocab,
      grad_scale);
  return launch_status("ce_softmax_grad_kernel");
}
