// Shared host/device helpers of libmolt_b200: error reporting, argument checks, small device utilities.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/molt_b200.h"

namespace molt {

// ---- host-side error channel (thread-local, so concurrent callers do not see each other's text) ----
char* error_buffer();
int fail(int code, const char* fmt, ...);

#define MOLT_REQUIRE(cond, code, ...)                 \
  do {                                                \
    if (!(cond)) return ::molt::fail(code, __VA_ARGS__); \
  } while (0)

#define MOLT_CUDA(call)                                                                      \
  do {                                                                                       \
    cudaError_t err__ = (call);                                                              \
    if (err__ != cudaSuccess)                                                                \
      return ::molt::fail(MOLT_E_RUNTIME, "%s failed: %s", #call, cudaGetErrorString(err__)); \
  } while (0)

void count_launch();

inline int launch_status(const char* what) {
  count_launch();
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MOLT_E_RUNTIME, "launch of %s failed: %s", what, cudaGetErrorString(err));
  return MOLT_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int sm_count();

// Validates a weight descriptor; fills blocks = number of absmax entries.
int check_desc(const molt_nf4_desc* w, int64_t* blocks);

// Device-visible copy of the parts of a descriptor a kernel needs (passed by value).
struct WeightView {
  const uint8_t* packed;
  const void* absmax;
  const float* absmax2;
  const float* code2;
  float offset;
  int absmax_kind;
  int block2;
  int block2_shift;   // log2(block2) when block2 is a power of two, else -1
  int blocksize;
  int nibble_order;
  long long n, k;
  float codebook[16];
};

inline WeightView make_view(const molt_nf4_desc* w) {
  WeightView v;
  v.packed = w->packed;
  v.absmax = w->absmax;
  v.absmax2 = w->absmax2;
  v.code2 = w->code2;
  v.offset = w->offset;
  v.absmax_kind = w->absmax_kind;
  v.block2 = w->block2 > 0 ? w->block2 : 256;
  v.block2_shift = -1;
  for (int sh = 0; sh < 31; ++sh)
    if ((1 << sh) == v.block2) v.block2_shift = sh;
  v.blocksize = w->blocksize;
  v.nibble_order = w->nibble_order;
  v.n = w->n;
  v.k = w->k;
  for (int i = 0; i < 16; ++i) v.codebook[i] = w->codebook[i];
  return v;
}

// The device status word shared by all kernels with bounded waits.
int32_t* device_status_word();

#ifdef __CUDACC__
// absmax of block `blk` in fp32.  The nested form is code2[u8] * absmax2 + offset with a separate
// multiply and add (no contraction), so every kernel resolves to the same bits.
__device__ __forceinline__ float load_absmax(const WeightView& w, long long blk) {
  if (w.absmax_kind == MOLT_ABSMAX_F32) return __ldg(reinterpret_cast<const float*>(w.absmax) + blk);
  unsigned code = __ldg(reinterpret_cast<const uint8_t*>(w.absmax) + blk);
  const long long group = w.block2_shift >= 0 ? (blk >> w.block2_shift) : blk / w.block2;
  float scaled = __fmul_rn(__ldg(w.code2 + code), __ldg(w.absmax2 + group));
  return __fadd_rn(scaled, w.offset);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
#endif

}  // namespace molt
