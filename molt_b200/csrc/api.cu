// extern "C" entry points of libmolt_b200: argument validation, kernel-path selection and the
// sequencing of the kernels that make up one linear / MLP-block forward or backward.
#include <string.h>

#include "internal.h"

namespace molt {

// ---- error channel ---------------------------------------------------------------------------------
static thread_local char g_error[512] = "";
char* error_buffer() { return g_error; }

int fail(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
  return code;
}

static unsigned long long g_launches = 0;
void count_launch() { __atomic_fetch_add(&g_launches, 1ULL, __ATOMIC_RELAXED); }

// ---- process-wide options --------------------------------------------------------------------------
static long long g_wait_limit_us = 1000000;   // one second
static int g_withheld_blocks = 0;

// SM clock cycles corresponding to the wait limit (at the device's maximum SM clock, so the limit is never shorter
// than asked for).
long long wait_limit_cycles() {
  static int khz[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (khz[dev] == 0) {
    int value = 0;
    if (cudaDeviceGetAttribute(&value, cudaDevAttrClockRate, dev) != cudaSuccess || value <= 0) value = 2000000;
    khz[dev] = value;
  }
  const long long us = __atomic_load_n(&g_wait_limit_us, __ATOMIC_RELAXED);
  return us * (long long)(khz[dev] / 1000);
}

int take_withheld_blocks() { return __atomic_exchange_n(&g_withheld_blocks, 0, __ATOMIC_RELAXED); }

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int count = 0;
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || count <= 0) count = 148;
    cached[dev] = count;
  }
  return cached[dev];
}

// One status word per device image of the library; kernels with bounded waits report here.
__device__ int32_t g_device_status = 0;

int32_t* device_status_word() {
  static thread_local int32_t* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
    cached[dev] = reinterpret_cast<int32_t*>(p);
  }
  return cached[dev];
}

int check_desc(const molt_nf4_desc* w, int64_t* blocks) {
  MOLT_REQUIRE(w != nullptr, MOLT_E_VALUE, "weight descriptor is NULL");
  MOLT_REQUIRE(w->packed != nullptr && w->absmax != nullptr, MOLT_E_VALUE, "weight descriptor holds a NULL pointer");
  MOLT_REQUIRE(w->n > 0 && w->k > 0, MOLT_E_VALUE, "weight shape must be positive, got [%lld, %lld]",
               (long long)w->n, (long long)w->k);
  MOLT_REQUIRE(w->blocksize >= 16 && w->blocksize % 2 == 0, MOLT_E_VALUE, "invalid NF4 block size %d", w->blocksize);
  MOLT_REQUIRE(w->nibble_order == MOLT_NIBBLE_LOW_FIRST || w->nibble_order == MOLT_NIBBLE_HIGH_FIRST, MOLT_E_VALUE,
               "invalid nibble order %d", w->nibble_order);
  MOLT_REQUIRE(w->absmax_kind == MOLT_ABSMAX_F32 || w->absmax_kind == MOLT_ABSMAX_NESTED, MOLT_E_CAPABILITY,
               "unsupported absmax kind %d", w->absmax_kind);
  if (w->absmax_kind == MOLT_ABSMAX_NESTED)
    MOLT_REQUIRE(w->absmax2 != nullptr && w->code2 != nullptr && w->block2 > 0, MOLT_E_VALUE,
                 "nested absmax needs absmax2, code2 and block2");
  const int64_t elements = w->n * w->k;
  *blocks = (elements + w->blocksize - 1) / w->blocksize;
  return MOLT_OK;
}

// ---- workspace carving -----------------------------------------------------------------------------
struct Arena {
  unsigned char* base;
  size_t size;
  size_t used;
  bool dry;
  bool size_optional;   // while sizing: count the optional regions too
  Arena(void* p, size_t bytes, bool sizing_only = false, bool with_optional = true)
      : base(reinterpret_cast<unsigned char*>(p)), size(bytes), used(0), dry(sizing_only), size_optional(with_optional) {}
  void* take(size_t bytes) {
    const size_t start = (used + 255) & ~size_t(255);
    used = start + bytes;
    if (dry) return reinterpret_cast<void*>(uintptr_t(256));  // non-NULL placeholder while sizing
    return base + start;
  }
  // A region the caller can do without: NULL when the workspace has no room for it.  Take it after the required ones.
  void* take_optional(size_t bytes) {
    const size_t start = (used + 255) & ~size_t(255);
    if (dry) {
      if (size_optional) used = start + bytes;
      return nullptr;
    }
    if (base == nullptr || start + bytes > size) return nullptr;
    used = start + bytes;
    return base + start;
  }
  bool fits() const { return dry || (used <= size && (used == 0 || base != nullptr)); }
};

static int padded_rank(int rank) { return (rank + 15) / 16 * 16; }

__global__ void add_bf16_kernel(const uint4* a, const uint4* b, uint4* out, long long vectors, long long count) {
  if (blockIdx.x == 0 && threadIdx.x < 8) {   // the tail past the last whole 16-byte vector
    const long long i = vectors * 8 + threadIdx.x;
    if (i < count) {
      const __nv_bfloat16* as = reinterpret_cast<const __nv_bfloat16*>(a);
      const __nv_bfloat16* bs = reinterpret_cast<const __nv_bfloat16*>(b);
      reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(__bfloat162float(as[i]) + __bfloat162float(bs[i]));
    }
  }
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < vectors;
       v += (long long)gridDim.x * blockDim.x) {
    const uint4 x = a[v], y = b[v];
    const uint32_t xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w};
    uint32_t r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      r[i] = pack_bf16x2(bf16_lo(xs[i]) + bf16_lo(ys[i]), bf16_hi(xs[i]) + bf16_hi(ys[i]));
    out[v] = make_uint4(r[0], r[1], r[2], r[3]);
  }
}

int add_bf16(const __nv_bfloat16* a, const __nv_bfloat16* b, __nv_bfloat16* out, long long count, cudaStream_t s) {
  if (count == 0) return MOLT_OK;
  const long long vectors = count / 8;
  long long blocks = (vectors + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  add_bf16_kernel<<<(unsigned)blocks, 256, 0, s>>>((const uint4*)a, (const uint4*)b, (uint4*)out, vectors, count);
  return launch_status("add_bf16_kernel");
}

static bool aligned_case(const molt_nf4_desc* w, int rank) {
  return w->blocksize == 64 && w->k % 64 == 0 && w->n % 64 == 0 && rank >= 1 && rank <= 64 &&
         (reinterpret_cast<uintptr_t>(w->packed) & 15) == 0;
}

// `requested` may carry MOLT_PATH_NO_SPLIT / MOLT_PATH_FORCE_SPLIT above the kernel path; *gemm_flags receives them.
static int pick_path(int requested, const molt_nf4_desc* w, int rank, int64_t m, bool forward, int* chosen,
                     int* gemm_flags = nullptr) {
  const bool aligned = aligned_case(w, rank);
  MOLT_REQUIRE((requested & ~(0xff | MOLT_PATH_NO_SPLIT | MOLT_PATH_FORCE_SPLIT | MOLT_PATH_TALL_TILES |
                              MOLT_PATH_SHORT_TILES | MOLT_PATH_EXACT_DECODE)) == 0,
               MOLT_E_VALUE, "unknown kernel path flags 0x%x", requested);
  if (gemm_flags != nullptr)
    *gemm_flags = ((requested & MOLT_PATH_NO_SPLIT) ? kGemmNoSplit : 0) | ((requested & MOLT_PATH_FORCE_SPLIT) ? kGemmForceSplit : 0) |
                  ((requested & MOLT_PATH_TALL_TILES) ? kGemmTallTiles : 0) | ((requested & MOLT_PATH_SHORT_TILES) ? kGemmShortTiles : 0) |
                  ((requested & MOLT_PATH_EXACT_DECODE) ? kGemmExactDecode : 0);
  requested &= 0xff;
  if (requested == MOLT_PATH_AUTO) {
    if (!aligned) *chosen = MOLT_PATH_GENERAL;
    else if (forward && m <= 8) *chosen = MOLT_PATH_GEMV;          // one token tile of the streaming kernel
    else if (forward && m <= 128) *chosen = MOLT_PATH_FEW_TOKENS;  // measured faster than the GEMV's second token tile
                                                                   // and than the GEMM's 256-token tiles
    else *chosen = MOLT_PATH_TCGEN05;
    return MOLT_OK;
  }
  MOLT_REQUIRE(requested == MOLT_PATH_GENERAL || requested == MOLT_PATH_TCGEN05 || requested == MOLT_PATH_GEMV ||
                   requested == MOLT_PATH_FEW_TOKENS,
               MOLT_E_VALUE, "unknown kernel path %d", requested);
  if (requested != MOLT_PATH_GENERAL)
    MOLT_REQUIRE(aligned, MOLT_E_CAPABILITY,
                 "the tcgen05 and GEMV kernels need blocksize 64, K %% 64 == 0, N %% 64 == 0, rank <= 64 and a packed "
                 "weight that starts on a 16-byte boundary "
                 "(got N=%lld K=%lld blocksize=%d rank=%d)",
                 (long long)w->n, (long long)w->k, w->blocksize, rank);
  if (requested == MOLT_PATH_GEMV)
    MOLT_REQUIRE(forward && m <= 16, MOLT_E_CAPABILITY, "the GEMV kernel handles forward with at most 16 tokens");
  if (requested == MOLT_PATH_FEW_TOKENS)
    MOLT_REQUIRE(forward && m <= 128, MOLT_E_CAPABILITY, "the few-token kernel handles forward with at most 128 tokens");
  *chosen = requested;
  return MOLT_OK;
}

// fp32 absmax for the tcgen05 GEMM: the descriptor's own array; NULL for a double-quantised absmax whose second-level
// block size is a power of two (the kernel reads that form itself); any other nested form resolved into the arena.
// With `deferred` the resolve is not launched here: *deferred gets the buffer and the caller folds the work into its
// next preparation kernel.
static int resolved_absmax(const molt_nf4_desc* w, Arena& arena, cudaStream_t s, const float** out,
                           float** deferred = nullptr) {
  if (deferred != nullptr) *deferred = nullptr;
  if (w->absmax_kind == MOLT_ABSMAX_F32) {
    *out = reinterpret_cast<const float*>(w->absmax);
    return MOLT_OK;
  }
  if (make_view(w).block2_shift >= 0) {   // the GEMM's decoders read this double-quantised form themselves
    *out = nullptr;
    return MOLT_OK;
  }
  const int64_t blocks = (w->n * w->k + w->blocksize - 1) / w->blocksize;
  float* buf = reinterpret_cast<float*>(arena.take((size_t)blocks * sizeof(float)));
  *out = buf;
  if (arena.dry) return MOLT_OK;
  MOLT_REQUIRE(arena.fits(), MOLT_E_VALUE, "workspace too small");
  if (deferred != nullptr) {
    *deferred = buf;
    return MOLT_OK;
  }
  return molt_nf4_resolve_absmax(w, buf, reinterpret_cast<uintptr_t>(s));
}

// ---- forward ---------------------------------------------------------------------------------------
static int lora_fwd_impl(const molt_nf4_desc* w, const void* x, const float* lora_a, const float* lora_b,
                         float scaling, int rank, void* y, int64_t m, void* t_out, Arena& arena, int path,
                         cudaStream_t s, int flags = 0, const molt_lora_shadow* shadow = nullptr,
                         const void* t_in = nullptr) {
  // t_in: T = bf16(x . bf16(A)^T) [m, 64] kept from an earlier call on the same x (tensor-core path only; the other
  // paths form it themselves)
  const WeightView view = make_view(w);
  const int rp = padded_rank(rank);
  auto* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  auto* yb = reinterpret_cast<__nv_bfloat16*>(y);
  if (path == MOLT_PATH_GEMV) {
    void* ws = arena.take(gemv_workspace_bytes(w->n, w->k));
    if (arena.dry) return MOLT_OK;
    MOLT_REQUIRE(arena.fits(), MOLT_E_VALUE, "molt_nf4_lora_fwd: workspace too small");
    WeightView gview = view;
    if (w->absmax_kind == MOLT_ABSMAX_NESTED && !gemv_reads_nested(view)) {
      // a nested layout the kernel cannot stage with 4-byte copies: resolve it to fp32 once per call
      float* resolved = gemv_resolved_absmax_slot(ws, w->n, w->k);
      if (int rc = molt_nf4_resolve_absmax(w, resolved, reinterpret_cast<uintptr_t>(s))) return rc;
      gview.absmax = resolved;
      gview.absmax_kind = MOLT_ABSMAX_F32;
    }
    return gemv_forward(gview, xb, lora_a, lora_b, scaling, rank, yb, (int)m, reinterpret_cast<__nv_bfloat16*>(t_out), ws,
                        gemv_workspace_bytes(w->n, w->k), s);
  }
  if (path == MOLT_PATH_FEW_TOKENS) {
    const size_t bytes = sm100_skinny_bytes(w->n, w->k, m);
    void* ws = arena.take(bytes);
    WeightView sview = view;
    float* resolved = nullptr;
    if (w->absmax_kind == MOLT_ABSMAX_NESTED && view.block2_shift < 0)   // a nested layout the kernel cannot read itself
      resolved = reinterpret_cast<float*>(arena.take((size_t)((w->n * w->k + 63) / 64) * sizeof(float)));
    if (arena.dry) return MOLT_OK;
    MOLT_REQUIRE(arena.fits(), MOLT_E_VALUE, "molt_nf4_lora_fwd: workspace too small");
    if (resolved != nullptr) {
      if (int rc = molt_nf4_resolve_absmax(w, resolved, reinterpret_cast<uintptr_t>(s))) return rc;
      sview.absmax = resolved;
      sview.absmax_kind = MOLT_ABSMAX_F32;
    }
    return sm100_skinny_forward(sview, xb, lora_a, lora_b, scaling, rank, yb, (int)m,
                                reinterpret_cast<__nv_bfloat16*>(t_out), ws, bytes, flags, s);
  }
  const bool t_given = t_in != nullptr && path == MOLT_PATH_TCGEN05 && t_out == nullptr;
  __nv_bfloat16* t = t_given ? const_cast<__nv_bfloat16*>(reinterpret_cast<const __nv_bfloat16*>(t_in))
                     : t_out != nullptr ? reinterpret_cast<__nv_bfloat16*>(t_out)
                                        : reinterpret_cast<__nv_bfloat16*>(arena.take((size_t)m * 64 * 2));
  if (path == MOLT_PATH_GENERAL) {
    if (arena.dry) return MOLT_OK;
    MOLT_REQUIRE(arena.fits(), MOLT_E_VALUE, "molt_nf4_lora_fwd: workspace too small");
    if (int rc = general_rowsum(true, xb, lora_a, 1.0f, m, w->k, rank, t, 64, s)) return rc;
    return general_forward(view, xb, t, 64, lora_b, scaling, rank, yb, m, s);
  }
  // tcgen05 path; with shadows the bf16 operands are the caller's and only a nested absmax is left to prepare
  const bool shadowed = shadow != nullptr && shadow->a16 != nullptr && shadow->bs != nullptr;
  auto* a16 = shadowed ? const_cast<__nv_bfloat16*>(reinterpret_cast<const __nv_bfloat16*>(shadow->a16))
                       : reinterpret_cast<__nv_bfloat16*>(arena.take((size_t)rp * w->k * 2));
  auto* bs = shadowed ? const_cast<__nv_bfloat16*>(reinterpret_cast<const __nv_bfloat16*>(shadow->bs))
                      : reinterpret_cast<__nv_bfloat16*>(arena.take((size_t)w->n * 64 * 2));
  const float* absmax = nullptr;
  float* to_resolve = nullptr;
  if (int rc = resolved_absmax(w, arena, s, &absmax, &to_resolve)) return rc;
  const bool fits = arena.fits();
  void* split = arena.take_optional(sm100_split_bytes());
  if (arena.dry) return MOLT_OK;
  MOLT_REQUIRE(fits, MOLT_E_VALUE, "molt_nf4_lora_fwd: workspace too small");
  MOLT_REQUIRE((reinterpret_cast<uintptr_t>(lora_a) & 15) == 0, MOLT_E_CAPABILITY,
               "molt_nf4_lora_fwd: lora_a must start on a 16-byte boundary for the tensor-core path");
  if (int rc = lora_prep(lora_a, lora_b, scaling, rank, rp, w->n, w->k, shadowed ? nullptr : a16, shadowed ? nullptr : bs,
                         nullptr, &view, to_resolve, s))
    return rc;
  if (!t_given)
    if (int rc = rowsum_mma(xb, a16, rp, m, w->k, t, s)) return rc;
  return sm100_gemm(false, view, absmax, xb, t, bs, rp, yb, m, split, flags, s);
}

// ---- backward --------------------------------------------------------------------------------------
static int lora_bwd_impl(const molt_nf4_desc* w, const void* x, const void* dy, const float* lora_a,
                         const float* lora_b, float scaling, int rank, void* dx, float* da, float* db, int64_t m,
                         const void* t_in, int accumulate, Arena& arena, int path, cudaStream_t s, int flags = 0,
                         const molt_lora_shadow* shadow = nullptr) {
  const WeightView view = make_view(w);
  const int rp = padded_rank(rank);
  auto* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  auto* gb = reinterpret_cast<const __nv_bfloat16*>(dy);
  auto* dxb = reinterpret_cast<__nv_bfloat16*>(dx);
  const bool want_grads = da != nullptr && db != nullptr;
  auto* u = reinterpret_cast<__nv_bfloat16*>(arena.take((size_t)m * 64 * 2));
  const __nv_bfloat16* t = reinterpret_cast<const __nv_bfloat16*>(t_in);
  __nv_bfloat16* t_own = nullptr;
  if (want_grads && t == nullptr) {
    t_own = reinterpret_cast<__nv_bfloat16*>(arena.take((size_t)m * 64 * 2));
    t = t_own;
  }
  if (path == MOLT_PATH_GENERAL) {
    if (arena.dry) return MOLT_OK;
    MOLT_REQUIRE(arena.fits(), MOLT_E_VALUE, "molt_nf4_lora_bwd: workspace too small");
    // U = bf16(s * dY . B)
    if (int rc = general_rowsum(false, gb, lora_b, scaling, m, w->n, rank, u, 64, s)) return rc;
    if (dxb != nullptr)
      if (int rc = general_backward_input(view, gb, u, 64, lora_a, MOLT_DTYPE_F32, 1.0f, rank, dxb, m, s)) return rc;
    if (want_grads) {
      if (t_own != nullptr)
        if (int rc = general_rowsum(true, xb, lora_a, 1.0f, m, w->k, rank, t_own, 64, s)) return rc;
      if (int rc = general_colsum(true, u, 64, xb, 1.0f, m, w->k, rank, da, accumulate, s)) return rc;
      if (int rc = general_colsum(false, t, 64, gb, scaling, m, w->n, rank, db, accumulate, s)) return rc;
    }
    return MOLT_OK;
  }
  const bool shadowed = shadow != nullptr && shadow->a16 != nullptr && shadow->bt != nullptr;
  auto* a16 = shadowed ? const_cast<__nv_bfloat16*>(reinterpret_cast<const __nv_bfloat16*>(shadow->a16))
                       : reinterpret_cast<__nv_bfloat16*>(arena.take((size_t)rp * w->k * 2));
  auto* bt = shadowed ? const_cast<__nv_bfloat16*>(reinterpret_cast<const __nv_bfloat16*>(shadow->bt))
                      : reinterpret_cast<__nv_bfloat16*>(arena.take((size_t)rp * w->n * 2));
  float* partial_a = nullptr;
  float* partial_b = nullptr;
  if (want_grads) {
    partial_a = reinterpret_cast<float*>(arena.take(colsum_partial_bytes(m, w->k, rp)));
    partial_b = reinterpret_cast<float*>(arena.take(colsum_partial_bytes(m, w->n, rp)));
  }
  const float* absmax = nullptr;
  float* to_resolve = nullptr;
  if (dxb != nullptr)
    if (int rc = resolved_absmax(w, arena, s, &absmax, &to_resolve)) return rc;
  const bool fits = arena.fits();
  void* split = dxb != nullptr ? arena.take_optional(sm100_split_bytes()) : nullptr;
  if (arena.dry) return MOLT_OK;
  MOLT_REQUIRE(fits, MOLT_E_VALUE, "molt_nf4_lora_bwd: workspace too small");
  MOLT_REQUIRE((reinterpret_cast<uintptr_t>(lora_a) & 15) == 0, MOLT_E_CAPABILITY,
               "molt_nf4_lora_bwd: lora_a must start on a 16-byte boundary for the tensor-core path");
  if (int rc = lora_prep(lora_a, lora_b, scaling, rank, rp, w->n, w->k, shadowed ? nullptr : a16, nullptr,
                         shadowed ? nullptr : bt, &view, to_resolve, s))
    return rc;
  if (int rc = rowsum_mma(gb, bt, rp, m, w->n, u, s)) return rc;  // U = dY . (sB)
  if (dxb != nullptr)
    if (int rc = sm100_gemm(true, view, absmax, gb, u, a16, rp, dxb, m, split, flags, s)) return rc;
  if (want_grads) {
    if (t_own != nullptr)
      if (int rc = rowsum_mma(xb, a16, rp, m, w->k, t_own, s)) return rc;
    if (int rc = colsum_pair(u, xb, w->k, partial_a, da, t, gb, w->n, scaling, partial_b, db, rp, rank, m, accumulate, s))
      return rc;
  }
  return MOLT_OK;
}

static int dx_impl(const molt_nf4_desc* w, const void* dy, const void* lora_grad, const void* lora_a,
                   int lora_a_dtype, float scaling, int rank, void* dx, int64_t m, Arena& arena, int path,
                   cudaStream_t s, int flags = 0) {
  const WeightView view = make_view(w);
  auto* gb = reinterpret_cast<const __nv_bfloat16*>(dy);
  auto* dxb = reinterpret_cast<__nv_bfloat16*>(dx);
  if (path == MOLT_PATH_TCGEN05) {
    // The low-rank term rides as one more contraction block: low = lora_grad zero-padded to [m, 64] and
    // ext = bf16(scaling * A) [rp, k].  Base and low-rank term are summed in fp32 and rounded once (the reference
    // rounds the base to bf16 first, methods/nf4_backward.py:127-136; the fused form is the more accurate one).
    const bool has_low = lora_grad != nullptr;
    const int rp = has_low ? padded_rank(rank) : 0;
    __nv_bfloat16* low = nullptr;
    __nv_bfloat16* a16 = nullptr;
    if (has_low) {
      low = reinterpret_cast<__nv_bfloat16*>(arena.take((size_t)m * 64 * 2));
      a16 = reinterpret_cast<__nv_bfloat16*>(arena.take((size_t)rp * w->k * 2));
    }
    const float* absmax = nullptr;
    if (int rc = resolved_absmax(w, arena, s, &absmax)) return rc;
    const bool fits = arena.fits();
    void* split = arena.take_optional(sm100_split_bytes());
    if (arena.dry) return MOLT_OK;
    MOLT_REQUIRE(fits, MOLT_E_VALUE, "molt_nf4_dx: workspace too small");
    if (has_low)
      if (int rc = dx_lora_prep(reinterpret_cast<const __nv_bfloat16*>(lora_grad), rank, m, lora_a, lora_a_dtype, scaling,
                                rp, w->k, low, a16, s))
        return rc;
    return sm100_gemm(true, view, absmax, gb, low, a16, rp, dxb, m, split, flags, s);
  }
  if (arena.dry) return MOLT_OK;
  return general_backward_input(view, gb, reinterpret_cast<const __nv_bfloat16*>(lora_grad), rank, lora_a,
                                lora_a_dtype, scaling, rank, dxb, m, s);
}

}  // namespace molt

using namespace molt;

extern "C" int molt_version(void) { return 100; }
extern "C" const char* molt_last_error(void) { return error_buffer(); }
extern "C" uint64_t molt_launch_count(void) { return __atomic_load_n(&g_launches, __ATOMIC_RELAXED); }

extern "C" int molt_set_option(int option, int64_t value) {
  switch (option) {
    case MOLT_OPT_WAIT_LIMIT_US:
      MOLT_REQUIRE(value >= 100 && value <= 60000000, MOLT_E_VALUE, "wait limit must lie in [100 us, 60 s]");
      __atomic_store_n(&g_wait_limit_us, (long long)value, __ATOMIC_RELAXED);
      return MOLT_OK;
    case MOLT_OPT_WITHHOLD_BLOCKS:
      MOLT_REQUIRE(value >= 0 && value <= 4, MOLT_E_VALUE, "withheld block count must lie in [0, 4]");
      __atomic_store_n(&g_withheld_blocks, (int)value, __ATOMIC_RELAXED);
      return MOLT_OK;
    default:
      return fail(MOLT_E_VALUE, "unknown option %d", option);
  }
}

extern "C" int molt_read_status(uintptr_t stream, int32_t* status_out) {
  MOLT_REQUIRE(status_out != nullptr, MOLT_E_VALUE, "molt_read_status: status_out is NULL");
  int32_t* word = device_status_word();
  MOLT_REQUIRE(word != nullptr, MOLT_E_RUNTIME, "molt_read_status: no device status word");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int32_t host = 0;
  MOLT_CUDA(cudaMemcpyAsync(&host, word, sizeof(host), cudaMemcpyDeviceToHost, s));
  MOLT_CUDA(cudaStreamSynchronize(s));
  if (host != 0) MOLT_CUDA(cudaMemsetAsync(word, 0, sizeof(host), s));
  *status_out = host;
  return MOLT_OK;
}

static int check_linear_args(const char* who, const molt_nf4_desc* w, int rank, int64_t m, int64_t* blocks) {
  if (int rc = check_desc(w, blocks)) return rc;
  MOLT_REQUIRE(m >= 0, MOLT_E_VALUE, "%s: negative token count", who);
  MOLT_REQUIRE(rank >= 1, MOLT_E_VALUE, "%s: LoRA rank must be positive", who);
  MOLT_REQUIRE(rank <= 64, MOLT_E_CAPABILITY, "%s: LoRA rank %d exceeds the supported maximum of 64", who, rank);
  return MOLT_OK;
}

// with_optional = false gives the smallest workspace the entry points accept (the tcgen05 GEMMs then keep their plain
// tile schedule instead of splitting the tiles of the last wave).
size_t molt::workspace_bytes(int op, int64_t m, int64_t n, int64_t k, int rank, bool with_optional) {
  if (m < 0 || n <= 0 || k <= 0 || rank < 1 || rank > 64) return 0;
  molt_nf4_desc fake;
  memset(&fake, 0, sizeof(fake));
  fake.n = n;
  fake.k = k;
  fake.blocksize = 64;
  fake.absmax_kind = MOLT_ABSMAX_NESTED;  // upper bound: room for a resolved absmax copy
  fake.packed = reinterpret_cast<const uint8_t*>(uintptr_t(256));
  fake.absmax = fake.packed;
  size_t best = 0;
  const int paths[4] = {MOLT_PATH_GENERAL, MOLT_PATH_TCGEN05, MOLT_PATH_GEMV, MOLT_PATH_FEW_TOKENS};
  for (int path : paths) {
    if (path != MOLT_PATH_GENERAL && !(k % 64 == 0 && n % 64 == 0)) continue;
    if (path == MOLT_PATH_GEMV && !(op == MOLT_OP_LORA_FWD && m <= 16)) continue;
    if (path == MOLT_PATH_FEW_TOKENS && !(op == MOLT_OP_LORA_FWD && m >= 1 && m <= 128)) continue;
    Arena arena(nullptr, 0, true, with_optional);
    if (op == MOLT_OP_LORA_FWD) lora_fwd_impl(&fake, nullptr, nullptr, nullptr, 1.f, rank, nullptr, m, nullptr, arena, path, 0);
    else if (op == MOLT_OP_LORA_BWD)
      lora_bwd_impl(&fake, nullptr, nullptr, nullptr, nullptr, 1.f, rank, reinterpret_cast<void*>(uintptr_t(256)),
                    reinterpret_cast<float*>(uintptr_t(256)), reinterpret_cast<float*>(uintptr_t(256)), m, nullptr, 0,
                    arena, path, 0);
    else if (op == MOLT_OP_DX)   // sized for a call with a low-rank term of this rank
      dx_impl(&fake, nullptr, reinterpret_cast<const void*>(uintptr_t(256)), nullptr, 0, 1.f, rank, nullptr, m, arena, path, 0);
    else return 0;
    if (arena.used > best) best = arena.used;
  }
  return best + 256;
}

extern "C" size_t molt_workspace_bytes(int op, int64_t m, int64_t n, int64_t k, int rank) {
  return molt::workspace_bytes(op, m, n, k, rank, true);
}

extern "C" int molt_nf4_lora_fwd(const molt_nf4_desc* w, const void* x, const float* lora_a, const float* lora_b,
                                 float scaling, int rank, void* y, int64_t m, void* t_out, void* workspace,
                                 size_t workspace_bytes, int path, uintptr_t stream) {
  return molt_nf4_lora_fwd_prepared(w, x, lora_a, lora_b, scaling, rank, nullptr, y, m, t_out, workspace, workspace_bytes,
                                    path, stream);
}

extern "C" int molt_nf4_lora_fwd_prepared(const molt_nf4_desc* w, const void* x, const float* lora_a,
                                          const float* lora_b, float scaling, int rank, const molt_lora_shadow* shadow,
                                          void* y, int64_t m, void* t_out, void* workspace, size_t workspace_bytes,
                                          int path, uintptr_t stream) {
  int64_t blocks = 0;
  if (int rc = check_linear_args("molt_nf4_lora_fwd", w, rank, m, &blocks)) return rc;
  MOLT_REQUIRE(x && lora_a && lora_b && y, MOLT_E_VALUE, "molt_nf4_lora_fwd: NULL tensor pointer");
  MOLT_REQUIRE(aligned16(x) && aligned16(y) && aligned16(w->packed) && (t_out == nullptr || aligned16(t_out)),
               MOLT_E_VALUE, "molt_nf4_lora_fwd: tensors must be 16-byte aligned");
  if (m == 0) return MOLT_OK;
  int chosen = 0, flags = 0;
  if (int rc = pick_path(path, w, rank, m, true, &chosen, &flags)) return rc;
  MOLT_REQUIRE(workspace != nullptr, MOLT_E_VALUE, "molt_nf4_lora_fwd: workspace is NULL");
  Arena arena(workspace, workspace_bytes);
  return lora_fwd_impl(w, x, lora_a, lora_b, scaling, rank, y, m, t_out, arena, chosen,
                       reinterpret_cast<cudaStream_t>(stream), flags, shadow);
}

extern "C" int molt_nf4_gemv(const molt_nf4_desc* w, const void* x, const float* lora_a, const float* lora_b,
                             float scaling, int rank, void* y, int64_t m, void* workspace, size_t workspace_bytes,
                             uintptr_t stream) {
  return molt_nf4_lora_fwd(w, x, lora_a, lora_b, scaling, rank, y, m, nullptr, workspace, workspace_bytes,
                           MOLT_PATH_GEMV, stream);
}

extern "C" int molt_nf4_lora_bwd(const molt_nf4_desc* w, const void* x, const void* dy, const float* lora_a,
                                 const float* lora_b, float scaling, int rank, void* dx, float* da, float* db,
                                 int64_t m, const void* t_in, int accumulate, void* workspace, size_t workspace_bytes,
                                 int path, uintptr_t stream) {
  return molt_nf4_lora_bwd_prepared(w, x, dy, lora_a, lora_b, scaling, rank, nullptr, dx, da, db, m, t_in, accumulate,
                                    workspace, workspace_bytes, path, stream);
}

extern "C" int molt_nf4_lora_bwd_prepared(const molt_nf4_desc* w, const void* x, const void* dy, const float* lora_a,
                                          const float* lora_b, float scaling, int rank, const molt_lora_shadow* shadow,
                                          void* dx, float* da, float* db, int64_t m, const void* t_in, int accumulate,
                                          void* workspace, size_t workspace_bytes, int path, uintptr_t stream) {
  int64_t blocks = 0;
  if (int rc = check_linear_args("molt_nf4_lora_bwd", w, rank, m, &blocks)) return rc;
  MOLT_REQUIRE(dy && lora_a && lora_b, MOLT_E_VALUE, "molt_nf4_lora_bwd: NULL tensor pointer");
  MOLT_REQUIRE((da == nullptr) == (db == nullptr), MOLT_E_VALUE,
               "molt_nf4_lora_bwd: da and db must both be given or both be NULL");
  MOLT_REQUIRE(da == nullptr || x != nullptr, MOLT_E_VALUE, "molt_nf4_lora_bwd: adapter gradients need x");
  MOLT_REQUIRE(aligned16(dy) && (x == nullptr || aligned16(x)) && (dx == nullptr || aligned16(dx)) &&
                   aligned16(w->packed) && (t_in == nullptr || aligned16(t_in)),
               MOLT_E_VALUE, "molt_nf4_lora_bwd: tensors must be 16-byte aligned");
  if (m == 0) {
    if (da != nullptr && !accumulate) {
      cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
      MOLT_CUDA(cudaMemsetAsync(da, 0, (size_t)rank * w->k * sizeof(float), s));
      MOLT_CUDA(cudaMemsetAsync(db, 0, (size_t)rank * w->n * sizeof(float), s));
    }
    return MOLT_OK;
  }
  int chosen = 0, flags = 0;
  if (int rc = pick_path(path, w, rank, m, false, &chosen, &flags)) return rc;
  MOLT_REQUIRE(workspace != nullptr, MOLT_E_VALUE, "molt_nf4_lora_bwd: workspace is NULL");
  Arena arena(workspace, workspace_bytes);
  return lora_bwd_impl(w, x, dy, lora_a, lora_b, scaling, rank, dx, da, db, m, t_in, accumulate, arena, chosen,
                       reinterpret_cast<cudaStream_t>(stream), flags, shadow);
}

extern "C" int molt_lora_shadow_refresh(const molt_lora_shadow_item* items, int count, int64_t max_n, int64_t max_k,
                                        uintptr_t stream) {
  MOLT_REQUIRE(count >= 0 && (count == 0 || items != nullptr), MOLT_E_VALUE, "molt_lora_shadow_refresh: bad item list");
  MOLT_REQUIRE(max_n > 0 && max_k > 0 && max_n % 64 == 0 && max_k % 64 == 0, MOLT_E_VALUE,
               "molt_lora_shadow_refresh: max_n and max_k must be positive multiples of 64");
  return lora_shadow_refresh(items, count, max_n, max_k, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int molt_nf4_dx(const molt_nf4_desc* w, const void* dy, const void* lora_grad, const void* lora_a,
                           int lora_a_dtype, float scaling, int rank, void* dx, int64_t m, void* workspace,
                           size_t workspace_bytes, int path, uintptr_t stream) {
  int64_t blocks = 0;
  if (int rc = check_desc(w, &blocks)) return rc;
  MOLT_REQUIRE(m >= 0, MOLT_E_VALUE, "molt_nf4_dx: negative token count");
  MOLT_REQUIRE(dy && dx, MOLT_E_VALUE, "molt_nf4_dx: NULL tensor pointer");
  MOLT_REQUIRE(aligned16(dy) && aligned16(dx) && aligned16(w->packed), MOLT_E_VALUE,
               "molt_nf4_dx: tensors must be 16-byte aligned");
  if (lora_grad != nullptr) {
    MOLT_REQUIRE(lora_a != nullptr, MOLT_E_VALUE, "molt_nf4_dx: lora_grad given without lora_a");
    MOLT_REQUIRE(rank >= 1, MOLT_E_VALUE, "molt_nf4_dx: LoRA rank must be positive");
    MOLT_REQUIRE(lora_a_dtype == MOLT_DTYPE_BF16 || lora_a_dtype == MOLT_DTYPE_F32, MOLT_E_CAPABILITY,
                 "molt_nf4_dx: LoRA A must be bf16 or fp32");
  }
  if (m == 0) return MOLT_OK;
  int chosen = 0, flags = 0;
  const int rank_for_path = lora_grad != nullptr ? rank : 1;
  if (lora_grad != nullptr)
    MOLT_REQUIRE(rank <= 64, MOLT_E_CAPABILITY, "molt_nf4_dx: LoRA rank %d exceeds the supported maximum of 64", rank);
  if (int rc = pick_path(path, w, rank_for_path, m, false, &chosen, &flags)) return rc;
  if (chosen == MOLT_PATH_TCGEN05 && lora_grad != nullptr && !aligned16(lora_a)) {
    MOLT_REQUIRE((path & 0xff) == MOLT_PATH_AUTO, MOLT_E_CAPABILITY,
                 "molt_nf4_dx: lora_a must start on a 16-byte boundary for the tensor-core path");
    chosen = MOLT_PATH_GENERAL;
  }
  MOLT_REQUIRE(chosen == MOLT_PATH_GENERAL || workspace != nullptr, MOLT_E_VALUE, "molt_nf4_dx: workspace is NULL");
  Arena arena(workspace, workspace_bytes);
  return dx_impl(w, dy, lora_grad, lora_a, lora_a_dtype, scaling, rank, dx, m, arena, chosen,
                 reinterpret_cast<cudaStream_t>(stream), flags);
}

// ---- dense frozen weight (LM head) -------------------------------------------------------------------
extern "C" size_t molt_dense_gemm_workspace_bytes(void) { return sm100_split_bytes() + 256; }

extern "C" int molt_dense_gemm(const void* weight, int64_t n, int64_t k, const void* in, void* out, int64_t m,
                               int contract_over_rows, void* workspace, size_t workspace_bytes, int flags,
                               uintptr_t stream) {
  MOLT_REQUIRE(weight && in && out, MOLT_E_VALUE, "molt_dense_gemm: NULL tensor pointer");
  MOLT_REQUIRE(n > 0 && k > 0 && m >= 0, MOLT_E_VALUE, "molt_dense_gemm: bad shape");
  MOLT_REQUIRE(n % 64 == 0 && k % 64 == 0, MOLT_E_CAPABILITY,
               "molt_dense_gemm: weight dimensions must be multiples of 64 (got [%lld, %lld])", (long long)n, (long long)k);
  MOLT_REQUIRE(aligned16(weight) && aligned16(in) && aligned16(out), MOLT_E_VALUE,
               "molt_dense_gemm: tensors must be 16-byte aligned");
  MOLT_REQUIRE((flags & ~(MOLT_PATH_NO_SPLIT | MOLT_PATH_FORCE_SPLIT | MOLT_PATH_TALL_TILES | MOLT_PATH_SHORT_TILES)) == 0,
               MOLT_E_VALUE, "molt_dense_gemm: unknown flags 0x%x", flags);
  if (m == 0) return MOLT_OK;
  const int gemm_flags = ((flags & MOLT_PATH_NO_SPLIT) ? kGemmNoSplit : 0) | ((flags & MOLT_PATH_FORCE_SPLIT) ? kGemmForceSplit : 0) |
                         ((flags & MOLT_PATH_TALL_TILES) ? kGemmTallTiles : 0) | ((flags & MOLT_PATH_SHORT_TILES) ? kGemmShortTiles : 0);
  // the split scratch is optional: without it the GEMM keeps the plain schedule
  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  void* split = nullptr;
  if (ws != nullptr) {
    const uintptr_t start = (reinterpret_cast<uintptr_t>(ws) + 255) & ~uintptr_t(255);
    if (start + sm100_split_bytes() <= reinterpret_cast<uintptr_t>(ws) + workspace_bytes) split = reinterpret_cast<void*>(start);
  }
  return sm100_dense_gemm(contract_over_rows != 0, reinterpret_cast<const __nv_bfloat16*>(weight), n, k,
                          reinterpret_cast<const __nv_bfloat16*>(in), reinterpret_cast<__nv_bfloat16*>(out), m, split,
                          gemm_flags, reinterpret_cast<cudaStream_t>(stream));
}

// ---- gated MLP block -------------------------------------------------------------------------------
static int check_proj(const char* who, const molt_lora_proj* p) {
  MOLT_REQUIRE(p != nullptr && p->w != nullptr && p->lora_a != nullptr && p->lora_b != nullptr, MOLT_E_VALUE,
               "%s: NULL projection", who);
  int64_t blocks = 0;
  return check_linear_args(who, p->w, p->rank, 0, &blocks);
}

static int check_block(const char* who, const molt_lora_proj* gate, const molt_lora_proj* up,
                       const molt_lora_proj* down) {
  if (int rc = check_proj(who, gate)) return rc;
  if (int rc = check_proj(who, up)) return rc;
  if (int rc = check_proj(who, down)) return rc;
  MOLT_REQUIRE(gate->w->n == up->w->n && gate->w->k == up->w->k, MOLT_E_VALUE,
               "%s: gate and up projections must have the same shape", who);
  MOLT_REQUIRE(down->w->k == gate->w->n && down->w->n == gate->w->k, MOLT_E_VALUE,
               "%s: down projection must map the intermediate width back to the hidden width", who);
  return MOLT_OK;
}

static int mlp_fwd_impl(const molt_lora_proj* gate, const molt_lora_proj* up, const molt_lora_proj* down,
                        const void* x, void* gate_out, void* up_out, void* y, void* t_out, int64_t m, Arena& arena,
                        cudaStream_t s) {
  // t_out: optional [3][m][64] bf16, the low-rank inputs T of gate, up and down, for the backward
  const int64_t inter = gate->w->n;
  void* up_buf = up_out != nullptr ? up_out : arena.take((size_t)m * inter * 2);
  void* hidden = arena.take((size_t)m * inter * 2);
  const size_t mark = arena.used;
  size_t high = mark;
  const molt_lora_proj* projs[3] = {gate, up, down};
  const void* ins[3] = {x, x, hidden};
  void* outs[3] = {gate_out, up_buf, y};
  for (int i = 0; i < 3; ++i) {
    arena.used = mark;  // the three linears run one after another on the stream and reuse the same scratch
    int chosen = 0;
    if (int rc = pick_path(MOLT_PATH_AUTO, projs[i]->w, projs[i]->rank, m, true, &chosen)) return rc;
    if (i == 2 && !arena.dry)
      if (int rc = molt_swiglu_fwd(gate_out, up_buf, hidden, m * inter, MOLT_DTYPE_BF16, reinterpret_cast<uintptr_t>(s)))
        return rc;
    if (int rc = lora_fwd_impl(projs[i]->w, ins[i], projs[i]->lora_a, projs[i]->lora_b, projs[i]->scaling,
                               projs[i]->rank, outs[i], m,
                               t_out != nullptr ? reinterpret_cast<unsigned char*>(t_out) + (size_t)i * m * 128 : nullptr,
                               arena, chosen, s, 0, projs[i]->shadow))
      return rc;
    if (arena.used > high) high = arena.used;
  }
  arena.used = high;
  return MOLT_OK;
}

static int mlp_bwd_impl(const molt_lora_proj* gate, const molt_lora_proj* up, const molt_lora_proj* down,
                        const void* x, const void* gate_saved, const void* up_saved, const void* t_saved,
                        const void* dy, void* dx, float* const grads[6], int accumulate, int64_t m, Arena& arena,
                        cudaStream_t s) {
  // t_saved: optional [3][m][64] bf16 from the forward (see mlp_fwd_impl).  With it no low-rank input is recomputed,
  // and h = silu(gate) * up is rebuilt by the SAME pass that forms dgate and dup (it is only needed for the down
  // projection's adapter gradients, which can wait until dh exists).
  const int64_t inter = gate->w->n, hidden_width = gate->w->k;
  auto kept_t = [&](int i) -> const void* {
    return t_saved != nullptr ? reinterpret_cast<const unsigned char*>(t_saved) + (size_t)i * m * 128 : nullptr;
  };
  const size_t act = (size_t)m * inter * 2;
  void* up_buf = up_saved != nullptr ? nullptr : arena.take(act);   // replayed `up`, later reused for dup
  void* dup_buf = up_saved != nullptr ? arena.take(act) : up_buf;
  void* hidden = arena.take(act);
  void* dh = arena.take(act);                                       // dh, overwritten in place by dgate
  void* dx_up = arena.take((size_t)m * hidden_width * 2);
  const size_t mark = arena.used;
  size_t high = mark;
  const uintptr_t st = reinterpret_cast<uintptr_t>(s);
  int chosen = 0;
  // 1. replay the up projection (reference gated_replay.py:360-368)
  const void* up_val = up_saved;
  if (up_saved == nullptr) {
    if (int rc = pick_path(MOLT_PATH_AUTO, up->w, up->rank, m, true, &chosen)) return rc;
    if (int rc = lora_fwd_impl(up->w, x, up->lora_a, up->lora_b, up->scaling, up->rank, up_buf, m, nullptr, arena,
                               chosen, s, 0, up->shadow, kept_t(1)))
      return rc;
    up_val = up_buf;
    if (arena.used > high) high = arena.used;
  }
  if (t_saved == nullptr) {
    // 2. rebuild h = silu(gate) * up (:373-375)
    if (!arena.dry)
      if (int rc = molt_swiglu_fwd(gate_saved, up_val, hidden, m * inter, MOLT_DTYPE_BF16, st)) return rc;
    // 3. down projection backward (:376-384)
    arena.used = mark;
    if (int rc = pick_path(MOLT_PATH_AUTO, down->w, down->rank, m, false, &chosen)) return rc;
    if (int rc = lora_bwd_impl(down->w, hidden, dy, down->lora_a, down->lora_b, down->scaling, down->rank, dh, grads[4],
                               grads[5], m, nullptr, accumulate, arena, chosen, s, 0, down->shadow))
      return rc;
    if (arena.used > high) high = arena.used;
    // 4. dup = dh * silu(gate), dgate = silu'(gate) * dh * up (:385-387); dgate overwrites dh
    if (!arena.dry)
      if (int rc = molt_swiglu_bwd(dh, gate_saved, up_val, dh, dup_buf, nullptr, m * inter, MOLT_DTYPE_BF16, st)) return rc;
  } else {
    // 2'. dh = dY . deq(W_down) + (dY . sB_down) . A_down: needs no h
    arena.used = mark;
    if (int rc = pick_path(MOLT_PATH_AUTO, down->w, down->rank, m, false, &chosen)) return rc;
    if (int rc = lora_bwd_impl(down->w, nullptr, dy, down->lora_a, down->lora_b, down->scaling, down->rank, dh, nullptr,
                               nullptr, m, nullptr, accumulate, arena, chosen, s, 0, down->shadow))
      return rc;
    if (arena.used > high) high = arena.used;
    // 3'. one pass over dh, gate, up: dgate (over dh), dup and h
    if (!arena.dry)
      if (int rc = molt_swiglu_bwd(dh, gate_saved, up_val, dh, dup_buf, hidden, m * inter, MOLT_DTYPE_BF16, st)) return rc;
    // 4'. the down projection's adapter gradients from h, dY and the kept T
    arena.used = mark;
    if (int rc = lora_bwd_impl(down->w, hidden, dy, down->lora_a, down->lora_b, down->scaling, down->rank, nullptr,
                               grads[4], grads[5], m, kept_t(2), accumulate, arena, chosen, s, 0, down->shadow))
      return rc;
    if (arena.used > high) high = arena.used;
  }
  // 5. gate and up projection backwards, dx = dx_gate + dx_up (:155-186)
  arena.used = mark;
  if (int rc = pick_path(MOLT_PATH_AUTO, gate->w, gate->rank, m, false, &chosen)) return rc;
  if (int rc = lora_bwd_impl(gate->w, x, dh, gate->lora_a, gate->lora_b, gate->scaling, gate->rank, dx, grads[0],
                             grads[1], m, kept_t(0), accumulate, arena, chosen, s, 0, gate->shadow))
    return rc;
  if (arena.used > high) high = arena.used;
  arena.used = mark;
  if (int rc = pick_path(MOLT_PATH_AUTO, up->w, up->rank, m, false, &chosen)) return rc;
  if (int rc = lora_bwd_impl(up->w, x, dup_buf, up->lora_a, up->lora_b, up->scaling, up->rank, dx_up, grads[2],
                             grads[3], m, kept_t(1), accumulate, arena, chosen, s, 0, up->shadow))
    return rc;
  if (arena.used > high) high = arena.used;
  arena.used = high;
  if (arena.dry) return MOLT_OK;
  return add_bf16(reinterpret_cast<const __nv_bfloat16*>(dx), reinterpret_cast<const __nv_bfloat16*>(dx_up),
                  reinterpret_cast<__nv_bfloat16*>(dx), m * hidden_width, s);
}

extern "C" size_t molt_mlp_workspace_bytes(int op, const molt_lora_proj* gate, const molt_lora_proj* up,
                                           const molt_lora_proj* down, int64_t m, int up_given) {
  if (check_block("molt_mlp_workspace_bytes", gate, up, down) != MOLT_OK || m < 0) return 0;
  Arena arena(nullptr, 0, true);
  void* fake = reinterpret_cast<void*>(uintptr_t(256));
  float* fake_grads[6];
  for (int i = 0; i < 6; ++i) fake_grads[i] = reinterpret_cast<float*>(fake);
  int rc = MOLT_E_VALUE;
  if (op == MOLT_OP_MLP_FWD) rc = mlp_fwd_impl(gate, up, down, fake, fake, up_given ? fake : nullptr, fake, nullptr, m, arena, 0);
  else if (op == MOLT_OP_MLP_BWD)
    rc = mlp_bwd_impl(gate, up, down, fake, fake, up_given ? fake : nullptr, nullptr, fake, fake, fake_grads, 0, m, arena, 0);
  return rc == MOLT_OK ? arena.used + 256 : 0;
}

extern "C" int molt_mlp_fwd_t(const molt_lora_proj* gate, const molt_lora_proj* up, const molt_lora_proj* down,
                              const void* x, void* gate_out, void* up_out, void* y, void* t_out, int64_t m,
                              void* workspace, size_t workspace_bytes, uintptr_t stream) {
  if (int rc = check_block("molt_mlp_fwd", gate, up, down)) return rc;
  MOLT_REQUIRE(m >= 0, MOLT_E_VALUE, "molt_mlp_fwd: negative token count");
  MOLT_REQUIRE(x && gate_out && y && workspace, MOLT_E_VALUE, "molt_mlp_fwd: NULL tensor pointer");
  MOLT_REQUIRE(aligned16(x) && aligned16(gate_out) && aligned16(y) && (up_out == nullptr || aligned16(up_out)) &&
                   (t_out == nullptr || aligned16(t_out)),
               MOLT_E_VALUE, "molt_mlp_fwd: tensors must be 16-byte aligned");
  if (m == 0) return MOLT_OK;
  Arena arena(workspace, workspace_bytes);
  return mlp_fwd_impl(gate, up, down, x, gate_out, up_out, y, t_out, m, arena, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int molt_mlp_fwd(const molt_lora_proj* gate, const molt_lora_proj* up, const molt_lora_proj* down,
                            const void* x, void* gate_out, void* up_out, void* y, int64_t m, void* workspace,
                            size_t workspace_bytes, uintptr_t stream) {
  return molt_mlp_fwd_t(gate, up, down, x, gate_out, up_out, y, nullptr, m, workspace, workspace_bytes, stream);
}

extern "C" int molt_mlp_bwd_t(const molt_lora_proj* gate, const molt_lora_proj* up, const molt_lora_proj* down,
                              const void* x, const void* gate_saved, const void* up_saved, const void* t_saved,
                              const void* dy, void* dx, float* const grads[6], int accumulate, int64_t m,
                              void* workspace, size_t workspace_bytes, uintptr_t stream) {
  if (int rc = check_block("molt_mlp_bwd", gate, up, down)) return rc;
  MOLT_REQUIRE(m >= 0, MOLT_E_VALUE, "molt_mlp_bwd: negative token count");
  MOLT_REQUIRE(x && gate_saved && dy && dx && grads && workspace, MOLT_E_VALUE, "molt_mlp_bwd: NULL tensor pointer");
  for (int i = 0; i < 6; ++i) MOLT_REQUIRE(grads[i] != nullptr, MOLT_E_VALUE, "molt_mlp_bwd: NULL gradient pointer");
  MOLT_REQUIRE(aligned16(x) && aligned16(gate_saved) && aligned16(dy) && aligned16(dx) &&
                   (up_saved == nullptr || aligned16(up_saved)) && (t_saved == nullptr || aligned16(t_saved)),
               MOLT_E_VALUE, "molt_mlp_bwd: tensors must be 16-byte aligned");
  if (m == 0) return MOLT_OK;
  Arena arena(workspace, workspace_bytes);
  return mlp_bwd_impl(gate, up, down, x, gate_saved, up_saved, t_saved, dy, dx, grads, accumulate, m, arena,
                      reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int molt_mlp_bwd(const molt_lora_proj* gate, const molt_lora_proj* up, const molt_lora_proj* down,
                            const void* x, const void* gate_saved, const void* up_saved, const void* dy, void* dx,
                            float* const grads[6], int accumulate, int64_t m, void* workspace, size_t workspace_bytes,
                            uintptr_t stream) {
  return molt_mlp_bwd_t(gate, up, down, x, gate_saved, up_saved, nullptr, dy, dx, grads, accumulate, m, workspace,
                        workspace_bytes, stream);
}
