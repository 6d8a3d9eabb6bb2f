// tcgen05 / TMEM GEMM for sm_100a with the NF4 decode fused in front of the tensor core.
//
//   forward : out[m, n] = in[m, k] . deq(W)[n, k]^T + low[m, r] . ext[n, r]^T        contraction over k
//   backward: out[m, k] = in[m, n] . deq(W)[n, k]   + low[m, r] . ext[r, k]          contraction over n
//
// The dequantised weight never exists in global memory.  Per 64-wide contraction block a CTA
//   * TMA-loads a 128 x 64 bf16 activation tile (128-byte swizzle) and the matching 8 KB of packed codes,
//   * eight decode warps expand the codes to bf16 (fp32 codebook value times fp32 absmax, rounded once --
//     the same bits the standalone dequantiser produces) straight into the swizzled shared-memory layout
//     that the UMMA descriptor reads: K-major rows for the forward, MN-major atoms for the backward,
//   * one thread issues tcgen05.mma (128 x 256 x 16, fp32 accumulators in TMEM),
//   * four epilogue warps drain the previous tile's accumulators (tcgen05.ld -> bf16 -> TMA store) while the
//     next tile is being accumulated in the other half of TMEM.
// The LoRA term rides along as one more contraction block whose operands are TMA-loaded ready-made.
// Kernels are persistent (one CTA per SM, static tile schedule).  Every mbarrier wait is bounded: on expiry
// the kernel records a code in the device status word, all roles leave their loops, TMEM is released and the
// kernel returns.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <stdlib.h>

#include "internal.h"
#include "sm100_ptx.cuh"

namespace molt {

constexpr int BM = 128;          // tokens per tile
constexpr int BN = 256;          // output columns per tile
constexpr int BK = 64;           // contraction elements per pipeline stage (= one absmax block)
constexpr int kStages = 3;
constexpr int kEpilogueWarps = 4;
constexpr int kDecodeWarps = 8;
constexpr int kProducerWarp = 4;
constexpr int kMmaWarp = 5;
constexpr int kFirstDecodeWarp = 6;
constexpr int kThreads = (kFirstDecodeWarp + kDecodeWarps) * 32;  // 448

constexpr uint32_t kTileABytes = BM * BK * 2;       // 16384
constexpr uint32_t kPackedBytes = BN * BK / 2;      // 8192
constexpr uint32_t kTileBBytes = BN * BK * 2;       // 32768
constexpr uint32_t kStageBytes = kTileABytes + kPackedBytes + kTileBBytes;  // 57344
constexpr uint32_t kStoreBytes = BM * 64 * 2;       // one TMA-store box: 128 rows x 64 bf16
constexpr uint32_t kLutBytes = 16 * 32 * 4;
constexpr uint32_t kSmemBytes = kStages * kStageBytes + 2 * kStoreBytes + kLutBytes + 256 /*barriers*/ + 1024 /*align*/;

struct GemmParams {
  const float* absmax;   // fp32 [n * k / 64]
  int32_t* status;
  long long m, n, k;
  int num_kb;            // contraction blocks of the base GEMM
  int ext_steps;         // rp / 16, 0 = no low-rank block
  int tiles_m, tiles_n;
  int nibble_high_first;
  float codebook[16];
};

// Static tile schedule: bands of 16 token tiles; inside a band the column tile is the slow index, so the
// CTAs running at one time share a few weight column tiles and one band of activations through L2.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int kBand = 16;
  const int band_tiles = kBand * tiles_n;
  const int band = tile / band_tiles;
  const int first_m = band * kBand;
  int rows = tiles_m - first_m;
  if (rows > kBand) rows = kBand;
  const int inside = tile - band * band_tiles;
  tn = inside / rows;
  tm = first_m + inside % rows;
}

template <bool BACKWARD>
__global__ void __launch_bounds__(kThreads, 1)
nf4_gemm_sm100_kernel(const __grid_constant__ CUtensorMap map_in, const __grid_constant__ CUtensorMap map_packed,
                      const __grid_constant__ CUtensorMap map_low, const __grid_constant__ CUtensorMap map_ext,
                      const __grid_constant__ CUtensorMap map_out, const GemmParams p) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag_s;
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_dyn + (base - raw);
  const uint32_t stage0 = base;
  const uint32_t store0 = base + kStages * kStageBytes;
  const uint32_t lut0 = store0 + 2 * kStoreBytes;
  const uint32_t bar0 = lut0 + kLutBytes;
  float* lut_ptr = reinterpret_cast<float*>(base_ptr + kStages * kStageBytes + 2 * kStoreBytes);
  // barriers: tma_full[s], b_full[s], empty[s], acc_full[2], acc_empty[2]
  auto bar_tma = [&](int s) { return bar0 + 8u * s; };
  auto bar_bfull = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto bar_empty = [&](int s) { return bar0 + 8u * (2 * kStages + s); };
  auto bar_accfull = [&](int b) { return bar0 + 8u * (3 * kStages + b); };
  auto bar_accempty = [&](int b) { return bar0 + 8u * (3 * kStages + 2 + b); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &abort_flag_s;

  if (threadIdx.x == 0) {
    abort_flag_s = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_tma(s), 1);
      mbar_init(bar_bfull(s), kDecodeWarps * 32);
      mbar_init(bar_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_accfull(b), 1);
      mbar_init(bar_accempty(b), kEpilogueWarps * 32);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // lane-private copies of the 16 codebook values: entry j of lane l at word j * 32 + l (bank = lane)
  for (int i = threadIdx.x; i < 16 * 32; i += kThreads) lut_ptr[i] = p.codebook[i >> 5];
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int blocks_per_tile = p.num_kb + (p.ext_steps > 0 ? 1 : 0);

  if (warp == kProducerWarp) {
    // ================= TMA producer =================
    int s = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      for (int kb = 0; kb < blocks_per_tile; ++kb) {
        ok = mbar_wait(bar_empty(s), phase ^ 1u, abort_flag, p.status, 1);
        if (!ok) break;
        if (lane == 0) {
          const uint32_t a_dst = stage0 + s * kStageBytes;
          const uint32_t pk_dst = a_dst + kTileABytes;
          const uint32_t b_dst = pk_dst + kPackedBytes;
          if (kb < p.num_kb) {
            mbar_expect_tx(bar_tma(s), kTileABytes + kPackedBytes);
            tma_load_2d(a_dst, &map_in, kb * BK, tm * BM, bar_tma(s));
            if (!BACKWARD) tma_load_2d(pk_dst, &map_packed, kb * (BK / 2), tn * BN, bar_tma(s));
            else tma_load_2d(pk_dst, &map_packed, tn * (BN / 2), kb * BK, bar_tma(s));
          } else {
            // low-rank block: both operands arrive ready for the tensor core
            const uint32_t ext_bytes = BACKWARD ? 4u * (uint32_t)p.ext_steps * 16u * 128u : kTileBBytes;
            mbar_expect_tx(bar_tma(s), kTileABytes + ext_bytes);
            tma_load_2d(a_dst, &map_low, 0, tm * BM, bar_tma(s));
            if (!BACKWARD) {
              tma_load_2d(b_dst, &map_ext, 0, tn * BN, bar_tma(s));
            } else {
              for (int a = 0; a < 4; ++a) tma_load_2d(b_dst + a * 8192u, &map_ext, tn * BN + a * 64, 0, bar_tma(s));
            }
          }
        }
        __syncwarp();
        if (++s == kStages) { s = 0; phase ^= 1u; }
      }
    }
  } else if (warp == kMmaWarp) {
    // ================= MMA issuer =================
    constexpr uint32_t idesc = make_idesc(BM, BN, BACKWARD ? 1 : 0);
    int s = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      ok = mbar_wait(bar_accempty(acc), acc_phase ^ 1u, abort_flag, p.status, 2);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + (uint32_t)acc * BN;
      for (int kb = 0; kb < blocks_per_tile; ++kb) {
        ok = mbar_wait(bar_tma(s), phase, abort_flag, p.status, 3) &&
             mbar_wait(bar_bfull(s), phase, abort_flag, p.status, 4);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_addr = stage0 + s * kStageBytes;
          const uint32_t b_addr = a_addr + kTileABytes + kPackedBytes;
          const uint64_t a_desc = make_desc(a_addr, 16, 1024);
          const uint64_t b_desc = BACKWARD ? make_desc(b_addr, 8192, 1024) : make_desc(b_addr, 16, 1024);
          const int steps = kb < p.num_kb ? BK / 16 : p.ext_steps;
          for (int ks = 0; ks < steps; ++ks) {
            // advance 16 contraction elements: 32 bytes along a K-major row, 16 rows (2048 bytes) in an MN-major atom
            const uint64_t a_k = a_desc + (uint64_t)(ks * 2);
            const uint64_t b_k = b_desc + (uint64_t)(BACKWARD ? ks * 128 : ks * 2);
            umma_bf16(d_tmem, a_k, b_k, idesc, (kb > 0 || ks > 0) ? 1u : 0u);
          }
          umma_commit(bar_empty(s));
          if (kb == blocks_per_tile - 1) umma_commit(bar_accfull(acc));
        }
        __syncwarp();
        if (++s == kStages) { s = 0; phase ^= 1u; }
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  } else if (warp >= kFirstDecodeWarp) {
    // ================= NF4 decoders =================
    const int dt = threadIdx.x - kFirstDecodeWarp * 32;   // 0..255 : one 64-element segment per thread and stage
    const float* my_lut = lut_ptr + lane;
    const long long kblocks_per_row = p.k / 64;
    int s = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      for (int kb = 0; kb < blocks_per_tile; ++kb) {
        float scale = 0.f;
        uint32_t src_off, dst_off, swz;
        if (!BACKWARD) {
          // segment = weight row tn*256 + dt, columns kb*64 .. +63
          const long long row = (long long)tn * BN + dt;
          if (kb < p.num_kb && row < p.n) scale = __ldg(p.absmax + row * kblocks_per_row + kb);
          src_off = (uint32_t)dt * 32u;
          dst_off = (uint32_t)dt * 128u;
          swz = (uint32_t)dt & 7u;
        } else {
          // segment = weight row kb*64 + j, columns tn*256 + a*64 .. +63
          const int a = dt >> 6, j = dt & 63;
          const long long row = (long long)kb * BK + j;
          const long long colblk = (long long)tn * (BN / 64) + a;
          if (kb < p.num_kb && row < p.n && colblk < kblocks_per_row)
            scale = __ldg(p.absmax + row * kblocks_per_row + colblk);
          swz = (uint32_t)j & 7u;
          src_off = (uint32_t)j * 128u + (((uint32_t)(2 * a) ^ swz) << 4);  // packed tile is 128B-swizzled by TMA
          dst_off = (uint32_t)a * 8192u + (uint32_t)j * 128u;
        }
        ok = mbar_wait(bar_tma(s), phase, abort_flag, p.status, 5);
        if (!ok) break;
        if (kb < p.num_kb) {
          const uint32_t pk = stage0 + s * kStageBytes + kTileABytes;
          const uint32_t bt = pk + kPackedBytes + dst_off;
          uint32_t words[8];
          {
            uint32_t a0 = pk + src_off;
            uint32_t a1 = BACKWARD ? (pk + (uint32_t)(dt & 63) * 128u + ((((uint32_t)(2 * (dt >> 6)) + 1u) ^ swz) << 4))
                                   : (a0 + 16u);
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(words[0]), "=r"(words[1]), "=r"(words[2]), "=r"(words[3]) : "r"(a0));
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(words[4]), "=r"(words[5]), "=r"(words[6]), "=r"(words[7]) : "r"(a1));
          }
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            uint32_t wd = words[c];
            if (p.nibble_high_first) wd = ((wd & 0x0f0f0f0fu) << 4) | ((wd >> 4) & 0x0f0f0f0fu);
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = __fmul_rn(my_lut[((wd >> (4 * e)) & 15u) * 32u], scale);
            const uint32_t o0 = pack_bf16x2(v[0], v[1]), o1 = pack_bf16x2(v[2], v[3]);
            const uint32_t o2 = pack_bf16x2(v[4], v[5]), o3 = pack_bf16x2(v[6], v[7]);
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(bt + (((uint32_t)c ^ swz) << 4)), "r"(o0),
                         "r"(o1), "r"(o2), "r"(o3)
                         : "memory");
          }
          fence_proxy_async();
        }
        mbar_arrive(bar_bfull(s));
        if (++s == kStages) { s = 0; phase ^= 1u; }
      }
    }
  } else {
    // ================= epilogue: TMEM -> bf16 -> shared -> TMA store =================
    const int row = warp * 32 + lane;  // accumulator lane = token row inside the tile
    int acc = 0;
    uint32_t acc_phase = 0;
    int store_buf = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      ok = mbar_wait(bar_accfull(acc), acc_phase, abort_flag, p.status, 6);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)acc * BN;
      for (int cg = 0; cg < BN / 64; ++cg) {
        const uint32_t stage_addr = store0 + (uint32_t)store_buf * kStoreBytes;
        // the store issued two groups ago read this buffer; make sure it has finished reading
        if (threadIdx.x == 0) tma_store_wait_read<1>();
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
          tma_store_2d(&map_out, stage_addr, tn * BN + cg * 64, tm * BM);
          tma_store_commit();
        }
        store_buf ^= 1;
      }
      tc_fence_before();
      mbar_arrive(bar_accempty(acc));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if (threadIdx.x == 0) tma_store_wait_all();
  }

  // ---- teardown ----
  if (*abort_flag) {
    // a wait expired somewhere: give copies and MMAs that are still in flight time to land before TMEM goes away
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

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

static int make_map(CUtensorMap* map, CUtensorMapDataType dtype, int elem_bytes, const void* ptr, uint64_t inner,
                    uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, bool swizzle128,
                    const char* what) {
  (void)elem_bytes;
  return make_tensor_map(map, dtype, ptr, inner, outer, row_stride_bytes, box_inner, box_outer,
                         swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, what);
}

bool sm100_gemm_supported(const WeightView& w, int rank) {
  return w.blocksize == 64 && w.k % 64 == 0 && w.n % 64 == 0 && rank <= 64;
}

int sm100_gemm_pair(bool backward, const WeightView& w, const float* absmax_f32, const __nv_bfloat16* in,
                    const __nv_bfloat16* low, const __nv_bfloat16* ext, int rp, __nv_bfloat16* out, long long m,
                    void* split_ws, cudaStream_t s);

// 0 = default (CTA-pair kernel), 1 = single-CTA kernel, 2 = CTA-pair kernel (MOLT_B200_GEMM_VARIANT; for testing)
static int forced_variant() {
  const char* env = getenv("MOLT_B200_GEMM_VARIANT");
  const int value = env != nullptr ? atoi(env) : 0;
  return (value < 0 || value > 2) ? 0 : value;
}

int sm100_gemm(bool backward, const WeightView& w, const float* absmax_f32, const __nv_bfloat16* in,
               const __nv_bfloat16* low, const __nv_bfloat16* ext, int rp, __nv_bfloat16* out, long long m,
               void* split_ws, cudaStream_t s) {
  // The CTA-pair kernel is the default for every token count: its pipeline is deeper and, even with half of a
  // pair tile empty (m <= 128), faster than the single-CTA kernel, which is kept as a selectable variant.
  const int variant = forced_variant();
  if (variant != 1)
    return sm100_gemm_pair(backward, w, absmax_f32, in, low, ext, rp, out, m, split_ws, s);
  if (!sm100_gemm_supported(w, rp)) return fail(MOLT_E_CAPABILITY, "tcgen05 GEMM: unsupported shape");
  const long long contraction = backward ? w.n : w.k;
  const long long out_cols = backward ? w.k : w.n;
  CUtensorMap map_in, map_packed, map_low, map_ext, map_out;
  if (int rc = make_map(&map_in, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, in, contraction, m, contraction * 2, BK, BM, true,
                        "activations"))
    return rc;
  if (!backward) {
    if (int rc = make_map(&map_packed, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w.packed, w.k / 2, w.n, w.k / 2, BK / 2, BN,
                          false, "packed weight"))
      return rc;
  } else {
    if (int rc = make_map(&map_packed, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w.packed, w.k / 2, w.n, w.k / 2, BN / 2, BK,
                          true, "packed weight"))
      return rc;
  }
  const bool has_low = low != nullptr && ext != nullptr && rp > 0;
  if (has_low) {
    if (int rc = make_map(&map_low, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, low, 64, m, 128, 64, BM, true, "low-rank input"))
      return rc;
    if (!backward) {
      if (int rc = make_map(&map_ext, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ext, 64, w.n, 128, 64, BN, true,
                            "scaled LoRA B"))
        return rc;
    } else {
      if (int rc = make_map(&map_ext, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ext, w.k, rp, w.k * 2, 64, rp, true,
                            "LoRA A"))
        return rc;
    }
  } else {
    map_low = map_in;
    map_ext = map_in;
  }
  if (int rc = make_map(&map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, out, out_cols, m, out_cols * 2, 64, BM, true,
                        "output"))
    return rc;

  GemmParams p;
  p.absmax = absmax_f32;
  p.status = device_status_word();
  if (p.status == nullptr) return fail(MOLT_E_RUNTIME, "tcgen05 GEMM: no device status word");
  p.m = m;
  p.n = w.n;
  p.k = w.k;
  p.num_kb = (int)(contraction / BK);
  p.ext_steps = has_low ? rp / 16 : 0;
  p.tiles_m = (int)((m + BM - 1) / BM);
  p.tiles_n = (int)((out_cols + BN - 1) / BN);
  p.nibble_high_first = w.nibble_order == MOLT_NIBBLE_HIGH_FIRST ? 1 : 0;
  for (int i = 0; i < 16; ++i) p.codebook[i] = w.codebook[i];

  static thread_local bool configured[64][2] = {};
  int dev = 0;
  MOLT_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev][backward ? 1 : 0]) {
    if (backward)
      MOLT_CUDA(cudaFuncSetAttribute(nf4_gemm_sm100_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)kSmemBytes));
    else
      MOLT_CUDA(cudaFuncSetAttribute(nf4_gemm_sm100_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)kSmemBytes));
    configured[dev][backward ? 1 : 0] = true;
  }
  const long long tiles = (long long)p.tiles_m * p.tiles_n;
  int grid = sm_count();
  if (tiles < grid) grid = (int)tiles;
  if (backward)
    nf4_gemm_sm100_kernel<true><<<grid, kThreads, kSmemBytes, s>>>(map_in, map_packed, map_low, map_ext, map_out, p);
  else
    nf4_gemm_sm100_kernel<false><<<grid, kThreads, kSmemBytes, s>>>(map_in, map_packed, map_low, map_ext, map_out, p);
  return launch_status("nf4_gemm_sm100_kernel");
}

}  // namespace molt
