// Prototypes shared between the translation units of libmolt_b200.
#pragma once

#include "common.cuh"

namespace molt {

// general.cu -- any shape
int general_forward(const WeightView& w, const __nv_bfloat16* x, const __nv_bfloat16* t, int t_ld, const float* lora_b,
                    float scaling, int rank, __nv_bfloat16* y, long long m, cudaStream_t s);
int general_backward_input(const WeightView& w, const __nv_bfloat16* dy, const __nv_bfloat16* u, int u_ld,
                           const void* lora_a, int lora_a_dtype, float scaling, int rank, __nv_bfloat16* dx,
                           long long m, cudaStream_t s);
int general_rowsum(bool by_rows, const __nv_bfloat16* in, const float* mat, float scale, long long m, long long cols,
                   int rank, __nv_bfloat16* low, int low_ld, cudaStream_t s);
int general_colsum(bool out_by_rows, const __nv_bfloat16* low, int low_ld, const __nv_bfloat16* in, float scale,
                   long long m, long long cols, int rank, float* grad, int accumulate, cudaStream_t s);

// skinny.cu -- aligned shapes
int lora_prep(const float* a, const float* b, float scaling, int rank, int rp, long long n, long long k,
              __nv_bfloat16* a16, __nv_bfloat16* bs, __nv_bfloat16* bt, const WeightView* w, float* resolved,
              cudaStream_t s);
int rowsum_mma(const __nv_bfloat16* in, const __nv_bfloat16* wt, int rp, long long m, long long cols,
               __nv_bfloat16* out, cudaStream_t s);
// the bf16 operands of `count` adapters in one launch (items: device array)
int lora_shadow_refresh(const molt_lora_shadow_item* items, int count, long long max_n, long long max_k, cudaStream_t s);
// low[m, 64] = lora_grad[m, rank] zero-padded; a16[rp, k] = bf16(scaling * A), rows >= rank zero (A bf16 or fp32)
int dx_lora_prep(const __nv_bfloat16* lora_grad, int rank, long long m, const void* lora_a, int lora_a_dtype,
                 float scaling, int rp, long long k, __nv_bfloat16* low, __nv_bfloat16* a16, cudaStream_t s);
size_t colsum_partial_bytes(long long m, long long cols, int rp);
int colsum_pair(const __nv_bfloat16* u, const __nv_bfloat16* x, long long k, float* partial_a, float* grad_a,
                const __nv_bfloat16* t, const __nv_bfloat16* dy, long long n, float scale_b, float* partial_b,
                float* grad_b, int rp, int rank, long long m, int accumulate, cudaStream_t s);

// gemv.cu -- small-token forward (m <= 16).  Workspace: [16][64] fp32 for the low-rank input, then room for a resolved
// fp32 absmax (used only for nested layouts the kernel cannot read itself).  t_out (optional): bf16 [m, 64] = x . A^T.
size_t gemv_workspace_bytes(long long n, long long k);
bool gemv_reads_nested(const WeightView& w);
float* gemv_resolved_absmax_slot(void* workspace, long long n, long long k);
int gemv_forward(const WeightView& w, const __nv_bfloat16* x, const float* lora_a, const float* lora_b, float scaling,
                 int rank, __nv_bfloat16* y, int m, __nv_bfloat16* t_out, void* workspace, size_t workspace_bytes,
                 cudaStream_t s);

// skinny_sm100.cu -- few-token forward (m <= 128) on the tensor cores with the operands swapped: weight rows are the
// MMA rows, tokens its columns; reads a nested absmax itself when the second-level block size is a power of two.
// t_out (optional): bf16 [m, 64] = x . A^T.  flags: kGemmExactDecode or 0.
bool sm100_skinny_supported(const WeightView& w, int rank, long long m);
size_t sm100_skinny_bytes(long long n, long long k, long long m);
int sm100_skinny_forward(const WeightView& w, const __nv_bfloat16* x, const float* lora_a, const float* lora_b,
                         float scaling, int rank, __nv_bfloat16* y, int m, __nv_bfloat16* t_out, void* workspace,
                         size_t workspace_bytes, int flags, cudaStream_t s);

// gemm_sm100_pair.cu -- tcgen05 / TMEM GEMM with the NF4 decode fused in front of the tensor core
//   forward : out[m, n] = in[m, k] . deq(W)^T + low[m, 0..rp) . ext[n, 0..rp)^T        (ext = bf16(s B) [n, 64])
//   backward: out[m, k] = in[m, n] . deq(W)   + low[m, 0..rp) . ext[0..rp, k]           (ext = bf16(A)   [rp, k])
// low is bf16 [m, 64]; low == nullptr skips the low-rank block.
// split_ws: sm100_split_bytes() bytes of scratch for splitting the tiles of the last wave, or NULL (plain schedule)
// flags: kGemmNoSplit keeps the plain schedule, kGemmForceSplit splits whenever the shape allows it; kGemmTallTiles /
// kGemmShortTiles force the tile height (512 / 256 tokens per CTA pair) instead of the library's own choice
constexpr int kGemmNoSplit = 1, kGemmForceSplit = 2, kGemmTallTiles = 4, kGemmShortTiles = 8;
// few-token kernel: the decode that reproduces the dequantiser's bits instead of the faster table decode
constexpr int kGemmExactDecode = 16;
int sm100_gemm(bool backward, const WeightView& w, const float* absmax_f32, const __nv_bfloat16* in,
               const __nv_bfloat16* low, const __nv_bfloat16* ext, int rp, __nv_bfloat16* out, long long m,
               void* split_ws, int flags, cudaStream_t s);
// the same kernel for a dense bf16 weight [n, k] (B tiles loaded ready-made): forward out[m, n] = in . weight^T,
// backward out[m, k] = in[m, n] . weight
int sm100_dense_gemm(bool backward, const __nv_bfloat16* weight, long long n, long long k, const __nv_bfloat16* in,
                     __nv_bfloat16* out, long long m, void* split_ws, int flags, cudaStream_t s);
size_t sm100_split_bytes();
size_t workspace_bytes(int op, int64_t m, int64_t n, int64_t k, int rank, bool with_optional);
bool sm100_gemm_supported(const WeightView& w, int rank);

// api.cu -- process-wide options (molt_set_option)
long long wait_limit_cycles();     // limit of every bounded device-side wait, in SM clock cycles
int take_withheld_blocks();        // failure injection for tests: returns the pending count and clears it

// elementwise helpers used by the block op
int add_bf16(const __nv_bfloat16* a, const __nv_bfloat16* b, __nv_bfloat16* out, long long count, cudaStream_t s);

}  // namespace molt
