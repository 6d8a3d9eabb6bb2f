/*
 * molt_b200 -- C ABI of the B200 (sm_100a) NF4 + LoRA hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (cudaStream_t passed as uintptr_t).  The library never allocates or frees
 * device memory and keeps no pointer after a call returns.  It never
 * synchronises the stream or the device (molt_read_status excepted).  All
 * tensors are row-major and contiguous.  The calling thread's current CUDA
 * device must be the device that owns the pointers.
 *
 * Return value of every int function: 0 = ok, otherwise one of MOLT_E_*; the
 * message of the last failure on the calling thread is molt_last_error().
 *
 * Paths cited as "reference" are files of the MOLT project (src/molt_stream/...).
 */
#ifndef MOLT_B200_H_
#define MOLT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOLT_OK 0
#define MOLT_E_VALUE 1      /* shape / argument mismatch   -> ValueError      (reference: nf4_backward.py:181-182) */
#define MOLT_E_CAPABILITY 2 /* unsupported dtype/rank/etc. -> CapabilityError (reference: core/errors.py:5-6)     */
#define MOLT_E_RUNTIME 3    /* CUDA launch / driver failure -> RuntimeError                                         */
#define MOLT_E_TIMEOUT 4    /* a bounded device-side wait expired (see molt_read_status)                            */

#define MOLT_ABSMAX_F32 0     /* absmax is float[blocks]                      (reference: streaming/nf4.py:58)      */
#define MOLT_ABSMAX_NESTED 1  /* absmax is uint8[blocks] + absmax2/code2/offset (reference: nf4_backward.py:154-160) */

#define MOLT_NIBBLE_LOW_FIRST 0  /* element 2i in bits 0-3 (reference: streaming/nf4.py:62)        */
#define MOLT_NIBBLE_HIGH_FIRST 1 /* element 2i in bits 4-7 (reference: nf4_backward.py:97-98)     */

#define MOLT_DTYPE_BF16 0
#define MOLT_DTYPE_F32 1

/* kernel selection for the linear ops; for aligned shapes (K % 64 == 0, N % 64 == 0, blocksize 64, rank <= 64) AUTO
 * picks, forward, GEMV for M <= 8 and the few-token kernel for M <= 128, else the tcgen05 GEMM; the general kernels
 * for every other shape. */
#define MOLT_PATH_AUTO 0
#define MOLT_PATH_GENERAL 1
#define MOLT_PATH_TCGEN05 2
#define MOLT_PATH_GEMV 3
#define MOLT_PATH_FEW_TOKENS 4 /* forward, M <= 128: tcgen05 with the weight rows as the MMA rows and the tokens as its columns */
/* Optional flags, OR-ed onto a path: schedule of the tensor-core GEMMs when the last wave of output tiles is partial. */
#define MOLT_PATH_NO_SPLIT 0x100    /* keep the plain tile schedule                                      */
#define MOLT_PATH_FORCE_SPLIT 0x200 /* cut the tiles of the last wave along the contraction whenever the shape allows it */
#define MOLT_PATH_TALL_TILES 0x400  /* tensor-core GEMMs: 512-token tiles per CTA pair (two MMAs per decoded weight tile) */
#define MOLT_PATH_SHORT_TILES 0x800 /* tensor-core GEMMs: 256-token tiles per CTA pair; neither flag = the library chooses */
#define MOLT_PATH_EXACT_DECODE 0x1000 /* few-token kernel: decode with the dequantiser's bits instead of the table decode */

/* operations for molt_workspace_bytes */
#define MOLT_OP_LORA_FWD 1
#define MOLT_OP_LORA_BWD 2
#define MOLT_OP_DX 3
#define MOLT_OP_MLP_FWD 4
#define MOLT_OP_MLP_BWD 5

/* A frozen NF4 weight W[n, k] as it lies in device memory.
 * Replaces the (packed, scales, shape, block_size) payload of reference streaming/nf4.py:21-35 and the
 * duck-typed bitsandbytes quant_state read at reference methods/nf4_backward.py:147-163. */
typedef struct molt_nf4_desc {
  const uint8_t* packed;  /* ceil(n*k / blocksize) * blocksize / 2 bytes, two codes per byte */
  const void* absmax;     /* float[blocks] or uint8[blocks], see absmax_kind                  */
  const float* absmax2;   /* nested only: float[ceil(blocks / block2)]                        */
  const float* code2;     /* nested only: float[256] lookup table                             */
  float offset;           /* nested only: added after code2[u8] * absmax2                     */
  int32_t absmax_kind;    /* MOLT_ABSMAX_*                                                    */
  int32_t block2;         /* nested only: absmax codes per absmax2 entry (256)                */
  int32_t blocksize;      /* weight elements per absmax (64)                                  */
  int32_t nibble_order;   /* MOLT_NIBBLE_*                                                    */
  int32_t reserved;
  int64_t n;              /* out_features (rows of W)                                         */
  int64_t k;              /* in_features  (columns of W)                                      */
  float codebook[16];     /* the 16 NF4 values (reference: streaming/nf4.py:10-18)            */
} molt_nf4_desc;

int molt_version(void);
/* Message of the last failing call on this thread ("" if none). */
const char* molt_last_error(void);

/* Number of kernels this library has launched in this process (all threads, all devices). */
uint64_t molt_launch_count(void);

/* Process-wide options.
 * MOLT_OPT_WAIT_LIMIT_US: limit of every bounded device-side wait in microseconds (default 1,000,000; 100 .. 60,000,000).
 * MOLT_OPT_WITHHOLD_BLOCKS: failure injection for tests, made on the host: the NEXT tensor-core GEMM launch is told to
 *   request this many contraction blocks fewer than its consumers expect, so that a bounded wait runs out, the kernel
 *   records MOLT_E_TIMEOUT in the status word and returns (its output is then incomplete).  Cleared by that launch. */
#define MOLT_OPT_WAIT_LIMIT_US 1
#define MOLT_OPT_WITHHOLD_BLOCKS 2
int molt_set_option(int option, int64_t value);

/* Device-side status word.  The kernels bound every wait; when one expires the kernel records
 * (MOLT_E_TIMEOUT << 24) | (wait site << 16) | block index here and returns with its output incomplete.
 * Reads and clears it (synchronises the given stream). 0 = clean.  Callers of the C ABI must poll this word at a
 * step boundary: it is the only report of an expired wait. */
int molt_read_status(uintptr_t stream, int32_t* status_out);

/* out[n, k] = codebook[code] * absmax, one fp32 multiply, cast last.
 * Replaces NF4DevicePayload.dequantize (reference streaming/nf4.py:29-35) and
 * bitsandbytes dequantize_4bit at reference methods/nf4_lora.py:98, nf4_layer_cache.py:51. */
int molt_nf4_dequant(const molt_nf4_desc* w, void* out, int out_dtype, uintptr_t stream);

/* out[blocks] = fp32 absmax (nested form resolved).  Replaces resolved_nf4_scales
 * (reference methods/nf4_backward.py:145-164). */
int molt_nf4_resolve_absmax(const molt_nf4_desc* w, float* out, uintptr_t stream);

/* Scratch bytes the given op uses for these sizes (0 if none).  The figure includes an optional part (about 38 MB on a
 * 148-SM device): room for the fp32 partial tiles with which the tensor-core GEMMs split the tiles of their last,
 * partial wave along the contraction.  A smaller workspace that still holds the required buffers is accepted; the
 * GEMMs then keep the plain tile schedule. */
size_t molt_workspace_bytes(int op, int64_t m, int64_t n, int64_t k, int rank);

/* y[m, n] = x[m, k] . deq(W)^T + scaling * (x . A^T) . B^T      (x, y bf16; A[rank, k], B[n, rank] fp32)
 * Replaces _ScheduledNF4LoRA.forward (reference methods/nf4_lora.py:23-69), _nf4_lora_forward
 * (reference methods/gated_replay.py:211-224) and _FrozenNF4LoRA.forward (reference streaming/engine.py:21-31).
 * t_out (optional, may be NULL): bf16 [m, 64] receives x . A^T zero-padded to 64 columns, for reuse in backward. */
int molt_nf4_lora_fwd(const molt_nf4_desc* w, const void* x, const float* lora_a, const float* lora_b,
                      float scaling, int rank, void* y, int64_t m, void* t_out, void* workspace,
                      size_t workspace_bytes, int path, uintptr_t stream);

/* dx[m, k] = dy . deq(W) + (scaling * dy . B) . A ; da[rank, k] = (scaling * dy . B)^T . x ;
 * db[n, rank] = scaling * dy^T . (x . A^T).   dx bf16 (may be NULL to skip), da/db fp32 (may both be NULL).
 * Replaces _ScheduledNF4LoRA.backward (reference methods/nf4_lora.py:71-113), _nf4_lora_backward
 * (reference methods/gated_replay.py:227-253) and _FrozenNF4LoRA.backward (reference streaming/engine.py:33-48).
 * t_in (optional): the t_out of the matching forward; recomputed from x when NULL.
 * accumulate != 0 adds into da/db instead of overwriting them. */
int molt_nf4_lora_bwd(const molt_nf4_desc* w, const void* x, const void* dy, const float* lora_a,
                      const float* lora_b, float scaling, int rank, void* dx, float* da, float* db,
                      int64_t m, const void* t_in, int accumulate, void* workspace, size_t workspace_bytes,
                      int path, uintptr_t stream);

/* dx[m, k] = dy[m, n] . deq(W) (+ scaling * lora_grad[m, rank] . A[rank, k] when lora_grad != NULL).
 * Replaces packed_nf4_backward_input and packed_nf4_lora_backward_input
 * (reference methods/nf4_backward.py:167-284).  lora_a_dtype: MOLT_DTYPE_BF16 or MOLT_DTYPE_F32.
 * On the tensor-core path both terms accumulate in fp32 and are rounded once; the general path rounds the base to
 * bf16 before adding the low-rank term as the reference does (:127-136). */
int molt_nf4_dx(const molt_nf4_desc* w, const void* dy, const void* lora_grad, const void* lora_a,
                int lora_a_dtype, float scaling, int rank, void* dx, int64_t m, void* workspace,
                size_t workspace_bytes, int path, uintptr_t stream);

/* Same operation and arguments as molt_nf4_lora_fwd, minus t_out and the workspace: the scratch is a fixed
 * MOLT_STATIC_SCRATCH_BYTES array inside the library's device image, so this call allocates nothing and asks the
 * caller for nothing.  It is meant for hosts that cannot allocate device memory where they call the library (a
 * server that pins its whole device budget at start-up, a plugin without an allocator of its own).  It has no
 * counterpart in the reference.  The result is that of molt_nf4_lora_fwd given a workspace without the optional
 * split region.  Problems whose scratch need exceeds the array are refused (MOLT_E_VALUE).  All
 * calls on a device share the array: calls that may overlap on the GPU must be serialised by the caller.  The
 * first call on a device looks the array's address up; make it before any stream capture. */
#define MOLT_STATIC_SCRATCH_BYTES (16u << 20)
int molt_nf4_lora_fwd_static(const molt_nf4_desc* w, const void* x, const float* lora_a, const float* lora_b,
                             float scaling, int rank, void* y, int64_t m, int path, uintptr_t stream);

/* Small-token forward (m <= 16): streams the packed weight once.  Same contract as molt_nf4_lora_fwd.
 * Replaces the bitsandbytes GEMV that bnb.matmul_4bit dispatches for few tokens (reference methods/nf4_lora.py:43-47). */
int molt_nf4_gemv(const molt_nf4_desc* w, const void* x, const float* lora_a, const float* lora_b,
                  float scaling, int rank, void* y, int64_t m, void* workspace, size_t workspace_bytes,
                  uintptr_t stream);

/* h = silu(g) * u, fp32 internal, one rounding.  Replaces _silu_mul_forward
 * (reference kernels/gated_activation.py:29-36).  dtype: MOLT_DTYPE_*. */
int molt_swiglu_fwd(const void* gate, const void* up, void* out, int64_t count, int dtype, uintptr_t stream);

/* dgate = dh * u * sig(g) * (1 + g * (1 - sig(g))), dup = dh * silu(g); optionally also re-emits
 * h = silu(g) * u (h_out != NULL) for the down-projection backward of the replay schedule.
 * Replaces _silu_mul_backward (reference kernels/gated_activation.py:38-51) and the eager replay
 * arithmetic at reference methods/gated_replay.py:373-387. */
int molt_swiglu_bwd(const void* grad_out, const void* gate, const void* up, void* dgate, void* dup,
                    void* h_out, int64_t count, int dtype, uintptr_t stream);

/* out = bf16(x * rsqrt(mean(x^2) + eps) * (weight + weight_offset)); x bf16 [rows, width], weight fp32 or bf16.
 * Replaces _RMSNormReplayRecipe.materialize (reference methods/gated_replay.py:22-29). */
int molt_rmsnorm_fwd(const void* x, const void* weight, int weight_dtype, float eps, float weight_offset,
                     void* out, int64_t rows, int64_t width, uintptr_t stream);

/* grad_x = bf16(inv * (dy (w + offset) - x inv * mean(dy (w + offset) * x inv))), inv = rsqrt(mean(x^2) + eps); the weight is
 * frozen, so there is no weight gradient.  Replaces _FrozenRMSNormFunction.backward
 * (reference kernels/frozen_rmsnorm.py:25-37); molt_rmsnorm_fwd is also its forward (:11-23). */
int molt_rmsnorm_bwd(const void* grad_out, const void* x, const void* weight, int weight_dtype, float eps,
                     float weight_offset, void* grad_x, int64_t rows, int64_t width, uintptr_t stream);

/* The residual add fused with the RMSNorm behind it: sum_out = bf16(x + delta), out = RMSNorm(sum_out) as
 * molt_rmsnorm_fwd computes it (one pass over the hidden states instead of two).  width a multiple of 8.  Fuses the
 * residual add of the decoder layer with reference kernels/frozen_rmsnorm.py:11-23. */
int molt_add_rmsnorm_fwd(const void* x, const void* delta, const void* weight, int weight_dtype, float eps,
                         float weight_offset, void* sum_out, void* out, int64_t rows, int64_t width, uintptr_t stream);

/* Its backward: grad_x = bf16(grad_sum + RMSNorm-backward(grad_out; sum)), the gradient of both x and delta
 * (reference kernels/frozen_rmsnorm.py:25-37 plus the gradient accumulation of the residual stream). */
int molt_add_rmsnorm_bwd(const void* grad_out, const void* grad_sum, const void* sum, const void* weight,
                         int weight_dtype, float eps, float weight_offset, void* grad_x, int64_t rows, int64_t width,
                         uintptr_t stream);

/* Rotary position embedding of q [batch, seq, heads, head_dim] and k [batch, seq, kv_heads, head_dim] (bf16) into
 * q_out / k_out (which may be q / k themselves): (x1, x2) -> (x1 cos - x2 sin, x2 cos + x1 sin) over the two halves of
 * every head vector; cos / sin are bf16 [seq, head_dim] tables with equal halves; inverse != 0 applies the transposed
 * rotation (the gradient).  head_dim a multiple of 16; kv_heads = 0 rotates q alone.  Part of the step driver around the path (the reference trainer
 * uses the model's own). */
int molt_rope(const void* q, const void* k, void* q_out, void* k_out, const void* cos_table, const void* sin_table,
              int64_t batch, int64_t seq, int heads, int kv_heads, int head_dim, int inverse, uintptr_t stream);

/* One AdamW step (decoupled weight decay, bias correction as in torch.optim.AdamW) over flat fp32 arrays of `count`
 * elements (a multiple of 4): every adapter's parameters, gradients and moments laid end to end, so one launch steps
 * them all.  grad is multiplied by grad_scale first (1 / world size after a summing all-reduce).  step counts from 1.
 * Replaces the per-parameter optimizer loop the reference builds at training/qlora.py:218-243 and steps at :982-986. */
int molt_adamw_step(float* param, const float* grad, float* exp_avg, float* exp_avg_sq, int64_t count, float lr,
                    float beta1, float beta2, float eps, float weight_decay, int64_t step, float grad_scale,
                    uintptr_t stream);

/* Frozen-head cross-entropy on bf16 logits [rows, vocab]: row_loss[row] = logsumexp(logits) - logits[target], and
 * logits is overwritten by (softmax - onehot) * grad_scale (bf16).  fp32 arithmetic, two passes over each row.
 * Replaces _fused_ce_loss_kernel_online / _fused_ce_softmax_grad_kernel_online
 * (reference kernels/frozen_linear_cross_entropy.py:27-139). */
int molt_ce_softmax_grad(void* logits, const int64_t* targets, float* row_loss, int64_t rows, int64_t vocab,
                         float grad_scale, uintptr_t stream);

/* GEMM against a dense, frozen bf16 weight [n, k] (the LM head), on the tensor-core kernel of the NF4 linears with its B
 * tiles loaded ready-made: contract_over_rows == 0: out[m, n] = in[m, k] . weight^T (logits = hidden . head^T);
 * contract_over_rows != 0: out[m, k] = in[m, n] . weight (dhidden = dlogits . head).  bf16 in and out, fp32 accumulation;
 * n and k multiples of 64.  workspace (optional, molt_dense_gemm_workspace_bytes()): scratch for splitting a partial last
 * wave of tiles; flags: MOLT_PATH_NO_SPLIT / FORCE_SPLIT / TALL_TILES / SHORT_TILES or 0.
 * Replaces the two F.linear calls around the cross-entropy kernels at reference
 * kernels/frozen_linear_cross_entropy.py:181-236 (with molt_ce_softmax_grad between them). */
size_t molt_dense_gemm_workspace_bytes(void);
int molt_dense_gemm(const void* weight, int64_t n, int64_t k, const void* in, void* out, int64_t m,
                    int contract_over_rows, void* workspace, size_t workspace_bytes, int flags, uintptr_t stream);

/* bf16 "shadow" operands of one adapter for the tensor-core kernels, so that they need not be rebuilt from the fp32
 * masters in front of every call: a16 [rp, k] = bf16(A) (rp = rank rounded up to 16, extra rows zero), bs [n, 64] =
 * bf16(scaling * B) (extra columns zero), bt [rp, n] = its transpose.  The caller owns the buffers and refreshes them
 * with molt_lora_shadow_refresh whenever A or B changed (i.e. after each optimizer step).  Counterpart of the
 * reference's bf16 LoRA shadows (methods/lora_shadow.py:19-141). */
typedef struct molt_lora_shadow {
  const void* a16;
  const void* bs;
  const void* bt;
} molt_lora_shadow;

/* One adapter of a refresh: masters in, shadows out (all device pointers). */
typedef struct molt_lora_shadow_item {
  const float* lora_a; /* [rank, k] */
  const float* lora_b; /* [n, rank] */
  float scaling;
  int32_t rank;
  int64_t n, k;        /* multiples of 64 */
  void* a16;
  void* bs;
  void* bt;
} molt_lora_shadow_item;

/* Rebuilds the shadows of `count` adapters in ONE launch; `items` is an array in DEVICE memory (the host builds it
 * once).  Meant to follow molt_adamw_step in the stream. */
int molt_lora_shadow_refresh(const molt_lora_shadow_item* items, int count, int64_t max_n, int64_t max_k,
                             uintptr_t stream);

/* molt_nf4_lora_fwd / molt_nf4_lora_bwd with the adapter's shadows given: the tensor-core path skips its operand
 * preparation (shadow may be NULL: then exactly the plain entry points).  lora_a / lora_b are still needed (kernels
 * for few tokens and general shapes read the masters). */
int molt_nf4_lora_fwd_prepared(const molt_nf4_desc* w, const void* x, const float* lora_a, const float* lora_b,
                               float scaling, int rank, const molt_lora_shadow* shadow, void* y, int64_t m, void* t_out,
                               void* workspace, size_t workspace_bytes, int path, uintptr_t stream);
int molt_nf4_lora_bwd_prepared(const molt_nf4_desc* w, const void* x, const void* dy, const float* lora_a,
                               const float* lora_b, float scaling, int rank, const molt_lora_shadow* shadow, void* dx,
                               float* da, float* db, int64_t m, const void* t_in, int accumulate, void* workspace,
                               size_t workspace_bytes, int path, uintptr_t stream);

/* Gated MLP block: gate = P_g(x), up = P_u(x), y = P_d(silu(gate) * up).
 * gate_out [m, inter] is always written (it is what the replay schedule saves); up_out may be NULL when the
 * caller re-materialises `up` in backward.  Replaces _ResidualRecipeGatedNF4LoRA.forward
 * (reference methods/gated_replay.py:53-133) / _AsymmetricGatedNF4LoRA.forward (:266-339). */
typedef struct molt_lora_proj {
  const molt_nf4_desc* w;
  const float* lora_a;  /* [rank, k] */
  const float* lora_b;  /* [n, rank] */
  float scaling;
  int32_t rank;
  const struct molt_lora_shadow* shadow; /* optional bf16 operands kept up to date by the caller (see below), or NULL */
} molt_lora_proj;

/* Scratch bytes of molt_mlp_fwd (op = MOLT_OP_MLP_FWD) / molt_mlp_bwd (op = MOLT_OP_MLP_BWD) for m tokens;
 * up_given != 0 when the caller passes up_out / up_saved. */
size_t molt_mlp_workspace_bytes(int op, const molt_lora_proj* gate, const molt_lora_proj* up,
                                const molt_lora_proj* down, int64_t m, int up_given);

int molt_mlp_fwd(const molt_lora_proj* gate, const molt_lora_proj* up, const molt_lora_proj* down,
                 const void* x, void* gate_out, void* up_out, void* y, int64_t m, void* workspace,
                 size_t workspace_bytes, uintptr_t stream);

/* Backward of the block with `up` replayed when up_saved == NULL.  Writes dx [m, hidden] and the six
 * adapter gradients grads[6] = {gate_a, gate_b, up_a, up_b, down_a, down_b} (fp32).
 * Replaces _ResidualRecipeGatedNF4LoRA.backward (reference methods/gated_replay.py:135-208) and
 * _AsymmetricGatedNF4LoRA.backward (:341-407). */
int molt_mlp_bwd(const molt_lora_proj* gate, const molt_lora_proj* up, const molt_lora_proj* down,
                 const void* x, const void* gate_saved, const void* up_saved, const void* dy, void* dx,
                 float* const grads[6], int accumulate, int64_t m, void* workspace, size_t workspace_bytes,
                 uintptr_t stream);

/* The same pair with the block's three low-rank inputs kept between them: t_out / t_saved is one buffer of
 * [3][m][64] bf16 (T = bf16(in . bf16(A)^T) of gate, up and down, zero padded to 64 columns), 3 * m * 128 bytes.
 * Given t_saved the backward recomputes none of them, and rebuilds h = silu(gate) * up in the same pass that forms
 * dgate and dup (after dh = dY . deq(W_down) + ..., which needs no h) instead of a pass of its own in front.  Same
 * results as molt_mlp_fwd / molt_mlp_bwd bit for bit; NULL gives exactly those.  The reference saves no such tensor
 * (methods/gated_replay.py:307-323 keeps x, gate and optionally up); it is 384 bytes per token. */
int molt_mlp_fwd_t(const molt_lora_proj* gate, const molt_lora_proj* up, const molt_lora_proj* down, const void* x,
                   void* gate_out, void* up_out, void* y, void* t_out, int64_t m, void* workspace,
                   size_t workspace_bytes, uintptr_t stream);
int molt_mlp_bwd_t(const molt_lora_proj* gate, const molt_lora_proj* up, const molt_lora_proj* down, const void* x,
                   const void* gate_saved, const void* up_saved, const void* t_saved, const void* dy, void* dx,
                   float* const grads[6], int accumulate, int64_t m, void* workspace, size_t workspace_bytes,
                   uintptr_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MOLT_B200_H_ */
