/*
 * bastile_b200 — C ABI of the sm_100a kernels behind the four Qwen3 training
 * ops that aghilann/bastile patches into HuggingFace transformers.
 *
 * Conventions shared by every entry point
 *   - plain device pointers, element counts and element strides; no torch types;
 *   - `dtype`: BT_BF16 / BT_FP16 / BT_FP32 storage, all arithmetic in fp32;
 *   - `stream`: a cudaStream_t passed as void* (NULL = legacy default stream);
 *   - return value: 0 on success, a negative BT_ERR_* code otherwise; the text of
 *     the last failure on the calling thread is available from bt_last_error();
 *   - nothing here allocates or frees device memory, synchronises the device or
 *     throws: the caller owns every buffer for the duration of the call only.
 *   - there is no CPU implementation behind this interface.
 *
 * Each declaration cites the function of the reference (path within the
 * aghilann/bastile source tree : lines) whose device work it replaces.
 */
#ifndef BASTILE_B200_H_
#define BASTILE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BT_BF16 0
#define BT_FP16 1
#define BT_FP32 2

#define BT_OK 0
#define BT_ERR_ARG (-1)      /* bad shape, stride, alignment or dtype            */
#define BT_ERR_LAUNCH (-2)   /* CUDA runtime error at launch (cudaGetLastError)  */
#define BT_ERR_DEVICE (-3)   /* a bounded device-side wait ran out (status word) */
#define BT_ERR_DRIVER (-4)   /* tensor-map encode / driver entry point failure   */
#define BT_ERR_LIMIT (-5)    /* size beyond a stated maximum                     */

/* Bits of the caller-owned int32 device status word that several entry points take.  The
 * low four are set by the tensor-core kernels when a bounded barrier wait runs out (producer,
 * MMA issuer waiting for an accumulator / for operands, epilogue): the results of that launch
 * are invalid.  BT_STATUS_BAD_LABEL reports invalid INPUT, not a device problem. */
#define BT_STATUS_WAIT_MASK 0x0f
#define BT_STATUS_BAD_LABEL 0x10

/* Library version (major*10000 + minor*100 + patch). No reference counterpart
 * (the reference is a JIT Python package: src/bastile/__init__.py:23). */
int bt_version(void);

/* Text of the last error raised on this thread ("" if none). */
const char* bt_last_error(void);

/* Number of SMs of the current device (src/bastile/ops/utils.py:8-13). */
int bt_sm_count(void);

/* Every device-side wait of this library (mbarrier waits of the tensor-core and bulk-copy
 * kernels, polls of the run-time tile hand-out) gives up after a limit and reports through the
 * status word / bt_device_wait_errors().  The limit is WALL time on the device clock (default
 * 1000 ms): it keeps counting while the context is descheduled (time-slicing between
 * processes, MPS, a debugger), so a process that shares its GPU that way should raise it.  Sets
 * the limit for kernels launched afterwards on the CURRENT device; 1 .. 600000 ms.  No reference
 * counterpart (CuTile kernels do not wait on one another). */
int bt_set_wait_limit_ms(int64_t ms);

/* Synchronising read-and-clear of the device word in which the RMSNorm kernels
 * record a bulk-copy wait that ran out (0 = none, -1 = the read failed).  For
 * tests and debugging; no reference counterpart. */
int bt_device_wait_errors(void);

/* ------------------------------------------------------------------ RMSNorm */

/* y[m,:] = x[m,:] * rsqrt(mean(x[m,:]^2) + eps) * w, rounded once to `dtype`;
 * rstd[m] (fp32) is saved for the backward.  x rows are ld_x elements apart,
 * y rows ld_y.  Replaces _rms_fwd + CuTileRMSNormFunction.forward
 * (src/bastile/ops/rms_norm.py:15-34, 105-126). */
int bt_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd,
                   int64_t M, int64_t N, int64_t ld_x, int64_t ld_y,
                   float eps, int dtype, void* stream);

/* dx = (dy*w - xhat*mean(xhat*dy*w)) * rstd, dw = sum_rows dy*xhat with
 * xhat = x*rstd.  `ws` is caller-owned scratch of bt_rmsnorm_bwd_ws_bytes(N)
 * bytes that must be ZERO on entry; the kernel leaves it zero again on exit, so
 * one zero-initialised buffer can be reused by successive calls on one stream.
 * Replaces _rms_bwd, the torch partial-sum reduction and the dtype cast
 * (src/bastile/ops/rms_norm.py:37-68, 128-153). */
int bt_rmsnorm_bwd(const void* dy, const void* x, const void* w,
                   const float* rstd, void* dx, void* dw, void* ws,
                   int64_t M, int64_t N, int64_t ld_dy, int64_t ld_x,
                   int64_t ld_dx, int dtype, void* stream);
int64_t bt_rmsnorm_bwd_ws_bytes(int64_t N);

/* The residual add in front of a norm, fused into it (the reference keeps them
 * apart: `hidden_states = residual + hidden_states` then the patched
 * Qwen3RMSNorm, transformers modeling_qwen3.py:326-333 around
 * src/bastile/ops/rms_norm.py:156-168):
 *   sum = T(x + residual)   (written out: it is the next residual stream)
 *   y   = sum * rstd * w,   rstd from the ROUNDED sum, as the unfused pair gives.
 * All of x, residual, sum, y are [M,N] with their own row strides. */
int bt_add_rmsnorm_fwd(const void* x, const void* residual, const void* w,
                       void* sum, void* y, float* rstd, int64_t M, int64_t N,
                       int64_t ld_x, int64_t ld_residual, int64_t ld_sum,
                       int64_t ld_y, float eps, int dtype, void* stream);

/* bt_rmsnorm_bwd whose dx also takes in the gradient that reaches the norm's
 * input along the residual path: dx = T(norm_backward(dy) + dresidual).  Saves
 * the separate gradient-accumulation pass autograd runs where the two branches
 * of a residual block meet.  Scratch contract as bt_rmsnorm_bwd. */
int bt_add_rmsnorm_bwd(const void* dy, const void* x, const void* w,
                       const float* rstd, const void* dresidual, void* dx,
                       void* dw, void* ws, int64_t M, int64_t N, int64_t ld_dy,
                       int64_t ld_x, int64_t ld_dresidual, int64_t ld_dx,
                       int dtype, void* stream);

/* bt_rmsnorm_bwd for callers that cannot provide scratch memory.  It has no
 * counterpart in the reference (there, torch allocates the partial-sum tensor).
 * Meant for hosts that reach this library through an FFI and hold no device
 * allocator - their tensors come from a framework that has reserved the device
 * memory for its own pool, so a cudaMalloc of their own is not theirs to make -
 * and for latency-critical paths that must avoid the device-wide
 * synchronisation of cudaMalloc/cudaFree.  The scratch is a fixed array inside
 * the library image: every GPU that loads the library holds it (about 64 KB)
 * until the process exits, and N may not exceed BT_RMSNORM_NOALLOC_MAX_N
 * (larger N returns BT_ERR_LIMIT).  The call allocates and frees nothing.
 * The first call on each device looks up the array's device address; make that
 * first call outside any stream capture.  All calls on a device share the one
 * array (it is cleared on the stream at the start of every call): two calls
 * whose kernels can overlap on the GPU - different streams, no ordering between
 * them - race on it and give wrong dw.  Arguments and results are otherwise
 * those of bt_rmsnorm_bwd. */
#define BT_RMSNORM_NOALLOC_MAX_N 16384
int bt_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w,
                           const float* rstd, void* dx, void* dw,
                           int64_t M, int64_t N, int64_t ld_dy, int64_t ld_x,
                           int64_t ld_dx, int dtype, void* stream);

/* --------------------------------------------------------------------- RoPE */

/* Rotate-half rotary embedding of q [B,Hq,T,D] and k [B,Hk,T,D]:
 *   out1 = in1*cos - in2*sin ; out2 = in2*cos + in1*sin   (halves of D)
 * using the FIRST D/2 columns of cos/sin rows [cos_bs in {1,B}, T, >=D/2].
 * Strides are in elements; the last dimension must be contiguous.  q_out may
 * equal q_in (in place, the forward) or be a separate buffer (the backward,
 * called with negate_sin = 1 on the incoming gradients).  Replaces
 * _rope_kernel / _reshape_and_launch / RoPEFunction
 * (src/bastile/ops/rope.py:13-90, 93-122, 125-136). */
int bt_rope(const void* q_in, const void* k_in, void* q_out, void* k_out,
            const void* cos, const void* sin,
            int64_t B, int64_t Hq, int64_t Hk, int64_t T, int64_t D,
            const int64_t q_in_strides[3],  /* b, h, t */
            const int64_t k_in_strides[3],
            const int64_t q_out_strides[3],
            const int64_t k_out_strides[3],
            const int64_t cos_strides[2],   /* b, t (shared by cos and sin) */
            int64_t cos_bs, int negate_sin, int dtype, void* stream);

/* ------------------------------------------------------ SwiGLU (elementwise) */

/* out = T(silu_fp32(gate)) * up, the product rounded to `dtype`
 * (swiglu_forward_kernel, src/bastile/ops/swiglu.py:23-50, 93-117). */
int bt_swiglu_fwd(const void* gate, const void* up, void* out,
                  int64_t rows, int64_t cols, int64_t ld_gate, int64_t ld_up,
                  int64_t ld_out, int dtype, void* stream);

/* dgate = dy*up*sig(g)*(1+g*(1-sig(g))), dup = dy*g*sig(g), fp32 math
 * (swiglu_backward_kernel, src/bastile/ops/swiglu.py:53-90, 120-146). */
int bt_swiglu_bwd(const void* dy, const void* gate, const void* up,
                  void* dgate, void* dup, int64_t rows, int64_t cols,
                  int64_t ld_dy, int64_t ld_gate, int64_t ld_up,
                  int64_t ld_dgate, int64_t ld_dup, int dtype, void* stream);

/* ------------------------------------------------------- tcgen05 GEMM core  */

/* D[M,N] = op(A) * op(B) with fp32 accumulation in tensor memory.  Operands are
 * BT_BF16 or BT_FP16 (result in the same type or fp32) or BT_FP32 (multiplied as
 * tf32, fp32 result); row strides must be multiples of 16 bytes.
 *   a_kmajor = 1: A is stored [M,K] with K contiguous (row stride lda)
 *   a_kmajor = 0: A is stored [K,M] with M contiguous (row stride lda)
 *   b_kmajor = 1: B is stored [N,K] with K contiguous (row stride ldb)
 *   b_kmajor = 0: B is stored [K,N] with N contiguous (row stride ldb)
 * The epilogue computes D = T_out(alpha[0] * (A*B + addend)): out_dtype selects
 * the storage of D (the operand dtype or BT_FP32, row stride ldd); `addend` is
 * an optional fp32 [M,N] matrix (row stride ld_addend; may alias an fp32 D to
 * accumulate in place); `alpha` is an optional DEVICE scalar (NULL = 1).
 * `status` points at a caller-owned, zero-initialised int32 device word that a
 * kernel sets non-zero if one of its bounded barrier waits runs out.
 * This is the library GEMM that the reference takes from cuBLAS through
 * torch.mm / nn.Linear (src/bastile/ops/swiglu.py:179-187,
 * src/bastile/ops/fused_linear_cross_entropy.py:167-185, 385). */
int bt_gemm(const void* A, const void* B, void* D,
            int64_t M, int64_t N, int64_t K,
            int64_t lda, int64_t ldb, int64_t ldd,
            int a_kmajor, int b_kmajor, int in_dtype, int out_dtype,
            const float* addend, int64_t ld_addend, const float* alpha,
            int32_t* status, void* stream);

/* bt_gemm with the rest of what the kernel can do, described by a struct (zero it, then
 * fill in what is needed):
 *   D = T_out(alpha[0] * (op(A)*op(B) + op(A1)*op(B1) + addend + addend_t))
 * A1/B1 is an optional second product (contraction length K1, same M, N and operand
 * layouts) accumulated in tensor memory before the epilogue; `addend_t` is an optional
 * [M,N] addend stored in the operand dtype, which may alias D (each element is read
 * before it is written).  With these, the input gradient of several linear layers that
 * share their input - dX = dQ Wq + dK Wk + dV Wv for the q/k/v projections of
 * Qwen3Attention (transformers modeling_qwen3.py:256-258), three cuBLAS GEMMs plus two
 * accumulation passes under autograd - is two launches and no elementwise pass. */
typedef struct bt_gemm_desc {
  const void* A;  const void* B;  int64_t lda, ldb, K;
  const void* A1; const void* B1; int64_t lda1, ldb1, K1;   /* A1 == NULL: no second product */
  void* D; int64_t ldd;
  int64_t M, N;
  int32_t a_kmajor, b_kmajor;      /* both products */
  int32_t in_dtype, out_dtype;
  const float* addend;  int64_t ld_addend;     /* fp32, or NULL */
  const void* addend_t; int64_t ld_addend_t;   /* operand dtype, or NULL */
  const float* alpha;                          /* device scalar, or NULL */
  /* A given as THREE tensors against one B (B1 unused); 0 = off.
   *   a_split = 1: side by side along K: D = [A | A1 | A2] * B with contraction lengths K, K1,
   *     K2 (K and K1 multiples of 64 elements, 32 for fp32) and B spanning K + K1 + K2 - the
   *     shared input gradient dX = [dQ | dK | dV] * [Wq; Wk; Wv] of the q/k/v projections
   *     (transformers modeling_qwen3.py:256-258) as ONE launch when the three weights lie one
   *     after the other in memory, without first copying dQ, dK, dV side by side.
   *   a_split = 2: stacked along M: rows [0, M0) of op(A) come from A, the next M1 from A1, the
   *     rest from A2 (M0, M1 multiples of 256; all three with contraction length K) - the three
   *     weight gradients [dQ | dK | dV]^T * X as one product into one stacked result. */
  const void* A2; int64_t lda2, K2;
  int32_t a_split;
  /* d_split = 1: the result is THREE tensors side by side along N: columns [0, N0) go to D (row
   * stride ldd), the next N1 to D1, the rest to D2 (N0, N1 multiples of 256; no addends) - the
   * q, k and v projections as one product x * [Wq; Wk; Wv]^T that still hands each its own
   * dense tensor. */
  int32_t d_split;
  int64_t M0, M1;
  void* D1; void* D2; int64_t ldd1, ldd2, N0, N1;
} bt_gemm_desc;
int bt_gemm_ex(const bt_gemm_desc* desc, int32_t* status, void* stream);

/* Selects how the tensor-core kernels tile their work: 0 = one CTA per 128x256
 * output tile (tcgen05 cta_group::1), 1 = pairs of CTAs in a 2-CTA cluster on
 * 256x256 tiles (cta_group::2).  A negative argument only queries.  Returns the
 * previous setting.  Process-wide; not a per-call option.  No reference
 * counterpart (cuBLAS picks its own kernels). */
int bt_set_gemm_cta_pairs(int enable);

/* How the tensor-core kernels write 16-bit results whose rows are 16-byte aligned: 1 (default) =
 * every epilogue warp stages 32 x 32 pieces in shared memory and issues tile stores
 * (cp.async.bulk.tensor), 0 = every thread stores its own row pieces from registers.  Same
 * bits either way.  A negative argument only queries; returns the previous setting.  Process-wide.
 * No reference counterpart. */
int bt_set_gemm_tile_stores(int enable);

/* Tile rasterisation of the tensor-core kernels: CTAs walk `row_tiles` row tiles of the result
 * for one column tile before moving to the next column tile, so that concurrently running CTAs
 * share operand tiles in L2.  0 (default) = the library's own choice per launch; a negative
 * argument only queries; returns the previous setting.  Process-wide; a tuning knob with no
 * reference counterpart (cuBLAS picks its own schedule). */
int bt_set_gemm_group_rows(int row_tiles);

/* 1 (default): the library launches its kernels as programmatic dependents of whatever precedes
 * them in the stream (cudaLaunchAttributeProgrammaticStreamSerialization): a kernel is set up on
 * the SMs while its predecessor drains and executes griddepcontrol.wait before its first access
 * to global memory, which takes the launch gap (about 2 us per launch on a B200) out of a chain
 * of short kernels.  0: ordinary launches.  Same results either way.  A negative argument only
 * queries; returns the previous setting.  Process-wide.  No reference counterpart. */
int bt_set_dependent_launch(int enable);

/* ------------------------------------------- per-head RMSNorm + RoPE, fused */

/* q_norm / k_norm followed by the rotary embedding, for the two tensors of
 * heads q [B,T,Hq,D] and k [B,T,Hk,D] (the projection outputs viewed per head;
 * element strides of batch, position, head; D contiguous), in one launch:
 *   y   = T(x * rstd * w)            per head row, rstd[b,t,h] = rsqrt(mean(x^2)+eps)
 *   out = rotate-half RoPE of y with cos/sin[b or 0, t, 0..D/2)
 * Replaces the patched Qwen3RMSNorm on head_dim-wide rows
 * (src/bastile/ops/rms_norm.py:105-126) and _rope_kernel
 * (src/bastile/ops/rope.py:13-90) that Qwen3Attention.forward runs back to
 * back (transformers modeling_qwen3.py:256-261).  rstd_q / rstd_k are
 * [B*T*H] in (b,t,h) order.  Head rows must be 128, 256 or 512 bytes
 * (D = 64/128/256 for 16-bit types); anything else returns BT_ERR_ARG and the
 * caller runs bt_rmsnorm_fwd and bt_rope instead.  Results are bit-identical
 * to that pair of calls. */
int bt_qk_norm_rope_fwd(const void* q, const void* k, const void* wq, const void* wk,
                        const void* cos, const void* sin, void* q_out, void* k_out,
                        float* rstd_q, float* rstd_k,
                        int64_t B, int64_t T, int64_t Hq, int64_t Hk, int64_t D,
                        const int64_t q_strides[3], const int64_t k_strides[3],
                        const int64_t q_out_strides[3], const int64_t k_out_strides[3],
                        const int64_t cos_strides[2], int64_t cos_bs,
                        float eps_q, float eps_k, int dtype, void* stream);

/* Backward of the pair: un-rotates dq_out / dk_out (rope.py:132-136), then the
 * RMSNorm backward (rms_norm.py:37-68, 128-153) gives dq, dk and the two weight
 * gradients dwq, dwk [D].  ws_q and ws_k: two separate scratch buffers of
 * bt_rmsnorm_bwd_ws_bytes(D) zeroed bytes each, left zero (as bt_rmsnorm_bwd). */
int bt_qk_norm_rope_bwd(const void* dq_out, const void* dk_out, const void* q, const void* k,
                        const void* wq, const void* wk, const float* rstd_q, const float* rstd_k,
                        const void* cos, const void* sin, void* dq, void* dk,
                        void* dwq, void* dwk, void* ws_q, void* ws_k,
                        int64_t B, int64_t T, int64_t Hq, int64_t Hk, int64_t D,
                        const int64_t dq_out_strides[3], const int64_t dk_out_strides[3],
                        const int64_t q_strides[3], const int64_t k_strides[3],
                        const int64_t dq_strides[3], const int64_t dk_strides[3],
                        const int64_t cos_strides[2], int64_t cos_bs, int dtype, void* stream);

/* How the CTA pairs of the tensor-core kernels get their output tiles: 0
 * (default) = dealt round-robin at launch, 1 = drawn from a global counter while
 * the kernel runs.  Dynamic hand-out is for a GPU whose SMs the GEMM has to
 * share with another stream's long-running kernels (NCCL collectives under
 * data-parallel training): a pair that gets its SMs late then finds few tiles
 * left instead of its whole fixed share.  It costs one small memset per launch
 * (the scheduler's words live in a fixed pool inside the library; nothing is
 * allocated).  A negative argument only queries.  Returns the previous
 * setting.  Process-wide.  No reference counterpart. */
int bt_set_gemm_dynamic_tiles(int enable);

/* ------------------------------------------------------ SwiGLU MLP (fused)  */

/* Forward of CuTileSwiGLUMLP (src/bastile/ops/swiglu.py:170-187):
 *   gate = x Wg^T, up = x Wu^T  (one tensor-core kernel, two accumulators),
 *   h = T(silu(gate)) * up fused in that kernel's epilogue,  y = h Wd^T.
 * x [T,H] (row stride ld_x), Wg/Wu [I,H], Wd [H,I] contiguous; gate, up, h
 * [T,I] and y [T,H] contiguous outputs (gate/up/h are what the backward needs).
 * `residual` [T,H] (row stride ld_residual, same dtype) may be NULL; otherwise
 * y = T(h Wd^T + residual): the `residual + hidden_states` that follows the MLP
 * in Qwen3DecoderLayer.forward (transformers modeling_qwen3.py:331-335) is added
 * to the fp32 accumulator in the down projection's epilogue. */
int bt_mlp_fwd(const void* x, const void* wg, const void* wu, const void* wd,
               void* gate, void* up, void* h, void* y,
               int64_t T, int64_t H, int64_t I, int64_t ld_x,
               const void* residual, int64_t ld_residual,
               int dtype, int32_t* status, void* stream);

/* Backward of the same block (autograd of src/bastile/ops/swiglu.py:186-187
 * plus swiglu_backward_kernel :53-90):
 *   dh = dy Wd (epilogue turns it into dgate, dup using saved gate/up),
 *   dWd = dy^T h, dWg = dgate^T x, dWu = dup^T x, dx = dgate Wg + dup Wu.
 * dgate/dup [T,I] are caller-owned scratch with row stride ld_dgate.  Any of
 * dx, dwg, dwu, dwd may be NULL to skip that product.  When dup starts I
 * elements after dgate in one [T, 2I] buffer (ld_dgate = 2I) and dwu starts
 * I*H elements after dwg, the two weight gradients are computed as ONE product
 * [dgate | dup]^T x. */
int bt_mlp_bwd(const void* dy, const void* x, const void* wg, const void* wu,
               const void* wd, const void* gate, const void* up, const void* h,
               void* dgate, void* dup, void* dx, void* dwg, void* dwu, void* dwd,
               int64_t T, int64_t H, int64_t I, int64_t ld_x, int64_t ld_dy,
               int64_t ld_dgate, int dtype, int32_t* status, void* stream);

/* ------------------------------------------- fused lm_head + cross-entropy  */

/* Step 1 of the fused loss for one chunk of rows and one vocabulary shard:
 * logits = hidden W^T on the tensor cores; the epilogue keeps, per row and per
 * 128-column block, (max, sum exp(logit-max)) and the target's logit, and writes
 * the logits once as 16-bit values into `logits` [rows, ld_logits] (the chunk
 * buffer, never [tokens, V]).  `tile_stats` has rows * bt_lce_num_vtiles(V)
 * float2 entries, `tgt_logit` one float per row (0 when the label is ignored or
 * outside [v_offset, v_offset+V)).  Replaces GEMM1 + pass 1 of
 * _ce_online_kernel + the target gather
 * (src/bastile/ops/fused_linear_cross_entropy.py:167, 46-100, 108-114). */
int bt_lce_logits_stats(const void* hidden, const void* W, const int64_t* labels,
                        void* logits, float* tile_stats, float* tgt_logit,
                        int64_t rows, int64_t H, int64_t V, int64_t ld_hidden,
                        int64_t ld_logits, int64_t v_offset, int64_t ignore_index,
                        int dtype, int32_t* status, void* stream);
int64_t bt_lce_num_vtiles(int64_t V);

/* Step 2: merge the per-tile statistics of each row into row_stats[rows,3] =
 * (max, sum exp, target logit) for this vocabulary shard
 * (the per-row reduction of _ce_online_kernel, :62-85). */
int bt_lce_row_stats(const float* tile_stats, const float* tgt_logit,
                     float* row_stats, int64_t rows, int64_t n_vtiles, void* stream);

/* Vocabulary-parallel form, between steps 2 and 3: shard_stats holds the row_stats of all
 * n_shards ranks as gathered by ONE collective (shard s at shard_stats + s * shard_stride floats,
 * [rows,3] each); row_stats[rows,3] receives their log-sum-exp merge - global max, sum exp
 * rescaled to it, and the target logit (non-zero on exactly one shard).  The reference has no
 * sharded loss; this is the exchange step of a vocabulary split of
 * src/bastile/ops/fused_linear_cross_entropy.py:46-100. */
int bt_lce_stats_combine(const float* shard_stats, float* row_stats, int64_t rows,
                         int64_t shard_stride, int n_shards, void* stream);

/* Step 3: given (possibly cross-shard merged) row statistics, write
 * loss_row = max + log(sum) - target (0 for ignored rows) and turn the logits
 * chunk in place into scaled gradients
 *   dlogits = (exp(logit - max)/sum - [col == label]) * grad_scale[0]
 * with ignored rows zeroed.  grad_scale is a DEVICE float (1/n_valid for mean,
 * 1 for sum).  write_loss = 0 skips the loss write.  Replaces pass 2 of
 * _ce_online_kernel and the torch fix-ups (:87-100, 126-130). */
int bt_lce_dlogits(void* logits, const float* row_stats, const int64_t* labels,
                   float* loss_row, const float* grad_scale,
                   int64_t rows, int64_t V, int64_t ld_logits, int64_t v_offset,
                   int64_t ignore_index, int write_loss, int dtype, void* stream);

/* Counts labels != ignore_index into n_valid[0] (fp32) and writes
 * grad_scale[0] = mean ? (n_valid > 0 ? 1/n_valid : 0) : 1 without a host
 * round trip (replaces the .item() sync of
 * src/bastile/ops/fused_linear_cross_entropy.py:334-343).  With vocab_size > 0 and a status
 * word, a label that is neither ignore_index nor inside [0, vocab_size) sets
 * BT_STATUS_BAD_LABEL in *status: the reference computes its loss with F.cross_entropy
 * (:127, :427), which asserts on such a label; here the row would silently count as valid with
 * no target term, so the caller is told instead (vocab_size is the FULL vocabulary when the
 * rows of lm_head are sharded over ranks). */
int bt_lce_count_valid(const int64_t* labels, int64_t n, int64_t ignore_index,
                       int mean, float* n_valid, float* grad_scale,
                       int64_t vocab_size, int32_t* status, void* stream);

/* loss[0] = sum(loss_row[0:n]) * (mean ? grad_scale[0] : 1)  (:333, 367). */
int bt_lce_reduce_loss(const float* loss_row, int64_t n, const float* grad_scale,
                       float* loss, void* stream);

/* out[i] = T(scale[0] * (float)in[i]) for i < n, `scale` a DEVICE float: the
 * dloss scaling of the saved gradients in the backward (:371-399). */
int bt_scale_cast(const void* in, void* out, int64_t n, const float* scale,
                  int in_dtype, int out_dtype, void* stream);

/* ------------------------------------------------------------------ AdamW  */

/* One AdamW step (decoupled weight decay, bias correction; the update rule of
 * torch.optim.AdamW) over a list of tensors that share one storage dtype for
 * parameter, gradient and both moments.  The four tables are HOST arrays of
 * n_tensors device pointers, `numel` a host array of element counts.  fp32
 * arithmetic, one rounding to the storage type.  `step` is the 1-based step
 * count used for the bias corrections.  The reference has no optimizer of its
 * own: its benchmark loop runs torch.optim.AdamW inside the timed region
 * (tests/benchmarks/e2e/qwen_8b_seqlen.py:122-125, 154-158); this is that step
 * as one streaming pass per tensor.  `ctas_per_sm` caps the resident CTAs per SM
 * of the large-tensor kernel (0 = default 16, which saturates HBM when the
 * kernel runs alone); a caller that runs the update on a side stream underneath
 * tensor-core work passes 1 or 2 so that the other stream's kernels still find
 * room on every SM. */
int bt_adamw_step(void* const* params, const void* const* grads,
                  void* const* exp_avg, void* const* exp_avg_sq,
                  const int64_t* numel, int n_tensors,
                  float lr, float beta1, float beta2, float eps, float weight_decay,
                  int64_t step, int ctas_per_sm, int dtype, void* stream);

/* The same step with fp32 MASTER weights, for one flat tensor: `master`, `exp_avg` and
 * `exp_avg_sq` are fp32 arrays of `numel` elements, `grad` holds the gradient in the model's
 * storage type `dtype`, and the updated parameter is written to `param_out` in that type for
 * the next forward pass ("bf16 parameters / fp32 master" of the reference's FSDP recipe,
 * tests/benchmarks/e2e/qwen_8b_fsdp.py:148-168, where FSDP mixed precision keeps fp32 shards
 * and hands bf16 copies to the layers).  The gradient is multiplied by `grad_scale` first
 * (1 / world size after a summing reduce-scatter, a clipping coefficient, ...).  A rank of
 * a sharded data-parallel job calls this on its slice of a flat bucket. */
int bt_adamw_master_step(float* master, float* exp_avg, float* exp_avg_sq,
                         const void* grad, void* param_out, int64_t numel,
                         float lr, float beta1, float beta2, float eps, float weight_decay,
                         int64_t step, float grad_scale, int ctas_per_sm, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BASTILE_B200_H_ */
