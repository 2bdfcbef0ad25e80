/*
 * mograd_b200 -- C ABI of the B200 (sm_100a) kernel library that replaces
 * mograd's Mojo kernel library (libmograd_gpu.so) on the training hot path.
 *
 * Conventions
 *   - every pointer is a DEVICE address unless its comment says "host";
 *     pointers already include any view offset, as AnyBuffer.data_ptr() does
 *     (mograd/buffer.mojo:62-67);
 *   - the callee never allocates and never frees: the caller passes outputs
 *     and, where a *_workspace_bytes query exists, a workspace of at least
 *     that many bytes (256-byte aligned), both from its own allocator
 *     (mograd/memory.mojo take_storage / scratch_take);
 *   - every call only enqueues work on `stream` (a cudaStream_t passed as
 *     void*; NULL = the legacy default stream) and returns; nothing
 *     synchronises the device;
 *   - return value 0 = enqueued; a negative MGB_E* code = nothing was
 *     launched and mograd_b200_last_error() (thread-local) says why.  The
 *     reference raises a Mojo Error in the same situations
 *     (mograd/runtime/gpu/kernels/dispatch.mojo:564-576 for dtypes);
 *   - dtype codes select the storage type of every tensor argument not
 *     documented otherwise.  bf16 runs the GEMMs and attention on the
 *     tcgen05 tensor cores with fp32 accumulation; f32 runs them on the
 *     CUDA cores in fp32.  Statistics, softmax and reductions are fp32 for
 *     both.
 */
#ifndef MOGRAD_B200_H_
#define MOGRAD_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOGRAD_B200_ABI_VERSION 1

enum mgb_status {
  MGB_OK = 0,
  MGB_EINVAL = -1,       /* null pointer, non-positive or inconsistent dims   */
  MGB_EDTYPE = -2,       /* dtype code not supported by this entry point      */
  MGB_EALIGN = -3,       /* pointer / leading dimension alignment not met     */
  MGB_EWORKSPACE = -4,   /* workspace missing or smaller than the query says  */
  MGB_ECUDA = -5,        /* a CUDA runtime / driver call reported an error    */
  MGB_EUNSUPPORTED = -6  /* valid request outside what the kernels implement  */
};

/* Storage types.  bfloat16 and float16 run on the tensor cores (fp32
 * accumulation); float32 runs on the CUDA cores.  float16 is the half type
 * mograd's buffers can carry today (mograd/buffer.mojo:136). */
enum mgb_dtype {
  MGB_BF16 = 0,
  MGB_F32 = 1,
  MGB_F16 = 2
};

/* Library identity.  No counterpart in the reference, whose Mojo ABI is
 * locked to the toolchain version instead (scripts/build_gpu.sh:46-48). */
int mograd_b200_abi_version(void);

/* Number of kernels this library has launched in this process so far (all
 * threads and devices).  No counterpart in the reference; its tracer counts
 * kernels per run in DebugStats (mograd/debug.mojo:23-46). */
unsigned long long mograd_b200_launch_count(void);

/* Message for the last negative status returned on this host thread. */
const char* mograd_b200_last_error(void);

/* Synchronises the device: reads (and clears) the status word the
 * tensor-core kernels write when one of their bounded waits on a TMA or MMA
 * barrier gives up (code 0 = none; 101 producer, 102 MMA issuer, 103 epilogue
 * of the GEMM; 2xx attention; 901 the self-test below).  A wait that gives up
 * is discovered on the GPU after the entry point has returned, so a 0 return
 * code of an entry point does NOT cover it: a host that wants that assurance
 * reads this word at a point where it synchronises anyway (the train-step
 * runner does so once per step) and must treat the outputs of the affected
 * step as garbage when the code is non-zero.  No counterpart in the
 * reference. */
int mograd_b200_device_status(int* code, int* detail);

/* The same word without a synchronisation of its own: enqueues a copy of the
 * status word (4 ints: code, detail, 2 reserved) into host_words (pinned
 * host memory) on `stream`; the caller looks at host_words[0] after its own
 * next synchronisation of that stream.  Does not clear the word: call
 * mograd_b200_device_status for that once a non-zero code has been seen. */
int mograd_b200_device_status_async(int* host_words, void* stream);

/* Self-test of the bounded waits: one warp waits up to limit_us microseconds
 * (1..100000) on a barrier that nothing completes, then records code 901 and
 * the microseconds it waited (detail) in the status word and returns; the
 * context stays usable.  No counterpart in the reference. */
int mograd_b200_selftest_wait_expiry(unsigned int limit_us, void* stream);

/* ------------------------------------------------------------------------
 * matmul_bias_bt:  Y[m,n] = sum_k A[m,k] * W[n,k] + bias[n]
 * Replaces mograd_matmul_bias_bt (mograd/runtime/gpu/kernels/__init__.mojo:
 * 758-840; signature MatmulBiasStrided, dispatch.mojo:247-257).  Batch dims
 * of A are collapsed into M by the caller, as the reference requires them to
 * be collapsible (__init__.mojo:775-776).  bias may be NULL (= the
 * reference's mograd_matmul_bt, __init__.mojo:688-755).  lda/ldw/ldy are row
 * strides in elements.  act: 0 = none, 1 = ReLU applied to Y before the
 * store (fuses the reference's separate mograd_relu launch).
 * bf16 fast path needs 16-byte aligned A/W and lda, ldw multiples of 8;
 * other bf16 shapes and all f32 calls take the CUDA-core kernel.
 * ---------------------------------------------------------------------- */
int mograd_b200_matmul_bias_bt(const void* a, const void* w, const void* bias, void* y, int64_t M, int64_t N,
                               int64_t K, int64_t lda, int64_t ldw, int64_t ldy, int act, int dtype,
                               void* stream);

/* ------------------------------------------------------------------------
 * Backward of matmul_bias_bt in one call (any of dx, dw, db may be NULL):
 *   dX[m,k] = sum_n dY[m,n] W[n,k];  dW[n,k] = sum_m dY[m,n] X[m,k];
 *   db[n] = sum_m dY[m,n].
 * Replaces the primitive chain the reference's rules build today:
 * matmul_grad (mograd/grad.mojo:180-183) + transpose_grad (:186-187) +
 * add_grad (:126-127) + expand_grad -> sum_axis (:278-288), which run on
 * mograd_matmul / mograd_matmul_bt (__init__.mojo:616-755) and mograd_sum.
 * dW and db are written in `dtype`.  db is produced inside the dW GEMM from
 * the dY tiles that pass through shared memory.
 * ---------------------------------------------------------------------- */
size_t mograd_b200_matmul_bias_bt_bwd_workspace_bytes(int64_t M, int64_t N, int64_t K, int dtype);
int mograd_b200_matmul_bias_bt_bwd(const void* dy, const void* x, const void* w, void* dx, void* dw, void* db,
                                   int64_t M, int64_t N, int64_t K, int64_t lddy, int64_t ldx, int64_t ldw,
                                   int64_t lddx, int64_t lddw, int dtype, void* workspace,
                                   size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------
 * LayerNorm forward over the last axis, biased variance:
 *   y = (x - mean) * rsqrt(var + eps) * gamma + beta
 * Replaces mograd_layer_norm_fwd (__init__.mojo:1309-1334; signature
 * LayerNormFwdKernel, dispatch.mojo:281-291).  mean / rstd (float32, one per
 * row) are optional extra outputs (NULL to skip); the reference saves none.
 * ---------------------------------------------------------------------- */
int mograd_b200_layer_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean,
                               float* rstd, int64_t rows, int64_t cols, float eps, int dtype, void* stream);

/* ------------------------------------------------------------------------
 * LayerNorm backward: dx (rows x cols), dgamma, dbeta (cols), mean / rstd
 * recomputed from x.  Replaces mograd_layer_norm_bwd (__init__.mojo:
 * 1337-1366; signature LayerNormBwdKernel, dispatch.mojo:317-329; kernels
 * mograd/runtime/gpu/kernels/normalization.mojo:85-400).  dgamma / dbeta are
 * plain stores: the caller need not zero them (the reference's dispatch
 * does, dispatch.mojo:343-344).  cols <= 16384, as in the reference.  dx may
 * alias dy (every row's dy is read before its dx is written).
 * ---------------------------------------------------------------------- */
size_t mograd_b200_layer_norm_bwd_workspace_bytes(int64_t rows, int64_t cols, int dtype);
int mograd_b200_layer_norm_bwd(const void* dy, const void* x, const void* gamma, void* dx, void* dgamma,
                               void* dbeta, int64_t rows, int64_t cols, float eps, int dtype, void* workspace,
                               size_t workspace_bytes, void* stream);

/* LayerNorm backward without a workspace argument.  It has no counterpart in
 * the reference.  It is for hosts that cannot hand the kernel a scratch
 * buffer because they are not allowed to allocate device memory at the point
 * of the call: a plugin running inside someone else's stream capture, a
 * runtime whose memory pool is frozen after start-up, or a callback that must
 * not re-enter the allocator.  The partial dgamma / dbeta rows go to an array
 * of 9.25 MiB that is part of the library image on every GPU that loads it.
 * On a B200 every shape with cols <= 4096 fits; wider rows fit only while
 * rows is small.  A request that needs more returns MGB_EUNSUPPORTED with the
 * sizes in the error text.  Inputs, outputs and results
 * are those of mograd_b200_layer_norm_bwd, bit for bit.
 *   - The first call on each device looks the array's address up (with that
 *     device current); make that first call outside any stream capture.
 *   - Neither this call nor anything it uses calls cudaMalloc / cudaFree.
 *   - All calls on a device share the one array.  Nothing in it has to be
 *     zero beforehand (every element that is read was written earlier in the
 *     same call), but two calls whose kernels overlap on the GPU (different
 *     streams, no dependency) race on it: keep them ordered. */
int mograd_b200_layer_norm_bwd_static(const void* dy, const void* x, const void* gamma, void* dx, void* dgamma,
                                      void* dbeta, int64_t rows, int64_t cols, float eps, int dtype, void* stream);

/* ------------------------------------------------------------------------
 * Cross-entropy with dense float labels of the logits' shape, mean over
 * rows; loss is one element of `dtype`.  Replaces mograd_cross_entropy /
 * _strided (__init__.mojo:1374-1454; kernels cross_entropy.mojo:14-77,
 * 155-177) without the reference's host synchronisation.  ldx / ldl are row
 * strides in elements (the reference's strided variant takes full Layouts;
 * row-strided views are what its callers produce).
 * ---------------------------------------------------------------------- */
size_t mograd_b200_cross_entropy_workspace_bytes(int64_t N, int64_t C, int dtype);
int mograd_b200_cross_entropy(const void* logits, const void* labels, void* loss, int64_t N, int64_t C,
                              int64_t ldx, int64_t ldl, int dtype, void* workspace, size_t workspace_bytes,
                              void* stream);

/* dst = (softmax(logits) - labels) * upstream[0] / N.  Replaces
 * mograd_cross_entropy_grad / _strided (__init__.mojo:1462-1528; kernel
 * cross_entropy.mojo:185-241; signature TernaryStrided, dispatch.mojo:
 * 545-554).  upstream is a one-element device tensor of `dtype`. */
int mograd_b200_cross_entropy_grad(const void* upstream, const void* logits, const void* labels, void* dst,
                                   int64_t N, int64_t C, int64_t ldx, int64_t ldl, int64_t lddst, int dtype,
                                   void* stream);

/* ------------------------------------------------------------------------
 * Fused softmax-cross-entropy forward + backward with one class index per
 * row (labels[r] in [0, C), int64): reads the logits once, writes
 *   loss (float32 scalar, mean over rows) and
 *   dlogits = (softmax - onehot) * upstream / N   (never materialising the
 * probabilities).  Same arithmetic as cross_entropy + cross_entropy_grad on
 * the one-hot labels the reference's train loop builds
 * (examples/tinyshakespear/train.mojo:38-41).  dlogits may alias logits.
 * dlogits == NULL computes the loss only; loss == NULL the gradient only.
 * ---------------------------------------------------------------------- */
size_t mograd_b200_softmax_xent_workspace_bytes(int64_t N, int64_t C, int dtype);
int mograd_b200_softmax_xent_fwd_bwd(const void* logits, const int64_t* labels, float* loss, void* dlogits,
                                     int64_t N, int64_t C, int64_t ldx, int64_t lddx, float upstream,
                                     int dtype, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------
 * Attention forward: O = softmax(scale * Q K^T [+ mask | causal]) V.
 * Q, K, V are BSHD (B,S,H,D); O is BHSD; lse is float32 (B,H,S), natural
 * log.  Replaces mograd_flash_attn_fwd (__init__.mojo:848-921; signature
 * FlashAttnFwdKernel, dispatch.mojo:361-377).  mask is an additive
 * (B,H,S,S) tensor of `dtype`, read only when has_bias != 0; causal and
 * has_bias together are rejected as in the reference (__init__.mojo:
 * 868-873).  1 <= D <= 512 (attention/dispatch.mojo:28-29).
 * bf16 or float16 with D in {64,128} (16-byte aligned tensors): tcgen05
 * kernels, with or without the additive mask (the mask tile is added to the
 * scores in registers before the exponentials, in the forward and in the
 * backward kernel, as the reference's fused half kernels do,
 * attention/nvidia_bwd.mojo:1061-1111); float32 and other head sizes:
 * CUDA-core kernels.
 * ---------------------------------------------------------------------- */
int mograd_b200_flash_attn_fwd(const void* q, const void* k, const void* v, const void* mask, void* dst,
                               float* lse, int64_t B, int64_t S, int64_t H, int64_t D, float scale, int causal,
                               int has_bias, int dtype, void* stream);

/* ------------------------------------------------------------------------
 * Attention backward: dQ, dK, dV (BSHD, `dtype`) from dO and O (BHSD),
 * Q, K, V (BSHD) and lse, recomputing the softmax tile by tile.  Replaces
 * mograd_flash_attn_bwd (__init__.mojo:924-1006; signature
 * FlashAttnBwdKernel, dispatch.mojo:418-438; kernels
 * attention/nvidia_bwd.mojo:784-1575).  The workspace holds
 * delta = rowsum(O * dO) and the float32 dQ accumulator.
 * ---------------------------------------------------------------------- */
size_t mograd_b200_flash_attn_bwd_workspace_bytes(int64_t B, int64_t S, int64_t H, int64_t D, int dtype);
int mograd_b200_flash_attn_bwd(const void* dy, const void* o, const void* q, const void* k, const void* v,
                               const void* mask, const float* lse, void* dq, void* dk, void* dv, int64_t B,
                               int64_t S, int64_t H, int64_t D, float scale, int causal, int has_bias,
                               int dtype, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------
 * Extended forms.  Same kernels and arithmetic as the entry points above with
 * extra operands that fold a neighbouring elementwise node of the reference's
 * graph into the kernel, or describe a non-default memory layout.  They have
 * no single counterpart in the reference: each note names the separate
 * reference launches it absorbs.  The plain entry points call these with the
 * extra operands NULL / default.
 * ---------------------------------------------------------------------- */

/* Y = act(A W^T + bias) + residual.  residual (M x N, row stride ldr, may be
 * NULL, may alias y) absorbs the mograd_add of a residual connection
 * (examples/tinyshakespear/model.mojo:64-66). */
int mograd_b200_matmul_bias_bt_ex(const void* a, const void* w, const void* bias, const void* residual, void* y,
                                  int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldr, int64_t ldy,
                                  int act, int dtype, void* stream);

/* dX = ((dY W) where relu_y > 0 else 0) + dx_residual.  relu_y (M x K: the
 * ReLU output that produced X, may be NULL) absorbs mograd_relu_grad
 * (mograd/grad.mojo:130-131); dx_residual (M x K, may be NULL, may alias dx)
 * absorbs the mograd_add that accumulates gradients reaching the same tensor
 * (accum, mograd/grad.mojo:93-95).  dW and db as in matmul_bias_bt_bwd. */
int mograd_b200_matmul_bias_bt_bwd_ex(const void* dy, const void* x, const void* w, const void* relu_y,
                                      const void* dx_residual, void* dx, void* dw, void* db, int64_t M, int64_t N,
                                      int64_t K, int64_t lddy, int64_t ldx, int64_t ldw, int64_t ld_relu_y,
                                      int64_t ld_dx_residual, int64_t lddx, int64_t lddw, int dtype, void* workspace,
                                      size_t workspace_bytes, void* stream);

/* The ReLU pair of a feed-forward block with the mask kept as one bit per element instead of re-reading the
 * activation (16x fewer bytes for the backward GEMM to fetch).  Forward: Y = relu(A W^T + bias) and
 * relu_bits[i][c / 32] bit (c % 32) = (Y[i][c] > 0); relu_bits is M rows of ld_bits uint32 words, ld_bits >=
 * ceil(N / 32).  Backward: as matmul_bias_bt_bwd_ex with the mask taken from relu_bits (M rows, one bit per column of
 * X, ld_bits >= ceil(K / 32)) instead of relu_y.  bf16 with 16-byte-aligned rows only (MGB_EUNSUPPORTED otherwise:
 * use relu_y).  Absorb mograd_relu / mograd_relu_grad (mograd/grad.mojo:130-131) like the _ex forms. */
int mograd_b200_matmul_bias_bt_relu_bits(const void* a, const void* w, const void* bias, void* y, void* relu_bits,
                                         int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldy,
                                         int64_t ld_bits, int dtype, void* stream);
int mograd_b200_matmul_bias_bt_bwd_relu_bits(const void* dy, const void* x, const void* w, const void* relu_bits,
                                             const void* dx_residual, void* dx, void* dw, void* db, int64_t M,
                                             int64_t N, int64_t K, int64_t lddy, int64_t ldx, int64_t ldw,
                                             int64_t ld_bits, int64_t ld_dx_residual, int64_t lddx, int64_t lddw,
                                             int dtype, void* workspace, size_t workspace_bytes, void* stream);

/* dx = layer_norm_bwd(...) + dx_residual (rows x cols, may be NULL, may alias
 * dx): absorbs the mograd_add of the residual branch's gradient. */
int mograd_b200_layer_norm_bwd_ex(const void* dy, const void* x, const void* gamma, const void* dx_residual, void* dx,
                                  void* dgamma, void* dbeta, int64_t rows, int64_t cols, float eps, int dtype,
                                  void* workspace, size_t workspace_bytes, void* stream);

/* Attention with explicit layouts.  ld_qkv / ld_dqkv: elements between
 * consecutive tokens of Q, K, V / dQ, dK, dV (H*D when each tensor is packed;
 * 3*H*D when they are the three column blocks of one fused projection
 * output).  o_layout: 0 = O and dO are BHSD as in the reference, 1 = BSHD,
 * which absorbs the reference's transpose(1,2)+contiguous copies around the
 * attention node (examples/tinyshakespear/model.mojo:100-108,
 * mograd/grad.mojo:336-339). */
int mograd_b200_flash_attn_fwd_ex(const void* q, const void* k, const void* v, const void* mask, void* dst, float* lse,
                                  int64_t B, int64_t S, int64_t H, int64_t D, float scale, int causal, int has_bias,
                                  int64_t ld_qkv, int o_layout, int dtype, void* stream);
int mograd_b200_flash_attn_bwd_ex(const void* dy, const void* o, const void* q, const void* k, const void* v,
                                  const void* mask, const float* lse, void* dq, void* dk, void* dv, int64_t B,
                                  int64_t S, int64_t H, int64_t D, float scale, int causal, int has_bias,
                                  int64_t ld_qkv, int64_t ld_dqkv, int o_layout, int dtype, void* workspace,
                                  size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------
 * Callers of the hot path inside a train step (elementwise, one pass each).
 * ---------------------------------------------------------------------- */

/* dx = dy where y > 0 else 0; y is the ReLU OUTPUT, as the reference's rule
 * passes it (relu_grad, mograd/grad.mojo:130-131; mograd_relu_grad,
 * __init__.mojo:546-560).  dx may alias dy. */
int mograd_b200_relu_grad(const void* y, const void* dy, void* dx, int64_t numel, int dtype, void* stream);

/* dst = a + b (residual connections and gradient accumulation; mograd_add,
 * mograd/runtime/gpu/kernels/elementwise.mojo).  dst may alias a or b. */
int mograd_b200_add(const void* a, const void* b, void* dst, int64_t numel, int dtype, void* stream);

/* out[t,:] = table[idx[t],:] (Embedding forward; mograd_gather,
 * mograd/runtime/gpu/kernels/gather_scatter.mojo:14-40).  idx is int64. */
int mograd_b200_gather_rows(const void* table, const int64_t* idx, void* out, int64_t rows, int64_t vocab, int64_t d,
                            int dtype, void* stream);

/* dtable[v,:] = sum_{t: idx[t]==v} dout[t,:] (Embedding backward;
 * mograd_scatter_add, gather_scatter.mojo:43-71).  Accumulates in fp32
 * (atomics; the summation order is not fixed), writes every row of dtable. */
size_t mograd_b200_scatter_add_rows_workspace_bytes(int64_t vocab, int64_t d, int dtype);
int mograd_b200_scatter_add_rows(const void* dout, const int64_t* idx, void* dtable, int64_t rows, int64_t vocab,
                                 int64_t d, int dtype, void* workspace, size_t workspace_bytes, void* stream);

/* One AdamW update with bias correction and decoupled weight decay, the
 * arithmetic of mograd/nn/optim/adam.mojo:6-58 in a single pass: m, v (and
 * the optional master copy of w) are float32, g is multiplied by grad_scale
 * first (1/world_size after a sum-allreduce), step counts from 1. */
int mograd_b200_adamw_step(void* w, const void* g, float* m, float* v, float* master, int64_t numel, float lr,
                           float beta1, float beta2, float eps, float weight_decay, int step, float grad_scale,
                           int dtype, void* stream);

/* The same update with the step number read from device memory, for callers
 * that replay a captured stream (a CUDA graph): a replay cannot carry a new
 * scalar argument, so the 1-based step lives in *step_dev.  advance != 0
 * first adds 1 to *step_dev on the stream (use it on the first range of a
 * step when the parameters are updated range by range). */
int mograd_b200_adamw_step_dev(void* w, const void* g, float* m, float* v, float* master, int64_t numel, float lr,
                               float beta1, float beta2, float eps, float weight_decay, int* step_dev, int advance,
                               float grad_scale, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOGRAD_B200_H_ */
