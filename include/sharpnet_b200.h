/*
 * sharpnet_b200 -- C ABI of the B200 (sm_100a) replacement for the fp32 matrix-multiply path of
 * SharpNet: Tensor.Dot, Tensor.BatchMatrixMultiplication and the Dense (Linear) layer forward /
 * backward with its bias and activation companions.
 *
 * Conventions shared by every entry point
 *   - every matrix is fp32, row-major and dense: the leading dimension equals the logical width,
 *     exactly as SharpNet's tensors are (Prod/Data/BlasServices.cs:17-19);
 *   - device pointers are owned by the caller, need only 4-byte alignment, and are never kept
 *     after the call returns.  The output never aliases an input; inputs may alias each other;
 *   - work is queued on the handle's stream (the legacy default stream unless snb200_set_stream
 *     was called) and the call returns without synchronising, like the cuBLAS/cuDNN calls it
 *     replaces (Prod/GPU/GpuTensor.cs:1196-1227);
 *   - the return value is 0 on success, otherwise one of the SNB200_STATUS_* codes, which reuse
 *     the numbering of cublasStatus_t (Prod/GPU/CublasWrapper.cs:8-20) so the caller's
 *     GPUWrapper.CheckStatus (Prod/GPU/GPUWrapper.cs:662-668) keeps printing meaningful names;
 *   - a handle is used by one host thread at a time; different handles are independent
 *     (one managed thread per device, Prod/GPU/GPUWrapper.cs:782-788,824-832);
 *   - there is no CPU fallback: without a CUDA device snb200_create fails.
 */
#ifndef SHARPNET_B200_H
#define SHARPNET_B200_H

#ifdef __cplusplus
extern "C" {
#endif

typedef struct snb200_context* snb200_handle_t;

enum {
  SNB200_STATUS_SUCCESS = 0,
  SNB200_STATUS_NOT_INITIALIZED = 1,
  SNB200_STATUS_ALLOC_FAILED = 3,
  SNB200_STATUS_INVALID_VALUE = 7,
  SNB200_STATUS_ARCH_MISMATCH = 8,
  SNB200_STATUS_EXECUTION_FAILED = 13,
  SNB200_STATUS_INTERNAL_ERROR = 14,
  SNB200_STATUS_NOT_SUPPORTED = 15
};

/* Arithmetic used by the tensor-core kernels.  SharpNet never sets a cuBLAS math mode
 * (classic fp32 SGEMM), so the default keeps fp32-level accuracy. */
enum {
  SNB200_MATH_3XTF32 = 0,    /* tcgen05 TF32 tensor cores, split fp32 = hi + lo, three products; default */
  SNB200_MATH_TF32 = 1,      /* single TF32 product: opt-in fast mode, ~1e-3 relative accuracy           */
  SNB200_MATH_FP32_SIMT = 2, /* fp32 FMA on the CUDA cores for every shape                               */
  /* opt-in: the hi * hi product in TF32 and both cross terms (a_lo * b_hi + a_hi * b_lo, 2^-11 of the result) as ONE
   * bf16 instruction over the concatenated K slices: two instruction times per slice instead of three, error about
   * 1.5x that of 3xTF32 and inside the same 1e-5 * sqrt(K) bound.  Implemented for Dot(a, false, b, true) shapes that
   * run on the CTA-pair kernel (both operands K-major); every other product runs 3xTF32. */
  SNB200_MATH_TF32_BF16X2 = 3
};

/* Activation selector: the values of cudnnActivationMode_t (Prod/GPU/CudnnWrapper.cs:267-281). */
enum {
  SNB200_ACT_SIGMOID = 0,
  SNB200_ACT_RELU = 1,
  SNB200_ACT_TANH = 2,
  /* min(max(x, 0), 1): the reference creates its cuDNN descriptors with coefficient 1.0 (Prod/GPU/GPUWrapper.cs:183) */
  SNB200_ACT_CLIPPED_RELU = 3,
  /* x >= 0 ? x : alpha * (exp(x) - 1), alpha from snb200_set_activation_parameter.  The reference itself always runs
   * ELU with alpha 1 (Prod/CPU/CpuTensor.cs:954,1000; the cuDNN descriptor of Prod/GPU/GPUWrapper.cs:183): a binding
   * sets 1.0 before an ELU call. */
  SNB200_ACT_ELU = 4,
  SNB200_ACT_IDENTITY = 5,
  SNB200_ACT_SWISH = 6,
  /* x >= 0 ? x : alpha * x, alpha from snb200_set_activation_parameter */
  SNB200_ACT_LEAKY_RELU = 1002,
  /* x <= 0 ? -100 : log(x); its gradient dy / x needs the input (Prod/CPU/CpuTensorActivationFunctions.cs:170-180) */
  SNB200_ACT_LN = 1004,
  /* snb200_dense_fwd only: y = softmax over every row of x * op(W) + bias, a Linear layer followed by an
   * ActivationLayer with CUDNN_ACTIVATION_SOFTMAX (Prod/GPU/GpuTensor.cs:411-413 -> cudnnSoftmaxForward): the output
   * layer of every classification network.  Its gradient enters through snb200_dense_bwd_from_loss. */
  SNB200_ACT_SOFTMAX = 1000
};

/* Losses whose gradient the library produces (Prod/Data/Tensor.cs:1182-1217): dy = scale * (yPredicted - yExpected)
 * with scale = 1/numClass, 1 and 2/numClass. */
enum { SNB200_LOSS_BINARY_CROSSENTROPY = 0, SNB200_LOSS_CATEGORICAL_CROSSENTROPY = 1, SNB200_LOSS_MSE = 2 };

/* Storage of the Dense weight matrix.
 * OUT_IN: W is [out_features, in_features], y = x * W^T   (Prod/Layers/Linear.cs:26-33,130).
 * IN_OUT: W is [in_features, out_features], y = x * W     (the Keras layout the golden network
 *         tests were produced with, Tests/NonReg/TestNetworkPropagation.cs:34,95). */
enum { SNB200_W_OUT_IN = 0, SNB200_W_IN_OUT = 1 };

/* ---- handle ---------------------------------------------------------------------------------
 * Replaces the per-device cuBLAS/cuDNN handles GPUWrapper creates and destroys
 * (Prod/GPU/GPUWrapper.cs:99-146,737-777; cublasCreate_v2/cublasDestroy_v2
 * Prod/GPU/CublasWrapper.cs:35-60).  The handle owns a small workspace (partial sums of the
 * column reductions, an error word); it never owns caller tensors. */
int snb200_create(snb200_handle_t* handle, int device_id);
int snb200_destroy(snb200_handle_t handle);
/* cudaStream_t passed as void*; NULL selects the legacy default stream (what SharpNet uses for
 * all cuBLAS/cuDNN work: it never calls cublasSetStream). */
int snb200_set_stream(snb200_handle_t handle, void* cuda_stream);
int snb200_set_math_mode(snb200_handle_t handle, int math_mode);
/* The coefficient of the parametric activations (ELU, LeakyRelu) for every call on this handle that follows: what
 * ActivationLayer hands to ActivationForward / ActivationBackward as activationParameter
 * (Prod/Layers/ActivationLayer.cs:21,36,66; Prod/CPU/CpuTensorActivationFunctions.cs:210-231).  0 by default. */
int snb200_set_activation_parameter(snb200_handle_t handle, float alpha);
int snb200_get_math_mode(snb200_handle_t handle, int* math_mode);
/* Text of the last error recorded on this handle (never NULL; empty when none). */
const char* snb200_last_error_string(snb200_handle_t handle);
/* Waits for the handle's stream and returns EXECUTION_FAILED if a kernel reported a
 * device-side pipeline time-out since the last check. */
int snb200_check_device_status(snb200_handle_t handle);
/* Runs the failure path of the tensor-core kernels on purpose, harmlessly (no counterpart in SharpNet): one small
 * kernel waits on a barrier that nothing signals, with a limit of limit_us microseconds (1 .. 100000) instead of
 * the kernels' two seconds, gives up, records the time-out in the handle's error word and returns normally.  The
 * next snb200_check_device_status reports EXECUTION_FAILED once; the handle and the context stay usable. */
int snb200_selftest_wait_timeout(snb200_handle_t handle, int limit_us);
/* Number of kernels this handle has launched so far, and the name of the kernel family chosen
 * by the last compute call ("umma_3xtf32", "umma_tf32", "simt", "skinny", ...). */
int snb200_get_launch_count(snb200_handle_t handle, long long* count);
int snb200_get_last_kernel(snb200_handle_t handle, char* buf, int buf_len);
int snb200_get_version(void);
/* Device time of the matrix products (no counterpart in SharpNet; the role of a profiler range).
 * Between _begin and _end the handle records a CUDA-event pair on its stream around every matrix
 * product it launches -- the Dot / batched entry points and the products inside the Dense and attention
 * entry points, with their reduction pass when K is cut -- at most 4096 of them.  _end waits for the
 * stream and returns the sum of the pairs' elapsed times and the number of products timed. */
int snb200_gemm_timing_begin(snb200_handle_t handle);
int snb200_gemm_timing_end(snb200_handle_t handle, double* total_ms, int* gemm_calls);
/* Kernel-selection overrides for experiments and tests (no counterpart in SharpNet).
 * key 3: K extent accumulated inside the tensor core before the sum moves to registers (3xTF32; default 128,
 *        0 = whole K); key 4: CTA-pair kernel (0 automatic, 1 always, 2 never); key 5: split-K and
 *        swapped-operand plans for problems with few tiles (0 automatic, 1 never); key 6: 1 selects the
 *        16-wide K blocks in 3xTF32 mode instead of the default 32-wide ones (A/B measurements).
 * key 0: path (0 automatic, 1 tensor cores whenever the operands allow TMA, 2 SIMT fp32);
 * key 1: tile width of the tensor-core kernel (0 automatic, else 32, 64, 128, 256, or 192 on the CTA-pair kernel);
 * key 2: 3xTF32 writes the rounded hi plane back to shared memory (1) or lets the
 *        tensor core truncate the raw fp32 words itself (0, default);
 * key 7: 1 launches the tensor-core kernels without programmatic dependent launch (by default their set-up
 *        overlaps the tail of the previous kernel in the stream; they wait for its completion before touching
 *        global memory);
 * key 8: n > 1 cuts K of the tiles of a partly filled last wave exactly n times (one of 2..8, 10, 12, 16),
 *        whatever the time estimate says (tests of the reduction pass);
 * key 9: 1 keeps the A operand of the single-CTA 3xTF32 kernel in shared memory instead of tensor memory
 *        (A/B measurements);
 * key 10: 1 runs the attention core as separate products instead of the single fused kernel;
 * key 11: 1 sends operands that TMA cannot load to the SIMT kernel instead of the tensor-core kernel with
 *         loader warps;
 * key 12: n keeps n SMs out of the persistent tensor-core grids launched from now on (0 = use all): a host that
 *         has just queued a collective on another stream sets it for the next product, so that the collective's
 *         CTAs find free SMs instead of displacing CTAs of a grid that counts on every SM;
 * key 13: K cut inside thread-block clusters, summed through distributed shared memory, for problems whose tiles
 *         leave SMs idle (0 automatic, 1 never, 2 or 4: always, in clusters of that size). */
int snb200_set_tuning(snb200_handle_t handle, int key, int value);

/* ---- Tensor.Dot -----------------------------------------------------------------------------
 * C = alpha * op(A) * op(B) + beta * C.
 * Replaces cublasSgemm_v2 as called by GPUTensor.Dot (Prod/GPU/GpuTensor.cs:1196-1227,
 * Prod/GPU/CublasWrapper.cs:105-122) and takes the argument list of BlasServices.DotMkl
 * (Prod/Data/BlasServices.cs:10-21): A is stored [aH x aW], B is stored [bH x bW],
 * M = transA ? aW : aH, N = transB ? bH : bW, K = transA ? aH : aW, and C is [M x N].
 * INVALID_VALUE when the inner dimensions disagree or a dimension is negative. */
int snb200_gemm(snb200_handle_t handle, int transA, int transB, int aH, int aW, int bH, int bW, float alpha,
                const float* A, const float* B, float beta, float* C);

/* ---- Tensor.BatchMatrixMultiplication -------------------------------------------------------
 * C[i] = alpha * op(A[i]) * op(B[i]) + beta * C[i] for i in [0, batchCount).
 * Replaces cublasSgemmStridedBatched as called by GPUTensor.BatchMatrixMultiplication
 * (Prod/GPU/GpuTensor.cs:1163-1194); strides are element counts between consecutive matrices
 * (MultDim0 of the 3-D tensors). */
int snb200_batched_gemm(snb200_handle_t handle, int transA, int transB, int aH, int aW, long long strideA, int bH,
                        int bW, long long strideB, long long strideC, int batchCount, float alpha, const float* A,
                        const float* B, float beta, float* C);

/* ---- Dense forward --------------------------------------------------------------------------
 * y = act(x * op(W) + bias), x [M x K], y [M x N], bias [N] or NULL: the bias, the activation and the
 * optional pre-activation copy are applied where the product is stored (the GEMM epilogue, or the
 * reduction pass when K is cut), never in a pass of their own.
 * Replaces Linear.DenseForwardPropagation (Prod/Layers/Linear.cs:125-132: Dot, then
 * BroadcastAddVectorToOutput -> cudnnAddTensor, Prod/GPU/GpuTensor.cs:633-644) followed by
 * ActivationLayer.ForwardPropagation (Prod/Layers/ActivationLayer.cs:32-38 ->
 * cudnnActivationForward, Prod/GPU/GpuTensor.cs:438-442).
 * z, when not NULL, receives the pre-activation x*op(W)+bias, which ActivationLayer keeps for the
 * Swish gradient (Prod/Layers/ActivationLayer.cs:73). */
int snb200_dense_fwd(snb200_handle_t handle, int w_layout, int M, int K, int N, const float* x, const float* W,
                     const float* bias, int act, float* z, float* y);

/* ---- Dense backward -------------------------------------------------------------------------
 * dz = act'(.) * dy ; dW = dW_multiplier * (dz, x) product in the layout of W ; db = column sums
 * of dz ; dx = dz * op(W)^T.
 * Replaces ActivationLayer.BackwardPropagation (Prod/Layers/ActivationLayer.cs:39-69 ->
 * cudnnActivationBackward, Prod/GPU/GpuTensor.cs:484-488) followed by
 * Linear.DenseBackwardPropagation (Prod/Layers/Linear.cs:142-191: Dot for dW with
 * multiplier = 1/batch or 1, Compute_BiasGradient_from_dy -> cudnnConvolutionBackwardBias
 * Prod/GPU/GpuTensor.cs:686-701, Dot for dx).
 * y is the activation output (needed unless act is IDENTITY), z the pre-activation (needed for
 * SWISH only).  dz_scratch is a caller-provided [M x N] buffer (the ActivationLayer's dx in
 * SharpNet); it may be NULL when act is IDENTITY.  dx may be NULL (previous layer is the input,
 * Linear.cs:184-187); db may be NULL (layer without bias).  dW may be NULL as well: the call then skips
 * the weight-gradient product, so a host that overlaps the gradient sum of several replicas with the
 * backward pass can run the two products of a layer as two calls (dW and db first, start their
 * all-reduce, then a second call with act = IDENTITY on the dz it already holds for dx alone), or
 * leave the smallest weight gradient for the very end of the step.  At least one output is required. */
int snb200_dense_bwd(snb200_handle_t handle, int w_layout, int M, int K, int N, const float* x, const float* W,
                     const float* dy, int act, const float* y, const float* z, float dW_multiplier,
                     float* dz_scratch, float* dx, float* dW, float* db);
/* Rows [row0, row0 + rows) of the same weight gradient (in the layout of W: rows are output features for
 * SNB200_W_OUT_IN, input features for SNB200_W_IN_OUT) from the layer's input x [M x K] and dz [M x N], the
 * gradient with respect to the pre-activation that snb200_dense_bwd leaves in dz_scratch (dy itself for an identity
 * layer): the product of Linear.cs:158 restricted to a panel of its result.  For hosts that sum gradients across
 * replicas (Prod/Networks/NetworkMultiGPUSupport.cs:161-173): the reduction of one panel runs while the next is
 * computed.  row0 must be a multiple of 4 for the tensor-core path. */
int snb200_dense_bwd_weight_rows(snb200_handle_t handle, int w_layout, int M, int K, int N, const float* x,
                                 const float* dz, float dW_multiplier, int row0, int rows, float* dW);

/* ---- loss gradient, alone and fused into the last Dense layer's backward ------------------------
 * dy = scale * (yPredicted - yExpected), [rows x cols].  Replaces
 * Tensor.ComputeGradientForEvaluationMetric for BinaryCrossentropy, CategoricalCrossentropy and Mse
 * (Prod/Data/Tensor.cs:1182-1217 -> :1379-1395 copy + cudnnAddTensor, and the MseGradient NVRTC kernel
 * Prod/GPU/Kernels/SinglePrecision.cu:1008-1020; CPU Prod/CPU/CpuTensor.cs:2458-2475). */
int snb200_loss_gradient(snb200_handle_t handle, int loss, int rows, int cols, const float* yExpected,
                         const float* yPredicted, float* dy);
/* Backward of the output Dense layer straight from the labels: one pass computes
 * dz = scale * (yPredicted - yExpected) into dz_scratch together with db (its column sums), then dW and dx as in
 * snb200_dense_bwd.  This folds three passes of SharpNet over the [M x N] output -- the loss gradient
 * (Tensor.cs:1182-1217), the output ActivationLayer's dy.CopyTo(dx) shortcut
 * (Prod/Layers/ActivationLayer.cs:60-63) and Compute_BiasGradient_from_dy (Prod/Layers/Linear.cs:160-165) --
 * into one. */
int snb200_dense_bwd_from_loss(snb200_handle_t handle, int w_layout, int M, int K, int N, const float* x,
                               const float* W, int loss, const float* yExpected, const float* yPredicted,
                               float dW_multiplier, float* dz_scratch, float* dx, float* dW, float* db);

/* ---- Dense companions, callable on their own ------------------------------------------------ */
/* y[m,n] += bias[n].  Tensor.BroadcastAddVectorToOutput (Prod/Data/Tensor.cs:495,
 * Prod/GPU/GpuTensor.cs:633-644, Prod/CPU/CpuTensor.cs:1468-1487). */
int snb200_bias_add(snb200_handle_t handle, int M, int N, const float* bias, float* y);
/* db[n] = sum_m dy[m,n].  Tensor.Compute_BiasGradient_from_dy (Prod/Data/Tensor.cs:710,
 * Prod/GPU/GpuTensor.cs:686-701, Prod/CPU/CpuTensor.cs:1736-1740,3343-3362). */
int snb200_bias_grad(snb200_handle_t handle, int M, int N, const float* dy, float* db);
/* db[n] = sum_m dy[m,n] without a handle and without any allocation.  It has no counterpart in
 * SharpNet.  It exists for hosts that cannot call cudaMalloc once they are running -- an engine
 * whose own pool already holds all of the device memory (a later cudaMalloc fails), or a
 * latency-critical loop that cannot take the device-wide synchronisation cudaMalloc / cudaFree
 * imply -- and that therefore cannot create a handle either (snb200_create allocates a workspace).
 * The slab partial sums of the reduction live in a fixed 1 MiB array inside the library's device
 * image (held by every GPU that loads the library until the process exits), which limits the
 * matrix to SNB200_NOALLOC_MAX_COLUMNS columns; wider matrices are refused with NOT_SUPPORTED and
 * a message.  The device address of that array is looked up on the first call on each device, so
 * make that first call before starting any stream capture -- and before the host's pool takes the
 * device memory: with CUDA's default lazy module loading that first call is also what loads the
 * library's device image (the array and the kernels) onto the device, the one moment that needs free
 * device memory (ALLOC_FAILED otherwise; CUDA_MODULE_LOADING=EAGER moves the load to start-up).  All calls on a device share the
 * array: calls queued on one stream are safe, calls that overlap on the GPU race.  Nothing needs
 * clearing between calls (every word read back is written first by the same call).
 * cuda_stream is a cudaStream_t (NULL = legacy default stream); err, when not NULL, receives the
 * text of a refusal or failure. */
#define SNB200_NOALLOC_MAX_COLUMNS 65536
int snb200_bias_grad_noalloc(int device_id, void* cuda_stream, int M, int N, const float* dy, float* db, char* err,
                             int err_len);
/* y = act(x) element-wise.  Tensor.ActivationForward (Prod/Data/Tensor.cs:618,
 * Prod/GPU/GpuTensor.cs:397-443, Prod/CPU/CpuTensorActivationFunctions.cs:152-244). */
int snb200_activation_fwd(snb200_handle_t handle, int act, long long count, const float* x, float* y);
/* dx = act'(x, y) * dy element-wise.  Tensor.ActivationBackward (Prod/Data/Tensor.cs:628,
 * Prod/GPU/GpuTensor.cs:445-490).  x is read for SWISH only and may be NULL otherwise. */
int snb200_activation_bwd(snb200_handle_t handle, int act, long long count, const float* dy, const float* x,
                          const float* y, float* dx);
/* y += alpha * x.  Tensor.Update_Adding_Alpha_X (Prod/Data/Tensor.cs:555,
 * Prod/GPU/GpuTensor.cs:1359-1362); used for weight decay on dW (Prod/Layers/Linear.cs:176). */
int snb200_axpy(snb200_handle_t handle, long long count, float alpha, const float* x, float* y);

/* ---- attention around BatchMatrixMultiplication ------------------------------------------------
 * Row softmax over the last dimension and its gradient.  Replace Tensor.ActivationForward /
 * ActivationBackward with CUDNN_ACTIVATION_SOFTMAX_LAST_DIMENSION (Prod/GPU/GpuTensor.cs:397-443 ->
 * cudnnSoftmaxForward, :445-490 -> cudnnSoftmaxBackward; CPU forward
 * Prod/CPU/CpuTensorActivationFunctions.cs:14-46).  The gradient is the softmax Jacobian
 * dx = y * (dy - sum(dy * y)), what the GPU path of SharpNet computes; x may equal y, dy may equal dx. */
int snb200_softmax_fwd(snb200_handle_t handle, long long rows, int cols, const float* x, float* y);
int snb200_softmax_bwd(snb200_handle_t handle, long long rows, int cols, const float* dy, const float* y, float* dx);
/* Scaled dot-product attention, Q [batch, q_steps, E], K and V [batch, v_steps, E], y [batch, q_steps, E]:
 * weights = softmax(mask(scaling * Q K^T)), y = weights V, scaling = use_scale ? 1/sqrt(E) : 1.
 * Replaces ScaledDotProductAttentionLayer.ScaledDotProductAttentionForwardPropagation
 * (Prod/Layers/ScaledDotProductAttentionLayer.cs:46-91): two strided-batched GEMMs with, between them, the
 * causal overwrite (SetAllElementsAboveMainDiagonal, -1e12) and the softmax applied where the scores are stored
 * (v_steps <= 256) or as ONE in-place pass over
 * `weights` [batch, q_steps, v_steps] (caller-provided; the layer's _weights_buffer, kept for the backward).
 * The separate scores buffer of the reference is not needed. */
int snb200_sdpa_fwd(snb200_handle_t handle, int batch, int q_steps, int v_steps, int embedding_dim, int use_scale,
                    int is_causal, const float* Q, const float* K, const float* V, float* weights, float* y);
/* Replaces ScaledDotProductAttentionBackwardPropagation (ScaledDotProductAttentionLayer.cs:108-129):
 * dV = weights^T dy; dScores = softmax'(scaling * dy V^T) in place in scores_grad_scratch
 * [batch, q_steps, v_steps] (caller-provided; the reference takes it from its memory pool);
 * dQ = dScores K; dK = dScores^T Q. */
int snb200_sdpa_bwd(snb200_handle_t handle, int batch, int q_steps, int v_steps, int embedding_dim, int use_scale,
                    const float* Q, const float* K, const float* V, const float* dy, const float* weights,
                    float* scores_grad_scratch, float* dQ, float* dK, float* dV);

/* ---- multi-head attention ------------------------------------------------------------------------
 * MultiheadAttention.ForwardPropagation / BackwardPropagation (Prod/Layers/MultiheadAttention.cs:178-295) as one
 * call each: the Dense projections of Q, K, V on the last dimension (Linear.DenseForwardPropagation), the head
 * split [b, t, h, d] -> [b, h, t, d] (TransposeSecondAndThirdDimension), scaled dot-product attention per head
 * (use_scale is always on, :32), the head merge and the output projection; the backward pass in the reverse order.
 * The permutations are not passes of their own: the product before each one stores its result already permuted.
 * The kernels of one call are queued back to back on the handle's stream, nothing is allocated.
 *   Q [batch, q_steps, embed_dim]; K, V [batch, v_steps, embed_dim]; y [batch, q_steps, embed_dim];
 *   embed_dim must equal num_heads * value_dim (the layer uses out_proj_weight that way, :121-126,236), and
 *   key_dim must equal value_dim (NOT_SUPPORTED otherwise): the layer's attention core multiplies Q by K^T over
 *   key_dim and takes V with the same embedding width (ScaledDotProductAttentionLayer.cs:56-60).
 * Weights are [out, in] rows (w_layout 0, Linear.cs:125-132) or [in, out] (w_layout 1); biases may be NULL.
 * snb200_mha_state holds what the layer keeps between the two passes (Q_heads_T, K_heads_T, V_heads_T,
 * attention_heads_T, weights_buffer; :73-77), caller-provided:
 *   Q_heads_T [batch*num_heads, q_steps, key_dim], K_heads_T [batch*num_heads, v_steps, key_dim],
 *   V_heads_T [batch*num_heads, v_steps, value_dim], attention_heads_T [batch, q_steps, num_heads*value_dim],
 *   weights_buffer [batch*num_heads, q_steps, v_steps].
 * `scratch` is caller-provided device memory of at least snb200_mha_scratch_floats(desc, backward) floats, 256-byte
 * aligned: nothing for the forward pass (0; scratch may be NULL), and for the backward pass the layer's
 * d_attention_heads, the gradients of the three projections' outputs and the gradient of the scores. */
typedef struct snb200_mha_desc {
  int w_layout, batch, q_steps, v_steps, embed_dim, num_heads, key_dim, value_dim, is_causal;
} snb200_mha_desc;
typedef struct snb200_mha_weights {
  const float *w_Q, *w_K, *w_V, *out_proj_weight;
  const float *w_Q_bias, *w_K_bias, *w_V_bias, *out_proj_bias;
} snb200_mha_weights;
typedef struct snb200_mha_state {
  float *Q_heads_T, *K_heads_T, *V_heads_T, *attention_heads_T, *weights_buffer;
} snb200_mha_state;
typedef struct snb200_mha_gradients {
  float *w_Q, *w_K, *w_V, *out_proj_weight;
  float *w_Q_bias, *w_K_bias, *w_V_bias, *out_proj_bias;      /* NULL where the layer has no bias */
} snb200_mha_gradients;
long long snb200_mha_scratch_floats(const snb200_mha_desc* desc, int backward);
int snb200_mha_fwd(snb200_handle_t handle, const snb200_mha_desc* desc, const snb200_mha_weights* weights,
                   const float* Q, const float* K, const float* V, const snb200_mha_state* state, float* scratch,
                   float* y);
/* dW_multiplier is the factor of the weight gradients (Linear.cs:152-158). */
int snb200_mha_bwd(snb200_handle_t handle, const snb200_mha_desc* desc, const snb200_mha_weights* weights,
                   const float* Q, const float* K, const float* V, const float* dy, const snb200_mha_state* state,
                   float dW_multiplier, float* scratch, const snb200_mha_gradients* gradients, float* dQ, float* dK,
                   float* dV);


/* dst[a, c, b, :] = src[a, b, c, :] for a dense src of shape [A, B, C, D] (D = product of the trailing
 * dimensions): Tensor.TransposeSecondAndThirdDimension (Prod/Data/Tensor.cs, GPU Prod/GPU/GpuTensor.cs:672-684,
 * CPU Prod/CPU/CpuTensor.cs:301-322), the head split and merge of MultiheadAttention
 * (Prod/Layers/MultiheadAttention.cs:209-236).  src and dst must not overlap. */
int snb200_transpose_second_third(snb200_handle_t handle, int A, int B, int C, int D, const float* src, float* dst);

/* ---- optimizer updates (the step right after the path in every training iteration) -----------
 * One kernel, one pass over the tensors.
 * SGD:  velocity = momentum * velocity - learning_rate * dW ;
 *       W += nesterov ? momentum * velocity - learning_rate * dW : velocity.
 * Replaces Tensor.UpdateSGDOptimizer (Prod/GPU/GpuTensor.cs:1147-1161: cudnnAddTensor + one or two
 * axpy passes; Prod/CPU/CpuTensor.cs:470-489) as called by Sgd.UpdateWeights
 * (Prod/Optimizers/Sgd.cs:43-52).  velocity == NULL gives W -= learning_rate * dW, the VanillaSgd
 * update (Prod/Optimizers/VanillaSgd.cs:12-21).  learning_rate is the already "pondered" rate
 * lr / batchSize (Prod/Optimizers/Optimizer.cs:26-29). */
int snb200_sgd_update(snb200_handle_t handle, long long count, float learning_rate, float momentum, int nesterov,
                      const float* dW, float* W, float* velocity);
/* Adam / AdamW:  v = beta1 v + (1 - beta1) dW ; s = beta2 s + (1 - beta2) dW^2 ;
 *       W -= lr * sqrt(1 - beta2^t) / (1 - beta1^t) * v / (sqrt(s) + epsilon) + weight_decay * W.
 * Replaces Tensor.UpdateAdamOptimizer (Prod/GPU/GpuTensor.cs:1136-1145 -> NVRTC kernel
 * Prod/GPU/Kernels/SinglePrecision.cu:19-28; Prod/CPU/CpuTensor.cs:1755-1769) as called by
 * Adam.UpdateWeights (Prod/Optimizers/Adam.cs:59-72); weight_decay is the pondered decay of :67. */
int snb200_adam_update(snb200_handle_t handle, long long count, double learning_rate, double beta1, double beta2,
                       double epsilon, double weight_decay, int time_step, const float* dW, float* W, float* adam_vW,
                       float* adam_sW);

/* ---- data-parallel gradient sum -------------------------------------------------------------
 * Sum of the per-replica dW/db buffers, left on every replica.  Replaces the
 * copy-to-master-and-add loop of Network.AddGradientFromSlaveNetwork
 * (Prod/Networks/NetworkMultiGPUSupport.cs:161-173: cudaMemcpyPeerAsync + cudnnAddTensor) by one
 * NCCL all-reduce over NVLink.  NCCL is loaded at run time (libnccl.so.2); without it these
 * calls return NOT_SUPPORTED and nothing else in the library is affected.
 *   one process per GPU:  rank 0 calls snb200_comm_get_unique_id, ships the 128 bytes to the
 *                         other ranks, every rank calls snb200_comm_init_rank;
 *   one thread per GPU :  snb200_comm_init_all on the array of handles (SharpNet's threading
 *                         model, Prod/Networks/Network.cs:71-83). */
int snb200_comm_get_unique_id(void* id_128_bytes);
int snb200_comm_init_rank(snb200_handle_t handle, int n_ranks, int rank, const void* id_128_bytes);
int snb200_comm_init_all(snb200_handle_t* handles, int n);
int snb200_allreduce_sum(snb200_handle_t handle, float* buf, long long count);
/* The same for n buffers at once (a layer's dW and db): one NCCL group, hence one collective launch, instead of
 * one launch per buffer -- for the small bias gradients the launch is all the cost. */
int snb200_allreduce_sum_group(snb200_handle_t handle, int n, float* const* bufs, const long long* counts);
int snb200_comm_destroy(snb200_handle_t handle);

/* ---- mini-batch staging ------------------------------------------------------------------------
 * The step before the path: SharpNet copies every mini-batch from pinned host memory to the device on its one
 * stream before it runs the step (Prod/Networks/Network.cs:1211-1258: x_miniBatch_cpu.CopyTo(x_miniBatch);
 * Prod/GPU/GpuTensor.cs:68-80 InitializeFromHostPinnedMemory -> cuMemcpyHtoDAsync_v2; pinning:
 * Prod/CPU/HostPinnedMemory.cs).  A stager runs those copies on a stream of its own, `slots`-fold buffered, so
 * that the copy of mini-batch i+1 overlaps the step on mini-batch i.  Device buffers and host memory belong to
 * the caller (one set of device buffers per slot).  Per step i, with s = i % slots:
 *   snb200_stager_issue(st, s, ...)   queue the host->device copies of that step's inputs into slot s; the copy
 *                                     stream first waits until the step that last read slot s has finished;
 *   snb200_stager_acquire(st, s)      the handle's stream waits for those copies (no host synchronisation);
 *   ... the step's compute calls on the handle, reading the slot's device buffers ...
 *   snb200_stager_release(st, s)      marks on the handle's stream where the slot's last reader ends.
 * Issue step i+1 before computing step i to get the overlap.  Copies are queued one cudaMemcpyAsync per pair. */
typedef struct snb200_stager* snb200_stager_t;
int snb200_stager_create(snb200_handle_t handle, int slots, snb200_stager_t* stager);
int snb200_stager_destroy(snb200_stager_t stager);
int snb200_stager_issue(snb200_stager_t stager, int slot, int n_copies, void* const* device_dst,
                        const void* const* host_src, const long long* bytes);
int snb200_stager_acquire(snb200_stager_t stager, int slot);
/* The same for ONE copy of the slot's last issue (the first 16 copies of an issue have an event of their own): the
 * handle's stream waits only for copies 0 .. part, so that work on the first rows of a mini-batch staged as several
 * row panels starts while the later panels are still on their way. */
int snb200_stager_acquire_part(snb200_stager_t stager, int slot, int part);
int snb200_stager_release(snb200_stager_t stager, int slot);
/* Page-locks / unlocks caller-owned host memory so that the copies above run asynchronously at full speed: what
 * HostPinnedMemory does for a managed array (Prod/CPU/HostPinnedMemory.cs:17-21; there the GC pin, here the CUDA
 * registration the async copy needs). */
int snb200_host_pin(void* host_ptr, long long bytes);
int snb200_host_unpin(void* host_ptr);

#ifdef __cplusplus
}
#endif
#endif /* SHARPNET_B200_H */
