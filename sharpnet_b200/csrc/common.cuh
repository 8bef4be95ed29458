// Types shared by the SIMT and tcgen05 GEMM kernels: the problem description and the fused
// epilogue  v = alpha*acc + beta*C + bias ; z = v ; C = act(v).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace snb {

// Programmatic dependent launch.  A kernel launched with the programmatic-stream-serialization attribute may
// start while the kernel before it in the stream is still running; grid_dependency_wait() returns once that
// kernel has completed and its memory operations are visible, and must come before the first access to global
// memory.  allow_dependent_launch() lets the next such kernel be scheduled as soon as every CTA of this grid
// has started; it does not weaken what that kernel's own wait guarantees.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void allow_dependent_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// First statement of every kernel of this library: let the next kernel of the stream be scheduled early, and wait
// for the previous one before touching global memory.  Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_prologue() {
  allow_dependent_launch();
  grid_dependency_wait();
}

// Values of cudnnActivationMode_t (Prod/GPU/CudnnWrapper.cs:267-281).
// ELU and LEAKY_RELU take a coefficient (the layer's activationParameter); it travels beside the code as act_alpha.
enum Act : int { ACT_SIGMOID = 0, ACT_RELU = 1, ACT_TANH = 2, ACT_CLIPPED_RELU = 3, ACT_ELU = 4, ACT_IDENTITY = 5, ACT_SWISH = 6, ACT_LEAKY_RELU = 1002, ACT_LN = 1004 };
// The reference builds every cuDNN activation descriptor with coefficient 1.0 (Prod/GPU/GPUWrapper.cs:183):
// its ClippedRelu is min(max(x, 0), 1).
#define SNB_CLIPPED_RELU_CEILING 1.0f
__host__ __device__ __forceinline__ bool act_needs_input(int act) { return act == ACT_SWISH || act == ACT_ELU || act == ACT_LN; }   // ActivationLayer.cs:73
// Internal selector of the fused column-sum pass: dz = scale * (yPredicted - yExpected), the gradient of
// the BinaryCrossentropy / CategoricalCrossentropy / Mse losses (Prod/Data/Tensor.cs:1379-1395,
// Prod/CPU/CpuTensor.cs:2458-2475).
constexpr int ACT_LOSS_DIFF = 100;

// Optional placement of the result: element (matrix i, row r, column c) of the logical [batch, M, N] result goes to
//   (i / H) * s_io + (i % H) * s_ii + (r / T) * s_ro + (r % T) * s_ri + (c / d) * s_co + (c % d).
// It lets a product store its result already permuted -- the head split [b, t, h, d] -> [b, h, t, d] of
// multi-head attention and its inverse -- instead of a separate pass.  `on` = 0: the plain dense layout
// i * strideC + r * ldc + c.  When on, d and every stride are multiples of 4 (whole float4s stay together).
struct OutMap {
  int on;
  int H, T, d;
  long long s_io, s_ii, s_ro, s_ri, s_co;
};
__host__ __device__ __forceinline__ long long out_offset(const OutMap& m, int i, int r, int c) {
  return static_cast<long long>(i / m.H) * m.s_io + static_cast<long long>(i % m.H) * m.s_ii +
         static_cast<long long>(r / m.T) * m.s_ro + static_cast<long long>(r % m.T) * m.s_ri +
         static_cast<long long>(c / m.d) * m.s_co + (c % m.d);
}

// One (possibly strided-batched) GEMM  C[b] = epi(alpha * op(A[b]) * op(B[b]) + beta * C[b]).
// All matrices are dense row-major fp32.
struct GemmProblem {
  int M, N, K;            // logical dims of op(A) [M x K], op(B) [K x N], C [M x N]
  int transA, transB;     // A stored [K x M] when transA, B stored [N x K] when transB
  int lda, ldb, ldc;      // row pitch (elements) of the stored matrices
  int batch;
  long long strideA, strideB, strideC;  // elements between consecutive matrices
  const float* A;
  const float* B;
  float* C;
  float alpha, beta;
  const float* bias;      // [N] or nullptr: added to every row
  float* Z;               // optional copy of the value before the activation (pitch ldc, stride strideC)
  int act;                // Act
  float act_alpha;        // coefficient of ACT_ELU / ACT_LEAKY_RELU
  // Row operation applied to alpha * op(A) * op(B) before it is stored, for products whose whole row lies in one
  // tile (N <= 128): the two softmax passes of scaled dot-product attention.
  int row_op;             // RowOp
  int causal;             // ROW_SOFTMAX: columns above the main diagonal of every matrix count as -1e12
  const float* aux;       // ROW_SOFTMAX_GRAD: the softmax output y, laid out like C
  OutMap omap;            // where C (and Z) go when not to the dense layout
};
enum RowOp : int { ROW_NONE = 0, ROW_SOFTMAX = 1, ROW_SOFTMAX_GRAD = 2 };

__device__ __forceinline__ float act_forward(int act, float v, float a = 0.0f) {
  // Formulas of Prod/CPU/CpuTensorActivationFunctions.cs:152-244 and Prod/Utils.cs:888-891.
  switch (act) {
    case ACT_RELU: return fmaxf(v, 0.0f);
    case ACT_CLIPPED_RELU: return fminf(fmaxf(v, 0.0f), SNB_CLIPPED_RELU_CEILING);
    case ACT_LEAKY_RELU: return v >= 0.0f ? v : a * v;                 // :210-213
    case ACT_LN: return v <= 0.0f ? -100.0f : logf(v);                   // :170-174
    case ACT_ELU: return v >= 0.0f ? v : a * expm1f(v);                // :223-226 (alpha * (exp(x) - 1), in double there)
    case ACT_SWISH: return v / (1.0f + expf(-v));
    case ACT_TANH: return tanhf(v);
    case ACT_SIGMOID: return 1.0f / (1.0f + expf(-v));
    default: return v;
  }
}

// For fully unrolled epilogues: Identity and Relu inline, the transcendental activations through one
// out-of-line copy, so that the unrolled code stays small enough for the instruction cache.
static __device__ __noinline__ float act_forward_call(int act, float v, float a) { return act_forward(act, v, a); }
__device__ __forceinline__ float act_forward_compact(int act, float v, float a = 0.0f) {
  if (act == ACT_IDENTITY) return v;
  if (act == ACT_RELU) return fmaxf(v, 0.0f);
  return act_forward_call(act, v, a);
}

// Gradient with respect to the pre-activation, from the upstream gradient dy, the activation
// output y and (SWISH and ELU only) the pre-activation x.
__device__ __forceinline__ float act_backward(int act, float dy, float x, float y, float a = 0.0f) {
  switch (act) {
    case ACT_RELU: return y > 0.0f ? dy : 0.0f;                       // CpuTensorActivationFunctions.cs:202-206
    case ACT_CLIPPED_RELU: return (y > 0.0f && y < SNB_CLIPPED_RELU_CEILING) ? dy : 0.0f;   // open interval: flat at both clips
    case ACT_LEAKY_RELU: return y >= 0.0f ? dy : a * dy;              // :214-219
    case ACT_ELU: return x >= 0.0f ? dy : dy * (y + a);               // :227-231
    case ACT_LN: return dy / x;                                       // :176-180
    case ACT_SWISH: {                                                  // :158-167
      float s = (fabsf(x) < 0.0001f) ? 0.5f : y / x;
      return dy * (s + x * s * (1.0f - s));
    }
    case ACT_TANH: return dy * (1.0f - y * y);                        // :190-194
    case ACT_SIGMOID: return dy * y * (1.0f - y);                     // :240-244
    default: return dy;
  }
}

struct Epilogue {
  float alpha, beta;
  const float* bias;
  float* Z;
  int act;
  __device__ __forceinline__ float apply(float acc, float c_old, float bias_v) const {
    float v = alpha * acc;
    if (beta != 0.0f) v = fmaf(beta, c_old, v);
    return v + bias_v;
  }
};

}  // namespace snb
