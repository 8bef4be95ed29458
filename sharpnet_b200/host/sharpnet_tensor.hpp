// C++ host-side mirror of SharpNet's GPU tensor API for the matrix-multiply path, on top of the
// C ABI of libsharpnet_b200.  SharpNet itself is C#; where no .NET toolchain exists this header is
// the compiled-language stand-in for the P/Invoke shim: same class and method names, same argument
// order and meaning, status codes turned into exceptions as GPUWrapper.CheckStatus does
// (Prod/GPU/GPUWrapper.cs:662-668).  Header only; link with -lsharpnet_b200 -lcudart.
#pragma once
#include <cuda_runtime.h>

#include <memory>
#include <numeric>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/sharpnet_b200.h"

namespace SharpNet {

enum class cudnnActivationMode_t : int {   // Prod/GPU/CudnnWrapper.cs:267-281
  CUDNN_ACTIVATION_SIGMOID = 0, CUDNN_ACTIVATION_RELU = 1, CUDNN_ACTIVATION_TANH = 2, CUDNN_ACTIVATION_CLIPPED_RELU = 3,
  CUDNN_ACTIVATION_ELU = 4, CUDNN_ACTIVATION_IDENTITY = 5, CUDNN_ACTIVATION_SWISH = 6, CUDNN_ACTIVATION_SOFTMAX = 1000,
  CUDNN_ACTIVATION_LEAKY_RELU = 1002, CUDNN_ACTIVATION_LN = 1004, CUDNN_ACTIVATION_SOFTMAX_LAST_DIMENSION = 1005
};

enum class EvaluationMetricEnum : int {   // the losses whose gradient the library produces (Prod/Data/Tensor.cs:1182-1217)
  BinaryCrossentropy = SNB200_LOSS_BINARY_CROSSENTROPY, CategoricalCrossentropy = SNB200_LOSS_CATEGORICAL_CROSSENTROPY,
  Mse = SNB200_LOSS_MSE
};

// One per device: owns the library handle (the role of Prod/GPU/GPUWrapper.cs:99-160).
class GPUWrapper {
 public:
  explicit GPUWrapper(int deviceId) : DeviceId(deviceId) {
    const int st = snb200_create(&handle_, deviceId);
    if (st != 0) throw std::runtime_error("snb200_create failed with status " + std::to_string(st));
  }
  ~GPUWrapper() { if (handle_) snb200_destroy(handle_); }
  GPUWrapper(const GPUWrapper&) = delete;
  GPUWrapper& operator=(const GPUWrapper&) = delete;
  void CheckStatus(int status) const {
    if (status != 0) throw std::runtime_error(std::string(snb200_last_error_string(handle_)) + " (status " +
                                              std::to_string(status) + ")");
  }
  snb200_handle_t Handle() const { return handle_; }
  void SetMathMode(int mode) { CheckStatus(snb200_set_math_mode(handle_, mode)); }
  // The coefficient SharpNet runs the activation with: the layer's activationParameter for LeakyRelu, 1 for Elu
  // whatever the parameter says (Prod/CPU/CpuTensor.cs:954,1000; the cuDNN descriptor of Prod/GPU/GPUWrapper.cs:183).
  void SetActivationCoefficient(cudnnActivationMode_t activationType, const float* activationParameterOrNull) {
    if (activationType == cudnnActivationMode_t::CUDNN_ACTIVATION_ELU) CheckStatus(snb200_set_activation_parameter(handle_, 1.0f));
    else if (activationParameterOrNull) CheckStatus(snb200_set_activation_parameter(handle_, *activationParameterOrNull));
  }
  const int DeviceId;
 private:
  snb200_handle_t handle_ = nullptr;
};

// fp32 tensor of up to 4 dimensions in device memory (Prod/GPU/GpuTensor.cs); owns its buffer unless
// it was made by Reshape (a view, like Prod/GPU/GpuTensor.cs:585-620).
class GPUTensor {
 public:
  GPUTensor(std::vector<int> shape, const float* hostDataOrNull, GPUWrapper& wrapper)
      : Shape(std::move(shape)), wrapper_(&wrapper), owner_(true) {
    const size_t bytes = sizeof(float) * static_cast<size_t>(std::max<long long>(Count(), 2));   // min 8 bytes, GpuTensor.cs:38
    if (cudaMalloc(&ptr_, bytes) != cudaSuccess) throw std::runtime_error("cudaMalloc failed");
    if (hostDataOrNull) cudaMemcpy(ptr_, hostDataOrNull, sizeof(float) * Count(), cudaMemcpyHostToDevice);
    else cudaMemset(ptr_, 0, bytes);
  }
  ~GPUTensor() { if (owner_ && ptr_) cudaFree(ptr_); }
  GPUTensor(const GPUTensor&) = delete;
  GPUTensor& operator=(const GPUTensor&) = delete;
  GPUTensor(GPUTensor&& o) noexcept : Shape(std::move(o.Shape)), wrapper_(o.wrapper_), ptr_(o.ptr_), owner_(o.owner_) {
    o.ptr_ = nullptr;
  }

  std::vector<int> Shape;
  long long Count() const { return std::accumulate(Shape.begin(), Shape.end(), 1LL, std::multiplies<long long>()); }
  int MultDim0() const {   // product of the trailing dimensions, Prod/Data/Tensor.cs:1521-1526
    return static_cast<int>(std::accumulate(Shape.begin() + 1, Shape.end(), 1LL, std::multiplies<long long>()));
  }
  float* Pointer() const { return ptr_; }
  GPUTensor Reshape(std::vector<int> shape) const {
    GPUTensor v(*this, std::move(shape));
    return v;
  }
  GPUTensor As2DTensor(bool flattenInputTensorOnLastDimension) const {   // Prod/Data/Tensor.cs:1645-1654
    if (flattenInputTensorOnLastDimension) return Reshape({static_cast<int>(Count() / Shape.back()), Shape.back()});
    return Reshape({Shape[0], MultDim0()});
  }
  std::vector<float> ContentAsFloatArray() const {
    std::vector<float> out(static_cast<size_t>(Count()));
    cudaMemcpy(out.data(), ptr_, sizeof(float) * out.size(), cudaMemcpyDeviceToHost);
    return out;
  }

  // this = alpha * op(a) * op(b) + beta * this          (Prod/Data/Tensor.cs:388-397, Prod/GPU/GpuTensor.cs:1196-1227)
  void Dot(const GPUTensor& a, bool transposeA, const GPUTensor& b, bool transposeB, float alpha, float beta) {
    wrapper_->CheckStatus(snb200_gemm(wrapper_->Handle(), transposeA, transposeB, a.Shape[0], a.MultDim0(), b.Shape[0],
                                      b.MultDim0(), alpha, a.ptr_, b.ptr_, beta, ptr_));
  }
  void Dot(const GPUTensor& a, const GPUTensor& b) { Dot(a, false, b, false, 1.0f, 0.0f); }   // Tensor.cs:60
  // this[i] = alpha * op(a[i]) * op(b[i]) + beta * this[i]   (Tensor.cs:400-415, GpuTensor.cs:1163-1194)
  void BatchMatrixMultiplication(const GPUTensor& a_3D, bool transposeA, const GPUTensor& b_3D, bool transposeB,
                                 float alpha, float beta) {
    wrapper_->CheckStatus(snb200_batched_gemm(wrapper_->Handle(), transposeA, transposeB, a_3D.Shape[1], a_3D.Shape[2],
                                              a_3D.MultDim0(), b_3D.Shape[1], b_3D.Shape[2], b_3D.MultDim0(), MultDim0(),
                                              a_3D.Shape[0], alpha, a_3D.ptr_, b_3D.ptr_, beta, ptr_));
  }
  // y[m, :] += this (the bias)                           (Tensor.cs:495, GpuTensor.cs:633-644)
  void BroadcastAddVectorToOutput(GPUTensor& y) const {
    wrapper_->CheckStatus(snb200_bias_add(wrapper_->Handle(), y.Shape[0], y.MultDim0(), ptr_, y.ptr_));
  }
  // biasGradient[n] = sum_m this[m, n] (this = dy)       (Tensor.cs:710, GpuTensor.cs:686-701)
  void Compute_BiasGradient_from_dy(GPUTensor& biasGradient_1D) const {
    wrapper_->CheckStatus(snb200_bias_grad(wrapper_->Handle(), Shape[0], MultDim0(), ptr_, biasGradient_1D.ptr_));
  }
  // y = act(this); activationParameter is the host value of SharpNet's one-element tensor (LeakyRelu's slope)
  //                                                       (Tensor.cs:618, GpuTensor.cs:397-443)
  void ActivationForward(cudnnActivationMode_t activationType, const float* activationParameterOrNull, GPUTensor& y) const {
    if (activationType == cudnnActivationMode_t::CUDNN_ACTIVATION_SOFTMAX ||
        activationType == cudnnActivationMode_t::CUDNN_ACTIVATION_SOFTMAX_LAST_DIMENSION) {
      // over the columns of the 2-D view (GpuTensor.cs:407-413), or over the last dimension
      const int cols = activationType == cudnnActivationMode_t::CUDNN_ACTIVATION_SOFTMAX ? MultDim0() : Shape.back();
      wrapper_->CheckStatus(snb200_softmax_fwd(wrapper_->Handle(), Count() / cols, cols, ptr_, y.ptr_));
      return;
    }
    wrapper_->SetActivationCoefficient(activationType, activationParameterOrNull);
    wrapper_->CheckStatus(snb200_activation_fwd(wrapper_->Handle(), static_cast<int>(activationType), Count(), ptr_, y.ptr_));
  }
  void ActivationForward(cudnnActivationMode_t activationType, GPUTensor& y) const { ActivationForward(activationType, nullptr, y); }
  // this = dx = act'(x, y) * dy                           (Tensor.cs:628, GpuTensor.cs:445-490)
  void ActivationBackward(cudnnActivationMode_t activationType, const float* activationParameterOrNull, const GPUTensor& dy,
                          const GPUTensor* x, const GPUTensor* y) {
    if (activationType == cudnnActivationMode_t::CUDNN_ACTIVATION_SOFTMAX ||
        activationType == cudnnActivationMode_t::CUDNN_ACTIVATION_SOFTMAX_LAST_DIMENSION) {
      const int cols = activationType == cudnnActivationMode_t::CUDNN_ACTIVATION_SOFTMAX ? MultDim0() : Shape.back();
      wrapper_->CheckStatus(snb200_softmax_bwd(wrapper_->Handle(), Count() / cols, cols, dy.ptr_, y->ptr_, ptr_));   // GpuTensor.cs:461-468
      return;
    }
    wrapper_->SetActivationCoefficient(activationType, activationParameterOrNull);
    wrapper_->CheckStatus(snb200_activation_bwd(wrapper_->Handle(), static_cast<int>(activationType), Count(), dy.ptr_,
                                                x ? x->ptr_ : nullptr, y ? y->ptr_ : nullptr, ptr_));
  }
  void ActivationBackward(cudnnActivationMode_t activationType, const GPUTensor& dy, const GPUTensor* x, const GPUTensor* y) {
    ActivationBackward(activationType, nullptr, dy, x, y);
  }
  // this += alpha * x                                     (Tensor.cs:555, GpuTensor.cs:1359-1362)
  void Update_Adding_Alpha_X(float alpha, const GPUTensor& x) {
    wrapper_->CheckStatus(snb200_axpy(wrapper_->Handle(), Count(), alpha, x.ptr_, ptr_));
  }
  // target[a, c, b, :] = this[a, b, c, :]                (GpuTensor.cs:672-684)
  void TransposeSecondAndThirdDimension(GPUTensor& target) const {
    const int A = Shape[0], B = Shape[1], C = Shape[2];
    const int D = static_cast<int>(Count() / (static_cast<long long>(A) * B * C));
    wrapper_->CheckStatus(snb200_transpose_second_third(wrapper_->Handle(), A, B, C, D, ptr_, target.ptr_));
    target.Shape = Shape;
    std::swap(target.Shape[1], target.Shape[2]);
  }
  // this = W: SGD with momentum; velocity null = the VanillaSgd update   (Tensor.cs:714, GpuTensor.cs:1147-1161)
  void UpdateSGDOptimizer(double learningRate, double momentum, bool nesterov, const GPUTensor& dW, GPUTensor* velocity) {
    wrapper_->CheckStatus(snb200_sgd_update(wrapper_->Handle(), Count(), static_cast<float>(learningRate),
                                            static_cast<float>(momentum), nesterov, dW.ptr_, ptr_,
                                            velocity ? velocity->ptr_ : nullptr));
  }
  // this = W: Adam / AdamW                                (Tensor.cs:712, GpuTensor.cs:1136-1145)
  void UpdateAdamOptimizer(double learningRate, double beta1, double beta2, double epsilon, double weight_decay,
                           const GPUTensor& dW, GPUTensor& adam_vW, GPUTensor& adam_sW, int timeStep) {
    wrapper_->CheckStatus(snb200_adam_update(wrapper_->Handle(), Count(), learningRate, beta1, beta2, epsilon, weight_decay,
                                             timeStep, dW.ptr_, ptr_, adam_vW.ptr_, adam_sW.ptr_));
  }
  // this = dyPredicted = scale * (yPredicted - yExpected)   (Tensor.cs:1182-1217)
  void ComputeGradientForEvaluationMetric(const GPUTensor& yExpected, const GPUTensor& yPredicted, EvaluationMetricEnum loss) {
    wrapper_->CheckStatus(snb200_loss_gradient(wrapper_->Handle(), static_cast<int>(loss), Shape[0], MultDim0(),
                                               yExpected.ptr_, yPredicted.ptr_, ptr_));
  }
  GPUWrapper& Wrapper() const { return *wrapper_; }

 private:
  GPUTensor(const GPUTensor& base, std::vector<int> shape)
      : Shape(std::move(shape)), wrapper_(base.wrapper_), ptr_(base.ptr_), owner_(false) {}
  GPUWrapper* wrapper_;
  float* ptr_ = nullptr;
  bool owner_;
};

// Static methods of the Dense layer (Prod/Layers/Linear.cs:125-191), weights stored [out, in].
struct Linear {
  static void DenseForwardPropagation(GPUTensor& y, const GPUTensor& x, const GPUTensor& weights,
                                      const GPUTensor* biasIfAny_1D, bool flattenInputTensorOnLastDimension) {
    GPUTensor x2 = x.As2DTensor(flattenInputTensorOnLastDimension);
    GPUTensor y2 = y.As2DTensor(flattenInputTensorOnLastDimension);
    y2.Dot(x2, false, weights, true, 1.0f, 0.0f);
    if (biasIfAny_1D) biasIfAny_1D->BroadcastAddVectorToOutput(y2);
  }
  static void DenseBackwardPropagation(GPUTensor* dx, GPUTensor& weightGradients, GPUTensor* biasGradients_1D,
                                       const GPUTensor& x, const GPUTensor& dy, const GPUTensor& weights,
                                       float multiplier, bool prevLayerIsInputLayer,
                                       bool flattenInputTensorOnLastDimension) {
    GPUTensor x2 = x.As2DTensor(flattenInputTensorOnLastDimension);
    GPUTensor dy2 = dy.As2DTensor(flattenInputTensorOnLastDimension);
    weightGradients.Dot(dy2, true, x2, false, multiplier, 0.0f);
    if (biasGradients_1D) dy2.Compute_BiasGradient_from_dy(*biasGradients_1D);
    if (prevLayerIsInputLayer || !dx) return;
    GPUTensor dx2 = dx->As2DTensor(flattenInputTensorOnLastDimension);
    dx2.Dot(dy2, false, weights, false, 1.0f, 0.0f);
  }
  // Dense + following ActivationLayer in one call each way (snb200_dense_fwd / snb200_dense_bwd).
  static void FusedForward(GPUTensor& y, const GPUTensor& x, const GPUTensor& weights, const GPUTensor* bias,
                           cudnnActivationMode_t act, GPUTensor* z) {
    GPUWrapper& w = y.Wrapper();
    w.CheckStatus(snb200_dense_fwd(w.Handle(), SNB200_W_OUT_IN, x.Shape[0], x.MultDim0(), y.MultDim0(), x.Pointer(),
                                   weights.Pointer(), bias ? bias->Pointer() : nullptr, static_cast<int>(act),
                                   z ? z->Pointer() : nullptr, y.Pointer()));
  }
  static void FusedBackward(GPUTensor* dx, GPUTensor& dW, GPUTensor* db, const GPUTensor& x, const GPUTensor& dy,
                            const GPUTensor& weights, cudnnActivationMode_t act, const GPUTensor* y, const GPUTensor* z,
                            float multiplier, GPUTensor* dzScratch) {
    GPUWrapper& w = dW.Wrapper();
    w.CheckStatus(snb200_dense_bwd(w.Handle(), SNB200_W_OUT_IN, x.Shape[0], x.MultDim0(), dy.MultDim0(), x.Pointer(),
                                   weights.Pointer(), dy.Pointer(), static_cast<int>(act), y ? y->Pointer() : nullptr,
                                   z ? z->Pointer() : nullptr, multiplier, dzScratch ? dzScratch->Pointer() : nullptr,
                                   dx ? dx->Pointer() : nullptr, dW.Pointer(), db ? db->Pointer() : nullptr));
  }
};

// The gradient sum of data-parallel training (Prod/Networks/NetworkMultiGPUSupport.cs:161-173) for SharpNet's
// one-thread-per-GPU model (Prod/Networks/Network.cs:71-83): one communicator over the wrappers of one process.
// AllReduceSum leaves the sum over all replicas in every replica's buffer; each wrapper's call is made from the
// thread that drives that wrapper.
class GradientCommunicator {
 public:
  explicit GradientCommunicator(const std::vector<GPUWrapper*>& wrappers) : wrappers_(wrappers) {
    std::vector<snb200_handle_t> handles;
    for (GPUWrapper* w : wrappers_) handles.push_back(w->Handle());
    wrappers_[0]->CheckStatus(snb200_comm_init_all(handles.data(), static_cast<int>(handles.size())));
  }
  ~GradientCommunicator() { for (GPUWrapper* w : wrappers_) snb200_comm_destroy(w->Handle()); }
  GradientCommunicator(const GradientCommunicator&) = delete;
  GradientCommunicator& operator=(const GradientCommunicator&) = delete;
  static void AllReduceSum(GPUTensor& gradients) {
    GPUWrapper& w = gradients.Wrapper();
    w.CheckStatus(snb200_allreduce_sum(w.Handle(), gradients.Pointer(), gradients.Count()));
  }
  // a layer's dW and db as one collective launch
  static void AllReduceSum(GPUTensor& weightGradients, GPUTensor& biasGradients) {
    GPUWrapper& w = weightGradients.Wrapper();
    float* bufs[2] = {weightGradients.Pointer(), biasGradients.Pointer()};
    const long long counts[2] = {weightGradients.Count(), biasGradients.Count()};
    w.CheckStatus(snb200_allreduce_sum_group(w.Handle(), 2, bufs, counts));
  }
 private:
  std::vector<GPUWrapper*> wrappers_;
};

// Page-locks a caller-owned host array for as long as the object lives, as HostPinnedMemory does for a managed
// array (Prod/CPU/HostPinnedMemory.cs:17-21): what the asynchronous host-to-device copies below need.
class HostPinnedMemory {
 public:
  HostPinnedMemory(void* hostPointer, long long bytes) : ptr_(hostPointer) {
    const int st = snb200_host_pin(hostPointer, bytes);
    if (st != 0) throw std::runtime_error("snb200_host_pin failed with status " + std::to_string(st));
  }
  ~HostPinnedMemory() { snb200_host_unpin(ptr_); }
  HostPinnedMemory(const HostPinnedMemory&) = delete;
  HostPinnedMemory& operator=(const HostPinnedMemory&) = delete;
  void* Pointer() const { return ptr_; }
 private:
  void* ptr_;
};

// The mini-batch copies of Network.cs:1211-1258 (x_miniBatch_cpu.CopyTo(x_miniBatch)) on a copy stream of their
// own, `slots`-fold buffered: Issue(slot, ...) queues the copies of a step's inputs, Acquire(slot) makes the
// wrapper's stream wait for them, Release(slot) marks where the slot's last reader ends.
class MiniBatchStager {
 public:
  MiniBatchStager(GPUWrapper& wrapper, int slots) : wrapper_(&wrapper) {
    wrapper_->CheckStatus(snb200_stager_create(wrapper_->Handle(), slots, &stager_));
  }
  ~MiniBatchStager() { if (stager_) snb200_stager_destroy(stager_); }
  MiniBatchStager(const MiniBatchStager&) = delete;
  MiniBatchStager& operator=(const MiniBatchStager&) = delete;
  // copies[i]: (device tensor of the slot, pinned host source holding at least its Count() floats)
  void Issue(int slot, const std::vector<std::pair<GPUTensor*, const float*>>& copies) {
    std::vector<void*> dst;
    std::vector<const void*> src;
    std::vector<long long> bytes;
    for (const auto& c : copies) {
      dst.push_back(c.first->Pointer());
      src.push_back(c.second);
      bytes.push_back(static_cast<long long>(sizeof(float)) * c.first->Count());
    }
    wrapper_->CheckStatus(snb200_stager_issue(stager_, slot, static_cast<int>(copies.size()), dst.data(), src.data(), bytes.data()));
  }
  void Acquire(int slot) { wrapper_->CheckStatus(snb200_stager_acquire(stager_, slot)); }
  void AcquirePart(int slot, int part) { wrapper_->CheckStatus(snb200_stager_acquire_part(stager_, slot, part)); }
  void Release(int slot) { wrapper_->CheckStatus(snb200_stager_release(stager_, slot)); }
 private:
  GPUWrapper* wrapper_;
  snb200_stager_t stager_ = nullptr;
};

// Static methods of the attention layer (Prod/Layers/ScaledDotProductAttentionLayer.cs:46-129); Q [batch, q, E],
// K and V [batch, v, E].  weights_buffer keeps the probabilities for the backward pass, scores_grad_scratch
// [batch, q, v] is what the reference takes from its memory pool there.
struct ScaledDotProductAttentionLayer {
  static void ScaledDotProductAttentionForwardPropagation(const GPUTensor& Q, const GPUTensor& K, const GPUTensor& V,
                                                          GPUTensor& y, GPUTensor& weights_buffer, bool use_scale,
                                                          bool is_causal) {
    GPUWrapper& w = y.Wrapper();
    w.CheckStatus(snb200_sdpa_fwd(w.Handle(), Q.Shape[0], Q.Shape[1], V.Shape[1], Q.Shape[2], use_scale, is_causal,
                                  Q.Pointer(), K.Pointer(), V.Pointer(), weights_buffer.Pointer(), y.Pointer()));
  }
  static void ScaledDotProductAttentionBackwardPropagation(GPUTensor& dQ, GPUTensor& dK, GPUTensor& dV, const GPUTensor& Q,
                                                           const GPUTensor& K, const GPUTensor& V, const GPUTensor& dy,
                                                           const GPUTensor& weights_buffer, GPUTensor& scores_grad_scratch,
                                                           bool use_scale) {
    GPUWrapper& w = dQ.Wrapper();
    w.CheckStatus(snb200_sdpa_bwd(w.Handle(), Q.Shape[0], Q.Shape[1], V.Shape[1], Q.Shape[2], use_scale, Q.Pointer(),
                                  K.Pointer(), V.Pointer(), dy.Pointer(), weights_buffer.Pointer(),
                                  scores_grad_scratch.Pointer(), dQ.Pointer(), dK.Pointer(), dV.Pointer()));
  }
};

// The multi-head attention layer (Prod/Layers/MultiheadAttention.cs:178-295) over snb200_mha_fwd / snb200_mha_bwd:
// the parameters (weights [out, in], biases or null) belong to the caller, the state the layer keeps between its
// two passes (:73-81) and the backward scratch are allocated on first use for the shapes of the call.
class MultiheadAttention {
 public:
  struct Parameters {
    const GPUTensor *w_Q, *w_K, *w_V, *out_proj_weight;
    const GPUTensor *w_Q_bias, *w_K_bias, *w_V_bias, *out_proj_bias;   // null: no bias
  };
  struct Gradients {
    GPUTensor *w_Q, *w_K, *w_V, *out_proj_weight;
    GPUTensor *w_Q_bias, *w_K_bias, *w_V_bias, *out_proj_bias;         // null where the layer has no bias
  };
  MultiheadAttention(int num_heads, int key_dim, int value_dim, bool is_causal, GPUWrapper& wrapper)
      : num_heads_(num_heads), key_dim_(key_dim), value_dim_(value_dim), is_causal_(is_causal), wrapper_(&wrapper) {}

  void ForwardPropagation(const GPUTensor& Q, const GPUTensor& K, const GPUTensor& V, const Parameters& p, GPUTensor& y) {
    const snb200_mha_desc d = Desc(Q, V);
    const int BH = d.batch * num_heads_;
    Q_heads_T.reset(new GPUTensor({BH, d.q_steps, key_dim_}, nullptr, *wrapper_));
    K_heads_T.reset(new GPUTensor({BH, d.v_steps, key_dim_}, nullptr, *wrapper_));
    V_heads_T.reset(new GPUTensor({BH, d.v_steps, value_dim_}, nullptr, *wrapper_));
    attention_heads_T.reset(new GPUTensor({d.batch, d.q_steps, num_heads_ * value_dim_}, nullptr, *wrapper_));
    weights_buffer.reset(new GPUTensor({BH, d.q_steps, d.v_steps}, nullptr, *wrapper_));
    const snb200_mha_weights w = Weights(p);
    const snb200_mha_state st = State();
    wrapper_->CheckStatus(snb200_mha_fwd(wrapper_->Handle(), &d, &w, Q.Pointer(), K.Pointer(), V.Pointer(), &st, nullptr,
                                         y.Pointer()));
  }
  // dW_multiplier: the factor of the weight gradients (Linear.cs:152-158)
  void BackwardPropagation(const GPUTensor& Q, const GPUTensor& K, const GPUTensor& V, const GPUTensor& dy,
                           const Parameters& p, float dW_multiplier, const Gradients& g, GPUTensor& dQ, GPUTensor& dK,
                           GPUTensor& dV) {
    const snb200_mha_desc d = Desc(Q, V);
    const long long need = snb200_mha_scratch_floats(&d, 1);
    if (!scratch_ || scratch_->Count() < need) scratch_.reset(new GPUTensor({static_cast<int>(need)}, nullptr, *wrapper_));
    const snb200_mha_weights w = Weights(p);
    const snb200_mha_state st = State();
    auto ptr = [](GPUTensor* t) { return t ? t->Pointer() : nullptr; };
    const snb200_mha_gradients gr = {ptr(g.w_Q), ptr(g.w_K), ptr(g.w_V), ptr(g.out_proj_weight),
                                     ptr(g.w_Q_bias), ptr(g.w_K_bias), ptr(g.w_V_bias), ptr(g.out_proj_bias)};
    wrapper_->CheckStatus(snb200_mha_bwd(wrapper_->Handle(), &d, &w, Q.Pointer(), K.Pointer(), V.Pointer(), dy.Pointer(), &st,
                                         dW_multiplier, scratch_->Pointer(), &gr, dQ.Pointer(), dK.Pointer(), dV.Pointer()));
  }
  // what the layer keeps between the passes (MultiheadAttention.cs:73-81)
  std::unique_ptr<GPUTensor> Q_heads_T, K_heads_T, V_heads_T, attention_heads_T, weights_buffer;

 private:
  snb200_mha_desc Desc(const GPUTensor& Q, const GPUTensor& V) const {
    return {SNB200_W_OUT_IN, Q.Shape[0], Q.Shape[1], V.Shape[1], Q.Shape[2], num_heads_, key_dim_, value_dim_, is_causal_};
  }
  static snb200_mha_weights Weights(const Parameters& p) {
    auto ptr = [](const GPUTensor* t) -> const float* { return t ? t->Pointer() : nullptr; };
    return {ptr(p.w_Q), ptr(p.w_K), ptr(p.w_V), ptr(p.out_proj_weight), ptr(p.w_Q_bias), ptr(p.w_K_bias), ptr(p.w_V_bias),
            ptr(p.out_proj_bias)};
  }
  snb200_mha_state State() const {
    return {Q_heads_T->Pointer(), K_heads_T->Pointer(), V_heads_T->Pointer(), attention_heads_T->Pointer(),
            weights_buffer->Pointer()};
  }
  int num_heads_, key_dim_, value_dim_;
  bool is_causal_;
  GPUWrapper* wrapper_;
  std::unique_ptr<GPUTensor> scratch_;
};

}  // namespace SharpNet
