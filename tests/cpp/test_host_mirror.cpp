// Drives the C ABI from compiled host code through the C++ mirror of SharpNet's tensor API, the way
// the C# shim would: the reference's exact Dot cases (Tests/GPU/TestGpuTensor.cs:50-120, 1e-9), a
// differential Dot / BatchMatrixMultiplication case against a double-precision host loop, and the
// Dense forward / backward call sequence of Prod/Layers/Linear.cs against the fused entry points.
// Prints "OK <n checks>" and exits 0, or the first mismatch and exits 1.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <random>
#include <string>

#include "../../sharpnet_b200/host/sharpnet_tensor.hpp"

using namespace SharpNet;

static int g_checks = 0;
#define EXPECT(cond, ...)                                             \
  do {                                                                \
    ++g_checks;                                                       \
    if (!(cond)) { std::printf("FAILED %s:%d: ", __FILE__, __LINE__); std::printf(__VA_ARGS__); std::printf("\n"); std::exit(1); } \
  } while (0)

static std::vector<float> uniform(size_t n, float lo, float hi, unsigned seed) {
  std::mt19937 g(seed);
  std::uniform_real_distribution<float> d(lo, hi);
  std::vector<float> v(n);
  for (auto& x : v) x = d(g);
  return v;
}
// C[m, n] = alpha * sum_k opA(m, k) * opB(k, n) + beta * C[m, n] in double
static std::vector<double> ref_gemm(const std::vector<float>& A, int aH, int aW, bool tA, const std::vector<float>& B,
                                    int bH, int bW, bool tB, const std::vector<float>& C, double alpha, double beta) {
  const int M = tA ? aW : aH, N = tB ? bH : bW, K = tA ? aH : aW;
  std::vector<double> out(static_cast<size_t>(M) * N);
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      double s = 0;
      for (int k = 0; k < K; ++k) {
        const double a = tA ? A[static_cast<size_t>(k) * aW + m] : A[static_cast<size_t>(m) * aW + k];
        const double b = tB ? B[static_cast<size_t>(n) * bW + k] : B[static_cast<size_t>(k) * bW + n];
        s += a * b;
      }
      out[static_cast<size_t>(m) * N + n] = alpha * s + beta * C[static_cast<size_t>(m) * N + n];
    }
  return out;
}
static double max_abs_diff(const std::vector<float>& got, const std::vector<double>& want) {
  double d = 0;
  for (size_t i = 0; i < got.size(); ++i) d = std::fmax(d, std::fabs(got[i] - want[i]));
  return d;
}

int main() {
  GPUWrapper gpu(0);
  {  // exact cases of the reference
    float a1[] = {2}, b1[] = {5};
    GPUTensor a({1, 1}, a1, gpu), b({1, 1}, b1, gpu), r({1, 1}, nullptr, gpu);
    r.Dot(a, false, b, false, 1, 0);
    EXPECT(std::fabs(r.ContentAsFloatArray()[0] - 10.0f) < 1e-9, "1x1");
    float a2[] = {1, 2, 3, 4};
    GPUTensor A2({2, 2}, a2, gpu), B2({2, 2}, a2, gpu), R2({2, 2}, nullptr, gpu);
    R2.Dot(A2, B2);
    const float want2[] = {7, 10, 15, 22};
    auto got2 = R2.ContentAsFloatArray();
    for (int i = 0; i < 4; ++i) EXPECT(std::fabs(got2[i] - want2[i]) < 1e-9, "2x2 element %d", i);
    float a3[] = {1, 2}, b3[] = {3, 4};
    GPUTensor A3({2, 1, 1}, a3, gpu), B3({1, 1, 2}, b3, gpu), R3({2, 2}, nullptr, gpu);   // 3-D inputs flattened
    R3.Dot(A3, false, B3, false, 1, 0);
    const float want3[] = {3, 4, 6, 8};
    auto got3 = R3.ContentAsFloatArray();
    for (int i = 0; i < 4; ++i) EXPECT(std::fabs(got3[i] - want3[i]) < 1e-9, "2x1x1 * 1x1x2 element %d", i);
  }
  for (int mode = 0; mode < 3; ++mode) {  // every math mode, every transposition, beta = 1
    gpu.SetMathMode(mode);
    const double tol = (mode == 1 ? 2e-3 : 1e-5);
    const int M = 200, N = 328, K = 100;
    unsigned seed = 1;
    for (int tA = 0; tA < 2; ++tA)
      for (int tB = 0; tB < 2; ++tB) {
        const int aH = tA ? K : M, aW = tA ? M : K, bH = tB ? N : K, bW = tB ? K : N;
        auto a = uniform(static_cast<size_t>(aH) * aW, -1, 1, seed++), b = uniform(static_cast<size_t>(bH) * bW, -1, 1, seed++);
        auto c = uniform(static_cast<size_t>(M) * N, -1, 1, seed++);
        GPUTensor A({aH, aW}, a.data(), gpu), B({bH, bW}, b.data(), gpu), C({M, N}, c.data(), gpu);
        C.Dot(A, tA, B, tB, 0.5f, 1.0f);
        const double e = max_abs_diff(C.ContentAsFloatArray(), ref_gemm(a, aH, aW, tA, b, bH, bW, tB, c, 0.5, 1.0)) / std::sqrt(K);
        EXPECT(e <= tol, "Dot mode %d tA %d tB %d: scaled error %.3e", mode, tA, tB, e);
      }
  }
  gpu.SetMathMode(0);
  {  // BatchMatrixMultiplication, batch 3, 12x12 * (12x7)^T ... as Tests/TestParallelRunCpuVersusGpu.cs:377-401
    const int nb = 3, L = 12, D = 7;
    auto dy = uniform(nb * L * D, -1.5f, 1.5f, 50), V = uniform(nb * L * D, -1.5f, 1.5f, 51);
    GPUTensor DY({nb, L, D}, dy.data(), gpu), Vt({nb, L, D}, V.data(), gpu), W({nb, L, L}, nullptr, gpu);
    W.BatchMatrixMultiplication(DY, false, Vt, true, 0.25f, 0.0f);
    auto got = W.ContentAsFloatArray();
    for (int i = 0; i < nb; ++i) {
      std::vector<float> a(dy.begin() + i * L * D, dy.begin() + (i + 1) * L * D), b(V.begin() + i * L * D, V.begin() + (i + 1) * L * D);
      std::vector<float> c(L * L, 0.0f), g(got.begin() + i * L * L, got.begin() + (i + 1) * L * L);
      EXPECT(max_abs_diff(g, ref_gemm(a, L, D, false, b, L, D, true, c, 0.25, 0.0)) < 1e-5, "batched matrix %d", i);
    }
  }
  {  // Dense: the Linear.cs sequence (Dot, bias add, activation) against the fused call, forward and backward
    const int M = 256, K = 192, N = 128;
    auto x = uniform(M * K, -2, 2, 60), W = uniform(N * K, -0.1f, 0.1f, 61), b = uniform(N, -0.5f, 0.5f, 62), dy = uniform(M * N, -2, 2, 63);
    GPUTensor X({M, K}, x.data(), gpu), Wt({N, K}, W.data(), gpu), Bt({N}, b.data(), gpu), DY({M, N}, dy.data(), gpu);
    GPUTensor z1({M, N}, nullptr, gpu), y1({M, N}, nullptr, gpu), z2({M, N}, nullptr, gpu), y2({M, N}, nullptr, gpu);
    Linear::DenseForwardPropagation(z1, X, Wt, &Bt, false);
    z1.ActivationForward(cudnnActivationMode_t::CUDNN_ACTIVATION_SWISH, y1);
    Linear::FusedForward(y2, X, Wt, &Bt, cudnnActivationMode_t::CUDNN_ACTIVATION_SWISH, &z2);
    auto a1 = y1.ContentAsFloatArray(), a2 = y2.ContentAsFloatArray();
    for (size_t i = 0; i < a1.size(); ++i) EXPECT(a1[i] == a2[i], "fused forward differs at %zu", i);
    std::vector<float> zeros(M * N, 0.0f);
    auto zref = ref_gemm(x, M, K, false, W, N, K, true, zeros, 1.0, 0.0);
    for (int m = 0; m < M; ++m) for (int n = 0; n < N; ++n) zref[m * N + n] += b[n];
    EXPECT(max_abs_diff(z2.ContentAsFloatArray(), zref) / std::sqrt(K) < 1e-5, "pre-activation vs double");
    GPUTensor dz1({M, N}, nullptr, gpu), dx1({M, K}, nullptr, gpu), dW1({N, K}, nullptr, gpu), db1({N}, nullptr, gpu);
    dz1.ActivationBackward(cudnnActivationMode_t::CUDNN_ACTIVATION_SWISH, DY, &z1, &y1);
    Linear::DenseBackwardPropagation(&dx1, dW1, &db1, X, dz1, Wt, 1.0f / M, false, false);
    GPUTensor dz2({M, N}, nullptr, gpu), dx2({M, K}, nullptr, gpu), dW2({N, K}, nullptr, gpu), db2({N}, nullptr, gpu);
    Linear::FusedBackward(&dx2, dW2, &db2, X, DY, Wt, cudnnActivationMode_t::CUDNN_ACTIVATION_SWISH, &y2, &z2, 1.0f / M, &dz2);
    auto w1 = dW1.ContentAsFloatArray(), w2 = dW2.ContentAsFloatArray();
    for (size_t i = 0; i < w1.size(); ++i) EXPECT(w1[i] == w2[i], "fused dW differs at %zu", i);
    auto g1 = dx1.ContentAsFloatArray(), g2 = dx2.ContentAsFloatArray();
    for (size_t i = 0; i < g1.size(); ++i) EXPECT(g1[i] == g2[i], "fused dx differs at %zu", i);
    auto dzv = dz2.ContentAsFloatArray();
    auto dWref = ref_gemm(dzv, M, N, true, x, M, K, false, std::vector<float>(N * K, 0.0f), 1.0 / M, 0.0);
    EXPECT(max_abs_diff(w2, dWref) * M / std::sqrt(M) / 8.0 < 1e-5, "dW vs double");
    auto dbv = db2.ContentAsFloatArray();
    for (int n = 0; n < N; ++n) {
      double s = 0;
      for (int m = 0; m < M; ++m) s += dzv[m * N + n];
      EXPECT(std::fabs(dbv[n] - s) < 1e-3, "db[%d]", n);
    }
  }
  {  // parametric activations: LeakyRelu with the layer's slope, Elu with SharpNet's fixed coefficient of 1
     // (Prod/CPU/CpuTensorActivationFunctions.cs:210-231, Prod/CPU/CpuTensor.cs:954,1000), Ln (:170-180)
    const int n = 1000;
    auto x = uniform(n, -1.5f, 1.5f, 70), dy = uniform(n, -1.5f, 1.5f, 71);
    GPUTensor X({n}, x.data(), gpu), DY({n}, dy.data(), gpu), Y({n}, nullptr, gpu), DX({n}, nullptr, gpu);
    const float slope = 0.3f, ignored = 0.0f;
    X.ActivationForward(cudnnActivationMode_t::CUDNN_ACTIVATION_LEAKY_RELU, &slope, Y);
    DX.ActivationBackward(cudnnActivationMode_t::CUDNN_ACTIVATION_LEAKY_RELU, &slope, DY, &X, &Y);
    auto y = Y.ContentAsFloatArray(), dx = DX.ContentAsFloatArray();
    for (int i = 0; i < n; ++i) {
      EXPECT(y[i] == (x[i] >= 0 ? x[i] : slope * x[i]), "LeakyRelu forward at %d", i);
      EXPECT(dx[i] == (y[i] >= 0 ? dy[i] : slope * dy[i]), "LeakyRelu backward at %d", i);
    }
    X.ActivationForward(cudnnActivationMode_t::CUDNN_ACTIVATION_ELU, &ignored, Y);
    DX.ActivationBackward(cudnnActivationMode_t::CUDNN_ACTIVATION_ELU, &ignored, DY, &X, &Y);
    y = Y.ContentAsFloatArray(); dx = DX.ContentAsFloatArray();
    for (int i = 0; i < n; ++i) {
      const double want = x[i] >= 0 ? x[i] : std::exp(static_cast<double>(x[i])) - 1.0;
      EXPECT(std::fabs(y[i] - want) <= 1e-6 * std::fabs(want) + 1e-7, "Elu forward at %d", i);
      EXPECT(std::fabs(dx[i] - (x[i] >= 0 ? dy[i] : dy[i] * (y[i] + 1.0f))) <= 1e-6, "Elu backward at %d", i);
    }
    X.ActivationForward(cudnnActivationMode_t::CUDNN_ACTIVATION_LN, Y);
    DX.ActivationBackward(cudnnActivationMode_t::CUDNN_ACTIVATION_LN, DY, &X, &Y);
    y = Y.ContentAsFloatArray(); dx = DX.ContentAsFloatArray();
    for (int i = 0; i < n; ++i) {
      const double want = x[i] <= 0 ? -100.0 : std::log(static_cast<double>(x[i]));
      EXPECT(std::fabs(y[i] - want) <= 1e-6 * std::fabs(want) + 1e-7, "Ln forward at %d", i);
      EXPECT(std::fabs(dx[i] - dy[i] / x[i]) <= 2e-6 * std::fabs(dy[i] / x[i]), "Ln backward at %d", i);
    }
    X.ActivationForward(cudnnActivationMode_t::CUDNN_ACTIVATION_CLIPPED_RELU, Y);
    y = Y.ContentAsFloatArray();
    for (int i = 0; i < n; ++i) EXPECT(y[i] == std::fmin(std::fmax(x[i], 0.0f), 1.0f), "ClippedRelu forward at %d", i);
  }
  {  // attention: the layer's static methods against the same arithmetic spelled out with the tensor calls
     // (Prod/Layers/ScaledDotProductAttentionLayer.cs:46-129), and the optimizer updates against host loops
    const int nb = 6, L = 40, E = 32;
    auto q = uniform(nb * L * E, -1, 1, 80), k = uniform(nb * L * E, -1, 1, 81), v = uniform(nb * L * E, -1, 1, 82), dy = uniform(nb * L * E, -1, 1, 83);
    GPUTensor Q({nb, L, E}, q.data(), gpu), K({nb, L, E}, k.data(), gpu), V({nb, L, E}, v.data(), gpu), DY({nb, L, E}, dy.data(), gpu);
    GPUTensor y({nb, L, E}, nullptr, gpu), wts({nb, L, L}, nullptr, gpu), scores({nb, L, L}, nullptr, gpu), p({nb, L, L}, nullptr, gpu), y2({nb, L, E}, nullptr, gpu);
    ScaledDotProductAttentionLayer::ScaledDotProductAttentionForwardPropagation(Q, K, V, y, wts, true, false);
    scores.BatchMatrixMultiplication(Q, false, K, true, 1.0f / std::sqrt(static_cast<float>(E)), 0.0f);
    scores.ActivationForward(cudnnActivationMode_t::CUDNN_ACTIVATION_SOFTMAX_LAST_DIMENSION, p);
    y2.BatchMatrixMultiplication(p, false, V, false, 1.0f, 0.0f);
    auto w1 = wts.ContentAsFloatArray(), w2 = p.ContentAsFloatArray(), o1 = y.ContentAsFloatArray(), o2 = y2.ContentAsFloatArray();
    for (size_t i = 0; i < w1.size(); ++i) EXPECT(std::fabs(w1[i] - w2[i]) < 2e-6, "attention weights at %zu", i);
    for (size_t i = 0; i < o1.size(); ++i) EXPECT(std::fabs(o1[i] - o2[i]) < 2e-5, "attention output at %zu", i);
    for (int r = 0; r < nb * L; ++r) {
      double sum = 0;
      for (int c = 0; c < L; ++c) sum += w1[r * L + c];
      EXPECT(std::fabs(sum - 1.0) < 1e-5, "probabilities of row %d sum to %f", r, sum);
    }
    GPUTensor dQ({nb, L, E}, nullptr, gpu), dK({nb, L, E}, nullptr, gpu), dV({nb, L, E}, nullptr, gpu), scratch({nb, L, L}, nullptr, gpu);
    ScaledDotProductAttentionLayer::ScaledDotProductAttentionBackwardPropagation(dQ, dK, dV, Q, K, V, DY, wts, scratch, true);
    GPUTensor dV2({nb, L, E}, nullptr, gpu), dW({nb, L, L}, nullptr, gpu), dS({nb, L, L}, nullptr, gpu), dQ2({nb, L, E}, nullptr, gpu), dK2({nb, L, E}, nullptr, gpu);
    dV2.BatchMatrixMultiplication(wts, true, DY, false, 1.0f, 0.0f);                                   // :113
    dW.BatchMatrixMultiplication(DY, false, V, true, 1.0f / std::sqrt(static_cast<float>(E)), 0.0f);   // :119
    dS.ActivationBackward(cudnnActivationMode_t::CUDNN_ACTIVATION_SOFTMAX_LAST_DIMENSION, dW, nullptr, &wts);   // :121
    dQ2.BatchMatrixMultiplication(dS, false, K, false, 1.0f, 0.0f);                                    // :123
    dK2.BatchMatrixMultiplication(dS, true, Q, false, 1.0f, 0.0f);                                     // :124
    auto a = dQ.ContentAsFloatArray(), b = dQ2.ContentAsFloatArray();
    for (size_t i = 0; i < a.size(); ++i) EXPECT(std::fabs(a[i] - b[i]) < 2e-5, "dQ at %zu", i);
    a = dK.ContentAsFloatArray(); b = dK2.ContentAsFloatArray();
    for (size_t i = 0; i < a.size(); ++i) EXPECT(std::fabs(a[i] - b[i]) < 2e-5, "dK at %zu", i);
    a = dV.ContentAsFloatArray(); b = dV2.ContentAsFloatArray();
    for (size_t i = 0; i < a.size(); ++i) EXPECT(std::fabs(a[i] - b[i]) < 2e-5, "dV at %zu", i);
    // head split: [b, t, h, d] -> [b, h, t, d]
    GPUTensor heads({2, 5, 3, 8}, q.data(), gpu), split({2, 3, 5, 8}, nullptr, gpu);
    heads.TransposeSecondAndThirdDimension(split);
    auto sp = split.ContentAsFloatArray();
    for (int bb = 0; bb < 2; ++bb) for (int t = 0; t < 5; ++t) for (int h = 0; h < 3; ++h) for (int d = 0; d < 8; ++d)
      EXPECT(sp[((bb * 3 + h) * 5 + t) * 8 + d] == q[((bb * 5 + t) * 3 + h) * 8 + d], "transposition at %d %d %d %d", bb, t, h, d);
    EXPECT(split.Shape[1] == 3 && split.Shape[2] == 5, "transposed shape");
    // SGD with momentum, then Adam, one step each against the formulas of Prod/CPU/CpuTensor.cs:470-489,1755-1769
    const int n = 777;
    auto w0 = uniform(n, -1, 1, 90), g = uniform(n, -1, 1, 91), vel0 = uniform(n, -0.1f, 0.1f, 92);
    GPUTensor W({n}, w0.data(), gpu), G({n}, g.data(), gpu), Vel({n}, vel0.data(), gpu);
    W.UpdateSGDOptimizer(0.1, 0.9, false, G, &Vel);
    auto wn = W.ContentAsFloatArray(), vn = Vel.ContentAsFloatArray();
    for (int i = 0; i < n; ++i) {
      const float vel = 0.9f * vel0[i] - 0.1f * g[i];
      EXPECT(std::fabs(vn[i] - vel) < 1e-6 && std::fabs(wn[i] - (w0[i] + vel)) < 1e-6, "SGD at %d", i);
    }
    GPUTensor W2({n}, w0.data(), gpu), M1({n}, nullptr, gpu), M2({n}, nullptr, gpu);
    W2.UpdateAdamOptimizer(0.01, 0.9, 0.999, 1e-8, 0.0, G, M1, M2, 1);
    wn = W2.ContentAsFloatArray();
    for (int i = 0; i < n; ++i) {
      const double m = 0.1 * g[i], s2 = 0.001 * g[i] * g[i];
      const double step = 0.01 * std::sqrt(1 - 0.999) / (1 - 0.9) * m / (std::sqrt(s2) + 1e-8);
      EXPECT(std::fabs(wn[i] - (w0[i] - step)) < 2e-6, "Adam at %d: %f against %f", i, wn[i], w0[i] - step);
    }
  }
  {  // multi-head attention as one call each way against the layer's own sequence of tensor calls
     // (Prod/Layers/MultiheadAttention.cs:178-295): projections on the last dimension, head split, attention per
     // head, head merge, output projection -- and the reverse
    const int B = 3, T = 24, H = 4, d = 8, E = H * d;
    auto q = uniform(B * T * E, -1, 1, 100), k = uniform(B * T * E, -1, 1, 101), v = uniform(B * T * E, -1, 1, 102), g = uniform(B * T * E, -1, 1, 103);
    auto wq = uniform(E * E, -0.3f, 0.3f, 104), wk = uniform(E * E, -0.3f, 0.3f, 105), wv = uniform(E * E, -0.3f, 0.3f, 106), wo = uniform(E * E, -0.3f, 0.3f, 107);
    auto bq = uniform(E, -0.2f, 0.2f, 108), bk = uniform(E, -0.2f, 0.2f, 109), bv = uniform(E, -0.2f, 0.2f, 110), bo = uniform(E, -0.2f, 0.2f, 111);
    GPUTensor Q({B, T, E}, q.data(), gpu), K({B, T, E}, k.data(), gpu), V({B, T, E}, v.data(), gpu), DY({B, T, E}, g.data(), gpu);
    GPUTensor Wq({E, E}, wq.data(), gpu), Wk({E, E}, wk.data(), gpu), Wv({E, E}, wv.data(), gpu), Wo({E, E}, wo.data(), gpu);
    GPUTensor Bq({E}, bq.data(), gpu), Bk({E}, bk.data(), gpu), Bv({E}, bv.data(), gpu), Bo({E}, bo.data(), gpu);
    MultiheadAttention mha(H, d, d, true, gpu);
    const MultiheadAttention::Parameters params = {&Wq, &Wk, &Wv, &Wo, &Bq, &Bk, &Bv, &Bo};
    GPUTensor y({B, T, E}, nullptr, gpu);
    mha.ForwardPropagation(Q, K, V, params, y);
    // the same with the layer's tensor calls
    auto project = [&](const GPUTensor& x, const GPUTensor& W, const GPUTensor& bias, GPUTensor& heads_T) {
      GPUTensor p({B, T, E}, nullptr, gpu);
      Linear::DenseForwardPropagation(p, x, W, &bias, true);
      GPUTensor split({B, H, T, d}, nullptr, gpu);
      p.Reshape({B, T, H, d}).TransposeSecondAndThirdDimension(split);
      cudaMemcpy(heads_T.Pointer(), split.Pointer(), sizeof(float) * B * T * E, cudaMemcpyDeviceToDevice);
    };
    GPUTensor QhT({B * H, T, d}, nullptr, gpu), KhT({B * H, T, d}, nullptr, gpu), VhT({B * H, T, d}, nullptr, gpu);
    project(Q, Wq, Bq, QhT); project(K, Wk, Bk, KhT); project(V, Wv, Bv, VhT);
    GPUTensor att({B * H, T, d}, nullptr, gpu), wts({B * H, T, T}, nullptr, gpu), attT({B, T, H, d}, nullptr, gpu), y2({B, T, E}, nullptr, gpu);
    ScaledDotProductAttentionLayer::ScaledDotProductAttentionForwardPropagation(QhT, KhT, VhT, att, wts, true, true);
    att.Reshape({B, H, T, d}).TransposeSecondAndThirdDimension(attT);
    GPUTensor attT3 = attT.Reshape({B, T, E});
    Linear::DenseForwardPropagation(y2, attT3, Wo, &Bo, true);
    auto a = y.ContentAsFloatArray(), b2 = y2.ContentAsFloatArray();
    for (size_t i = 0; i < a.size(); ++i) EXPECT(std::fabs(a[i] - b2[i]) < 3e-5, "multi-head attention output at %zu: %f against %f", i, a[i], b2[i]);
    // backward
    GPUTensor dWq({E, E}, nullptr, gpu), dWk({E, E}, nullptr, gpu), dWv({E, E}, nullptr, gpu), dWo({E, E}, nullptr, gpu);
    GPUTensor dBq({E}, nullptr, gpu), dBk({E}, nullptr, gpu), dBv({E}, nullptr, gpu), dBo({E}, nullptr, gpu);
    GPUTensor dQ({B, T, E}, nullptr, gpu), dK({B, T, E}, nullptr, gpu), dV({B, T, E}, nullptr, gpu);
    const MultiheadAttention::Gradients grads = {&dWq, &dWk, &dWv, &dWo, &dBq, &dBk, &dBv, &dBo};
    mha.BackwardPropagation(Q, K, V, DY, params, 1.0f, grads, dQ, dK, dV);
    GPUTensor dAttT({B, T, E}, nullptr, gpu), dWo2({E, E}, nullptr, gpu), dBo2({E}, nullptr, gpu);
    Linear::DenseBackwardPropagation(&dAttT, dWo2, &dBo2, attT3, DY, Wo, 1.0f, false, true);
    GPUTensor dAtt({B, H, T, d}, nullptr, gpu);
    dAttT.Reshape({B, T, H, d}).TransposeSecondAndThirdDimension(dAtt);
    GPUTensor dAtt3 = dAtt.Reshape({B * H, T, d});
    GPUTensor dQh({B * H, T, d}, nullptr, gpu), dKh({B * H, T, d}, nullptr, gpu), dVh({B * H, T, d}, nullptr, gpu), scratch({B * H, T, T}, nullptr, gpu);
    ScaledDotProductAttentionLayer::ScaledDotProductAttentionBackwardPropagation(dQh, dKh, dVh, QhT, KhT, VhT, dAtt3, wts, scratch, true);
    auto unproject = [&](const GPUTensor& dheads, const GPUTensor& x, const GPUTensor& W, GPUTensor& dx, GPUTensor& dW, GPUTensor& db) {
      GPUTensor merged({B, T, H, d}, nullptr, gpu);
      dheads.Reshape({B, H, T, d}).TransposeSecondAndThirdDimension(merged);
      GPUTensor merged3 = merged.Reshape({B, T, E});
      Linear::DenseBackwardPropagation(&dx, dW, &db, x, merged3, W, 1.0f, false, true);
    };
    GPUTensor dQ2({B, T, E}, nullptr, gpu), dK2({B, T, E}, nullptr, gpu), dV2({B, T, E}, nullptr, gpu);
    GPUTensor dWq2({E, E}, nullptr, gpu), dWk2({E, E}, nullptr, gpu), dWv2({E, E}, nullptr, gpu), dBq2({E}, nullptr, gpu), dBk2({E}, nullptr, gpu), dBv2({E}, nullptr, gpu);
    unproject(dQh, Q, Wq, dQ2, dWq2, dBq2); unproject(dKh, K, Wk, dK2, dWk2, dBk2); unproject(dVh, V, Wv, dV2, dWv2, dBv2);
    auto close = [&](const GPUTensor& x1, const GPUTensor& x2, double tol, const char* what) {
      auto u = x1.ContentAsFloatArray(), w2 = x2.ContentAsFloatArray();
      for (size_t i = 0; i < u.size(); ++i) EXPECT(std::fabs(u[i] - w2[i]) < tol, "%s at %zu: %f against %f", what, i, u[i], w2[i]);
    };
    close(dQ, dQ2, 5e-5, "dQ"); close(dK, dK2, 5e-5, "dK"); close(dV, dV2, 5e-5, "dV");
    close(dWq, dWq2, 2e-4, "dW_Q"); close(dWk, dWk2, 2e-4, "dW_K"); close(dWv, dWv2, 2e-4, "dW_V"); close(dWo, dWo2, 2e-4, "dW_O");
    close(dBq, dBq2, 2e-4, "db_Q"); close(dBo, dBo2, 2e-4, "db_O");
  }
  {  // loss gradients (Prod/Data/Tensor.cs:1182-1217) and the mini-batch staging of Network.cs:1211-1258:
     // three steps, double buffered, each step's input copied from pinned host memory while the step before runs
    const int rows = 50, cols = 7;
    auto t = uniform(rows * cols, 0, 1, 120), pr = uniform(rows * cols, 0, 1, 121);
    GPUTensor Tt({rows, cols}, t.data(), gpu), P({rows, cols}, pr.data(), gpu), D({rows, cols}, nullptr, gpu);
    D.ComputeGradientForEvaluationMetric(Tt, P, EvaluationMetricEnum::CategoricalCrossentropy);
    auto dv = D.ContentAsFloatArray();
    for (int i = 0; i < rows * cols; ++i) EXPECT(dv[i] == pr[i] - t[i], "categorical cross-entropy gradient at %d", i);
    D.ComputeGradientForEvaluationMetric(Tt, P, EvaluationMetricEnum::Mse);
    dv = D.ContentAsFloatArray();
    for (int i = 0; i < rows * cols; ++i) EXPECT(std::fabs(dv[i] - 2.0f * (pr[i] - t[i]) / cols) < 1e-7, "Mse gradient at %d", i);
    D.ComputeGradientForEvaluationMetric(Tt, P, EvaluationMetricEnum::BinaryCrossentropy);
    dv = D.ContentAsFloatArray();
    for (int i = 0; i < rows * cols; ++i) EXPECT(std::fabs(dv[i] - (pr[i] - t[i]) / cols) < 1e-7, "binary cross-entropy gradient at %d", i);

    const int M = 512, Kd = 64, N = 32, steps = 3;
    std::vector<std::vector<float>> batches;
    for (int i = 0; i < steps; ++i) batches.push_back(uniform(M * Kd, -1, 1, 130 + i));
    std::vector<std::unique_ptr<HostPinnedMemory>> pins;
    for (auto& bt : batches) pins.emplace_back(new HostPinnedMemory(bt.data(), static_cast<long long>(sizeof(float)) * bt.size()));
    auto wv = uniform(Kd * N, -1, 1, 140);
    GPUTensor Wm({Kd, N}, wv.data(), gpu);
    GPUTensor x0({M, Kd}, nullptr, gpu), x1({M, Kd}, nullptr, gpu);
    GPUTensor* slot_x[2] = {&x0, &x1};
    std::vector<std::unique_ptr<GPUTensor>> outs;
    for (int i = 0; i < steps; ++i) outs.emplace_back(new GPUTensor({M, N}, nullptr, gpu));
    MiniBatchStager stager(gpu, 2);
    stager.Issue(0, {{slot_x[0], batches[0].data()}});
    for (int i = 0; i < steps; ++i) {
      if (i + 1 < steps) stager.Issue((i + 1) % 2, {{slot_x[(i + 1) % 2], batches[i + 1].data()}});
      stager.Acquire(i % 2);
      outs[i]->Dot(*slot_x[i % 2], false, Wm, false, 1.0f, 0.0f);
      stager.Release(i % 2);
    }
    std::vector<float> zeros(M * N, 0.0f);
    for (int i = 0; i < steps; ++i)
      EXPECT(max_abs_diff(outs[i]->ContentAsFloatArray(), ref_gemm(batches[i], M, Kd, false, wv, Kd, N, false, zeros, 1.0, 0.0)) / 8.0 < 1e-5,
             "staged step %d", i);
  }
  {  // the gradient sum over the replicas of one process; with the one GPU this program drives the sum is the
     // buffer itself (the two-GPU form runs in the Python suite, one thread per GPU)
    auto gw = uniform(1000, -1, 1, 150), gb = uniform(10, -1, 1, 151);
    GPUTensor GW({100, 10}, gw.data(), gpu), GB({10}, gb.data(), gpu);
    std::unique_ptr<GradientCommunicator> comm;
    try {
      comm.reset(new GradientCommunicator({&gpu}));
    } catch (const std::runtime_error& e) {   // status 15: no NCCL library on this machine, the one accepted reason
      EXPECT(std::string(e.what()).find("status 15") != std::string::npos, "communicator: %s", e.what());
    }
    if (comm) {
      GradientCommunicator::AllReduceSum(GW);
      GradientCommunicator::AllReduceSum(GW, GB);
      auto r = GW.ContentAsFloatArray(), rb = GB.ContentAsFloatArray();
      for (size_t i = 0; i < r.size(); ++i) EXPECT(r[i] == gw[i], "all-reduce over one replica at %zu", i);
      for (size_t i = 0; i < rb.size(); ++i) EXPECT(rb[i] == gb[i], "grouped all-reduce over one replica at %zu", i);
    }
  }
  {  // errors surface as exceptions, like GPUWrapper.CheckStatus
    GPUTensor A({4, 3}, nullptr, gpu), B({5, 4}, nullptr, gpu), C({4, 4}, nullptr, gpu);
    bool thrown = false;
    try { C.Dot(A, false, B, false, 1, 0); } catch (const std::runtime_error&) { thrown = true; }
    EXPECT(thrown, "mismatched inner dimensions must throw");
  }
  std::printf("OK %d checks\n", g_checks);
  return 0;
}
