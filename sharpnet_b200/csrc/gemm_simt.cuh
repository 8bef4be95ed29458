// fp32 FMA GEMM on the CUDA cores.  It takes every shape, transposition, pitch and 4-byte
// aligned pointer, so it serves the shapes the tensor-core path cannot be fed with (tiny or
// odd-sized matrices, pointers or pitches that are not 16-byte multiples) and the
// SNB200_MATH_FP32_SIMT mode.  Same fused epilogue as the tcgen05 kernel.
#pragma once
#include "common.cuh"

namespace snb {

constexpr int kSimtBM = 64, kSimtBN = 64, kSimtBK = 16, kSimtThreads = 256;

struct SimtParams {
  int M, N, K, batch;
  // element strides of the logical operands: A(m,k) = A[m*sAm + k*sAk], B(k,n) = B[k*sBk + n*sBn]
  long long sAm, sAk, sBk, sBn;
  long long strideA, strideB, strideC;
  int ldc;
  const float* A;
  const float* B;
  float* C;
  float* Z;
  const float* bias;
  float alpha, beta;
  int act;
  int tiles_m, tiles_n;
};

__global__ void __launch_bounds__(kSimtThreads)
simt_gemm_kernel(const SimtParams p) {
  __shared__ float As[kSimtBK][kSimtBM + 4];
  __shared__ float Bs[kSimtBK][kSimtBN + 4];
  const int tid = threadIdx.x;
  const int tiles = p.tiles_m * p.tiles_n;
  const int b = blockIdx.x / tiles;
  const int r = blockIdx.x - b * tiles;
  const int m0 = (r % p.tiles_m) * kSimtBM;
  const int n0 = (r / p.tiles_m) * kSimtBN;
  const float* A = p.A + b * p.strideA;
  const float* B = p.B + b * p.strideB;
  const int ty = tid >> 4, tx = tid & 15;  // 16 x 16 threads, 4 x 4 outputs each

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  const bool a_k_contig = (p.sAk == 1);
  const bool b_n_contig = (p.sBn == 1);

  for (int k0 = 0; k0 < p.K; k0 += kSimtBK) {
    // Global -> shared; the thread mapping follows whichever dimension is contiguous in memory.
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int m, k;
      if (a_k_contig) { k = tid & 15; m = (tid >> 4) + 16 * i; }
      else            { m = tid & 63; k = (tid >> 6) + 4 * i; }
      const int gm = m0 + m, gk = k0 + k;
      As[k][m] = (gm < p.M && gk < p.K) ? __ldg(A + gm * p.sAm + gk * p.sAk) : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int n, k;
      if (b_n_contig) { n = tid & 63; k = (tid >> 6) + 4 * i; }
      else            { k = tid & 15; n = (tid >> 4) + 16 * i; }
      const int gn = n0 + n, gk = k0 + k;
      Bs[k][n] = (gn < p.N && gk < p.K) ? __ldg(B + gk * p.sBk + gn * p.sBn) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kSimtBK; ++k) {
      const float4 a4 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 b4 = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
      const float a[4] = {a4.x, a4.y, a4.z, a4.w};
      const float bb[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = m0 + ty * 4 + i;
    if (row >= p.M) continue;
    const size_t off = static_cast<size_t>(b) * p.strideC + static_cast<size_t>(row) * p.ldc;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = n0 + tx * 4 + j;
      if (col >= p.N) continue;
      float o = p.alpha * acc[i][j];
      if (p.beta != 0.0f) o = fmaf(p.beta, p.C[off + col], o);
      if (p.bias) o += __ldg(p.bias + col);
      if (p.Z) p.Z[off + col] = o;
      p.C[off + col] = act_forward(p.act, o);
    }
  }
}

}  // namespace snb
