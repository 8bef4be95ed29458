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
  float act_alpha;
  int tiles_m, tiles_n;
  OutMap omap;
};

__global__ void __launch_bounds__(kSimtThreads)
simt_gemm_kernel(const SimtParams p) {
  pdl_prologue();
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

  // Result placement: the column part of the address once per column, the row part once per row (with a mapped
  // result each is an integer division, too long to repeat for every element of the unrolled loops).
  long long cpart[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int col = n0 + tx * 4 + j;
    cpart[j] = col;
    if (p.omap.on) cpart[j] = static_cast<long long>(col / p.omap.d) * p.omap.s_co + (col % p.omap.d);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = m0 + ty * 4 + i;
    if (row >= p.M) continue;
    long long rpart = static_cast<long long>(b) * p.strideC + static_cast<long long>(row) * p.ldc;
    if (p.omap.on)
      rpart = static_cast<long long>(b / p.omap.H) * p.omap.s_io + static_cast<long long>(b % p.omap.H) * p.omap.s_ii +
              static_cast<long long>(row / p.omap.T) * p.omap.s_ro + static_cast<long long>(row % p.omap.T) * p.omap.s_ri;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = n0 + tx * 4 + j;
      if (col >= p.N) continue;
      const long long off = rpart + cpart[j];
      float o = p.alpha * acc[i][j];
      if (p.beta != 0.0f) o = fmaf(p.beta, p.C[off], o);
      if (p.bias) o += __ldg(p.bias + col);
      if (p.Z) p.Z[off] = o;
      p.C[off] = act_forward_compact(p.act, o, p.act_alpha);
    }
  }
}

// The same product for problems large enough to fill the SMs with 128 x 128 tiles: 256 threads, 8 x 8 outputs per
// thread (two 4-wide groups 64 apart in each direction, so that shared-memory reads are conflict free), 8-deep K
// slices double buffered in shared memory with the next slice prefetched into registers while the current one is
// multiplied.  Same operand generality (any strides, any 4-byte aligned pointer) and the same epilogue.
constexpr int kSimtBigBM = 128, kSimtBigBN = 128, kSimtBigBK = 8;

__global__ void __launch_bounds__(kSimtThreads, 2)
simt_gemm_big_kernel(const SimtParams p) {
  pdl_prologue();
  __shared__ float As[2][kSimtBigBK][kSimtBigBM + 4];
  __shared__ float Bs[2][kSimtBigBK][kSimtBigBN + 4];
  const int tid = threadIdx.x;
  const int tiles = p.tiles_m * p.tiles_n;
  const int b = blockIdx.x / tiles;
  const int r = blockIdx.x - b * tiles;
  const int m0 = (r % p.tiles_m) * kSimtBigBM;
  const int n0 = (r / p.tiles_m) * kSimtBigBN;
  const float* A = p.A + b * p.strideA;
  const float* B = p.B + b * p.strideB;
  const int ty = tid >> 4, tx = tid & 15;

  // Each thread moves 4 elements of A and 4 of B per slice; the mapping follows the contiguous dimension.
  const bool a_k_contig = (p.sAk == 1);
  const bool b_n_contig = (p.sBn == 1);
  int am[4], ak[4], bn[4], bk[4];
  const float* ap[4];
  const float* bp[4];
  bool a_ok[4], b_ok[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (a_k_contig) { ak[i] = tid & 7; am[i] = (tid >> 3) + 32 * i; }
    else            { am[i] = tid & 127; ak[i] = (tid >> 7) + 2 * i; }
    if (b_n_contig) { bn[i] = tid & 127; bk[i] = (tid >> 7) + 2 * i; }
    else            { bk[i] = tid & 7; bn[i] = (tid >> 3) + 32 * i; }
    a_ok[i] = (m0 + am[i]) < p.M;
    b_ok[i] = (n0 + bn[i]) < p.N;
    ap[i] = A + static_cast<long long>(m0 + am[i]) * p.sAm + static_cast<long long>(ak[i]) * p.sAk;
    bp[i] = B + static_cast<long long>(bk[i]) * p.sBk + static_cast<long long>(n0 + bn[i]) * p.sBn;
  }
  const long long a_step = static_cast<long long>(kSimtBigBK) * p.sAk;
  const long long b_step = static_cast<long long>(kSimtBigBK) * p.sBk;

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

  float ra[4], rb[4];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      ra[i] = (a_ok[i] && k0 + ak[i] < p.K) ? __ldg(ap[i]) : 0.0f;
      rb[i] = (b_ok[i] && k0 + bk[i] < p.K) ? __ldg(bp[i]) : 0.0f;
      ap[i] += a_step;
      bp[i] += b_step;
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      As[buf][ak[i]][am[i]] = ra[i];
      Bs[buf][bk[i]][bn[i]] = rb[i];
    }
  };

  fetch(0);
  stash(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < p.K; k0 += kSimtBigBK) {
    const bool more = k0 + kSimtBigBK < p.K;
    if (more) fetch(k0 + kSimtBigBK);
#pragma unroll
    for (int k = 0; k < kSimtBigBK; ++k) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tx * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
    }
    if (more) {
      stash(buf ^ 1);       // the other buffer was last read before the previous barrier
      __syncthreads();
      buf ^= 1;
    }
  }

  long long cpart[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int col = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
    cpart[j] = col;
    if (p.omap.on) cpart[j] = static_cast<long long>(col / p.omap.d) * p.omap.s_co + (col % p.omap.d);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (row >= p.M) continue;
    long long rpart = static_cast<long long>(b) * p.strideC + static_cast<long long>(row) * p.ldc;
    if (p.omap.on)
      rpart = static_cast<long long>(b / p.omap.H) * p.omap.s_io + static_cast<long long>(b % p.omap.H) * p.omap.s_ii +
              static_cast<long long>(row / p.omap.T) * p.omap.s_ro + static_cast<long long>(row % p.omap.T) * p.omap.s_ri;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int col = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
      if (col >= p.N) continue;
      const long long off = rpart + cpart[j];
      float o = p.alpha * acc[i][j];
      if (p.beta != 0.0f) o = fmaf(p.beta, p.C[off], o);
      if (p.bias) o += __ldg(p.bias + col);
      if (p.Z) p.Z[off] = o;
      p.C[off] = act_forward_compact(p.act, o, p.act_alpha);
    }
  }
}

}  // namespace snb
