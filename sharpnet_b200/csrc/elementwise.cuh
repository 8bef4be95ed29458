// Bandwidth-bound companions of the Dense layer: bias broadcast, column sums (bias gradient),
// activations and their gradients, axpy, and the fused "activation gradient + bias gradient"
// pass of the Dense backward.  All are grid-stride / slab kernels sized from the SM count.
#pragma once
#include "common.cuh"

namespace snb {

// y[m, n] += bias[n]                               (Prod/CPU/CpuTensor.cs:1468-1487)
static __global__ void bias_add_kernel(long long total, int N, const float* __restrict__ bias, float* __restrict__ y) {
  pdl_prologue();
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += stride)
    y[i] += __ldg(bias + (i % N));
}
static __global__ void bias_add_vec4_kernel(long long total4, int N4, const float4* __restrict__ bias,
                                     float4* __restrict__ y) {
  pdl_prologue();
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total4; i += stride) {
    float4 v = y[i];
    const float4 b = __ldg(bias + (i % N4));
    v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
    y[i] = v;
  }
}

// Element-wise kernels: grid-stride over 16-byte vectors when every pointer is 16-byte aligned
// (VEC = 4), scalar otherwise (VEC = 1); the last n % 4 elements of the vector form are done one by one.
// Copy of `cols` columns of a row-major fp32 matrix (row pitch src_pitch) whose base is only 4-byte aligned, or whose
// pitch is not a multiple of 4 floats, into a 16-byte aligned buffer with a row pitch that is a multiple of 4
// floats: what TMA needs.  One thread per four consecutive destination floats (one 16-byte store); the four source
// floats are separate 4-byte loads, coalesced across the warp.  The padding columns are written as zeros.
static __global__ void realign_rows_kernel(const float* __restrict__ src, float* __restrict__ dst, long long rows_total,
                                           int cols, int src_pitch, int dst_pitch) {
  pdl_prologue();
  const int quads = dst_pitch >> 2;
  const long long total = rows_total * quads;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += stride) {
    const long long row = i / quads;
    const int c = static_cast<int>(i - row * quads) << 2;
    const float* s0 = src + row * src_pitch + c;
    float4 v;
    v.x = c < cols ? __ldg(s0) : 0.0f;
    v.y = c + 1 < cols ? __ldg(s0 + 1) : 0.0f;
    v.z = c + 2 < cols ? __ldg(s0 + 2) : 0.0f;
    v.w = c + 3 < cols ? __ldg(s0 + 3) : 0.0f;
    *reinterpret_cast<float4*>(dst + row * dst_pitch + c) = v;
  }
}

template <int VEC> struct Pack;
template <> struct Pack<4> { typedef float4 type; };
template <> struct Pack<1> { typedef float type; };
__device__ __forceinline__ float lane_get(const float4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }
__device__ __forceinline__ float lane_get(const float& v, int) { return v; }
__device__ __forceinline__ void lane_set(float4& v, int i, float x) { if (i == 0) v.x = x; else if (i == 1) v.y = x; else if (i == 2) v.z = x; else v.w = x; }
__device__ __forceinline__ void lane_set(float& v, int, float x) { v = x; }

template <int VEC>
static __global__ void activation_fwd_kernel(int act, float act_alpha, long long n, const float* __restrict__ x,
                                             float* __restrict__ y) {
  pdl_prologue();
  typedef typename Pack<VEC>::type P;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nv = n / VEC;
  for (long long i = tid; i < nv; i += stride) {
    const P xv = reinterpret_cast<const P*>(x)[i];
    P yv;
#pragma unroll
    for (int k = 0; k < VEC; ++k) lane_set(yv, k, act_forward(act, lane_get(xv, k), act_alpha));
    reinterpret_cast<P*>(y)[i] = yv;
  }
  for (long long i = nv * VEC + tid; i < n; i += stride) y[i] = act_forward(act, x[i], act_alpha);
}
template <int VEC>
static __global__ void activation_bwd_kernel(int act, float act_alpha, long long n, const float* __restrict__ dy, const float* __restrict__ x,
                                             const float* __restrict__ y, float* __restrict__ dx) {
  pdl_prologue();
  typedef typename Pack<VEC>::type P;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nv = n / VEC;
  const bool need_x = act_needs_input(act), need_y = (act != ACT_IDENTITY);
  for (long long i = tid; i < nv; i += stride) {
    const P g = reinterpret_cast<const P*>(dy)[i];
    P xv = P(), yv = P(), o;
    if (need_x) xv = reinterpret_cast<const P*>(x)[i];
    if (need_y) yv = reinterpret_cast<const P*>(y)[i];
#pragma unroll
    for (int k = 0; k < VEC; ++k) lane_set(o, k, act_backward(act, lane_get(g, k), lane_get(xv, k), lane_get(yv, k), act_alpha));
    reinterpret_cast<P*>(dx)[i] = o;
  }
  for (long long i = nv * VEC + tid; i < n; i += stride)
    dx[i] = act_backward(act, dy[i], need_x ? x[i] : 0.0f, need_y ? y[i] : 0.0f, act_alpha);
}
// y += alpha * x                                    (Prod/CPU/CpuTensor.cs:1032-1038)
template <int VEC>
static __global__ void axpy_kernel(long long n, float alpha, const float* __restrict__ x, float* __restrict__ y) {
  pdl_prologue();
  typedef typename Pack<VEC>::type P;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nv = n / VEC;
  for (long long i = tid; i < nv; i += stride) {
    const P xv = reinterpret_cast<const P*>(x)[i];
    P yv = reinterpret_cast<P*>(y)[i];
#pragma unroll
    for (int k = 0; k < VEC; ++k) lane_set(yv, k, fmaf(alpha, lane_get(xv, k), lane_get(yv, k)));
    reinterpret_cast<P*>(y)[i] = yv;
  }
  for (long long i = nv * VEC + tid; i < n; i += stride) y[i] = fmaf(alpha, x[i], y[i]);
}

// dst[a, c, b, :] = src[a, b, c, :] for src [A, B, C, D]: the head split / merge of multi-head attention
// (Prod/CPU/CpuTensor.cs:301-322, Prod/GPU/GpuTensor.cs:672-684).  One thread per VEC consecutive floats
// of a D-run, enumerated in destination order so that writes are fully coalesced; reads are D-long runs.
template <int VEC>
static __global__ void transpose_second_third_kernel(long long total_vec, int B, int C, int Dv,
                                                     const float* __restrict__ src, float* __restrict__ dst) {
  pdl_prologue();
  typedef typename Pack<VEC>::type P;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total_vec; i += stride) {
    const int d = static_cast<int>(i % Dv);
    long long r = i / Dv;                       // destination row index (a, c, b)
    const int b = static_cast<int>(r % B);
    r /= B;
    const int c = static_cast<int>(r % C);
    const long long a = r / C;
    const long long s = ((a * B + b) * C + c) * Dv + d;
    reinterpret_cast<P*>(dst)[i] = reinterpret_cast<const P*>(src)[s];
  }
}

// Column sums of g[M x N] over a slab of rows, optionally fused with the activation gradient:
//   g = dy                        (FUSE_ACT = false:  db = sum_m dy,  CpuTensor.cs:3343-3362)
//   g = act'(z, y) * dy -> dz     (FUSE_ACT = true:   ActivationBackward + bias gradient in one pass)
//   g = scale * (p - t)  -> dz     (FUSE_ACT = true, act = ACT_LOSS_DIFF: loss gradient + bias gradient in one pass)
// Block = 256 threads = 8 warps; a warp covers 32*VEC consecutive columns, the 8 warps stride over
// the rows of the slab.  The slab's sums go to partial[slab, N] (or straight to db when there is
// one slab); colsum_finish_kernel adds the slabs in a fixed order, so results are deterministic.
template <int VEC, bool FUSE_ACT>
__global__ void __launch_bounds__(256)
colsum_slab_kernel(int M, int N, int rows_per_slab, int act, const float* __restrict__ dy,
                   const float* __restrict__ y, const float* __restrict__ z, float* __restrict__ dz,
                   float* __restrict__ out, float scale = 1.0f, float act_alpha = 0.0f) {
  pdl_prologue();
  __shared__ float red[8][32 * VEC];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = (blockIdx.x * 32 + lane) * VEC;
  const int r0 = blockIdx.y * rows_per_slab;
  const int r1 = min(M, r0 + rows_per_slab);
  float s[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) s[v] = 0.0f;
  if (col < N) {
    for (int r = r0 + warp; r < r1; r += 8) {
      const size_t off = static_cast<size_t>(r) * N + col;
      float g[VEC], yv[VEC], zv[VEC];
      if (VEC == 4) {
        const float4 t = *reinterpret_cast<const float4*>(dy + off);
        g[0] = t.x; g[1] = t.y; g[2] = t.z; g[3] = t.w;
      } else {
        g[0] = dy[off];
      }
      if (FUSE_ACT) {
        if (VEC == 4) {
          const float4 t = *reinterpret_cast<const float4*>(y + off);
          yv[0] = t.x; yv[1] = t.y; yv[2] = t.z; yv[3] = t.w;
          if (act_needs_input(act)) {
            const float4 u = *reinterpret_cast<const float4*>(z + off);
            zv[0] = u.x; zv[1] = u.y; zv[2] = u.z; zv[3] = u.w;
          }
        } else {
          yv[0] = y[off];
          if (act_needs_input(act)) zv[0] = z[off];
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v)
          g[v] = (act == ACT_LOSS_DIFF) ? scale * (g[v] - yv[v])      // dy = yPredicted, y = yExpected
                                        : act_backward(act, g[v], act_needs_input(act) ? zv[v] : 0.0f, yv[v], act_alpha);
        if (VEC == 4) {
          *reinterpret_cast<float4*>(dz + off) = make_float4(g[0], g[1], g[2], g[3]);
        } else {
          dz[off] = g[0];
        }
      }
#pragma unroll
      for (int v = 0; v < VEC; ++v) s[v] += g[v];
    }
  }
  if (out == nullptr) return;   // caller only wanted dz
#pragma unroll
  for (int v = 0; v < VEC; ++v) red[warp][lane * VEC + v] = s[v];
  __syncthreads();
  if (warp == 0 && col < N) {
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      float t = 0.0f;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += red[w][lane * VEC + v];
      out[static_cast<size_t>(blockIdx.y) * N + col + v] = t;
    }
  }
}

static __global__ void colsum_finish_kernel(int N, int slabs, const float* __restrict__ partial, float* __restrict__ db) {
  pdl_prologue();
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= N) return;
  float t = 0.0f;
  for (int s = 0; s < slabs; ++s) t += partial[static_cast<size_t>(s) * N + col];
  db[col] = t;
}

// dy = scale * (yPredicted - yExpected)
template <int VEC>
static __global__ void loss_gradient_kernel(long long n, float scale, const float* __restrict__ expected,
                                            const float* __restrict__ predicted, float* __restrict__ dy) {
  pdl_prologue();
  typedef typename Pack<VEC>::type P;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nv = n / VEC;
  for (long long i = tid; i < nv; i += stride) {
    const P e = reinterpret_cast<const P*>(expected)[i], p = reinterpret_cast<const P*>(predicted)[i];
    P o;
#pragma unroll
    for (int k = 0; k < VEC; ++k) lane_set(o, k, scale * (lane_get(p, k) - lane_get(e, k)));
    reinterpret_cast<P*>(dy)[i] = o;
  }
  for (long long i = nv * VEC + tid; i < n; i += stride) dy[i] = scale * (predicted[i] - expected[i]);
}

// ---------------------------------------------------------------- row softmax (attention weights)
// y[r, :] = softmax(x[r, :]) over the last dimension, one warp per row; `causal_rows` > 0 masks the
// columns above the main diagonal of every [causal_rows x cols] matrix first, i.e. the -1e12 overwrite of
// Tensor.SetAllElementsAboveMainDiagonal (Prod/CPU/CpuTensor.cs:3037-3052) that
// ScaledDotProductAttentionLayer applies before the softmax (Prod/Layers/ScaledDotProductAttentionLayer.cs:73-81),
// folded into the same pass.  Formula of CpuTensorActivationFunctions.Softmax (Prod/CPU/CpuTensorActivationFunctions.cs:19-46).
// x may equal y.  Rows of up to 1024 columns stay in registers; longer rows are re-read.
template <int PER_LANE>
static __global__ void __launch_bounds__(256)
softmax_fwd_kernel(long long rows, int cols, int causal_rows, const float* x, float* y) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long n_warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long r = warp; r < rows; r += n_warps) {
    const float* xr = x + r * cols;
    float* yr = y + r * cols;
    const int limit = causal_rows > 0 ? static_cast<int>(r % causal_rows) : cols;   // columns > limit are masked
    float v[PER_LANE > 0 ? PER_LANE : 1];
    float mx = -3.402823466e38f;
    if (PER_LANE > 0) {
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i) {
        const int c = lane + 32 * i;
        v[i] = (c < cols) ? ((c > limit) ? -1e12f : xr[c]) : -3.402823466e38f;
        mx = fmaxf(mx, v[i]);
      }
    } else {
      for (int c = lane; c < cols; c += 32) mx = fmaxf(mx, (c > limit) ? -1e12f : xr[c]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.0f;
    if (PER_LANE > 0) {
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i) {
        const int c = lane + 32 * i;
        v[i] = (c < cols) ? expf(v[i] - mx) : 0.0f;
        sum += v[i];
      }
    } else {
      for (int c = lane; c < cols; c += 32) sum += expf(((c > limit) ? -1e12f : xr[c]) - mx);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (PER_LANE > 0) {
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i) {
        const int c = lane + 32 * i;
        if (c < cols) yr[c] = v[i] / sum;
      }
    } else {
      for (int c = lane; c < cols; c += 32) yr[c] = expf(((c > limit) ? -1e12f : xr[c]) - mx) / sum;
    }
  }
}

// The same for short rows (up to 32 * PER_LANE columns), R rows per warp at a time: with one 512-byte row in flight
// per warp the kernel is bound by memory latency (0.69 of the HBM rate at 128 columns); R independent rows give every
// lane R * PER_LANE loads in flight.  Per row the arithmetic and its order are those of the kernel above.
template <int PER_LANE, int R>
static __global__ void __launch_bounds__(256)
softmax_fwd_rows_kernel(long long rows, int cols, int causal_rows, const float* x, float* y) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long n_warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long r0 = warp * R; r0 < rows; r0 += n_warps * R) {
    float v[R][PER_LANE];
    float mx[R], sum[R];
#pragma unroll
    for (int q = 0; q < R; ++q) {
      const long long r = r0 + q;
      const bool live = r < rows;
      const float* xr = x + (live ? r : r0) * cols;
      const int limit = causal_rows > 0 ? static_cast<int>((live ? r : r0) % causal_rows) : cols;
      mx[q] = -3.402823466e38f;
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i) {
        const int c = lane + 32 * i;
        v[q][i] = (c < cols) ? ((c > limit) ? -1e12f : xr[c]) : -3.402823466e38f;
        mx[q] = fmaxf(mx[q], v[q][i]);
      }
    }
#pragma unroll
    for (int q = 0; q < R; ++q) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx[q] = fmaxf(mx[q], __shfl_xor_sync(0xffffffffu, mx[q], o));
      sum[q] = 0.0f;
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i) {
        const int c = lane + 32 * i;
        v[q][i] = (c < cols) ? expf(v[q][i] - mx[q]) : 0.0f;
        sum[q] += v[q][i];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum[q] += __shfl_xor_sync(0xffffffffu, sum[q], o);
    }
#pragma unroll
    for (int q = 0; q < R; ++q) {
      const long long r = r0 + q;
      if (r < rows) {
        float* yr = y + r * cols;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
          const int c = lane + 32 * i;
          if (c < cols) yr[c] = v[q][i] / sum[q];
        }
      }
    }
  }
}

// dx[r, :] = y[r, :] * (dy[r, :] - sum_j dy[r, j] * y[r, j]): the softmax Jacobian that
// cudnnSoftmaxBackward applies on SharpNet's GPU path (Prod/GPU/GpuTensor.cs:445-490).  dx may equal dy.
static __global__ void __launch_bounds__(256)
softmax_bwd_kernel(long long rows, int cols, const float* dy, const float* __restrict__ y, float* dx) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long n_warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long r = warp; r < rows; r += n_warps) {
    const float* gr = dy + r * cols;
    const float* yr = y + r * cols;
    float* dr = dx + r * cols;
    float dot = 0.0f;
    for (int c = lane; c < cols; c += 32) dot = fmaf(gr[c], yr[c], dot);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    for (int c = lane; c < cols; c += 32) dr[c] = yr[c] * (gr[c] - dot);
  }
}

// ---------------------------------------------------------------- optimizer updates
// One pass each over the parameter tensors; SharpNet's GPU path makes two or three
// (cudnnAddTensor + axpy, Prod/GPU/GpuTensor.cs:1147-1161) or launches an NVRTC kernel
// (UpdateAdamOptimizer, Prod/GPU/Kernels/SinglePrecision.cu:19-28).

// velocity = momentum * velocity - lr * dW ;  W += nesterov ? momentum * velocity - lr * dW : velocity
// (Prod/CPU/CpuTensor.cs:470-489).  velocity == nullptr: plain W -= lr * dW (Prod/Optimizers/VanillaSgd.cs:18-20).
__device__ __forceinline__ void sgd_one(float lr, float momentum, int nesterov, bool has_v, float g, float& w, float& v) {
  if (!has_v) { w = fmaf(-lr, g, w); return; }
  v = momentum * v - g * lr;
  w += nesterov ? (momentum * v - g * lr) : v;
}
template <int VEC>
static __global__ void sgd_update_kernel(long long n, float lr, float momentum, int nesterov,
                                         const float* __restrict__ dW, float* __restrict__ W,
                                         float* __restrict__ velocity) {
  pdl_prologue();
  typedef typename Pack<VEC>::type P;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nv = n / VEC;
  const bool has_v = velocity != nullptr;
  for (long long i = tid; i < nv; i += stride) {
    const P g = reinterpret_cast<const P*>(dW)[i];
    P w = reinterpret_cast<P*>(W)[i];
    P v = P();
    if (has_v) v = reinterpret_cast<P*>(velocity)[i];
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      float wk = lane_get(w, k), vk = lane_get(v, k);
      sgd_one(lr, momentum, nesterov, has_v, lane_get(g, k), wk, vk);
      lane_set(w, k, wk); lane_set(v, k, vk);
    }
    reinterpret_cast<P*>(W)[i] = w;
    if (has_v) reinterpret_cast<P*>(velocity)[i] = v;
  }
  for (long long i = nv * VEC + tid; i < n; i += stride) {
    float wk = W[i], vk = has_v ? velocity[i] : 0.0f;
    sgd_one(lr, momentum, nesterov, has_v, dW[i], wk, vk);
    W[i] = wk;
    if (has_v) velocity[i] = vk;
  }
}

// v = beta1 v + (1 - beta1) dW ; s = beta2 s + (1 - beta2) dW^2 ;
// W -= factor * v / (sqrt(s) + eps) + weight_decay * W, factor = lr * sqrt(1 - beta2^t) / (1 - beta1^t) computed
// by the host in double (Prod/GPU/GpuTensor.cs:1136-1145, Prod/CPU/CpuTensor.cs:1755-1769).
__device__ __forceinline__ void adam_one(float beta1, float beta2, float eps, float wd, float factor, float g, float& w,
                                         float& v, float& s) {
  v = beta1 * v + (1.0f - beta1) * g;
  s = beta2 * s + (1.0f - beta2) * g * g;
  w = w - ((factor * v) / (sqrtf(s) + eps) + wd * w);
}
template <int VEC>
static __global__ void adam_update_kernel(long long n, float beta1, float beta2, float eps, float weight_decay,
                                          float factor, const float* __restrict__ dW, float* __restrict__ W,
                                          float* __restrict__ vW, float* __restrict__ sW) {
  pdl_prologue();
  typedef typename Pack<VEC>::type P;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nv = n / VEC;
  for (long long i = tid; i < nv; i += stride) {
    const P g = reinterpret_cast<const P*>(dW)[i];
    P w = reinterpret_cast<P*>(W)[i], v = reinterpret_cast<P*>(vW)[i], s = reinterpret_cast<P*>(sW)[i];
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      float wk = lane_get(w, k), vk = lane_get(v, k), sk = lane_get(s, k);
      adam_one(beta1, beta2, eps, weight_decay, factor, lane_get(g, k), wk, vk, sk);
      lane_set(w, k, wk); lane_set(v, k, vk); lane_set(s, k, sk);
    }
    reinterpret_cast<P*>(W)[i] = w;
    reinterpret_cast<P*>(vW)[i] = v;
    reinterpret_cast<P*>(sW)[i] = s;
  }
  for (long long i = nv * VEC + tid; i < n; i += stride) {
    float wk = W[i], vk = vW[i], sk = sW[i];
    adam_one(beta1, beta2, eps, weight_decay, factor, dW[i], wk, vk, sk);
    W[i] = wk; vW[i] = vk; sW[i] = sk;
  }
}

}  // namespace snb
