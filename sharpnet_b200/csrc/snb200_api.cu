// Host side of libsharpnet_b200: handle, argument validation, kernel selection and launch.
// Nothing in this file computes on the host; without a CUDA device every entry point fails.
#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/sharpnet_b200.h"
#include "elementwise.cuh"
#include "gemm_simt.cuh"
#include "gemm_umma.cuh"
#include "gemm_umma2.cuh"
#include "attention_umma.cuh"

using namespace snb;

// ------------------------------------------------------------------------------------ handle
enum { TUNE_FORCE_PATH = 0, TUNE_FORCE_BN = 1, TUNE_REWRITE_HI = 2, TUNE_CHUNK_K = 3, TUNE_PAIR = 4, TUNE_SPLITK = 5, TUNE_VARIANT = 6, TUNE_PDL = 7, TUNE_FORCE_SPLITS = 8, TUNE_NO_TS = 9, TUNE_NO_FUSED_ATTN = 10, TUNE_NO_SWLOAD = 11, TUNE_SM_RESERVE = 12, TUNE_CLUSTER = 13, TUNE_COUNT = 14 };

struct snb200_context {
  int device;
  int sm_count;
  cudaStream_t stream;
  int math_mode;
  int tune[TUNE_COUNT];
  float act_alpha;          // coefficient of ELU / LeakyRelu for the calls that follow (snb200_set_activation_parameter)
  float* workspace;            // partial sums of the column reductions
  size_t workspace_floats;
  int* error_word;             // device word set by a kernel whose pipeline wait timed out
  long long launches;
  char last_kernel[64];
  char last_error[256];
  void* nccl_comm;
  int realigning;              // inside the product of realigned operand copies (no second realignment)
  int time_gemms;              // snb200_gemm_timing_begin .. _end: an event pair around every GEMM
  cudaEvent_t* gemm_events;
  int gemm_events_used;        // events recorded so far (two per GEMM)
};
constexpr int kMaxTimedGemms = 4096;
// SMs the persistent tensor-core grids may use: all of them, minus the ones the caller keeps free for a concurrent
// kernel (a collective on another stream), rounded so that CTA pairs stay whole.
static int usable_sms(const snb200_context* h) {
  int r = h->tune[TUNE_SM_RESERVE];
  if (r < 0) r = 0;
  if (r > h->sm_count - 2) r = h->sm_count - 2;
  return h->sm_count - r;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode_tiled = nullptr;

static int fail(snb200_handle_t h, int status, const char* fmt, ...) {
  if (h) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(h->last_error, sizeof(h->last_error), fmt, ap);
    va_end(ap);
  }
  return status;
}
static int cuda_fail(snb200_handle_t h, cudaError_t e, const char* what) {
  return fail(h, SNB200_STATUS_EXECUTION_FAILED, "%s: %s", what, cudaGetErrorString(e));
}
#define SNB_CUDA(h, call)                                        \
  do {                                                           \
    cudaError_t e__ = (call);                                    \
    if (e__ != cudaSuccess) return cuda_fail((h), e__, #call);   \
  } while (0)

static int enter(snb200_handle_t h) {
  if (!h) return SNB200_STATUS_NOT_INITIALIZED;
  cudaError_t e = cudaSetDevice(h->device);
  if (e != cudaSuccess) return cuda_fail(h, e, "cudaSetDevice");
  return 0;
}
static void note_kernel(snb200_handle_t h, const char* name, int launches) {
  snprintf(h->last_kernel, sizeof(h->last_kernel), "%s", name);
  h->launches += launches;
}
static int check_launch(snb200_handle_t h, const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(h, e, what);
  return 0;
}

extern "C" int snb200_get_version(void) { return 100; }
#ifdef SNB_TRACE
// development builds only: the %globaltimer stamps CTA 0 of the last tensor-core kernel left behind
extern "C" int snb200_trace_read(snb200_handle_t h, unsigned long long* out32) {
  if (!h || !out32) return SNB200_STATUS_INVALID_VALUE;
  cudaSetDevice(h->device);
  cudaStreamSynchronize(h->stream);
  return cudaMemcpy(out32, h->workspace + (h->workspace_floats - 128), 512, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : 13;
}
#endif

extern "C" int snb200_create(snb200_handle_t* handle, int device_id) {
  if (!handle) return SNB200_STATUS_INVALID_VALUE;
  *handle = nullptr;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) return SNB200_STATUS_NOT_INITIALIZED;
  if (device_id < 0 || device_id >= n) return SNB200_STATUS_INVALID_VALUE;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device_id) != cudaSuccess) return SNB200_STATUS_NOT_INITIALIZED;
  if (prop.major != 10) return SNB200_STATUS_ARCH_MISMATCH;  // kernels are built for sm_100a only
  if (cudaSetDevice(device_id) != cudaSuccess) return SNB200_STATUS_NOT_INITIALIZED;
  if (!g_encode_tiled) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn ||
        q != cudaDriverEntryPointSuccess)
      return SNB200_STATUS_NOT_INITIALIZED;
    g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
  }
  snb200_context* h = static_cast<snb200_context*>(calloc(1, sizeof(snb200_context)));
  if (!h) return SNB200_STATUS_ALLOC_FAILED;
  h->device = device_id;
  h->sm_count = prop.multiProcessorCount;
  h->stream = 0;
  h->math_mode = SNB200_MATH_3XTF32;
  h->tune[TUNE_REWRITE_HI] = 0;
  h->tune[TUNE_CHUNK_K] = 128;
  const char* env = getenv("SNB200_MATH_MODE");
  if (env && env[0] >= '0' && env[0] <= '2' && env[1] == 0) h->math_mode = env[0] - '0';
  env = getenv("SNB200_NO_FUSED_ATTENTION");          // A/B measurements: the attention core as separate products
  if (env && env[0] == '1' && env[1] == 0) h->tune[TUNE_NO_FUSED_ATTN] = 1;
  env = getenv("SNB200_TS");                         // A operand from tensor memory: off until SNB200_TS=1 says otherwise
  h->tune[TUNE_NO_TS] = (env && env[0] == '1' && env[1] == 0) ? 0 : 1;
  h->workspace_floats = 32u << 20;   // 128 MB: column-sum slabs and split-K partial sums
  if (cudaMalloc(&h->workspace, h->workspace_floats * sizeof(float)) != cudaSuccess ||
      cudaMalloc(&h->error_word, sizeof(int)) != cudaSuccess ||
      cudaMemset(h->error_word, 0, sizeof(int)) != cudaSuccess) {
    cudaFree(h->workspace);
    cudaFree(h->error_word);
    free(h);
    return SNB200_STATUS_ALLOC_FAILED;
  }
  *handle = h;
  return 0;
}

extern "C" int snb200_destroy(snb200_handle_t h) {
  if (!h) return SNB200_STATUS_NOT_INITIALIZED;
  cudaSetDevice(h->device);
  if (h->nccl_comm) snb200_comm_destroy(h);
  cudaFree(h->workspace);
  cudaFree(h->error_word);
  if (h->gemm_events) {
    for (int i = 0; i < 2 * kMaxTimedGemms; ++i) cudaEventDestroy(h->gemm_events[i]);
    free(h->gemm_events);
  }
  free(h);
  return 0;
}

extern "C" int snb200_set_stream(snb200_handle_t h, void* s) {
  if (!h) return SNB200_STATUS_NOT_INITIALIZED;
  h->stream = static_cast<cudaStream_t>(s);
  return 0;
}
extern "C" int snb200_set_math_mode(snb200_handle_t h, int m) {
  if (!h) return SNB200_STATUS_NOT_INITIALIZED;
  if (m < 0 || m > 3) return fail(h, SNB200_STATUS_INVALID_VALUE, "math mode %d is not one of 0, 1, 2, 3", m);
  h->math_mode = m;
  return 0;
}
extern "C" int snb200_get_math_mode(snb200_handle_t h, int* m) {
  if (!h) return SNB200_STATUS_NOT_INITIALIZED;
  if (!m) return SNB200_STATUS_INVALID_VALUE;
  *m = h->math_mode;
  return 0;
}
extern "C" int snb200_set_tuning(snb200_handle_t h, int key, int value) {
  if (!h) return SNB200_STATUS_NOT_INITIALIZED;
  if (key < 0 || key >= TUNE_COUNT) return fail(h, SNB200_STATUS_INVALID_VALUE, "unknown tuning key %d", key);
  if (key == TUNE_CLUSTER && value != 0 && value != 1 && value != 2 && value != 4)
    return fail(h, SNB200_STATUS_INVALID_VALUE, "cluster size %d: 0 (automatic), 1 (never), 2 or 4", value);
  h->tune[key] = value;
  return 0;
}
extern "C" int snb200_set_activation_parameter(snb200_handle_t h, float alpha) {
  if (!h) return SNB200_STATUS_NOT_INITIALIZED;
  h->act_alpha = alpha;
  return 0;
}
extern "C" const char* snb200_last_error_string(snb200_handle_t h) { return h ? h->last_error : "null handle"; }
extern "C" int snb200_get_launch_count(snb200_handle_t h, long long* c) {
  if (!h) return SNB200_STATUS_NOT_INITIALIZED;
  if (!c) return SNB200_STATUS_INVALID_VALUE;
  *c = h->launches;
  return 0;
}
extern "C" int snb200_get_last_kernel(snb200_handle_t h, char* buf, int len) {
  if (!h) return SNB200_STATUS_NOT_INITIALIZED;
  if (!buf || len <= 0) return SNB200_STATUS_INVALID_VALUE;
  snprintf(buf, len, "%s", h->last_kernel);
  return 0;
}
extern "C" int snb200_check_device_status(snb200_handle_t h) {
  int st = enter(h);
  if (st) return st;
  SNB_CUDA(h, cudaStreamSynchronize(h->stream));
  int w = 0;
  SNB_CUDA(h, cudaMemcpy(&w, h->error_word, sizeof(int), cudaMemcpyDeviceToHost));
  if (w) {
    cudaMemset(h->error_word, 0, sizeof(int));
    return fail(h, SNB200_STATUS_EXECUTION_FAILED, "a tensor-core pipeline wait timed out on the device");
  }
  return 0;
}

// The failure path of the tensor-core kernels, run on purpose and harmlessly: one warp waits on an mbarrier that
// nothing ever arrives at, with a short limit; the wait gives up, raises the CTA's abort flag, and the kernel leaves
// through the same teardown as the GEMM kernels (error word set, normal return).
static __global__ void wait_timeout_selftest_kernel(int* error_word, unsigned long long limit_ns) {
  __shared__ uint64_t never_signalled;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&never_signalled, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  volatile int* abortp = &abort_flag;
  if (threadIdx.x == 0) mbar_wait_limit(&never_signalled, 0, abortp, limit_ns);
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag) atomicExch(error_word, 1);
}

extern "C" int snb200_selftest_wait_timeout(snb200_handle_t h, int limit_us) {
  int st = enter(h);
  if (st) return st;
  if (limit_us < 1 || limit_us > 100000)
    return fail(h, SNB200_STATUS_INVALID_VALUE, "the limit must lie between 1 and 100000 microseconds");
  wait_timeout_selftest_kernel<<<1, 32, 0, h->stream>>>(h->error_word, 1000ull * static_cast<unsigned long long>(limit_us));
  h->launches += 1;
  return check_launch(h, "wait_timeout_selftest_kernel launch");
}

// Launch of one of this library's kernels on the handle's stream with programmatic dependent launch: every kernel
// here starts with pdl_prologue() (or, for the tensor-core kernels, runs its set-up first), so its launch latency
// overlaps the tail of the previous kernel and it waits for that kernel before touching memory.
template <typename... KArgs, typename... Args>
static void launch_pdl(snb200_handle_t h, void (*kernel)(KArgs...), dim3 grid, dim3 block, Args&&... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = h->stream;
  cfg.attrs = attr;
  cfg.numAttrs = h->tune[TUNE_PDL] == 1 ? 0 : 1;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);   // errors surface in check_launch (cudaGetLastError)
}

// ------------------------------------------------------------------------------------ GEMM
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static bool encode_3d(CUtensorMap* m, const float* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t pitch1,
                      uint64_t pitch2, uint32_t b0, uint32_t b1, CUtensorMapSwizzle sw) {
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {pitch1 * sizeof(float), pitch2 * sizeof(float)};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode_tiled(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(ptr), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// The TMA path needs 16-byte aligned bases and pitches that are multiples of 16 bytes.
static bool tma_eligible(const GemmProblem& g) {
  if (!aligned16(g.A) || !aligned16(g.B)) return false;
  if ((g.lda & 3) || (g.ldb & 3)) return false;
  if (g.batch > 1 && ((g.strideA & 3) || (g.strideB & 3))) return false;
  if (g.K < 1) return false;
  return true;
}

// Result placement (OutMap): may the stores move whole float4s?
static bool omap_vec(const OutMap& m) {
  return !m.on || (!(m.d & 3) && !(m.s_io & 3) && !(m.s_ii & 3) && !(m.s_ro & 3) && !(m.s_ri & 3) && !(m.s_co & 3));
}
constexpr int kNoDiv = 1 << 30;   // a divisor larger than any index: x / kNoDiv = 0, x % kNoDiv = x
// A [B*T, H*d] result stored as [B, H, T, d]: the head split of multi-head attention.
static OutMap head_split_map(int T, int H, int d) {
  OutMap m;
  m.on = 1; m.H = 1; m.s_io = 0; m.s_ii = 0;
  m.T = T; m.s_ro = static_cast<long long>(H) * T * d; m.s_ri = d;
  m.d = d; m.s_co = static_cast<long long>(T) * d;
  return m;
}
// A batch of B*H [T x d] results stored as [B, T, H, d]: the head merge.
static OutMap head_merge_map(int T, int H, int d) {
  OutMap m;
  m.on = 1; m.H = H; m.s_io = static_cast<long long>(T) * H * d; m.s_ii = d;
  m.T = kNoDiv; m.s_ro = 0; m.s_ri = static_cast<long long>(H) * d;
  m.d = kNoDiv; m.s_co = 0;
  return m;
}

// Tensor maps and kernel parameters shared by the single-CTA and the CTA-pair kernels.  `bn_box` is
// the number of B columns one CTA loads per stage (BN, or BN / 2 in a pair).
template <class T>
static int fill_umma_args(snb200_handle_t h, const GemmProblem& g, int bn_box, CUtensorMap* tmA, CUtensorMap* tmB,
                          UmmaParams* pp) {
  const uint64_t a_rows = g.transA ? g.K : g.M, b_rows = g.transB ? g.N : g.K;
  const uint64_t pitchA2 = g.batch > 1 ? static_cast<uint64_t>(g.strideA) : a_rows * g.lda;
  const uint64_t pitchB2 = g.batch > 1 ? static_cast<uint64_t>(g.strideB) : b_rows * g.ldb;
  const CUtensorMapSwizzle kmaj_sw = (T::BK == 32) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  bool ok;
  if (!tma_eligible(g)) {       // the kernel's loader warps read the operands through plain pointers
    memset(tmA, 0, sizeof(*tmA));
    memset(tmB, 0, sizeof(*tmB));
    ok = true;
  } else {
  if (!g.transA)
    ok = encode_3d(tmA, g.A, g.K, g.M, g.batch, g.lda, pitchA2, T::BK, T::BM, kmaj_sw);
  else
    ok = encode_3d(tmA, g.A, g.M, g.K, g.batch, g.lda, pitchA2, 32, T::BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
  if (g.transB)
    ok = ok && encode_3d(tmB, g.B, g.K, g.N, g.batch, g.ldb, pitchB2, T::BK, bn_box, kmaj_sw);
  else
    ok = ok && encode_3d(tmB, g.B, g.N, g.K, g.batch, g.ldb, pitchB2, 32, T::BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
  }
  if (!ok) return fail(h, SNB200_STATUS_INTERNAL_ERROR, "cuTensorMapEncodeTiled rejected the operand layout");
  UmmaParams& p = *pp;
  p.M = g.M; p.N = g.N; p.K = g.K; p.batch = g.batch;
  p.tiles_m = (g.M + T::BM - 1) / T::BM;
  p.tiles_n = (g.N + T::BN - 1) / T::BN;
  p.k_blocks = (g.K + T::BK - 1) / T::BK;
  int chunk_k = T::SPLIT ? h->tune[TUNE_CHUNK_K] : 0;
  p.chunk_kblocks = chunk_k > 0 ? (chunk_k + T::BK - 1) / T::BK : p.k_blocks;
  if (p.chunk_kblocks < 1) p.chunk_kblocks = 1;
  p.a_mn = g.transA ? 1 : 0;
  p.b_mn = g.transB ? 0 : 1;
  p.ldc = g.ldc; p.strideC = g.strideC;
  p.C = g.C; p.Z = g.Z; p.bias = g.bias;
  p.alpha = g.alpha; p.beta = g.beta; p.act = g.act; p.act_alpha = g.act_alpha;
  p.rewrite_hi = h->tune[TUNE_REWRITE_HI];
  p.vec_ok = aligned16(g.C) && (g.ldc % 4 == 0) && (g.batch == 1 || g.strideC % 4 == 0) &&
             (!g.Z || aligned16(g.Z)) && (!g.bias || aligned16(g.bias));
  p.error_word = h->error_word;
  p.splits = 1;
  p.kb_per_split = p.k_blocks;
  p.row_op = g.row_op; p.causal = g.causal; p.aux = g.aux;
  p.omap = g.omap;
  if (!omap_vec(g.omap)) p.vec_ok = 0;
  p.A = g.A; p.B = g.B; p.lda = g.lda; p.ldb = g.ldb;
  p.strideA = g.batch > 1 ? g.strideA : 0; p.strideB = g.batch > 1 ? g.strideB : 0;
#ifdef SNB_TRACE
  p.trace = reinterpret_cast<unsigned long long*>(h->workspace + (h->workspace_floats - 128));   // last 512 bytes of the workspace
#endif
  p.cluster = 1;
  p.store_t = 0;
  p.group_batch = 0;
  p.c_shift = 0;
  p.whole_tiles = 0;       // set by the launcher: it knows the tile grid of its kernel
  p.partial_tiled = 0;
  p.partial = nullptr;
  p.partial_stride = 0;
  return 0;
}

// How a problem is cut along K when its output tiles do not fill the SMs evenly.  The first
// `whole_tiles` tiles run whole; each remaining tile becomes `splits` work units of `k_per_split` of K that
// write raw partial sums to the workspace (`tiled`: one tile per unit; otherwise one dense matrix per
// split, all tiles split), and a second kernel combines them.
struct SplitPlan {
  int splits; int k_per_split; int transposed;
  int parts;        // out: partial results per tail tile actually written (0 = none, C is final)
  int tiled; int whole_tiles;
  int tail;         // out: tiles whose partial sums are in the workspace
  int tiles_m;      // out: tile rows of the grid the kernel walked
  // cluster > 1: instead of all the above, every tile is cut into `cluster` K parts computed by the CTAs of one
  // thread-block cluster, which sum them through distributed shared memory and store C themselves (store_t: as the
  // transpose of what the kernel computed)
  int cluster; int store_t;
};

template <class T>
static void apply_split_plan(snb200_handle_t h, const GemmProblem& g, int tile_rows, long long n_tiles, UmmaParams& p,
                             SplitPlan& plan) {
  p.whole_tiles = static_cast<int>(n_tiles);
  plan.parts = 0; plan.tail = 0;
  if (plan.splits <= 0) return;
  const int chunk = p.chunk_kblocks < p.k_blocks ? p.chunk_kblocks : 1;
  int kbps = (plan.k_per_split + T::BK - 1) / T::BK;
  kbps = (kbps + chunk - 1) / chunk * chunk;          // whole accumulation chunks per unit
  p.kb_per_split = kbps;
  p.splits = (p.k_blocks + kbps - 1) / kbps;
  p.partial = h->workspace;
  if (plan.tiled) {
    p.partial_tiled = 1;
    p.whole_tiles = plan.whole_tiles;
    p.partial_stride = static_cast<long long>(tile_rows) * T::BN;
  } else {
    p.whole_tiles = 0;
    p.partial_stride = static_cast<long long>(g.batch) * g.M * g.N;
  }
  plan.parts = p.splits;
  plan.tail = static_cast<int>(n_tiles) - p.whole_tiles;
}

// K blocks per CTA when a tile's K range is shared by a cluster of `cs` CTAs (whole accumulation chunks of
// `chunk` blocks each), or 0 when that would leave a CTA without work.
static long long cluster_kblocks(long long k_blocks, int cs, long long chunk) {
  long long kbps = (k_blocks + cs - 1) / cs;
  if (chunk > 1 && chunk < k_blocks) kbps = (kbps + chunk - 1) / chunk * chunk;
  return kbps * (cs - 1) < k_blocks ? kbps : 0;
}

template <class T, bool ROWOP = false, int CLUSTER = 1>
static int launch_umma_t(snb200_handle_t h, const GemmProblem& g, SplitPlan& plan) {
  static bool configured[64] = {};
  CUtensorMap tmA, tmB;
  UmmaParams p;
  int st = fill_umma_args<T>(h, g, T::BN, &tmA, &tmB, &p);
  if (st) return st;
  const long long n_tiles = static_cast<long long>(p.batch) * p.tiles_m * p.tiles_n;
  if (CLUSTER > 1) {
    // one work unit per CTA: CTA r of a cluster takes K part r of the cluster's tile
    const int kbps = static_cast<int>(cluster_kblocks(p.k_blocks, CLUSTER, p.chunk_kblocks));
    if (kbps == 0 || n_tiles * CLUSTER > 0x7fffffffLL)
      return fail(h, SNB200_STATUS_INTERNAL_ERROR, "K = %d is too short for a cluster of %d", g.K, CLUSTER);
    p.cluster = CLUSTER; p.splits = CLUSTER; p.kb_per_split = kbps; p.whole_tiles = 0;
    p.store_t = plan.store_t;
    plan.parts = 0; plan.tail = 0;
  } else {
    apply_split_plan<T>(h, g, T::BM, n_tiles, p, plan);
  }
  plan.tiles_m = p.tiles_m;
  if (!configured[h->device]) {
    SNB_CUDA(h, cudaFuncSetAttribute(umma_gemm_kernel<T, ROWOP, CLUSTER>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     T::SMEM_BYTES));
    configured[h->device] = true;
  }
  if (CLUSTER > 1) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CLUSTER; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3(static_cast<unsigned>(n_tiles * CLUSTER));
    cfg.blockDim = dim3(T::THREADS);
    cfg.dynamicSmemBytes = T::SMEM_BYTES;
    cfg.stream = h->stream;
    cfg.attrs = attr;
    cfg.numAttrs = h->tune[TUNE_PDL] == 1 ? 1 : 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, umma_gemm_kernel<T, ROWOP, CLUSTER>, tmA, tmB, p);
    if (e != cudaSuccess) return cuda_fail(h, e, "umma_gemm_kernel (cluster) launch");
    return check_launch(h, "umma_gemm_kernel (cluster) launch");
  }
  const long long units = p.whole_tiles + (n_tiles - p.whole_tiles) * p.splits;
  const int grid = static_cast<int>(units < usable_sms(h) ? units : usable_sms(h));
  // launched so that its set-up may overlap the tail of the previous kernel in the stream; the kernel waits for
  // that kernel's completion before it touches global memory
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(T::THREADS);
  cfg.dynamicSmemBytes = T::SMEM_BYTES;
  cfg.stream = h->stream;
  cfg.attrs = attr;
  cfg.numAttrs = h->tune[TUNE_PDL] == 1 ? 0 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, umma_gemm_kernel<T, ROWOP, 1>, tmA, tmB, p);
  if (e != cudaSuccess) return cuda_fail(h, e, "umma_gemm_kernel launch");
  return check_launch(h, "umma_gemm_kernel launch");
}

template <class T>
static int launch_umma2_t(snb200_handle_t h, const GemmProblem& g, SplitPlan& plan) {
  static bool configured[64] = {};
  static int max_pairs[64] = {};
  CUtensorMap tmA, tmB;
  UmmaParams p;
  int st = fill_umma_args<T>(h, g, T::BNH, &tmA, &tmB, &p);
  if (st) return st;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see launch_umma_t
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.blockDim = dim3(T::THREADS);
  cfg.dynamicSmemBytes = T::SMEM_BYTES;
  cfg.stream = h->stream;
  cfg.attrs = attr;
  cfg.numAttrs = h->tune[TUNE_PDL] == 1 ? 1 : 2;
  if (!configured[h->device]) {
    SNB_CUDA(h, cudaFuncSetAttribute(umma2_gemm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES));
    cfg.gridDim = dim3(h->sm_count & ~1);
    int n = 0;
    SNB_CUDA(h, cudaOccupancyMaxActiveClusters(&n, umma2_gemm_kernel<T>, &cfg));
    if (n < 1) return fail(h, SNB200_STATUS_NOT_SUPPORTED, "no CTA pair of this kernel fits on the device");
    max_pairs[h->device] = n;
    configured[h->device] = true;
  }
  const int pair_tiles_m = (g.M + 2 * T::BM - 1) / (2 * T::BM);
  const long long tiles = static_cast<long long>(p.batch) * pair_tiles_m * p.tiles_n;
  apply_split_plan<T>(h, g, 2 * T::BM, tiles, p, plan);
  plan.tiles_m = pair_tiles_m;
  const long long units = p.whole_tiles + (tiles - p.whole_tiles) * p.splits;
  const int pair_cap = max_pairs[h->device] < usable_sms(h) / 2 ? max_pairs[h->device] : usable_sms(h) / 2;
  const long long pairs = units < pair_cap ? units : pair_cap;
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
  {
    const size_t len = strlen(h->last_kernel);
    snprintf(h->last_kernel + len, sizeof(h->last_kernel) - len, "_p%lld", pairs);
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, umma2_gemm_kernel<T>, tmA, tmB, p);
  if (e != cudaSuccess) return cuda_fail(h, e, "umma2_gemm_kernel launch");
  return check_launch(h, "umma2_gemm_kernel launch");
}

static int launch_umma2(snb200_handle_t h, const GemmProblem& g, bool split, int bn, SplitPlan& plan, bool hybrid) {
  char name[64];
  hybrid = hybrid && split && (bn == 128 || bn == 256);
  snprintf(name, sizeof(name), "umma2_%s_256x%d%s", hybrid ? "tf32bf16x2" : split ? "3xtf32" : "tf32", bn,
           plan.splits > 0 ? "_splitk" : "");
  note_kernel(h, name, 1);
  if (hybrid) {
    if (bn == 256) return launch_umma2_t<Umma2Tile<256, 32, true, true>>(h, g, plan);
    return launch_umma2_t<Umma2Tile<128, 32, true, true>>(h, g, plan);
  }
  if (split) {
    switch (bn) {
      // 32-wide K blocks: three 64 KB stages beat six 32 KB ones (fewer hand-offs per byte), measured +8..35 %
      case 256:
        if (h->tune[TUNE_VARIANT] == 1) return launch_umma2_t<Umma2Tile<256, 16, true>>(h, g, plan);
        return launch_umma2_t<Umma2Tile<256, 32, true>>(h, g, plan);
      case 192: return launch_umma2_t<Umma2Tile<192, 32, true>>(h, g, plan);
      case 128: return launch_umma2_t<Umma2Tile<128, 32, true>>(h, g, plan);
      default: return launch_umma2_t<Umma2Tile<64, 32, true>>(h, g, plan);
    }
  }
  switch (bn) {
    case 256: return launch_umma2_t<Umma2Tile<256, 32, false>>(h, g, plan);
    case 192: return launch_umma2_t<Umma2Tile<192, 32, false>>(h, g, plan);
    case 128: return launch_umma2_t<Umma2Tile<128, 32, false>>(h, g, plan);
    default: return launch_umma2_t<Umma2Tile<64, 32, false>>(h, g, plan);
  }
}

// How many clusters of `cs` CTAs of the tensor-core kernel (one CTA per SM) the device runs at once: fewer than
// SMs / cs, because a cluster lives inside one GPC.  0 when the query fails.
template <int CS>
static int cluster_capacity_t(snb200_handle_t h) {
  static int cap[64] = {};
  static bool known[64] = {};
  if (!known[h->device]) {
    using T = UmmaTile<128, 32, true>;
    int n = 0;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.gridDim = dim3(static_cast<unsigned>(h->sm_count / CS * CS));
    cfg.blockDim = dim3(T::THREADS);
    cfg.dynamicSmemBytes = T::SMEM_BYTES;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaFuncSetAttribute(umma_gemm_kernel<T, false, CS>, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES) !=
            cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, umma_gemm_kernel<T, false, CS>, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
    cap[h->device] = n;
    known[h->device] = true;
  }
  return cap[h->device];
}
static int cluster_capacity(snb200_handle_t h, int cs) { return cs == 4 ? cluster_capacity_t<4>(h) : cluster_capacity_t<2>(h); }

template <int CS>
static int launch_umma_cluster(snb200_handle_t h, const GemmProblem& g, bool split, int bn, SplitPlan& plan) {
  if (split) {
    switch (bn) {
      case 256: return launch_umma_t<UmmaTile<256, 32, true>, false, CS>(h, g, plan);
      case 128: return launch_umma_t<UmmaTile<128, 32, true>, false, CS>(h, g, plan);
      case 64: return launch_umma_t<UmmaTile<64, 32, true>, false, CS>(h, g, plan);
      default: return launch_umma_t<UmmaTile<32, 32, true>, false, CS>(h, g, plan);
    }
  }
  switch (bn) {
    case 256: return launch_umma_t<UmmaTile<256, 32, false>, false, CS>(h, g, plan);
    case 128: return launch_umma_t<UmmaTile<128, 32, false>, false, CS>(h, g, plan);
    case 64: return launch_umma_t<UmmaTile<64, 32, false>, false, CS>(h, g, plan);
    default: return launch_umma_t<UmmaTile<32, 32, false>, false, CS>(h, g, plan);
  }
}

static int launch_umma(snb200_handle_t h, const GemmProblem& g, bool split, int bn, SplitPlan& plan) {
  char name[64];
  if (plan.cluster > 1) {
    snprintf(name, sizeof(name), "umma_%s_128x%d%s_clusterk%d", split ? "3xtf32" : "tf32", bn,
             plan.store_t ? "_swapAB" : "", plan.cluster);
    note_kernel(h, name, 1);
    return plan.cluster == 4 ? launch_umma_cluster<4>(h, g, split, bn, plan) : launch_umma_cluster<2>(h, g, split, bn, plan);
  }
  snprintf(name, sizeof(name), "umma_%s_128x%d%s", split ? "3xtf32" : "tf32", bn,
           plan.splits > 0 ? (plan.transposed ? "_swapAB_splitk" : "_splitk") : "");
  note_kernel(h, name, 1);
  if (split) {
    const bool ts = h->tune[TUNE_NO_TS] == 0;   // A operand from tensor memory (tiles up to 128 wide)
    switch (bn) {
      case 256:
        if (h->tune[TUNE_VARIANT] == 1) return launch_umma_t<UmmaTile<256, 16, true>>(h, g, plan);
        return launch_umma_t<UmmaTile<256, 32, true>>(h, g, plan);
      case 128:
        if (h->tune[TUNE_VARIANT] == 1) return launch_umma_t<UmmaTile<128, 16, true>>(h, g, plan);
        if (ts) return launch_umma_t<UmmaTile<128, 32, true, 0, true>>(h, g, plan);
        return launch_umma_t<UmmaTile<128, 32, true>>(h, g, plan);
      // narrow tiles leave room for 32-wide K blocks: half as many stage hand-offs per unit of K
      case 64:
        if (ts) return launch_umma_t<UmmaTile<64, 32, true, 0, true>>(h, g, plan);
        return launch_umma_t<UmmaTile<64, 32, true>>(h, g, plan);
      default:
        if (ts) return launch_umma_t<UmmaTile<32, 32, true, 0, true>>(h, g, plan);
        return launch_umma_t<UmmaTile<32, 32, true>>(h, g, plan);
    }
  }
  switch (bn) {
    case 256: return launch_umma_t<UmmaTile<256, 32, false>>(h, g, plan);
    case 128: return launch_umma_t<UmmaTile<128, 32, false>>(h, g, plan);
    case 64: return launch_umma_t<UmmaTile<64, 32, false>>(h, g, plan);
    default: return launch_umma_t<UmmaTile<32, 32, false>>(h, g, plan);
  }
}

// Operands TMA cannot load (4-byte aligned base, pitch not a multiple of 16 bytes): the same tensor-core kernel fed
// by loader warps.  Whole tiles only: K is not cut and operands are not swapped on this path.
static int launch_umma_swload(snb200_handle_t h, const GemmProblem& g, bool split) {
  const int bn = g.N > 64 ? 128 : g.N > 32 ? 64 : 32;
  char name[64];
  snprintf(name, sizeof(name), "umma_%s_128x%d_swload", split ? "3xtf32" : "tf32", bn);
  note_kernel(h, name, 1);
  SplitPlan none = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
  if (split) {
    if (bn == 128) return launch_umma_t<UmmaTile<128, 32, true, 0, false, true>>(h, g, none);
    if (bn == 64) return launch_umma_t<UmmaTile<64, 32, true, 0, false, true>>(h, g, none);
    return launch_umma_t<UmmaTile<32, 32, true, 0, false, true>>(h, g, none);
  }
  if (bn == 128) return launch_umma_t<UmmaTile<128, 32, false, 0, false, true>>(h, g, none);
  if (bn == 64) return launch_umma_t<UmmaTile<64, 32, false, 0, false, true>>(h, g, none);
  return launch_umma_t<UmmaTile<32, 32, false, 0, false, true>>(h, g, none);
}

static int launch_simt(snb200_handle_t h, const GemmProblem& g) {
  SimtParams p;
  p.M = g.M; p.N = g.N; p.K = g.K; p.batch = g.batch;
  p.sAm = g.transA ? 1 : g.lda;
  p.sAk = g.transA ? g.lda : 1;
  p.sBk = g.transB ? 1 : g.ldb;
  p.sBn = g.transB ? g.ldb : 1;
  p.strideA = g.strideA; p.strideB = g.strideB; p.strideC = g.strideC;
  p.ldc = g.ldc;
  p.A = g.A; p.B = g.B; p.C = g.C; p.Z = g.Z; p.bias = g.bias;
  p.alpha = g.alpha; p.beta = g.beta; p.act = g.act; p.act_alpha = g.act_alpha;
  p.omap = g.omap;
  // 128 x 128 tiles once they fill most of the SMs; 64 x 64 tiles for everything smaller
  const long long big_tiles = static_cast<long long>((g.M + kSimtBigBM - 1) / kSimtBigBM) *
                              ((g.N + kSimtBigBN - 1) / kSimtBigBN) * g.batch;
  const bool big = big_tiles >= h->sm_count && g.K >= 64;
  const int bm = big ? kSimtBigBM : kSimtBM, bn = big ? kSimtBigBN : kSimtBN;
  p.tiles_m = (g.M + bm - 1) / bm;
  p.tiles_n = (g.N + bn - 1) / bn;
  const long long blocks = static_cast<long long>(p.tiles_m) * p.tiles_n * g.batch;
  if (blocks > 0x7fffffffLL) return fail(h, SNB200_STATUS_NOT_SUPPORTED, "too many tiles for one launch");
  note_kernel(h, big ? "simt_fp32_128x128" : "simt_fp32_64x64", 1);
  if (big)
    launch_pdl(h, simt_gemm_big_kernel, dim3(static_cast<unsigned>(blocks)), dim3(kSimtThreads), p);
  else
    launch_pdl(h, simt_gemm_kernel, dim3(static_cast<unsigned>(blocks)), dim3(kSimtThreads), p);
  return check_launch(h, "simt_gemm_kernel launch");
}

// Picks the kernel (one CTA per 128 x BN tile, or a CTA pair per 256 x BN tile), the tile width and the
// K split of the last, partly filled wave, by a time estimate in microseconds:
//   fixed + [whole waves * K blocks + tail waves * K blocks per split] * (time of one 32-deep K block)
//   + the reduction pass over the workspace.
// Both constants are measured on a B200, one wave of tiles at K = 1024 and K = 4096, per kernel, tile width and
// operand layout.  What they show: the tensor core reads both operand slices from shared memory for every
// instruction, so a narrow tile (which re-reads its 128 rows of A for few columns) costs almost as much per K
// block as a tile twice as wide -- narrow tiles only pay when they fill a wave that wide tiles cannot -- and a
// pair, where each SM holds half of B, runs a 256-wide tile 1.45x faster than one CTA does in 3xTF32 mode.
struct TileChoice { int pair; int bn; int splits; int whole_tiles; int cluster; };   // splits > 1: cut K of the tail tiles; cluster > 1: of every tile, inside a cluster
struct TileCost { double kblock_us, fixed_us; };
static TileCost tile_cost(bool split3x, int pair, int bn, const GemmProblem& g) {
  const int i = bn == 256 ? 0 : bn == 128 ? 1 : bn == 64 ? 2 : 3;
  if (bn == 192) {   // CTA pairs only: between the 256- and the 128-wide tile
    if (split3x) return {0.91, 11.4};
    if (g.transA) return {0.515, 8.3};
    return g.transB ? TileCost{0.369, 9.1} : TileCost{0.402, 8.9};
  }
  if (split3x) {   // the hi/lo split and three products per block hide the operand layout
    static const TileCost single[4] = {{1.46, 13.3}, {0.90, 8.5}, {0.81, 6.7}, {0.69, 5.7}};
    static const TileCost paired[4] = {{1.00, 13.3}, {0.82, 9.4}, {0.72, 7.6}, {0.72, 7.6}};
    return pair ? paired[i] : single[i];
  }
  // TF32: K-major operands (A not transposed, B transposed) are the fastest to feed
  static const TileCost single_nt[4] = {{0.381, 9.2}, {0.357, 6.2}, {0.340, 4.8}, {0.307, 5.6}};
  static const TileCost paired_nt[4] = {{0.371, 10.7}, {0.366, 7.4}, {0.345, 6.4}, {0.345, 6.4}};
  static const TileCost single_nn[4] = {{0.489, 8.3}, {0.380, 6.0}, {0.332, 5.2}, {0.316, 4.7}};
  static const TileCost paired_nn[4] = {{0.439, 10.1}, {0.365, 7.7}, {0.350, 6.2}, {0.350, 6.2}};
  static const TileCost single_tn[4] = {{0.567, 7.8}, {0.454, 6.1}, {0.381, 5.1}, {0.336, 4.8}};
  static const TileCost paired_tn[4] = {{0.551, 9.5}, {0.476, 7.0}, {0.420, 6.0}, {0.420, 6.0}};
  if (g.transA) return pair ? paired_tn[i] : single_tn[i];
  if (!g.transB) return pair ? paired_nn[i] : single_nn[i];
  return pair ? paired_nt[i] : single_nt[i];
}
static TileChoice choose_tile(const snb200_context* h, const GemmProblem& g, bool split, bool hybrid) {
  TileChoice best = {0, 256, 1, 0, 1};
  const bool allow_splitk = h->tune[TUNE_SPLITK] == 0;
  double best_cost = 1e300;
  const int pair_mode = h->tune[TUNE_PAIR];   // 0 automatic, 1 always, 2 never
  const int forced_bn = h->tune[TUNE_FORCE_BN];
  const int forced_splits = allow_splitk ? h->tune[TUNE_FORCE_SPLITS] : 0;
  const int cand[5] = {256, 192, 128, 64, 32};
  const int ks_cand[11] = {1, 2, 3, 4, 5, 6, 7, 8, 10, 12, 16};
  const long long kb = (g.K + 31) / 32;
  for (int pair = 0; pair < 2; ++pair) {
    if (pair == 0 && pair_mode == 1) continue;
    if (pair == 1 && (pair_mode == 2 || (pair_mode == 0 && g.M <= 128))) continue;
    for (int i = 0; i < 5; ++i) {
      const int bn = cand[i];
      if (pair && bn < 64) continue;
      if (!pair && bn == 192) continue;
      if (forced_bn && bn != forced_bn) continue;
      const int rows = pair ? 256 : 128;
      const long long tiles = static_cast<long long>(g.batch) * ((g.M + rows - 1) / rows) * ((g.N + bn - 1) / bn);
      const long long slots = pair ? usable_sms(h) / 2 : usable_sms(h);
      const long long whole = tiles / slots * slots, tail = tiles - whole;
      const TileCost tc = tile_cost(split, pair, bn, g);
      // TF32 + bf16 cross terms: two instruction times per K slice instead of three, on the pair kernel's wide tiles
      const double c = tc.kblock_us * ((hybrid && pair && (bn == 128 || bn == 256)) ? 0.7 : 1.0), fixed = tc.fixed_us;
      // One wave of tiles that leaves SMs idle: clusters of 2 or 4 CTAs share a tile's K range and sum their parts
      // through distributed shared memory.  No workspace pass, and every CTA stores only its share of the rows.
      const int cluster_mode = h->tune[TUNE_CLUSTER];   // 0 automatic, 1 never, 2 / 4 forced
      if (!pair && cluster_mode != 1 && allow_splitk && g.row_op == ROW_NONE && forced_splits <= 1) {
        static const double store_us[5] = {4.5, 0.0, 2.0, 1.3, 0.9};   // the store phase of a whole tile (nothing overlaps it)
        for (int cs = 2; cs <= 4; cs *= 2) {
          if (cluster_mode > 1 && cs != cluster_mode) continue;
          // left to itself: pairs of CTAs, all resident at once (measured: clusters of four lose to pairs on wider
          // tiles or to the workspace plans wherever they fit, and a second wave of clusters loses to everything)
          if (cluster_mode == 0 && (cs != 2 || kb / cs < 4 ||
                                    tiles > cluster_capacity(const_cast<snb200_context*>(h), cs) || tiles * cs > slots))
            continue;
          const long long kbps = cluster_kblocks(kb, cs, split ? (h->tune[TUNE_CHUNK_K] + 31) / 32 : 0);
          if (kbps == 0) continue;                                  // every CTA needs a part of K
          const long long waves = (tiles * cs + slots - 1) / slots;
          // the exchange: every CTA reads (cs - 1) / cs of a tile from the other CTAs' shared memory, about 20 KB / us
          const double exchange_us = 0.5 + 128.0 * bn * 4.0 * (cs - 1) / cs / 20.0e3;
          // + 1.5: where the estimates tie, the workspace plans of the CTA-pair kernel measured faster
          double cost = waves * (fixed + c * kbps) + exchange_us - store_us[i] * (1.0 - 1.0 / cs) + 1.5;
          if (cluster_mode > 1) cost -= 1.0e6;                      // forced: beats every other plan
          if (cost < best_cost * 0.999) {
            best_cost = cost; best.pair = 0; best.bn = bn; best.splits = 1; best.whole_tiles = 0; best.cluster = cs;
          }
        }
      }
      for (int j = 0; j < 11; ++j) {
        const long long ks = ks_cand[j];
        if (forced_splits > 1) {            // tests: cut the tail tiles this many times whatever it costs
          if (ks != forced_splits) { if (ks > forced_splits) break; continue; }
          if (tail == 0 || kb / ks < 1) break;
        } else
        if (ks > 1 && (!allow_splitk || tail == 0 || kb / ks < 8)) break;   // at least 256 of K per unit
        const long long tail_floats = tail * rows * bn;
        if (ks > 1 && ks * tail_floats > static_cast<long long>(h->workspace_floats)) break;
        const long long kbps = ((kb + ks - 1) / ks + 3) / 4 * 4;
        const long long tail_waves = (tail * ks + slots - 1) / slots;
        double cost = fixed + c * (static_cast<double>(whole / slots) * kb + static_cast<double>(tail_waves) * (ks > 1 ? kbps : kb));
        // a cut costs: the reduction kernel (launch + its traffic) and, per wave of cut units, one more
        // pipeline fill and a partial-tile store that nothing overlaps
        if (ks > 1) cost += 2.0 + static_cast<double>(ks + 1) * tail_floats * 4.0 / 4.0e6 + 2.0 * tail_waves;
        if (cost < best_cost * 0.999) {
          best_cost = cost; best.pair = pair; best.bn = bn; best.splits = static_cast<int>(ks);
          best.whole_tiles = static_cast<int>(whole); best.cluster = 1;
        }
      }
    }
  }
  if (best_cost > 1e299) { best.pair = (pair_mode == 1); best.bn = 256; best.splits = 1; }   // forced width not offered by the forced kernel
  return best;
}

static int launch_tail_reduce(snb200_handle_t h, const GemmProblem& g, const SplitPlan& plan, int tile_rows, int bn) {
  TailReduceParams r;
  r.M = g.M; r.N = g.N;
  r.tiles_m = plan.tiles_m; r.tiles_n = (g.N + bn - 1) / bn;
  r.tile_rows = tile_rows; r.bn = bn; r.rows_per_block = bn == 192 ? 4 : 1024 / bn;   // divides the tile's rows
  r.whole_tiles = plan.whole_tiles; r.tail = plan.tail; r.splits = plan.parts;
  r.partial = h->workspace;
  r.tile_elems = static_cast<long long>(tile_rows) * bn;
  r.C = g.C; r.Z = g.Z; r.bias = g.bias; r.ldc = g.ldc; r.strideC = g.strideC;
  r.alpha = g.alpha; r.beta = g.beta; r.act = g.act; r.act_alpha = g.act_alpha;
  r.omap = g.omap;
  r.vec_ok = aligned16(g.C) && (g.ldc % 4 == 0) && (g.batch == 1 || g.strideC % 4 == 0) &&
             (!g.Z || aligned16(g.Z)) && (!g.bias || aligned16(g.bias)) && omap_vec(g.omap);
  dim3 grid(plan.tail, tile_rows / r.rows_per_block);
  launch_pdl(h, tail_reduce_kernel, grid, dim3(256), r);
  h->launches += 1;
  return check_launch(h, "tail_reduce_kernel launch");
}

static int launch_reduce(snb200_handle_t h, const GemmProblem& g, int parts, int transposed) {
  SplitKReduceParams r;
  r.M = g.M; r.N = g.N; r.batch = g.batch; r.splits = parts; r.transposed = transposed;
  r.partial = h->workspace;
  r.partial_stride = static_cast<long long>(g.batch) * g.M * g.N;
  r.C = g.C; r.Z = g.Z; r.bias = g.bias; r.ldc = g.ldc; r.strideC = g.strideC;
  r.alpha = g.alpha; r.beta = g.beta; r.act = g.act; r.act_alpha = g.act_alpha;
  r.omap = g.omap;
  const long long total = r.partial_stride;
  long long blocks = (total + 255) / 256;
  if (blocks > 8LL * h->sm_count) blocks = 8LL * h->sm_count;
  if (transposed && g.batch <= 65535 && (g.M + 31) / 32 <= 65535) {
    dim3 grid((g.N + 31) / 32, (g.M + 31) / 32, g.batch);
    launch_pdl(h, splitk_reduce_transposed_kernel, grid, dim3(256), r);
  } else {
    launch_pdl(h, splitk_reduce_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), r);
  }
  h->launches += 1;
  return check_launch(h, "splitk_reduce_kernel launch");
}

static int run_gemm_untimed(snb200_handle_t h, const GemmProblem& g);
static int run_gemm(snb200_handle_t h, const GemmProblem& g);

// Two strided-batched products of one shape (same dimensions, transposes, pitches and strides; beta = 0, no bias, no
// activation) as ONE launch of the single-CTA tensor-core kernel: the grid walks 2 x batch matrices and takes the
// second half's operands from their own tensor maps.  Used where two small products follow each other and each
// would be mostly launch (the dV and dK products of the attention backward pass).  Falls back to two calls when the
// pair does not qualify.
template <class T>
static int launch_umma_grouped_t(snb200_handle_t h, const GemmProblem& g1, const GemmProblem& g2, long long c_shift) {
  static bool configured[64] = {};
  CUtensorMap tmA, tmB, tmA2, tmB2;
  UmmaParams p, p2;
  int st = fill_umma_args<T>(h, g1, T::BN, &tmA, &tmB, &p);
  if (!st) st = fill_umma_args<T>(h, g2, T::BN, &tmA2, &tmB2, &p2);
  if (st) return st;
  p.group_batch = g1.batch;
  p.batch = 2 * g1.batch;
  p.c_shift = c_shift;
  p.vec_ok = p.vec_ok && p2.vec_ok && !(c_shift & 3);
  const long long n_tiles = static_cast<long long>(p.batch) * p.tiles_m * p.tiles_n;
  p.whole_tiles = static_cast<int>(n_tiles);
  if (!configured[h->device]) {
    SNB_CUDA(h, cudaFuncSetAttribute(umma_gemm_grouped_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES));
    configured[h->device] = true;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.gridDim = dim3(static_cast<unsigned>(n_tiles < usable_sms(h) ? n_tiles : usable_sms(h)));
  cfg.blockDim = dim3(T::THREADS);
  cfg.dynamicSmemBytes = T::SMEM_BYTES;
  cfg.stream = h->stream;
  cfg.attrs = attr;
  cfg.numAttrs = h->tune[TUNE_PDL] == 1 ? 0 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, umma_gemm_grouped_kernel<T>, tmA, tmB, tmA2, tmB2, p);
  if (e != cudaSuccess) return cuda_fail(h, e, "umma_gemm_grouped_kernel launch");
  return check_launch(h, "umma_gemm_grouped_kernel launch");
}

static int run_gemm_pair(snb200_handle_t h, const GemmProblem& g1, const GemmProblem& g2) {
  const bool same = g1.M == g2.M && g1.N == g2.N && g1.K == g2.K && g1.batch == g2.batch && g1.transA == g2.transA &&
                    g1.transB == g2.transB && g1.lda == g2.lda && g1.ldb == g2.ldb && g1.ldc == g2.ldc &&
                    g1.strideA == g2.strideA && g1.strideB == g2.strideB && g1.strideC == g2.strideC &&
                    g1.alpha == g2.alpha && memcmp(&g1.omap, &g2.omap, sizeof(OutMap)) == 0;
  const bool plain = g1.beta == 0.0f && g2.beta == 0.0f && !g1.bias && !g2.bias && !g1.Z && !g2.Z &&
                     g1.act == ACT_IDENTITY && g2.act == ACT_IDENTITY && g1.row_op == ROW_NONE && g2.row_op == ROW_NONE;
  const bool tensor = h->math_mode != SNB200_MATH_FP32_SIMT && h->tune[TUNE_FORCE_PATH] != 2 &&
                      h->tune[TUNE_NO_FUSED_ATTN] == 0 && tma_eligible(g1) && tma_eligible(g2);
  // few K blocks per tile: launch-bound products that no K cut would help
  const long long tiles = static_cast<long long>(g1.batch) * ((g1.M + 127) / 128) * ((g1.N + 127) / 128);
  const bool small = g1.N <= 128 && g1.M >= 16 && g1.N >= 8 && g1.K <= 512 && 2 * tiles <= 0x3fffffffLL &&
                     static_cast<double>(g1.M) * g1.N * g1.K * g1.batch >= 64.0 * 64 * 64;
  long long c_shift = 0;
  bool placed = ((reinterpret_cast<uintptr_t>(g1.C) | reinterpret_cast<uintptr_t>(g2.C)) & 3u) == 0;
  if (same && placed) {
    // where matrix b of the doubled batch would land from g1.C, against where matrix b - batch of g2 must land
    const long long base = g1.omap.on ? (g1.batch % g1.omap.H == 0 ? static_cast<long long>(g1.batch / g1.omap.H) * g1.omap.s_io : -1)
                                      : static_cast<long long>(g1.batch) * g1.strideC;
    if (g1.omap.on && base < 0) placed = false;
    c_shift = (reinterpret_cast<intptr_t>(g2.C) - reinterpret_cast<intptr_t>(g1.C)) / 4 - base;
  }
  if (!(same && plain && tensor && small && placed)) {
    const int st = run_gemm(h, g1);
    return st ? st : run_gemm(h, g2);
  }
  const bool timed = h->time_gemms && h->gemm_events_used + 2 <= 2 * kMaxTimedGemms;
  if (timed) SNB_CUDA(h, cudaEventRecord(h->gemm_events[h->gemm_events_used], h->stream));
  const bool split = h->math_mode == SNB200_MATH_3XTF32 || h->math_mode == SNB200_MATH_TF32_BF16X2;
  const int bn = g1.N <= 32 ? 32 : g1.N <= 64 ? 64 : 128;
  char name[64];
  snprintf(name, sizeof(name), "umma_%s_128x%d_grouped", split ? "3xtf32" : "tf32", bn);
  note_kernel(h, name, 1);
  int st;
  if (split) {
    st = bn == 32 ? launch_umma_grouped_t<UmmaTile<32, 32, true>>(h, g1, g2, c_shift)
       : bn == 64 ? launch_umma_grouped_t<UmmaTile<64, 32, true>>(h, g1, g2, c_shift)
                  : launch_umma_grouped_t<UmmaTile<128, 32, true>>(h, g1, g2, c_shift);
  } else {
    st = bn == 32 ? launch_umma_grouped_t<UmmaTile<32, 32, false>>(h, g1, g2, c_shift)
       : bn == 64 ? launch_umma_grouped_t<UmmaTile<64, 32, false>>(h, g1, g2, c_shift)
                  : launch_umma_grouped_t<UmmaTile<128, 32, false>>(h, g1, g2, c_shift);
  }
  if (timed) {
    SNB_CUDA(h, cudaEventRecord(h->gemm_events[h->gemm_events_used + 1], h->stream));
    h->gemm_events_used += 2;
  }
  return st;
}

static int run_gemm(snb200_handle_t h, const GemmProblem& g) {
  const bool timed = h->time_gemms && h->gemm_events_used + 2 <= 2 * kMaxTimedGemms;
  if (timed) SNB_CUDA(h, cudaEventRecord(h->gemm_events[h->gemm_events_used], h->stream));
  const int st = run_gemm_untimed(h, g);
  if (timed) {
    SNB_CUDA(h, cudaEventRecord(h->gemm_events[h->gemm_events_used + 1], h->stream));
    h->gemm_events_used += 2;
  }
  return st;
}

extern "C" int snb200_gemm_timing_begin(snb200_handle_t h) {
  int st = enter(h);
  if (st) return st;
  if (!h->gemm_events) {
    h->gemm_events = static_cast<cudaEvent_t*>(calloc(2 * kMaxTimedGemms, sizeof(cudaEvent_t)));
    if (!h->gemm_events) return fail(h, SNB200_STATUS_ALLOC_FAILED, "out of host memory");
    for (int i = 0; i < 2 * kMaxTimedGemms; ++i) SNB_CUDA(h, cudaEventCreate(&h->gemm_events[i]));
  }
  h->gemm_events_used = 0;
  h->time_gemms = 1;
  return 0;
}

extern "C" int snb200_gemm_timing_end(snb200_handle_t h, double* total_ms, int* gemm_calls) {
  int st = enter(h);
  if (st) return st;
  if (!h->time_gemms) return fail(h, SNB200_STATUS_INVALID_VALUE, "snb200_gemm_timing_begin was not called");
  h->time_gemms = 0;
  SNB_CUDA(h, cudaStreamSynchronize(h->stream));
  double sum = 0.0;
  for (int i = 0; i + 1 < h->gemm_events_used; i += 2) {
    float ms = 0.0f;
    SNB_CUDA(h, cudaEventElapsedTime(&ms, h->gemm_events[i], h->gemm_events[i + 1]));
    sum += ms;
  }
  if (total_ms) *total_ms = sum;
  if (gemm_calls) *gemm_calls = h->gemm_events_used / 2;
  return 0;
}

static int run_gemm_untimed(snb200_handle_t h, const GemmProblem& g) {
  if (g.M == 0 || g.N == 0 || g.batch == 0) return 0;
  const int force = h->tune[TUNE_FORCE_PATH];  // 0 auto, 1 tensor cores whenever eligible, 2 SIMT
  bool use_umma = h->math_mode != SNB200_MATH_FP32_SIMT && force != 2 && tma_eligible(g);
  if (use_umma && force != 1) {
    // Tiny problems do not amortise a 128-row tensor-core tile.
    const double macs = static_cast<double>(g.M) * g.N * g.K * g.batch;
    const bool swappable = h->tune[TUNE_SPLITK] == 0 && g.N >= 256 && g.K >= 256;   // few rows run transposed
    if (macs < 64.0 * 64 * 64 || (g.M < 16 && !swappable) || g.N < 8) use_umma = false;
  }
  const bool split = h->math_mode == SNB200_MATH_3XTF32 || h->math_mode == SNB200_MATH_TF32_BF16X2;
  // Operands TMA cannot load (a base that is only float-aligned, a width that is not a multiple of 4 floats): when
  // the product is large against its operands and they fit the front half of the workspace, they are first copied
  // into aligned, padded rows there (one bandwidth-bound pass, O(n^2) bytes before O(n^3) flops) and the product
  // then runs on the TMA kernels like any other, with the rest of the workspace for its partial sums.
  if (!use_umma && h->math_mode != SNB200_MATH_FP32_SIMT && force != 2 && !tma_eligible(g) && g.K >= 1 &&
      h->tune[TUNE_NO_SWLOAD] == 0 && !h->realigning &&
      g.M >= 64 && g.N >= 16 && static_cast<double>(g.M) * g.N * g.K * g.batch >= 128.0 * 128 * 128) {
    const bool fixA = !aligned16(g.A) || (g.lda & 3) || (g.batch > 1 && (g.strideA & 3));
    const bool fixB = !aligned16(g.B) || (g.ldb & 3) || (g.batch > 1 && (g.strideB & 3));
    const long long a_rows = g.transA ? g.K : g.M, b_rows = g.transB ? g.N : g.K;
    const int a_pitch = (g.lda + 3) & ~3, b_pitch = (g.ldb + 3) & ~3;
    auto granules = [](long long floats) { return (floats + 63) / 64 * 64; };   // 256-byte granules
    const long long a_mat = granules(a_rows * a_pitch), b_mat = granules(b_rows * b_pitch);
    const long long budget = static_cast<long long>(h->workspace_floats / 4 * 3);   // a quarter stays for partial sums
    const long long need_b = fixB ? b_mat * g.batch : 0;
    // A may go through in panels of rows of op(A) (one matrix, dense result only) when it does not fit beside B
    const bool panels_ok = g.batch == 1 && !g.omap.on;
    int m_panel = g.M;
    if (fixA && need_b + a_mat * g.batch > budget && panels_ok) {
      const long long per_row = g.transA ? granules(static_cast<long long>(g.K) * 256) / 256 : a_pitch;   // floats per row of op(A)
      const long long rows_fit = (budget - need_b) / (per_row > 0 ? per_row : 1);
      m_panel = static_cast<int>(rows_fit / 256 * 256);
    }
    const long long a_panel_rows = g.transA ? g.K : m_panel;
    const int a_panel_pitch = g.transA ? ((m_panel + 3) & ~3) : a_pitch;
    const long long need_a = fixA ? granules(a_panel_rows * a_panel_pitch) * g.batch : 0;
    const long long need = need_a + need_b;
    // the copies move 8 bytes per operand float; worth it when the product does far more work than that
    const double copied = static_cast<double>((fixA ? a_mat : 0) + (fixB ? b_mat : 0)) * g.batch;
    const double flops_per_copied_float = 2.0 * g.M * g.N * g.K * g.batch / (copied > 0 ? copied : 1.0);
    // one copy launch per matrix: worth it for a few large matrices, not for a batch of many small ones
    if (need > 0 && m_panel >= 256 - (g.M < 256 ? 256 : 0) && m_panel > 0 && need <= budget &&
        flops_per_copied_float >= 256.0 && g.batch <= 16) {
      float* ws = h->workspace;
      auto copy = [&](const float* src, float* dst, long long rows, int cols, int src_pitch, int pitch) {
        const long long quads = rows * (pitch >> 2);
        long long blocks = (quads + 255) / 256;
        if (blocks > 16LL * h->sm_count) blocks = 16LL * h->sm_count;
        launch_pdl(h, realign_rows_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), src, dst, rows, cols, src_pitch, pitch);
        h->launches += 1;
      };
      GemmProblem t = g;
      float* b_copy = nullptr;
      if (fixB) {
        b_copy = ws;
        for (int b = 0; b < g.batch; ++b) copy(g.B + b * g.strideB, ws + b * b_mat, b_rows, g.ldb, g.ldb, b_pitch);
        t.B = b_copy; t.ldb = b_pitch; t.strideB = b_mat;
        ws += need_b;
      }
      float* a_copy = ws;
      if (fixA) ws += need_a;
      // the products see the rest of the workspace
      float* ws0 = h->workspace;
      const size_t wf0 = h->workspace_floats;
      h->workspace_floats -= static_cast<size_t>(ws - ws0);
      h->workspace = ws;
      h->realigning = 1;
      int st = 0;
      for (int m0 = 0; m0 < g.M && !st; m0 += m_panel) {
        const int mp = g.M - m0 < m_panel ? g.M - m0 : m_panel;
        if (fixA) {
          if (!g.transA) {          // rows m0 .. m0 + mp of A
            const long long mat = granules(static_cast<long long>(mp) * a_pitch);
            for (int b = 0; b < g.batch; ++b)
              copy(g.A + b * g.strideA + static_cast<long long>(m0) * g.lda, a_copy + b * mat, mp, g.lda, g.lda, a_pitch);
            t.A = a_copy; t.lda = a_pitch; t.strideA = mat;
          } else {                  // columns m0 .. m0 + mp of the stored [K x M] matrix
            const int pitch = (mp + 3) & ~3;
            const long long mat = granules(static_cast<long long>(g.K) * pitch);
            for (int b = 0; b < g.batch; ++b) copy(g.A + b * g.strideA + m0, a_copy + b * mat, g.K, mp, g.lda, pitch);
            t.A = a_copy; t.lda = pitch; t.strideA = mat;
          }
        } else {
          t.A = g.transA ? g.A + m0 : g.A + static_cast<long long>(m0) * g.lda;   // an aligned A walks in place
        }
        t.M = mp;
        t.C = g.C + static_cast<long long>(m0) * g.ldc;
        t.Z = g.Z ? g.Z + static_cast<long long>(m0) * g.ldc : nullptr;
        st = check_launch(h, "realign_rows_kernel launch");
        if (!st) st = run_gemm_untimed(h, t);
      }
      h->realigning = 0;
      h->workspace = ws0;
      h->workspace_floats = wf0;
      if (!st) {
        const size_t len = strlen(h->last_kernel);
        snprintf(h->last_kernel + len, sizeof(h->last_kernel) - len, "_realigned");
      }
      return st;
    }
  }
  // unaligned operands of a problem large enough for 128-row tiles: tensor cores fed by loader warps
  if (!use_umma && h->math_mode != SNB200_MATH_FP32_SIMT && force != 2 && !tma_eligible(g) && g.K >= 1 &&
      g.row_op == ROW_NONE && h->tune[TUNE_NO_SWLOAD] == 0 &&
      (force == 1 || (g.M >= 64 && g.N >= 16 && static_cast<double>(g.M) * g.N * g.K * g.batch >= 128.0 * 128 * 128)))
    return launch_umma_swload(h, g, split);
  if (!use_umma) return launch_simt(h, g);
  // the bf16 cross-term scheme exists for K-major operands on the pair kernel; everything else runs 3xTF32
  const bool hybrid = h->math_mode == SNB200_MATH_TF32_BF16X2 && !g.transA && g.transB;
  if (g.row_op != ROW_NONE) {
    // whole rows in one tile of the single-CTA kernel, K never cut (the caller checked row_op_fits)
    SplitPlan none = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
    const int bn = g.N <= 32 ? 32 : g.N <= 64 ? 64 : g.N <= 128 ? 128 : 256;
    char name[64];
    snprintf(name, sizeof(name), "umma_%s_128x%d_%s", split ? "3xtf32" : "tf32", bn,
             g.row_op == ROW_SOFTMAX ? "softmax" : "softmax_grad");
    note_kernel(h, name, 1);
    // two epilogue warps per row (UmmaTile<..., 2>) except for the 32-wide tile
    if (split) {
      if (h->tune[TUNE_NO_TS] == 0) {
        if (bn == 32) return launch_umma_t<UmmaTile<32, 32, true, 0, true>, true>(h, g, none);
        if (bn == 64) return launch_umma_t<UmmaTile<64, 32, true, 2, true>, true>(h, g, none);
        if (bn == 128) return launch_umma_t<UmmaTile<128, 32, true, 2, true>, true>(h, g, none);
      }
      if (bn == 32) return launch_umma_t<UmmaTile<32, 32, true>, true>(h, g, none);
      if (bn == 64) return launch_umma_t<UmmaTile<64, 32, true, 2>, true>(h, g, none);
      if (bn == 128) return launch_umma_t<UmmaTile<128, 32, true, 2>, true>(h, g, none);
      return launch_umma_t<UmmaTile<256, 32, true, 2>, true>(h, g, none);
    }
    if (bn == 32) return launch_umma_t<UmmaTile<32, 32, false>, true>(h, g, none);
    if (bn == 64) return launch_umma_t<UmmaTile<64, 32, false, 2>, true>(h, g, none);
    if (bn == 128) return launch_umma_t<UmmaTile<128, 32, false, 2>, true>(h, g, none);
    return launch_umma_t<UmmaTile<256, 32, false, 2>, true>(h, g, none);
  }
  const int splitk_mode = h->tune[TUNE_SPLITK];   // 0 automatic, 1 never
  // Few rows (M <= 64): run the transposed problem C^T = op(B)^T * op(A)^T, so that the long N dimension
  // fills the 128 rows of the tensor-core tile and the short M dimension becomes a narrow tile width.
  if (splitk_mode == 0 && h->tune[TUNE_PAIR] != 1 && g.M <= 64 && g.N >= 256 && g.K >= 256) {
    GemmProblem t = g;
    t.M = g.N; t.N = g.M;
    t.A = g.B; t.lda = g.ldb; t.strideA = g.strideB; t.transA = g.transB ? 0 : 1;
    t.B = g.A; t.ldb = g.lda; t.strideB = g.strideA; t.transB = g.transA ? 0 : 1;
    const int bn = t.N <= 32 ? 32 : 64;
    const long long tiles = static_cast<long long>(t.batch) * ((t.M + 127) / 128) * ((t.N + bn - 1) / bn);
    long long s = usable_sms(h) / (tiles > 0 ? tiles : 1);
    if (s < 1) s = 1;
    if (s > g.K / 256) s = g.K / 256;
    const size_t per_split = static_cast<size_t>(g.batch) * g.M * g.N;
    if (s * per_split > h->workspace_floats) s = static_cast<long long>(h->workspace_floats / per_split);
    const int cluster_mode = h->tune[TUNE_CLUSTER];
    int cs = cluster_mode > 1 ? cluster_mode : (s >= 4 ? 4 : s >= 2 ? 2 : 1);
    const long long chunk = split ? (h->tune[TUNE_CHUNK_K] + 31) / 32 : 0;
    while (cs > 1 && (g.K / cs < 128 || cluster_kblocks((g.K + 31) / 32, cs, chunk) == 0 ||
                      (cluster_mode == 0 && tiles > cluster_capacity(h, cs)))) cs /= 2;
    // worth it while the cluster keeps about as many CTAs busy as the workspace plan would (s K parts per tile)
    if (cluster_mode != 1 && cs > 1 && !g.omap.on && (cluster_mode > 1 || 5 * cs >= 4 * s)) {
      // K parts summed inside clusters; the owners store the transposed tile straight into C
      SplitPlan plan = {0, 0, 0, 0, 0, 0, 0, 0, cs, 1};
      return launch_umma(h, t, split, bn, plan);
    }
    if (s >= 1) {
      SplitPlan plan = {static_cast<int>(s), static_cast<int>((g.K + s - 1) / s), 1, 0, 0, 0, 0, 0, 0, 0};
      plan.k_per_split = (plan.k_per_split + 127) / 128 * 128;
      const int st = launch_umma(h, t, split, bn, plan);
      if (st) return st;
      return launch_reduce(h, g, plan.parts, 1);
    }
  }
  const TileChoice c = choose_tile(h, g, split, hybrid);
  // Tiles that would leave most SMs idle in the last wave are cut along K.
  SplitPlan plan = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
  if (c.cluster > 1) {
    plan.cluster = c.cluster;
  } else if (c.splits > 1) {
    plan.splits = c.splits;
    plan.k_per_split = (g.K + c.splits - 1) / c.splits;
    plan.tiled = 1;
    plan.whole_tiles = c.whole_tiles;
  }
  const int st = c.pair ? launch_umma2(h, g, split, c.bn, plan, hybrid) : launch_umma(h, g, split, c.bn, plan);
  if (st || plan.parts == 0) return st;
  return launch_tail_reduce(h, g, plan, c.pair ? 256 : 128, c.bn);
}

static int check_ptrs(snb200_handle_t h, const void* a, const void* b, const void* c) {
  if (!a || !b || !c) return fail(h, SNB200_STATUS_INVALID_VALUE, "null matrix pointer");
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 3u)
    return fail(h, SNB200_STATUS_INVALID_VALUE, "matrix pointers must be 4-byte aligned");
  return 0;
}

extern "C" int snb200_batched_gemm(snb200_handle_t h, int transA, int transB, int aH, int aW, long long strideA,
                                   int bH, int bW, long long strideB, long long strideC, int batchCount,
                                   float alpha, const float* A, const float* B, float beta, float* C) {
  int st = enter(h);
  if (st) return st;
  if (aH < 0 || aW < 0 || bH < 0 || bW < 0 || batchCount < 0)
    return fail(h, SNB200_STATUS_INVALID_VALUE, "negative dimension");
  GemmProblem g;
  memset(&g, 0, sizeof(g));
  // Dimension rules of BlasServices.DotMkl (Prod/Data/BlasServices.cs:14-19).
  g.M = transA ? aW : aH;
  g.N = transB ? bH : bW;
  g.K = transA ? aH : aW;
  const int kB = transB ? bW : bH;
  if (g.K != kB)
    return fail(h, SNB200_STATUS_INVALID_VALUE, "inner dimensions differ: op(A) is %dx%d, op(B) is %dx%d", g.M, g.K,
                kB, g.N);
  g.transA = transA ? 1 : 0; g.transB = transB ? 1 : 0;
  g.lda = aW; g.ldb = bW; g.ldc = g.N;
  g.batch = batchCount;
  g.strideA = strideA; g.strideB = strideB; g.strideC = strideC;
  if (batchCount > 1 && (strideA < 0 || strideB < 0 || strideC < static_cast<long long>(g.M) * g.N))
    return fail(h, SNB200_STATUS_INVALID_VALUE, "batch strides must be non-negative and C matrices must not overlap");
  if (g.M == 0 || g.N == 0 || batchCount == 0) return 0;
  st = check_ptrs(h, A, B, C);
  if (st) return st;
  g.A = A; g.B = B; g.C = C;
  g.alpha = alpha; g.beta = beta;
  g.act = ACT_IDENTITY;
  return run_gemm(h, g);
}

extern "C" int snb200_gemm(snb200_handle_t h, int transA, int transB, int aH, int aW, int bH, int bW, float alpha,
                           const float* A, const float* B, float beta, float* C) {
  return snb200_batched_gemm(h, transA, transB, aH, aW, 0, bH, bW, 0, 0, 1, alpha, A, B, beta, C);
}

// ------------------------------------------------------------------------------------ Dense
static bool act_supported(int act) {
  return act == ACT_SIGMOID || act == ACT_RELU || act == ACT_TANH || act == ACT_IDENTITY || act == ACT_SWISH ||
         act == ACT_ELU || act == ACT_LEAKY_RELU || act == ACT_LN || act == ACT_CLIPPED_RELU;
}

static int dense_fwd_impl(snb200_handle_t h, int w_layout, int M, int K, int N, const float* x, const float* W,
                          const float* bias, int act, float* z, float* y, const OutMap* y_map);
static bool row_op_fits(const snb200_context* h, const GemmProblem& g, int max_cols);
static int launch_softmax_fwd(snb200_handle_t h, long long rows, int cols, int causal_rows, const float* x, float* y);
extern "C" int snb200_dense_fwd(snb200_handle_t h, int w_layout, int M, int K, int N, const float* x, const float* W,
                                const float* bias, int act, float* z, float* y) {
  return dense_fwd_impl(h, w_layout, M, K, N, x, W, bias, act, z, y, nullptr);
}
// `y_map`, when given, places y (and z) somewhere else than the dense [M, N] layout.
static int dense_fwd_impl(snb200_handle_t h, int w_layout, int M, int K, int N, const float* x, const float* W,
                          const float* bias, int act, float* z, float* y, const OutMap* y_map) {
  int st = enter(h);
  if (st) return st;
  if (M < 0 || K < 0 || N < 0) return fail(h, SNB200_STATUS_INVALID_VALUE, "negative dimension");
  if (w_layout != SNB200_W_OUT_IN && w_layout != SNB200_W_IN_OUT)
    return fail(h, SNB200_STATUS_INVALID_VALUE, "unknown weight layout %d", w_layout);
  const bool softmax = act == SNB200_ACT_SOFTMAX;   // Dense + Softmax over every row: forward only
  if (softmax) act = ACT_IDENTITY;
  if (!act_supported(act)) return fail(h, SNB200_STATUS_NOT_SUPPORTED, "activation %d is not fused", act);
  if (M == 0 || N == 0) return 0;
  st = check_ptrs(h, x, W, y);
  if (st) return st;
  GemmProblem g;
  memset(&g, 0, sizeof(g));
  g.M = M; g.N = N; g.K = K;
  g.transA = 0; g.lda = K;
  if (w_layout == SNB200_W_OUT_IN) { g.transB = 1; g.ldb = K; }   // y = x * W^T, W [N x K]
  else                             { g.transB = 0; g.ldb = N; }   // y = x * W,   W [K x N]
  g.ldc = N; g.batch = 1;
  g.A = x; g.B = W; g.C = y;
  g.alpha = 1.0f; g.beta = 0.0f;
  g.bias = bias; g.Z = z; g.act = act; g.act_alpha = h->act_alpha;
  if (y_map) g.omap = *y_map;
  if (!softmax) return run_gemm(h, g);
  if (y_map) return fail(h, SNB200_STATUS_NOT_SUPPORTED, "a softmax result is stored densely");
  if (!z && row_op_fits(h, g, 256)) {   // softmax applied where the product is stored
    g.row_op = ROW_SOFTMAX;
    return run_gemm(h, g);
  }
  st = run_gemm(h, g);                   // logits (also kept in z when asked for), then one in-place pass
  if (st) return st;
  return launch_softmax_fwd(h, M, N, 0, y, y);
}

template <bool FUSE>
static int launch_colsum(snb200_handle_t h, int M, int N, int act, const float* dy, const float* y, const float* z,
                         float* dz, float* db, float scale = 1.0f) {
  const bool vec = (N % 4 == 0) && aligned16(dy) && (!FUSE || (aligned16(y) && aligned16(dz) && (!z || aligned16(z))));
  const int cols_per_block = vec ? 128 : 32;
  const int col_blocks = (N + cols_per_block - 1) / cols_per_block;
  int slabs = (4 * h->sm_count + col_blocks - 1) / col_blocks;
  const int max_slabs_rows = (M + 7) / 8;
  if (slabs > max_slabs_rows) slabs = max_slabs_rows;
  const long long ws_slabs = static_cast<long long>(h->workspace_floats / (N > 0 ? N : 1));
  if (slabs > ws_slabs) slabs = static_cast<int>(ws_slabs);
  if (slabs < 1) slabs = 1;
  if (slabs > 65535) slabs = 65535;
  const int rows_per_slab = (M + slabs - 1) / slabs;
  slabs = (M + rows_per_slab - 1) / rows_per_slab;
  if (slabs > 1 && static_cast<size_t>(slabs) * N > h->workspace_floats)
    return fail(h, SNB200_STATUS_NOT_SUPPORTED, "row width %d exceeds the reduction workspace", N);
  float* out = db ? (slabs == 1 ? db : h->workspace) : nullptr;
  dim3 grid(col_blocks, slabs);
  if (vec)
    launch_pdl(h, colsum_slab_kernel<4, FUSE>, grid, dim3(256), M, N, rows_per_slab, act, dy, y, z, dz, out, scale, h->act_alpha);
  else
    launch_pdl(h, colsum_slab_kernel<1, FUSE>, grid, dim3(256), M, N, rows_per_slab, act, dy, y, z, dz, out, scale, h->act_alpha);
  int launches = 1;
  if (db && slabs > 1) {
    launch_pdl(h, colsum_finish_kernel, dim3((N + 255) / 256), dim3(256), N, slabs, h->workspace, db);
    ++launches;
  }
  note_kernel(h, FUSE ? "dz_db_colsum" : "colsum", launches);
  return check_launch(h, "colsum launch");
}

static int ew_grid(const snb200_context* h, long long n, int block) {
  long long want = (n + block - 1) / block;
  const long long cap = static_cast<long long>(h->sm_count) * 16;
  if (want > cap) want = cap;
  return static_cast<int>(want < 1 ? 1 : want);
}

static bool loss_scale(int loss, int N, float* scale) {
  switch (loss) {
    case SNB200_LOSS_BINARY_CROSSENTROPY: *scale = 1.0f / N; return true;      // Prod/Data/Tensor.cs:1379-1387
    case SNB200_LOSS_CATEGORICAL_CROSSENTROPY: *scale = 1.0f; return true;     // :1389-1395
    case SNB200_LOSS_MSE: *scale = 2.0f / N; return true;                      // Prod/CPU/CpuTensor.cs:2466-2475
    default: return false;
  }
}

// dW and dx of the Dense backward from dz (the gradient w.r.t. the pre-activation).
static int dense_bwd_gemms(snb200_handle_t h, int w_layout, int M, int K, int N, const float* x, const float* W,
                           const float* dz, float dW_multiplier, float* dx, float* dW, const OutMap* dx_map = nullptr) {
  int st = 0;
  GemmProblem g;
  memset(&g, 0, sizeof(g));
  g.batch = 1; g.act = ACT_IDENTITY; g.beta = 0.0f;
  // dW, in the layout of W.
  if (w_layout == SNB200_W_OUT_IN) {   // dW [N x K] = mult * dz^T * x          (Linear.cs:158)
    g.M = N; g.N = K; g.K = M;
    g.transA = 1; g.A = dz; g.lda = N;
    g.transB = 0; g.B = x; g.ldb = K;
  } else {                             // dW [K x N] = mult * x^T * dz
    g.M = K; g.N = N; g.K = M;
    g.transA = 1; g.A = x; g.lda = K;
    g.transB = 0; g.B = dz; g.ldb = N;
  }
  g.C = dW; g.ldc = g.N; g.alpha = dW_multiplier;
  if (dW) {
    st = run_gemm(h, g);
    if (st) return st;
  }
  if (dx) {
    g.M = M; g.N = K; g.K = N;
    g.transA = 0; g.A = dz; g.lda = N;
    if (w_layout == SNB200_W_OUT_IN) { g.transB = 0; g.B = W; g.ldb = K; }   // dx = dz * W      (Linear.cs:190)
    else                             { g.transB = 1; g.B = W; g.ldb = N; }   // dx = dz * W^T
    g.C = dx; g.ldc = K; g.alpha = 1.0f;
    if (dx_map) g.omap = *dx_map;
    st = run_gemm(h, g);
    if (st) return st;
  }
  return 0;
}

// Rows [row0, row0 + rows) of the weight gradient, in the layout of W, from the layer's input and dz: the product
// dense_bwd_gemms runs for dW, restricted to a panel of its result.  A host that sums gradients across replicas
// cuts the last large weight gradient of a backward pass into panels and starts the reduction of each panel while
// the next one is computed, so that only the last panel's reduction has nothing to hide behind.
extern "C" int snb200_dense_bwd_weight_rows(snb200_handle_t h, int w_layout, int M, int K, int N, const float* x,
                                            const float* dz, float dW_multiplier, int row0, int rows, float* dW) {
  int st = enter(h);
  if (st) return st;
  if (M < 0 || K < 0 || N < 0 || row0 < 0 || rows < 0) return fail(h, SNB200_STATUS_INVALID_VALUE, "negative dimension");
  if (w_layout != SNB200_W_OUT_IN && w_layout != SNB200_W_IN_OUT)
    return fail(h, SNB200_STATUS_INVALID_VALUE, "unknown weight layout %d", w_layout);
  const int w_rows = w_layout == SNB200_W_OUT_IN ? N : K, w_cols = w_layout == SNB200_W_OUT_IN ? K : N;
  if (row0 + static_cast<long long>(rows) > w_rows)
    return fail(h, SNB200_STATUS_INVALID_VALUE, "rows %d .. %lld of a weight matrix of %d rows", row0,
                row0 + static_cast<long long>(rows), w_rows);
  if (rows == 0 || w_cols == 0) return 0;
  st = check_ptrs(h, x, dz, dW);
  if (st) return st;
  GemmProblem g;
  memset(&g, 0, sizeof(g));
  g.batch = 1; g.act = ACT_IDENTITY; g.beta = 0.0f;
  g.M = rows; g.N = w_cols; g.K = M;
  g.transA = 1; g.transB = 0;
  if (w_layout == SNB200_W_OUT_IN) { g.A = dz + row0; g.lda = N; g.B = x; g.ldb = K; }    // dz[:, row0 ..]^T * x
  else                             { g.A = x + row0; g.lda = K; g.B = dz; g.ldb = N; }    // x[:, row0 ..]^T * dz
  g.C = dW + static_cast<long long>(row0) * w_cols; g.ldc = w_cols; g.alpha = dW_multiplier;
  return run_gemm(h, g);
}

extern "C" int snb200_loss_gradient(snb200_handle_t h, int loss, int rows, int cols, const float* yExpected,
                                    const float* yPredicted, float* dy) {
  int st = enter(h);
  if (st) return st;
  if (rows < 0 || cols < 0) return fail(h, SNB200_STATUS_INVALID_VALUE, "negative dimension");
  float scale;
  if (!loss_scale(loss, cols, &scale)) return fail(h, SNB200_STATUS_NOT_SUPPORTED, "loss %d is not implemented", loss);
  const long long n = static_cast<long long>(rows) * cols;
  if (n == 0) return 0;
  if (!yExpected || !yPredicted || !dy) return fail(h, SNB200_STATUS_INVALID_VALUE, "null pointer");
  if (aligned16(yExpected) && aligned16(yPredicted) && aligned16(dy))
    launch_pdl(h, loss_gradient_kernel<4>, dim3(ew_grid(h, n / 4 + 1, 256)), dim3(256), n, scale, yExpected, yPredicted, dy);
  else
    launch_pdl(h, loss_gradient_kernel<1>, dim3(ew_grid(h, n, 256)), dim3(256), n, scale, yExpected, yPredicted, dy);
  note_kernel(h, "loss_gradient", 1);
  return check_launch(h, "loss_gradient launch");
}

extern "C" int snb200_dense_bwd_from_loss(snb200_handle_t h, int w_layout, int M, int K, int N, const float* x,
                                          const float* W, int loss, const float* yExpected, const float* yPredicted,
                                          float dW_multiplier, float* dz_scratch, float* dx, float* dW, float* db) {
  int st = enter(h);
  if (st) return st;
  if (M < 0 || K < 0 || N < 0) return fail(h, SNB200_STATUS_INVALID_VALUE, "negative dimension");
  if (w_layout != SNB200_W_OUT_IN && w_layout != SNB200_W_IN_OUT)
    return fail(h, SNB200_STATUS_INVALID_VALUE, "unknown weight layout %d", w_layout);
  float scale;
  if (!loss_scale(loss, N, &scale)) return fail(h, SNB200_STATUS_NOT_SUPPORTED, "loss %d is not implemented", loss);
  st = check_ptrs(h, x, W, yPredicted);
  if (st) return st;
  if (!yExpected || !dz_scratch || !dW) return fail(h, SNB200_STATUS_INVALID_VALUE, "null pointer");
  if (M > 0 && N > 0) {
    st = launch_colsum<true>(h, M, N, ACT_LOSS_DIFF, yPredicted, yExpected, nullptr, dz_scratch, db, scale);
    if (st) return st;
  }
  return dense_bwd_gemms(h, w_layout, M, K, N, x, W, dz_scratch, dW_multiplier, dx, dW);
}

static int dense_bwd_impl(snb200_handle_t h, int w_layout, int M, int K, int N, const float* x, const float* W,
                          const float* dy, int act, const float* y, const float* z, float dW_multiplier,
                          float* dz_scratch, float* dx, float* dW, float* db, const OutMap* dx_map);
extern "C" int snb200_dense_bwd(snb200_handle_t h, int w_layout, int M, int K, int N, const float* x, const float* W,
                                const float* dy, int act, const float* y, const float* z, float dW_multiplier,
                                float* dz_scratch, float* dx, float* dW, float* db) {
  return dense_bwd_impl(h, w_layout, M, K, N, x, W, dy, act, y, z, dW_multiplier, dz_scratch, dx, dW, db, nullptr);
}
// `dx_map`, when given, places dx somewhere else than the dense [M, K] layout.
static int dense_bwd_impl(snb200_handle_t h, int w_layout, int M, int K, int N, const float* x, const float* W,
                          const float* dy, int act, const float* y, const float* z, float dW_multiplier,
                          float* dz_scratch, float* dx, float* dW, float* db, const OutMap* dx_map) {
  int st = enter(h);
  if (st) return st;
  if (M < 0 || K < 0 || N < 0) return fail(h, SNB200_STATUS_INVALID_VALUE, "negative dimension");
  if (w_layout != SNB200_W_OUT_IN && w_layout != SNB200_W_IN_OUT)
    return fail(h, SNB200_STATUS_INVALID_VALUE, "unknown weight layout %d", w_layout);
  if (!act_supported(act)) return fail(h, SNB200_STATUS_NOT_SUPPORTED, "activation %d is not fused", act);
  st = check_ptrs(h, x, W, dy);
  if (st) return st;
  if (!dW && !dx && !db) return fail(h, SNB200_STATUS_INVALID_VALUE, "dW, dx and db are all null: nothing to compute");
  const float* dz = dy;
  if (act != ACT_IDENTITY) {
    if (!y) return fail(h, SNB200_STATUS_INVALID_VALUE, "activation output y is required for this activation");
    if (act_needs_input(act) && !z) return fail(h, SNB200_STATUS_INVALID_VALUE, "pre-activation z is required for SWISH, ELU and LN");
    if (!dz_scratch) return fail(h, SNB200_STATUS_INVALID_VALUE, "dz_scratch is required for this activation");
    if (M > 0 && N > 0) {
      st = launch_colsum<true>(h, M, N, act, dy, y, z, dz_scratch, db);   // dz and db in one pass over dy
      if (st) return st;
    }
    dz = dz_scratch;
  } else if (db && M > 0 && N > 0) {
    st = launch_colsum<false>(h, M, N, act, dy, nullptr, nullptr, nullptr, db);
    if (st) return st;
  }
  return dense_bwd_gemms(h, w_layout, M, K, N, x, W, dz, dW_multiplier, dx, dW, dx_map);
}

// ------------------------------------------------------------------------------------ companions

extern "C" int snb200_bias_add(snb200_handle_t h, int M, int N, const float* bias, float* y) {
  int st = enter(h);
  if (st) return st;
  if (M < 0 || N < 0) return fail(h, SNB200_STATUS_INVALID_VALUE, "negative dimension");
  if (M == 0 || N == 0) return 0;
  if (!bias || !y) return fail(h, SNB200_STATUS_INVALID_VALUE, "null pointer");
  const long long total = static_cast<long long>(M) * N;
  if (N % 4 == 0 && aligned16(bias) && aligned16(y))
    launch_pdl(h, bias_add_vec4_kernel, dim3(ew_grid(h, total / 4, 256)), dim3(256), 
        total / 4, N / 4, reinterpret_cast<const float4*>(bias), reinterpret_cast<float4*>(y));
  else
    launch_pdl(h, bias_add_kernel, dim3(ew_grid(h, total, 256)), dim3(256), total, N, bias, y);
  note_kernel(h, "bias_add", 1);
  return check_launch(h, "bias_add launch");
}

extern "C" int snb200_bias_grad(snb200_handle_t h, int M, int N, const float* dy, float* db) {
  int st = enter(h);
  if (st) return st;
  if (M < 0 || N < 0) return fail(h, SNB200_STATUS_INVALID_VALUE, "negative dimension");
  if (N == 0) return 0;
  if (!db || (M > 0 && !dy)) return fail(h, SNB200_STATUS_INVALID_VALUE, "null pointer");
  if (M == 0) {
    SNB_CUDA(h, cudaMemsetAsync(db, 0, sizeof(float) * N, h->stream));
    return 0;
  }
  return launch_colsum<false>(h, M, N, ACT_IDENTITY, dy, nullptr, nullptr, nullptr, db);
}

extern "C" int snb200_activation_fwd(snb200_handle_t h, int act, long long count, const float* x, float* y) {
  int st = enter(h);
  if (st) return st;
  if (count < 0) return fail(h, SNB200_STATUS_INVALID_VALUE, "negative count");
  if (!act_supported(act)) return fail(h, SNB200_STATUS_NOT_SUPPORTED, "activation %d is not implemented", act);
  if (count == 0) return 0;
  if (!x || !y) return fail(h, SNB200_STATUS_INVALID_VALUE, "null pointer");
  if (aligned16(x) && aligned16(y))
    launch_pdl(h, activation_fwd_kernel<4>, dim3(ew_grid(h, count / 4 + 1, 256)), dim3(256), act, h->act_alpha, count, x, y);
  else
    launch_pdl(h, activation_fwd_kernel<1>, dim3(ew_grid(h, count, 256)), dim3(256), act, h->act_alpha, count, x, y);
  note_kernel(h, "activation_fwd", 1);
  return check_launch(h, "activation_fwd launch");
}

extern "C" int snb200_activation_bwd(snb200_handle_t h, int act, long long count, const float* dy, const float* x,
                                     const float* y, float* dx) {
  int st = enter(h);
  if (st) return st;
  if (count < 0) return fail(h, SNB200_STATUS_INVALID_VALUE, "negative count");
  if (!act_supported(act)) return fail(h, SNB200_STATUS_NOT_SUPPORTED, "activation %d is not implemented", act);
  if (count == 0) return 0;
  if (!dy || !dx || (act != ACT_IDENTITY && !y) || (act_needs_input(act) && !x))
    return fail(h, SNB200_STATUS_INVALID_VALUE, "null pointer");
  if (aligned16(dy) && aligned16(dx) && (!x || aligned16(x)) && (!y || aligned16(y)))
    launch_pdl(h, activation_bwd_kernel<4>, dim3(ew_grid(h, count / 4 + 1, 256)), dim3(256), act, h->act_alpha, count, dy, x, y, dx);
  else
    launch_pdl(h, activation_bwd_kernel<1>, dim3(ew_grid(h, count, 256)), dim3(256), act, h->act_alpha, count, dy, x, y, dx);
  note_kernel(h, "activation_bwd", 1);
  return check_launch(h, "activation_bwd launch");
}

extern "C" int snb200_axpy(snb200_handle_t h, long long count, float alpha, const float* x, float* y) {
  int st = enter(h);
  if (st) return st;
  if (count < 0) return fail(h, SNB200_STATUS_INVALID_VALUE, "negative count");
  if (count == 0) return 0;
  if (!x || !y) return fail(h, SNB200_STATUS_INVALID_VALUE, "null pointer");
  if (aligned16(x) && aligned16(y))
    launch_pdl(h, axpy_kernel<4>, dim3(ew_grid(h, count / 4 + 1, 256)), dim3(256), count, alpha, x, y);
  else
    launch_pdl(h, axpy_kernel<1>, dim3(ew_grid(h, count, 256)), dim3(256), count, alpha, x, y);
  note_kernel(h, "axpy", 1);
  return check_launch(h, "axpy launch");
}

extern "C" int snb200_transpose_second_third(snb200_handle_t h, int A, int B, int C, int D, const float* src,
                                             float* dst) {
  int st = enter(h);
  if (st) return st;
  if (A < 0 || B < 0 || C < 0 || D < 0) return fail(h, SNB200_STATUS_INVALID_VALUE, "negative dimension");
  const long long total = static_cast<long long>(A) * B * C * D;
  if (total == 0) return 0;
  if (!src || !dst) return fail(h, SNB200_STATUS_INVALID_VALUE, "null pointer");
  if (src == dst) return fail(h, SNB200_STATUS_INVALID_VALUE, "the permutation is not done in place");
  if (D % 4 == 0 && aligned16(src) && aligned16(dst))
    launch_pdl(h, transpose_second_third_kernel<4>, dim3(ew_grid(h, total / 4, 256)), dim3(256), total / 4, B, C, D / 4, src, dst);
  else
    launch_pdl(h, transpose_second_third_kernel<1>, dim3(ew_grid(h, total, 256)), dim3(256), total, B, C, D, src, dst);
  note_kernel(h, "transpose_second_third", 1);
  return check_launch(h, "transpose_second_third launch");
}

extern "C" int snb200_sgd_update(snb200_handle_t h, long long count, float learning_rate, float momentum, int nesterov,
                                 const float* dW, float* W, float* velocity) {
  int st = enter(h);
  if (st) return st;
  if (count < 0) return fail(h, SNB200_STATUS_INVALID_VALUE, "negative count");
  if (count == 0) return 0;
  if (!dW || !W) return fail(h, SNB200_STATUS_INVALID_VALUE, "null pointer");
  if (aligned16(dW) && aligned16(W) && (!velocity || aligned16(velocity)))
    launch_pdl(h, sgd_update_kernel<4>, dim3(ew_grid(h, count / 4 + 1, 256)), dim3(256), count, learning_rate, momentum,
                                                                               nesterov ? 1 : 0, dW, W, velocity);
  else
    launch_pdl(h, sgd_update_kernel<1>, dim3(ew_grid(h, count, 256)), dim3(256), count, learning_rate, momentum,
                                                                       nesterov ? 1 : 0, dW, W, velocity);
  note_kernel(h, "sgd_update", 1);
  return check_launch(h, "sgd_update launch");
}

extern "C" int snb200_adam_update(snb200_handle_t h, long long count, double learning_rate, double beta1, double beta2,
                                  double epsilon, double weight_decay, int time_step, const float* dW, float* W,
                                  float* adam_vW, float* adam_sW) {
  int st = enter(h);
  if (st) return st;
  if (count < 0 || time_step < 1) return fail(h, SNB200_STATUS_INVALID_VALUE, "negative count or time step below 1");
  if (count == 0) return 0;
  if (!dW || !W || !adam_vW || !adam_sW) return fail(h, SNB200_STATUS_INVALID_VALUE, "null pointer");
  const double b1p = pow(beta1, time_step), b2p = pow(beta2, time_step);
  const double factor = learning_rate * (sqrt(1.0 - b2p) / (1.0 - b1p));
  const float b1 = static_cast<float>(beta1), b2 = static_cast<float>(beta2), ep = static_cast<float>(epsilon);
  const float wd = static_cast<float>(weight_decay), fc = static_cast<float>(factor);
  if (aligned16(dW) && aligned16(W) && aligned16(adam_vW) && aligned16(adam_sW))
    launch_pdl(h, adam_update_kernel<4>, dim3(ew_grid(h, count / 4 + 1, 256)), dim3(256), count, b1, b2, ep, wd, fc, dW, W, adam_vW,
                                                                                adam_sW);
  else
    launch_pdl(h, adam_update_kernel<1>, dim3(ew_grid(h, count, 256)), dim3(256), count, b1, b2, ep, wd, fc, dW, W, adam_vW, adam_sW);
  note_kernel(h, "adam_update", 1);
  return check_launch(h, "adam_update launch");
}

// ------------------------------------------------------------------------------------ attention
static int launch_softmax_fwd(snb200_handle_t h, long long rows, int cols, int causal_rows, const float* x, float* y) {
  long long blocks = (rows + 7) / 8;   // 8 warps (rows) per block
  const long long cap = 16LL * h->sm_count;
  if (blocks > cap) blocks = cap;
  const unsigned g = static_cast<unsigned>(blocks < 1 ? 1 : blocks);
  // many short rows: several rows per warp at a time (more loads in flight per lane)
  const bool many = rows >= 64LL * h->sm_count;
  if (cols <= 128 && many) {
    const long long b4 = (rows + 31) / 32;
    launch_pdl(h, softmax_fwd_rows_kernel<4, 4>, dim3(static_cast<unsigned>(b4 < cap ? b4 : cap)), dim3(256), rows, cols, causal_rows, x, y);
  } else if (cols <= 256 && many) {
    const long long b2 = (rows + 15) / 16;
    launch_pdl(h, softmax_fwd_rows_kernel<8, 2>, dim3(static_cast<unsigned>(b2 < cap ? b2 : cap)), dim3(256), rows, cols, causal_rows, x, y);
  } else if (cols <= 128) launch_pdl(h, softmax_fwd_kernel<4>, dim3(g), dim3(256), rows, cols, causal_rows, x, y);
  else if (cols <= 256) launch_pdl(h, softmax_fwd_kernel<8>, dim3(g), dim3(256), rows, cols, causal_rows, x, y);
  else if (cols <= 512) launch_pdl(h, softmax_fwd_kernel<16>, dim3(g), dim3(256), rows, cols, causal_rows, x, y);
  else if (cols <= 1024) launch_pdl(h, softmax_fwd_kernel<32>, dim3(g), dim3(256), rows, cols, causal_rows, x, y);
  else launch_pdl(h, softmax_fwd_kernel<0>, dim3(g), dim3(256), rows, cols, causal_rows, x, y);
  note_kernel(h, "softmax_fwd", 1);
  return check_launch(h, "softmax_fwd launch");
}
static int launch_softmax_bwd(snb200_handle_t h, long long rows, int cols, const float* dy, const float* y, float* dx) {
  long long blocks = (rows + 7) / 8;
  const long long cap = 16LL * h->sm_count;
  if (blocks > cap) blocks = cap;
  launch_pdl(h, softmax_bwd_kernel, dim3(static_cast<unsigned>(blocks < 1 ? 1 : blocks)), dim3(256), rows, cols, dy, y, dx);
  note_kernel(h, "softmax_bwd", 1);
  return check_launch(h, "softmax_bwd launch");
}

extern "C" int snb200_softmax_fwd(snb200_handle_t h, long long rows, int cols, const float* x, float* y) {
  int st = enter(h);
  if (st) return st;
  if (rows < 0 || cols < 0) return fail(h, SNB200_STATUS_INVALID_VALUE, "negative dimension");
  if (rows == 0 || cols == 0) return 0;
  if (!x || !y) return fail(h, SNB200_STATUS_INVALID_VALUE, "null pointer");
  return launch_softmax_fwd(h, rows, cols, 0, x, y);
}
extern "C" int snb200_softmax_bwd(snb200_handle_t h, long long rows, int cols, const float* dy, const float* y,
                                  float* dx) {
  int st = enter(h);
  if (st) return st;
  if (rows < 0 || cols < 0) return fail(h, SNB200_STATUS_INVALID_VALUE, "negative dimension");
  if (rows == 0 || cols == 0) return 0;
  if (!dy || !y || !dx) return fail(h, SNB200_STATUS_INVALID_VALUE, "null pointer");
  return launch_softmax_bwd(h, rows, cols, dy, y, dx);
}

static void bmm_problem(GemmProblem* g, int batch, int M, int N, int K, int tA, int tB, const float* A, int lda,
                        long long sA, const float* B, int ldb, long long sB, float* C, float alpha) {
  memset(g, 0, sizeof(*g));
  g->M = M; g->N = N; g->K = K; g->transA = tA; g->transB = tB;
  g->A = A; g->lda = lda; g->strideA = sA;
  g->B = B; g->ldb = ldb; g->strideB = sB;
  g->C = C; g->ldc = N; g->strideC = static_cast<long long>(M) * N;
  g->batch = batch; g->alpha = alpha; g->beta = 0.0f; g->act = ACT_IDENTITY;
}

// Can the product run on the tensor-core kernel with its whole rows in one tile, so that a row operation
// (softmax, softmax gradient; rows of up to 256 columns) can be applied where the product is stored?  Otherwise the caller runs the plain
// product and a separate row pass.
static bool row_op_fits(const snb200_context* h, const GemmProblem& g, int max_cols) {
  if (h->math_mode == SNB200_MATH_FP32_SIMT || h->tune[TUNE_FORCE_PATH] == 2 || !tma_eligible(g)) return false;
  if (g.N > max_cols || g.N < 8 || g.M < 16) return false;
  // the row operation reads and writes whole float4s of 16-byte aligned rows
  if ((g.N & 3) || !aligned16(g.C) || (g.aux && !aligned16(g.aux)) || (g.batch > 1 && (g.strideC & 3))) return false;
  return static_cast<double>(g.M) * g.N * g.K * g.batch >= 64.0 * 64 * 64;
}

// The attention core as one kernel (attn_fwd_kernel): score rows of up to 128 columns, embeddings of up to 128, the
// 3xTF32 mode, operands TMA can load.  Returns -1 when the case does not qualify (the caller then runs the products
// one by one).
template <class T, bool GRAD = false>
static int launch_attn_fwd_t(snb200_handle_t h, const AttnParams& ap, const float* Q, const float* K, const float* V) {
  static bool configured[64] = {};
  auto kernel = GRAD ? attn_bwd_kernel<T> : attn_fwd_kernel<T>;
  CUtensorMap tmQ, tmK, tmV;
  const uint64_t B = ap.batch, Tq = ap.q_steps, Tk = ap.v_steps, E = ap.embedding_dim;
  bool ok = encode_3d(&tmQ, Q, E, Tq, B, E, Tq * E, 32, 128, CU_TENSOR_MAP_SWIZZLE_128B) &&
            encode_3d(&tmK, K, E, Tk, B, E, Tk * E, 32, T::TKN, CU_TENSOR_MAP_SWIZZLE_128B) &&
            encode_3d(&tmV, V, E, Tk, B, E, Tk * E, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
  if (!ok) return fail(h, SNB200_STATUS_INTERNAL_ERROR, "cuTensorMapEncodeTiled rejected an attention operand");
  if (!configured[h->device]) {
    SNB_CUDA(h, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES));
    configured[h->device] = true;
  }
  const long long units = static_cast<long long>(ap.batch) * ap.tiles_q;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.gridDim = dim3(static_cast<unsigned>(units < h->sm_count ? units : h->sm_count));
  cfg.blockDim = dim3(T::THREADS);
  cfg.dynamicSmemBytes = T::SMEM_BYTES;
  cfg.stream = h->stream;
  cfg.attrs = attr;
  cfg.numAttrs = h->tune[TUNE_PDL] == 1 ? 0 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tmQ, tmK, tmV, ap);
  if (e != cudaSuccess) return cuda_fail(h, e, "attention kernel launch");
  return check_launch(h, "attention kernel launch");
}

static int try_fused_attention_fwd(snb200_handle_t h, int batch, int Tq, int Tk, int E, float scaling, int is_causal,
                                   const float* Q, const float* K, const float* V, float* weights, float* y,
                                   const OutMap* y_map) {
  if (h->tune[TUNE_NO_FUSED_ATTN] == 1 || h->tune[TUNE_FORCE_PATH] == 2) return -1;
  if (h->math_mode != SNB200_MATH_3XTF32 && h->math_mode != SNB200_MATH_TF32_BF16X2) return -1;
  if (Tk > 128 || E > 128 || Tk < 8 || Tq < 16 || (E & 3)) return -1;
  if (!aligned16(Q) || !aligned16(K) || !aligned16(V)) return -1;
  if (static_cast<double>(batch) * Tq * Tk * E < 64.0 * 64 * 64) return -1;
  if (static_cast<long long>(batch) * ((Tq + 127) / 128) > 0x7fffffffLL) return -1;
  AttnParams ap;
  memset(&ap, 0, sizeof(ap));
  ap.batch = batch; ap.q_steps = Tq; ap.v_steps = Tk; ap.embedding_dim = E;
  ap.tiles_q = (Tq + 127) / 128;
  ap.error_word = h->error_word;
  UmmaParams& s = ap.s;
  s.M = Tq; s.N = Tk; s.K = E; s.batch = batch;
  s.ldc = Tk; s.strideC = static_cast<long long>(Tq) * Tk;
  s.C = weights; s.alpha = scaling; s.beta = 0.0f; s.act = ACT_IDENTITY;
  s.row_op = ROW_SOFTMAX; s.causal = is_causal ? 1 : 0;
  s.vec_ok = aligned16(weights) && (Tk % 4 == 0);
  UmmaParams& o = ap.o;
  o.M = Tq; o.N = E; o.K = Tk; o.batch = batch;
  o.ldc = E; o.strideC = static_cast<long long>(Tq) * E;
  o.C = y; o.alpha = 1.0f; o.beta = 0.0f; o.act = ACT_IDENTITY;
  o.vec_ok = aligned16(y);
  if (y_map) { o.omap = *y_map; if (!omap_vec(*y_map)) o.vec_ok = 0; }
#ifdef SNB_TRACE
  s.trace = reinterpret_cast<unsigned long long*>(h->workspace + (h->workspace_floats - 128));
#endif
  const int tkn = Tk <= 32 ? 32 : Tk <= 64 ? 64 : 128, en = E <= 32 ? 32 : E <= 64 ? 64 : 128;
  char name[64];
  snprintf(name, sizeof(name), "attention_fwd_3xtf32_%dx%d", tkn, en);
  note_kernel(h, name, 1);
#define SNB_ATTN_CASE(TK, EE) if (tkn == TK && en == EE) return launch_attn_fwd_t<AttnTile<TK, EE>>(h, ap, Q, K, V)
  SNB_ATTN_CASE(32, 32); SNB_ATTN_CASE(32, 64); SNB_ATTN_CASE(32, 128);
  SNB_ATTN_CASE(64, 32); SNB_ATTN_CASE(64, 64); SNB_ATTN_CASE(64, 128);
  SNB_ATTN_CASE(128, 32); SNB_ATTN_CASE(128, 64); SNB_ATTN_CASE(128, 128);
#undef SNB_ATTN_CASE
  return -1;
}

// The middle of the backward pass in one launch of the same kernel body: dScores = softmax'(scaling dy V^T; weights)
// stored to `scores_grad` (the dK product reads it) and dQ = dScores K.  Same conditions as the forward kernel, plus
// probability rows that are 16-byte aligned.  Returns -1 when the case does not qualify.
static int try_fused_attention_bwd(snb200_handle_t h, int batch, int Tq, int Tk, int E, float scaling, const float* dy,
                                   const float* V, const float* K, const float* weights, float* scores_grad, float* dQ,
                                   const OutMap* dq_map) {
  if (h->tune[TUNE_NO_FUSED_ATTN] == 1 || h->tune[TUNE_FORCE_PATH] == 2) return -1;
  if (h->math_mode != SNB200_MATH_3XTF32 && h->math_mode != SNB200_MATH_TF32_BF16X2) return -1;
  if (Tk > 128 || E > 128 || Tk < 8 || Tq < 16 || (E & 3) || (Tk & 3)) return -1;
  if (!aligned16(dy) || !aligned16(K) || !aligned16(V) || !aligned16(weights) || !aligned16(scores_grad)) return -1;
  if (static_cast<double>(batch) * Tq * Tk * E < 64.0 * 64 * 64) return -1;
  if (static_cast<long long>(batch) * ((Tq + 127) / 128) > 0x7fffffffLL) return -1;
  AttnParams ap;
  memset(&ap, 0, sizeof(ap));
  ap.batch = batch; ap.q_steps = Tq; ap.v_steps = Tk; ap.embedding_dim = E;
  ap.tiles_q = (Tq + 127) / 128;
  ap.error_word = h->error_word;
  UmmaParams& s = ap.s;
  s.M = Tq; s.N = Tk; s.K = E; s.batch = batch;
  s.ldc = Tk; s.strideC = static_cast<long long>(Tq) * Tk;
  s.C = scores_grad; s.aux = weights; s.alpha = scaling; s.beta = 0.0f; s.act = ACT_IDENTITY;
  s.row_op = ROW_SOFTMAX_GRAD;
  s.vec_ok = 1;
  UmmaParams& o = ap.o;
  o.M = Tq; o.N = E; o.K = Tk; o.batch = batch;
  o.ldc = E; o.strideC = static_cast<long long>(Tq) * E;
  o.C = dQ; o.alpha = 1.0f; o.beta = 0.0f; o.act = ACT_IDENTITY;
  o.vec_ok = aligned16(dQ);
  if (dq_map) { o.omap = *dq_map; if (!omap_vec(*dq_map)) o.vec_ok = 0; }
#ifdef SNB_TRACE
  s.trace = reinterpret_cast<unsigned long long*>(h->workspace + (h->workspace_floats - 128));
#endif
  const int tkn = Tk <= 32 ? 32 : Tk <= 64 ? 64 : 128, en = E <= 32 ? 32 : E <= 64 ? 64 : 128;
  char name[64];
  snprintf(name, sizeof(name), "attention_bwd_3xtf32_%dx%d", tkn, en);
  note_kernel(h, name, 1);
#define SNB_ATTN_CASE(TK, EE) if (tkn == TK && en == EE) return launch_attn_fwd_t<AttnTile<TK, EE>, true>(h, ap, dy, V, K)
  SNB_ATTN_CASE(32, 32); SNB_ATTN_CASE(32, 64); SNB_ATTN_CASE(32, 128);
  SNB_ATTN_CASE(64, 32); SNB_ATTN_CASE(64, 64); SNB_ATTN_CASE(64, 128);
  SNB_ATTN_CASE(128, 32); SNB_ATTN_CASE(128, 64); SNB_ATTN_CASE(128, 128);
#undef SNB_ATTN_CASE
  return -1;
}

static int sdpa_fwd_impl(snb200_handle_t h, int batch, int q_steps, int v_steps, int embedding_dim, int use_scale,
                         int is_causal, const float* Q, const float* K, const float* V, float* weights, float* y,
                         const OutMap* y_map);
extern "C" int snb200_sdpa_fwd(snb200_handle_t h, int batch, int q_steps, int v_steps, int embedding_dim,
                               int use_scale, int is_causal, const float* Q, const float* K, const float* V,
                               float* weights, float* y) {
  return sdpa_fwd_impl(h, batch, q_steps, v_steps, embedding_dim, use_scale, is_causal, Q, K, V, weights, y, nullptr);
}
static int sdpa_fwd_impl(snb200_handle_t h, int batch, int q_steps, int v_steps, int embedding_dim, int use_scale,
                         int is_causal, const float* Q, const float* K, const float* V, float* weights, float* y,
                         const OutMap* y_map) {
  int st = enter(h);
  if (st) return st;
  if (batch < 0 || q_steps < 0 || v_steps < 0 || embedding_dim < 0)
    return fail(h, SNB200_STATUS_INVALID_VALUE, "negative dimension");
  if (batch == 0 || q_steps == 0 || v_steps == 0 || embedding_dim == 0) return 0;
  st = check_ptrs(h, Q, K, V);
  if (st) return st;
  if (!weights || !y) return fail(h, SNB200_STATUS_INVALID_VALUE, "null pointer");
  const int Tq = q_steps, Tk = v_steps, E = embedding_dim;
  const float scaling = use_scale ? 1.0f / sqrtf(static_cast<float>(E)) : 1.0f;
  // both products, the mask and the softmax in one kernel where a score row fits one tile
  st = try_fused_attention_fwd(h, batch, Tq, Tk, E, scaling, is_causal, Q, K, V, weights, y, y_map);
  if (st >= 0) return st;
  GemmProblem g;
  // scores = scaling * Q * K^T                       (ScaledDotProductAttentionLayer.cs:66-71)
  bmm_problem(&g, batch, Tq, Tk, E, 0, 1, Q, E, static_cast<long long>(Tq) * E, K, E, static_cast<long long>(Tk) * E,
              weights, scaling);
  if (row_op_fits(h, g, 256)) {
    // causal mask + softmax over the last dimension where the scores are stored   (:73-81)
    g.row_op = ROW_SOFTMAX; g.causal = is_causal ? 1 : 0;
    st = run_gemm(h, g);
    if (st) return st;
  } else {
    st = run_gemm(h, g);
    if (st) return st;
    // causal mask + softmax over the last dimension, in place   (:73-81)
    st = launch_softmax_fwd(h, static_cast<long long>(batch) * Tq, Tk, is_causal ? Tq : 0, weights, weights);
    if (st) return st;
  }
  // y = weights * V                                   (:85)
  bmm_problem(&g, batch, Tq, E, Tk, 0, 0, weights, Tk, static_cast<long long>(Tq) * Tk, V, E,
              static_cast<long long>(Tk) * E, y, 1.0f);
  if (y_map) g.omap = *y_map;
  return run_gemm(h, g);
}

static int sdpa_bwd_impl(snb200_handle_t h, int batch, int q_steps, int v_steps, int embedding_dim, int use_scale,
                         const float* Q, const float* K, const float* V, const float* dy, const float* weights,
                         float* scores_grad_scratch, float* dQ, float* dK, float* dV, const OutMap* dq_map,
                         const OutMap* dkv_map);
extern "C" int snb200_sdpa_bwd(snb200_handle_t h, int batch, int q_steps, int v_steps, int embedding_dim,
                               int use_scale, const float* Q, const float* K, const float* V, const float* dy,
                               const float* weights, float* scores_grad_scratch, float* dQ, float* dK, float* dV) {
  return sdpa_bwd_impl(h, batch, q_steps, v_steps, embedding_dim, use_scale, Q, K, V, dy, weights, scores_grad_scratch,
                       dQ, dK, dV, nullptr, nullptr);
}
// `dq_map` places dQ, `dkv_map` places dK and dV, when they do not go to the dense per-matrix layout.
static int sdpa_bwd_impl(snb200_handle_t h, int batch, int q_steps, int v_steps, int embedding_dim, int use_scale,
                         const float* Q, const float* K, const float* V, const float* dy, const float* weights,
                         float* scores_grad_scratch, float* dQ, float* dK, float* dV, const OutMap* dq_map,
                         const OutMap* dkv_map) {
  int st = enter(h);
  if (st) return st;
  if (batch < 0 || q_steps < 0 || v_steps < 0 || embedding_dim < 0)
    return fail(h, SNB200_STATUS_INVALID_VALUE, "negative dimension");
  if (batch == 0 || q_steps == 0 || v_steps == 0 || embedding_dim == 0) return 0;
  st = check_ptrs(h, Q, K, V);
  if (st) return st;
  if (!dy || !weights || !scores_grad_scratch || !dQ || !dK || !dV)
    return fail(h, SNB200_STATUS_INVALID_VALUE, "null pointer");
  const int Tq = q_steps, Tk = v_steps, E = embedding_dim;
  const long long sQ = static_cast<long long>(Tq) * E, sK = static_cast<long long>(Tk) * E;
  const long long sW = static_cast<long long>(Tq) * Tk;
  const float scaling = use_scale ? 1.0f / sqrtf(static_cast<float>(E)) : 1.0f;
  GemmProblem g;
  // dScores and dQ in one kernel where a score row fits one tile                       (:119-123)
  st = try_fused_attention_bwd(h, batch, Tq, Tk, E, scaling, dy, V, K, weights, scores_grad_scratch, dQ, dq_map);
  if (st > 0) return st;
  if (st == 0) {
    // dV = weights^T * dy and dK = dScores^T * Q: two products of one shape, one launch where they qualify  (:113,124)
    GemmProblem gk;
    bmm_problem(&g, batch, Tk, E, Tq, 1, 0, weights, Tk, sW, dy, E, sQ, dV, 1.0f);
    bmm_problem(&gk, batch, Tk, E, Tq, 1, 0, scores_grad_scratch, Tk, sW, Q, E, sQ, dK, 1.0f);
    if (dkv_map) { g.omap = *dkv_map; gk.omap = *dkv_map; }
    return run_gemm_pair(h, g, gk);
  }
  // dV = weights^T * dy                               (ScaledDotProductAttentionLayer.cs:113)
  bmm_problem(&g, batch, Tk, E, Tq, 1, 0, weights, Tk, sW, dy, E, sQ, dV, 1.0f);
  if (dkv_map) g.omap = *dkv_map;
  st = run_gemm(h, g);
  if (st) return st;
  // gradient w.r.t. the weights, scaled: scaling * dy * V^T    (:119)
  bmm_problem(&g, batch, Tq, Tk, E, 0, 1, dy, E, sQ, V, E, sK, scores_grad_scratch, scaling);
  g.aux = weights;
  if (row_op_fits(h, g, 128)) {   // measured: beyond 128 columns the 256-wide single-CTA tile loses to pair tiles + a pass
    // ... turned into the gradient w.r.t. the scores by the softmax Jacobian where it is stored    (:121)
    g.row_op = ROW_SOFTMAX_GRAD;
    st = run_gemm(h, g);
    if (st) return st;
  } else {
    st = run_gemm(h, g);
    if (st) return st;
    // ... turned into the gradient w.r.t. the scores by the softmax Jacobian, in place    (:121)
    st = launch_softmax_bwd(h, static_cast<long long>(batch) * Tq, Tk, scores_grad_scratch, weights, scores_grad_scratch);
    if (st) return st;
  }
  // dQ = dScores * K ; dK = dScores^T * Q             (:123-124)
  bmm_problem(&g, batch, Tq, E, Tk, 0, 0, scores_grad_scratch, Tk, sW, K, E, sK, dQ, 1.0f);
  if (dq_map) g.omap = *dq_map;
  st = run_gemm(h, g);
  if (st) return st;
  bmm_problem(&g, batch, Tk, E, Tq, 1, 0, scores_grad_scratch, Tk, sW, Q, E, sQ, dK, 1.0f);
  if (dkv_map) g.omap = *dkv_map;
  return run_gemm(h, g);
}

// ------------------------------------------------------------------------------------ multi-head attention
static long long round64(long long n) { return (n + 63) / 64 * 64; }   // 256-byte granules keep sub-buffers TMA-eligible

static int mha_check(snb200_handle_t h, const snb200_mha_desc* d) {
  if (!d) return fail(h, SNB200_STATUS_INVALID_VALUE, "null descriptor");
  if (d->batch < 0 || d->q_steps < 0 || d->v_steps < 0 || d->embed_dim < 0 || d->num_heads <= 0 || d->key_dim <= 0 ||
      d->value_dim <= 0)
    return fail(h, SNB200_STATUS_INVALID_VALUE, "negative or zero dimension");
  if (d->w_layout != SNB200_W_OUT_IN && d->w_layout != SNB200_W_IN_OUT)
    return fail(h, SNB200_STATUS_INVALID_VALUE, "unknown weight layout %d", d->w_layout);
  if (d->num_heads * d->value_dim != d->embed_dim)
    return fail(h, SNB200_STATUS_INVALID_VALUE, "num_heads * value_dim (%d) must equal embed_dim (%d)",
                d->num_heads * d->value_dim, d->embed_dim);
  return 0;
}

extern "C" long long snb200_mha_scratch_floats(const snb200_mha_desc* d, int backward) {
  if (!d || !backward) return 0;   // the forward pass writes straight into the state tensors
  const long long B = d->batch, Tq = d->q_steps, Tk = d->v_steps, H = d->num_heads, kd = d->key_dim, vd = d->value_dim;
  // d_attention_heads, the gradients of the Q, K, V projections' outputs, the gradient of the scores
  return round64(B * H * Tq * vd) + round64(B * Tq * H * kd) + round64(B * Tk * H * kd) + round64(B * Tk * H * vd) +
         round64(B * H * Tq * Tk);
}

extern "C" int snb200_mha_fwd(snb200_handle_t h, const snb200_mha_desc* d, const snb200_mha_weights* w, const float* Q,
                              const float* K, const float* V, const snb200_mha_state* s, float* scratch, float* y) {
  int st = enter(h);
  if (st) return st;
  st = mha_check(h, d);
  if (st) return st;
  if (!w || !s || !Q || !K || !V || !y || !w->w_Q || !w->w_K || !w->w_V || !w->out_proj_weight ||
      !s->Q_heads_T || !s->K_heads_T || !s->V_heads_T || !s->attention_heads_T || !s->weights_buffer)
    return fail(h, SNB200_STATUS_INVALID_VALUE, "null pointer");
  const int B = d->batch, Tq = d->q_steps, Tk = d->v_steps, E = d->embed_dim, H = d->num_heads, kd = d->key_dim,
            vd = d->value_dim;
  if (B == 0 || Tq == 0 || Tk == 0 || E == 0) return 0;
  // Projections on the last dimension; each product stores its result already split by head, [b, t, h, d] ->
  // [b, h, t, d] (the layer's TransposeSecondAndThirdDimension, :201-218), so no permutation pass runs.
  const OutMap split_q = head_split_map(Tq, H, kd), split_k = head_split_map(Tk, H, kd), split_v = head_split_map(Tk, H, vd);
  st = dense_fwd_impl(h, d->w_layout, B * Tq, E, H * kd, Q, w->w_Q, w->w_Q_bias, ACT_IDENTITY, nullptr, s->Q_heads_T, &split_q);
  if (!st) st = dense_fwd_impl(h, d->w_layout, B * Tk, E, H * kd, K, w->w_K, w->w_K_bias, ACT_IDENTITY, nullptr, s->K_heads_T, &split_k);
  if (!st) st = dense_fwd_impl(h, d->w_layout, B * Tk, E, H * vd, V, w->w_V, w->w_V_bias, ACT_IDENTITY, nullptr, s->V_heads_T, &split_v);
  // attention per head (always scaled, :32,221); its second product stores the heads merged, [b, h, t, d] ->
  // [b, t, h, d]                                                                                        (:220-226)
  if (!st && kd != vd) st = fail(h, SNB200_STATUS_NOT_SUPPORTED, "key_dim and value_dim must be equal");
  const OutMap merge = head_merge_map(Tq, H, vd);
  if (!st) st = sdpa_fwd_impl(h, B * H, Tq, Tk, kd, 1, d->is_causal, s->Q_heads_T, s->K_heads_T, s->V_heads_T,
                              s->weights_buffer, s->attention_heads_T, &merge);
  // output projection                                                                                   (:227)
  if (!st) st = snb200_dense_fwd(h, d->w_layout, B * Tq, H * vd, E, s->attention_heads_T, w->out_proj_weight,
                                 w->out_proj_bias, ACT_IDENTITY, nullptr, y);
  (void)scratch;
  if (!st) note_kernel(h, "multihead_attention_fwd", 0);
  return st;
}

extern "C" int snb200_mha_bwd(snb200_handle_t h, const snb200_mha_desc* d, const snb200_mha_weights* w, const float* Q,
                              const float* K, const float* V, const float* dy, const snb200_mha_state* s,
                              float dW_multiplier, float* scratch, const snb200_mha_gradients* g, float* dQ, float* dK,
                              float* dV) {
  int st = enter(h);
  if (st) return st;
  st = mha_check(h, d);
  if (st) return st;
  if (!w || !s || !g || !scratch || !Q || !K || !V || !dy || !dQ || !dK || !dV || !w->w_Q || !w->w_K || !w->w_V ||
      !w->out_proj_weight || !g->w_Q || !g->w_K || !g->w_V || !g->out_proj_weight || !s->Q_heads_T || !s->K_heads_T ||
      !s->V_heads_T || !s->attention_heads_T || !s->weights_buffer)
    return fail(h, SNB200_STATUS_INVALID_VALUE, "null pointer");
  const int B = d->batch, Tq = d->q_steps, Tk = d->v_steps, E = d->embed_dim, H = d->num_heads, kd = d->key_dim,
            vd = d->value_dim;
  if (B == 0 || Tq == 0 || Tk == 0 || E == 0) return 0;
  if (kd != vd) return fail(h, SNB200_STATUS_NOT_SUPPORTED, "key_dim and value_dim must be equal");
  float* d_heads = scratch;
  float* dQh = d_heads + round64(static_cast<long long>(B) * H * Tq * vd);
  float* dKh = dQh + round64(static_cast<long long>(B) * H * Tq * kd);
  float* dVh = dKh + round64(static_cast<long long>(B) * H * Tk * kd);
  float* dscores = dVh + round64(static_cast<long long>(B) * H * Tk * vd);
  // output projection backward; its dx product stores the gradient already split by head             (:253-260)
  const OutMap split_o = head_split_map(Tq, H, vd);
  st = dense_bwd_impl(h, d->w_layout, B * Tq, H * vd, E, s->attention_heads_T, w->out_proj_weight, dy, ACT_IDENTITY,
                      nullptr, nullptr, dW_multiplier, nullptr, d_heads, g->out_proj_weight, g->out_proj_bias, &split_o);
  // attention backward per head; dQ, dK, dV come out merged, [b, h, t, d] -> [b, t, h, d]               (:266-278)
  const OutMap merge_q = head_merge_map(Tq, H, kd), merge_kv = head_merge_map(Tk, H, kd);
  if (!st) st = sdpa_bwd_impl(h, B * H, Tq, Tk, kd, 1, s->Q_heads_T, s->K_heads_T, s->V_heads_T, d_heads,
                              s->weights_buffer, dscores, dQh, dKh, dVh, &merge_q, &merge_kv);
  // the three input projections backward
  if (!st) st = snb200_dense_bwd(h, d->w_layout, B * Tq, E, H * kd, Q, w->w_Q, dQh, ACT_IDENTITY, nullptr, nullptr,
                                 dW_multiplier, nullptr, dQ, g->w_Q, g->w_Q_bias);
  if (!st) st = snb200_dense_bwd(h, d->w_layout, B * Tk, E, H * kd, K, w->w_K, dKh, ACT_IDENTITY, nullptr, nullptr,
                                 dW_multiplier, nullptr, dK, g->w_K, g->w_K_bias);
  if (!st) st = snb200_dense_bwd(h, d->w_layout, B * Tk, E, H * vd, V, w->w_V, dVh, ACT_IDENTITY, nullptr, nullptr,
                                 dW_multiplier, nullptr, dV, g->w_V, g->w_V_bias);
  if (!st) note_kernel(h, "multihead_attention_bwd", 0);
  return st;
}

// ------------------------------------------------------------------------------------ mini-batch staging
// Host -> device copies of the next mini-batch on a stream of their own, double (or n-fold) buffered: slot s is
// written by the copy stream and read by the handle's compute stream, and two events per slot order them --
// `copied` (the compute stream waits for it before it reads the slot) and `consumed` (the copy stream waits for it
// before it overwrites the slot).  The device buffers and the pinned host memory belong to the caller.
struct snb200_stager {
  snb200_handle_t h;
  int slots;
  cudaStream_t copy_stream;
  cudaEvent_t* copied;
  cudaEvent_t* consumed;
  unsigned char* has_copied;
  unsigned char* has_consumed;
  cudaEvent_t* part_copied;   // [slots][kStagerParts]: behind each of the first copies of an issue
  int* n_parts;               // copies of the slot's last issue that have an event of their own
};
constexpr int kStagerParts = 16;

extern "C" int snb200_stager_create(snb200_handle_t h, int slots, snb200_stager_t* out) {
  int st = enter(h);
  if (st) return st;
  if (!out || slots < 1 || slots > 16) return fail(h, SNB200_STATUS_INVALID_VALUE, "1 to 16 slots");
  *out = nullptr;
  snb200_stager* s = static_cast<snb200_stager*>(calloc(1, sizeof(snb200_stager)));
  if (!s) return fail(h, SNB200_STATUS_ALLOC_FAILED, "out of host memory");
  s->h = h; s->slots = slots;
  s->copied = static_cast<cudaEvent_t*>(calloc(slots, sizeof(cudaEvent_t)));
  s->consumed = static_cast<cudaEvent_t*>(calloc(slots, sizeof(cudaEvent_t)));
  s->has_copied = static_cast<unsigned char*>(calloc(slots, 1));
  s->has_consumed = static_cast<unsigned char*>(calloc(slots, 1));
  s->part_copied = static_cast<cudaEvent_t*>(calloc(static_cast<size_t>(slots) * kStagerParts, sizeof(cudaEvent_t)));
  s->n_parts = static_cast<int*>(calloc(slots, sizeof(int)));
  bool ok = s->copied && s->consumed && s->has_copied && s->has_consumed && s->part_copied && s->n_parts &&
            cudaStreamCreateWithFlags(&s->copy_stream, cudaStreamNonBlocking) == cudaSuccess;
  for (int i = 0; ok && i < slots; ++i)
    ok = cudaEventCreateWithFlags(&s->copied[i], cudaEventDisableTiming) == cudaSuccess &&
         cudaEventCreateWithFlags(&s->consumed[i], cudaEventDisableTiming) == cudaSuccess;
  for (int i = 0; ok && i < slots * kStagerParts; ++i)
    ok = cudaEventCreateWithFlags(&s->part_copied[i], cudaEventDisableTiming) == cudaSuccess;
  if (!ok) {
    snb200_stager_destroy(s);
    return fail(h, SNB200_STATUS_ALLOC_FAILED, "could not create the copy stream or its events");
  }
  *out = s;
  return 0;
}

extern "C" int snb200_stager_destroy(snb200_stager_t s) {
  if (!s) return SNB200_STATUS_NOT_INITIALIZED;
  cudaSetDevice(s->h->device);
  if (s->copy_stream) { cudaStreamSynchronize(s->copy_stream); cudaStreamDestroy(s->copy_stream); }
  for (int i = 0; i < s->slots; ++i) {
    if (s->copied && s->copied[i]) cudaEventDestroy(s->copied[i]);
    if (s->consumed && s->consumed[i]) cudaEventDestroy(s->consumed[i]);
  }
  for (int i = 0; s->part_copied && i < s->slots * kStagerParts; ++i)
    if (s->part_copied[i]) cudaEventDestroy(s->part_copied[i]);
  free(s->part_copied); free(s->n_parts);
  free(s->copied); free(s->consumed); free(s->has_copied); free(s->has_consumed);
  free(s);
  return 0;
}

extern "C" int snb200_stager_issue(snb200_stager_t s, int slot, int n_copies, void* const* device_dst,
                                   const void* const* host_src, const long long* bytes) {
  if (!s) return SNB200_STATUS_NOT_INITIALIZED;
  snb200_handle_t h = s->h;
  int st = enter(h);
  if (st) return st;
  if (slot < 0 || slot >= s->slots) return fail(h, SNB200_STATUS_INVALID_VALUE, "slot %d of %d", slot, s->slots);
  if (n_copies < 0 || (n_copies > 0 && (!device_dst || !host_src || !bytes)))
    return fail(h, SNB200_STATUS_INVALID_VALUE, "bad copy list");
  for (int i = 0; i < n_copies; ++i)
    if (bytes[i] < 0 || (bytes[i] > 0 && (!device_dst[i] || !host_src[i])))
      return fail(h, SNB200_STATUS_INVALID_VALUE, "bad copy %d", i);
  // the slot may still be read by the step it was staged for
  if (s->has_consumed[slot]) SNB_CUDA(h, cudaStreamWaitEvent(s->copy_stream, s->consumed[slot], 0));
  for (int i = 0; i < n_copies; ++i) {
    if (bytes[i] > 0)
      SNB_CUDA(h, cudaMemcpyAsync(device_dst[i], host_src[i], static_cast<size_t>(bytes[i]), cudaMemcpyHostToDevice,
                                  s->copy_stream));
    if (i < kStagerParts) SNB_CUDA(h, cudaEventRecord(s->part_copied[slot * kStagerParts + i], s->copy_stream));
  }
  s->n_parts[slot] = n_copies < kStagerParts ? n_copies : kStagerParts;
  SNB_CUDA(h, cudaEventRecord(s->copied[slot], s->copy_stream));
  s->has_copied[slot] = 1;
  return 0;
}

extern "C" int snb200_stager_acquire_part(snb200_stager_t s, int slot, int part) {
  if (!s) return SNB200_STATUS_NOT_INITIALIZED;
  snb200_handle_t h = s->h;
  int st = enter(h);
  if (st) return st;
  if (slot < 0 || slot >= s->slots) return fail(h, SNB200_STATUS_INVALID_VALUE, "slot %d of %d", slot, s->slots);
  if (!s->has_copied[slot]) return fail(h, SNB200_STATUS_INVALID_VALUE, "nothing was staged into slot %d", slot);
  if (part < 0 || part >= s->n_parts[slot])
    return fail(h, SNB200_STATUS_INVALID_VALUE, "copy %d of the %d with their own event in slot %d", part, s->n_parts[slot], slot);
  SNB_CUDA(h, cudaStreamWaitEvent(h->stream, s->part_copied[slot * kStagerParts + part], 0));
  return 0;
}

extern "C" int snb200_stager_acquire(snb200_stager_t s, int slot) {
  if (!s) return SNB200_STATUS_NOT_INITIALIZED;
  snb200_handle_t h = s->h;
  int st = enter(h);
  if (st) return st;
  if (slot < 0 || slot >= s->slots) return fail(h, SNB200_STATUS_INVALID_VALUE, "slot %d of %d", slot, s->slots);
  if (!s->has_copied[slot]) return fail(h, SNB200_STATUS_INVALID_VALUE, "nothing was staged into slot %d", slot);
  SNB_CUDA(h, cudaStreamWaitEvent(h->stream, s->copied[slot], 0));
  return 0;
}

extern "C" int snb200_stager_release(snb200_stager_t s, int slot) {
  if (!s) return SNB200_STATUS_NOT_INITIALIZED;
  snb200_handle_t h = s->h;
  int st = enter(h);
  if (st) return st;
  if (slot < 0 || slot >= s->slots) return fail(h, SNB200_STATUS_INVALID_VALUE, "slot %d of %d", slot, s->slots);
  SNB_CUDA(h, cudaEventRecord(s->consumed[slot], h->stream));
  s->has_consumed[slot] = 1;
  return 0;
}

extern "C" int snb200_host_pin(void* host_ptr, long long bytes) {
  if (!host_ptr || bytes <= 0) return SNB200_STATUS_INVALID_VALUE;
  cudaError_t e = cudaHostRegister(host_ptr, static_cast<size_t>(bytes), cudaHostRegisterPortable);
  if (e == cudaErrorHostMemoryAlreadyRegistered) { cudaGetLastError(); return 0; }
  return e == cudaSuccess ? 0 : SNB200_STATUS_ALLOC_FAILED;
}
extern "C" int snb200_host_unpin(void* host_ptr) {
  if (!host_ptr) return SNB200_STATUS_INVALID_VALUE;
  cudaError_t e = cudaHostUnregister(host_ptr);
  if (e != cudaSuccess) cudaGetLastError();
  return e == cudaSuccess ? 0 : SNB200_STATUS_INVALID_VALUE;
}

// ------------------------------------------------------------------------------------ NCCL (loaded at run time)
struct NcclId { char bytes[128]; };
typedef int (*nccl_get_id_t)(NcclId*);
typedef int (*nccl_init_rank_t)(void**, int, NcclId, int);
typedef int (*nccl_init_all_t)(void**, int, const int*);
typedef int (*nccl_allreduce_t)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef int (*nccl_destroy_t)(void*);
typedef int (*nccl_group_t)(void);
typedef const char* (*nccl_errstr_t)(int);
static struct {
  void* lib;
  nccl_get_id_t get_id;
  nccl_init_rank_t init_rank;
  nccl_init_all_t init_all;
  nccl_allreduce_t allreduce;
  nccl_destroy_t destroy;
  nccl_group_t group_start, group_end;
  nccl_errstr_t errstr;
} g_nccl;

static bool load_nccl() {
  if (g_nccl.lib) return true;
  const char* names[3] = {getenv("SNB200_NCCL_LIBRARY"), "libnccl.so.2", "libnccl.so"};
  void* lib = nullptr;
  for (int i = 0; i < 3 && !lib; ++i)
    if (names[i] && names[i][0]) lib = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
  if (!lib) return false;
  g_nccl.get_id = reinterpret_cast<nccl_get_id_t>(dlsym(lib, "ncclGetUniqueId"));
  g_nccl.init_rank = reinterpret_cast<nccl_init_rank_t>(dlsym(lib, "ncclCommInitRank"));
  g_nccl.init_all = reinterpret_cast<nccl_init_all_t>(dlsym(lib, "ncclCommInitAll"));
  g_nccl.allreduce = reinterpret_cast<nccl_allreduce_t>(dlsym(lib, "ncclAllReduce"));
  g_nccl.destroy = reinterpret_cast<nccl_destroy_t>(dlsym(lib, "ncclCommDestroy"));
  g_nccl.errstr = reinterpret_cast<nccl_errstr_t>(dlsym(lib, "ncclGetErrorString"));
  g_nccl.group_start = reinterpret_cast<nccl_group_t>(dlsym(lib, "ncclGroupStart"));
  g_nccl.group_end = reinterpret_cast<nccl_group_t>(dlsym(lib, "ncclGroupEnd"));
  if (!g_nccl.get_id || !g_nccl.init_rank || !g_nccl.init_all || !g_nccl.allreduce || !g_nccl.destroy ||
      !g_nccl.group_start || !g_nccl.group_end) {
    dlclose(lib);
    return false;
  }
  g_nccl.lib = lib;
  return true;
}
static int nccl_fail(snb200_handle_t h, int r, const char* what) {
  return fail(h, SNB200_STATUS_EXECUTION_FAILED, "%s: %s", what, g_nccl.errstr ? g_nccl.errstr(r) : "NCCL error");
}

extern "C" int snb200_comm_get_unique_id(void* id) {
  if (!id) return SNB200_STATUS_INVALID_VALUE;
  if (!load_nccl()) return SNB200_STATUS_NOT_SUPPORTED;
  return g_nccl.get_id(static_cast<NcclId*>(id)) == 0 ? 0 : SNB200_STATUS_EXECUTION_FAILED;
}
extern "C" int snb200_comm_init_rank(snb200_handle_t h, int n_ranks, int rank, const void* id) {
  int st = enter(h);
  if (st) return st;
  if (!id || n_ranks < 1 || rank < 0 || rank >= n_ranks) return fail(h, SNB200_STATUS_INVALID_VALUE, "bad rank %d of %d", rank, n_ranks);
  if (h->nccl_comm) return fail(h, SNB200_STATUS_INVALID_VALUE, "communicator already initialised");
  if (!load_nccl()) return fail(h, SNB200_STATUS_NOT_SUPPORTED, "libnccl.so.2 could not be loaded");
  NcclId nid;
  memcpy(&nid, id, sizeof(nid));
  int r = g_nccl.init_rank(&h->nccl_comm, n_ranks, nid, rank);
  if (r) { h->nccl_comm = nullptr; return nccl_fail(h, r, "ncclCommInitRank"); }
  return 0;
}
extern "C" int snb200_comm_init_all(snb200_handle_t* handles, int n) {
  if (!handles || n < 1 || n > 64) return SNB200_STATUS_INVALID_VALUE;
  if (!load_nccl()) return SNB200_STATUS_NOT_SUPPORTED;
  void* comms[64];
  int devs[64];
  for (int i = 0; i < n; ++i) {
    if (!handles[i]) return SNB200_STATUS_NOT_INITIALIZED;
    if (handles[i]->nccl_comm) return fail(handles[i], SNB200_STATUS_INVALID_VALUE, "communicator already initialised");
    devs[i] = handles[i]->device;
  }
  int r = g_nccl.init_all(comms, n, devs);
  if (r) return nccl_fail(handles[0], r, "ncclCommInitAll");
  for (int i = 0; i < n; ++i) handles[i]->nccl_comm = comms[i];
  return 0;
}
extern "C" int snb200_allreduce_sum(snb200_handle_t h, float* buf, long long count) {
  int st = enter(h);
  if (st) return st;
  if (count < 0 || (count > 0 && !buf)) return fail(h, SNB200_STATUS_INVALID_VALUE, "bad buffer");
  if (!h->nccl_comm) return fail(h, SNB200_STATUS_NOT_INITIALIZED, "no communicator on this handle");
  if (count == 0) return 0;
  int r = g_nccl.allreduce(buf, buf, static_cast<size_t>(count), /*ncclFloat32*/ 7, /*ncclSum*/ 0, h->nccl_comm, h->stream);
  if (r) return nccl_fail(h, r, "ncclAllReduce");
  return 0;
}
extern "C" int snb200_allreduce_sum_group(snb200_handle_t h, int n, float* const* bufs, const long long* counts) {
  int st = enter(h);
  if (st) return st;
  if (n < 0 || (n > 0 && (!bufs || !counts))) return fail(h, SNB200_STATUS_INVALID_VALUE, "bad buffer list");
  for (int i = 0; i < n; ++i)
    if (counts[i] < 0 || (counts[i] > 0 && !bufs[i])) return fail(h, SNB200_STATUS_INVALID_VALUE, "bad buffer %d", i);
  if (!h->nccl_comm) return fail(h, SNB200_STATUS_NOT_INITIALIZED, "no communicator on this handle");
  int r = g_nccl.group_start();
  if (r) return nccl_fail(h, r, "ncclGroupStart");
  int first_error = 0;
  for (int i = 0; i < n && !first_error; ++i)
    if (counts[i] > 0)
      first_error = g_nccl.allreduce(bufs[i], bufs[i], static_cast<size_t>(counts[i]), /*ncclFloat32*/ 7, /*ncclSum*/ 0,
                                     h->nccl_comm, h->stream);
  r = g_nccl.group_end();   // always closes the group, also after a failed call inside it
  if (first_error) return nccl_fail(h, first_error, "ncclAllReduce");
  if (r) return nccl_fail(h, r, "ncclGroupEnd");
  return 0;
}
extern "C" int snb200_comm_destroy(snb200_handle_t h) {
  if (!h) return SNB200_STATUS_NOT_INITIALIZED;
  if (!h->nccl_comm) return 0;
  cudaSetDevice(h->device);
  int r = g_nccl.destroy(h->nccl_comm);
  h->nccl_comm = nullptr;
  return r ? nccl_fail(h, r, "ncclCommDestroy") : 0;
}
