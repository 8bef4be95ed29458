// snb200_bias_grad_noalloc: the bias gradient (column sums of dy) for callers that cannot allocate.
//
// Every other entry point of this library needs a handle, and creating a handle calls cudaMalloc
// for its workspace.  Some hosts cannot do that once they are up and running: an engine that hands
// the whole device memory to its own pool at start-up (SharpNet's TensorMemoryPool grown to the
// limit, or any framework that reserves the GPU) makes a later cudaMalloc fail with out-of-memory,
// and a latency-critical loop cannot afford the device-wide synchronisation that cudaMalloc and
// cudaFree imply.  This entry point therefore takes no handle and calls no allocating routine:
// the slab partial sums that the column reduction needs live in a fixed array in the library's own
// device image.
//
// One moment does need free device memory: the library's device image (the array and the kernels) is loaded
// onto a device on first use -- with CUDA's default lazy loading, in the first call of this entry point on that
// device.  That first call must therefore come before the host's pool takes the memory (it is also the call that
// must precede any stream capture), or the process runs with CUDA_MODULE_LOADING=EAGER; an out-of-memory at that
// point is reported as ALLOC_FAILED with that advice.
//
// The array is 1 MiB per GPU that loads the library, for the life of the process.  All calls on a
// device share it, so two calls that overlap on the GPU (different streams, or different host
// threads) race on it; calls on one stream are safe.  The kernels overwrite every word of it that
// they read back, so nothing has to be cleared between calls.
#include <cuda_runtime.h>
#include <stdio.h>

#include <mutex>

#include "../../include/sharpnet_b200.h"
#include "elementwise.cuh"

using namespace snb;

namespace {

constexpr int kScratchFloats = 1 << 18;   // 1 MiB
constexpr int kMaxDevices = 64;

// Scratch for the slab partial sums.  In host code this name is only a handle for the symbol, not
// a device address; the address is asked for once per device (below) and passed to the kernels.
static __device__ __align__(256) float g_noalloc_scratch[kScratchFloats];

std::mutex g_setup_mutex;
float* g_scratch_addr[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};

int report(char* err, int err_len, int status, const char* msg, const char* detail = "") {
  if (err && err_len > 0) snprintf(err, err_len, "%s%s", msg, detail);
  return status;
}

}  // namespace

extern "C" int snb200_bias_grad_noalloc(int device_id, void* cuda_stream, int M, int N, const float* dy, float* db,
                                        char* err, int err_len) {
  if (err && err_len > 0) err[0] = 0;
  if (device_id < 0 || device_id >= kMaxDevices)
    return report(err, err_len, SNB200_STATUS_INVALID_VALUE, "device id out of range");
  if (M < 0 || N < 0) return report(err, err_len, SNB200_STATUS_INVALID_VALUE, "negative dimension");
  if (N > SNB200_NOALLOC_MAX_COLUMNS)
    return report(err, err_len, SNB200_STATUS_NOT_SUPPORTED,
                  "snb200_bias_grad_noalloc handles at most 65536 columns (its scratch is a fixed 1 MiB array); "
                  "use snb200_bias_grad with a handle for wider matrices");
  if (N == 0) return 0;
  if (!db || (M > 0 && !dy)) return report(err, err_len, SNB200_STATUS_INVALID_VALUE, "null pointer");
  cudaError_t e = cudaSetDevice(device_id);
  if (e != cudaSuccess)
    return report(err, err_len, SNB200_STATUS_NOT_INITIALIZED, "cudaSetDevice: ", cudaGetErrorString(e));
  {
    // First call on this device: resolve the device address of the scratch array and the SM count.
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_addr[device_id]) {
      float* p = nullptr;
      // With CUDA's lazy module loading this is where the device image that holds the array (1 MiB plus the
      // kernels) is loaded onto the device -- the one moment this entry point needs free device memory.
      e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
      if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        return report(err, err_len, SNB200_STATUS_ALLOC_FAILED,
                      "no device memory left to load the library's device image: make the first call on a device "
                      "before the host's pool takes the memory, or run with CUDA_MODULE_LOADING=EAGER");
      }
      if (e != cudaSuccess || !p)
        return report(err, err_len, SNB200_STATUS_NOT_INITIALIZED, "cudaGetSymbolAddress: ", cudaGetErrorString(e));
      int sms = 0;
      e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device_id);
      if (e != cudaSuccess || sms <= 0)
        return report(err, err_len, SNB200_STATUS_NOT_INITIALIZED, "cudaDeviceGetAttribute: ", cudaGetErrorString(e));
      g_sm_count[device_id] = sms;
      g_scratch_addr[device_id] = p;
    }
  }
  float* scratch = g_scratch_addr[device_id];
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (M == 0) {
    e = cudaMemsetAsync(db, 0, sizeof(float) * N, stream);
    return e == cudaSuccess ? 0 : report(err, err_len, SNB200_STATUS_EXECUTION_FAILED, "cudaMemsetAsync: ",
                                         cudaGetErrorString(e));
  }
  const bool vec = (N % 4 == 0) && ((reinterpret_cast<uintptr_t>(dy) & 15u) == 0);
  const int cols_per_block = vec ? 128 : 32;
  const int col_blocks = (N + cols_per_block - 1) / cols_per_block;
  int slabs = (4 * g_sm_count[device_id] + col_blocks - 1) / col_blocks;
  if (slabs > (M + 7) / 8) slabs = (M + 7) / 8;
  if (slabs > kScratchFloats / N) slabs = kScratchFloats / N;   // >= 4 because N <= 65536
  if (slabs > 65535) slabs = 65535;
  if (slabs < 1) slabs = 1;
  const int rows_per_slab = (M + slabs - 1) / slabs;
  slabs = (M + rows_per_slab - 1) / rows_per_slab;
  float* out = slabs == 1 ? db : scratch;
  dim3 grid(col_blocks, slabs);
  if (vec)
    colsum_slab_kernel<4, false><<<grid, 256, 0, stream>>>(M, N, rows_per_slab, ACT_IDENTITY, dy, nullptr, nullptr,
                                                           nullptr, out);
  else
    colsum_slab_kernel<1, false><<<grid, 256, 0, stream>>>(M, N, rows_per_slab, ACT_IDENTITY, dy, nullptr, nullptr,
                                                           nullptr, out);
  if (slabs > 1) colsum_finish_kernel<<<(N + 255) / 256, 256, 0, stream>>>(N, slabs, scratch, db);
  e = cudaGetLastError();
  if (e != cudaSuccess)
    return report(err, err_len, SNB200_STATUS_EXECUTION_FAILED, "kernel launch: ", cudaGetErrorString(e));
  return 0;
}
