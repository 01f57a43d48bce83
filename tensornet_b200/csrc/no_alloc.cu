// Allocation-free entry point of the batch dedup; see no_alloc.h for the contract.
#include <mutex>
#include <string>

#include "no_alloc.h"
#include "tn_device.cuh"
#include "tn_ops.h"

namespace {

constexpr unsigned kScratchCap = 2u * TN_UNIQUE_STATIC_MAX_IDS;             // power of two, load factor <= 0.5
constexpr size_t kKeysBytes = (size_t)kScratchCap * sizeof(unsigned long long);
constexpr size_t kValsBytes = (size_t)kScratchCap * sizeof(int);
constexpr size_t kStatusBytes = 64;
constexpr size_t kScratchBytes = kKeysBytes + kValsBytes + kStatusBytes;

// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) unsigned char g_unique_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char* g_scratch_ptr[kMaxDevices] = {nullptr};
thread_local std::string g_error;

__global__ void static_prepare_kernel(unsigned long long* keys, unsigned cap, int* status, int* count, float* show, float* click,
                                      int n_out) {
  const unsigned tid = blockIdx.x * blockDim.x + threadIdx.x, nth = gridDim.x * blockDim.x;
  for (unsigned i = tid; i < cap; i += nth) keys[i] = tn::kEmptyKey;
  for (unsigned i = tid; i < (unsigned)n_out; i += nth) {
    if (show) show[i] = 0.f;
    if (click) click[i] = 0.f;
  }
  if (tid < 4) status[tid] = 0;
  if (tid == 0) *count = 0;
}

int fail(int code, const std::string& msg) {
  g_error = msg;
  return code;
}

// Device address of the scratch on the current device; looked up once per device.
int scratch_for_current_device(unsigned char** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(TN_NOALLOC_CUDA_ERROR, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(TN_NOALLOC_BAD_ARGUMENT, "device index out of range");
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_unique_scratch);
    if (e != cudaSuccess) return fail(TN_NOALLOC_CUDA_ERROR, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
    g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_ptr[dev];
  return TN_NOALLOC_OK;
}

}  // namespace

extern "C" int tn_unique_assign_static(const long long* ids, int n, const float* labels, unsigned long long* uniq, int uniq_cap,
                                       int* inverse, float* show, float* click, int* count, cudaStream_t stream) {
  g_error.clear();
  if (n < 0 || uniq_cap < 0) return fail(TN_NOALLOC_BAD_ARGUMENT, "tn_unique_assign_static: negative size");
  if (n > TN_UNIQUE_STATIC_MAX_IDS)
    return fail(TN_NOALLOC_TOO_LARGE, "tn_unique_assign_static: " + std::to_string(n) + " ids exceed the built-in scratch (max " +
                                          std::to_string(TN_UNIQUE_STATIC_MAX_IDS) + "); use the allocating entry point");
  if (!count || (n > 0 && (!ids || !uniq || !inverse))) return fail(TN_NOALLOC_BAD_ARGUMENT, "tn_unique_assign_static: null buffer");
  unsigned char* base = nullptr;
  int rc = scratch_for_current_device(&base);
  if (rc != TN_NOALLOC_OK) return rc;
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(base);
  int* vals = reinterpret_cast<int*>(base + kKeysBytes);
  int* status = reinterpret_cast<int*>(base + kKeysBytes + kValsBytes);
  const int n_out = n < uniq_cap ? n : uniq_cap;
  static_prepare_kernel<<<148, 256, 0, stream>>>(keys, kScratchCap, status, count, show, click, n_out);
  tn::launch_unique_assign(ids, n, labels, keys, vals, kScratchCap, uniq, uniq_cap, inverse, show, click, count, status, stream);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(TN_NOALLOC_CUDA_ERROR, std::string("kernel launch: ") + cudaGetErrorString(e));
  return TN_NOALLOC_OK;
}

extern "C" const char* tn_unique_assign_static_error(void) { return g_error.c_str(); }

extern "C" int tn_unique_assign_static_status(int* host_out, cudaStream_t stream) {
  unsigned char* base = nullptr;
  int rc = scratch_for_current_device(&base);
  if (rc != TN_NOALLOC_OK) return rc;
  cudaError_t e = cudaMemcpyAsync(host_out, base + kKeysBytes + kValsBytes, 4 * sizeof(int), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return fail(TN_NOALLOC_CUDA_ERROR, std::string("status read: ") + cudaGetErrorString(e));
  return TN_NOALLOC_OK;
}
