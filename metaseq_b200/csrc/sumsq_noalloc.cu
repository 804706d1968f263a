// Sum of squares of a flat tensor without any device allocation: the per-CTA partial sums
// live in a file-scope __device__ array.  See msq_noalloc.h for who needs this and the rules
// for calling it.  The arithmetic matches msq_sumsq (optim.cu): each CTA reduces a
// grid-strided slice to one fp32 partial, a single-CTA second kernel adds the partials.
#include "msq_noalloc.h"

#include <cstdio>
#include <mutex>

#include "sm100_common.cuh"

namespace {

constexpr int NA_THREADS = 512;
constexpr int NA_MAX_DEVICES = 64;

// Scratch shared by every call on a device.  In host code this name is only a handle for
// cudaGetSymbolAddress; it is never passed to a kernel directly.
static __device__ __align__(256) float g_noalloc_partials[MSQ_NOALLOC_MAX_PARTS];

std::mutex g_setup_mutex;
float* g_partials_addr[NA_MAX_DEVICES] = {nullptr};
int g_sm_count[NA_MAX_DEVICES] = {0};

template <int DT>  // 0 fp16, 1 bf16, 2 fp32
__global__ void __launch_bounds__(NA_THREADS)
noalloc_partial_kernel(const void* __restrict__ g, long long n, float* __restrict__ partials) {
  __shared__ float red[32];
  float acc = 0.f;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  if constexpr (DT == 2) {
    const float* p = static_cast<const float*>(g);
    const long long n4 = n >> 2;
    const float4* p4 = static_cast<const float4*>(g);
    for (long long i = tid; i < n4; i += stride) {
      const float4 v = p4[i];
      acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    for (long long i = (n4 << 2) + tid; i < n; i += stride) acc += p[i] * p[i];
  } else {
    const long long n8 = n >> 3;
    const uint4* p8 = static_cast<const uint4*>(g);
    for (long long i = tid; i < n8; i += stride) {
      const uint4 v = p8[i];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = msq::unpack2<DT == 1>(w[j]);
        acc += t.x * t.x + t.y * t.y;
      }
    }
    const uint16_t* p = static_cast<const uint16_t*>(g);
    for (long long i = (n8 << 3) + tid; i < n; i += stride) {
      const uint32_t raw = p[i];
      const float2 t = msq::unpack2<DT == 1>(raw);  // low half holds the element
      acc += t.x * t.x;
    }
  }
  const float total = msq::block_sum(acc, red);
  if (threadIdx.x == 0) partials[blockIdx.x] = total;  // every slot in [0, gridDim.x) is rewritten
}

__global__ void __launch_bounds__(NA_THREADS)
noalloc_finalize_kernel(const float* __restrict__ partials, int parts, float* __restrict__ out, int accumulate) {
  __shared__ float red[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < parts; i += blockDim.x) acc += partials[i];  // reads only what this call wrote
  const float total = msq::block_sum(acc, red);
  if (threadIdx.x == 0) out[0] = total + (accumulate ? out[0] : 0.f);
}

// Device address of the scratch array for the current device, looked up on first use.
int scratch_for_current_device(float** addr, int* sms) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NA_MAX_DEVICES) return MSQ_NOALLOC_ERR_SYMBOL;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_partials_addr[dev] == nullptr) {
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_partials);
    if (e != cudaSuccess || p == nullptr) {
      std::fprintf(stderr, "msq_sumsq_noalloc: cudaGetSymbolAddress failed on device %d: %s\n", dev,
                   cudaGetErrorString(e));
      return MSQ_NOALLOC_ERR_SYMBOL;
    }
    int n_sm = 0;
    if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 1;
    g_sm_count[dev] = n_sm;
    g_partials_addr[dev] = p;
  }
  *addr = g_partials_addr[dev];
  *sms = g_sm_count[dev];
  return MSQ_NOALLOC_OK;
}

}  // namespace

extern "C" int msq_sumsq_noalloc(const void* g, long long n, int dtype, float* out, int accumulate,
                                 cudaStream_t stream) {
  if (n < 0 || n > MSQ_NOALLOC_MAX_ELEMS) {
    std::fprintf(stderr, "msq_sumsq_noalloc: n = %lld is outside [0, %lld]; nothing was launched\n", n,
                 static_cast<long long>(MSQ_NOALLOC_MAX_ELEMS));
    return MSQ_NOALLOC_ERR_SIZE;
  }
  if (dtype < 0 || dtype > 2) {
    std::fprintf(stderr, "msq_sumsq_noalloc: dtype %d is not 0 (fp16), 1 (bf16) or 2 (fp32)\n", dtype);
    return MSQ_NOALLOC_ERR_DTYPE;
  }
  if (out == nullptr || (n > 0 && g == nullptr) || (reinterpret_cast<uintptr_t>(g) & 15)) {
    std::fprintf(stderr, "msq_sumsq_noalloc: null output, null input with n > 0, or input not 16-byte aligned\n");
    return MSQ_NOALLOC_ERR_ARG;
  }
  float* partials = nullptr;
  int sms = 1;
  const int rc = scratch_for_current_device(&partials, &sms);
  if (rc != MSQ_NOALLOC_OK) return rc;
  const long long per_cta = 8LL * NA_THREADS;
  long long parts = (n + per_cta - 1) / per_cta;
  const long long cap = 4LL * sms < MSQ_NOALLOC_MAX_PARTS ? 4LL * sms : MSQ_NOALLOC_MAX_PARTS;
  if (parts > cap) parts = cap;
  if (parts < 1) parts = 1;
  const int grid = static_cast<int>(parts);
  if (dtype == 0) noalloc_partial_kernel<0><<<grid, NA_THREADS, 0, stream>>>(g, n, partials);
  else if (dtype == 1) noalloc_partial_kernel<1><<<grid, NA_THREADS, 0, stream>>>(g, n, partials);
  else noalloc_partial_kernel<2><<<grid, NA_THREADS, 0, stream>>>(g, n, partials);
  noalloc_finalize_kernel<<<1, NA_THREADS, 0, stream>>>(partials, grid, out, accumulate);
  if (cudaGetLastError() != cudaSuccess) {
    std::fprintf(stderr, "msq_sumsq_noalloc: kernel launch failed\n");
    return MSQ_NOALLOC_ERR_LAUNCH;
  }
  return MSQ_NOALLOC_OK;
}
