// Optimizer-side kernels: squared-L2-norm of a flat gradient shard, the
// device-side clip / overflow decision, and the fused AdamW update for the
// memory-efficient fp16 optimizer (16-bit params and grads, fp32 moments, no
// fp32 master copy).
//
// Reference behaviour being reproduced:
//   * grad norm: metaseq/utils.py:104-127 (multi_tensor_l2norm) + :199-229 (clip)
//   * lazy _multiply_factor folding 1/loss_scale, dp/sample_size and the clip
//     coefficient: metaseq/optim/fp16_optimizer.py:397-455
//   * Adam math: metaseq/optim/adam.py:170-213 (decoupled weight decay, bias
//     correction folded into the step size, eps added outside the sqrt)
// Unlike the reference, the overflow / clip decision stays on the device: the
// update kernel reads a two-float control block, so no host sync sits between
// the norm and the step.
#include "sm100_common.cuh"

namespace msq {

constexpr int SUMSQ_THREADS = 512;

template <int DT>  // 0 fp16, 1 bf16, 2 fp32
__device__ __forceinline__ float load_as_float(const void* base, long long i) {
  if constexpr (DT == 0) return __half2float(static_cast<const __half*>(base)[i]);
  else if constexpr (DT == 1) return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[i]);
  else return static_cast<const float*>(base)[i];
}

// Each CTA writes one partial sum of squares to scratch[blockIdx.x].
template <int DT>
__global__ void __launch_bounds__(SUMSQ_THREADS)
sumsq_partial_kernel(const void* __restrict__ g, long long n, float* __restrict__ scratch) {
  __shared__ float red[32];
  float acc = 0.f;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  if constexpr (DT == 2) {
    const long long n4 = n >> 2;
    const float4* g4 = static_cast<const float4*>(g);
    for (long long i = tid; i < n4; i += stride) {
      const float4 v = g4[i];
      acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    for (long long i = (n4 << 2) + tid; i < n; i += stride) {
      const float v = static_cast<const float*>(g)[i];
      acc += v * v;
    }
  } else {
    const long long n8 = n >> 3;
    const uint4* g8 = static_cast<const uint4*>(g);
    for (long long i = tid; i < n8; i += stride) {
      const uint4 v = g8[i];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = unpack2<DT == 1>(w[j]);
        acc += t.x * t.x + t.y * t.y;
      }
    }
    for (long long i = (n8 << 3) + tid; i < n; i += stride) {
      const float v = load_as_float<DT>(g, i);
      acc += v * v;
    }
  }
  const float total = block_sum(acc, red);
  if (threadIdx.x == 0) scratch[blockIdx.x] = total;
}

// Single CTA: out[0] = (accumulate ? out[0] : 0) + sum(scratch[0..parts)).
__global__ void __launch_bounds__(SUMSQ_THREADS)
sumsq_finalize_kernel(const float* __restrict__ scratch, int parts, float* __restrict__ out, int accumulate) {
  __shared__ float red[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < parts; i += blockDim.x) acc += scratch[i];
  const float total = block_sum(acc, red);
  if (threadIdx.x == 0) out[0] = total + (accumulate ? out[0] : 0.f);
}

// List form (the reference's apex multi_tensor_l2norm: metaseq/modules/apex/multi_tensor_l2norm_kernel.cu:58-140):
// one launch covers every tensor of a table in device memory.  CTA b works on the tensor whose block range
// [first_block, next first_block) contains b, writes its partial to scratch[b], and the CTA that finishes last
// (a ticket counter, reset for the next call) adds all partials in index order, so the result does not depend on
// the order in which CTAs ran.
struct SumsqTensor {
  const void* g;
  long long n;
  long long first_block;  // of a table with count + 1 entries; the last entry holds the total block count
};

// INF = false: sum of squares; INF = true: largest magnitude (the inf-norm of the list; a non-finite element,
// NaN included, gives +inf so that overflow checks see it).
template <bool INF>
__device__ __forceinline__ void norm_fold(float& acc, float v) {
  if constexpr (INF) {
    const float a = fabsf(v);
    acc = fmaxf(acc, a <= 3.402823466e38f ? a : INFINITY);
  } else {
    acc += v * v;
  }
}

template <int DT, bool INF>
__global__ void __launch_bounds__(SUMSQ_THREADS)
sumsq_multi_kernel(const SumsqTensor* __restrict__ table, int count, float* __restrict__ scratch,
                   unsigned* __restrict__ ticket, float* __restrict__ out, int accumulate) {
  __shared__ float red[32];
  __shared__ int s_idx;
  __shared__ bool s_last;
  const int b = blockIdx.x;
  if (threadIdx.x == 0) {
    int lo = 0, hi = count - 1;  // last tensor whose first_block <= b
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (table[mid].first_block <= b) lo = mid; else hi = mid - 1;
    }
    s_idx = lo;
  }
  __syncthreads();
  const SumsqTensor t = table[s_idx];
  const long long nblk = table[s_idx + 1].first_block - t.first_block;
  const long long tid = (static_cast<long long>(b) - t.first_block) * blockDim.x + threadIdx.x;
  const long long stride = nblk * blockDim.x;
  float acc = 0.f;
  const bool aligned = (reinterpret_cast<uintptr_t>(t.g) & 15) == 0;
  long long done = 0;
  if (aligned) {
    if constexpr (DT == 2) {
      const long long n4 = t.n >> 2;
      const float4* g4 = static_cast<const float4*>(t.g);
      for (long long i = tid; i < n4; i += stride) {
        const float4 v = g4[i];
        norm_fold<INF>(acc, v.x);
        norm_fold<INF>(acc, v.y);
        norm_fold<INF>(acc, v.z);
        norm_fold<INF>(acc, v.w);
      }
      done = n4 << 2;
    } else {
      const long long n8 = t.n >> 3;
      const uint4* g8 = static_cast<const uint4*>(t.g);
      for (long long i = tid; i < n8; i += stride) {
        const uint4 v = g8[i];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack2<DT == 1>(w[j]);
          norm_fold<INF>(acc, f.x);
          norm_fold<INF>(acc, f.y);
        }
      }
      done = n8 << 3;
    }
  }
  for (long long i = done + tid; i < t.n; i += stride) norm_fold<INF>(acc, load_as_float<DT>(t.g, i));
  const float total = INF ? block_max(acc, red) : block_sum(acc, red);
  if (threadIdx.x == 0) {
    scratch[b] = total;
    __threadfence();
    s_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  float sum = 0.f;
  for (int i = threadIdx.x; i < static_cast<int>(gridDim.x); i += blockDim.x) {
    const float v = __ldcg(scratch + i);
    sum = INF ? fmaxf(sum, v) : sum + v;
  }
  sum = INF ? block_max(sum, red) : block_sum(sum, red);
  if (threadIdx.x == 0) {
    if (INF) out[0] = accumulate ? fmaxf(sum, out[0]) : sum;
    else out[0] = sum + (accumulate ? out[0] : 0.f);
    *ticket = 0;
  }
}

// List form of an in-place scale (the reference's apex multi_tensor_scale, metaseq/modules/apex/multi_tensor_scale_kernel.cu):
// every tensor of the table is multiplied by host_scale * (dev_scale ? dev_scale[0] : 1), the device factor being
// e.g. a clip coefficient that the host never reads.
template <int DT>
__global__ void __launch_bounds__(SUMSQ_THREADS)
scale_multi_kernel(const SumsqTensor* __restrict__ table, int count, const float* __restrict__ dev_scale,
                   float host_scale) {
  __shared__ int s_idx;
  const int b = blockIdx.x;
  if (threadIdx.x == 0) {
    int lo = 0, hi = count - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (table[mid].first_block <= b) lo = mid; else hi = mid - 1;
    }
    s_idx = lo;
  }
  __syncthreads();
  const SumsqTensor t = table[s_idx];
  const float f = host_scale * (dev_scale ? dev_scale[0] : 1.f);
  if (f == 1.f) return;
  const long long nblk = table[s_idx + 1].first_block - t.first_block;
  const long long tid = (static_cast<long long>(b) - t.first_block) * blockDim.x + threadIdx.x;
  const long long stride = nblk * blockDim.x;
  void* g = const_cast<void*>(t.g);
  const bool aligned = (reinterpret_cast<uintptr_t>(g) & 15) == 0;
  long long done = 0;
  if (aligned) {
    if constexpr (DT == 2) {
      const long long n4 = t.n >> 2;
      float4* g4 = static_cast<float4*>(g);
      for (long long i = tid; i < n4; i += stride) {
        float4 v = g4[i];
        v.x *= f; v.y *= f; v.z *= f; v.w *= f;
        g4[i] = v;
      }
      done = n4 << 2;
    } else {
      const long long n8 = t.n >> 3;
      uint4* g8 = static_cast<uint4*>(g);
      for (long long i = tid; i < n8; i += stride) {
        const uint4 v = g8[i];
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 x = unpack2<DT == 1>(w[j]);
          w[j] = pack2<DT == 1>(x.x * f, x.y * f);
        }
        g8[i] = make_uint4(w[0], w[1], w[2], w[3]);
      }
      done = n8 << 3;
    }
  }
  for (long long i = done + tid; i < t.n; i += stride) {
    const float v = load_as_float<DT>(g, i) * f;
    if constexpr (DT == 0) static_cast<__half*>(g)[i] = __float2half(v);
    else if constexpr (DT == 1) static_cast<__nv_bfloat16*>(g)[i] = __float2bfloat16(v);
    else static_cast<float*>(g)[i] = v;
  }
}

// ctrl_out[0] = multiplier the update applies to raw grads (pre_factor * clip_coef)
// ctrl_out[1] = 1 when the step must be skipped (non-finite norm), else 0
// ctrl_out[2] = unclipped gradient norm (pre_factor * sqrt(sum of squares))
// ctrl_out[3] = clip coefficient
__global__ void clip_decision_kernel(const float* __restrict__ sumsq, int n_terms, float pre_factor, float max_norm,
                                     float* __restrict__ ctrl_out) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  float s = 0.f;
  for (int i = 0; i < n_terms; ++i) s += sumsq[i];
  const float norm = pre_factor * sqrtf(s);
  const bool bad = !isfinite(norm);
  float coef = 1.f;
  if (!bad && max_norm > 0.f) coef = fminf(1.f, max_norm / (norm + 1e-6f));
  ctrl_out[0] = pre_factor * coef;
  ctrl_out[1] = bad ? 1.f : 0.f;
  ctrl_out[2] = norm;
  ctrl_out[3] = coef;
}

// AdamW on a flat shard.  P and G are 16-bit (PDT / GDT codes as above; PDT may be
// fp32 for a master-weight flavour, in which case p16_out, if given, receives the
// 16-bit copy).  m, v fp32.
template <int PDT, int GDT>
__global__ void __launch_bounds__(512)
adamw_kernel(void* __restrict__ p, const void* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
             void* __restrict__ p16_out, int p16_bf16, long long n, float lr, float beta1, float beta2, float eps,
             float weight_decay, float step_size, float inv_sqrt_bc2_unused, const float* __restrict__ ctrl) {
  const float gmul = ctrl ? ctrl[0] : 1.f;
  if (ctrl && ctrl[1] != 0.f) return;  // overflow: leave params and moments untouched
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float gi = load_as_float<GDT>(g, i) * gmul;
    float pi = load_as_float<PDT>(p, i);
    const float mi = beta1 * m[i] + (1.f - beta1) * gi;
    const float vi = beta2 * v[i] + (1.f - beta2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    const float denom = sqrtf(vi) + eps;
    pi = pi - lr * weight_decay * pi;
    pi = pi - step_size * (mi / denom);
    if constexpr (PDT == 0) static_cast<__half*>(p)[i] = __float2half(pi);
    else if constexpr (PDT == 1) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16(pi);
    else {
      static_cast<float*>(p)[i] = pi;
      if (p16_out) {
        if (p16_bf16) static_cast<__nv_bfloat16*>(p16_out)[i] = __float2bfloat16(pi);
        else static_cast<__half*>(p16_out)[i] = __float2half(pi);
      }
    }
  }
}

// List form: one launch updates every tensor of a table in device memory (blockIdx.y = tensor).  16-bit
// parameters and gradients with 16-byte aligned storage are processed eight elements per thread and iteration
// (one 16-byte load each for p and g, two each for m and v); other cases take the scalar loop.
struct AdamTensor {
  void* p;
  const void* g;
  float* m;
  float* v;
  long long n;
};

template <int PDT, int GDT>
__global__ void __launch_bounds__(512)
adamw_multi_kernel(const AdamTensor* __restrict__ table, float lr, float beta1, float beta2, float eps,
                   float weight_decay, float step_size, const float* __restrict__ ctrl) {
  const float gmul = ctrl ? ctrl[0] : 1.f;
  if (ctrl && ctrl[1] != 0.f) return;  // overflow: leave params and moments untouched
  const AdamTensor t = table[blockIdx.y];
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  auto update = [&](float pi, float gi, float& mi, float& vi) -> float {
    gi *= gmul;
    mi = beta1 * mi + (1.f - beta1) * gi;
    vi = beta2 * vi + (1.f - beta2) * gi * gi;
    pi = pi - lr * weight_decay * pi;
    return pi - step_size * (mi / (sqrtf(vi) + eps));
  };
  long long done = 0;
  if constexpr (PDT != 2 && GDT != 2) {
    const bool aligned = ((reinterpret_cast<uintptr_t>(t.p) | reinterpret_cast<uintptr_t>(t.g) |
                           reinterpret_cast<uintptr_t>(t.m) | reinterpret_cast<uintptr_t>(t.v)) & 15) == 0;
    if (aligned) {
      const long long n8 = t.n >> 3;
      for (long long i = tid; i < n8; i += stride) {
        const uint4 pv = static_cast<const uint4*>(t.p)[i];
        const uint4 gv = static_cast<const uint4*>(t.g)[i];
        float4 m0 = reinterpret_cast<float4*>(t.m)[2 * i], m1 = reinterpret_cast<float4*>(t.m)[2 * i + 1];
        float4 v0 = reinterpret_cast<float4*>(t.v)[2 * i], v1 = reinterpret_cast<float4*>(t.v)[2 * i + 1];
        const uint32_t pw[4] = {pv.x, pv.y, pv.z, pv.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w};
        float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
        float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        uint32_t out[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 pf = unpack2<PDT == 1>(pw[j]);
          const float2 gf = unpack2<GDT == 1>(gw[j]);
          const float a = update(pf.x, gf.x, mm[2 * j], vv[2 * j]);
          const float b = update(pf.y, gf.y, mm[2 * j + 1], vv[2 * j + 1]);
          out[j] = pack2<PDT == 1>(a, b);
        }
        static_cast<uint4*>(t.p)[i] = make_uint4(out[0], out[1], out[2], out[3]);
        reinterpret_cast<float4*>(t.m)[2 * i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
        reinterpret_cast<float4*>(t.m)[2 * i + 1] = make_float4(mm[4], mm[5], mm[6], mm[7]);
        reinterpret_cast<float4*>(t.v)[2 * i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
        reinterpret_cast<float4*>(t.v)[2 * i + 1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
      }
      done = n8 << 3;
    }
  }
  for (long long i = done + tid; i < t.n; i += stride) {
    float mi = t.m[i], vi = t.v[i];
    const float pi = update(load_as_float<PDT>(t.p, i), load_as_float<GDT>(t.g, i), mi, vi);
    t.m[i] = mi;
    t.v[i] = vi;
    if constexpr (PDT == 0) static_cast<__half*>(t.p)[i] = __float2half(pi);
    else if constexpr (PDT == 1) static_cast<__nv_bfloat16*>(t.p)[i] = __float2bfloat16(pi);
    else static_cast<float*>(t.p)[i] = pi;
  }
}

static int device_sms() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return sms;
}

}  // namespace msq

// Number of scratch floats msq_sumsq needs for an n-element tensor.
extern "C" int msq_sumsq_parts(long long n) {
  const long long per = 8LL * msq::SUMSQ_THREADS;
  long long b = (n + per - 1) / per;
  const long long cap = 4LL * msq::device_sms();
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

// out[0] (+)= sum(g^2).  `scratch` holds msq_sumsq_parts(n) floats of global memory.
extern "C" int msq_sumsq(const void* g, long long n, int dtype, float* scratch, float* out, int accumulate,
                         cudaStream_t stream) {
  using namespace msq;
  const int parts = msq_sumsq_parts(n);
  if (dtype == 0) sumsq_partial_kernel<0><<<parts, SUMSQ_THREADS, 0, stream>>>(g, n, scratch);
  else if (dtype == 1) sumsq_partial_kernel<1><<<parts, SUMSQ_THREADS, 0, stream>>>(g, n, scratch);
  else if (dtype == 2) sumsq_partial_kernel<2><<<parts, SUMSQ_THREADS, 0, stream>>>(g, n, scratch);
  else return -2;
  sumsq_finalize_kernel<<<1, SUMSQ_THREADS, 0, stream>>>(scratch, parts, out, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// List form of msq_sumsq.  `table`: count + 1 records {pointer, elements, first block} (3 x 8 bytes) in device
// memory, the block ranges consecutive and the last record's first block = total_blocks; `scratch`: total_blocks
// floats; `ticket`: one zero-initialised unsigned that the kernel leaves at zero.  All tensors share `dtype`.
// Note block_sum sums per-thread values in a fixed order, so equal inputs give equal bits from call to call.
extern "C" int msq_sumsq_multi(const void* table, int count, int total_blocks, int dtype, float* scratch,
                               unsigned* ticket, float* out, int accumulate, cudaStream_t stream) {
  using namespace msq;
  if (count <= 0 || total_blocks <= 0) return 0;
  const SumsqTensor* tb = static_cast<const SumsqTensor*>(table);
  if (dtype == 0) sumsq_multi_kernel<0, false><<<total_blocks, SUMSQ_THREADS, 0, stream>>>(tb, count, scratch, ticket, out, accumulate);
  else if (dtype == 1) sumsq_multi_kernel<1, false><<<total_blocks, SUMSQ_THREADS, 0, stream>>>(tb, count, scratch, ticket, out, accumulate);
  else if (dtype == 2) sumsq_multi_kernel<2, false><<<total_blocks, SUMSQ_THREADS, 0, stream>>>(tb, count, scratch, ticket, out, accumulate);
  else return -2;
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Same table and scratch as msq_sumsq_multi; out[0] = max |element| over the list (max with the old out[0] when
// `accumulate`), +inf when an element is not finite.
extern "C" int msq_absmax_multi(const void* table, int count, int total_blocks, int dtype, float* scratch,
                                unsigned* ticket, float* out, int accumulate, cudaStream_t stream) {
  using namespace msq;
  if (count <= 0 || total_blocks <= 0) return 0;
  const SumsqTensor* tb = static_cast<const SumsqTensor*>(table);
  if (dtype == 0) sumsq_multi_kernel<0, true><<<total_blocks, SUMSQ_THREADS, 0, stream>>>(tb, count, scratch, ticket, out, accumulate);
  else if (dtype == 1) sumsq_multi_kernel<1, true><<<total_blocks, SUMSQ_THREADS, 0, stream>>>(tb, count, scratch, ticket, out, accumulate);
  else if (dtype == 2) sumsq_multi_kernel<2, true><<<total_blocks, SUMSQ_THREADS, 0, stream>>>(tb, count, scratch, ticket, out, accumulate);
  else return -2;
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Every tensor of the table *= host_scale * (dev_scale ? dev_scale[0] : 1), in place, in one launch.
extern "C" int msq_scale_multi(const void* table, int count, int total_blocks, int dtype, const float* dev_scale,
                               float host_scale, cudaStream_t stream) {
  using namespace msq;
  if (count <= 0 || total_blocks <= 0) return 0;
  const SumsqTensor* tb = static_cast<const SumsqTensor*>(table);
  if (dtype == 0) scale_multi_kernel<0><<<total_blocks, SUMSQ_THREADS, 0, stream>>>(tb, count, dev_scale, host_scale);
  else if (dtype == 1) scale_multi_kernel<1><<<total_blocks, SUMSQ_THREADS, 0, stream>>>(tb, count, dev_scale, host_scale);
  else if (dtype == 2) scale_multi_kernel<2><<<total_blocks, SUMSQ_THREADS, 0, stream>>>(tb, count, dev_scale, host_scale);
  else return -2;
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int msq_clip_decision(const float* sumsq, int n_terms, float pre_factor, float max_norm, float* ctrl_out,
                                 cudaStream_t stream) {
  msq::clip_decision_kernel<<<1, 32, 0, stream>>>(sumsq, n_terms, pre_factor, max_norm, ctrl_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int msq_adamw(void* p, const void* g, float* m, float* v, void* p16_out, int p16_bf16, long long n,
                         int p_dtype, int g_dtype, float lr, float beta1, float beta2, float eps, float weight_decay,
                         float step_size, const float* ctrl, cudaStream_t stream) {
  using namespace msq;
  if (n <= 0) return 0;
  long long blocks = (n + 511) / 512;
  const long long cap = 16LL * device_sms();
  if (blocks > cap) blocks = cap;
  const int b = static_cast<int>(blocks);
#define MSQ_ADAM(PD, GD)                                                                                       \
  adamw_kernel<PD, GD><<<b, 512, 0, stream>>>(p, g, m, v, p16_out, p16_bf16, n, lr, beta1, beta2, eps,        \
                                              weight_decay, step_size, 0.f, ctrl)
  if (p_dtype == 0 && g_dtype == 0) MSQ_ADAM(0, 0);
  else if (p_dtype == 1 && g_dtype == 1) MSQ_ADAM(1, 1);
  else if (p_dtype == 2 && g_dtype == 0) MSQ_ADAM(2, 0);
  else if (p_dtype == 2 && g_dtype == 1) MSQ_ADAM(2, 1);
  else if (p_dtype == 2 && g_dtype == 2) MSQ_ADAM(2, 2);
  else if (p_dtype == 0 && g_dtype == 2) MSQ_ADAM(0, 2);
  else if (p_dtype == 1 && g_dtype == 2) MSQ_ADAM(1, 2);
  else return -2;
#undef MSQ_ADAM
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// List form of msq_adamw (the reference's apex multi_tensor_adam: metaseq/modules/apex/multi_tensor_adam.cu).
// `table`: `count` records {p, g, m, v, n} (5 x 8 bytes each) in device memory; `max_n`: the largest n, which sizes
// the grid.  All tensors share the data types and hyper-parameters.
extern "C" int msq_adamw_multi(const void* table, int count, long long max_n, int p_dtype, int g_dtype, float lr,
                               float beta1, float beta2, float eps, float weight_decay, float step_size,
                               const float* ctrl, cudaStream_t stream) {
  using namespace msq;
  if (count <= 0 || max_n <= 0) return 0;
  if (count > 65535) return -2;
  long long blocks = (max_n / 8 + 511) / 512;
  const long long cap = (16LL * device_sms() + count - 1) / count;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  const dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(count));
  const AdamTensor* tb = static_cast<const AdamTensor*>(table);
#define MSQ_ADAM_MULTI(PD, GD) \
  adamw_multi_kernel<PD, GD><<<grid, 512, 0, stream>>>(tb, lr, beta1, beta2, eps, weight_decay, step_size, ctrl)
  if (p_dtype == 0 && g_dtype == 0) MSQ_ADAM_MULTI(0, 0);
  else if (p_dtype == 1 && g_dtype == 1) MSQ_ADAM_MULTI(1, 1);
  else if (p_dtype == 2 && g_dtype == 0) MSQ_ADAM_MULTI(2, 0);
  else if (p_dtype == 2 && g_dtype == 1) MSQ_ADAM_MULTI(2, 1);
  else if (p_dtype == 2 && g_dtype == 2) MSQ_ADAM_MULTI(2, 2);
  else if (p_dtype == 0 && g_dtype == 2) MSQ_ADAM_MULTI(0, 2);
  else if (p_dtype == 1 && g_dtype == 2) MSQ_ADAM_MULTI(1, 2);
  else return -2;
#undef MSQ_ADAM_MULTI
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

