// LayerNorm forward / backward over rows of a [rows, D] 16-bit matrix with fp32
// statistics.  Replaces the vendored apex kernels the reference calls
// (metaseq/modules/apex/layer_norm_cuda_kernel.cu:382-455 forward,
// :570-864 backward) with a row-in-registers design: each thread owns the same
// 8-wide column vectors for every row its CTA visits, so a row is read from HBM
// exactly once and dgamma/dbeta accumulate in registers across rows.
#include "sm100_common.cuh"

namespace msq {

constexpr int LN_THREADS = 256;

template <bool BF16>
__device__ __forceinline__ void load8(const uint16_t* p, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 t = unpack2<BF16>(w[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
template <bool BF16>
__device__ __forceinline__ void store8(uint16_t* p, const float (&f)[8]) {
  uint4 o;
  o.x = pack2<BF16>(f[0], f[1]);
  o.y = pack2<BF16>(f[2], f[3]);
  o.z = pack2<BF16>(f[4], f[5]);
  o.w = pack2<BF16>(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = o;
}

template <bool BF16, int VPT>
__global__ void __launch_bounds__(LN_THREADS)
layernorm_fwd_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ gamma,
                     const uint16_t* __restrict__ beta, uint16_t* __restrict__ y, float* __restrict__ mean_out,
                     float* __restrict__ rstd_out, int rows, int D, float eps, int rms) {
  __shared__ float red[32];
  const int nvec = D >> 3;
  float g[VPT][8], b[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * LN_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) { g[i][j] = 1.f; b[i][j] = 0.f; }
    if (v < nvec) {
      if (gamma) load8<BF16>(gamma + v * 8, g[i]);
      if (beta) load8<BF16>(beta + v * 8, b[i]);
    }
  }
  const float inv_d = 1.f / static_cast<float>(D);
  dependents_launch();
  dependents_wait();  // gamma / beta above are parameters; x comes from the preceding kernel
  // The row after this one is requested before this one is reduced: the two block-wide sums of a row are
  // latency, and without the prefetch nothing of this CTA is in flight while they run.
  float nxt[VPT][8];
  auto fetch = [&](int row) {
    const uint16_t* xr = x + static_cast<long long>(row) * D;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * LN_THREADS;
      if (v < nvec) {
        load8<BF16>(xr + v * 8, nxt[i]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) nxt[i][j] = 0.f;
      }
    }
  };
  if (static_cast<int>(blockIdx.x) < rows) fetch(blockIdx.x);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    float f[VPT][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        f[i][j] = nxt[i][j];
        s += f[i][j];
      }
    }
    if (row + static_cast<int>(gridDim.x) < rows) fetch(row + gridDim.x);
    const float mean = rms ? 0.f : block_sum(s, red) * inv_d;  // RMS norm: no centring (uniform per launch)
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * LN_THREADS;
      if (v < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = f[i][j] - mean;
          q += d * d;
        }
      }
    }
    const float var = block_sum(q, red) * inv_d;
    const float rstd = rsqrtf(var + eps);
    if (threadIdx.x == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
    uint16_t* yr = y + static_cast<long long>(row) * D;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * LN_THREADS;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (f[i][j] - mean) * rstd * g[i][j] + b[i][j];
        store8<BF16>(yr + v * 8, o);
      }
    }
  }
}

// Forward for rows of at most 2048 elements: one warp per row.  A lane holds VPW 16-byte vectors of the row (all
// requested at once, kept packed), the two sums are warp shuffles, and nothing waits on a block-wide barrier, so
// a CTA has eight independent rows in flight.  gamma / beta are re-read per row (they stay in L1).
template <bool BF16, int VPW>
__global__ void __launch_bounds__(LN_THREADS)
layernorm_fwd_warp_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ gamma,
                          const uint16_t* __restrict__ beta, uint16_t* __restrict__ y, float* __restrict__ mean_out,
                          float* __restrict__ rstd_out, int rows, int D, float eps, int rms) {
  const int nvec = D >> 3;
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * (LN_THREADS / 32);
  const float inv_d = 1.f / static_cast<float>(D);
  dependents_launch();
  dependents_wait();  // x comes from the preceding kernel
  for (int row = blockIdx.x * (LN_THREADS / 32) + (threadIdx.x >> 5); row < rows; row += warps) {
    const uint16_t* xr = x + static_cast<long long>(row) * D;
    uint4 raw[VPW];
#pragma unroll
    for (int i = 0; i < VPW; ++i) {
      const int v = lane + 32 * i;
      raw[i] = v < nvec ? *reinterpret_cast<const uint4*>(xr + v * 8) : make_uint4(0u, 0u, 0u, 0u);
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPW; ++i) {
      const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = unpack2<BF16>(w[j]);
        s += t.x + t.y;
      }
    }
    const float mean = rms ? 0.f : warp_sum(s) * inv_d;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < VPW; ++i) {
      if (lane + 32 * i < nvec) {
        const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 t = unpack2<BF16>(w[j]);
          q += (t.x - mean) * (t.x - mean) + (t.y - mean) * (t.y - mean);
        }
      }
    }
    const float rstd = rsqrtf(warp_sum(q) * inv_d + eps);
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
    uint16_t* yr = y + static_cast<long long>(row) * D;
#pragma unroll
    for (int i = 0; i < VPW; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        float f[8], g[8], b[8];
        const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 t = unpack2<BF16>(w[j]);
          f[2 * j] = t.x;
          f[2 * j + 1] = t.y;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) { g[j] = 1.f; b[j] = 0.f; }
        if (gamma) load8<BF16>(gamma + v * 8, g);
        if (beta) load8<BF16>(beta + v * 8, b);
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (f[j] - mean) * rstd * g[j] + b[j];
        store8<BF16>(yr + v * 8, o);
      }
    }
  }
}

// dx = rstd * (gdy - mean(gdy) - xhat * mean(gdy * xhat)) [+ add], gdy = gamma * dy.
// Per-CTA partial sums of dgamma (= dy * xhat) and dbeta (= dy) go to
// part_g / part_b, each [gridDim.x, D] fp32, reduced by layernorm_bwd_finalize.
template <bool BF16, int VPT>
__global__ void __launch_bounds__(LN_THREADS)
layernorm_bwd_kernel(const uint16_t* __restrict__ dy, const uint16_t* __restrict__ x,
                     const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                     const uint16_t* __restrict__ gamma, const uint16_t* __restrict__ add,
                     uint16_t* __restrict__ dx, float* __restrict__ part_g, float* __restrict__ part_b, int rows,
                     int D, int rms) {
  __shared__ float red[32];
  const int nvec = D >> 3;
  float g[VPT][8], ag[VPT][8], ab[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * LN_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) { g[i][j] = 1.f; ag[i][j] = 0.f; ab[i][j] = 0.f; }
    if (v < nvec && gamma) load8<BF16>(gamma + v * 8, g[i]);
  }
  const float inv_d = 1.f / static_cast<float>(D);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long off = static_cast<long long>(row) * D;
    const float mean = rms ? 0.f : mean_in[row], rstd = rstd_in[row];
    float xh[VPT][8], gd[VPT][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * LN_THREADS;
      if (v < nvec) {
        float xv[8], dv[8];
        load8<BF16>(x + off + v * 8, xv);
        load8<BF16>(dy + off + v * 8, dv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xv[j] - mean) * rstd;
          gd[i][j] = dv[j] * g[i][j];
          s1 += gd[i][j];
          s2 += gd[i][j] * xh[i][j];
          ag[i][j] += dv[j] * xh[i][j];
          ab[i][j] += dv[j];
        }
      }
    }
    const float m1 = rms ? 0.f : block_sum(s1, red) * inv_d;
    const float m2 = block_sum(s2, red) * inv_d;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * LN_THREADS;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (gd[i][j] - m1 - xh[i][j] * m2);
        if (add) {
          float a[8];
          load8<BF16>(add + off + v * 8, a);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += a[j];
        }
        store8<BF16>(dx + off + v * 8, o);
      }
    }
  }
  if (part_g) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * LN_THREADS;
      if (v < nvec) {
        float* pg = part_g + static_cast<long long>(blockIdx.x) * D + v * 8;
        float* pb = part_b + static_cast<long long>(blockIdx.x) * D + v * 8;
        *reinterpret_cast<float4*>(pg) = make_float4(ag[i][0], ag[i][1], ag[i][2], ag[i][3]);
        *reinterpret_cast<float4*>(pg + 4) = make_float4(ag[i][4], ag[i][5], ag[i][6], ag[i][7]);
        *reinterpret_cast<float4*>(pb) = make_float4(ab[i][0], ab[i][1], ab[i][2], ab[i][3]);
        *reinterpret_cast<float4*>(pb + 4) = make_float4(ab[i][4], ab[i][5], ab[i][6], ab[i][7]);
      }
    }
  }
}

// Sums `parts` partial rows per column, then writes (or adds to) the 16-bit gradient.  A CTA owns 32
// columns; its 8 warps each sum every 8th partial row (coalesced 128-byte reads) and the eight
// partial results meet in shared memory.
template <bool BF16>
__global__ void __launch_bounds__(256)
layernorm_bwd_finalize(const float* __restrict__ part_g, const float* __restrict__ part_b, int parts,
                       int D, uint16_t* __restrict__ dgamma, uint16_t* __restrict__ dbeta,
                       int accumulate) {
  __shared__ float red_g[8][33], red_b[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + tx;
  float ag = 0.f, ab = 0.f;
  if (col < D) {
#pragma unroll 4
    for (int p = ty; p < parts; p += 8) {
      ag += part_g[static_cast<long long>(p) * D + col];
      ab += part_b[static_cast<long long>(p) * D + col];
    }
  }
  red_g[ty][tx] = ag;
  red_b[ty][tx] = ab;
  __syncthreads();
  if (ty != 0 || col >= D) return;
  float sg = 0.f, sb = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) { sg += red_g[i][tx]; sb += red_b[i][tx]; }
  auto rd = [](const uint16_t* p) -> float {
    if constexpr (BF16) return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(p));
    else return __half2float(*reinterpret_cast<const __half*>(p));
  };
  auto wr = [](uint16_t* p, float v) {
    if constexpr (BF16) *reinterpret_cast<__nv_bfloat16*>(p) = __float2bfloat16(v);
    else *reinterpret_cast<__half*>(p) = __float2half(v);
  };
  if (dgamma) wr(dgamma + col, sg + (accumulate ? rd(dgamma + col) : 0.f));
  if (dbeta) wr(dbeta + col, sb + (accumulate ? rd(dbeta + col) : 0.f));
}

static int ln_grid(int rows) {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int cap = sms * 4;
  return rows < cap ? rows : cap;
}

// The forward kernel keeps fewer registers per thread, so five CTAs share an SM.
static int ln_grid_fwd(int rows) {
  const int cap = ln_grid(1 << 30) / 4 * 5;
  return rows < cap ? rows : cap;
}

}  // namespace msq

#define MSQ_LN_DISPATCH(NVEC, CALL)                          \
  if (NVEC <= 256) { constexpr int VPT = 1; CALL; }          \
  else if (NVEC <= 512) { constexpr int VPT = 2; CALL; }     \
  else if (NVEC <= 1024) { constexpr int VPT = 4; CALL; }    \
  else if (NVEC <= 1536) { constexpr int VPT = 6; CALL; }    \
  else if (NVEC <= 2048) { constexpr int VPT = 8; CALL; }    \
  else return -1;

// Number of CTAs the backward kernel uses for `rows` rows; the caller sizes the
// partial buffers as [msq_layernorm_bwd_parts(rows), D] fp32 each.
extern "C" int msq_layernorm_bwd_parts(int rows) { return msq::ln_grid(rows); }

namespace msq {
static int norm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd, int rows, int D,
                    float eps, int bf16, int rms, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D & 7) return -2;
  const int nvec = D >> 3;
  const int grid = ln_grid_fwd(rows);
  auto X = static_cast<const uint16_t*>(x);
  auto G = static_cast<const uint16_t*>(gamma);
  auto B = static_cast<const uint16_t*>(beta);
  auto Y = static_cast<uint16_t*>(y);
  if (nvec <= 256 && rows >= 2048) {
    // Many rows: one warp per row, each warp looping over rows.  With few rows (a decode step) the block-per-row
    // kernel below is quicker: a row is spread over 256 threads instead of walked by 32.
    const int vpw = (nvec + 31) / 32;
    const int want = (rows + LN_THREADS / 32 - 1) / (LN_THREADS / 32);
    const int cap = ln_grid(1 << 30) * 2;
    const dim3 g(want < cap ? want : cap), t(LN_THREADS);
#define MSQ_LN_WARP(V)                                                                                                  \
  case V:                                                                                                               \
    if (bf16) launch_chained(layernorm_fwd_warp_kernel<true, V>, g, t, 0, stream, 1u, X, G, B, Y, mean, rstd, rows, D, eps, rms); \
    else launch_chained(layernorm_fwd_warp_kernel<false, V>, g, t, 0, stream, 1u, X, G, B, Y, mean, rstd, rows, D, eps, rms);    \
    break;
    switch (vpw) {
      MSQ_LN_WARP(1) MSQ_LN_WARP(2) MSQ_LN_WARP(3) MSQ_LN_WARP(4) MSQ_LN_WARP(5) MSQ_LN_WARP(6) MSQ_LN_WARP(7) MSQ_LN_WARP(8)
      default: return -1;
    }
#undef MSQ_LN_WARP
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
  }
  if (bf16) {
    MSQ_LN_DISPATCH(nvec, (launch_chained(layernorm_fwd_kernel<true, VPT>, dim3(grid), dim3(LN_THREADS), 0, stream, 1u, X, G, B, Y, mean, rstd, rows, D, eps, rms)))
  } else {
    MSQ_LN_DISPATCH(nvec, (launch_chained(layernorm_fwd_kernel<false, VPT>, dim3(grid), dim3(LN_THREADS), 0, stream, 1u, X, G, B, Y, mean, rstd, rows, D, eps, rms)))
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

static int norm_bwd(const void* dy, const void* x, const float* mean, const float* rstd, const void* gamma,
                    const void* add, void* dx, float* part_g, float* part_b, void* dgamma, void* dbeta, int accumulate,
                    int rows, int D, int bf16, int rms, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D & 7) return -2;
  const int nvec = D >> 3;
  const int grid = ln_grid(rows);
  auto DY = static_cast<const uint16_t*>(dy);
  auto X = static_cast<const uint16_t*>(x);
  auto G = static_cast<const uint16_t*>(gamma);
  auto A = static_cast<const uint16_t*>(add);
  auto DX = static_cast<uint16_t*>(dx);
  if (bf16) {
    MSQ_LN_DISPATCH(nvec, (layernorm_bwd_kernel<true, VPT><<<grid, LN_THREADS, 0, stream>>>(DY, X, mean, rstd, G, A, DX, part_g, part_b, rows, D, rms)))
  } else {
    MSQ_LN_DISPATCH(nvec, (layernorm_bwd_kernel<false, VPT><<<grid, LN_THREADS, 0, stream>>>(DY, X, mean, rstd, G, A, DX, part_g, part_b, rows, D, rms)))
  }
  if (part_g && (dgamma || dbeta)) {
    const int t = 256, b = (D + 31) / 32;
    if (bf16)
      layernorm_bwd_finalize<true><<<b, t, 0, stream>>>(part_g, part_b, grid, D, static_cast<uint16_t*>(dgamma),
                                                        static_cast<uint16_t*>(dbeta), accumulate);
    else
      layernorm_bwd_finalize<false><<<b, t, 0, stream>>>(part_g, part_b, grid, D, static_cast<uint16_t*>(dgamma),
                                                         static_cast<uint16_t*>(dbeta), accumulate);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
}  // namespace msq

extern "C" int msq_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean,
                                 float* rstd, int rows, int D, float eps, int bf16, cudaStream_t stream) {
  return msq::norm_fwd(x, gamma, beta, y, mean, rstd, rows, D, eps, bf16, 0, stream);
}

extern "C" int msq_layernorm_bwd(const void* dy, const void* x, const float* mean, const float* rstd,
                                 const void* gamma, const void* add, void* dx, float* part_g, float* part_b,
                                 void* dgamma, void* dbeta, int accumulate, int rows, int D, int bf16,
                                 cudaStream_t stream) {
  return msq::norm_bwd(dy, x, mean, rstd, gamma, add, dx, part_g, part_b, dgamma, dbeta, accumulate, rows, D, bf16, 0,
                       stream);
}

// RMS norm, y = x * rsqrt(mean(x^2) + eps) * gamma: the LayerNorm kernels without the centring terms (the
// reference exposes it from the same extension: metaseq/modules/apex/layer_norm_cuda.cpp:459-471, rms_* entries).
// `part_b` is still required as scratch by the backward kernel; its column sums are not used.
extern "C" int msq_rmsnorm_fwd(const void* x, const void* gamma, void* y, float* rstd, int rows, int D, float eps, int bf16,
                               cudaStream_t stream) {
  return msq::norm_fwd(x, gamma, nullptr, y, nullptr, rstd, rows, D, eps, bf16, 1, stream);
}

extern "C" int msq_rmsnorm_bwd(const void* dy, const void* x, const float* rstd, const void* gamma, const void* add,
                               void* dx, float* part_g, float* part_b, void* dgamma, int accumulate, int rows, int D,
                               int bf16, cudaStream_t stream) {
  return msq::norm_bwd(dy, x, nullptr, rstd, gamma, add, dx, part_g, part_b, dgamma, nullptr, accumulate, rows, D, bf16, 1,
                       stream);
}
