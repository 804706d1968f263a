// Nucleus (top-p) sampling of one token per row from log-probabilities, without sorting.
//
// The reference sorts the whole vocabulary of every row, takes a cumulative sum, masks the tail, renormalises and
// calls multinomial (metaseq/sequence_generator.py:399-437): half a dozen full passes over [rows, V] per
// generated token, which costs more than the decode step of a small model.  Here one CTA owns a row, keeps its
// probabilities in shared memory (V fp32 values; 50272 of them are 196 KB) and
//   1. finds by bisection on the float bit pattern the largest threshold t with mass{p_i >= t} >= top_p, i.e.
//      the nucleus is {p_i >= t} (the sorted-prefix definition, except that tokens tied with the last one are
//      all kept);
//   2. draws from the nucleus in index order with the caller's uniform number: a block-wide scan of per-thread
//      partial masses finds the thread whose segment holds the draw, and that thread walks its segment.
// The log-probability reported for the token is the input value, as in the reference.
#include "sm100_common.cuh"

namespace msq {

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ float sample_block_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // scratch may still be read from the previous call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = lane < (SAMPLE_THREADS / 32) ? scratch[lane] : 0.f;
  return warp_sum(t);  // every warp reduces the same 32 partials: the result is uniform across the block
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_topp_kernel(const float* __restrict__ lprobs, long long ld, int V, const float* __restrict__ top_p, int p_per_row,
                   const float* __restrict__ uniform, long long* __restrict__ token, float* __restrict__ token_lprob) {
  extern __shared__ float probs[];
  __shared__ float scratch[32];
  __shared__ float seg_mass[SAMPLE_THREADS];
  __shared__ int chosen;
  const int row = blockIdx.x;
  const float* lp = lprobs + static_cast<long long>(row) * ld;
  // contiguous segment per thread (the draw walks one segment in index order)
  const int per = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int i0 = min(V, static_cast<int>(threadIdx.x) * per), i1 = min(V, i0 + per);
  float total = 0.f, biggest = 0.f;
  for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {  // coalesced load; -inf and NaN become 0
    const float x = lp[i];
    const float p = (x == x && x > -INFINITY) ? __expf(x) : 0.f;
    probs[i] = p;
    total += p;
    biggest = fmaxf(biggest, p);
  }
  total = sample_block_sum(total, scratch);
  biggest = warp_max(biggest);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = biggest;
  __syncthreads();
  biggest = warp_max((threadIdx.x & 31) < SAMPLE_THREADS / 32 ? scratch[threadIdx.x & 31] : 0.f);
  const float want = top_p[p_per_row ? row : 0];

  // largest t (as a bit pattern of a non-negative float) with mass{p >= t} >= want; t = 0 keeps everything
  uint32_t lo = 0u, hi = __float_as_uint(biggest);  // invariant: mass(lo) >= want (or lo = 0), answer in [lo, hi]
  if (want < total) {
    for (int it = 0; it < 32 && lo < hi; ++it) {
      const uint32_t mid = lo + ((hi - lo + 1u) >> 1);
      const float t = __uint_as_float(mid);
      float m = 0.f;
      for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
        const float p = probs[i];
        m += p >= t ? p : 0.f;
      }
      m = sample_block_sum(m, scratch);
      if (m >= want) {
        lo = mid;
      } else {
        hi = mid - 1u;
      }
    }
  }
  const float thr = __uint_as_float(lo);

  // draw in index order from {p >= thr, p > 0}
  float mine = 0.f;
  for (int i = i0; i < i1; ++i) {
    const float p = probs[i];
    mine += (p >= thr && p > 0.f) ? p : 0.f;
  }
  seg_mass[threadIdx.x] = mine;
  if (threadIdx.x == 0) chosen = -1;
  __syncthreads();
  if (threadIdx.x < 32) {  // warp 0 scans the 1024 segment masses, 32 per lane
    float run = 0.f;
    float part[SAMPLE_THREADS / 32];
#pragma unroll
    for (int j = 0; j < SAMPLE_THREADS / 32; ++j) {
      part[j] = seg_mass[threadIdx.x * (SAMPLE_THREADS / 32) + j];
      run += part[j];
    }
    float incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, incl, o);
      if (static_cast<int>(threadIdx.x) >= o) incl += up;
    }
    float excl = incl - run;
#pragma unroll
    for (int j = 0; j < SAMPLE_THREADS / 32; ++j) {
      seg_mass[threadIdx.x * (SAMPLE_THREADS / 32) + j] = excl;  // exclusive prefix of every segment
      excl += part[j];
    }
  }
  __syncthreads();
  float u = uniform[row];
  u = fminf(fmaxf(u, 0.f), 0.99999994f);
  // scale the draw by the scanned total (it differs from the bisection's mass by rounding)
  __shared__ float scanned_total;
  if (threadIdx.x == SAMPLE_THREADS - 1) scanned_total = seg_mass[threadIdx.x] + mine;
  __syncthreads();
  const float draw = u * scanned_total;
  const float begin = seg_mass[threadIdx.x];
  if (mine > 0.f && draw >= begin && draw < begin + mine) {
    float run = begin;
    int pick = -1;
    for (int i = i0; i < i1; ++i) {
      const float p = probs[i];
      if (p >= thr && p > 0.f) {
        pick = i;  // the last kept token of the segment takes whatever rounding leaves over
        run += p;
        if (draw < run) break;
      }
    }
    chosen = pick;  // normally one thread; if rounding lets two neighbouring segments claim the draw, either token is a valid draw
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int tok = chosen;
    if (tok < 0) {
      // rounding at a segment boundary (or an all-zero row): fall back to the most probable token
      tok = 0;
      float best = -1.f;
      for (int i = 0; i < V; ++i) {
        if (probs[i] > best) { best = probs[i]; tok = i; }
      }
    }
    token[row] = tok;
    token_lprob[row] = lp[tok];
  }
}

}  // namespace msq

// lprobs: fp32 [rows, V] (row stride ld), -inf for banned tokens; top_p: one value, or one per row when p_per_row;
// uniform: one number in [0, 1) per row; outputs: token ids (int64) and their input log-probabilities.
// V fp32 values must fit in shared memory (V <= 56000).
extern "C" int msq_sample_topp(const float* lprobs, long long ld, int rows, int V, const float* top_p, int p_per_row,
                               const float* uniform, long long* token, float* token_lprob, cudaStream_t stream) {
  using namespace msq;
  if (rows <= 0) return 0;
  if (V <= 0 || V > 56000) return -2;
  const size_t smem = static_cast<size_t>(V) * sizeof(float);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(sample_topp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 56000 * 4) != cudaSuccess)
      return -10;
    configured = true;
  }
  sample_topp_kernel<<<rows, SAMPLE_THREADS, smem, stream>>>(lprobs, ld, V, top_p, p_per_row, uniform, token, token_lprob);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
