// Single-query attention over a preallocated key/value cache (incremental decoding).
//
// The reference concatenates the new key/value onto the cached ones with torch.cat and runs
// bmm + fp32 softmax + bmm per generated token (metaseq/modules/multihead_attention.py:428-476).  Here the
// cache is a preallocated [B, Tmax, H*HD] buffer that the caller appends to in place, and one kernel
// reads every cached key and value exactly once: the operation is bound by that read, so the kernel is
// organised around 16-byte loads with HD/8 lanes per key, an online softmax per lane group, and a merge
// of the groups' (max, sum, accumulator) triples at the end.  Long sequences with few (batch, head)
// pairs are split along the sequence; a second kernel merges the splits.
//
// The "step" form serves a decode step captured in a CUDA graph: the number of cached positions is read
// from device memory (the graph is replayed with a growing cache), and the new token's key/value are taken
// from the projection output and written into the cache by the block that owns the last position, so that
// the append needs no launch of its own.
#include "sm100_common.cuh"

namespace msq {

constexpr int DEC_THREADS = 128;
constexpr float DEC_LOG2E = 1.4426950408889634f;
constexpr int DEC_UNROLL = 2;

// 16-byte load of data that is read once per launch: do not keep it in L1.
__device__ __forceinline__ uint4 ld_stream_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

struct Partial {
  float m, l;
};

template <int HD, bool BF16>
__global__ void __launch_bounds__(DEC_THREADS, 7)
decode_attn_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ kc, const uint16_t* __restrict__ vc,
                   uint16_t* __restrict__ out, const uint8_t* __restrict__ mask, int S, long long q_bs, long long kv_rs,
                   long long kv_bs, long long o_bs, long long mask_bs, float scale_log2, int splits,
                   float* __restrict__ ws, const int* __restrict__ len_ptr, const uint16_t* __restrict__ k_new,
                   const uint16_t* __restrict__ v_new, long long new_bs, int capacity, int hd) {
  // hd: the real head size (a multiple of 8, <= HD).  Lanes whose eight columns lie past it hold zeros and touch no
  // memory, so head sizes such as 80 and 96 run the HD = 128 instantiation.
  constexpr int G = HD / 8;    // lanes per key
  constexpr int KPW = 32 / G;  // keys per warp and iteration
  const int h = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / G, part = lane % G;
  dependents_launch();
  dependents_wait();
  int fresh = -1;  // index of the position whose key/value still sit in the projection output
  if (len_ptr) {
    S = min(*len_ptr + 1, capacity);
    fresh = S - 1;
  }
  const int chunk = (S + splits - 1) / splits;
  const int s0 = split * chunk, s1 = min(S, s0 + chunk);

  const bool live = part * 8 < hd;
  float qv[8];
  {
    const uint4 v = live ? *reinterpret_cast<const uint4*>(q + b * q_bs + h * hd + part * 8) : make_uint4(0u, 0u, 0u, 0u);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack2<BF16>(w[j]);
      qv[2 * j] = f.x * scale_log2;
      qv[2 * j + 1] = f.y * scale_log2;
    }
  }
  float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  const uint16_t* kb = kc + b * kv_bs + h * hd + part * 8;
  const uint16_t* vb = vc + b * kv_bs + h * hd + part * 8;
  const uint8_t* mb = mask ? mask + b * mask_bs : nullptr;
  // Warp-uniform trip count: the shuffles are executed by all 32 lanes in every iteration.  The kernel is bound
  // by the cache read, so the rows of the next iteration are requested before the current ones are used (two
  // register buffers), and DEC_UNROLL keys share one update of the running maximum.
  constexpr int STEP = (DEC_THREADS / 32) * KPW * DEC_UNROLL;
  auto fetch = [&](uint4 (&kq)[DEC_UNROLL], uint4 (&vq)[DEC_UNROLL], int base) {
#pragma unroll
    for (int u = 0; u < DEC_UNROLL; ++u) {
      const long long s = base + u * (STEP / DEC_UNROLL) + sub;
      kq[u] = make_uint4(0u, 0u, 0u, 0u);
      vq[u] = make_uint4(0u, 0u, 0u, 0u);
      if (s < s1 && live) {
        if (s == fresh) {
          kq[u] = *reinterpret_cast<const uint4*>(k_new + b * new_bs + h * hd + part * 8);
          vq[u] = *reinterpret_cast<const uint4*>(v_new + b * new_bs + h * hd + part * 8);
          *reinterpret_cast<uint4*>(const_cast<uint16_t*>(kb) + s * kv_rs) = kq[u];
          *reinterpret_cast<uint4*>(const_cast<uint16_t*>(vb) + s * kv_rs) = vq[u];
        } else {
          kq[u] = ld_stream_16(kb + s * kv_rs);
          vq[u] = ld_stream_16(vb + s * kv_rs);
        }
      }
    }
  };
  auto consume = [&](const uint4 (&kq)[DEC_UNROLL], const uint4 (&vq)[DEC_UNROLL], int base) {
    float dot[DEC_UNROLL];
    float m_new = m;
#pragma unroll
    for (int u = 0; u < DEC_UNROLL; ++u) {
      const long long s = base + u * (STEP / DEC_UNROLL) + sub;
      const uint32_t kw[4] = {kq[u].x, kq[u].y, kq[u].z, kq[u].w};
      float d = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack2<BF16>(kw[j]);
        d = fmaf(qv[2 * j], f.x, d);
        d = fmaf(qv[2 * j + 1], f.y, d);
      }
#pragma unroll
      for (int o = G / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      if (!(s < s1) || (mb && mb[s])) d = -INFINITY;
      dot[u] = d;
      m_new = fmaxf(m_new, d);
    }
    if (m_new > -INFINITY) {  // uniform within a lane group; no shuffles below
      const float alpha = exp2f(m - m_new);  // 0 for the first keys (m = -inf)
      float pr[DEC_UNROLL];
      float psum = 0.f;
#pragma unroll
      for (int u = 0; u < DEC_UNROLL; ++u) {
        pr[u] = exp2f(dot[u] - m_new);  // 0 for an excluded key
        psum += pr[u];
      }
      l = fmaf(l, alpha, psum);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] *= alpha;
#pragma unroll
      for (int u = 0; u < DEC_UNROLL; ++u) {
        const uint32_t vw[4] = {vq[u].x, vq[u].y, vq[u].z, vq[u].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack2<BF16>(vw[j]);
          acc[2 * j] = fmaf(pr[u], f.x, acc[2 * j]);
          acc[2 * j + 1] = fmaf(pr[u], f.y, acc[2 * j + 1]);
        }
      }
      m = m_new;
    }
  };
  {
    uint4 ka[DEC_UNROLL], va[DEC_UNROLL], kb2[DEC_UNROLL], vb2[DEC_UNROLL];
    int base = s0 + warp * KPW;
    if (base < s1) {
      fetch(ka, va, base);
      while (true) {
        int next = base + STEP;
        if (next < s1) fetch(kb2, vb2, next);
        consume(ka, va, base);
        base = next;
        if (base >= s1) break;
        next = base + STEP;
        if (next < s1) fetch(ka, va, next);
        consume(kb2, vb2, base);
        base = next;
        if (base >= s1) break;
      }
    }
  }
  // merge the lane groups of the warp (they hold different keys, same dimensions)
#pragma unroll
  for (int o = G; o < 32; o <<= 1) {
    const float m_o = __shfl_xor_sync(0xffffffffu, m, o);
    const float l_o = __shfl_xor_sync(0xffffffffu, l, o);
    const float m_new = fmaxf(m, m_o);
    const float a = (m == -INFINITY) ? 0.f : exp2f(m - m_new);
    const float bsc = (m_o == -INFINITY) ? 0.f : exp2f(m_o - m_new);
    l = l * a + l_o * bsc;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = acc[j] * a + __shfl_xor_sync(0xffffffffu, acc[j], o) * bsc;
    m = m_new;
  }
  // merge the warps through shared memory
  __shared__ float s_acc[DEC_THREADS / 32][HD];
  __shared__ float s_m[DEC_THREADS / 32], s_l[DEC_THREADS / 32];
  if (sub == 0) {
#pragma unroll
    for (int j = 0; j < 8; ++j) s_acc[warp][part * 8 + j] = acc[j];
    if (part == 0) { s_m[warp] = m; s_l[warp] = l; }
  }
  __syncthreads();
  if (threadIdx.x < HD) {
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_THREADS / 32; ++w) mm = fmaxf(mm, s_m[w]);
    float ll = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_THREADS / 32; ++w) {
      const float sc = (s_m[w] == -INFINITY) ? 0.f : exp2f(s_m[w] - mm);
      ll += s_l[w] * sc;
      a += s_acc[w][threadIdx.x] * sc;
    }
    if (splits == 1) {
      const float r = ll > 0.f ? a / ll : 0.f;
      uint16_t* o = out + b * o_bs + h * hd + threadIdx.x;
      if (static_cast<int>(threadIdx.x) < hd) {
        if (BF16) *reinterpret_cast<__nv_bfloat16*>(o) = __float2bfloat16(r);
        else *reinterpret_cast<__half*>(o) = __float2half(r);
      }
    } else {
      float* w = ws + ((static_cast<long long>(b) * gridDim.x + h) * splits + split) * (HD + 2);
      w[threadIdx.x] = a;
      if (threadIdx.x == 0) { w[HD] = mm; w[HD + 1] = ll; }
    }
  }
}

template <int HD, bool BF16>
__global__ void decode_attn_merge_kernel(const float* __restrict__ ws, uint16_t* __restrict__ out, long long o_bs, int splits,
                                         int hd) {
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  dependents_launch();
  dependents_wait();
  const float* w = ws + (static_cast<long long>(b) * gridDim.x + h) * splits * (HD + 2);
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, w[s * (HD + 2) + HD]);
  float ll = 0.f, a = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = w[s * (HD + 2) + HD];
    const float sc = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
    ll += w[s * (HD + 2) + HD + 1] * sc;
    a += w[s * (HD + 2) + d] * sc;
  }
  const float r = ll > 0.f ? a / ll : 0.f;
  if (d >= hd) return;
  uint16_t* o = out + b * o_bs + h * hd + d;
  if (BF16) *reinterpret_cast<__nv_bfloat16*>(o) = __float2bfloat16(r);
  else *reinterpret_cast<__half*>(o) = __float2half(r);
}

template <int HD, bool BF16>
static int launch_decode(const void* q, const void* kc, const void* vc, void* out, const void* mask, int B, int H, int S,
                         long long q_bs, long long kv_rs, long long kv_bs, long long o_bs, long long mask_bs, float scale,
                         int splits, float* ws, cudaStream_t stream, int hd, const int* len_ptr = nullptr,
                         const void* k_new = nullptr, const void* v_new = nullptr, long long new_bs = 0, int capacity = 0) {
  dim3 grid(H, B, splits);
  launch_chained(decode_attn_kernel<HD, BF16>, grid, dim3(DEC_THREADS), 0, stream, 1u,
                 static_cast<const uint16_t*>(q), static_cast<const uint16_t*>(kc), static_cast<const uint16_t*>(vc),
                 static_cast<uint16_t*>(out), static_cast<const uint8_t*>(mask), S, q_bs, kv_rs, kv_bs, o_bs, mask_bs,
                 scale * DEC_LOG2E, splits, ws, len_ptr, static_cast<const uint16_t*>(k_new),
                 static_cast<const uint16_t*>(v_new), new_bs, capacity, hd);
  if (splits > 1) {
    dim3 g2(H, B);
    launch_chained(decode_attn_merge_kernel<HD, BF16>, g2, dim3(HD), 0, stream, 1u, static_cast<const float*>(ws),
                   static_cast<uint16_t*>(out), o_bs, splits, hd);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace msq

// Number of sequence splits the launch will use for this problem (the caller sizes the workspace:
// B * H * splits * (P + 2) floats with P = 64 for head sizes up to 64 and 128 above; none needed when the answer is 1).
extern "C" int msq_decode_attn_splits(int B, int H, int S) {
  // The kernel keeps seven CTAs per SM busy (148 * 7 = 1036 CTAs in one wave); with fewer (batch, head) pairs
  // than about five per SM the sequence is split so that the grid comes close to one full wave.
  const long long pairs = static_cast<long long>(B) * H;
  if (pairs >= 740 || S < 256) return 1;
  long long want = (1036 + pairs / 2) / pairs;
  const long long cap = S / 128;
  if (want > cap) want = cap;
  if (want > 32) want = 32;
  return want < 1 ? 1 : static_cast<int>(want);
}

// q: [B, H*HD] rows (batch stride q_bs); k/v cache: [B, >=S, H*HD] with row stride kv_rs and batch stride
// kv_bs; out: [B, H*HD] (batch stride o_bs); mask: optional uint8 [B, >=S], non-zero = key excluded.
// Strides in elements.  All 16-bit pointers 16-byte aligned, strides multiples of 8.
extern "C" int msq_decode_attn(const void* q, const void* kc, const void* vc, void* out, const void* mask, int B, int H,
                               int HD, int S, long long q_bs, long long kv_rs, long long kv_bs, long long o_bs,
                               long long mask_bs, float scale, int bf16, float* workspace, int splits,
                               cudaStream_t stream) {
  using namespace msq;
  if (B <= 0 || H <= 0 || S <= 0) return 0;
  if (HD < 8 || HD > 128 || (HD & 7)) return -4;
  if ((q_bs & 7) || (kv_rs & 7) || (kv_bs & 7) || (reinterpret_cast<uintptr_t>(q) & 15) ||
      (reinterpret_cast<uintptr_t>(kc) & 15) || (reinterpret_cast<uintptr_t>(vc) & 15))
    return -2;
  if (splits < 1) splits = 1;
  if (splits > 1 && !workspace) return -3;
#define MSQ_DEC(HDV, BF) \
  return launch_decode<HDV, BF>(q, kc, vc, out, mask, B, H, S, q_bs, kv_rs, kv_bs, o_bs, mask_bs, scale, splits, workspace, stream, HD)
  if (HD <= 64) { if (bf16) MSQ_DEC(64, true); else MSQ_DEC(64, false); }
  if (bf16) MSQ_DEC(128, true); else MSQ_DEC(128, false);
#undef MSQ_DEC
}

// Decode step with the cache length on the device: ``*len_ptr`` positions are cached; the new token's key and
// value (rows of ``k_new`` / ``v_new``, batch stride ``new_bs``) become position ``*len_ptr``, are written into
// the cache (row capacity ``capacity``) and take part in the attention.  The caller increments ``*len_ptr``
// afterwards.  ``s_hint`` (a host estimate of the length) only sizes the sequence split.
extern "C" int msq_decode_attn_step(const void* q, const void* k_new, const void* v_new, long long new_bs, void* kc, void* vc,
                                    void* out, const void* mask, int B, int H, int HD, const int* len_ptr, int capacity,
                                    long long q_bs, long long kv_rs, long long kv_bs, long long o_bs, long long mask_bs,
                                    float scale, int bf16, float* workspace, int splits, cudaStream_t stream) {
  using namespace msq;
  if (B <= 0 || H <= 0 || capacity <= 0) return 0;
  if (HD < 8 || HD > 128 || (HD & 7)) return -4;
  if (!len_ptr || !k_new || !v_new) return -5;
  if ((q_bs & 7) || (kv_rs & 7) || (kv_bs & 7) || (new_bs & 7) || (reinterpret_cast<uintptr_t>(q) & 15) ||
      (reinterpret_cast<uintptr_t>(kc) & 15) || (reinterpret_cast<uintptr_t>(vc) & 15) ||
      (reinterpret_cast<uintptr_t>(k_new) & 15) || (reinterpret_cast<uintptr_t>(v_new) & 15))
    return -2;
  if (splits < 1) splits = 1;
  if (splits > 1 && !workspace) return -3;
#define MSQ_DEC(HDV, BF) \
  return launch_decode<HDV, BF>(q, kc, vc, out, mask, B, H, 0, q_bs, kv_rs, kv_bs, o_bs, mask_bs, scale, splits, workspace, \
                                stream, HD, len_ptr, k_new, v_new, new_bs, capacity)
  if (HD <= 64) { if (bf16) MSQ_DEC(64, true); else MSQ_DEC(64, false); }
  if (bf16) MSQ_DEC(128, true); else MSQ_DEC(128, false);
#undef MSQ_DEC
}
