// Token + learned-position embedding (forward gather, backward scatter-add),
// softmax cross-entropy over a [rows, V] logits matrix with the gradient
// written in place, and a column-sum reduction used for bias gradients.
//
// Reference behaviour:
//   * embedding: token row * embed_scale + position row, positions counted from
//     padding_idx + 1 over non-pad tokens (metaseq/models/transformer_decoder.py:263-346,
//     metaseq/utils.py:83-93, metaseq/modules/learned_positional_embedding.py:23-54)
//   * cross entropy: fp32 log-softmax, summed NLL, ignore pad targets
//     (metaseq/criterions/cross_entropy.py:40-136,
//      metaseq/modules/megatron/mpu/cross_entropy.py:19-109 for the in-place
//      "overwrite logits with softmax" trick the backward relies on)
#include "sm100_common.cuh"

namespace msq {

// ------------------------------------------------------------ embedding fwd
// out[r, :] = tok_w[tokens[r] - vocab_start, :] * scale + pos_w[positions[r], :]
// Rows whose token is outside [vocab_start, vocab_end) contribute only the
// position term on partition 0 and nothing elsewhere (vocab-parallel masking).
template <bool BF16>
__global__ void embed_fwd_kernel(const long long* __restrict__ tokens, const long long* __restrict__ positions,
                                 const uint16_t* __restrict__ tok_w, const uint16_t* __restrict__ pos_w,
                                 uint16_t* __restrict__ out, int rows, int D, float scale, long long vocab_start,
                                 long long vocab_end, int add_positions) {
  const int nvec = D >> 3;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const long long tok = tokens[r];
    const bool in_range = tok >= vocab_start && tok < vocab_end;
    const uint16_t* tw = tok_w + (tok - vocab_start) * D;
    const uint16_t* pw = (pos_w && add_positions) ? pos_w + positions[r] * D : nullptr;
    uint16_t* o = out + static_cast<long long>(r) * D;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = 0.f;
      if (in_range) {
        const uint4 a = *reinterpret_cast<const uint4*>(tw + v * 8);
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 t = unpack2<BF16>(w[j]);
          f[2 * j] = t.x * scale;
          f[2 * j + 1] = t.y * scale;
        }
      }
      if (pw) {
        const uint4 a = *reinterpret_cast<const uint4*>(pw + v * 8);
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 t = unpack2<BF16>(w[j]);
          f[2 * j] += t.x;
          f[2 * j + 1] += t.y;
        }
      }
      uint4 ov;
      ov.x = pack2<BF16>(f[0], f[1]);
      ov.y = pack2<BF16>(f[2], f[3]);
      ov.z = pack2<BF16>(f[4], f[5]);
      ov.w = pack2<BF16>(f[6], f[7]);
      *reinterpret_cast<uint4*>(o + v * 8) = ov;
    }
  }
}

// ------------------------------------------------------------ embedding bwd
// Scatter-add of dy rows into fp32 gradient tables (atomics); the caller folds
// the fp32 tables into the 16-bit flat gradient afterwards.
template <bool BF16>
__global__ void embed_bwd_kernel(const long long* __restrict__ tokens, const long long* __restrict__ positions,
                                 const uint16_t* __restrict__ dy, float* __restrict__ dtok, float* __restrict__ dpos,
                                 int rows, int D, float scale, long long vocab_start, long long vocab_end,
                                 long long pad_idx) {
  const int nh = D >> 1;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const long long tok = tokens[r];
    const bool in_range = tok >= vocab_start && tok < vocab_end && tok != pad_idx;
    const long long pos = positions ? positions[r] : -1;
    const uint32_t* d = reinterpret_cast<const uint32_t*>(dy + static_cast<long long>(r) * D);
    float* tw = dtok + (tok - vocab_start) * D;
    float* pw = (dpos && pos >= 0 && pos != pad_idx) ? dpos + pos * D : nullptr;
    for (int h = threadIdx.x; h < nh; h += blockDim.x) {
      const float2 t = unpack2<BF16>(d[h]);
      if (in_range && dtok) {
        atomicAdd(tw + 2 * h, t.x * scale);
        atomicAdd(tw + 2 * h + 1, t.y * scale);
      }
      if (pw) {
        atomicAdd(pw + 2 * h, t.x);
        atomicAdd(pw + 2 * h + 1, t.y);
      }
    }
  }
}

// dst16[i] = (accumulate ? dst16[i] : 0) + src32[i]
template <bool BF16>
__global__ void fold_fp32_kernel(const float* __restrict__ src, uint16_t* __restrict__ dst, long long n,
                                 int accumulate) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long n2 = n >> 1;
  uint32_t* d2 = reinterpret_cast<uint32_t*>(dst);
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n2; i += stride) {
    float a = src[2 * i], b = src[2 * i + 1];
    if (accumulate) {
      const float2 o = unpack2<BF16>(d2[i]);
      a += o.x;
      b += o.y;
    }
    d2[i] = pack2<BF16>(a, b);
  }
}

// x[r, c] *= g[r] (or g[0] when `per_row` is 0), in place, 8 elements per thread: the chain-rule factor applied to
// a stored gradient (the loss scale on d(loss)/d(logits)), read from device memory so that no host sync is needed.
template <bool BF16, typename G>
__global__ void scale_rows_kernel(uint16_t* __restrict__ x, long long ld, long long rows, int cols,
                                  const G* __restrict__ g, int per_row) {
  const int vec_per_row = cols >> 3;
  const long long total = rows * vec_per_row;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i - r * vec_per_row) * 8;
    const float f = static_cast<float>(g[per_row ? r : 0]);
    uint4* p = reinterpret_cast<uint4*>(x + r * ld + c);
    uint4 v = *p;
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = unpack2<BF16>(w[j]);
      w[j] = pack2<BF16>(t.x * f, t.y * f);
    }
    *p = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// dst16[r, c] = src32[r, c]: contiguous fp32 rows to 16-bit rows of a strided view, 8 elements per thread.
template <bool BF16>
__global__ void convert_rows_kernel(const float* __restrict__ src, uint16_t* __restrict__ dst, long long rows,
                                    int cols, long long dst_ld) {
  const int vec_per_row = cols >> 3;
  const long long total = rows * vec_per_row;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / vec_per_row;
    const int v = static_cast<int>(i - r * vec_per_row);
    const float4 a = *reinterpret_cast<const float4*>(src + r * cols + v * 8);
    const float4 b = *reinterpret_cast<const float4*>(src + r * cols + v * 8 + 4);
    uint4 o;
    o.x = pack2<BF16>(a.x, a.y);
    o.y = pack2<BF16>(a.z, a.w);
    o.z = pack2<BF16>(b.x, b.y);
    o.w = pack2<BF16>(b.z, b.w);
    *reinterpret_cast<uint4*>(dst + r * dst_ld + v * 8) = o;
  }
}

// ------------------------------------------------------------ cross entropy
// One CTA per row.  The row (V 16-bit logits) is staged in shared memory, so
// HBM sees one read and, when the gradient is requested, one write.
//   loss[r]  = logsumexp(logits[r, :]) - logits[r, target[r]]      (0 for ignored rows)
//   lse[r]   = logsumexp
//   grad     : logits[r, :] <- (softmax - onehot) * grad_scale      (0 for ignored rows)
// vocab_valid <= V lets the caller exclude padded columns at the end of a row.
template <bool BF16>
__global__ void __launch_bounds__(512)
cross_entropy_kernel(uint16_t* __restrict__ logits, long long ld, const long long* __restrict__ target,
                     float* __restrict__ loss, float* __restrict__ lse_out, int rows, int V, long long ignore_index,
                     float grad_scale, int write_grad) {
  extern __shared__ uint4 row_smem[];
  __shared__ float red[32];
  uint16_t* srow = reinterpret_cast<uint16_t*>(row_smem);
  const int nvec = V >> 3;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    uint16_t* grow = logits + static_cast<long long>(r) * ld;
    const long long tgt = target[r];
    const bool ignored = tgt == ignore_index;
    float mx = -INFINITY;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const uint4 a = *reinterpret_cast<const uint4*>(grow + v * 8);
      row_smem[v] = a;
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = unpack2<BF16>(w[j]);
        mx = fmaxf(mx, fmaxf(t.x, t.y));
      }
    }
    mx = block_max(mx, red);
    float se = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const uint4 a = row_smem[v];
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = unpack2<BF16>(w[j]);
        se += __expf(t.x - mx) + __expf(t.y - mx);
      }
    }
    se = block_sum(se, red);
    const float lse = mx + __logf(se);
    if (threadIdx.x == 0) {
      float tl = 0.f;
      if (!ignored) {
        const uint16_t raw = srow[tgt];
        tl = BF16 ? __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&raw))
                  : __half2float(*reinterpret_cast<const __half*>(&raw));
      }
      if (loss) loss[r] = ignored ? 0.f : (lse - tl);
      if (lse_out) lse_out[r] = lse;
    }
    if (write_grad) {
      const float gs = ignored ? 0.f : grad_scale;
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        const uint4 a = row_smem[v];
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
        float f[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 t = unpack2<BF16>(w[j]);
          f[2 * j] = __expf(t.x - lse) * gs;
          f[2 * j + 1] = __expf(t.y - lse) * gs;
        }
        const long long c0 = static_cast<long long>(v) * 8;
        if (!ignored && tgt >= c0 && tgt < c0 + 8) f[tgt - c0] -= gs;
        uint4 o;
        o.x = pack2<BF16>(f[0], f[1]);
        o.y = pack2<BF16>(f[2], f[3]);
        o.z = pack2<BF16>(f[4], f[5]);
        o.w = pack2<BF16>(f[6], f[7]);
        *reinterpret_cast<uint4*>(grow + v * 8) = o;
      }
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------ dropout
// out[r, c] = residual[r, c] + keep(r, c) ? (y[r, c] + bias[c]) / (1 - p) : 0      (residual, bias optional)
// With y == dy, no bias and no residual this is also the backward of the dropped branch.  The mask is the hash of
// (seed, r * cols + c); rows of y / residual / out may be strided.
template <bool BF16>
__global__ void dropout_add_kernel(const uint16_t* __restrict__ y, long long ldy, const uint16_t* __restrict__ bias,
                                   const uint16_t* __restrict__ residual, long long ldr, uint16_t* __restrict__ out,
                                   long long ldo, long long rows, int cols, uint32_t threshold16, float inv_keep,
                                   unsigned long long seed) {
  const int vec_per_row = cols >> 3;
  const long long total = rows * vec_per_row;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i - r * vec_per_row) * 8;
    const uint4 a = *reinterpret_cast<const uint4*>(y + r * ldy + c);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
    uint32_t bw[4] = {0u, 0u, 0u, 0u}, rw[4] = {0u, 0u, 0u, 0u};
    if (bias) {
      const uint4 b4 = *reinterpret_cast<const uint4*>(bias + c);
      bw[0] = b4.x; bw[1] = b4.y; bw[2] = b4.z; bw[3] = b4.w;
    }
    if (residual) {
      const uint4 r4 = *reinterpret_cast<const uint4*>(residual + r * ldr + c);
      rw[0] = r4.x; rw[1] = r4.y; rw[2] = r4.z; rw[3] = r4.w;
    }
    const unsigned long long pair0 = (static_cast<unsigned long long>(r) * cols + c) >> 1;
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 v = unpack2<BF16>(w[j]);
      if (bias) {
        const float2 b2 = unpack2<BF16>(bw[j]);
        v.x += b2.x;
        v.y += b2.y;
      }
      bool k0, k1;
      dropout_keep2(dropout_bits(seed, pair0 + j), threshold16, k0, k1);
      v.x = k0 ? v.x * inv_keep : 0.f;
      v.y = k1 ? v.y * inv_keep : 0.f;
      if (residual) {
        const float2 r2 = unpack2<BF16>(rw[j]);
        v.x += r2.x;
        v.y += r2.y;
      }
      o[j] = pack2<BF16>(v.x, v.y);
    }
    *reinterpret_cast<uint4*>(out + r * ldo + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ------------------------------------------------- vocabulary-parallel cross entropy
// Each tensor-parallel rank holds logits[rows, V_local] for vocabulary ids [vocab_start, vocab_start + V_local).
// Phase 1 writes, per row, (local max, sum of exp(x - local max), target logit or 0) into this rank's block of a
// [world, rows, 3] fp32 table whose other blocks stay zero, so one SUM all-reduce of the table is an all-gather.
// Phase 2 combines the `world` triples of a row into the global log-sum-exp, writes the loss and overwrites the
// local logits with (softmax - onehot) * grad_scale.  Reference: three separate all-reduces around unfused ops
// (metaseq/modules/megatron/mpu/cross_entropy.py:19-109).
template <bool BF16>
__global__ void __launch_bounds__(256)
vp_ce_partial_kernel(const uint16_t* __restrict__ logits, long long ld, const long long* __restrict__ target,
                     float* __restrict__ stats_block, int rows, int V, long long vocab_start) {
  __shared__ float red[32];
  const int nvec = V >> 3;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const uint16_t* grow = logits + static_cast<long long>(r) * ld;
    float mx = -INFINITY;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const uint4 a = *reinterpret_cast<const uint4*>(grow + v * 8);
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = unpack2<BF16>(w[j]);
        mx = fmaxf(mx, fmaxf(t.x, t.y));
      }
    }
    mx = block_max(mx, red);
    float se = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {  // second read comes from L2 / L1
      const uint4 a = *reinterpret_cast<const uint4*>(grow + v * 8);
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = unpack2<BF16>(w[j]);
        se += __expf(t.x - mx) + __expf(t.y - mx);
      }
    }
    se = block_sum(se, red);
    if (threadIdx.x == 0) {
      const long long lt = target[r] - vocab_start;
      float tl = 0.f;
      if (lt >= 0 && lt < V) {
        const uint16_t raw = grow[lt];
        tl = BF16 ? __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&raw))
                  : __half2float(*reinterpret_cast<const __half*>(&raw));
      }
      float* o = stats_block + static_cast<long long>(r) * 3;
      o[0] = mx;
      o[1] = se;
      o[2] = tl;
    }
    __syncthreads();
  }
}

template <bool BF16>
__global__ void __launch_bounds__(256)
vp_ce_finish_kernel(uint16_t* __restrict__ logits, long long ld, const long long* __restrict__ target,
                    const float* __restrict__ stats, int world, float* __restrict__ loss, int rows, int V,
                    long long vocab_start, long long ignore_index, float grad_scale) {
  const int nvec = V >> 3;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    float gmax = -INFINITY;
    for (int w = 0; w < world; ++w) gmax = fmaxf(gmax, stats[(static_cast<long long>(w) * rows + r) * 3]);
    float gsum = 0.f, tl = 0.f;
    for (int w = 0; w < world; ++w) {
      const float* st = stats + (static_cast<long long>(w) * rows + r) * 3;
      gsum += st[1] * __expf(st[0] - gmax);
      tl += st[2];
    }
    const float lse = gmax + __logf(gsum);
    const long long tgt = target[r];
    const bool ignored = tgt == ignore_index;
    if (threadIdx.x == 0 && loss) loss[r] = ignored ? 0.f : (lse - tl);
    const float gs = ignored ? 0.f : grad_scale;
    const long long lt = tgt - vocab_start;
    uint16_t* grow = logits + static_cast<long long>(r) * ld;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const uint4 a = *reinterpret_cast<const uint4*>(grow + v * 8);
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
      float f[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = unpack2<BF16>(w[j]);
        f[2 * j] = __expf(t.x - lse) * gs;
        f[2 * j + 1] = __expf(t.y - lse) * gs;
      }
      const long long c0 = static_cast<long long>(v) * 8;
      if (!ignored && lt >= c0 && lt < c0 + 8) f[lt - c0] -= gs;
      uint4 o;
      o.x = pack2<BF16>(f[0], f[1]);
      o.y = pack2<BF16>(f[2], f[3]);
      o.z = pack2<BF16>(f[4], f[5]);
      o.w = pack2<BF16>(f[6], f[7]);
      *reinterpret_cast<uint4*>(grow + v * 8) = o;
    }
  }
}

// ---------------------------------------- cross entropy from the logits product's row statistics
// The logits GEMM (msq_gemm2_rowstats) leaves, per column tile and row, the maximum of the stored logits and the sum
// of exp(logit - max).  One warp per row folds the tiles into this rank's triple (max, sum-exp, target logit) and
// delivers it: to a local [rows, 3] table (one rank), or into the exchange table of every tensor-parallel peer over
// NVLink (plain peer stores, no library collective).  An exchanged value travels as an 8-byte unit {fp32 value,
// epoch}; 8-byte stores are indivisible, so a reader that sees the epoch it waits for also sees the value, and no
// separate flag, fence or remote load is needed.  Table layout on every rank: unit[(src_rank * rows_cap + row) * 3 + k].
struct CePeers {
  unsigned long long* table[16];
};

template <bool BF16>
__global__ void __launch_bounds__(256)
ce_merge_rowstats_kernel(const float* __restrict__ rs_max, const float* __restrict__ rs_sum, int tiles_n, int rows,
                         const uint16_t* __restrict__ logits, long long ld, const long long* __restrict__ target,
                         int V, long long vocab_start, float* __restrict__ local_stats, CePeers peers, int world,
                         int rank, int rows_cap, uint32_t epoch) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    float m = -INFINITY;
    for (int t = lane; t < tiles_n; t += 32) m = fmaxf(m, rs_max[static_cast<long long>(t) * rows + r]);
    m = warp_max(m);
    float s = 0.f;
    for (int t = lane; t < tiles_n; t += 32) {
      const long long i = static_cast<long long>(t) * rows + r;
      s += rs_sum[i] * __expf(rs_max[i] - m);
    }
    s = warp_sum(s);
    if (lane < 3) {
      float val = lane == 0 ? m : s;
      if (lane == 2) {
        const long long lt = target[r] - vocab_start;
        val = 0.f;
        if (lt >= 0 && lt < V) {
          const uint16_t raw = logits[static_cast<long long>(r) * ld + lt];
          val = BF16 ? __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&raw))
                     : __half2float(*reinterpret_cast<const __half*>(&raw));
        }
      }
      if (world <= 1) {
        local_stats[static_cast<long long>(r) * 3 + lane] = val;
      } else {
        const unsigned long long unit =
            (static_cast<unsigned long long>(epoch) << 32) | static_cast<unsigned long long>(__float_as_uint(val));
        const long long slot = (static_cast<long long>(rank) * rows_cap + r) * 3 + lane;
        for (int w = 0; w < world; ++w) {
          unsigned long long* dst = peers.table[(rank + w) % world] + slot;  // own table first, then round the ring
          asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(unit) : "memory");
        }
      }
    }
  }
}

// Second half on every rank: waits (bounded) until the triples of all ranks for a row carry `epoch`, combines them
// into the global log-sum-exp, writes the loss and overwrites the local logits with (softmax - onehot) * grad_scale.
template <bool BF16>
__global__ void __launch_bounds__(256)
vp_ce_finish_exchanged_kernel(uint16_t* __restrict__ logits, long long ld, const long long* __restrict__ target,
                              const unsigned long long* __restrict__ table, int world, int rows_cap, uint32_t epoch,
                              float* __restrict__ loss, int rows, int V, long long vocab_start,
                              long long ignore_index, float grad_scale, int* __restrict__ status) {
  __shared__ float trip[16 * 3];
  __shared__ int failed;
  const int nvec = V >> 3;
  if (threadIdx.x == 0) failed = (status && *reinterpret_cast<volatile int*>(status) != 0) ? 1 : 0;
  __syncthreads();
  if (failed) return;  // an earlier kernel timed out: do nothing until the host has cleared the status word
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    if (threadIdx.x < world * 3) {
      const int w = threadIdx.x / 3, k = threadIdx.x - w * 3;
      const unsigned long long* src = table + (static_cast<long long>(w) * rows_cap + r) * 3 + k;
      const unsigned long long t0 = globaltimer_ns();
      unsigned long long unit;
      uint32_t spins = 0;
      while (true) {
        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(unit) : "l"(src) : "memory");
        if (static_cast<uint32_t>(unit >> 32) == epoch) break;
        if ((++spins & 0x3f) == 0) {
          if (globaltimer_ns() - t0 > WAIT_NS_PEER) {
            if (status) atomicCAS(status, 0, ST_TIMEOUT_PEER_FLAG);
            failed = 1;
            break;
          }
          __nanosleep(200);
        }
      }
      trip[threadIdx.x] = __uint_as_float(static_cast<uint32_t>(unit));
    }
    __syncthreads();
    if (failed) return;
    float gmax = -INFINITY;
    for (int w = 0; w < world; ++w) gmax = fmaxf(gmax, trip[w * 3]);
    float gsum = 0.f, tl = 0.f;
    for (int w = 0; w < world; ++w) {
      gsum += trip[w * 3 + 1] * __expf(trip[w * 3] - gmax);
      tl += trip[w * 3 + 2];
    }
    __syncthreads();  // trip is rewritten for the next row
    const float lse = gmax + __logf(gsum);
    const long long tgt = target[r];
    const bool ignored = tgt == ignore_index;
    if (threadIdx.x == 0 && loss) loss[r] = ignored ? 0.f : (lse - tl);
    const float gs = ignored ? 0.f : grad_scale;
    const long long lt = tgt - vocab_start;
    uint16_t* grow = logits + static_cast<long long>(r) * ld;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const uint4 a = *reinterpret_cast<const uint4*>(grow + v * 8);
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
      float f[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = unpack2<BF16>(w[j]);
        f[2 * j] = __expf(t.x - lse) * gs;
        f[2 * j + 1] = __expf(t.y - lse) * gs;
      }
      const long long c0 = static_cast<long long>(v) * 8;
      if (!ignored && lt >= c0 && lt < c0 + 8) f[lt - c0] -= gs;
      uint4 o;
      o.x = pack2<BF16>(f[0], f[1]);
      o.y = pack2<BF16>(f[2], f[3]);
      o.z = pack2<BF16>(f[4], f[5]);
      o.w = pack2<BF16>(f[6], f[7]);
      *reinterpret_cast<uint4*>(grow + v * 8) = o;
    }
  }
}

// x[r, :] *= g[r or 0] * inv_ref, rows whose factor is exactly 1 left untouched (not even read).  The forward pass
// stores a gradient already multiplied by the factor it expects from upstream (the loss scale, 1 / inv_ref); when
// the backward pass brings exactly that factor this launch costs a few microseconds instead of a pass over memory.
template <bool BF16, typename G>
__global__ void __launch_bounds__(256)
scale_rows_rel_kernel(uint16_t* __restrict__ x, long long ld, long long rows, int cols, const G* __restrict__ g,
                      int per_row, float inv_ref) {
  const int nvec = cols >> 3;
  if (!per_row && static_cast<float>(g[0]) * inv_ref == 1.f) return;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const float f = static_cast<float>(g[per_row ? r : 0]) * inv_ref;
    if (f == 1.f) continue;
    uint16_t* row = x + r * ld;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      uint4* p = reinterpret_cast<uint4*>(row + v * 8);
      const uint4 a = *p;
      uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = unpack2<BF16>(w[j]);
        w[j] = pack2<BF16>(t.x * f, t.y * f);
      }
      *p = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// ------------------------------------------------------------------ colsum
// acc[n] += sum over a slice of rows of x[m, n]; fp32 atomics, one per column
// per CTA.  Block = 32 x 8 threads, each thread owns 8 adjacent columns.
template <bool BF16>
__global__ void __launch_bounds__(256)
colsum_kernel(const uint16_t* __restrict__ x, long long ld, int rows, int N, float* __restrict__ acc,
              int rows_per_cta) {
  __shared__ float sm[8][256 + 8];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + tx * 8;
  const int r0 = blockIdx.y * rows_per_cta;
  const int r1 = min(rows, r0 + rows_per_cta);
  float s[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s[j] = 0.f;
  if (col < N) {
    for (int r = r0 + ty; r < r1; r += 8) {
      const uint4 a = *reinterpret_cast<const uint4*>(x + static_cast<long long>(r) * ld + col);
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = unpack2<BF16>(w[j]);
        s[2 * j] += t.x;
        s[2 * j + 1] += t.y;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) sm[ty][tx * 8 + j] = s[j];
  __syncthreads();
  const int c = threadIdx.x;
  if (blockIdx.x * 256 + c < N) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += sm[k][c];
    atomicAdd(acc + blockIdx.x * 256 + c, t);
  }
}

// One-launch form of the bias gradient: the same slice sums and fp32 atomics as colsum_kernel, after which the CTA
// that arrives last at a column block (a ticket per block) turns the block's fp32 sums into the 16-bit output
// (added to it when `accumulate`) and leaves accumulator and ticket at zero for the next call, so the scratch needs
// no fill and the result no separate conversion pass.
template <bool BF16>
__global__ void __launch_bounds__(256)
colsum_direct_kernel(const uint16_t* __restrict__ x, long long ld, int rows, int N, float* __restrict__ acc,
                     unsigned* __restrict__ tickets, uint16_t* __restrict__ out, int accumulate, int rows_per_cta) {
  __shared__ float sm[8][256 + 8];
  __shared__ bool last;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + tx * 8;
  const int r0 = blockIdx.y * rows_per_cta;
  const int r1 = min(rows, r0 + rows_per_cta);
  float s[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s[j] = 0.f;
  if (col < N) {
    for (int r = r0 + ty; r < r1; r += 8) {
      const uint4 a = *reinterpret_cast<const uint4*>(x + static_cast<long long>(r) * ld + col);
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = unpack2<BF16>(w[j]);
        s[2 * j] += t.x;
        s[2 * j + 1] += t.y;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) sm[ty][tx * 8 + j] = s[j];
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < N) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += sm[k][threadIdx.x];
    atomicAdd(acc + c, t);
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(tickets + blockIdx.x, 1u) == gridDim.y - 1;
  __syncthreads();
  if (!last) return;
  __threadfence();
  if (c < N) {
    float t = __ldcg(acc + c);
    if (accumulate) {
      const uint16_t prev = out[c];
      t += BF16 ? __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&prev))
                : __half2float(*reinterpret_cast<const __half*>(&prev));
    }
    if (BF16) *reinterpret_cast<__nv_bfloat16*>(out + c) = __float2bfloat16(t);
    else *reinterpret_cast<__half*>(out + c) = __float2half(t);
    acc[c] = 0.f;
  }
  if (threadIdx.x == 0) tickets[blockIdx.x] = 0;
}

}  // namespace msq

extern "C" int msq_embed_fwd(const long long* tokens, const long long* positions, const void* tok_w,
                             const void* pos_w, void* out, int rows, int D, float scale, long long vocab_start,
                             long long vocab_end, int add_positions, int bf16, cudaStream_t stream) {
  using namespace msq;
  if (rows <= 0) return 0;
  if (D & 7) return -2;
  const int threads = (D >> 3) < 256 ? (((D >> 3) + 31) / 32 * 32) : 256;
  const int grid = rows < 148 * 16 ? rows : 148 * 16;
  if (bf16)
    embed_fwd_kernel<true><<<grid, threads, 0, stream>>>(tokens, positions, static_cast<const uint16_t*>(tok_w),
                                                         static_cast<const uint16_t*>(pos_w),
                                                         static_cast<uint16_t*>(out), rows, D, scale, vocab_start,
                                                         vocab_end, add_positions);
  else
    embed_fwd_kernel<false><<<grid, threads, 0, stream>>>(tokens, positions, static_cast<const uint16_t*>(tok_w),
                                                          static_cast<const uint16_t*>(pos_w),
                                                          static_cast<uint16_t*>(out), rows, D, scale, vocab_start,
                                                          vocab_end, add_positions);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int msq_embed_bwd(const long long* tokens, const long long* positions, const void* dy, float* dtok,
                             float* dpos, int rows, int D, float scale, long long vocab_start, long long vocab_end,
                             long long pad_idx, int bf16, cudaStream_t stream) {
  using namespace msq;
  if (rows <= 0) return 0;
  if (D & 1) return -2;
  const int grid = rows < 148 * 16 ? rows : 148 * 16;
  if (bf16)
    embed_bwd_kernel<true><<<grid, 256, 0, stream>>>(tokens, positions, static_cast<const uint16_t*>(dy), dtok, dpos,
                                                     rows, D, scale, vocab_start, vocab_end, pad_idx);
  else
    embed_bwd_kernel<false><<<grid, 256, 0, stream>>>(tokens, positions, static_cast<const uint16_t*>(dy), dtok, dpos,
                                                      rows, D, scale, vocab_start, vocab_end, pad_idx);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int msq_fold_fp32(const float* src, void* dst, long long n, int accumulate, int bf16,
                             cudaStream_t stream) {
  using namespace msq;
  if (n <= 0) return 0;
  if (n & 1) return -2;
  long long blocks = (n / 2 + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (bf16) fold_fp32_kernel<true><<<static_cast<int>(blocks), 256, 0, stream>>>(src, static_cast<uint16_t*>(dst), n, accumulate);
  else fold_fp32_kernel<false><<<static_cast<int>(blocks), 256, 0, stream>>>(src, static_cast<uint16_t*>(dst), n, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// src: contiguous fp32 [rows, cols]; dst: 16-bit [rows, cols] with row stride dst_ld (elements).
extern "C" int msq_convert_rows(const float* src, void* dst, long long rows, int cols, long long dst_ld, int bf16,
                                cudaStream_t stream) {
  using namespace msq;
  if (rows <= 0 || cols <= 0) return 0;
  if ((cols & 7) || (dst_ld & 7) || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) return -2;
  long long blocks = (rows * (cols >> 3) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (bf16) convert_rows_kernel<true><<<static_cast<int>(blocks), 256, 0, stream>>>(src, static_cast<uint16_t*>(dst), rows, cols, dst_ld);
  else convert_rows_kernel<false><<<static_cast<int>(blocks), 256, 0, stream>>>(src, static_cast<uint16_t*>(dst), rows, cols, dst_ld);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// x: 16-bit [rows, cols] with row stride ld, scaled in place by g (fp32 when g_fp32, else the type of x): one
// factor per row, or a single factor when per_row is 0.
extern "C" int msq_scale_rows(void* x, long long ld, long long rows, int cols, const void* g, int g_fp32, int per_row,
                              int bf16, cudaStream_t stream) {
  using namespace msq;
  if (rows <= 0 || cols <= 0) return 0;
  if ((cols & 7) || (ld & 7) || (reinterpret_cast<uintptr_t>(x) & 15)) return -2;
  long long blocks = (rows * (cols >> 3) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  const int nb = static_cast<int>(blocks);
  uint16_t* xp = static_cast<uint16_t*>(x);
  if (g_fp32) {
    if (bf16) scale_rows_kernel<true, float><<<nb, 256, 0, stream>>>(xp, ld, rows, cols, static_cast<const float*>(g), per_row);
    else scale_rows_kernel<false, float><<<nb, 256, 0, stream>>>(xp, ld, rows, cols, static_cast<const float*>(g), per_row);
  } else if (bf16) {
    scale_rows_kernel<true, __nv_bfloat16><<<nb, 256, 0, stream>>>(xp, ld, rows, cols, static_cast<const __nv_bfloat16*>(g), per_row);
  } else {
    scale_rows_kernel<false, __half><<<nb, 256, 0, stream>>>(xp, ld, rows, cols, static_cast<const __half*>(g), per_row);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int msq_cross_entropy(void* logits, long long ld, const long long* target, float* loss, float* lse,
                                 int rows, int V, long long ignore_index, float grad_scale, int write_grad, int bf16,
                                 cudaStream_t stream) {
  using namespace msq;
  if (rows <= 0) return 0;
  if ((V & 7) || (ld & 7)) return -2;
  const size_t smem = static_cast<size_t>(V) * 2;
  if (smem > 200 * 1024) return -3;
  static bool configured[2] = {false, false};
  if (!configured[bf16 ? 1 : 0]) {
    cudaError_t e = bf16 ? cudaFuncSetAttribute(cross_entropy_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
                         : cudaFuncSetAttribute(cross_entropy_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return -10;
    configured[bf16 ? 1 : 0] = true;
  }
  const int grid = rows < 148 * 2 ? rows : 148 * 2;
  if (bf16)
    cross_entropy_kernel<true><<<grid, 512, smem, stream>>>(static_cast<uint16_t*>(logits), ld, target, loss, lse, rows,
                                                            V, ignore_index, grad_scale, write_grad);
  else
    cross_entropy_kernel<false><<<grid, 512, smem, stream>>>(static_cast<uint16_t*>(logits), ld, target, loss, lse, rows,
                                                             V, ignore_index, grad_scale, write_grad);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// p in [0, 1); cols a multiple of 8; all pointers 16-byte aligned, strides multiples of 8 elements.
extern "C" int msq_dropout_add(const void* y, long long ldy, const void* bias, const void* residual, long long ldr,
                               void* out, long long ldo, long long rows, int cols, float p, unsigned long long seed,
                               int bf16, cudaStream_t stream) {
  using namespace msq;
  if (rows <= 0 || cols <= 0) return 0;
  if ((cols & 7) || (ldy & 7) || (ldr & 7) || (ldo & 7) || p < 0.f || p >= 1.f) return -2;
  const uint32_t thr = static_cast<uint32_t>(p * 65536.f + 0.5f);
  const float inv_keep = 1.f / (1.f - static_cast<float>(thr) / 65536.f);
  long long blocks = (rows * (cols >> 3) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (bf16)
    dropout_add_kernel<true><<<static_cast<int>(blocks), 256, 0, stream>>>(
        static_cast<const uint16_t*>(y), ldy, static_cast<const uint16_t*>(bias), static_cast<const uint16_t*>(residual), ldr,
        static_cast<uint16_t*>(out), ldo, rows, cols, thr, inv_keep, seed);
  else
    dropout_add_kernel<false><<<static_cast<int>(blocks), 256, 0, stream>>>(
        static_cast<const uint16_t*>(y), ldy, static_cast<const uint16_t*>(bias), static_cast<const uint16_t*>(residual), ldr,
        static_cast<uint16_t*>(out), ldo, rows, cols, thr, inv_keep, seed);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// stats_block: this rank's [rows, 3] block of the zero-initialised [world, rows, 3] table.
extern "C" int msq_vp_ce_partial(const void* logits, long long ld, const long long* target, float* stats_block, int rows,
                                 int V, long long vocab_start, int bf16, cudaStream_t stream) {
  using namespace msq;
  if (rows <= 0) return 0;
  if ((V & 7) || (ld & 7) || (reinterpret_cast<uintptr_t>(logits) & 15)) return -2;
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  if (bf16) vp_ce_partial_kernel<true><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(logits), ld, target, stats_block, rows, V, vocab_start);
  else vp_ce_partial_kernel<false><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(logits), ld, target, stats_block, rows, V, vocab_start);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// stats: the all-reduced [world, rows, 3] table.  The logits are overwritten with the gradient.
extern "C" int msq_vp_ce_finish(void* logits, long long ld, const long long* target, const float* stats, int world,
                                float* loss, int rows, int V, long long vocab_start, long long ignore_index,
                                float grad_scale, int bf16, cudaStream_t stream) {
  using namespace msq;
  if (rows <= 0) return 0;
  if ((V & 7) || (ld & 7) || (reinterpret_cast<uintptr_t>(logits) & 15)) return -2;
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  if (bf16) vp_ce_finish_kernel<true><<<grid, 256, 0, stream>>>(static_cast<uint16_t*>(logits), ld, target, stats, world, loss, rows, V, vocab_start, ignore_index, grad_scale);
  else vp_ce_finish_kernel<false><<<grid, 256, 0, stream>>>(static_cast<uint16_t*>(logits), ld, target, stats, world, loss, rows, V, vocab_start, ignore_index, grad_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Folds the row statistics of msq_gemm2_rowstats (rs_max / rs_sum: [tiles_n, rows]) into per-row triples (max,
// sum-exp, target logit).  world <= 1: written to local_stats ([rows, 3] fp32).  world > 1: stored as {value, epoch}
// units into peer_tables[w] (one table of world * rows_cap * 3 units per rank, this rank's included) at this rank's
// block; `epoch` must differ from the one of the previous use of the same tables.
extern "C" int msq_ce_merge_rowstats(const float* rs_max, const float* rs_sum, int tiles_n, int rows, const void* logits,
                                     long long ld, const long long* target, int V, long long vocab_start,
                                     float* local_stats, void* const* peer_tables, int world, int rank, int rows_cap,
                                     unsigned epoch, int bf16, cudaStream_t stream) {
  using namespace msq;
  if (rows <= 0) return 0;
  if (tiles_n <= 0 || world > 16 || (world > 1 && (!peer_tables || rows > rows_cap)) || (world <= 1 && !local_stats)) return -2;
  CePeers peers;
  for (int i = 0; i < 16; ++i)
    peers.table[i] = (world > 1 && i < world) ? static_cast<unsigned long long*>(peer_tables[i]) : nullptr;
  int grid = (rows + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  const uint16_t* lg = static_cast<const uint16_t*>(logits);
  if (bf16) ce_merge_rowstats_kernel<true><<<grid, 256, 0, stream>>>(rs_max, rs_sum, tiles_n, rows, lg, ld, target, V, vocab_start, local_stats, peers, world, rank, rows_cap, epoch);
  else ce_merge_rowstats_kernel<false><<<grid, 256, 0, stream>>>(rs_max, rs_sum, tiles_n, rows, lg, ld, target, V, vocab_start, local_stats, peers, world, rank, rows_cap, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// msq_vp_ce_finish reading the triples from this rank's exchange table (filled by msq_ce_merge_rowstats on every
// rank).  Waits are bounded; a timeout sets *status and leaves the remaining rows untouched.
extern "C" int msq_vp_ce_finish_exchanged(void* logits, long long ld, const long long* target, const void* table,
                                          int world, int rows_cap, unsigned epoch, float* loss, int rows, int V,
                                          long long vocab_start, long long ignore_index, float grad_scale, int bf16,
                                          int* status, cudaStream_t stream) {
  using namespace msq;
  if (rows <= 0) return 0;
  if ((V & 7) || (ld & 7) || (reinterpret_cast<uintptr_t>(logits) & 15) || world < 1 || world > 16 || rows > rows_cap) return -2;
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  const unsigned long long* tb = static_cast<const unsigned long long*>(table);
  if (bf16) vp_ce_finish_exchanged_kernel<true><<<grid, 256, 0, stream>>>(static_cast<uint16_t*>(logits), ld, target, tb, world, rows_cap, epoch, loss, rows, V, vocab_start, ignore_index, grad_scale, status);
  else vp_ce_finish_exchanged_kernel<false><<<grid, 256, 0, stream>>>(static_cast<uint16_t*>(logits), ld, target, tb, world, rows_cap, epoch, loss, rows, V, vocab_start, ignore_index, grad_scale, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// msq_scale_rows relative to a reference: factors are g * inv_ref and rows whose factor is 1 are skipped.
extern "C" int msq_scale_rows_rel(void* x, long long ld, long long rows, int cols, const void* g, int g_fp32, int per_row,
                                  float inv_ref, int bf16, cudaStream_t stream) {
  using namespace msq;
  if (rows <= 0 || cols <= 0) return 0;
  if ((cols & 7) || (ld & 7) || (reinterpret_cast<uintptr_t>(x) & 15)) return -2;
  const int nb = rows < 148 * 16 ? static_cast<int>(rows) : 148 * 16;
  uint16_t* xp = static_cast<uint16_t*>(x);
  if (g_fp32) {
    if (bf16) scale_rows_rel_kernel<true, float><<<nb, 256, 0, stream>>>(xp, ld, rows, cols, static_cast<const float*>(g), per_row, inv_ref);
    else scale_rows_rel_kernel<false, float><<<nb, 256, 0, stream>>>(xp, ld, rows, cols, static_cast<const float*>(g), per_row, inv_ref);
  } else if (bf16) {
    scale_rows_rel_kernel<true, __nv_bfloat16><<<nb, 256, 0, stream>>>(xp, ld, rows, cols, static_cast<const __nv_bfloat16*>(g), per_row, inv_ref);
  } else {
    scale_rows_rel_kernel<false, __half><<<nb, 256, 0, stream>>>(xp, ld, rows, cols, static_cast<const __half*>(g), per_row, inv_ref);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// acc (fp32, [N], zeroed or holding a running sum) += column sums of x[rows, N].
extern "C" int msq_colsum(const void* x, long long ld, int rows, int N, float* acc, int bf16, cudaStream_t stream) {
  using namespace msq;
  if (rows <= 0 || N <= 0) return 0;
  if ((N & 7) || (ld & 7)) return -2;
  const int gx = (N + 255) / 256;
  int gy = (148 * 8 + gx - 1) / gx;
  int rows_per = (rows + gy - 1) / gy;
  rows_per = (rows_per + 7) / 8 * 8;
  gy = (rows + rows_per - 1) / rows_per;
  dim3 grid(gx, gy);
  if (bf16) colsum_kernel<true><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(x), ld, rows, N, acc, rows_per);
  else colsum_kernel<false><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(x), ld, rows, N, acc, rows_per);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// out16[n] (+)= column sums of x[rows, N] in one launch.  `acc` (N floats) and `tickets` ((N + 255) / 256 words) are
// scratch that must be zero before the first call; every call leaves them zero.  Calls that share scratch must not
// overlap on the GPU.
extern "C" int msq_colsum_direct(const void* x, long long ld, int rows, int N, float* acc, unsigned* tickets, void* out16,
                                 int accumulate, int bf16, cudaStream_t stream) {
  using namespace msq;
  if (rows <= 0 || N <= 0) return 0;
  if ((N & 7) || (ld & 7)) return -2;
  const int gx = (N + 255) / 256;
  int gy = (148 * 8 + gx - 1) / gx;
  int rows_per = (rows + gy - 1) / gy;
  rows_per = (rows_per + 7) / 8 * 8;
  gy = (rows + rows_per - 1) / rows_per;
  dim3 grid(gx, gy);
  if (bf16) colsum_direct_kernel<true><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(x), ld, rows, N, acc, tickets, static_cast<uint16_t*>(out16), accumulate, rows_per);
  else colsum_direct_kernel<false><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(x), ld, rows, N, acc, tickets, static_cast<uint16_t*>(out16), accumulate, rows_per);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
