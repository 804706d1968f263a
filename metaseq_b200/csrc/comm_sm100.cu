// Collectives over NVLink peer memory, written as plain kernels over peer pointers.
//
// Every rank owns one symmetric region (same layout on every GPU of the node) that its peers
// have mapped; `PeerPtrs` carries the base address of that region on each rank as seen from the
// calling process.  Data moves with 16-byte peer stores ("push"), so a consumer always reads its
// own HBM; completion is published with a system-scope release store to a flag word in the
// destination's signal pad and observed with acquire loads under a bounded wait.
//
// These kernels replace the NCCL calls of the reference's FSDP and tensor-parallel paths:
//   parameter all-gather      (fairscale FSDP `_rebuild_full_params`, all_gather_base)
//   gradient reduce-scatter   (fairscale FSDP `_post_backward_hook`, reduce_scatter_base)
//   activations all-reduce    (metaseq/modules/megatron/mpu/mappings.py:27 `_reduce`)
// and add what the reference leaves to separate kernels: the reduce-scatter epilogue also
// unscales, accumulates the squared gradient norm and raises the overflow flag.
//
// No kernel here waits on another launch of the same GPU: a wait is always on a flag written by a
// different rank's kernel, and every wait gives up after WAIT_NS_PEER, records a code in the
// status word and lets the kernel finish.
#include "sm100_common.cuh"

#include <cstring>

namespace msq {

constexpr int MAX_PEERS = 16;

struct PeerPtrs {
  void* p[MAX_PEERS];
};

// ------------------------------------------------------------------ barrier
// Flag words [flag_base, flag_base + world) of every rank's signal pad: word `src` is written by rank src.
__global__ void comm_barrier_kernel(PeerPtrs sig, int rank, int world, long long flag_base, uint32_t epoch, int* status) {
  const int t = threadIdx.x;
  if (t < world) {
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(sig.p[t]) + flag_base + rank, epoch);
    wait_flag(static_cast<const uint32_t*>(sig.p[rank]) + flag_base + t, epoch, status);
  }
}

// Waits until flags [lo, hi) of the local signal pad, except [skip_lo, skip_hi), have reached `epoch`.
// The skipped range is for flags that a kernel of this same GPU publishes: those are ordered with
// stream events instead, so that no launch ever waits on another launch of its own device.
__global__ void comm_wait_flags_kernel(const uint32_t* flags, long long lo, long long hi, long long skip_lo,
                                       long long skip_hi, uint32_t epoch, int* status) {
  for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    if (i >= skip_lo && i < skip_hi) continue;
    if (!wait_flag(flags + i, epoch, status)) break;
  }
}

struct FlagList {
  int idx[32];
  int n;
};
// Waits for an explicit list of flag words (the chunks that hold a unit's small parameters, while the
// GEMMs poll the chunks of their own weight tiles).
__global__ void comm_wait_flag_list_kernel(const uint32_t* flags, FlagList list, uint32_t epoch, int* status) {
  if (threadIdx.x < list.n) wait_flag(flags + list.idx[threadIdx.x], epoch, status);
}

// ------------------------------------------------------------- all-gather
// Rank `rank` owns bytes [rank * shard_bytes, (rank + 1) * shard_bytes) of the gathered buffer, cut
// into chunks of `chunk_bytes`.  A CTA reads one chunk of the local shard once and stores it into the
// gathered buffer of every rank (its own included), then publishes flag `flag_base + global chunk
// index` on each destination.  Consumers (the GEMM producer warp, or comm_wait_flags_kernel) poll
// those flags, so a weight tile can be multiplied as soon as its chunks have landed.
__global__ void __launch_bounds__(512)
comm_allgather_push_kernel(PeerPtrs dst, long long dst_off_bytes, const uint4* __restrict__ src, long long shard_bytes,
                           int chunk_bytes, int rank, int world, PeerPtrs sig, long long flag_base, uint32_t epoch,
                           int* status) {
  if (status && *reinterpret_cast<volatile int*>(status) != 0) return;
  const long long chunks = (shard_bytes + chunk_bytes - 1) / chunk_bytes;
  for (long long c = blockIdx.x; c < chunks; c += gridDim.x) {
    const long long b0 = c * chunk_bytes;
    const long long nb = (shard_bytes - b0 < chunk_bytes) ? (shard_bytes - b0) : chunk_bytes;
    const int nvec = static_cast<int>(nb >> 4);
    const uint4* s = src + (b0 >> 4);
    // four independent 16-byte loads per thread keep enough bytes in flight to fill the links
    for (int i0 = threadIdx.x; i0 < nvec; i0 += 4 * blockDim.x) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < nvec) v[u] = s[i];
      }
      for (int pp = 0; pp < world; ++pp) {
        const int peer = (rank + pp) % world;  // spread the first stores over different links
        uint4* d = reinterpret_cast<uint4*>(static_cast<uint8_t*>(dst.p[peer]) + dst_off_bytes + rank * shard_bytes + b0);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + u * blockDim.x;
          if (i < nvec) d[i] = v[u];
        }
      }
    }
    __syncthreads();
    if (threadIdx.x < world) {
      __threadfence_system();
      st_release_sys(static_cast<uint32_t*>(sig.p[threadIdx.x]) + flag_base + rank * chunks + c, epoch);
    }
    __syncthreads();
  }
}

// Publishes `count` consecutive flags starting at flag_base + first on every rank.  Used after copy-engine
// transfers (stream order guarantees they have completed) so that the data path needs no SM at all.
__global__ void comm_signal_kernel(PeerPtrs sig, int world, long long flag_base, long long first, long long count,
                                   uint32_t epoch) {
  __threadfence_system();
  for (long long i = threadIdx.x; i < count * world; i += blockDim.x) {
    const int peer = static_cast<int>(i / count);
    st_release_sys(static_cast<uint32_t*>(sig.p[peer]) + flag_base + first + (i - peer * count), epoch);
  }
}

// --------------------------------------------------------- reduce-scatter
// Push phase: slice p of the local full-size buffer goes to slot `rank` of rank p's slot area
// (slot area = world slots of shard_bytes each), then flag `flag_base + rank` is published on rank p.
__global__ void __launch_bounds__(512)
comm_reduce_scatter_push_kernel(PeerPtrs slots, long long slots_off_bytes, const uint4* __restrict__ full,
                                long long shard_bytes, int rank, int world, PeerPtrs sig, long long flag_base,
                                uint32_t epoch, unsigned int* done_counter, int* status) {
  if (status && *reinterpret_cast<volatile int*>(status) != 0) return;
  const long long vec_per_shard = shard_bytes >> 4;
  const long long total = vec_per_shard * world;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total; i0 += 4 * stride) {
    uint4 v[4];
    uint4* d[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * stride;
      if (i < total) {
        const int pp = static_cast<int>(i / vec_per_shard);
        const long long off = i - pp * vec_per_shard;
        const int peer = (rank + pp) % world;
        d[u] = reinterpret_cast<uint4*>(static_cast<uint8_t*>(slots.p[peer]) + slots_off_bytes + rank * shard_bytes) + off;
        v[u] = full[peer * vec_per_shard + off];
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i0 + u * stride < total) *d[u] = v[u];
  }
  // the last CTA to finish publishes the flags (every CTA's stores are fenced before it counts itself)
  __threadfence_system();
  __syncthreads();
  __shared__ bool last;
  if (threadIdx.x == 0) last = (atomicAdd(done_counter, 1u) == gridDim.x - 1);
  __syncthreads();
  if (last) {
    if (threadIdx.x < world) {
      __threadfence_system();
      st_release_sys(static_cast<uint32_t*>(sig.p[threadIdx.x]) + flag_base + rank, epoch);
    }
    if (threadIdx.x == 0) *done_counter = 0;
  }
}

// Reduce phase (local reads only): waits for the `world` source flags, sums the slots in fp32, applies
// `scale`, writes the 16-bit (or fp32) shard and accumulates sum(g^2) of the scaled result into
// sumsq_acc; a non-finite value sets *overflow.
template <bool BF16, bool OUT32>
__global__ void __launch_bounds__(256)
comm_reduce_slots_kernel(const uint4* __restrict__ slots, long long shard_numel, int world, float scale,
                         void* __restrict__ out, float* sumsq_acc, int* overflow, const uint32_t* flags,
                         long long flag_base, uint32_t epoch, int* status) {
  __shared__ bool ok_s;
  if (threadIdx.x == 0) ok_s = true;
  __syncthreads();
  if (threadIdx.x < world) {
    if (!wait_flag(flags + flag_base + threadIdx.x, epoch, status)) ok_s = false;
  }
  __syncthreads();
  if (!ok_s) return;
  const long long nvec = shard_numel >> 3;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  float ss = 0.f;
  bool bad = false;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < world; ++s) {
      const uint4 v = slots[s * nvec + i];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack2<BF16>(w[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      acc[j] *= scale;
      ss += acc[j] * acc[j];
      bad |= !isfinite(acc[j]);
    }
    if (OUT32) {
      float4* o = reinterpret_cast<float4*>(out) + 2 * i;
      o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    } else {
      uint4 o;
      o.x = pack2<BF16>(acc[0], acc[1]);
      o.y = pack2<BF16>(acc[2], acc[3]);
      o.z = pack2<BF16>(acc[4], acc[5]);
      o.w = pack2<BF16>(acc[6], acc[7]);
      reinterpret_cast<uint4*>(out)[i] = o;
    }
  }
  __shared__ float red[32];
  ss = block_sum(ss, red);
  if (threadIdx.x == 0 && sumsq_acc) atomicAdd(sumsq_acc, ss);
  if (bad && overflow) *overflow = 1;
}

// Owner-side ("pull") reduce-scatter, fused with the unscale / norm / overflow epilogue.  Every rank's full-size
// gradient buffer lives at the same offset of its symmetric region.  A rank publishes flag `flag_base + rank` on
// every peer when its buffer is complete (msq_comm_signal); the owner of a shard waits for all `world` flags and
// then reads its slice of all ranks at once:
//   MC   : one multimem.ld_reduce per 16 bytes on the multicast address: the additions happen inside NVSwitch
//          (fp32 accumulation for 16-bit inputs) and only the sum crosses the owner's link (ingress 1 x shard);
//   !MC  : plain 16-byte loads from each peer's mapping, summed in fp32 registers (ingress (world - 1) x shard).
// No landing slots and no second pass: the value is scaled, squared into the norm accumulator, checked for
// non-finite values and written as the 16-bit or fp32 shard straight from registers.
template <bool BF16, bool OUT32, bool MC>
__global__ void __launch_bounds__(256)
comm_reduce_scatter_pull_kernel(const void* mc_shard, PeerPtrs src, long long src_off_bytes, long long shard_numel,
                                int rank, int world, float scale, void* __restrict__ out, float* sumsq_acc,
                                int* overflow, const uint32_t* flags, long long flag_base, uint32_t epoch, int* status) {
  __shared__ bool ok_s;
  if (threadIdx.x == 0) ok_s = !(status && *reinterpret_cast<volatile int*>(status) != 0);
  __syncthreads();
  if (threadIdx.x < world && ok_s) {
    if (!wait_flag(flags + flag_base + threadIdx.x, epoch, status)) ok_s = false;
  }
  __syncthreads();
  if (!ok_s) return;
  const long long nvec = shard_numel >> 3;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  float ss = 0.f;
  bool bad = false;
  // Four independent 16-byte requests per thread are in flight before the first result is used: a request that
  // crosses the switch takes microseconds, so the link is filled by the number of requests outstanding.
  constexpr int U = 4;
  for (long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < nvec; i0 += U * stride) {
    uint32_t w[U][4];
    float acc[U][8];
    if (MC) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < nvec) {
          const uint8_t* a = static_cast<const uint8_t*>(mc_shard) + (i << 4);
          if (BF16)
            asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                         : "=r"(w[u][0]), "=r"(w[u][1]), "=r"(w[u][2]), "=r"(w[u][3]) : "l"(a) : "memory");
          else
            asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                         : "=r"(w[u][0]), "=r"(w[u][1]), "=r"(w[u][2]), "=r"(w[u][3]) : "l"(a) : "memory");
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack2<BF16>(w[u][j]);
          acc[u][2 * j] = f.x;
          acc[u][2 * j + 1] = f.y;
        }
      }
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
      for (int s = 0; s < world; ++s) {
        const int peer = (rank + s) % world;  // own slice first, then round the ring
        const uint4* base = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(src.p[peer]) + src_off_bytes);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * stride;
          if (i < nvec)
            asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(w[u][0]), "=r"(w[u][1]), "=r"(w[u][2]), "=r"(w[u][3]) : "l"(base + i) : "memory");
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (i0 + u * stride < nvec) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = unpack2<BF16>(w[u][j]);
              acc[u][2 * j] += f.x;
              acc[u][2 * j + 1] += f.y;
            }
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= nvec) continue;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc[u][j] *= scale;
        ss += acc[u][j] * acc[u][j];
        bad |= !isfinite(acc[u][j]);
      }
      if (OUT32) {
        float4* o = reinterpret_cast<float4*>(out) + 2 * i;
        o[0] = make_float4(acc[u][0], acc[u][1], acc[u][2], acc[u][3]);
        o[1] = make_float4(acc[u][4], acc[u][5], acc[u][6], acc[u][7]);
      } else {
        uint4 o;
        o.x = pack2<BF16>(acc[u][0], acc[u][1]);
        o.y = pack2<BF16>(acc[u][2], acc[u][3]);
        o.z = pack2<BF16>(acc[u][4], acc[u][5]);
        o.w = pack2<BF16>(acc[u][6], acc[u][7]);
        reinterpret_cast<uint4*>(out)[i] = o;
      }
    }
  }
  __shared__ float red[32];
  ss = block_sum(ss, red);
  if (threadIdx.x == 0 && sumsq_acc) atomicAdd(sumsq_acc, ss);
  if (bad && overflow) *overflow = 1;
}

// All-gather through the switch: a CTA reads one chunk of the local shard and writes it with multimem.st to the
// multicast address of the gathered buffer, which NVSwitch delivers to every rank (this one included): the shard
// leaves the GPU once instead of once per peer.  The per-chunk arrival flags are then published on every rank as
// in comm_allgather_push_kernel, so the GEMM that consumes the gathered weights polls them the same way.
__global__ void __launch_bounds__(512)
comm_allgather_multimem_kernel(void* mc_dst, const uint4* __restrict__ src, long long shard_bytes, int chunk_bytes,
                               int rank, int world, PeerPtrs sig, long long flag_base, uint32_t epoch, int* status) {
  if (status && *reinterpret_cast<volatile int*>(status) != 0) return;
  const long long chunks = (shard_bytes + chunk_bytes - 1) / chunk_bytes;
  for (long long c = blockIdx.x; c < chunks; c += gridDim.x) {
    const long long b0 = c * chunk_bytes;
    const long long nb = (shard_bytes - b0 < chunk_bytes) ? (shard_bytes - b0) : chunk_bytes;
    const int nvec = static_cast<int>(nb >> 4);
    const uint4* s = src + (b0 >> 4);
    uint8_t* d = static_cast<uint8_t*>(mc_dst) + static_cast<long long>(rank) * shard_bytes + b0;
    for (int i0 = threadIdx.x; i0 < nvec; i0 += 4 * blockDim.x) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < nvec) v[u] = s[i];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < nvec)
          asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                       ::"l"(d + (static_cast<long long>(i) << 4)), "r"(v[u].x), "r"(v[u].y), "r"(v[u].z), "r"(v[u].w)
                       : "memory");
      }
    }
    __syncthreads();
    if (threadIdx.x < world) {
      __threadfence_system();
      st_release_sys(static_cast<uint32_t*>(sig.p[threadIdx.x]) + flag_base + rank * chunks + c, epoch);
    }
    __syncthreads();
  }
}

// Row-block reduction behind a scattering GEMM: this rank owns `rows` rows of an [*, N] matrix; slot s holds
// the partial product computed by rank s.  out_row = sum_s slot_s + bias + residual, written to `out_local`
// (reduce-scatter) and, when bcast.p[0] is set, also stored into every rank's copy of the full matrix at
// row row0 + r (all-reduce = reduce-scatter + all-gather), after which flag `bcast_flag_base + rank` is
// published on every rank by the last CTA.
template <bool BF16>
__global__ void __launch_bounds__(256)
comm_reduce_rows_kernel(const uint4* __restrict__ slots, long long slot_stride_vec, int world, int rows, int N,
                        const uint16_t* __restrict__ bias, const uint16_t* __restrict__ residual, long long ldr,
                        uint16_t* __restrict__ out_local, long long ldo, PeerPtrs bcast, long long bcast_off_bytes,
                        long long ld_bcast, int row0, int rank, const uint32_t* flags, long long flag_base, uint32_t epoch,
                        PeerPtrs sig, long long bcast_flag_base, unsigned int* done_counter, int* status) {
  __shared__ bool ok_s, last_s;
  if (threadIdx.x == 0) ok_s = true;
  __syncthreads();
  if (threadIdx.x < world) {
    if (!wait_flag(flags + flag_base + threadIdx.x, epoch, status)) ok_s = false;
  }
  __syncthreads();
  if (!ok_s) return;
  const int vec_per_row = N >> 3;
  const long long total = static_cast<long long>(rows) * vec_per_row;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const bool do_bcast = bcast.p[0] != nullptr;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int r = static_cast<int>(i / vec_per_row);
    const int c = static_cast<int>(i - static_cast<long long>(r) * vec_per_row) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    auto add16 = [&](const uint4& v) {
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack2<BF16>(w[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    };
    for (int s = 0; s < world; ++s) add16(slots[s * slot_stride_vec + i]);
    if (bias) add16(*reinterpret_cast<const uint4*>(bias + c));
    if (residual) add16(*reinterpret_cast<const uint4*>(residual + static_cast<long long>(r) * ldr + c));
    uint4 o;
    o.x = pack2<BF16>(acc[0], acc[1]);
    o.y = pack2<BF16>(acc[2], acc[3]);
    o.z = pack2<BF16>(acc[4], acc[5]);
    o.w = pack2<BF16>(acc[6], acc[7]);
    if (out_local) *reinterpret_cast<uint4*>(out_local + static_cast<long long>(r) * ldo + c) = o;
    if (do_bcast) {
      for (int pp = 0; pp < world; ++pp) {
        const int peer = (rank + pp) % world;
        uint16_t* d = reinterpret_cast<uint16_t*>(static_cast<uint8_t*>(bcast.p[peer]) + bcast_off_bytes);
        *reinterpret_cast<uint4*>(d + static_cast<long long>(row0 + r) * ld_bcast + c) = o;
      }
    }
  }
  if (!do_bcast) return;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) last_s = (atomicAdd(done_counter, 1u) == gridDim.x - 1);
  __syncthreads();
  if (last_s) {
    if (threadIdx.x < world) {
      __threadfence_system();
      st_release_sys(static_cast<uint32_t*>(sig.p[threadIdx.x]) + bcast_flag_base + rank, epoch);
    }
    if (threadIdx.x == 0) *done_counter = 0;
  }
}

// ------------------------------------------------------- one-shot all-reduce
// For small tensors (decode activations, vocab-parallel loss statistics): every rank stores its
// input into slot `rank` of every peer's slot area, publishes a flag, waits for the other ranks'
// flags and sums the slots locally.  Slot areas alternate with the epoch's parity, so a fast rank
// starting the next all-reduce never overwrites data a slow rank is still reading.
template <int MODE>  // 0: 16-bit fp16, 1: bf16, 2: fp32
__global__ void __launch_bounds__(512)
comm_allreduce_oneshot_kernel(PeerPtrs slots, long long slots_off_bytes, long long slot_stride, const void* in, void* out,
                              long long bytes, int rank, int world, PeerPtrs sig, long long flag_base, uint32_t epoch,
                              int* status) {
  if (status && *reinterpret_cast<volatile int*>(status) != 0) return;
  const long long parity_off = (epoch & 1u) ? slot_stride * world : 0;
  const long long nvec = bytes >> 4;
  const uint4* src = static_cast<const uint4*>(in);
  for (long long i = threadIdx.x; i < nvec; i += blockDim.x) {
    const uint4 v = src[i];
    for (int pp = 0; pp < world; ++pp) {
      const int peer = (rank + pp) % world;
      uint4* d = reinterpret_cast<uint4*>(static_cast<uint8_t*>(slots.p[peer]) + slots_off_bytes + parity_off + rank * slot_stride);
      d[i] = v;
    }
  }
  __syncthreads();
  __shared__ bool ok_s;
  if (threadIdx.x == 0) ok_s = true;
  __syncthreads();
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(sig.p[threadIdx.x]) + flag_base + rank, epoch);
    if (!wait_flag(static_cast<const uint32_t*>(sig.p[rank]) + flag_base + threadIdx.x, epoch, status)) ok_s = false;
  }
  __syncthreads();
  if (!ok_s) return;
  const uint8_t* mine = static_cast<const uint8_t*>(slots.p[rank]) + slots_off_bytes + parity_off;
  for (long long i = threadIdx.x; i < nvec; i += blockDim.x) {
    if (MODE == 2) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < world; ++s) {
        const float4 v = reinterpret_cast<const float4*>(mine + s * slot_stride)[i];
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      static_cast<float4*>(out)[i] = acc;
    } else {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < world; ++s) {
        const uint4 v = reinterpret_cast<const uint4*>(mine + s * slot_stride)[i];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack2<MODE == 1>(w[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      uint4 o;
      o.x = pack2<MODE == 1>(acc[0], acc[1]);
      o.y = pack2<MODE == 1>(acc[2], acc[3]);
      o.z = pack2<MODE == 1>(acc[4], acc[5]);
      o.w = pack2<MODE == 1>(acc[6], acc[7]);
      static_cast<uint4*>(out)[i] = o;
    }
  }
}

// Multi-CTA form of the one-shot all-reduce: CTA c owns slice c of the tensor and shakes hands only with the
// CTAs of the same index on the other ranks (flag words flag_base + c * world + src), so no grid-wide or
// cross-CTA synchronisation is needed and large tensors use many SMs.
template <int MODE>
__global__ void __launch_bounds__(512)
comm_allreduce_sliced_kernel(PeerPtrs slots, long long slots_off_bytes, long long slot_stride, const void* in, void* out,
                             long long bytes, long long slice_bytes, int rank, int world, PeerPtrs sig, long long flag_base,
                             uint32_t epoch, int* status) {
  if (status && *reinterpret_cast<volatile int*>(status) != 0) return;
  const long long parity_off = (epoch & 1u) ? slot_stride * world : 0;
  const long long b0 = static_cast<long long>(blockIdx.x) * slice_bytes;
  const long long nb = (bytes - b0 < slice_bytes) ? (bytes - b0) : slice_bytes;
  if (nb <= 0) return;
  const long long v0 = b0 >> 4, nvec = nb >> 4;
  const uint4* src = static_cast<const uint4*>(in) + v0;
  for (long long i = threadIdx.x; i < nvec; i += blockDim.x) {
    const uint4 v = src[i];
    for (int pp = 0; pp < world; ++pp) {
      const int peer = (rank + pp) % world;
      uint4* d = reinterpret_cast<uint4*>(static_cast<uint8_t*>(slots.p[peer]) + slots_off_bytes + parity_off + rank * slot_stride) + v0;
      d[i] = v;
    }
  }
  __syncthreads();
  __shared__ bool ok_s;
  if (threadIdx.x == 0) ok_s = true;
  __syncthreads();
  const long long my_flags = flag_base + static_cast<long long>(blockIdx.x) * world;
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(sig.p[threadIdx.x]) + my_flags + rank, epoch);
    if (!wait_flag(static_cast<const uint32_t*>(sig.p[rank]) + my_flags + threadIdx.x, epoch, status)) ok_s = false;
  }
  __syncthreads();
  if (!ok_s) return;
  const uint8_t* mine = static_cast<const uint8_t*>(slots.p[rank]) + slots_off_bytes + parity_off;
  for (long long i = threadIdx.x; i < nvec; i += blockDim.x) {
    if (MODE == 2) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < world; ++s) {
        const float4 v = reinterpret_cast<const float4*>(mine + s * slot_stride)[v0 + i];
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      static_cast<float4*>(out)[v0 + i] = acc;
    } else {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < world; ++s) {
        const uint4 v = reinterpret_cast<const uint4*>(mine + s * slot_stride)[v0 + i];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack2<MODE == 1>(w[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      uint4 o;
      o.x = pack2<MODE == 1>(acc[0], acc[1]);
      o.y = pack2<MODE == 1>(acc[2], acc[3]);
      o.z = pack2<MODE == 1>(acc[4], acc[5]);
      o.w = pack2<MODE == 1>(acc[6], acc[7]);
      static_cast<uint4*>(out)[v0 + i] = o;
    }
  }
}

// One-launch in-switch all-reduce.  CTA c stages slice c of the input in this rank's symmetric buffer, shakes
// hands with the same-index CTAs of the other ranks, reduces its 1/world share of the slice inside NVSwitch
// (multimem.ld_reduce on the multicast address) and broadcasts it (multimem.st), shakes hands again and copies
// the finished slice to the output.
template <int MODE>
__global__ void __launch_bounds__(512)
comm_allreduce_multimem_fused_kernel(void* mc, void* stage_local, const void* in, void* out, long long bytes,
                                     long long slice_bytes, int rank, int world, PeerPtrs sig, long long flag_base,
                                     uint32_t epoch, int* status) {
  if (status && *reinterpret_cast<volatile int*>(status) != 0) return;
  const long long b0 = static_cast<long long>(blockIdx.x) * slice_bytes;
  const long long nb = (bytes - b0 < slice_bytes) ? (bytes - b0) : slice_bytes;
  if (nb <= 0) return;
  const long long v0 = b0 >> 4, nvec = nb >> 4;
  const uint4* src = static_cast<const uint4*>(in) + v0;
  uint4* stg = static_cast<uint4*>(stage_local) + v0;
  for (long long i = threadIdx.x; i < nvec; i += blockDim.x) stg[i] = src[i];
  __shared__ bool ok_s;
  if (threadIdx.x == 0) ok_s = true;
  __syncthreads();
  const long long f1 = flag_base + static_cast<long long>(blockIdx.x) * 2 * world;
  const long long f2 = f1 + world;
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(sig.p[threadIdx.x]) + f1 + rank, epoch);
    if (!wait_flag(static_cast<const uint32_t*>(sig.p[rank]) + f1 + threadIdx.x, epoch, status)) ok_s = false;
  }
  __syncthreads();
  if (!ok_s) return;
  const long long per = (nvec + world - 1) / world;
  const long long lo = rank * per, hi = (lo + per < nvec) ? lo + per : nvec;
  for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    uint8_t* a = static_cast<uint8_t*>(mc) + ((v0 + i) << 4);
    uint32_t x, y, z, w;
    if (MODE == 2)
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(x), "=r"(y), "=r"(z), "=r"(w) : "l"(a) : "memory");
    else if (MODE == 1)
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                   : "=r"(x), "=r"(y), "=r"(z), "=r"(w) : "l"(a) : "memory");
    else
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                   : "=r"(x), "=r"(y), "=r"(z), "=r"(w) : "l"(a) : "memory");
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
  }
  __syncthreads();
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(sig.p[threadIdx.x]) + f2 + rank, epoch);
    if (!wait_flag(static_cast<const uint32_t*>(sig.p[rank]) + f2 + threadIdx.x, epoch, status)) ok_s = false;
  }
  __syncthreads();
  if (!ok_s) return;
  uint4* dst = static_cast<uint4*>(out) + v0;
  for (long long i = threadIdx.x; i < nvec; i += blockDim.x) dst[i] = stg[i];
}

// In-switch variant: `mc` is the multicast address of the input buffers (same offset on every rank).
// After a barrier each rank asks the switch for the sum of its share of the elements
// (multimem.ld_reduce) and broadcasts the result to all ranks (multimem.st), i.e. a two-shot
// all-reduce whose additions happen inside NVSwitch.  fp32 accumulation for 16-bit inputs.
template <int MODE>
__global__ void __launch_bounds__(512)
comm_allreduce_multimem_kernel(void* mc, long long bytes, int rank, int world, PeerPtrs sig, long long flag_base,
                               uint32_t epoch, int* status) {
  if (status && *reinterpret_cast<volatile int*>(status) != 0) return;
  __shared__ bool ok_s;
  if (threadIdx.x == 0) ok_s = true;
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(sig.p[threadIdx.x]) + flag_base + rank, epoch);
  }
  if (threadIdx.x < world) {
    if (!wait_flag(static_cast<const uint32_t*>(sig.p[rank]) + flag_base + threadIdx.x, epoch, status)) ok_s = false;
  }
  __syncthreads();
  if (!ok_s) return;
  const long long nvec = bytes >> 4;
  const long long per = (nvec + world - 1) / world;
  const long long lo = rank * per, hi = (lo + per < nvec) ? lo + per : nvec;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = lo + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < hi; i += stride) {
    uint8_t* a = static_cast<uint8_t*>(mc) + (i << 4);
    uint32_t x, y, z, w;
    if (MODE == 2)
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(x), "=r"(y), "=r"(z), "=r"(w) : "l"(a) : "memory");
    else if (MODE == 1)
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                   : "=r"(x), "=r"(y), "=r"(z), "=r"(w) : "l"(a) : "memory");
    else
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                   : "=r"(x), "=r"(y), "=r"(z), "=r"(w) : "l"(a) : "memory");
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
  }
}

// ------------------------------------------- small exchange that a CUDA graph can replay
// Every rank contributes `words` 32-bit words (two 16-bit values each in the summing modes); every rank ends up with
// the sum over ranks (MODE 0: fp16 pairs, 1: bf16 pairs, fp32 accumulation) or with all ranks' words side by side
// (MODE 2: out[src * words + i]).  A word travels as the 8-byte unit {word, epoch}: a thread stores its unit into
// the receive buffer of every rank at [rank * cap + i] and then polls its own buffer until the unit of every source
// at index i carries the epoch, so there is no flag, fence or remote load, and the reader of a word is the same
// thread index on every rank.  The epoch is a counter in device memory that the kernel itself advances (the last CTA
// to finish stores the new value), which is what allows a captured launch to be replayed; receive buffers
// alternate with its parity so that a rank that is one call ahead does not overwrite units still being read.
template <int MODE>
__global__ void __launch_bounds__(256)
comm_words_exchange_kernel(const uint32_t* __restrict__ in, long long words, PeerPtrs recv0, PeerPtrs recv1,
                           long long cap, int rank, int world, uint32_t* epoch_dev, unsigned* ticket,
                           uint32_t* __restrict__ out, int* status) {
  if (status && *reinterpret_cast<volatile int*>(status) != 0) return;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(epoch_dev) + 1u;
  const PeerPtrs& recv = (epoch & 1u) ? recv1 : recv0;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  bool ok = true;
  const long long first = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  // all of this thread's units leave before it starts to wait for anybody else's
  for (long long i = first; i < words; i += stride) {
    const unsigned long long unit = (static_cast<unsigned long long>(epoch) << 32) | in[i];
    for (int w = 0; w < world; ++w) {
      unsigned long long* dst = static_cast<unsigned long long*>(recv.p[(rank + w) % world]) + rank * cap + i;
      asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(unit) : "memory");
    }
  }
  for (long long i = first; i < words && ok; i += stride) {
    float sx = 0.f, sy = 0.f;
    const unsigned long long* mine = static_cast<const unsigned long long*>(recv.p[rank]) + i;
    for (int s = 0; s < world && ok; ++s) {
      const unsigned long long* src = mine + s * cap;
      unsigned long long got;
      const unsigned long long t0 = globaltimer_ns();
      uint32_t spins = 0;
      while (true) {
        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(got) : "l"(src) : "memory");
        if (static_cast<uint32_t>(got >> 32) == epoch) break;
        if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > WAIT_NS_PEER) {
          if (status) atomicCAS(status, 0, ST_TIMEOUT_PEER_FLAG);
          ok = false;
          break;
        }
      }
      if (!ok) break;
      const uint32_t word = static_cast<uint32_t>(got);
      if (MODE == 2) {
        out[s * words + i] = word;
      } else {
        const float2 f = unpack2<MODE == 1>(word);
        sx += f.x;
        sy += f.y;
      }
    }
    if (MODE != 2 && ok) out[i] = pack2<MODE == 1>(sx, sy);
  }
  // advance the epoch once every CTA of this launch has read it (all of them are done when the last one is)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
      *epoch_dev = epoch;
      *ticket = 0;
    }
  }
}

}  // namespace msq

using msq::PeerPtrs;

static PeerPtrs make_ptrs(void* const* ptrs, int world) {
  PeerPtrs r;
  for (int i = 0; i < msq::MAX_PEERS; ++i) r.p[i] = i < world ? ptrs[i] : nullptr;
  return r;
}

// ---------------------------------------------------------------- IPC heap
// Symmetric regions for processes that cannot share a CUDA virtual-memory handle: plain cudaMalloc
// plus cudaIpc handles exchanged by the caller.
extern "C" int msq_symm_alloc(long long bytes, void** ptr, void* handle64) {
  if (cudaMalloc(ptr, static_cast<size_t>(bytes)) != cudaSuccess) return -1;
  if (cudaMemset(*ptr, 0, static_cast<size_t>(bytes)) != cudaSuccess) return -2;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, *ptr) != cudaSuccess) return -3;
  static_assert(sizeof(h) == 64, "ipc handle size");
  memcpy(handle64, &h, 64);
  return 0;
}
extern "C" int msq_symm_open(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? 0 : -1;
}
extern "C" int msq_symm_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : -1; }
extern "C" int msq_symm_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : -1; }

// ------------------------------------------------------------ entry points
extern "C" int msq_comm_barrier(void* const* sig_ptrs, int rank, int world, long long flag_base, unsigned epoch,
                                int* status, cudaStream_t stream) {
  if (world > msq::MAX_PEERS) return -2;
  msq::comm_barrier_kernel<<<1, 32, 0, stream>>>(make_ptrs(sig_ptrs, world), rank, world, flag_base, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int msq_comm_wait_flags(const void* flags, long long lo, long long hi, long long skip_lo, long long skip_hi,
                                   unsigned epoch, int* status, cudaStream_t stream) {
  if (hi <= lo) return 0;
  msq::comm_wait_flags_kernel<<<1, 128, 0, stream>>>(static_cast<const uint32_t*>(flags), lo, hi, skip_lo, skip_hi, epoch,
                                                     status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int msq_comm_wait_flag_list(const void* flags, const int* idx, int n, unsigned epoch, int* status,
                                       cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n > 32) return -2;
  msq::FlagList l;
  for (int i = 0; i < 32; ++i) l.idx[i] = i < n ? idx[i] : 0;
  l.n = n;
  msq::comm_wait_flag_list_kernel<<<1, 32, 0, stream>>>(static_cast<const uint32_t*>(flags), l, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Publishes one flag (flag_base + rank) on every rank; stream order makes everything launched before it on
// this stream (for instance the peer stores of a scattering GEMM) visible first.
extern "C" int msq_comm_signal(void* const* sig_ptrs, int rank, int world, long long flag_base, unsigned epoch,
                               cudaStream_t stream) {
  if (world > msq::MAX_PEERS) return -2;
  msq::comm_signal_kernel<<<1, 128, 0, stream>>>(make_ptrs(sig_ptrs, world), world, flag_base, rank, 1, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int msq_comm_reduce_rows(const void* slots, long long slot_stride_bytes, int world, int rows, int N,
                                    const void* bias, const void* residual, long long ldr, void* out_local, long long ldo,
                                    void* const* bcast_ptrs, long long bcast_off_bytes, long long ld_bcast, int row0,
                                    int rank, int bf16, const void* flags, long long flag_base, unsigned epoch,
                                    void* const* sig_ptrs, long long bcast_flag_base, unsigned* done_counter, int max_ctas,
                                    int* status, cudaStream_t stream) {
  if (world > msq::MAX_PEERS) return -2;
  if ((N & 7) || (slot_stride_bytes & 15) || (ldr & 7) || (ldo & 7) || (ld_bcast & 7)) return -2;
  if (rows <= 0) return 0;
  long long want = (static_cast<long long>(rows) * (N >> 3) + 255) / 256;
  int grid = static_cast<int>(want < max_ctas ? want : max_ctas);
  if (grid < 1) grid = 1;
  PeerPtrs bc;
  for (int i = 0; i < msq::MAX_PEERS; ++i) bc.p[i] = (bcast_ptrs && i < world) ? bcast_ptrs[i] : nullptr;
  PeerPtrs sg = make_ptrs(sig_ptrs, world);
  if (bf16)
    msq::comm_reduce_rows_kernel<true><<<grid, 256, 0, stream>>>(
        static_cast<const uint4*>(slots), slot_stride_bytes >> 4, world, rows, N, static_cast<const uint16_t*>(bias),
        static_cast<const uint16_t*>(residual), ldr, static_cast<uint16_t*>(out_local), ldo, bc, bcast_off_bytes, ld_bcast,
        row0, rank, static_cast<const uint32_t*>(flags), flag_base, epoch, sg, bcast_flag_base, done_counter, status);
  else
    msq::comm_reduce_rows_kernel<false><<<grid, 256, 0, stream>>>(
        static_cast<const uint4*>(slots), slot_stride_bytes >> 4, world, rows, N, static_cast<const uint16_t*>(bias),
        static_cast<const uint16_t*>(residual), ldr, static_cast<uint16_t*>(out_local), ldo, bc, bcast_off_bytes, ld_bcast,
        row0, rank, static_cast<const uint32_t*>(flags), flag_base, epoch, sg, bcast_flag_base, done_counter, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int msq_comm_allgather_push(void* const* dst_ptrs, long long dst_off_bytes, const void* src, long long shard_bytes,
                                       int chunk_bytes, int rank, int world, void* const* sig_ptrs, long long flag_base,
                                       unsigned epoch, int max_ctas, int* status, cudaStream_t stream) {
  if (world > msq::MAX_PEERS) return -2;
  if ((shard_bytes & 15) || (chunk_bytes & 15) || (dst_off_bytes & 15) || (reinterpret_cast<uintptr_t>(src) & 15)) return -2;
  if (shard_bytes <= 0) return 0;
  long long chunks = (shard_bytes + chunk_bytes - 1) / chunk_bytes;
  int grid = static_cast<int>(chunks < max_ctas ? chunks : max_ctas);
  if (grid < 1) grid = 1;
  msq::comm_allgather_push_kernel<<<grid, 512, 0, stream>>>(make_ptrs(dst_ptrs, world), dst_off_bytes,
                                                           static_cast<const uint4*>(src), shard_bytes, chunk_bytes, rank,
                                                           world, make_ptrs(sig_ptrs, world), flag_base, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Copy-engine variants: the shard (or gradient slice) travels by peer-to-peer DMA, one asynchronous copy
// per destination, and a one-CTA kernel publishes the arrival flags afterwards.  No SM is taken from the
// GEMMs that run concurrently on the compute stream.
extern "C" int msq_comm_allgather_ce(void* const* dst_ptrs, long long dst_off_bytes, const void* src, long long shard_bytes,
                                     int chunk_bytes, int rank, int world, void* const* sig_ptrs, long long flag_base,
                                     unsigned epoch, cudaStream_t stream, cudaStream_t local_stream) {
  // The copy into this rank's own gathered buffer goes to `local_stream` (normally the consumer's stream), so
  // its completion is ordered by the stream itself and consumers only poll the flags of other ranks.
  if (world > msq::MAX_PEERS) return -2;
  if (shard_bytes <= 0) return 0;
  for (int pp = 0; pp < world; ++pp) {
    const int peer = (rank + pp) % world;
    void* d = static_cast<uint8_t*>(dst_ptrs[peer]) + dst_off_bytes + static_cast<long long>(rank) * shard_bytes;
    if (cudaMemcpyAsync(d, src, static_cast<size_t>(shard_bytes), cudaMemcpyDeviceToDevice,
                        peer == rank ? local_stream : stream) != cudaSuccess)
      return -12;
  }
  const long long chunks = (shard_bytes + chunk_bytes - 1) / chunk_bytes;
  msq::comm_signal_kernel<<<1, 128, 0, stream>>>(make_ptrs(sig_ptrs, world), world, flag_base, rank * chunks, chunks, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int msq_comm_reduce_scatter_ce(void* const* slot_ptrs, long long slots_off_bytes, const void* full,
                                          long long shard_bytes, int rank, int world, void* const* sig_ptrs,
                                          long long flag_base, unsigned epoch, cudaStream_t stream) {
  if (world > msq::MAX_PEERS) return -2;
  if (shard_bytes <= 0) return 0;
  for (int pp = 0; pp < world; ++pp) {
    const int peer = (rank + pp) % world;
    void* d = static_cast<uint8_t*>(slot_ptrs[peer]) + slots_off_bytes + static_cast<long long>(rank) * shard_bytes;
    const void* sl = static_cast<const uint8_t*>(full) + static_cast<long long>(peer) * shard_bytes;
    if (cudaMemcpyAsync(d, sl, static_cast<size_t>(shard_bytes), cudaMemcpyDeviceToDevice, stream) != cudaSuccess) return -12;
  }
  msq::comm_signal_kernel<<<1, 128, 0, stream>>>(make_ptrs(sig_ptrs, world), world, flag_base, rank, 1, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int msq_comm_reduce_scatter_push(void* const* slot_ptrs, long long slots_off_bytes, const void* full,
                                            long long shard_bytes, int rank, int world, void* const* sig_ptrs,
                                            long long flag_base, unsigned epoch, unsigned* done_counter, int max_ctas,
                                            int* status, cudaStream_t stream) {
  if (world > msq::MAX_PEERS) return -2;
  if ((shard_bytes & 15) || (slots_off_bytes & 15) || (reinterpret_cast<uintptr_t>(full) & 15)) return -2;
  if (shard_bytes <= 0) return 0;
  long long want = ((shard_bytes >> 4) * world + 511) / 512;
  int grid = static_cast<int>(want < max_ctas ? want : max_ctas);
  if (grid < 1) grid = 1;
  msq::comm_reduce_scatter_push_kernel<<<grid, 512, 0, stream>>>(make_ptrs(slot_ptrs, world), slots_off_bytes,
                                                                static_cast<const uint4*>(full), shard_bytes, rank, world,
                                                                make_ptrs(sig_ptrs, world), flag_base, epoch, done_counter,
                                                                status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Owner-side reduce-scatter (see comm_reduce_scatter_pull_kernel).  `mc_base` (or null): multicast address of the
// symmetric regions; `src_ptrs`: the regions as mapped here; `buf_off_bytes`: offset of the full-size gradient
// buffer inside them.  This rank reduces elements [rank * shard_numel, (rank + 1) * shard_numel) of that buffer
// over all ranks into `out`.  Sources announce their buffers with msq_comm_signal(flag_base, epoch) beforehand.
extern "C" int msq_comm_reduce_scatter_pull(void* mc_base, void* const* src_ptrs, long long buf_off_bytes,
                                            long long shard_numel, int rank, int world, float scale, void* out,
                                            int out_fp32, int bf16, float* sumsq_acc, int* overflow, const void* flags,
                                            long long flag_base, unsigned epoch, int max_ctas, int* status,
                                            cudaStream_t stream) {
  if (world > msq::MAX_PEERS) return -2;
  if ((shard_numel & 7) || (buf_off_bytes & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return -2;
  if (shard_numel <= 0) return 0;
  long long want = ((shard_numel >> 3) + 255) / 256;
  int grid = static_cast<int>(want < max_ctas ? want : max_ctas);
  if (grid < 1) grid = 1;
  const long long shard_off = buf_off_bytes + static_cast<long long>(rank) * shard_numel * 2;
  const void* mc_shard = mc_base ? static_cast<const uint8_t*>(mc_base) + shard_off : nullptr;
  const uint32_t* f = static_cast<const uint32_t*>(flags);
  PeerPtrs sp = make_ptrs(src_ptrs, world);
#define MSQ_PULL(BF, O32, MC) \
  msq::comm_reduce_scatter_pull_kernel<BF, O32, MC><<<grid, 256, 0, stream>>>(mc_shard, sp, shard_off, shard_numel, rank, world, scale, out, sumsq_acc, overflow, f, flag_base, epoch, status)
  if (mc_base) {
    if (bf16) { if (out_fp32) MSQ_PULL(true, true, true); else MSQ_PULL(true, false, true); }
    else { if (out_fp32) MSQ_PULL(false, true, true); else MSQ_PULL(false, false, true); }
  } else {
    if (bf16) { if (out_fp32) MSQ_PULL(true, true, false); else MSQ_PULL(true, false, false); }
    else { if (out_fp32) MSQ_PULL(false, true, false); else MSQ_PULL(false, false, false); }
  }
#undef MSQ_PULL
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// All-gather by multimem.st (see comm_allgather_multimem_kernel).  `mc_dst`: multicast address of the gathered
// buffer; flags as for msq_comm_allgather_push.
extern "C" int msq_comm_allgather_multimem(void* mc_dst, const void* src, long long shard_bytes, int chunk_bytes, int rank,
                                           int world, void* const* sig_ptrs, long long flag_base, unsigned epoch,
                                           int max_ctas, int* status, cudaStream_t stream) {
  if (world > msq::MAX_PEERS || !mc_dst) return -2;
  if ((shard_bytes & 15) || (chunk_bytes & 15) || (reinterpret_cast<uintptr_t>(mc_dst) & 15) ||
      (reinterpret_cast<uintptr_t>(src) & 15))
    return -2;
  if (shard_bytes <= 0) return 0;
  long long chunks = (shard_bytes + chunk_bytes - 1) / chunk_bytes;
  int grid = static_cast<int>(chunks < max_ctas ? chunks : max_ctas);
  if (grid < 1) grid = 1;
  msq::comm_allgather_multimem_kernel<<<grid, 512, 0, stream>>>(mc_dst, static_cast<const uint4*>(src), shard_bytes,
                                                               chunk_bytes, rank, world, make_ptrs(sig_ptrs, world),
                                                               flag_base, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int msq_comm_reduce_slots(const void* slots, long long shard_numel, int world, float scale, void* out,
                                     int out_fp32, int bf16, float* sumsq_acc, int* overflow, const void* flags,
                                     long long flag_base, unsigned epoch, int max_ctas, int* status, cudaStream_t stream) {
  if ((shard_numel & 7) || (reinterpret_cast<uintptr_t>(slots) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return -2;
  if (shard_numel <= 0) return 0;
  long long want = ((shard_numel >> 3) + 255) / 256;
  int grid = static_cast<int>(want < max_ctas ? want : max_ctas);
  if (grid < 1) grid = 1;
  const uint4* s = static_cast<const uint4*>(slots);
  const uint32_t* f = static_cast<const uint32_t*>(flags);
#define MSQ_RS(BF, O32) \
  msq::comm_reduce_slots_kernel<BF, O32><<<grid, 256, 0, stream>>>(s, shard_numel, world, scale, out, sumsq_acc, overflow, f, flag_base, epoch, status)
  if (bf16) { if (out_fp32) MSQ_RS(true, true); else MSQ_RS(true, false); }
  else { if (out_fp32) MSQ_RS(false, true); else MSQ_RS(false, false); }
#undef MSQ_RS
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// dtype: 0 fp16, 1 bf16, 2 fp32.  bytes must be a multiple of 16 and at most slot_stride; the slot area
// holds 2 * world slots of slot_stride bytes at slots_off_bytes (one set per epoch parity).  in == out is allowed.
extern "C" int msq_comm_allreduce_oneshot(void* const* slot_ptrs, long long slots_off_bytes, long long slot_stride,
                                          const void* in, void* out,
                                          long long bytes, int dtype, int rank, int world, void* const* sig_ptrs,
                                          long long flag_base, unsigned epoch, int* status, cudaStream_t stream) {
  if (world > msq::MAX_PEERS) return -2;
  if ((bytes & 15) || (slot_stride & 15) || bytes > slot_stride || (reinterpret_cast<uintptr_t>(in) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return -2;
  if (bytes <= 0) return 0;
  PeerPtrs sl = make_ptrs(slot_ptrs, world), sg = make_ptrs(sig_ptrs, world);
  if (dtype == 0) msq::comm_allreduce_oneshot_kernel<0><<<1, 512, 0, stream>>>(sl, slots_off_bytes, slot_stride, in, out, bytes, rank, world, sg, flag_base, epoch, status);
  else if (dtype == 1) msq::comm_allreduce_oneshot_kernel<1><<<1, 512, 0, stream>>>(sl, slots_off_bytes, slot_stride, in, out, bytes, rank, world, sg, flag_base, epoch, status);
  else msq::comm_allreduce_oneshot_kernel<2><<<1, 512, 0, stream>>>(sl, slots_off_bytes, slot_stride, in, out, bytes, rank, world, sg, flag_base, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Multi-CTA one-shot all-reduce (see comm_allreduce_sliced_kernel).  Needs ceil(bytes / slice_bytes) * world flag
// words at flag_base; slots as for msq_comm_allreduce_oneshot.
extern "C" int msq_comm_allreduce_sliced(void* const* slot_ptrs, long long slots_off_bytes, long long slot_stride,
                                         const void* in, void* out, long long bytes, long long slice_bytes, int dtype,
                                         int rank, int world, void* const* sig_ptrs, long long flag_base, unsigned epoch,
                                         int* status, cudaStream_t stream) {
  if (world > msq::MAX_PEERS) return -2;
  if ((bytes & 15) || (slice_bytes & 15) || slice_bytes <= 0 || bytes > slot_stride || (reinterpret_cast<uintptr_t>(in) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return -2;
  if (bytes <= 0) return 0;
  const int grid = static_cast<int>((bytes + slice_bytes - 1) / slice_bytes);
  PeerPtrs sl = make_ptrs(slot_ptrs, world), sg = make_ptrs(sig_ptrs, world);
  if (dtype == 0) msq::comm_allreduce_sliced_kernel<0><<<grid, 512, 0, stream>>>(sl, slots_off_bytes, slot_stride, in, out, bytes, slice_bytes, rank, world, sg, flag_base, epoch, status);
  else if (dtype == 1) msq::comm_allreduce_sliced_kernel<1><<<grid, 512, 0, stream>>>(sl, slots_off_bytes, slot_stride, in, out, bytes, slice_bytes, rank, world, sg, flag_base, epoch, status);
  else msq::comm_allreduce_sliced_kernel<2><<<grid, 512, 0, stream>>>(sl, slots_off_bytes, slot_stride, in, out, bytes, slice_bytes, rank, world, sg, flag_base, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// One-launch in-switch all-reduce: `mc` is the multicast address and `stage_local` this rank's address of the
// same symmetric staging buffer.  Needs 2 * world flag words per slice at flag_base.
extern "C" int msq_comm_allreduce_multimem_fused(void* mc, void* stage_local, const void* in, void* out, long long bytes,
                                                 long long slice_bytes, int dtype, int rank, int world,
                                                 void* const* sig_ptrs, long long flag_base, unsigned epoch, int* status,
                                                 cudaStream_t stream) {
  if (world > msq::MAX_PEERS) return -2;
  if ((bytes & 15) || (slice_bytes & 15) || slice_bytes <= 0 || (reinterpret_cast<uintptr_t>(mc) & 15) ||
      (reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return -2;
  if (bytes <= 0) return 0;
  const int grid = static_cast<int>((bytes + slice_bytes - 1) / slice_bytes);
  PeerPtrs sg = make_ptrs(sig_ptrs, world);
  if (dtype == 0) msq::comm_allreduce_multimem_fused_kernel<0><<<grid, 512, 0, stream>>>(mc, stage_local, in, out, bytes, slice_bytes, rank, world, sg, flag_base, epoch, status);
  else if (dtype == 1) msq::comm_allreduce_multimem_fused_kernel<1><<<grid, 512, 0, stream>>>(mc, stage_local, in, out, bytes, slice_bytes, rank, world, sg, flag_base, epoch, status);
  else msq::comm_allreduce_multimem_fused_kernel<2><<<grid, 512, 0, stream>>>(mc, stage_local, in, out, bytes, slice_bytes, rank, world, sg, flag_base, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// In-place all-reduce of the symmetric buffer whose multicast address is `mc`.  The caller follows it
// with msq_comm_barrier before reading the result.
extern "C" int msq_comm_allreduce_multimem(void* mc, long long bytes, int dtype, int rank, int world, void* const* sig_ptrs,
                                           long long flag_base, unsigned epoch, int max_ctas, int* status,
                                           cudaStream_t stream) {
  if (world > msq::MAX_PEERS) return -2;
  if ((bytes & 15) || (reinterpret_cast<uintptr_t>(mc) & 15)) return -2;
  if (bytes <= 0) return 0;
  long long want = (((bytes >> 4) + world - 1) / world + 511) / 512;
  int grid = static_cast<int>(want < max_ctas ? want : max_ctas);
  if (grid < 1) grid = 1;
  PeerPtrs sg = make_ptrs(sig_ptrs, world);
  if (dtype == 0) msq::comm_allreduce_multimem_kernel<0><<<grid, 512, 0, stream>>>(mc, bytes, rank, world, sg, flag_base, epoch, status);
  else if (dtype == 1) msq::comm_allreduce_multimem_kernel<1><<<grid, 512, 0, stream>>>(mc, bytes, rank, world, sg, flag_base, epoch, status);
  else msq::comm_allreduce_multimem_kernel<2><<<grid, 512, 0, stream>>>(mc, bytes, rank, world, sg, flag_base, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Small sum / gather over ranks that may be captured in a CUDA graph (see comm_words_exchange_kernel).  `in`: `words`
// 32-bit words; recv0 / recv1: the two receive buffers of every rank (world * cap units of 8 bytes each, zero-filled
// at creation); `epoch_dev` and `ticket`: one zero-initialised word each, owned by this exchange.  mode 0 / 1: `out`
// gets the sum of fp16 / bf16 pairs (`words` words); mode 2: `out` gets world * words words, source-major.  Every
// rank must issue the same sequence of calls (same `words`) on buffers used by nothing else.
extern "C" int msq_comm_words_exchange(const void* in, long long words, void* const* recv0, void* const* recv1,
                                       long long cap, int rank, int world, unsigned* epoch_dev, unsigned* ticket,
                                       void* out, int mode, int* status, cudaStream_t stream) {
  if (world > msq::MAX_PEERS || words > cap || mode < 0 || mode > 2) return -2;
  if (words <= 0) return 0;
  long long want = (words + 255) / 256;
  const int grid = static_cast<int>(want < 64 ? want : 64);
  const uint32_t* i32 = static_cast<const uint32_t*>(in);
  uint32_t* o32 = static_cast<uint32_t*>(out);
  PeerPtrs r0 = make_ptrs(recv0, world), r1 = make_ptrs(recv1, world);
  if (mode == 0) msq::comm_words_exchange_kernel<0><<<grid, 256, 0, stream>>>(i32, words, r0, r1, cap, rank, world, epoch_dev, ticket, o32, status);
  else if (mode == 1) msq::comm_words_exchange_kernel<1><<<grid, 256, 0, stream>>>(i32, words, r0, r1, cap, rank, world, epoch_dev, ticket, o32, status);
  else msq::comm_words_exchange_kernel<2><<<grid, 256, 0, stream>>>(i32, words, r0, r1, cap, rank, world, epoch_dev, ticket, o32, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
