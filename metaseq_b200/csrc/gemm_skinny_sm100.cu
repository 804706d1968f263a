// Linear layer for a handful of rows (one decode step):  C[M,N] = epilogue(X[M,K] * W[N,K]^T),  M <= 64.
//
// With so few rows the product is a single pass over the weight matrix, so the kernel is built to stream W at
// memory speed rather than to fill the tensor cores:
//
//   * operands are swapped: a tile is 128 rows of W (the tcgen05 "M" side) against all rows of X padded to
//     16 / 32 / 64 (the "N" side), so no tensor-core lanes or shared memory are spent on padding of X to 128;
//   * the K range of a tile is split over the CTAs of a thread-block cluster (1, 2, 4 or 8), which gives
//     every SM a slice of W to fetch even when N / 128 is far below the SM count (out-projection, fc2);
//   * the cluster adds the partial products through distributed shared memory: CTA c owns rows
//     [c*128/S, (c+1)*128/S) of the tile; every CTA stores its fp32 partial rows straight into the owner's shared
//     memory (remote stores need no round trip), and after one cluster barrier the owner sums its S slots and
//     applies the epilogue (+bias -> ReLU -> +residual).  No workspace, no atomics, and the result does not
//     depend on the order in which CTAs finish;
//   * shared memory stays near 100 KB so that two CTAs share an SM and about 200 KB of loads are in flight
//     per SM.
//
// Tensor parallelism: a row-parallel product (K sharded over the ranks) ends in a sum over the ranks.  Here the
// owner CTA stores its finished partial rows (16-bit, like the all-reduce payload of the reference) straight into
// a receive buffer of every rank over NVLink, each 4 bytes of payload paired with a 4-byte epoch in one 8-byte
// unit, and then polls its own receive buffer until the units of every source rank carry the epoch: the data
// is its own arrival flag, so the exchange costs one one-way store latency, with no fence, no separate flag and
// no remote load.  It then adds the ranks' rows in fp32 and applies bias and residual: GEMM and all-reduce in
// one launch, tile by tile, without a grid-wide or rank-wide barrier.  Epochs live in device memory (one counter
// per CTA, advanced by the kernel), so the launch can be replayed from a CUDA graph; consecutive products
// alternate between two receive buffers (chosen by the caller), which keeps a fast rank from overwriting units
// that a slow rank has not consumed yet, provided every such product of the sequence uses the same grid (CTA i
// sends product n+2 only after it received product n+1 from CTA i of every peer, which they send after consuming
// product n).
//
// The reference runs these products as torch.matmul plus separate bias / activation / residual kernels
// (metaseq/modules/megatron/mpu/layers.py:290,373; metaseq/modules/feedforward.py:21-22) and the sum over ranks
// as an NCCL all-reduce after the product (metaseq/modules/megatron/mpu/mappings.py:27-40).
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 2..5 move the
// accumulator to the owners' shared memory; all threads take part in the final sum.
#include <cstdio>

#include "sm100_common.cuh"

namespace msq {

int make_tmap_2d(CUtensorMap* out, const void* base, long long rows, long long cols, long long ld, int box_rows,
                 int bf16);  // gemm_sm100.cu

constexpr int SK_MAX_RANKS = 8;

struct SkinnyParams {
  int M, N, K;
  int k_blocks_per_cta;
  int split;  // cluster size along K
  void* C;
  long long ldc;
  const void* bias;      // [N] or null
  const void* residual;  // [M, ldr] or null
  long long ldr;
  int relu;  // activation after the bias: 0 none, 1 ReLU, 2 GELU (erf form)
  int bf16;
  int* status;
  // sum over tensor-parallel ranks (world <= 1: none)
  int world, rank;
  void* recv_buf[SK_MAX_RANKS];  // every rank's receive buffer for this product: [world][slot_rows][N] 4-byte cells,
                                 // cell (src, m, n) = {two 16-bit values for columns n, n+1 | epoch} at even n
  int slot_rows;                 // rows reserved per source rank
  uint32_t* epoch_dev;           // this rank's per-CTA epoch counters
  long long* prof;               // debug: per-CTA cycle stamps (see msq_gemm_skinny_set_prof)
};

constexpr int SK_BM = 128;  // rows of W per tile
constexpr int SK_BK = 64;
constexpr int SK_THREADS = 192;

template <int MP>
struct SkinnyCfg {
  static constexpr uint32_t W_BYTES = SK_BM * SK_BK * 2;
  static constexpr uint32_t X_BYTES = MP * SK_BK * 2;
  static constexpr int STAGES = (MP == 64) ? 3 : (MP == 32 ? 4 : 5);
  static constexpr uint32_t RECV_BYTES = SK_BM * MP * 4;  // S slots of [MP][128 / S] fp32, whatever S is
  static constexpr uint32_t SMEM = STAGES * (W_BYTES + X_BYTES) + RECV_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
  static constexpr uint32_t TMEM_COLS = MP < 32 ? 32 : MP;
  static_assert(2 * SMEM <= 227 * 1024, "two CTAs must fit in one SM");
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Barrier 1 only establishes that every CTA of the cluster has started (its shared memory exists) before a
// peer stores into it: arrive early, wait just before the first remote store.  Not `.aligned`: the roles diverge.
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
// Barrier 2 publishes the remote stores to their owners.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t remote_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote_addr), "f"(v) : "memory");
}

__device__ __forceinline__ float activate(float x, int kind) {
  if (kind == 1) return fmaxf(x, 0.f);
  if (kind == 2) return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
  return x;
}

// 16-byte load of two {payload, epoch} units that a peer GPU writes: never from L1.
__device__ __forceinline__ uint4 ld_units(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// 16-byte store of two units into (possibly) another GPU's memory.  Each 8-byte half is self-validating, so no
// ordering between stores is needed.
__device__ __forceinline__ void st_units(void* p, uint32_t d0, uint32_t d1, uint32_t epoch) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(d0), "r"(epoch), "r"(d1), "r"(epoch)
               : "memory");
}

template <int MP>
__global__ void __launch_bounds__(SK_THREADS, 2)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                   const SkinnyParams p) {
  using Cfg = SkinnyCfg<MP>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sW = smem;
  uint8_t* sX = smem + STAGES * Cfg::W_BYTES;
  float* recv = reinterpret_cast<float*>(sX + STAGES * Cfg::X_BYTES);  // [S][MP][128 / S]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sX + STAGES * Cfg::X_BYTES + Cfg::RECV_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t crank = cluster_ctarank();
  const int tile = blockIdx.x / p.split;
  const int n0 = tile * SK_BM;
  const int total_kb = (p.K + SK_BK - 1) / SK_BK;
  const int kb0 = static_cast<int>(crank) * p.k_blocks_per_cta;
  const int kb1 = min(total_kb, kb0 + p.k_blocks_per_cta);
  const int my_kb = max(0, kb1 - kb0);

  // A wait that ran out earlier on this stream left its code in the status word: do no work until the host has
  // read and cleared it.  The CTA still walks through the cluster barriers below, because its peers may have
  // read the word before it was set and will address this CTA's shared memory.
  const bool skip = p.status && *reinterpret_cast<volatile int*>(p.status) != 0;
  const long long prof_t0 = p.prof ? clock64() : 0;
  dependents_launch();

  const int head = (!skip) ? min(STAGES, my_kb) : 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tfull_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
    // The weights are not written by any kernel of the stream, so the first ring of W tiles is requested at
    // once: before the rest of the set-up and before the wait for the preceding kernels.
    for (int i = 0; i < head; ++i) {
      mbar_expect_tx(&full_bar[i], Cfg::W_BYTES + Cfg::X_BYTES);
      tma_load_2d(sW + i * Cfg::W_BYTES, &tmW, &full_bar[i], (kb0 + i) * SK_BK, n0);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  cluster_arrive_relaxed();  // barrier 1
  bool waited = false;
  const uint32_t tmem_base = *tmem_slot;
  const int R = SK_BM / p.split;  // rows of the tile that each CTA of the cluster owns

  if (!skip && my_kb > 0) {
    if (warp == 0) {
      // ---------------------------------------------------------- producer
      if (lane == 0) {
        dependents_wait();
        for (int i = 0; i < head; ++i)
          tma_load_2d(sX + i * Cfg::X_BYTES, &tmX, &full_bar[i], (kb0 + i) * SK_BK, 0);
        int stage = 0;  // head == STAGES whenever the loop below runs
        uint32_t phase = 1;
        bool ok = true;
        for (int kb = kb0 + head; kb < kb1; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, ST_TIMEOUT_SMEM_EMPTY);
          if (!ok) break;
          mbar_expect_tx(&full_bar[stage], Cfg::W_BYTES + Cfg::X_BYTES);
          tma_load_2d(sW + stage * Cfg::W_BYTES, &tmW, &full_bar[stage], kb * SK_BK, n0);
          tma_load_2d(sX + stage * Cfg::X_BYTES, &tmX, &full_bar[stage], kb * SK_BK, 0);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) {
          // Leaving early: give the copies already issued a bounded time to land before this CTA's shared
          // memory can be handed to another CTA.
          const unsigned long long t0 = globaltimer_ns();
          while (globaltimer_ns() - t0 < 2000000ull) { }
        }
      }
    } else if (warp == 1) {
      // -------------------------------------------------------- MMA issuer
      if (lane == 0) {
        const uint32_t idesc = make_idesc_f16(p.bf16, 0, 0, SK_BM, MP);
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int i = 0; i < my_kb; ++i) {
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t w_addr = smem_u32(sW + stage * Cfg::W_BYTES);
          const uint32_t x_addr = smem_u32(sX + stage * Cfg::X_BYTES);
#pragma unroll
          for (int kk = 0; kk < SK_BK / 16; ++kk) {
            const uint64_t dw = make_smem_desc_sw128(w_addr + kk * 32, 16, 1024);
            const uint64_t dx = make_smem_desc_sw128(x_addr + kk * 32, 16, 1024);
            tc_mma_f16(tmem_base, dw, dx, idesc, (i > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit(tfull_bar);
      }
    } else {
      // --------------------------- accumulator -> the owners' shared memory
      const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) = rows of the W tile
      const bool ok = mbar_wait_warp(tfull_bar, 0, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
      cluster_wait();  // barrier 1: the owners' shared memory exists
      waited = true;
      if (ok) {
        tc_fence_after();
        const int r = quarter * 32 + lane;
        const uint32_t slot = smem_u32(recv) + static_cast<uint32_t>((static_cast<int>(crank) * MP) * R + (r % R)) * 4u;
        const uint32_t dst = map_to_cta(slot, static_cast<uint32_t>(r / R));
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll
        for (int c = 0; c < MP / 16; ++c) {
          uint32_t v[16];
          tmem_ld_32x16(taddr + c * 16, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j)
            st_cluster_f32(dst + static_cast<uint32_t>((c * 16 + j) * R) * 4u, __uint_as_float(v[j]));
        }
      }
    }
  } else if (warp >= 2) {
    // no K range (or skipping): contribute zeros
    cluster_wait();
    waited = true;
    const int r = (warp & 3) * 32 + lane;
    const uint32_t slot = smem_u32(recv) + static_cast<uint32_t>((static_cast<int>(crank) * MP) * R + (r % R)) * 4u;
    const uint32_t dst = map_to_cta(slot, static_cast<uint32_t>(r / R));
    for (int m = 0; m < MP; ++m) st_cluster_f32(dst + static_cast<uint32_t>(m * R) * 4u, 0.f);
  }
  if (!waited) cluster_wait();  // barrier 1 for the threads that store nothing

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
  dependents_wait();   // the residual is an output of the preceding kernels, and C may be memory they still read
  const long long prof_wait = p.prof ? clock64() : 0;
  cluster_sync_all();  // barrier 2: every partial row has reached its owner
  const long long prof_sum = p.prof ? clock64() : 0;

  const bool reduce_ranks = p.world > 1;
  const uint32_t epoch = reduce_ranks ? p.epoch_dev[blockIdx.x] + 1u : 0u;
  long long prof_sent = 0;
  if (!skip && !reduce_ranks) {
    // This CTA finishes rows [crank*R, crank*R + R) of the tile, two adjacent rows (= output columns) per item.
    const int half = R >> 1;
    const int items = half * p.M;
    for (int e = threadIdx.x; e < items; e += SK_THREADS) {
      const int m = e / half;
      const int rl = (e - m * half) * 2;
      const int n = n0 + static_cast<int>(crank) * R + rl;
      if (n >= p.N) continue;  // N is even, so a pair is inside or outside as a whole
      uint32_t bw = 0u, rw = 0u;  // requested before the sum so that their latency overlaps it
      if (p.bias) bw = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint16_t*>(p.bias) + n);
      if (p.residual)
        rw = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint16_t*>(p.residual) +
                                                static_cast<long long>(m) * p.ldr + n);
      float2 acc = make_float2(0.f, 0.f);
      for (int j = 0; j < p.split; ++j) {
        const float2 v = *reinterpret_cast<const float2*>(recv + (j * MP + m) * R + rl);
        acc.x += v.x;
        acc.y += v.y;
      }
      if (p.bias) {
        const float2 b2 = p.bf16 ? unpack2<true>(bw) : unpack2<false>(bw);
        acc.x += b2.x;
        acc.y += b2.y;
      }
      acc.x = activate(acc.x, p.relu);
      acc.y = activate(acc.y, p.relu);
      if (p.residual) {
        const float2 r2 = p.bf16 ? unpack2<true>(rw) : unpack2<false>(rw);
        acc.x += r2.x;
        acc.y += r2.y;
      }
      uint32_t* dst = reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(p.C) + static_cast<long long>(m) * p.ldc + n);
      *dst = p.bf16 ? pack2<true>(acc.x, acc.y) : pack2<false>(acc.x, acc.y);
    }
  }
  if (!reduce_ranks || skip) return;

  // ------------------------------------------------------- sum over ranks
  // 8 adjacent columns of one row per item: R is a multiple of 16 and N of 8, so a chunk is inside or outside N as
  // a whole.  A chunk is four {payload, epoch} units = two 16-byte stores per destination rank.
  const int chunks = R >> 3;
  const int items = chunks * p.M;
  for (int e = threadIdx.x; e < items; e += SK_THREADS) {
    const int m = e / chunks;
    const int rl = (e - m * chunks) * 8;
    const int n = n0 + static_cast<int>(crank) * R + rl;
    if (n >= p.N) continue;
    uint32_t d[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float2 acc = make_float2(0.f, 0.f);
      for (int j = 0; j < p.split; ++j) {
        const float2 v = *reinterpret_cast<const float2*>(recv + (j * MP + m) * R + rl + 2 * q);
        acc.x += v.x;
        acc.y += v.y;
      }
      d[q] = p.bf16 ? pack2<true>(acc.x, acc.y) : pack2<false>(acc.x, acc.y);
    }
    const long long cell = (static_cast<long long>(p.rank) * p.slot_rows + m) * p.N + n;  // 4-byte cells
#pragma unroll
    for (int r = 0; r < SK_MAX_RANKS; ++r) {
      if (r < p.world) {
        uint8_t* dst = static_cast<uint8_t*>(p.recv_buf[r]) + cell * 4;
        st_units(dst, d[0], d[1], epoch);
        st_units(dst + 16, d[2], d[3], epoch);
      }
    }
  }
  if (p.prof) prof_sent = clock64();
  bool all_ok = true;
  for (int e = threadIdx.x; e < items && all_ok; e += SK_THREADS) {
    const int m = e / chunks;
    const int n = n0 + static_cast<int>(crank) * R + (e - m * chunks) * 8;
    if (n >= p.N) continue;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int r = 0; r < p.world && all_ok; ++r) {
      const uint8_t* src = static_cast<const uint8_t*>(p.recv_buf[p.rank]) +
                           ((static_cast<long long>(r) * p.slot_rows + m) * p.N + n) * 4;
      uint4 u0 = ld_units(src), u1 = ld_units(src + 16);
      if (u0.y != epoch || u0.w != epoch || u1.y != epoch || u1.w != epoch) {
        const unsigned long long t0 = globaltimer_ns();
        uint32_t spins = 0;
        while (true) {
          u0 = ld_units(src);
          u1 = ld_units(src + 16);
          if (u0.y == epoch && u0.w == epoch && u1.y == epoch && u1.w == epoch) break;
          if ((++spins & 0x3f) == 0) {
            if ((p.status && *reinterpret_cast<volatile int*>(p.status) != 0) || globaltimer_ns() - t0 > WAIT_NS_PEER) {
              if (p.status) atomicCAS(p.status, 0, ST_TIMEOUT_PEER_FLAG);
              all_ok = false;
              break;
            }
          }
        }
      }
      const uint32_t w4[4] = {u0.x, u0.z, u1.x, u1.z};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 v = p.bf16 ? unpack2<true>(w4[j]) : unpack2<false>(w4[j]);
        acc[2 * j] += v.x;
        acc[2 * j + 1] += v.y;
      }
    }
    if (!all_ok) break;
    const uint16_t* bias16 = reinterpret_cast<const uint16_t*>(p.bias);
    const uint16_t* res16 = reinterpret_cast<const uint16_t*>(p.residual);
    uint32_t out4[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float a0 = acc[2 * j], a1 = acc[2 * j + 1];
      if (bias16) {
        const uint32_t bw = *reinterpret_cast<const uint32_t*>(bias16 + n + 2 * j);
        const float2 b2 = p.bf16 ? unpack2<true>(bw) : unpack2<false>(bw);
        a0 += b2.x;
        a1 += b2.y;
      }
      a0 = activate(a0, p.relu);
      a1 = activate(a1, p.relu);
      if (res16) {
        const uint32_t rw = *reinterpret_cast<const uint32_t*>(res16 + static_cast<long long>(m) * p.ldr + n + 2 * j);
        const float2 r2 = p.bf16 ? unpack2<true>(rw) : unpack2<false>(rw);
        a0 += r2.x;
        a1 += r2.y;
      }
      out4[j] = p.bf16 ? pack2<true>(a0, a1) : pack2<false>(a0, a1);
    }
    uint32_t* dst = reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(p.C) + static_cast<long long>(m) * p.ldc + n);
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[j] = out4[j];
  }
  // The counter advances only when every thread got its units: after a timeout the status word tells the host.
  if (__syncthreads_and(all_ok ? 1 : 0) && threadIdx.x == 0) p.epoch_dev[blockIdx.x] = epoch;
  if (p.prof && threadIdx.x == 0) {
    long long* o = p.prof + static_cast<long long>(blockIdx.x) * 6;
    o[0] = prof_wait - prof_t0;   // start -> previous kernels done, own K range multiplied (before the cluster barrier)
    o[1] = prof_sum - prof_wait;  // cluster barrier
    o[2] = prof_sent - prof_sum;  // cluster sum, units stored to every rank
    o[3] = clock64() - prof_sent; // units of every rank received, epilogue
    o[4] = 0;
    o[5] = clock64() - prof_t0;
  }
}

static int g_skinny_sms = 0;

template <int MP>
static int launch_skinny(const CUtensorMap& tmW, const CUtensorMap& tmX, const SkinnyParams& p, cudaStream_t stream) {
  using Cfg = SkinnyCfg<MP>;
  auto kern = gemm_skinny_kernel<MP>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess) return -10;
    configured = true;
  }
  const int tiles = (p.N + SK_BM - 1) / SK_BM;
  if (launch_chained(kern, dim3(static_cast<unsigned>(tiles * p.split), 1, 1), dim3(SK_THREADS, 1, 1), Cfg::SMEM, stream,
                     static_cast<unsigned>(p.split), tmW, tmX, p) != cudaSuccess) {
    cudaGetLastError();
    return -11;
  }
  return 0;
}

thread_local int g_dependent_launch = 0;
static long long* g_skinny_prof = nullptr;

}  // namespace msq

// Cluster size along K that the launch will use (exposed for tests and benchmarks).
extern "C" int msq_gemm_skinny_split(int N, int K) {
  using namespace msq;
  if (g_skinny_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&g_skinny_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || g_skinny_sms <= 0)
      g_skinny_sms = 148;
  }
  const int tiles = (N + SK_BM - 1) / SK_BM;
  const int k_blocks = (K + SK_BK - 1) / SK_BK;
  const int slots = 2 * g_skinny_sms;  // two CTAs per SM
  int split = 1;
  for (int s = 8; s > 1; s >>= 1) {
    if (tiles * s <= slots && k_blocks >= 2 * s) { split = s; break; }
  }
  return split;
}

namespace msq {

static int skinny_common(const void* X, const void* W, void* C, int M, int N, int K, long long ldx, long long ldw,
                         long long ldc, int bf16, const void* bias, const void* residual, long long ldr, int relu,
                         int* status, cudaStream_t stream, SkinnyParams& p, int split) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || (N & 7) || (K & 7) || (ldc & 1) || (ldr & 1) || (reinterpret_cast<uintptr_t>(C) & 3) ||
      (reinterpret_cast<uintptr_t>(residual) & 3) || (reinterpret_cast<uintptr_t>(bias) & 3))
    return -4;
  const int mp = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  CUtensorMap tmW, tmX;
  int rc = make_tmap_2d(&tmW, W, N, K, ldw, SK_BM, bf16);
  if (rc) return rc;
  rc = make_tmap_2d(&tmX, X, M, K, ldx, mp, bf16);
  if (rc) return rc - 100;
  p.M = M; p.N = N; p.K = K;
  p.split = split;
  const int k_blocks = (K + SK_BK - 1) / SK_BK;
  p.k_blocks_per_cta = (k_blocks + p.split - 1) / p.split;
  p.C = C; p.ldc = ldc;
  p.bias = bias; p.residual = residual; p.ldr = ldr;
  p.relu = relu; p.bf16 = bf16; p.status = status;
  if (mp == 16) return launch_skinny<16>(tmW, tmX, p, stream);
  if (mp == 32) return launch_skinny<32>(tmW, tmX, p, stream);
  return launch_skinny<64>(tmW, tmX, p, stream);
}

}  // namespace msq

// X: [M, K] (row stride ldx), W: [N, K] (row stride ldw), C: [M, N] (row stride ldc), all 16-bit of one type,
// strides in elements.  `relu`: 0 none, 1 ReLU, 2 GELU after the bias.  M <= 64; K and N multiples of 8; base pointers 16-byte aligned, C / residual / bias 4-byte
// aligned with even strides.  Returns 0 on a successful launch, a negative code for unsupported arguments.
extern "C" int msq_gemm_skinny(const void* X, const void* W, void* C, int M, int N, int K, long long ldx, long long ldw,
                               long long ldc, int bf16, const void* bias, const void* residual, long long ldr, int relu,
                               int* status, cudaStream_t stream) {
  msq::SkinnyParams p = {};
  p.world = 1;
  return msq::skinny_common(X, W, C, M, N, K, ldx, ldw, ldc, bf16, bias, residual, ldr, relu, status, stream, p,
                            msq_gemm_skinny_split(N, K));
}

// Row-parallel product of a tensor-parallel layer: C = epilogue(sum over ranks of X_r W_r^T), every rank ending
// with the full sum.  `recv_ptrs[r]` is rank r's receive buffer for this call: world * slot_rows * N 4-byte cells
// (zero-initialised once; the same offset of a symmetric allocation on every rank; the caller alternates between
// two such buffers from call to call); `epoch_dev` holds one zero-initialised counter per CTA.  `split` fixes the
// cluster size (0 = choose as msq_gemm_skinny does): every product that shares buffers and counters must use one
// grid.  Returns the number of CTAs launched, or a negative code.
extern "C" int msq_gemm_skinny_allreduce(const void* X, const void* W, void* C, int M, int N, int K, long long ldx,
                                         long long ldw, long long ldc, int bf16, const void* bias, const void* residual,
                                         long long ldr, int relu, int rank, int world, void* const* recv_ptrs,
                                         int slot_rows, unsigned* epoch_dev, int split, int* status, cudaStream_t stream) {
  using namespace msq;
  if (world < 1 || world > SK_MAX_RANKS || rank < 0 || rank >= world) return -6;
  if (world > 1 && (!recv_ptrs || !epoch_dev || M > slot_rows)) return -6;
  SkinnyParams p = {};
  p.world = world;
  p.rank = rank;
  for (int r = 0; r < world && world > 1; ++r) {
    p.recv_buf[r] = recv_ptrs[r];
    if (!p.recv_buf[r] || (reinterpret_cast<uintptr_t>(p.recv_buf[r]) & 15)) return -6;
  }
  p.slot_rows = slot_rows;
  p.epoch_dev = epoch_dev;
  p.prof = g_skinny_prof;
  if (split != 1 && split != 2 && split != 4 && split != 8) split = msq_gemm_skinny_split(N, K);
  const int k_blocks = (K + SK_BK - 1) / SK_BK;
  while (split > 1 && k_blocks < split) split >>= 1;
  const int rc = skinny_common(X, W, C, M, N, K, ldx, ldw, ldc, bf16, bias, residual, ldr, relu, status, stream, p, split);
  return rc < 0 ? rc : ((N + SK_BM - 1) / SK_BM) * split;
}

// Debug aid: device buffer of 6 int64 per CTA that the next launches of msq_gemm_skinny_allreduce fill with the
// cycle counts of their phases (null switches it off).
extern "C" void msq_gemm_skinny_set_prof(long long* buf) { msq::g_skinny_prof = buf; }

// Non-zero: the calling thread's launches of the few-row GEMM, the LayerNorm forward and the decode attention
// carry the programmatic-dependent-launch attribute, so that each may start (and the GEMM may request its
// first weight tiles) while its predecessor drains.  Only for call sequences in which the GEMM's W operand is
// not written by any kernel in flight (a decode step: W are model weights).
extern "C" int msq_set_dependent_launch(int on) {
  msq::g_dependent_launch = on ? 1 : 0;
  return 0;
}
