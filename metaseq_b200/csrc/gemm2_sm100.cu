// Two-CTA (cta_group::2) variant of the persistent tcgen05 GEMM: a cluster of two CTAs on
// neighbouring SMs computes one 256 x 256 output tile.  Each CTA loads its own 128 rows of A
// and half (128 rows) of the B tile, the leader CTA issues one tcgen05.mma.cta_group::2 per
// 16-wide k step that drives the tensor cores of both SMs, and each CTA keeps its 128 x 256
// fp32 accumulator in its own TMEM.  Against the one-CTA kernel (gemm_sm100.cu) this halves
// the B traffic from L2 into each SM (32 KB instead of 48 KB per 64-wide k block), which is
// what limits that kernel, and leaves room for six pipeline stages.
//
// No load uses cluster multicast: every CTA issues plain tiled TMA loads into its own shared
// memory and only the completion is signalled on the leader's mbarrier (cta_group::2 form).
//
// Same operand layouts and epilogue as msq_gemm; see gemm_sm100.cu.
#include <cstdio>

#include "sm100_common.cuh"

namespace msq {

struct Gemm2Params {
  int M, N, K;
  void* C;
  long long ldc;
  const void* bias;
  const void* residual;
  long long ldr;
  const void* mask;
  long long ldm;
  int relu;
  int accumulate;
  int bf16;
  int* status;
  // Arrival flags of the B operand when it is (part of) a gathered buffer that peer GPUs fill over NVLink:
  // the buffer is cut into `ready_world` shards of ready_shard_bytes, each into chunks of ready_chunk_bytes with
  // one flag word per chunk; a chunk is usable once its flag has reached ready_epoch.  B starts
  // ready_b_offset bytes into the buffer.  The producer warp polls (bounded) the flags covering the rows it is
  // about to load, so the product starts while later chunks are still in flight.  Chunks of shard
  // ready_skip_shard (the local rank's own, ordered by the stream) are not polled.  Null = no waiting.
  const uint32_t* ready_flags;
  long long ready_b_offset;
  long long ready_ldb_bytes;
  long long ready_shard_bytes;
  long long ready_chunk_bytes;
  int ready_chunks_per_shard;
  int ready_skip_shard;
  uint32_t ready_epoch;
  int ready_operand;  // 0: the flags describe B (weights arriving, FSDP); 1: they describe A (rows arriving, sequence parallel)
  long long* prof;  // debug: cycle counters of the first pair's MMA thread (see msq_gemm2_set_prof)
  // Row-scatter output (GEMM -> reduce-scatter over NVLink): when scatter_world > 0 the tile rows are not
  // written to C but stored into peer memory: row r belongs to rank r / scatter_rows and lands at
  // scatter_base[that rank] + (r % scatter_rows) * ldc.  Each base already points at the slot reserved for
  // this source rank, so the owner later sums one slot per source.  Epilogue options are not applied.
  void* scatter_base[16];
  int scatter_world;
  int scatter_rows;
  // Row statistics of the stored output (softmax pieces for a cross entropy that follows a logits product):
  // for column tile tn, rs_max[tn * M + r] = max over the tile's columns of row r and rs_sum[tn * M + r] =
  // sum of exp(value - that max), both over the values as rounded for storage.  Null = not computed.
  float* rs_max;
  float* rs_sum;
};

// Bounded wait until every chunk overlapping bytes [lo, hi) of the gathered buffer has arrived.
__device__ __forceinline__ bool wait_operand_ready(const Gemm2Params& p, long long lo, long long hi, volatile int* abort_flag) {
  if (hi <= lo) return true;
  const long long last = hi - 1;
  long long shard = lo / p.ready_shard_bytes;
  long long chunk = (lo - shard * p.ready_shard_bytes) / p.ready_chunk_bytes;
  const long long shard_end = last / p.ready_shard_bytes;
  const long long chunk_end = (last - shard_end * p.ready_shard_bytes) / p.ready_chunk_bytes;
  while (shard < shard_end || (shard == shard_end && chunk <= chunk_end)) {
    if (shard != p.ready_skip_shard) {
      const uint32_t* f = p.ready_flags + shard * p.ready_chunks_per_shard + chunk;
      const unsigned long long t0 = globaltimer_ns();
      uint32_t spins = 0;
      while (true) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
        if (static_cast<int32_t>(v - p.ready_epoch) >= 0) break;
        if ((++spins & 0x3f) == 0) {
          if (*abort_flag) return false;
          if (globaltimer_ns() - t0 > WAIT_NS_PEER) {
            *abort_flag = 1;
            if (p.status) atomicCAS(p.status, 0, ST_TIMEOUT_PEER_FLAG);
            return false;
          }
          __nanosleep(100);
        }
      }
    }
    if (++chunk == p.ready_chunks_per_shard) { chunk = 0; ++shard; }
  }
  // the chunks were written through the generic proxy (peer stores or DMA); the loads below use the async proxy
  asm volatile("fence.proxy.async.global;" ::: "memory");
  return true;
}

constexpr int G2_BM = 128;   // rows per CTA (256 per pair)
constexpr int G2_BN = 256;   // columns per pair; each CTA stages half of the B tile
constexpr int G2_BK = 64;
constexpr int G2_STAGES = 6;
constexpr int G2_THREADS = 192;
constexpr uint32_t G2_A_BYTES = G2_BM * G2_BK * 2;        // 16 KB
constexpr uint32_t G2_B_BYTES = (G2_BN / 2) * G2_BK * 2;  // 16 KB
constexpr uint32_t G2_EPI_BYTES = 4 * 2048;  // per epilogue warp: 32 rows x 64 bytes of output being transposed
constexpr uint32_t G2_SMEM = G2_STAGES * (G2_A_BYTES + G2_B_BYTES) + G2_EPI_BYTES + 1024 + 256;
constexpr uint32_t G2_TMEM_COLS = 2 * G2_BN;
constexpr uint32_t PEER_BIT_MASK = 0xFEFFFFFFu;  // clears the CTA-parity bit of a shared address

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_shared_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// Tiled load into this CTA's shared memory; completion bytes are credited to the barrier at the
// same offset in the even (leader) CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int c0,
                                                 int c1) {
  const uint32_t leader_bar = smem_u32(bar) & PEER_BIT_MASK;
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(leader_bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this offset in both CTAs of the pair once all earlier MMAs are done.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  const uint16_t mask = 0x3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(mask)
      : "memory");
}

__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int GROUP = 8;  // 8 x 256 rows share the same sweep over column tiles
  const int per_group = GROUP * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP;
  const int gsize = min(GROUP, tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + (r % gsize);
  tn = r / gsize;
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G2_THREADS, 1)
gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const Gemm2Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + G2_STAGES * G2_A_BYTES;
  uint8_t* sEpi = sB + G2_STAGES * G2_B_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sEpi + G2_EPI_BYTES);
  uint64_t* empty_bar = full_bar + G2_STAGES;
  uint64_t* tfull_bar = empty_bar + G2_STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile uint32_t* skip_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  const int tiles_m = (p.M + 2 * G2_BM - 1) / (2 * G2_BM);
  const int tiles_n = (p.N + G2_BN - 1) / G2_BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (p.K + G2_BK - 1) / G2_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < G2_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 8);  // 4 epilogue warps in each CTA of the pair
    }
    *abort_flag = 0;
    if (rank == 0) {
      // One decision for the pair: skip all work when an earlier launch left a timeout code behind.
      const uint32_t skip = (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1u : 0u;
      *skip_flag = skip;
      st_shared_cluster_u32(map_to_cta(smem_u32(const_cast<uint32_t*>(skip_flag)), 1), skip);
    }
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  __syncthreads();
  cluster_sync_all();  // barriers of both CTAs are initialised, skip flag is in place
  if (*skip_flag) return;

  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, G2_TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const long long ldb_bytes = p.ready_ldb_bytes;
      const bool poll_b = p.ready_flags && p.ready_operand == 0;
      const bool poll_a = p.ready_flags && p.ready_operand == 1 && !A_MN;
      if (poll_b && B_MN)  // every tile reads all k-rows of an MN-major B: the whole operand must be here
        ok = wait_operand_ready(p, p.ready_b_offset, p.ready_b_offset + static_cast<long long>(p.K) * ldb_bytes, abort_flag);
      if (p.ready_flags && p.ready_operand == 1 && A_MN)  // MN-major A: all k-rows of the operand
        ok = wait_operand_ready(p, p.ready_b_offset, p.ready_b_offset + static_cast<long long>(p.K) * ldb_bytes, abort_flag);
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int tm, tn;
        pair_tile_coords(tile, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * 2 * G2_BM + static_cast<int>(rank) * G2_BM;
        const int n0 = tn * G2_BN + static_cast<int>(rank) * (G2_BN / 2);
        // Rows n0 .. n0+127 of a K-major B are one contiguous byte range.  The first tile is checked here; every
        // later tile was checked one tile ahead (below), while the pipeline was full, so the system-scope
        // acquire loads cost no issue time.
        if (poll_b && !B_MN && tile == pair) {
          const long long r1 = min(n0 + G2_BN / 2, p.N);
          ok = wait_operand_ready(p, p.ready_b_offset + n0 * ldb_bytes, p.ready_b_offset + r1 * ldb_bytes, abort_flag);
          if (!ok) break;
        }
        if (poll_a && tile == pair) {  // rows m0 .. m0+127 of a K-major A (ready_ldb_bytes is its row pitch here)
          const long long r1 = min(m0 + G2_BM, p.M);
          ok = wait_operand_ready(p, p.ready_b_offset + m0 * ldb_bytes, p.ready_b_offset + r1 * ldb_bytes, abort_flag);
          if (!ok) break;
        }
        const int check_kb = k_blocks > G2_STAGES ? G2_STAGES - 1 : k_blocks - 1;
        for (int kb = 0; kb < k_blocks; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, ST_TIMEOUT_SMEM_EMPTY);
          if (!ok) break;
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * (G2_A_BYTES + G2_B_BYTES));
          uint8_t* a_dst = sA + stage * G2_A_BYTES;
          uint8_t* b_dst = sB + stage * G2_B_BYTES;
          const int k0 = kb * G2_BK;
          if constexpr (!A_MN) {
            tma_load_2d_pair(a_dst, &tmA, &full_bar[stage], k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < G2_BM / 64; ++c)
              tma_load_2d_pair(a_dst + c * (G2_BK * 128), &tmA, &full_bar[stage], m0 + c * 64, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(b_dst, &tmB, &full_bar[stage], k0, n0);
          } else {
#pragma unroll
            for (int c = 0; c < (G2_BN / 2) / 64; ++c)
              tma_load_2d_pair(b_dst + c * (G2_BK * 128), &tmB, &full_bar[stage], n0 + c * 64, k0);
          }
          if (++stage == G2_STAGES) { stage = 0; phase ^= 1; }
          if ((poll_a || (poll_b && !B_MN)) && kb == check_kb && tile + num_pairs < num_tiles) {
            int ntm, ntn;
            pair_tile_coords(tile + num_pairs, tiles_m, tiles_n, ntm, ntn);
            long long lo, hi;
            if (poll_a) {
              lo = ntm * 2 * G2_BM + static_cast<int>(rank) * G2_BM;
              hi = min(lo + G2_BM, static_cast<long long>(p.M));
            } else {
              lo = ntn * G2_BN + static_cast<int>(rank) * (G2_BN / 2);
              hi = min(lo + G2_BN / 2, static_cast<long long>(p.N));
            }
            ok = wait_operand_ready(p, p.ready_b_offset + lo * ldb_bytes, p.ready_b_offset + hi * ldb_bytes, abort_flag);
            if (!ok) break;
          }
        }
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) { }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = make_idesc_f16(p.bf16, A_MN ? 1 : 0, B_MN ? 1 : 0, 2 * G2_BM, G2_BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
#ifdef MSQ_GEMM2_PROF
      long long prof_tempty = 0, prof_full = 0;
      const long long prof_t0 = clock64();
#endif
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++it) {
        const int buf = it & 1;
        const uint32_t acc = tmem_base + buf * G2_BN;
#ifdef MSQ_GEMM2_PROF
        const long long c0 = clock64();
#endif
        ok = mbar_wait(&tempty_bar[buf], ((it >> 1) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY);
        if (!ok) break;
#ifdef MSQ_GEMM2_PROF
        prof_tempty += clock64() - c0;
#endif
        tc_fence_after();
        for (int kb = 0; kb < k_blocks; ++kb) {
#ifdef MSQ_GEMM2_PROF
          const long long c1 = clock64();
#endif
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL);
          if (!ok) break;
#ifdef MSQ_GEMM2_PROF
          prof_full += clock64() - c1;
#endif
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * G2_A_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * G2_B_BYTES);
#pragma unroll
          for (int kk = 0; kk < G2_BK / 16; ++kk) {
            uint64_t da, db;
            if constexpr (!A_MN) da = make_smem_desc_sw128(a_addr + kk * 32, 16, 1024);
            else da = make_smem_desc_sw128(a_addr + kk * 2048, G2_BK * 128, 1024);
            if constexpr (!B_MN) db = make_smem_desc_sw128(b_addr + kk * 32, 16, 1024);
            else db = make_smem_desc_sw128(b_addr + kk * 2048, G2_BK * 128, 1024);
            tc_mma_f16_pair(acc, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit_pair(&empty_bar[stage]);  // frees this stage in both CTAs
          if (++stage == G2_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit_pair(&tfull_bar[buf]);  // accumulator ready in both CTAs
      }
#ifdef MSQ_GEMM2_PROF
      if (p.prof && pair == 0) {
        p.prof[0] = clock64() - prof_t0;
        p.prof[1] = prof_tempty;
        p.prof[2] = prof_full;
        p.prof[3] = it;
      }
#endif
    }
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs)
    const int quarter = warp & 3;
    const uint32_t leader_tempty0 = map_to_cta(smem_u32(&tempty_bar[0]), 0);
    const uint32_t leader_tempty1 = map_to_cta(smem_u32(&tempty_bar[1]), 0);
    bool ok = true;
    int it = 0;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++it) {
      int tm, tn;
      pair_tile_coords(tile, tiles_m, tiles_n, tm, tn);
      const int buf = it & 1;
      ok = mbar_wait_warp(&tfull_bar[buf], (it >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      const int row_base = tm * 2 * G2_BM + static_cast<int>(rank) * G2_BM + quarter * 32;
      const int row = row_base + lane;
      const bool row_ok = row < p.M;
      // Output path: each lane owns one row of the accumulator, so direct stores would touch 32 different
      // lines with 16 bytes each.  The packed values go through a swizzled shared-memory tile instead and
      // leave as 8 rows x 64 contiguous bytes per store instruction (full 32-byte sectors).
      uint8_t* stage = sEpi + (warp - 2) * 2048;
      const int st_row = lane >> 2, st_vec = lane & 3;
      const uint32_t taddr0 = tmem_base + buf * G2_BN + (static_cast<uint32_t>(quarter * 32) << 16);
      float rs_m = -INFINITY, rs_s = 0.f;  // this lane's row: running max and sum of exp(x - max) over the tile
#pragma unroll 1
      for (int c = 0; c < G2_BN / 32; ++c) {
        const int col0 = tn * G2_BN + c * 32;
        if (col0 >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32(taddr0 + c * 32, r);
        tmem_ld_wait();
        if (row_ok) {
          const uint16_t* crow = reinterpret_cast<const uint16_t*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int col = col0 + v * 8;
            if (col < p.N) {
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]);
              if (p.bias) {
                const uint4 bv = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.bias) + col);
                const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float2 b2 = p.bf16 ? unpack2<true>(bw[j]) : unpack2<false>(bw[j]);
                  f[2 * j] += b2.x;
                  f[2 * j + 1] += b2.y;
                }
              }
              if (p.relu) {
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = fmaxf(f[j], 0.f);
              }
              if (p.mask) {
                const uint4 mv = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.mask) +
                                                                 static_cast<long long>(row) * p.ldm + col);
                const uint32_t mw[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float2 m2 = p.bf16 ? unpack2<true>(mw[j]) : unpack2<false>(mw[j]);
                  if (!(m2.x > 0.f)) f[2 * j] = 0.f;
                  if (!(m2.y > 0.f)) f[2 * j + 1] = 0.f;
                }
              }
              if (p.residual) {
                const uint4 rv = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.residual) +
                                                                 static_cast<long long>(row) * p.ldr + col);
                const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float2 r2 = p.bf16 ? unpack2<true>(rw[j]) : unpack2<false>(rw[j]);
                  f[2 * j] += r2.x;
                  f[2 * j + 1] += r2.y;
                }
              }
              if (p.accumulate) {
                const uint4 cv = *reinterpret_cast<const uint4*>(crow + v * 8);
                const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float2 c2 = p.bf16 ? unpack2<true>(cw[j]) : unpack2<false>(cw[j]);
                  f[2 * j] += c2.x;
                  f[2 * j + 1] += c2.y;
                }
              }
              uint4 o;
              if (p.bf16) {
                o.x = pack2<true>(f[0], f[1]); o.y = pack2<true>(f[2], f[3]);
                o.z = pack2<true>(f[4], f[5]); o.w = pack2<true>(f[6], f[7]);
              } else {
                o.x = pack2<false>(f[0], f[1]); o.y = pack2<false>(f[2], f[3]);
                o.z = pack2<false>(f[4], f[5]); o.w = pack2<false>(f[6], f[7]);
              }
              *reinterpret_cast<uint4*>(stage + lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4)) = o;
              if (p.rs_max) {
                const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
                float g[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 t = p.bf16 ? unpack2<true>(ow[j]) : unpack2<false>(ow[j]);
                  g[2 * j] = t.x;
                  g[2 * j + 1] = t.y;
                }
                float vm = g[0];
#pragma unroll
                for (int j = 1; j < 8; ++j) vm = fmaxf(vm, g[j]);
                if (vm > rs_m) {
                  rs_s *= __expf(rs_m - vm);  // exp(-inf) = 0 on the first vector
                  rs_m = vm;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) rs_s += __expf(g[j] - rs_m);
              }
            }
          }
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = j * 8 + st_row;
          const int col = col0 + st_vec * 8;
          if (row_base + r < p.M && col < p.N) {
            const uint4 o = *reinterpret_cast<const uint4*>(stage + r * 64 + ((st_vec ^ ((r >> 1) & 3)) << 4));
            const int grow = row_base + r;
            if (p.scatter_world > 0) {
              const int owner = grow / p.scatter_rows;
              *reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.scatter_base[owner]) +
                                        static_cast<long long>(grow - owner * p.scatter_rows) * p.ldc + col) = o;
            } else {
              *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.C) + static_cast<long long>(grow) * p.ldc + col) = o;
            }
          }
        }
        __syncwarp();
      }
      if (p.rs_max && row_ok) {
        p.rs_max[static_cast<long long>(tn) * p.M + row] = rs_m;
        p.rs_sum[static_cast<long long>(tn) * p.M + row] = rs_s;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(buf ? leader_tempty1 : leader_tempty0);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer may still signal or read this CTA until it, too, is done
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, G2_TMEM_COLS);
  }
}

int make_tmap_2d(CUtensorMap* out, const void* base, long long rows, long long cols, long long ld, int box_rows,
                 int bf16);  // gemm_sm100.cu

static int g2_num_sms = 0;

template <bool A_MN, bool B_MN>
static int launch_gemm2(const CUtensorMap& tmA, const CUtensorMap& tmB, const Gemm2Params& p, int max_ctas,
                        cudaStream_t stream) {
  auto kern = gemm_tcgen05_2cta_kernel<A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM) != cudaSuccess) return -10;
    configured = true;
  }
  const int tiles = ((p.M + 2 * G2_BM - 1) / (2 * G2_BM)) * ((p.N + G2_BN - 1) / G2_BN);
  int pairs = g2_num_sms / 2;
  if (max_ctas > 0 && pairs > max_ctas / 2) pairs = max_ctas / 2;
  if (pairs > tiles) pairs = tiles;
  if (pairs <= 0) return 0;
  kern<<<2 * pairs, G2_THREADS, G2_SMEM, stream>>>(tmA, tmB, p);  // cluster shape comes from __cluster_dims__
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace msq

static long long* g_gemm2_prof = nullptr;
// Debug aid (builds with -DMSQ_GEMM2_PROF only; otherwise the MMA thread carries no timing code and the buffer
// stays untouched): device buffer of 4 int64 that receives, from the MMA thread of pair 0 of the next launches,
// {total cycles, cycles waiting for a free accumulator, cycles waiting for operand stages, tiles}.
extern "C" void msq_gemm2_set_prof(long long* buf) { g_gemm2_prof = buf; }

struct MsqGemmReady {
  const void* flags;
  long long b_offset, shard_bytes, chunk_bytes;
  int chunks_per_shard, skip_shard;
  unsigned epoch;
  int operand;  // 0 = B, 1 = A
};

extern "C" int msq_gemm2_ready(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                               long long ldc, int a_mn, int b_mn, int bf16, const void* bias, const void* residual,
                               long long ldr, const void* mask, long long ldm, int relu, int accumulate, int bn,
                               int max_ctas, int* status, cudaStream_t stream, const MsqGemmReady* ready);

// Same contract as msq_gemm.  Intended for M >= 256; smaller problems should use msq_gemm.
extern "C" int msq_gemm2(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                         long long ldc, int a_mn, int b_mn, int bf16, const void* bias, const void* residual,
                         long long ldr, const void* mask, long long ldm, int relu, int accumulate, int bn,
                         int max_ctas, int* status, cudaStream_t stream) {
  return msq_gemm2_ready(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, bf16, bias, residual, ldr, mask, ldm, relu,
                         accumulate, bn, max_ctas, status, stream, nullptr);
}

// msq_gemm2 whose B operand lives in a gathered buffer that peers are still filling: `ready` describes the
// arrival flags (see Gemm2Params).  This is the consumer half of the fused all-gather -> GEMM path.
static int gemm2_common(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                        long long ldc, int a_mn, int b_mn, int bf16, const void* bias, const void* residual,
                        long long ldr, const void* mask, long long ldm, int relu, int accumulate,
                        int max_ctas, int* status, cudaStream_t stream, const MsqGemmReady* ready,
                        void* const* scatter_ptrs, int scatter_world, int scatter_rows, float* rs_max = nullptr,
                        float* rs_sum = nullptr);

// Column tiles of the pair kernel for N output columns: the first dimension of the row-statistics tables.
extern "C" int msq_gemm2_tiles_n(int N) { return (N + msq::G2_BN - 1) / msq::G2_BN; }

// msq_gemm2_ready that also fills the row-statistics tables rs_max / rs_sum ([msq_gemm2_tiles_n(N), M] fp32 each):
// the producer half of cross entropy fused with the logits product.
extern "C" int msq_gemm2_rowstats(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                  long long ldb, long long ldc, int a_mn, int b_mn, int bf16, const void* bias,
                                  float* rs_max, float* rs_sum, int max_ctas, int* status, cudaStream_t stream,
                                  const MsqGemmReady* ready) {
  if (!rs_max || !rs_sum) return -4;
  return gemm2_common(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, bf16, bias, nullptr, 0, nullptr, 0, 0, 0, max_ctas,
                      status, stream, ready, nullptr, 0, 0, rs_max, rs_sum);
}

extern "C" int msq_gemm2_ready(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                               long long ldc, int a_mn, int b_mn, int bf16, const void* bias, const void* residual,
                               long long ldr, const void* mask, long long ldm, int relu, int accumulate, int bn,
                               int max_ctas, int* status, cudaStream_t stream, const MsqGemmReady* ready) {
  (void)bn;
  return gemm2_common(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, bf16, bias, residual, ldr, mask, ldm, relu, accumulate,
                      max_ctas, status, stream, ready, nullptr, 0, 0);
}

// Producer half of the fused GEMM -> reduce-scatter path: rows [r * rows_per_rank, (r+1) * rows_per_rank) of
// op(A) @ op(B) are stored into dst_ptrs[r] (peer memory, row stride ldc) instead of a local C.
extern "C" int msq_gemm2_scatter(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb,
                                 long long ldc, int a_mn, int b_mn, int bf16, void* const* dst_ptrs, int world,
                                 int rows_per_rank, int max_ctas, int* status, cudaStream_t stream) {
  if (world <= 0 || world > 16 || rows_per_rank <= 0 || static_cast<long long>(rows_per_rank) * world < M) return -7;
  for (int i = 0; i < world; ++i)
    if (reinterpret_cast<uintptr_t>(dst_ptrs[i]) & 15) return -4;
  return gemm2_common(A, B, nullptr, M, N, K, lda, ldb, ldc, a_mn, b_mn, bf16, nullptr, nullptr, 0, nullptr, 0, 0, 0,
                      max_ctas, status, stream, nullptr, dst_ptrs, world, rows_per_rank);
}

static int gemm2_common(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                        long long ldc, int a_mn, int b_mn, int bf16, const void* bias, const void* residual,
                        long long ldr, const void* mask, long long ldm, int relu, int accumulate,
                        int max_ctas, int* status, cudaStream_t stream, const MsqGemmReady* ready,
                        void* const* scatter_ptrs, int scatter_world, int scatter_rows, float* rs_max, float* rs_sum) {
  using namespace msq;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (N & 7) || (ldc & 7) || (reinterpret_cast<uintptr_t>(C) & 15)) return -4;
  if (g2_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g2_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap tmA, tmB;
  int rc;
  rc = a_mn ? make_tmap_2d(&tmA, A, K, M, lda, G2_BK, bf16) : make_tmap_2d(&tmA, A, M, K, lda, G2_BM, bf16);
  if (rc) return rc;
  rc = b_mn ? make_tmap_2d(&tmB, B, K, N, ldb, G2_BK, bf16) : make_tmap_2d(&tmB, B, N, K, ldb, G2_BN / 2, bf16);
  if (rc) return rc - 100;
  Gemm2Params p;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.bias = bias; p.residual = residual; p.ldr = ldr; p.mask = mask; p.ldm = ldm;
  p.relu = relu; p.accumulate = accumulate; p.bf16 = bf16; p.status = status;
  p.prof = g_gemm2_prof;
  p.rs_max = rs_max;
  p.rs_sum = rs_sum;
  p.scatter_world = scatter_world;
  p.scatter_rows = scatter_rows;
  for (int i = 0; i < 16; ++i) p.scatter_base[i] = (scatter_ptrs && i < scatter_world) ? scatter_ptrs[i] : nullptr;
  p.ready_flags = nullptr;
  p.ready_b_offset = p.ready_ldb_bytes = p.ready_shard_bytes = p.ready_chunk_bytes = 0;
  p.ready_chunks_per_shard = 0; p.ready_skip_shard = -1; p.ready_epoch = 0; p.ready_operand = 0;
  if (ready && ready->flags) {
    if (ready->shard_bytes <= 0 || ready->chunk_bytes <= 0 || ready->chunks_per_shard <= 0) return -6;
    p.ready_flags = static_cast<const uint32_t*>(ready->flags);
    p.ready_b_offset = ready->b_offset;
    p.ready_operand = ready->operand ? 1 : 0;
    p.ready_ldb_bytes = (ready->operand ? lda : ldb) * 2;
    p.ready_shard_bytes = ready->shard_bytes;
    p.ready_chunk_bytes = ready->chunk_bytes;
    p.ready_chunks_per_shard = ready->chunks_per_shard;
    p.ready_skip_shard = ready->skip_shard;
    p.ready_epoch = ready->epoch;
  }
  if (!a_mn && !b_mn) return launch_gemm2<false, false>(tmA, tmB, p, max_ctas, stream);
  if (!a_mn && b_mn) return launch_gemm2<false, true>(tmA, tmB, p, max_ctas, stream);
  if (a_mn && !b_mn) return launch_gemm2<true, false>(tmA, tmB, p, max_ctas, stream);
  return launch_gemm2<true, true>(tmA, tmB, p, max_ctas, stream);
}
