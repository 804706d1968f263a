// Persistent warp-specialised GEMM for sm_100a: TMA -> 128B-swizzled shared
// memory -> tcgen05.mma with the fp32 accumulator in TMEM -> fused epilogue.
//
//   C[M,N] = epilogue( op(A)[M,K] * op(B)[K,N] )
//
// Operand storage (16-bit, fp16 or bf16):
//   a_mn = 0 : A stored [M,K], K contiguous          (activations in y = x W^T)
//   a_mn = 1 : A stored [K,M], M contiguous          (dy^T in wgrad)
//   b_mn = 0 : B stored [N,K], K contiguous          (nn.Linear weight in forward)
//   b_mn = 1 : B stored [K,N], N contiguous          (weight in dgrad, x in wgrad)
// Epilogue, applied in this order on the fp32 accumulator:
//   + bias[n]  ->  ReLU  ->  * (mask[m,n] > 0)  ->  + residual[m,n]  ->  + C_old[m,n]
// This covers the linear layers of the decoder block that the reference runs as
// torch.matmul plus separate bias / ReLU / residual kernels
// (metaseq/modules/megatron/mpu/layers.py:290,323,373; metaseq/modules/feedforward.py:21-22).
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner,
// warps 2..5 = epilogue (one TMEM lane quarter each).  Two accumulator buffers in
// TMEM let the epilogue of tile i overlap the main loop of tile i+1.
#include <cstdio>

#include "sm100_common.cuh"

namespace msq {

struct GemmParams {
  int M, N, K;
  void* C;
  long long ldc;
  const void* bias;      // [N] or null
  const void* residual;  // [M, ldr] or null
  long long ldr;
  const void* mask;  // [M, ldm] or null; output is zeroed where mask <= 0
  long long ldm;
  int relu;
  int accumulate;  // add the previous contents of C
  int bf16;        // 0 = fp16, 1 = bf16
  int* status;
};

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 192;

template <int BN>
struct GemmCfg {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr uint32_t A_BYTES = BM * BK * 2;
  static constexpr uint32_t B_BYTES = BN * BK * 2;
  static constexpr uint32_t SMEM = STAGES * (A_BYTES + B_BYTES) + 1024 /*align slack*/ + 256 /*barriers*/;
  static constexpr uint32_t TMEM_COLS = 2 * BN;  // 512 or 256: a power of two >= 32
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  // Groups of 16 row-tiles sweep all column-tiles, so a wave of CTAs shares
  // B tiles and a bounded set of A tiles in L2.
  constexpr int GROUP = 16;
  const int per_group = GROUP * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP;
  const int gsize = min(GROUP, tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + (r % gsize);
  tn = r / gsize;
}

template <bool A_MN, bool B_MN, int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * Cfg::A_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sB + STAGES * Cfg::B_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (p.K + BK - 1) / BK;

  // A wait that ran out earlier on this stream left its code in the status word: do no work
  // until the host has read and cleared it (uniform per CTA, taken before any TMEM allocation).
  if (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) return;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int issued = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, ST_TIMEOUT_SMEM_EMPTY);
          if (!ok) break;
          mbar_expect_tx(&full_bar[stage], Cfg::A_BYTES + Cfg::B_BYTES);
          uint8_t* a_dst = sA + stage * Cfg::A_BYTES;
          uint8_t* b_dst = sB + stage * Cfg::B_BYTES;
          const int k0 = kb * BK;
          if constexpr (!A_MN) {
            tma_load_2d(a_dst, &tmA, &full_bar[stage], k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(a_dst + c * (BK * 128), &tmA, &full_bar[stage], m0 + c * 64, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d(b_dst, &tmB, &full_bar[stage], k0, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(b_dst + c * (BK * 128), &tmB, &full_bar[stage], n0 + c * 64, k0);
          }
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Leaving early: give the copies already issued a bounded time to land
        // before this CTA's shared memory can be handed to another CTA.
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) { }
      }
      (void)issued;
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(p.bf16, A_MN ? 1 : 0, B_MN ? 1 : 0, BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int buf = it & 1;
        const uint32_t acc = tmem_base + buf * BN;
        ok = mbar_wait(&tempty_bar[buf], ((it >> 1) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after();
        for (int kb = 0; kb < k_blocks; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * Cfg::A_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * Cfg::B_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            uint64_t da, db;
            if constexpr (!A_MN) da = make_smem_desc_sw128(a_addr + kk * 32, 16, 1024);
            else da = make_smem_desc_sw128(a_addr + kk * 2048, BK * 128, 1024);
            if constexpr (!B_MN) db = make_smem_desc_sw128(b_addr + kk * 32, 16, 1024);
            else db = make_smem_desc_sw128(b_addr + kk * 2048, BK * 128, 1024);
            tc_mma_f16(acc, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&tfull_bar[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32)
    bool ok = true;
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, tm, tn);
      const int buf = it & 1;
      ok = mbar_wait_warp(&tfull_bar[buf], (it >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      const int row = tm * BM + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr0 = tmem_base + buf * BN + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = tn * BN + c * 32;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(taddr0 + c * 32, r);
        tmem_ld_wait();
        if (row_ok) {
          uint16_t* crow = reinterpret_cast<uint16_t*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int col = col0 + v * 8;
            if (col < p.N) {  // N is a multiple of 8
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
              *reinterpret_cast<uint4*>(crow + v * 8) = o;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ------------------------------------------------------------------- host
// 2-D map over a row-major 16-bit matrix [rows, cols] with row stride `ld` elements;
// box = [box_rows, 64 columns] (128 bytes), 128-byte swizzle, zero fill out of range.
int make_tmap_2d(CUtensorMap* out, const void* base, long long rows, long long cols, long long ld, int box_rows,
                 int bf16) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15)) return -2;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
  CUresult r = encode_tiled_16bit(out, base, 2, dims, strides, box, bf16);
  if (r != CUDA_SUCCESS) {
    std::fprintf(stderr,
                 "msq_gemm: cuTensorMapEncodeTiled failed (CUresult %d): base=%p rows=%lld cols=%lld ld=%lld "
                 "box_rows=%d bf16=%d\n",
                 static_cast<int>(r), base, rows, cols, ld, box_rows, bf16);
    return -3;
  }
  return 0;
}

static int g_num_sms = 0;

template <bool A_MN, bool B_MN, int BN>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int max_ctas,
                       cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_tcgen05_kernel<A_MN, B_MN, BN>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess) return -10;
    configured = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  int grid = tiles < g_num_sms ? tiles : g_num_sms;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (grid <= 0) return 0;
  kern<<<grid, GEMM_THREADS, Cfg::SMEM, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace msq

// C entry point.  All pointers are device pointers; leading dimensions are in
// elements.  K and N must be multiples of 8 and every base pointer 16-byte
// aligned (TMA and the vector epilogue need it).  Returns 0 on a successful launch.
extern "C" int msq_gemm(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                        long long ldc, int a_mn, int b_mn, int bf16, const void* bias, const void* residual,
                        long long ldr, const void* mask, long long ldm, int relu, int accumulate, int bn,
                        int max_ctas, int* status, cudaStream_t stream) {
  using namespace msq;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (N & 7) || (ldc & 7) || (reinterpret_cast<uintptr_t>(C) & 15)) return -4;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  if (bn != 128 && bn != 256) bn = (N >= 256) ? 256 : 128;
  CUtensorMap tmA, tmB;
  int rc;
  // K-major operand: matrix [MN, K], box [tile_mn rows, 64 k].  MN-major operand:
  // matrix [K, MN], box [64 k rows, 64 mn]; one box per 64-wide chunk of the tile.
  rc = a_mn ? make_tmap_2d(&tmA, A, K, M, lda, BK, bf16) : make_tmap_2d(&tmA, A, M, K, lda, BM, bf16);
  if (rc) return rc;
  rc = b_mn ? make_tmap_2d(&tmB, B, K, N, ldb, BK, bf16) : make_tmap_2d(&tmB, B, N, K, ldb, bn, bf16);
  if (rc) return rc - 100;
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.bias = bias; p.residual = residual; p.ldr = ldr; p.mask = mask; p.ldm = ldm;
  p.relu = relu; p.accumulate = accumulate; p.bf16 = bf16; p.status = status;
#define MSQ_DISPATCH(AM, BMJ)                                                                 \
  (bn == 256 ? launch_gemm<AM, BMJ, 256>(tmA, tmB, p, max_ctas, stream)                       \
             : launch_gemm<AM, BMJ, 128>(tmA, tmB, p, max_ctas, stream))
  if (!a_mn && !b_mn) return MSQ_DISPATCH(false, false);
  if (!a_mn && b_mn) return MSQ_DISPATCH(false, true);
  if (a_mn && !b_mn) return MSQ_DISPATCH(true, false);
  return MSQ_DISPATCH(true, true);
#undef MSQ_DISPATCH
}
