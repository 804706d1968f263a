// Causal flash attention, forward and backward, on tcgen05 tensor cores with
// the score / probability tiles in TMEM and shared memory only: the [T, T]
// score matrix never reaches HBM.
//
// Replaces the reference training path that materialises scores with baddbmm,
// runs the scaled upper-triangular masked softmax kernel and a second bmm
// (metaseq/modules/multihead_attention.py:356-426,
//  metaseq/modules/megatron/fused_kernels/scaled_upper_triang_masked_softmax.h:113-330),
// and lifts that kernel's 2048-token limit.  The reference scales q and k by
// d^-1/4 each before the product; here the product is scaled once by d^-1/2,
// which is the same function in exact arithmetic.
//
// Layout: q, k, v are [B, T, H, hd] views with arbitrary row / batch strides
// (they are column slices of the fused qkv projection output); the output is
// [B, T, H*hd].  One TMA box is 128 rows x 64 columns of one head with 128-byte swizzle, and a
// tile of HD columns is HD/64 such boxes.  Two instantiations of every kernel: the plain one
// (head sizes 64 and 128, causal mask only; 3-D tensor maps: all heads' columns, token, batch)
// and the general one, which adds the masks below and head sizes that are other multiples of 8
// (80 and 96: OPT-2.7B, OPT-760M; run on the HD = 128 kernels, up to 64 on the HD = 64 ones).
// It uses 4-D maps (hd, head, token, batch): columns past hd lie outside the map's first
// dimension, so the loads fill them with zeros, which contribute nothing to Q K^T and leave
// the padded columns of O, dQ, dK, dV unused.
//
// Masks beyond causality (both optional): `doc_start[b, t]` = first position of the document
// that token t belongs to; a query attends to keys in [doc_start, t] only (the reference's
// --self-attn-doc-sep block-diagonal mask, metaseq/modules/multihead_attention.py:400-409,
// built there as a [B, T, T] tensor for the masked-softmax kernel).  Blocks that lie wholly
// before the documents of a query tile are skipped.  `alibi_slopes[h]` adds slope * key
// position to the scaled scores (metaseq/models/transformer_decoder.py:193-230).  The same physical tile serves as a
// K-major operand (rows = M or N, 64 columns = K) and as an MN-major operand
// (rows = K, 64 columns = M or N), which is what lets the backward pass reuse
// Q, dO, P and dS for the transposed products without any transposed copy.
#include "sm100_common.cuh"

namespace msq {

constexpr int ATT_THREADS = 192;      // forward: TMA warp, MMA warp, 4 softmax warps
constexpr int ATT_BWD_THREADS = 448;  // backward: TMA warp, MMA warp, 8 element-wise warps, 4 dQ-drain warps
constexpr int TILE = 128;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

// Byte offset of the 16-byte unit `unit` (0..7) of row `r` inside a
// [rows x 128 B] 128-byte-swizzled chunk.
__device__ __forceinline__ uint32_t sw128_offset(int r, int unit) {
  return static_cast<uint32_t>(r) * 128u + (static_cast<uint32_t>(unit ^ (r & 7)) << 4);
}

// One 64-column box of head `h` at token row `row`: native head sizes use the 3-D map (columns of all heads in
// one dimension, so that 256-byte L2 promotion spans neighbouring heads), other sizes the 4-D map whose first
// dimension ends at the head size and zero-fills beyond it.
__device__ __forceinline__ void attn_load_box(void* dst, const CUtensorMap* tm, uint64_t* bar, bool native, int hd,
                                              int c, int h, int row, int b) {
  if (native) tma_load_3d(dst, tm, bar, h * hd + c * 64, row, b);
  else tma_load_4d(dst, tm, bar, c * 64, h, row, b);
}
__device__ __forceinline__ void attn_reduce_box(const CUtensorMap* tm, const void* src, bool native, int hd, int col,
                                                int h, int row, int b) {
  if (native) tma_reduce_add_3d(tm, src, h * hd + col, row, b);
  else tma_reduce_add_4d(tm, src, col, h, row, b);
}

struct AttnFwdParams {
  void* out;  // [B, T, H*HD]
  long long o_row_stride, o_batch_stride;
  float* lse;  // [B, H, T]
  int T, H;
  float scale_log2;  // softmax scale * log2(e)
  int causal;
  int bf16;
  int* status;
  long long* prof;  // optional phase timestamps of CTA (0,0,0), see msq_attn_set_prof
  // attention dropout: weights are dropped with probability threshold16 / 65536 and the kept ones scaled by
  // inv_keep; the mask of element (b, h, q, k) is a hash of the seed and its index (see dropout_bits)
  uint32_t drop_threshold16;
  float inv_keep;
  unsigned long long seed;
  int hd;                     // real head size (<= HD of the kernel)
  const int* doc_start;       // [B, T] or null
  const float* alibi_slopes;  // [H] or null
  int B, n_qblocks;           // work items: one per (batch, head, q tile)
  unsigned* work;             // {next item, CTAs finished} of this launch, both zero before and after it
};

// The forward kernel is persistent: CTAs (two per SM at HD = 64) draw work items from a counter.  Item w is q tile
// n_qblocks - 1 - w % n_qblocks of (batch, head) group w / n_qblocks: the q tiles of one head run at about the same
// time (its K / V stay in L2) and the heavy ones of each head start first.
struct FwdItem {
  int qb, h, b, j0, n_kv;
};
template <bool GEN>
__device__ __forceinline__ FwdItem fwd_item(const AttnFwdParams& p, int w) {
  FwdItem it;
  const int group = w / p.n_qblocks;
  it.qb = p.n_qblocks - 1 - (w - group * p.n_qblocks);
  it.h = group % p.H;
  it.b = group / p.H;
  // With document starts the first row of the tile has the earliest start: kv blocks before it are skipped.
  it.j0 = (GEN && p.doc_start) ? p.doc_start[static_cast<long long>(it.b) * p.T + min(it.qb * TILE, p.T - 1)] / TILE : 0;
  it.n_kv = (p.causal ? (it.qb + 1) : (p.T + TILE - 1) / TILE) - it.j0;  // blocks j0 .. j0 + n_kv - 1
  return it;
}

// 2^x for a pair of x <= 8 on the FMA pipe (no special-function unit): x = n + f with n = round(x), f in [-0.5, 0.5];
// 2^f by a cubic (relative error 1.0e-4, under the rounding of the 16-bit result), scaled by adding n to the
// exponent field.  Inputs below -126 are clamped (their result is a denormal-range value that rounds to zero).
__device__ __forceinline__ void exp2_poly2(uint64_t x2, float& a, float& b) {
  const uint64_t magic2 = f2_pack(12582912.f, 12582912.f);  // 1.5 * 2^23
  const uint64_t neg_magic2 = f2_pack(-12582912.f, -12582912.f);
  const uint64_t one2 = f2_pack(1.f, 1.f);
  float x0, x1;
  f2_unpack(x2, x0, x1);
  x2 = f2_pack(fmaxf(x0, -126.f), fmaxf(x1, -126.f));
  const uint64_t t2 = f2_add(x2, magic2);
  const uint64_t f2 = f2_add(x2, f2_mul(f2_add(t2, neg_magic2), f2_pack(-1.f, -1.f)));
  uint64_t p2 = f2_fma(f2, f2_pack(0.05500893f, 0.05500893f), f2_pack(0.24221096f, 0.24221096f));
  p2 = f2_fma(p2, f2, f2_pack(0.69328293f, 0.69328293f));
  p2 = f2_fma(p2, f2, one2);
  float t0, t1, p0, p1;
  f2_unpack(t2, t0, t1);
  f2_unpack(p2, p0, p1);
  a = __int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23));
  b = __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23));
}

template <int HD>
struct FwdCfg {
  static constexpr int CHUNKS = HD / 64;
  static constexpr uint32_t TILE_BYTES = TILE * HD * 2;  // one Q/K/V tile
  static constexpr uint32_t CHUNK_BYTES = TILE * 128;    // 16 KB
  // K/V ring.  Four slots at HD = 64 also keep the footprint above a third of an SM's shared memory, so
  // at most two CTAs (2 x 256 TMEM columns) are ever co-resident and tcgen05.alloc never has to wait.
  static constexpr int SLOTS = (HD == 64) ? 4 : 3;
  static constexpr uint32_t EPI_BYTES = 4 * 2048;  // per softmax warp: a 32-row x 64-byte transposition buffer for O
  static constexpr uint32_t SMEM = TILE_BYTES * (2 + SLOTS) + EPI_BYTES + 1024 + 256;  // two Q tiles: the next item's is prefetched
  // TMEM columns: S (128 fp32), O (HD fp32), P (128 16-bit values = 64 columns)
  static constexpr uint32_t O_COL = 128;
  static constexpr uint32_t P_COL = 128 + HD;
  static constexpr uint32_t TMEM_COLS = (HD == 64) ? 256 : 512;
};

// GEN: the instantiation that also handles document starts, ALiBi and head sizes below HD (4-D tensor maps).  The
// plain instantiation carries none of that code: the softmax loop is the critical path of the kernel and its speed
// proved sensitive to the amount of code around it.
template <int HD, bool BF16, bool DROP, bool GEN>
__global__ void __launch_bounds__(ATT_THREADS, (HD == 64) ? 2 : 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const AttnFwdParams p) {
  using Cfg = FwdCfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;  // two tiles
  uint8_t* sKV = sQ + 2 * Cfg::TILE_BYTES;
  uint8_t* sEpi = sKV + Cfg::SLOTS * Cfg::TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sEpi + Cfg::EPI_BYTES);
  uint64_t* q_full = bars;        // [2]
  uint64_t* q_empty = bars + 2;   // [2]
  uint64_t* kv_full = bars + 4;
  uint64_t* kv_empty = kv_full + Cfg::SLOTS;
  uint64_t* s_full = kv_empty + Cfg::SLOTS;
  uint64_t* p_full = s_full + 1;
  uint64_t* o_full = p_full + 1;
  uint64_t* o_empty = o_full + 1;
  uint64_t* s_free = o_empty + 1;
  volatile int* work_item = reinterpret_cast<volatile int*>(s_free + 1);  // [2]: item in each Q buffer, -1 = no more
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(const_cast<int*>(work_item) + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_items = p.n_qblocks * p.H * p.B;
  const int hd = GEN ? p.hd : HD;

  if (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) return;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 5);  // the commit behind the item's last score product + one arrival per softmax warp
    }
    for (int s = 0; s < Cfg::SLOTS; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
    mbar_init(o_full, 1);
    mbar_init(o_empty, 128);
    mbar_init(s_free, 128);
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tO = tmem_base + Cfg::O_COL, tP = tmem_base + Cfg::P_COL;

  if (warp == 0) {
    if (lane == 0) {
      int slot = 0;
      uint32_t phase = 0;
      bool ok = true;
      int w = static_cast<int>(atomicAdd(p.work, 1u));
      for (int seq = 0; ok; ++seq) {
        const int qbuf = seq & 1;
        ok = mbar_wait(&q_empty[qbuf], ((seq >> 1) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_SMEM_EMPTY);
        if (!ok) break;
        if (w >= total_items) {
          work_item[qbuf] = -1;
          mbar_arrive(&q_full[qbuf]);
          break;
        }
        work_item[qbuf] = w;
        const FwdItem it = fwd_item<GEN>(p, w);
        mbar_expect_tx(&q_full[qbuf], Cfg::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < Cfg::CHUNKS; ++c)
          attn_load_box(sQ + qbuf * Cfg::TILE_BYTES + c * Cfg::CHUNK_BYTES, &tmQ, &q_full[qbuf], !GEN, hd, c, it.h,
                        it.qb * TILE, it.b);
        w = static_cast<int>(atomicAdd(p.work, 1u));  // the next item; its latency hides behind the loads below
        for (int j = 0; j < it.n_kv && ok; ++j) {
#pragma unroll 1
          for (int which = 0; which < 2; ++which) {
            ok = mbar_wait(&kv_empty[slot], phase ^ 1, abort_flag, p.status, ST_TIMEOUT_SMEM_EMPTY);
            if (!ok) break;
            mbar_expect_tx(&kv_full[slot], Cfg::TILE_BYTES);
            uint8_t* dst = sKV + slot * Cfg::TILE_BYTES;
            const CUtensorMap* tm = which ? &tmV : &tmK;
#pragma unroll
            for (int c = 0; c < Cfg::CHUNKS; ++c)
              attn_load_box(dst + c * Cfg::CHUNK_BYTES, tm, &kv_full[slot], !GEN, hd, c, it.h, (it.j0 + j) * TILE, it.b);
            if (++slot == Cfg::SLOTS) { slot = 0; phase ^= 1; }
          }
        }
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) { }
      }
    }
  } else if (warp == 1) {
    // The whole warp runs the control flow (so addresses and descriptors stay warp-uniform); one elected
    // lane issues the tensor-core instructions.  Descriptors are built once and advanced by adding the
    // byte offset >> 4 to their address field: the issue loop is the latency-critical path of the kernel.
    const bool leader = elect_one();
    const uint32_t idesc_s = make_idesc_f16(BF16 ? 1 : 0, 0, 0, TILE, TILE);
    const uint32_t idesc_o = make_idesc_f16(BF16 ? 1 : 0, 0, 1, TILE, HD);
    const uint64_t q_desc0 = make_smem_desc_sw128(smem_u32(sQ), 16, 1024);
    const uint64_t k_desc0 = make_smem_desc_sw128(smem_u32(sKV), 16, 1024);                 // K-major (S = Q K^T)
    const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(sKV), Cfg::CHUNK_BYTES, 1024);   // MN-major (O = P V)
    // Ring order is K0 V0 K1 V1 ... over all items of this CTA: tile i (K of block i/2 when even, V when odd) sits
    // in slot i % SLOTS and completes phase (i / SLOTS) & 1 of that slot's barriers.  `g` counts the blocks of the
    // items before the current one, so block j of the item is block G = g + j of the CTA, whose parity the
    // S / P / O barriers follow.
    // The score product runs one block ahead of the P V product, across item boundaries too: the first scores of
    // the next item are computed while the softmax warps finish the last block of this one and store its output.
    bool ok = true;
    int n_kv_of[2] = {0, 0};  // blocks of the item in each Q buffer
    int s_seq = 0, s_j = 0;   // the block whose scores were issued last: block s_j of item s_seq
    bool s_done = false;      // no further scores to issue
    auto issue_s = [&](int qbuf, bool last_of_item, uint32_t G) -> bool {  // scores of the CTA's block G
      const uint32_t i = 2 * G, slot = i % Cfg::SLOTS;
      if (!mbar_wait_warp(&kv_full[slot], (i / Cfg::SLOTS) & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL)) return false;
      tc_fence_after();
      if (leader) {
        const uint64_t q_desc = q_desc0 + ((qbuf * Cfg::TILE_BYTES) >> 4);
        const uint64_t k_desc = k_desc0 + ((slot * Cfg::TILE_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = ((kk >> 2) * Cfg::CHUNK_BYTES + (kk & 3) * 32) >> 4;
          tc_mma_f16(tS, q_desc + off, k_desc + off, idesc_s, kk > 0 ? 1u : 0u);
        }
        tc_commit(&kv_empty[slot]);
        tc_commit(s_full);
        if (last_of_item) tc_commit(&q_empty[qbuf]);  // the item's last use of its Q tile
      }
      __syncwarp();
      return true;
    };
    // waits for the item in Q buffer seq & 1 and records its length; false when there is none (or on a timeout)
    auto open_item = [&](int seq) -> bool {
      const int qbuf = seq & 1;
      ok = mbar_wait_warp(&q_full[qbuf], (seq >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL);
      if (!ok) return false;
      const int w = work_item[qbuf];
      if (w < 0) return false;
      n_kv_of[qbuf] = fwd_item<GEN>(p, w).n_kv;
      return true;
    };
    if (open_item(0)) {
      ok = issue_s(0, n_kv_of[0] == 1, 0);
      int p_seq = 0, p_j = 0;  // the block whose P V product comes next
      for (uint32_t G = 0; ok; ++G) {
        // scores of block G + 1, as soon as the softmax threads hold the last of S(G) in registers (a quarter of
        // the exponential pass before P(G) is complete)
        if (!s_done) {
          if (s_j + 1 < n_kv_of[s_seq & 1]) {
            ++s_j;
          } else if (open_item(s_seq + 1)) {
            ++s_seq;
            s_j = 0;
          } else {
            s_done = true;
          }
          if (!ok) break;
          if (!s_done) {
            ok = mbar_wait_warp(s_free, G & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY);
            if (!ok) break;
            ok = issue_s(s_seq & 1, s_j == n_kv_of[s_seq & 1] - 1, G + 1);
            if (!ok) break;
          }
        }
        // p_full(G): every softmax thread has written P(G) and finished any rescale of O.
        ok = mbar_wait_warp(p_full, G & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY);
        if (!ok) break;
        if (p_j == 0 && p_seq > 0) {  // the first product of an item overwrites O: the previous item's must have been read
          ok = mbar_wait_warp(o_empty, (p_seq - 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY);
          if (!ok) break;
        }
        const uint32_t i = 2 * G + 1, slot = i % Cfg::SLOTS;
        ok = mbar_wait_warp(&kv_full[slot], (i / Cfg::SLOTS) & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL);
        if (!ok) break;
        tc_fence_after();
        if (leader) {
          const uint64_t v_desc = v_desc0 + ((slot * Cfg::TILE_BYTES) >> 4);
#pragma unroll
          for (int kk = 0; kk < TILE / 16; ++kk)  // O += P V: P read from TMEM (8 columns per K = 16), O accumulated there
            tc_mma_f16_ts(tO, tP + kk * 8, v_desc + ((kk * 2048) >> 4), idesc_o, (kk > 0 || p_j > 0) ? 1u : 0u);
          tc_commit(&kv_empty[slot]);
          tc_commit(o_full);
        }
        __syncwarp();
        if (++p_j == n_kv_of[p_seq & 1]) {
          p_j = 0;
          ++p_seq;
          if (s_done && p_seq > s_seq) break;  // the last block of the last item
        }
      }
    }
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;       // row inside the q tile == TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    // m_run is the reference maximum used for P and l; it may lag the true running maximum by up to
    // RESCALE_LOG2 (so P <= 2^RESCALE_LOG2), which keeps rescales of the TMEM accumulator rare.
    constexpr float RESCALE_LOG2 = 8.f;
    bool ok = true;
    uint32_t g = 0;  // blocks of the items before the current one (see the MMA warp)
    for (int seq = 0; ok; ++seq) {
    const int qbuf = seq & 1;
    ok = mbar_wait_warp(&q_full[qbuf], (seq >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL);
    if (!ok) break;
    const int w = work_item[qbuf];
    __syncwarp();
    if (lane == 0) mbar_arrive(&q_empty[qbuf]);  // the item number has been read by this warp
    if (w < 0) break;
    const FwdItem it = fwd_item<GEN>(p, w);
    const int qb = it.qb, h = it.h, b = it.b, j0 = it.j0, n_kv = it.n_kv;
    const int* dstart = (GEN && p.doc_start) ? p.doc_start + static_cast<long long>(b) * p.T : nullptr;
    const int q_idx = qb * TILE + row;         // position in the sequence
    float m_run = -INFINITY, l_run = 0.f;
    // first pair index of this thread's row in the dropout mask: ((b*H + h)*T + q) * ceil(T/2)
    const unsigned long long drop_row =
        ((static_cast<unsigned long long>(b) * p.H + h) * p.T + q_idx) * static_cast<unsigned long long>((p.T + 1) >> 1);
    const int row_start = (GEN && dstart && q_idx < p.T) ? dstart[q_idx] : 0;  // first key this row may attend to
    const float slope2 = (GEN && p.alibi_slopes) ? p.alibi_slopes[h] * LOG2E : 0.f;
    for (int j = 0; j < n_kv && ok; ++j) {
      const uint32_t G = g + j;
      ok = mbar_wait_warp(s_full, G & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      const int ja = j0 + j;  // kv block index in the sequence
      // Columns of this block that row q_idx may attend to: [lo, limit).  Only the diagonal block of a
      // causal problem, the last block of a ragged sequence, blocks that a document start cuts and ALiBi need
      // the per-element path; every other block takes the unmasked one (uniform over the warp).
      const bool prof_on = p.prof != nullptr && row == 0 && blockIdx.x == 0 && seq == 0 && j < 32;
      if (prof_on) p.prof[j * 8 + 0] = clock64();
      const int lo = row_start - ja * TILE;
      // `general`: a document start cuts this block for some row of the warp, or ALiBi is on: the per-element path
      // then also applies the lower bound and the position bias (a separate code path, so that plain causal
      // attention pays nothing for it)
      const bool general = GEN && (p.alibi_slopes != nullptr || (dstart != nullptr && __any_sync(0xffffffffu, lo > 0)));
      const bool need_mask = (p.causal && ja == qb) || ((ja + 1) * TILE > p.T) || general;
      int limit = p.T - ja * TILE;
      if (p.causal) limit = min(limit, q_idx - ja * TILE + 1);
      limit = max(0, min(limit, TILE));
      const float bias0 = slope2 * static_cast<float>(ja * TILE);  // ALiBi: bias of column i is bias0 + slope2 * i
      // Unmasked blocks after the first take one pass over S: the exponentials use the running reference maximum
      // while the block maximum is collected alongside; only if some row of the warp outgrew the reference by more
      // than RESCALE_LOG2 (rare once a few blocks have been seen) is the block redone by the two-pass code below.
      bool one_pass_done = false;
      if (!DROP && !need_mask && j == 0 && n_kv > 1) {
        // First block of an item: the maximum of its first 32 columns serves as the reference (in a causal
        // language model the first key of the sequence, a common attention sink, is among them); should the rest of
        // the block outgrow it, the block is redone like any other.
        uint32_t r[32];
        tmem_ld_32x32(tS + lane_off, r);
        tmem_ld_wait();
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 16; ++i) m4[i & 3] = fmax3(m4[i & 3], __uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
        m_run = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;
      }
      if (!DROP && !need_mask && (j > 0 || n_kv > 1) && __all_sync(0xffffffffu, m_run != -INFINITY)) {
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        uint64_t ps2[2] = {0ull, 0ull};
        const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2), neg_m2 = f2_pack(-m_run, -m_run);
        uint32_t r[2][32];
        tmem_ld_32x32(tS + lane_off, r[0]);
        bool overflow = false;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          tmem_ld_wait();
          if (c + 1 < 4) tmem_ld_32x32(tS + lane_off + (c + 1) * 32, r[(c + 1) & 1]);
#pragma unroll
          for (int i = 0; i < 16; ++i)
            m4[i & 3] = fmax3(m4[i & 3], __uint_as_float(r[c & 1][2 * i]), __uint_as_float(r[c & 1][2 * i + 1]));
          if (c == 3) {
            const float bm = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;
            overflow = __any_sync(0xffffffffu, bm - m_run > RESCALE_LOG2);
            if (overflow) break;
            tc_fence_before();
            mbar_arrive(s_free);  // all of S(j) is in registers: the tensor pipe may write S(j+1)
          }
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float x0, x1, a, bb;
            const uint64_t xx = f2_fma(f2_pack_bits(r[c & 1][2 * i], r[c & 1][2 * i + 1]), scale2, neg_m2);
            if ((i & 3) == 3) {  // every fourth pair on the FMA pipe
              exp2_poly2(xx, a, bb);
            } else {
              f2_unpack(xx, x0, x1);
              a = exp2f(x0);
              bb = exp2f(x1);
            }
            ps2[i & 1] = f2_add(ps2[i & 1], f2_pack(a, bb));
            packed[i] = pack2<BF16>(a, bb);
          }
          if (c == 0 && j > 0) {
            // P V (j-1) must have read P before it is overwritten; it ran under the first chunk's exponentials
            ok = mbar_wait_warp(o_full, (G - 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
            if (!ok) break;
            tc_fence_after();
          }
          tmem_st_32x16(tP + lane_off + c * 16, packed);
        }
        if (!ok) break;
        if (!overflow) {
          float s0, s1, s2, s3;
          f2_unpack(ps2[0], s0, s1);
          f2_unpack(ps2[1], s2, s3);
          l_run += (s0 + s1) + (s2 + s3);
          one_pass_done = true;
        }
      }
      // The diagonal block of a causal problem, likewise in one pass: the warp that owns rows 32 q .. 32 q + 31 of
      // the tile sees chunk c < q whole, chunk q up to its own column, and nothing of the chunks behind it, which
      // it neither loads nor exponentiates.
      if (!DROP && !GEN && p.causal && ja == qb && j > 0 && (ja + 1) * TILE <= p.T &&
          __all_sync(0xffffffffu, m_run != -INFINITY)) {
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        float lsum = 0.f;
        uint64_t ps2[2] = {0ull, 0ull};
        const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2), neg_m2 = f2_pack(-m_run, -m_run);
        bool overflow = false;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t packed[16];
          if (c <= quarter) {
            uint32_t r[32];
            tmem_ld_32x32(tS + lane_off + c * 32, r);
            tmem_ld_wait();
            if (c < quarter) {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                m4[i & 3] = fmax3(m4[i & 3], __uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                float x0, x1;
                f2_unpack(f2_fma(f2_pack_bits(r[2 * i], r[2 * i + 1]), scale2, neg_m2), x0, x1);
                const float a = exp2f(x0), bb = exp2f(x1);
                ps2[i & 1] = f2_add(ps2[i & 1], f2_pack(a, bb));
                packed[i] = pack2<BF16>(a, bb);
              }
            } else {
              // columns 32 q + i of this chunk are visible to row 32 q + lane for i <= lane
              float bm = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (i <= lane) bm = fmaxf(bm, __uint_as_float(r[i]));
              overflow = __any_sync(0xffffffffu, bm * p.scale_log2 - m_run > RESCALE_LOG2);
              if (overflow) break;
              tc_fence_before();
              mbar_arrive(s_free);  // the rest of S(j) is not needed: the tensor pipe may write S(j+1)
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const float a = (2 * i <= lane) ? exp2f(fmaf(__uint_as_float(r[2 * i]), p.scale_log2, -m_run)) : 0.f;
                const float bb = (2 * i + 1 <= lane) ? exp2f(fmaf(__uint_as_float(r[2 * i + 1]), p.scale_log2, -m_run)) : 0.f;
                lsum += a + bb;
                packed[i] = pack2<BF16>(a, bb);
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) packed[i] = 0u;
          }
          if (c == 0) {
            ok = mbar_wait_warp(o_full, (G - 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
            if (!ok) break;
            tc_fence_after();
          }
          tmem_st_32x16(tP + lane_off + c * 16, packed);
        }
        if (!ok) break;
        if (!overflow) {
          float s0, s1, s2, s3;
          f2_unpack(ps2[0], s0, s1);
          f2_unpack(ps2[1], s2, s3);
          l_run += ((s0 + s1) + (s2 + s3)) + lsum;
          one_pass_done = true;
        }
      }
      if (!one_pass_done) {
      float mx;  // row maximum of this block in log2 units (scaled, biased)
      {
        // four independent running maxima keep the dependency chains short
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        uint32_t r[2][32];
        tmem_ld_32x32(tS + lane_off, r[0]);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          tmem_ld_wait();
          if (c + 1 < 4) tmem_ld_32x32(tS + lane_off + (c + 1) * 32, r[(c + 1) & 1]);
          if (GEN && general) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int col = c * 32 + i;
              if (col < limit && col >= lo)
                m4[i & 3] = fmaxf(m4[i & 3], fmaf(__uint_as_float(r[c & 1][i]), p.scale_log2,
                                                  fmaf(slope2, static_cast<float>(c * 32 + i), bias0)));
            }
          } else if (need_mask) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i < limit) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(r[c & 1][i]));
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              m4[i & 3] = fmax3(m4[i & 3], __uint_as_float(r[c & 1][2 * i]), __uint_as_float(r[c & 1][2 * i + 1]));
          }
        }
        mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        if (!general) mx *= p.scale_log2;  // the general path already works in scaled, biased units
      }
      if (prof_on) p.prof[j * 8 + 1] = clock64();
      const float m_new = fmaxf(m_run, mx);
      if (j == 0) {
        m_run = m_new;  // the first P V product overwrites O: nothing to rescale
      } else {
        // P V (j-1) was issued after S(j); it must have completed before P(j) overwrites its operand or O
        // is rescaled.  It ran under the pass above, so this wait is normally already satisfied.
        ok = mbar_wait_warp(o_full, (G - 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, m_new - m_run > RESCALE_LOG2)) {
          const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m_run - m_new);
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tO + lane_off + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32(tO + lane_off + c * 32, r);
          }
          l_run *= alpha;
          m_run = m_new;
        }
      }
      // A row with nothing to attend to yet (only rows past T) keeps m = -inf; guard the subtraction.
      const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
      float psum;
      float ps4[4] = {0.f, 0.f, 0.f, 0.f};
      uint64_t ps2[2] = {0ull, 0ull};  // packed pairs of partial sums (unmasked path)
      const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2), neg_m2 = f2_pack(-m_use, -m_use);
      {
        uint32_t r[2][32];
        tmem_ld_32x32(tS + lane_off, r[0]);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          tmem_ld_wait();
          if (c + 1 < 4) {
            tmem_ld_32x32(tS + lane_off + (c + 1) * 32, r[(c + 1) & 1]);
          } else {
            tc_fence_before();
            mbar_arrive(s_free);  // all of S(j) is in registers: the tensor pipe may write S(j+1)
          }
          uint32_t packed[16];
          if (need_mask) {
            const float off0 = bias0 - m_use;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int col = c * 32 + 2 * i;
              float a, bb;
              if (GEN && general) {
                a = (col < limit && col >= lo)
                        ? exp2f(fmaf(__uint_as_float(r[c & 1][2 * i]), p.scale_log2,
                                     fmaf(slope2, static_cast<float>(c * 32 + 2 * i), off0))) : 0.f;
                bb = (col + 1 < limit && col + 1 >= lo)
                         ? exp2f(fmaf(__uint_as_float(r[c & 1][2 * i + 1]), p.scale_log2,
                                      fmaf(slope2, static_cast<float>(c * 32 + 2 * i + 1), off0))) : 0.f;
              } else {
                a = (col < limit) ? exp2f(fmaf(__uint_as_float(r[c & 1][2 * i]), p.scale_log2, -m_use)) : 0.f;
                bb = (col + 1 < limit) ? exp2f(fmaf(__uint_as_float(r[c & 1][2 * i + 1]), p.scale_log2, -m_use)) : 0.f;
              }
              ps4[i & 3] += a + bb;
              float da = a, db = bb;
              if (DROP) {
                bool k0, k1;
                dropout_keep2(dropout_bits(p.seed, drop_row + ((ja * TILE + c * 32) >> 1) + i), p.drop_threshold16, k0, k1);
                da = k0 ? a * p.inv_keep : 0.f;
                db = k1 ? bb * p.inv_keep : 0.f;
              }
              packed[i] = pack2<BF16>(da, db);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float x0, x1;
              f2_unpack(f2_fma(f2_pack_bits(r[c & 1][2 * i], r[c & 1][2 * i + 1]), scale2, neg_m2), x0, x1);
              const float a = exp2f(x0), bb = exp2f(x1);
              ps2[i & 1] = f2_add(ps2[i & 1], f2_pack(a, bb));  // the normaliser uses the undropped weights
              float da = a, db = bb;
              if (DROP) {
                bool k0, k1;
                dropout_keep2(dropout_bits(p.seed, drop_row + ((ja * TILE + c * 32) >> 1) + i), p.drop_threshold16, k0, k1);
                da = k0 ? a * p.inv_keep : 0.f;
                db = k1 ? bb * p.inv_keep : 0.f;
              }
              packed[i] = pack2<BF16>(da, db);
            }
          }
          tmem_st_32x16(tP + lane_off + c * 16, packed);  // row = lane, two 16-bit probabilities per column
        }
      }
      {
        float s0, s1, s2, s3;
        f2_unpack(ps2[0], s0, s1);
        f2_unpack(ps2[1], s2, s3);
        psum = ((ps4[0] + ps4[1]) + (ps4[2] + ps4[3])) + ((s0 + s1) + (s2 + s3));
      }
      l_run += psum;
      }  // two-pass path
      tmem_st_wait();
      if (prof_on) p.prof[j * 8 + 2] = clock64();
      tc_fence_before();
      mbar_arrive(p_full);
    }
    if (ok) ok = mbar_wait_warp(o_full, (g + n_kv - 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
    tc_fence_after();
    if (ok) {
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      // Each lane owns one row of O, so direct stores would touch 32 lines with 16 bytes each.  The packed values go
      // through a swizzled 32-row x 64-byte buffer of this warp and leave as 8 rows x 64 contiguous bytes per store.
      uint8_t* tbuf = sEpi + quarter * 2048;
      const int st_row = lane >> 2, st_vec = lane & 3;
      const int row0 = qb * TILE + quarter * 32;
      uint16_t* obase = reinterpret_cast<uint16_t*>(p.out) + static_cast<long long>(b) * p.o_batch_stride + h * hd;
      uint32_t r[2][32];
      tmem_ld_32x32(tO + lane_off, r[0]);
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        tmem_ld_wait();
        if (c + 1 < HD / 32) {
          tmem_ld_32x32(tO + lane_off + (c + 1) * 32, r[(c + 1) & 1]);
        } else {
          tc_fence_before();
          mbar_arrive(o_empty);  // O is in registers: the next item's first product may overwrite the accumulator
        }
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 ov;
          ov.x = pack2<BF16>(__uint_as_float(r[c & 1][v * 8 + 0]) * inv_l, __uint_as_float(r[c & 1][v * 8 + 1]) * inv_l);
          ov.y = pack2<BF16>(__uint_as_float(r[c & 1][v * 8 + 2]) * inv_l, __uint_as_float(r[c & 1][v * 8 + 3]) * inv_l);
          ov.z = pack2<BF16>(__uint_as_float(r[c & 1][v * 8 + 4]) * inv_l, __uint_as_float(r[c & 1][v * 8 + 5]) * inv_l);
          ov.w = pack2<BF16>(__uint_as_float(r[c & 1][v * 8 + 6]) * inv_l, __uint_as_float(r[c & 1][v * 8 + 7]) * inv_l);
          *reinterpret_cast<uint4*>(tbuf + lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4)) = ov;
        }
        __syncwarp();
        if (!GEN || c * 32 + st_vec * 8 < hd) {  // padded columns of a head size below HD are not stored
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const int rr = jj * 8 + st_row;
            if (row0 + rr < p.T) {
              const uint4 ov = *reinterpret_cast<const uint4*>(tbuf + rr * 64 + ((st_vec ^ ((rr >> 1) & 3)) << 4));
              *reinterpret_cast<uint4*>(obase + static_cast<long long>(row0 + rr) * p.o_row_stride + c * 32 + st_vec * 8) = ov;
            }
          }
        }
        __syncwarp();
      }
      if (p.lse && q_idx < p.T) p.lse[(static_cast<long long>(b) * p.H + h) * p.T + q_idx] = (m_run + log2f(l_run)) * LN2;
    }
    g += n_kv;
    }  // items
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
  // Every CTA has drawn its last (refused) item by now; the one that finishes last leaves the counters at zero for
  // the next launch that is given this pair.
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.work + 1, 1u) == gridDim.x - 1) {
      p.work[0] = 0;
      p.work[1] = 0;
    }
  }
}


// ---------------------------------------------------------- forward, head size 128
// Two q tiles (256 rows) per work item on one CTA per SM: the tensor pipe alternates between the tiles, so that the
// score and P V products of one tile run while the softmax warps of the other tile are busy.  With 128 fp32
// columns each for S and O of both tiles the 512 TMEM columns are full: P is written over the first 64 columns of
// its own S (the columns it overwrites have been read by then), and the next score product of a tile is issued
// behind its P V product.  Warps: TMA, MMA issue, four softmax warps per tile (320 threads).  Causal masking only;
// dropout, document starts, ALiBi and padded head sizes stay on the one-tile kernel above.
constexpr int ATT128_THREADS = 320;
struct Fwd128Cfg {
  static constexpr int HD = 128;
  static constexpr int CHUNKS = 2;
  static constexpr uint32_t TILE_BYTES = TILE * HD * 2;  // 32 KB
  static constexpr uint32_t CHUNK_BYTES = TILE * 128;    // 16 KB
  static constexpr int SLOTS = 4;                        // K0 V0 K1 V1
  static constexpr uint32_t EPI_BYTES = 8 * 2048;
  static constexpr uint32_t SMEM = TILE_BYTES * (2 + SLOTS) + EPI_BYTES + 1024 + 256;
};

struct Fwd128Item {
  int qp, h, b;
  int n[2];    // kv blocks of tile 0 / 1 (0: the tile lies beyond the sequence)
  int n_iter;  // max of the two
};
__device__ __forceinline__ Fwd128Item fwd128_item(const AttnFwdParams& p, int w) {
  Fwd128Item it;
  const int group = w / p.n_qblocks;  // n_qblocks counts tile pairs for this kernel
  it.qp = p.n_qblocks - 1 - (w - group * p.n_qblocks);
  it.h = group % p.H;
  it.b = group / p.H;
  const int n_kv = (p.T + TILE - 1) / TILE;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int qb = 2 * it.qp + t;
    it.n[t] = qb * TILE < p.T ? (p.causal ? min(qb + 1, n_kv) : n_kv) : 0;
  }
  it.n_iter = max(it.n[0], it.n[1]);
  return it;
}

template <bool BF16>
__global__ void __launch_bounds__(ATT128_THREADS, 1)
flash_fwd128_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const AttnFwdParams p) {
  using Cfg = Fwd128Cfg;
  constexpr int HD = 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;  // tile 0, tile 1
  uint8_t* sKV = sQ + 2 * Cfg::TILE_BYTES;
  uint8_t* sEpi = sKV + Cfg::SLOTS * Cfg::TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sEpi + Cfg::EPI_BYTES);
  uint64_t* q_full = bars;
  uint64_t* q_empty = bars + 1;
  uint64_t* kv_full = bars + 2;
  uint64_t* kv_empty = kv_full + Cfg::SLOTS;
  uint64_t* s_full = kv_empty + Cfg::SLOTS;  // [2]
  uint64_t* p_full = s_full + 2;             // [2]
  uint64_t* o_full = p_full + 2;             // [2]
  uint64_t* o_empty = o_full + 2;            // [2]
  volatile int* work_item = reinterpret_cast<volatile int*>(o_empty + 2);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(const_cast<int*>(work_item) + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_items = p.n_qblocks * p.H * p.B;

  if (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) return;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1 + 8);  // the commit behind the item's last score product + one arrival per softmax warp
    for (int s = 0; s < Cfg::SLOTS; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 128);
      mbar_init(&o_full[t], 1);
      mbar_init(&o_empty[t], 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int slot = 0;
      uint32_t phase = 0;
      bool ok = true;
      int w = static_cast<int>(atomicAdd(p.work, 1u));
      for (int seq = 0; ok; ++seq) {
        ok = mbar_wait(q_empty, (seq & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_SMEM_EMPTY);
        if (!ok) break;
        if (w >= total_items) {
          *work_item = -1;
          mbar_arrive(q_full);
          break;
        }
        *work_item = w;
        const Fwd128Item it = fwd128_item(p, w);
        mbar_expect_tx(q_full, 2 * Cfg::TILE_BYTES);
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
          for (int c = 0; c < Cfg::CHUNKS; ++c)  // rows past the sequence are filled with zeros by the copy engine
            attn_load_box(sQ + t * Cfg::TILE_BYTES + c * Cfg::CHUNK_BYTES, &tmQ, q_full, true, HD, c, it.h,
                          (2 * it.qp + t) * TILE, it.b);
        w = static_cast<int>(atomicAdd(p.work, 1u));
        for (int j = 0; j < it.n_iter && ok; ++j) {
#pragma unroll 1
          for (int which = 0; which < 2; ++which) {
            ok = mbar_wait(&kv_empty[slot], phase ^ 1, abort_flag, p.status, ST_TIMEOUT_SMEM_EMPTY);
            if (!ok) break;
            mbar_expect_tx(&kv_full[slot], Cfg::TILE_BYTES);
            uint8_t* dst = sKV + slot * Cfg::TILE_BYTES;
            const CUtensorMap* tm = which ? &tmV : &tmK;
#pragma unroll
            for (int c = 0; c < Cfg::CHUNKS; ++c)
              attn_load_box(dst + c * Cfg::CHUNK_BYTES, tm, &kv_full[slot], true, HD, c, it.h, j * TILE, it.b);
            if (++slot == Cfg::SLOTS) { slot = 0; phase ^= 1; }
          }
        }
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) { }
      }
    }
  } else if (warp == 1) {
    const bool leader = elect_one();
    const uint32_t idesc_s = make_idesc_f16(BF16 ? 1 : 0, 0, 0, TILE, TILE);
    const uint32_t idesc_o = make_idesc_f16(BF16 ? 1 : 0, 0, 1, TILE, HD);
    const uint64_t q_desc0 = make_smem_desc_sw128(smem_u32(sQ), 16, 1024);
    const uint64_t k_desc0 = make_smem_desc_sw128(smem_u32(sKV), 16, 1024);                // K-major (S = Q K^T)
    const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(sKV), Cfg::CHUNK_BYTES, 1024);  // MN-major (O = P V)
    bool ok = true;
    uint32_t gkv = 0;             // kv blocks of the items before the current one (ring position)
    uint32_t g[2] = {0, 0};       // blocks of each tile before the current item (parity of its barriers)
    uint32_t items_of[2] = {0, 0};  // items in which each tile was active (parity of o_empty)
    for (int seq = 0; ok; ++seq) {
      ok = mbar_wait_warp(q_full, seq & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL);
      if (!ok) break;
      const int w = *work_item;
      if (w < 0) break;
      const Fwd128Item it = fwd128_item(p, w);
      // S_t (j): waits for K (j); frees it if no later product of the item reads it; the item's last score product
      // also frees the Q tiles
      auto issue_s = [&](int t, int j) -> bool {
        const uint32_t i = 2 * (gkv + j), slot = i % Cfg::SLOTS;
        if (!mbar_wait_warp(&kv_full[slot], (i / Cfg::SLOTS) & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL)) return false;
        tc_fence_after();
        if (leader) {
          const uint64_t q_desc = q_desc0 + ((t * Cfg::TILE_BYTES) >> 4);
          const uint64_t k_desc = k_desc0 + ((slot * Cfg::TILE_BYTES) >> 4);
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            const uint32_t off = ((kk >> 2) * Cfg::CHUNK_BYTES + (kk & 3) * 32) >> 4;
            tc_mma_f16(tmem_base + t * 128, q_desc + off, k_desc + off, idesc_s, kk > 0 ? 1u : 0u);
          }
          tc_commit(&s_full[t]);
          if (t == 1 || j >= it.n[1]) tc_commit(&kv_empty[slot]);  // tile 1 is the later reader when it is active
          const bool last_s = (t == 1) ? (j == it.n[1] - 1 && it.n[1] >= it.n[0]) : (j == it.n[0] - 1 && it.n[0] > it.n[1]);
          if (last_s) tc_commit(q_empty);
        }
        __syncwarp();
        return true;
      };
      for (int t = 0; t < 2 && ok; ++t)
        if (it.n[t] > 0) ok = issue_s(t, 0);
      for (int j = 0; j < it.n_iter && ok; ++j) {
#pragma unroll 1
        for (int t = 0; t < 2 && ok; ++t) {
          if (j >= it.n[t]) continue;
          // P_t (j) is in TMEM (over the first half of S_t) and any rescale of O_t is done
          ok = mbar_wait_warp(&p_full[t], (g[t] + j) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY);
          if (!ok) break;
          if (j == 0 && items_of[t] > 0) {  // the first product of an item overwrites O_t: the previous item's must have been read
            ok = mbar_wait_warp(&o_empty[t], (items_of[t] - 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY);
            if (!ok) break;
          }
          const uint32_t i = 2 * (gkv + j) + 1, slot = i % Cfg::SLOTS;
          ok = mbar_wait_warp(&kv_full[slot], (i / Cfg::SLOTS) & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL);
          if (!ok) break;
          tc_fence_after();
          if (leader) {
            const uint64_t v_desc = v_desc0 + ((slot * Cfg::TILE_BYTES) >> 4);
#pragma unroll
            for (int kk = 0; kk < TILE / 16; ++kk)
              tc_mma_f16_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + kk * 8, v_desc + ((kk * 2048) >> 4), idesc_o,
                            (kk > 0 || j > 0) ? 1u : 0u);
            tc_commit(&o_full[t]);
            if (t == 1 || j >= it.n[1]) tc_commit(&kv_empty[slot]);
          }
          __syncwarp();
          // the next scores of this tile go behind its P V product (they overwrite P); the other tile's softmax
          // runs meanwhile
          if (j + 1 < it.n[t]) ok = issue_s(t, j + 1);
        }
      }
      gkv += it.n_iter;
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        g[t] += it.n[t];
        if (it.n[t] > 0) ++items_of[t];
      }
    }
  } else {
    const int t = (warp - 2) >> 2;  // tile of this warp
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tS = tmem_base + t * 128, tO = tmem_base + 256 + t * 128, tP = tS;
    constexpr float RESCALE_LOG2 = 8.f;
    bool ok = true;
    uint32_t g = 0;
    for (int seq = 0; ok; ++seq) {
      ok = mbar_wait_warp(q_full, seq & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL);
      if (!ok) break;
      const int w = *work_item;
      __syncwarp();
      if (lane == 0) mbar_arrive(q_empty);
      if (w < 0) break;
      const Fwd128Item it = fwd128_item(p, w);
      const int n_kv = it.n[t];
      if (n_kv == 0) continue;
      const int qb = 2 * it.qp + t, h = it.h, b = it.b;
      const int q_idx = qb * TILE + row;
      float m_run = -INFINITY, l_run = 0.f;
      for (int j = 0; j < n_kv && ok; ++j) {
        const uint32_t G = g + j;
        // S (j) was issued behind P V (j - 1) of this tile: O and the P columns are free as soon as it is here
        ok = mbar_wait_warp(&s_full[t], G & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
        if (!ok) break;
        tc_fence_after();
        const bool need_mask = (p.causal && j == qb) || ((j + 1) * TILE > p.T);
        int limit = p.T - j * TILE;
        if (p.causal) limit = min(limit, q_idx - j * TILE + 1);
        limit = max(0, min(limit, TILE));
        bool done = false;
        // The diagonal tile of a causal problem (full tiles only): the warp that owns rows 32 q .. 32 q + 31 sees chunk
        // c < q whole, chunk q up to its own column and nothing behind it.
        const bool diag = p.causal && j == qb && (j + 1) * TILE <= p.T;
        if (j == 0 && n_kv > 1 && !need_mask) {
          // first block of an item: the maximum of its first 32 columns serves as the reference; should the rest of
          // the block outgrow it, the block is redone like any other
          uint32_t r0[32];
          tmem_ld_32x32(tS + lane_off, r0);
          tmem_ld_wait();
          float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int i = 0; i < 16; ++i) m4[i & 3] = fmax3(m4[i & 3], __uint_as_float(r0[2 * i]), __uint_as_float(r0[2 * i + 1]));
          m_run = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;
        }
        if ((!need_mask || (diag && j > 0)) && (j > 0 || n_kv > 1) && __all_sync(0xffffffffu, m_run != -INFINITY)) {
          // one pass: exponentials against the running reference, P kept in registers until the block maximum has
          // shown that the reference still holds (P overwrites S, so a redo must be decided before any store)
          float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
          uint64_t ps2[2] = {0ull, 0ull};
          float lsum = 0.f;
          const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2), neg_m2 = f2_pack(-m_run, -m_run);
          uint32_t r[2][32];
          uint32_t packed[4][16];
          const int last_c = diag ? quarter : 3;  // chunks behind it are invisible to this warp's rows
          tmem_ld_32x32(tS + lane_off, r[0]);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (c <= last_c) {
              tmem_ld_wait();
              if (c + 1 < 4 && c + 1 <= last_c) tmem_ld_32x32(tS + lane_off + (c + 1) * 32, r[(c + 1) & 1]);
              if (diag && c == last_c) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  const bool v0 = 2 * i <= lane, v1 = 2 * i + 1 <= lane;
                  const float e0 = __uint_as_float(r[c & 1][2 * i]), e1 = __uint_as_float(r[c & 1][2 * i + 1]);
                  if (v0) m4[i & 3] = fmaxf(m4[i & 3], e0);
                  if (v1) m4[i & 3] = fmaxf(m4[i & 3], e1);
                  const float a = v0 ? exp2f(fmaf(e0, p.scale_log2, -m_run)) : 0.f;
                  const float bb = v1 ? exp2f(fmaf(e1, p.scale_log2, -m_run)) : 0.f;
                  lsum += a + bb;
                  packed[c][i] = pack2<BF16>(a, bb);
                }
              } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  m4[i & 3] = fmax3(m4[i & 3], __uint_as_float(r[c & 1][2 * i]), __uint_as_float(r[c & 1][2 * i + 1]));
                  float x0, x1, a, bb;
                  const uint64_t xx = f2_fma(f2_pack_bits(r[c & 1][2 * i], r[c & 1][2 * i + 1]), scale2, neg_m2);
                  if ((i & 3) == 3) {
                    exp2_poly2(xx, a, bb);
                  } else {
                    f2_unpack(xx, x0, x1);
                    a = exp2f(x0);
                    bb = exp2f(x1);
                  }
                  ps2[i & 1] = f2_add(ps2[i & 1], f2_pack(a, bb));
                  packed[c][i] = pack2<BF16>(a, bb);
                }
              }
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) packed[c][i] = 0u;
            }
          }
          const float bm = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;
          if (!__any_sync(0xffffffffu, bm - m_run > RESCALE_LOG2)) {
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_st_32x16(tP + lane_off + c * 16, packed[c]);
            float s0, s1, s2, s3;
            f2_unpack(ps2[0], s0, s1);
            f2_unpack(ps2[1], s2, s3);
            l_run += ((s0 + s1) + (s2 + s3)) + lsum;
            done = true;
          }
        }
        if (!done) {
          float mx;
          {
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            uint32_t r[2][32];
            tmem_ld_32x32(tS + lane_off, r[0]);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              tmem_ld_wait();
              if (c + 1 < 4) tmem_ld_32x32(tS + lane_off + (c + 1) * 32, r[(c + 1) & 1]);
              if (need_mask) {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (c * 32 + i < limit) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(r[c & 1][i]));
              } else {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                  m4[i & 3] = fmax3(m4[i & 3], __uint_as_float(r[c & 1][2 * i]), __uint_as_float(r[c & 1][2 * i + 1]));
              }
            }
            mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;
          }
          const float m_new = fmaxf(m_run, mx);
          if (j == 0) {
            m_run = m_new;
          } else if (__any_sync(0xffffffffu, m_new - m_run > RESCALE_LOG2)) {
            const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m_run - m_new);
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
              uint32_t r[32];
              tmem_ld_32x32(tO + lane_off + c * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st_32x32(tO + lane_off + c * 32, r);
            }
            l_run *= alpha;
            m_run = m_new;
          }
          const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
          float psum = 0.f;
          uint32_t r[2][32];
          tmem_ld_32x32(tS + lane_off, r[0]);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            tmem_ld_wait();
            if (c + 1 < 4) tmem_ld_32x32(tS + lane_off + (c + 1) * 32, r[(c + 1) & 1]);
            uint32_t packed[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int col = c * 32 + 2 * i;
              const float a = (!need_mask || col < limit) ? exp2f(fmaf(__uint_as_float(r[c & 1][2 * i]), p.scale_log2, -m_use)) : 0.f;
              const float bb = (!need_mask || col + 1 < limit) ? exp2f(fmaf(__uint_as_float(r[c & 1][2 * i + 1]), p.scale_log2, -m_use)) : 0.f;
              psum += a + bb;
              packed[i] = pack2<BF16>(a, bb);
            }
            // P chunk c lands in columns 16 c .. 16 c + 15 of S, inside chunks that have already been read
            tmem_st_32x16(tP + lane_off + c * 16, packed);
          }
          l_run += psum;
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&p_full[t]);
      }
      if (ok) ok = mbar_wait_warp(&o_full[t], (g + n_kv - 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
      tc_fence_after();
      if (ok) {
        const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
        uint8_t* tbuf = sEpi + (warp - 2) * 2048;
        const int st_row = lane >> 2, st_vec = lane & 3;
        const int row0 = qb * TILE + quarter * 32;
        uint16_t* obase = reinterpret_cast<uint16_t*>(p.out) + static_cast<long long>(b) * p.o_batch_stride + h * HD;
        uint32_t r[2][32];
        tmem_ld_32x32(tO + lane_off, r[0]);
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          tmem_ld_wait();
          if (c + 1 < HD / 32) {
            tmem_ld_32x32(tO + lane_off + (c + 1) * 32, r[(c + 1) & 1]);
          } else {
            tc_fence_before();
            mbar_arrive(&o_empty[t]);
          }
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 ov;
            ov.x = pack2<BF16>(__uint_as_float(r[c & 1][v * 8 + 0]) * inv_l, __uint_as_float(r[c & 1][v * 8 + 1]) * inv_l);
            ov.y = pack2<BF16>(__uint_as_float(r[c & 1][v * 8 + 2]) * inv_l, __uint_as_float(r[c & 1][v * 8 + 3]) * inv_l);
            ov.z = pack2<BF16>(__uint_as_float(r[c & 1][v * 8 + 4]) * inv_l, __uint_as_float(r[c & 1][v * 8 + 5]) * inv_l);
            ov.w = pack2<BF16>(__uint_as_float(r[c & 1][v * 8 + 6]) * inv_l, __uint_as_float(r[c & 1][v * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(tbuf + lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4)) = ov;
          }
          __syncwarp();
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const int rr = jj * 8 + st_row;
            if (row0 + rr < p.T) {
              const uint4 ov = *reinterpret_cast<const uint4*>(tbuf + rr * 64 + ((st_vec ^ ((rr >> 1) & 3)) << 4));
              *reinterpret_cast<uint4*>(obase + static_cast<long long>(row0 + rr) * p.o_row_stride + c * 32 + st_vec * 8) = ov;
            }
          }
          __syncwarp();
        }
        if (p.lse && q_idx < p.T) p.lse[(static_cast<long long>(b) * p.H + h) * p.T + q_idx] = (m_run + log2f(l_run)) * LN2;
      }
      g += n_kv;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.work + 1, 1u) == gridDim.x - 1) {
      p.work[0] = 0;
      p.work[1] = 0;
    }
  }
}

// ------------------------------------------------------------------ backward
struct AttnBwdParams {
  const float* lse;    // [B, H, T]
  const float* delta;  // [B, H, T] rowsum(dO * O)
  float* dq_accum;     // [B, T, H*HD] fp32, zero-initialised; receives sum over kv blocks
  void* dk;            // [B, T, H, HD] view
  void* dv;
  long long dk_row_stride, dk_batch_stride, dv_row_stride, dv_batch_stride;
  int T, H;
  float scale;  // softmax scale
  int causal;
  int bf16;
  int* status;
  long long* prof;
  uint32_t drop_threshold16;
  float inv_keep;
  unsigned long long seed;
  int hd;                     // real head size (<= HD of the kernel)
  const int* doc_start;       // [B, T] or null
  const float* alibi_slopes;  // [H] or null
  int B, n_kvblocks;          // work items: one per (batch, head, kv block)
  unsigned* work;             // {next item, CTAs finished} of this launch, both zero before and after it
};

// The backward kernel is persistent too (one CTA per SM).  Item w is kv block w % n_kvblocks of (batch, head) group
// w / n_kvblocks: low blocks have the longest causal q range and are drawn first within their head.
struct BwdItem {
  int nb, h, b, m_start, n_it;
};
template <bool GEN>
__device__ __forceinline__ BwdItem bwd_item(const AttnBwdParams& p, int w) {
  BwdItem it;
  const int group = w / p.n_kvblocks;
  it.nb = w - group * p.n_kvblocks;
  it.h = group % p.H;
  it.b = group / p.H;
  const int n_q = (p.T + TILE - 1) / TILE;
  it.m_start = p.causal ? it.nb : 0;
  int m_end = n_q;
  // Document starts never decrease along the sequence: once the first row of a q tile starts after the last key of
  // this block, that tile and every later one see none of its keys.
  if (GEN && p.doc_start) {
    const int* dstart = p.doc_start + static_cast<long long>(it.b) * p.T;
    const int kv_last = it.nb * TILE + TILE - 1;
    for (int m = it.m_start + 1; m < n_q; ++m)
      if (dstart[min(m * TILE, p.T - 1)] > kv_last) { m_end = m; break; }
  }
  it.n_it = m_end - it.m_start;
  return it;
}

template <int HD>
struct BwdCfg {
  static constexpr int CHUNKS = HD / 64;
  static constexpr uint32_t TILE_BYTES = TILE * HD * 2;
  static constexpr uint32_t CHUNK_BYTES = TILE * 128;
  // Q / dO ring: a stage is released by the last products of its iteration and refilled from L2 in one to two
  // thousand cycles, about two thirds of an iteration, so three stages are needed for the refill to be early enough
  static constexpr int QSTAGES = (HD == 64) ? 3 : 1;
  static constexpr int KVBUFS = 1;
  static constexpr uint32_t P_BYTES = TILE * TILE * 2;
  static constexpr uint32_t STAGE_BYTES = 8 * 4096;  // one 32 x 32 fp32 box per element-wise warp
  static constexpr uint32_t SMEM = TILE_BYTES * (2 * KVBUFS + 2 * QSTAGES) + 2 * P_BYTES + STAGE_BYTES + 1024 + 256;
  static constexpr uint32_t TMEM_COLS = 512;
  static constexpr uint32_t S_COL = 0, DP_COL = 128, DV_COL = 256, DK_COL = 256 + HD;
  static constexpr uint32_t DQ_COL = (HD == 64) ? 384 : 0;  // HD = 128 reuses the S columns
  static constexpr bool DQ_ALIASES_S = (HD != 64);
  // At HD = 64 the last 64 columns hold dS as 16-bit values (row = q, two per column): the dQ = dS K product takes
  // its A operand from there instead of from shared memory, which is the bottleneck of this kernel.
  static constexpr bool DS_IN_TMEM = (HD == 64);
  static constexpr uint32_t DS16_COL = 448;
};

template <int HD, bool BF16, bool DROP, bool GEN>
__global__ void __launch_bounds__(ATT_BWD_THREADS, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                 const __grid_constant__ CUtensorMap tmDQ, const AttnBwdParams p) {
  using Cfg = BwdCfg<HD>;
  constexpr int QS = Cfg::QSTAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int KVB = Cfg::KVBUFS;
  uint8_t* sK = smem;                          // KVB tiles
  uint8_t* sV = sK + KVB * Cfg::TILE_BYTES;    // KVB tiles
  uint8_t* sQ = sV + KVB * Cfg::TILE_BYTES;
  uint8_t* sDO = sQ + QS * Cfg::TILE_BYTES;
  uint8_t* sP = sDO + QS * Cfg::TILE_BYTES;
  uint8_t* sDS = sP + Cfg::P_BYTES;
  uint8_t* sStage = sDS + Cfg::P_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStage + Cfg::STAGE_BYTES);
  uint64_t* kv_full = bars;              // [KVB]
  uint64_t* kv_empty = kv_full + KVB;    // [KVB]
  uint64_t* qdo_full = kv_empty + KVB;
  uint64_t* qdo_empty = qdo_full + QS;
  uint64_t* sdp_full = qdo_empty + QS;
  uint64_t* pds_full = sdp_full + 1;
  uint64_t* dq_full = pds_full + 1;
  uint64_t* dq_empty = dq_full + 1;
  uint64_t* dkv_full = dq_empty + 1;
  uint64_t* dkv_empty = dkv_full + 1;
  uint64_t* pds_free = dkv_empty + 1;
  uint64_t* sdp_free = pds_free + 1;
  uint64_t* epi_done = sdp_free + 1;
  volatile int* work_item = reinterpret_cast<volatile int*>(epi_done + 1);  // [KVB]: item in each K / V buffer, -1 = none
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(const_cast<int*>(work_item) + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_items = p.n_kvblocks * p.H * p.B;
  const int hd = GEN ? p.hd : HD;
  // readers of work_item besides the MMA warp: the element-wise warps and, when they have work, the drain warps
  constexpr int ITEM_READERS = 8 + (Cfg::DQ_ALIASES_S ? 0 : 4);

  if (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) return;

  if (threadIdx.x == 0) {
    for (int s = 0; s < KVB; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1 + ITEM_READERS);  // the commit behind the item's last products + one arrival per reader warp
    }
    for (int s = 0; s < QS; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, 256);
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, Cfg::DQ_ALIASES_S ? 256 : 128);  // drained by the element-wise warps when aliased, else by the drain warps
    mbar_init(dkv_full, 1);
    mbar_init(dkv_empty, 256);
    mbar_init(epi_done, 256);
    mbar_init(pds_free, 1);
    mbar_init(sdp_free, 256);
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
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
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int w = static_cast<int>(atomicAdd(p.work, 1u));
      for (int seq = 0; ok; ++seq) {
        const int kb = seq % KVB;
        ok = mbar_wait(&kv_empty[kb], ((seq / KVB) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_SMEM_EMPTY);
        if (!ok) break;
        if (w >= total_items) {
          work_item[kb] = -1;
          mbar_arrive(&kv_full[kb]);
          break;
        }
        work_item[kb] = w;
        const BwdItem it = bwd_item<GEN>(p, w);
        mbar_expect_tx(&kv_full[kb], 2 * Cfg::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < Cfg::CHUNKS; ++c) {
          attn_load_box(sK + kb * Cfg::TILE_BYTES + c * Cfg::CHUNK_BYTES, &tmK, &kv_full[kb], !GEN, hd, c, it.h, it.nb * TILE, it.b);
          attn_load_box(sV + kb * Cfg::TILE_BYTES + c * Cfg::CHUNK_BYTES, &tmV, &kv_full[kb], !GEN, hd, c, it.h, it.nb * TILE, it.b);
        }
        w = static_cast<int>(atomicAdd(p.work, 1u));  // the next item; its latency hides behind the loads below
        for (int i = 0; i < it.n_it && ok; ++i) {
          const int m = it.m_start + i;
          ok = mbar_wait(&qdo_empty[stage], phase ^ 1, abort_flag, p.status, ST_TIMEOUT_SMEM_EMPTY);
          if (!ok) break;
          mbar_expect_tx(&qdo_full[stage], 2 * Cfg::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < Cfg::CHUNKS; ++c) {
            attn_load_box(sQ + stage * Cfg::TILE_BYTES + c * Cfg::CHUNK_BYTES, &tmQ, &qdo_full[stage], !GEN, hd, c, it.h,
                          m * TILE, it.b);
            attn_load_box(sDO + stage * Cfg::TILE_BYTES + c * Cfg::CHUNK_BYTES, &tmDO, &qdo_full[stage], !GEN, hd, c, it.h,
                          m * TILE, it.b);
          }
          if (++stage == QS) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) { }
      }
    }
  } else if (warp == 1) {
    // Whole-warp control flow, one elected issuing lane, descriptors built once (see the forward kernel).
    const bool leader = elect_one();
    const int dt = BF16 ? 1 : 0;
    const uint32_t idesc_s = make_idesc_f16(dt, 0, 0, TILE, TILE);   // Q K^T and dO V^T
    const uint32_t idesc_t = make_idesc_f16(dt, 1, 1, TILE, HD);     // P^T dO and dS^T Q
    const uint32_t idesc_q = make_idesc_f16(dt, 0, 1, TILE, HD);     // dS K
    const uint64_t k_km0 = make_smem_desc_sw128(smem_u32(sK), 16, 1024);
    const uint64_t v_km0 = make_smem_desc_sw128(smem_u32(sV), 16, 1024);
    const uint64_t k_mn0 = make_smem_desc_sw128(smem_u32(sK), Cfg::CHUNK_BYTES, 1024);
    const uint64_t p_mn = make_smem_desc_sw128(smem_u32(sP), Cfg::CHUNK_BYTES, 1024);
    const uint64_t ds_mn = make_smem_desc_sw128(smem_u32(sDS), Cfg::CHUNK_BYTES, 1024);
    const uint64_t ds_km = make_smem_desc_sw128(smem_u32(sDS), 16, 1024);
    const uint64_t q_km0 = make_smem_desc_sw128(smem_u32(sQ), 16, 1024);
    const uint64_t q_mn0 = make_smem_desc_sw128(smem_u32(sQ), Cfg::CHUNK_BYTES, 1024);
    const uint64_t do_km0 = make_smem_desc_sw128(smem_u32(sDO), 16, 1024);
    const uint64_t do_mn0 = make_smem_desc_sw128(smem_u32(sDO), Cfg::CHUNK_BYTES, 1024);
    // Without aliasing (HD = 64) the scores of the next iteration are issued before the three gradient products
    // of this one: the element-wise warps then work on S / dP (it+1) while dQ, dV, dK (it) run on the tensor
    // pipe.  With dQ aliased onto the S columns (HD = 128) the order stays strictly sequential.
    constexpr bool PIPELINED = !Cfg::DQ_ALIASES_S;
    bool ok = true;
    uint32_t gi = 0;  // iterations of the items before the current one: iteration `it` of the item is iteration
                      // G = gi + it of the CTA, whose parity the per-iteration barriers follow; its Q / dO tiles sit in
                      // stage G % QS and complete phase (G / QS) & 1 of that stage's barriers
    for (int seq = 0; ok; ++seq) {
      const int kb = seq % KVB;
      ok = mbar_wait_warp(&kv_full[kb], (seq / KVB) & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL);
      if (!ok) break;
      const int w = work_item[kb];
      if (w < 0) break;
      const int n_it = bwd_item<GEN>(p, w).n_it;
      const uint32_t kb_off = (kb * Cfg::TILE_BYTES) >> 4;
      const uint64_t k_km = k_km0 + kb_off, v_km = v_km0 + kb_off, k_mn = k_mn0 + kb_off;
      auto issue_sdp = [&](uint32_t G) -> bool {  // S = Q K^T and dP = dO V^T of the CTA's iteration G
        const int stage = G % QS;
        if (!mbar_wait_warp(&qdo_full[stage], (G / QS) & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL)) return false;
        tc_fence_after();
        const uint32_t st_off = (stage * Cfg::TILE_BYTES) >> 4;
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            const uint32_t off = ((kk >> 2) * Cfg::CHUNK_BYTES + (kk & 3) * 32) >> 4;
            tc_mma_f16(tmem_base + Cfg::S_COL, q_km0 + st_off + off, k_km + off, idesc_s, kk > 0 ? 1u : 0u);
          }
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            const uint32_t off = ((kk >> 2) * Cfg::CHUNK_BYTES + (kk & 3) * 32) >> 4;
            tc_mma_f16(tmem_base + Cfg::DP_COL, do_km0 + st_off + off, v_km + off, idesc_s, kk > 0 ? 1u : 0u);
          }
          tc_commit(sdp_full);
        }
        __syncwarp();
        return true;
      };
      // The S / dP columns of the previous item's last iteration must be free: read into registers (pipelined), or
      // the dQ that aliases them drained (HD = 128).
      if (gi > 0) {
        ok = PIPELINED ? mbar_wait_warp(sdp_free, (gi - 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)
                       : mbar_wait_warp(dq_empty, (gi - 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY);
        if (!ok) break;
      }
      ok = issue_sdp(gi);
      for (int it = 0; it < n_it && ok; ++it) {
        const uint32_t G = gi + it;
        const int stage = G % QS;
        const uint32_t st_off = (stage * Cfg::TILE_BYTES) >> 4;
        if (PIPELINED && it + 1 < n_it) {
          // S / dP of this iteration are in the element-wise warps' registers: the next pair is computed while
          // they finish P and dS
          ok = mbar_wait_warp(sdp_free, G & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY);
          if (!ok) break;
          ok = issue_sdp(G + 1);
          if (!ok) break;
        }
        // P and dS of this iteration are in shared memory
        ok = mbar_wait_warp(pds_full, G & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY);
        if (!ok) break;
        if (G > 0) {  // dQ of the previous iteration has been drained from TMEM
          ok = mbar_wait_warp(dq_empty, (G - 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY);
          if (!ok) break;
        }
        if (it == 0 && seq > 0) {  // dK / dV of the previous item have been read out of their accumulators
          ok = mbar_wait_warp(dkv_empty, (seq - 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY);
          if (!ok) break;
        }
        tc_fence_after();
        if (leader) {
          const uint32_t acc = it > 0 ? 1u : 0u;
#pragma unroll
          for (int kk = 0; kk < TILE / 16; ++kk) {  // dQ = dS K      (K = kv rows)
            if (Cfg::DS_IN_TMEM) {
              tc_mma_f16_ts(tmem_base + Cfg::DQ_COL, tmem_base + Cfg::DS16_COL + kk * 8, k_mn + ((kk * 2048) >> 4), idesc_q,
                            kk > 0 ? 1u : 0u);
            } else {
              const uint32_t a_off = ((kk >> 2) * Cfg::CHUNK_BYTES + (kk & 3) * 32) >> 4;
              tc_mma_f16(tmem_base + Cfg::DQ_COL, ds_km + a_off, k_mn + ((kk * 2048) >> 4), idesc_q, kk > 0 ? 1u : 0u);
            }
          }
          tc_commit(dq_full);
#pragma unroll
          for (int kk = 0; kk < TILE / 16; ++kk) {  // dV += P^T dO   (K = q rows)
            const uint32_t off = (kk * 2048) >> 4;
            tc_mma_f16(tmem_base + Cfg::DV_COL, p_mn + off, do_mn0 + st_off + off, idesc_t, (kk > 0) ? 1u : acc);
          }
#pragma unroll
          for (int kk = 0; kk < TILE / 16; ++kk) {  // dK += dS^T Q
            const uint32_t off = (kk * 2048) >> 4;
            tc_mma_f16(tmem_base + Cfg::DK_COL, ds_mn + off, q_mn0 + st_off + off, idesc_t, (kk > 0) ? 1u : acc);
          }
          tc_commit(&qdo_empty[stage]);
          tc_commit(pds_free);  // P / dS in shared memory may be overwritten
          if (it == n_it - 1) {
            tc_commit(dkv_full);
            tc_commit(&kv_empty[kb]);  // the item's last use of its K / V tiles
          }
        }
        __syncwarp();
        if (!PIPELINED && it + 1 < n_it) {
          // dQ (it) lives in the S columns: it must be drained before the next scores are written there
          ok = mbar_wait_warp(dq_empty, G & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY);
          if (!ok) break;
          ok = issue_sdp(G + 1);
        }
      }
      gi += n_it;
    }
  } else if (warp >= 10) {
    // dQ drain warps (one per TMEM lane quarter): TMEM -> swizzled fp32 staging -> bulk add into dq_accum, off
    // the element-wise warps' critical path.  Idle when dQ aliases the score columns (HD = 128).
    if (!Cfg::DQ_ALIASES_S) {
      const int quarter = warp & 3;
      const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
      uint8_t* boxes = sStage + (warp - 10) * 8192;  // two 32 x 32 fp32 boxes (dQ columns 0-31 and 32-63)
      bool ok = true;
      uint32_t gi = 0;
      for (int seq = 0; ok; ++seq) {
      const int kb = seq % KVB;
      ok = mbar_wait_warp(&kv_full[kb], (seq / KVB) & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL);
      if (!ok) break;
      const int w = work_item[kb];
      __syncwarp();
      if (lane == 0) mbar_arrive(&kv_empty[kb]);  // the item number has been read by this warp
      if (w < 0) break;
      const BwdItem item = bwd_item<GEN>(p, w);
      const int n_it = item.n_it, m_start = item.m_start, h = item.h, b = item.b;
      for (int dit = 0; dit < n_it && ok; ++dit) {
        const uint32_t G = gi + dit;
        ok = mbar_wait_warp(dq_full, G & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
        if (!ok) break;
        tc_fence_after();
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(tmem_base + Cfg::DQ_COL + lane_off, r0);
        tmem_ld_32x32(tmem_base + Cfg::DQ_COL + lane_off + 32, r1);
        if (G > 0) {  // the bulk adds of the previous iteration must have read the boxes
          if (lane == 0) bulk_wait_read_all();
          __syncwarp();
        }
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(dq_empty);  // dQ is in registers: the tensor pipe may overwrite the accumulator
        uint8_t* d0 = boxes + lane * 128;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int sw = (u ^ (lane & 7)) << 4;
          *reinterpret_cast<uint4*>(d0 + sw) = make_uint4(r0[4 * u], r0[4 * u + 1], r0[4 * u + 2], r0[4 * u + 3]);
          *reinterpret_cast<uint4*>(d0 + 4096 + sw) = make_uint4(r1[4 * u], r1[4 * u + 1], r1[4 * u + 2], r1[4 * u + 3]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const int row0 = (m_start + dit) * TILE + quarter * 32;
          if (row0 < p.T) {  // rows past T inside a box are dropped by the copy engine
            attn_reduce_box(&tmDQ, boxes, !GEN, hd, 0, h, row0, b);
            if (hd > 32) attn_reduce_box(&tmDQ, boxes + 4096, !GEN, hd, 32, h, row0, b);
          }
          bulk_commit_group();
        }
      }
      gi += n_it;
      }  // items
      if (lane == 0) bulk_wait_all();  // shared memory must outlive the bulk adds that read it
    }
  } else {
    // Eight warps: warp w owns TMEM lanes / tile rows 32 * (w % 4) .. +31 (the hardware's lane window of
    // that warp) and the column half (w - 2) / 4 of every tile it reads.
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t col0 = half * 64;
    const float scale_log2 = p.scale * LOG2E;
    // dQ staging for the bulk reduce: one swizzled 32-row x 32-column fp32 box per warp
    constexpr int DQ_BOXES = HD / 64;  // boxes per warp and iteration
    uint8_t* stage_buf = sStage + (warp - 2) * 4096;
    bool ok = true;
    int staged = 0;  // bulk reduces issued so far from this warp's staging box
    uint32_t gi = 0;  // iterations of the items before the current one (see the MMA warp)
    for (int seq = 0; ok; ++seq) {
    const int kb = seq % KVB;
    ok = mbar_wait_warp(&kv_full[kb], (seq / KVB) & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL);
    if (!ok) break;
    const int w = work_item[kb];
    __syncwarp();
    if (lane == 0) mbar_arrive(&kv_empty[kb]);  // the item number has been read by this warp
    if (w < 0) break;
    const BwdItem item = bwd_item<GEN>(p, w);
    const int nb = item.nb, h = item.h, b = item.b, m_start = item.m_start, n_it = item.n_it;
    const int* dstart = (GEN && p.doc_start) ? p.doc_start + static_cast<long long>(b) * p.T : nullptr;
    const long long bh = static_cast<long long>(b) * p.H + h;
    // dQ tile of the CTA's iteration G (q tile dm): TMEM -> swizzled fp32 staging -> one bulk add per 32 x 32 box
    auto drain_dq = [&](uint32_t G, int dm) -> bool {
      if (!mbar_wait_warp(dq_full, G & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) return false;
      tc_fence_after();
      const bool rows_in_range = dm * TILE + quarter * 32 < p.T;  // rows past T inside a box are dropped by the copy engine
#pragma unroll
      for (int c = 0; c < DQ_BOXES; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + Cfg::DQ_COL + lane_off + half * (HD / 2) + c * 32, r);
        if (staged > 0) {  // the previous bulk add must have read the staging box
          if (lane == 0) bulk_wait_read_all();
          __syncwarp();
        }
        tmem_ld_wait();
        uint8_t* dst = stage_buf + lane * 128;
#pragma unroll
        for (int u = 0; u < 8; ++u)
          *reinterpret_cast<uint4*>(dst + ((u ^ (lane & 7)) << 4)) = make_uint4(r[4 * u], r[4 * u + 1], r[4 * u + 2], r[4 * u + 3]);
        if (c == DQ_BOXES - 1) {
          tc_fence_before();
          mbar_arrive(dq_empty);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          // a box that starts in the padded columns of a smaller head is dropped; one that straddles the end
          // of the head is clipped by the copy engine
          if (rows_in_range && half * (HD / 2) + c * 32 < hd)
            attn_reduce_box(&tmDQ, stage_buf, !GEN, hd, half * (HD / 2) + c * 32, h, dm * TILE + quarter * 32, b);
          bulk_commit_group();
        }
        ++staged;
      }
      return true;
    };
    // the row statistics of an iteration are fetched one iteration ahead: their latency would otherwise sit in front
    // of every iteration
    float lse_next = 0.f, delta_next = 0.f;
    if (m_start * TILE + row < p.T) {
      lse_next = p.lse[bh * p.T + m_start * TILE + row];
      delta_next = p.delta[bh * p.T + m_start * TILE + row];
    }
    for (int it = 0; it < n_it && ok; ++it) {
      const int m = m_start + it;
      const int q_idx = m * TILE + row;
      const bool q_ok = q_idx < p.T;
      const float lse_raw = lse_next, delta = delta_next;
      if (it + 1 < n_it && q_idx + TILE < p.T) {
        lse_next = p.lse[bh * p.T + q_idx + TILE];
        delta_next = p.delta[bh * p.T + q_idx + TILE];
      } else {
        lse_next = 0.f;
        delta_next = 0.f;
      }
      const float lse2 = lse_raw * LOG2E;
      int limit = p.T - nb * TILE;
      if (p.causal) limit = min(limit, q_idx - nb * TILE + 1);
      limit = q_ok ? max(0, min(limit, TILE)) : 0;
      const int lo = (GEN && dstart && q_ok) ? dstart[q_idx] - nb * TILE : 0;  // keys before the row's document are masked
      const float slope2 = (GEN && p.alibi_slopes) ? p.alibi_slopes[h] * LOG2E : 0.f;
      // uniform over the warp: only diagonal blocks, ragged tails (rows or columns past T), blocks cut by a
      // document start and ALiBi need the per-element path
      const bool general = GEN && (p.alibi_slopes != nullptr || (dstart != nullptr && __any_sync(0xffffffffu, lo > 0)));
      const bool need_mask = (p.causal && m == nb) || ((m + 1) * TILE > p.T) || ((nb + 1) * TILE > p.T) || general;
      const uint32_t G = gi + it;
      ok = mbar_wait_warp(sdp_full, G & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      // P and dS of this thread's 64 columns, kept in registers until shared memory is free to take them
      uint32_t pp[2][16], dd[2][16];
      {
        uint32_t s[32], dp[32];
        tmem_ld_32x32(tmem_base + Cfg::S_COL + lane_off + col0, s);
        tmem_ld_32x32(tmem_base + Cfg::DP_COL + lane_off + col0, dp);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          tmem_ld_wait();
          if (c == 1) {
            tc_fence_before();
            mbar_arrive(sdp_free);  // S and dP of this iteration are in registers
          }
          const int cbase = col0 + c * 32;
          if (need_mask || DROP) {
            // general path: per-element bounds and, with dropout, the keep factor of each weight.  dV uses the
            // dropped and rescaled weights; dS = P * (keep / (1-p) * dP - delta) * scale.
            const unsigned long long drop_row =
                ((static_cast<unsigned long long>(b) * p.H + h) * p.T + (q_ok ? q_idx : 0)) *
                    static_cast<unsigned long long>((p.T + 1) >> 1) + ((nb * TILE + cbase) >> 1);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float p0 = 0.f, p1 = 0.f, d0 = 0.f, d1 = 0.f, ks0 = 1.f, ks1 = 1.f;
              if (DROP) {
                bool k0, k1;
                dropout_keep2(dropout_bits(p.seed, drop_row + i), p.drop_threshold16, k0, k1);
                ks0 = k0 ? p.inv_keep : 0.f;
                ks1 = k1 ? p.inv_keep : 0.f;
              }
              const int col = cbase + 2 * i;
              // plain causal / ragged blocks: lo <= 0 for every row and the bias is zero, so the extra terms fold away
              const float b0 = (GEN && general) ? fmaf(slope2, static_cast<float>(nb * TILE + col), -lse2) : -lse2;
              const float b1 = (GEN && general) ? b0 + slope2 : -lse2;
              if (col < limit && (!(GEN && general) || col >= lo)) {
                p0 = exp2f(fmaf(__uint_as_float(s[2 * i]), scale_log2, b0));
                d0 = p0 * (ks0 * __uint_as_float(dp[2 * i]) - delta) * p.scale;
                p0 *= ks0;
              }
              if (col + 1 < limit && (!(GEN && general) || col + 1 >= lo)) {
                p1 = exp2f(fmaf(__uint_as_float(s[2 * i + 1]), scale_log2, b1));
                d1 = p1 * (ks1 * __uint_as_float(dp[2 * i + 1]) - delta) * p.scale;
                p1 *= ks1;
              }
              pp[c][i] = pack2<BF16>(p0, p1);
              dd[c][i] = pack2<BF16>(d0, d1);
            }
          } else {
            const float nds = -delta * p.scale;
            const uint64_t sl2 = f2_pack(scale_log2, scale_log2), nl2 = f2_pack(-lse2, -lse2);
            const uint64_t sc2 = f2_pack(p.scale, p.scale), nds2 = f2_pack(nds, nds);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float x0, x1, d0, d1;
              f2_unpack(f2_fma(f2_pack_bits(s[2 * i], s[2 * i + 1]), sl2, nl2), x0, x1);
              const float p0 = exp2f(x0), p1 = exp2f(x1);
              const uint64_t g = f2_fma(f2_pack_bits(dp[2 * i], dp[2 * i + 1]), sc2, nds2);
              f2_unpack(f2_mul(f2_pack(p0, p1), g), d0, d1);
              pp[c][i] = pack2<BF16>(p0, p1);
              dd[c][i] = pack2<BF16>(d0, d1);
            }
          }
          if (c == 0) {
            tmem_ld_32x32(tmem_base + Cfg::S_COL + lane_off + col0 + 32, s);
            tmem_ld_32x32(tmem_base + Cfg::DP_COL + lane_off + col0 + 32, dp);
          }
        }
      }
      if (G > 0) {
        // the products of the previous iteration that read P / dS from shared memory have completed
        ok = mbar_wait_warp(pds_free, (G - 1) & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_EMPTY);
        if (!ok) break;
      }
      if (Cfg::DS_IN_TMEM) {
        // pds_free (G - 1) above also covers the dQ product of the previous iteration, the reader of these columns
#pragma unroll
        for (int c = 0; c < 2; ++c) tmem_st_32x16(tmem_base + Cfg::DS16_COL + lane_off + half * 32 + c * 16, dd[c]);
      }
      {
        const uint32_t chunk_off = half * Cfg::CHUNK_BYTES;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const uint32_t off = chunk_off + sw128_offset(row, c * 4 + u);
            *reinterpret_cast<uint4*>(sP + off) = make_uint4(pp[c][4 * u], pp[c][4 * u + 1], pp[c][4 * u + 2], pp[c][4 * u + 3]);
            *reinterpret_cast<uint4*>(sDS + off) = make_uint4(dd[c][4 * u], dd[c][4 * u + 1], dd[c][4 * u + 2], dd[c][4 * u + 3]);
          }
        }
      }
      if (Cfg::DS_IN_TMEM) tmem_st_wait();
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(pds_full);
      // With aliasing (HD = 128) dQ (it) is drained here, before the next scores overwrite its columns; otherwise
      // the drain warps take care of it concurrently.
      if (Cfg::DQ_ALIASES_S) {
        ok = drain_dq(G, m);
        if (!ok) break;
      }
    }
    // dK / dV of this kv block are complete when the products of the last iteration have been committed.
    if (ok) ok = mbar_wait_warp(dkv_full, seq & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
    tc_fence_after();
    if (ok) {
      // The TMEM loads are warp-wide (.sync.aligned): every lane runs them; only the
      // global stores are predicated on the row being inside the sequence.
      // Each lane owns one row of the accumulators, so direct stores would touch 32 lines with 16 bytes each.  The
      // packed values go through a swizzled 32 x 64-byte tile of shared memory instead (this warp's 4 KB of the P
      // tile, idle until the next item's first iteration) and leave as 8 rows x 64 contiguous bytes per instruction.
      uint8_t* tbuf = sP + (warp - 2) * 4096;
      const int st_row = lane >> 2, st_vec = lane & 3;
      const int row0 = nb * TILE + quarter * 32;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        uint16_t* base = reinterpret_cast<uint16_t*>(which ? p.dv : p.dk) +
                         static_cast<long long>(b) * (which ? p.dv_batch_stride : p.dk_batch_stride) + h * hd + half * (HD / 2);
        const long long rs = which ? p.dv_row_stride : p.dk_row_stride;
        const uint32_t col = (which ? Cfg::DV_COL : Cfg::DK_COL) + half * (HD / 2);
#pragma unroll 1
        for (int c = 0; c < HD / 64; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + col + lane_off + c * 32, r);
          tmem_ld_wait();
          if (which == 1 && c == HD / 64 - 1) {
            tc_fence_before();
            mbar_arrive(dkv_empty);  // the accumulators are in registers: the next item's products may overwrite them
          }
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 ov;
            ov.x = pack2<BF16>(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
            ov.y = pack2<BF16>(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
            ov.z = pack2<BF16>(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
            ov.w = pack2<BF16>(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
            *reinterpret_cast<uint4*>(tbuf + lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4)) = ov;
          }
          __syncwarp();
          const int colh = half * (HD / 2) + c * 32 + st_vec * 8;  // first of this lane's 8 columns inside the head
          if (!GEN || colh < hd) {
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              const int rr = jj * 8 + st_row;
              if (row0 + rr < p.T) {
                const uint4 ov = *reinterpret_cast<const uint4*>(tbuf + rr * 64 + ((st_vec ^ ((rr >> 1) & 3)) << 4));
                *reinterpret_cast<uint4*>(base + static_cast<long long>(row0 + rr) * rs + c * 32 + st_vec * 8) = ov;
              }
            }
          }
          __syncwarp();
        }
      }
    }
    // the transposition buffers are part of the P tile: every warp must be done with its own before any warp
    // writes P of the next item
    if (ok) {
      mbar_arrive(epi_done);
      ok = mbar_wait_warp(epi_done, seq & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_EMPTY);
    }
    gi += n_it;
    }  // items
    // shared memory must outlive the bulk reduces that read it
    if (lane == 0) bulk_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
  // Every CTA has drawn its last (refused) item by now; the one that finishes last leaves the counters at zero for
  // the next launch that is given this pair.
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.work + 1, 1u) == gridDim.x - 1) {
      p.work[0] = 0;
      p.work[1] = 0;
    }
  }
}

// delta[b, h, t] = sum_d dO[b, t, h, d] * O[b, t, h, d].  LPG (a power of two >= hd / 8) adjacent lanes own one
// (b, t, h) row and load 16 bytes each where they fall inside the head, so a warp reads contiguous runs of a token
// row from each tensor.
template <bool BF16, int LPG>
__global__ void __launch_bounds__(256)
attn_delta_kernel(const uint16_t* __restrict__ o, const uint16_t* __restrict__ d_o, long long row_stride,
                  long long batch_stride, float* __restrict__ delta, int B, int T, int H, int hd) {
  const long long gt = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long item = gt / LPG;
  const int sub = static_cast<int>(gt % LPG);
  const long long total = static_cast<long long>(B) * T * H;
  float s = 0.f;
  int hh = 0, t = 0, bb = 0;
  if (item < total) {
    hh = static_cast<int>(item % H);
    const long long bt = item / H;
    t = static_cast<int>(bt % T);
    bb = static_cast<int>(bt / T);
    if (sub * 8 < hd) {
      const long long off = static_cast<long long>(bb) * batch_stride + static_cast<long long>(t) * row_stride + hh * hd + sub * 8;
      const uint4 a = *reinterpret_cast<const uint4*>(o + off);
      const uint4 g = *reinterpret_cast<const uint4*>(d_o + off);
      const uint32_t av[4] = {a.x, a.y, a.z, a.w}, gv[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 x = unpack2<BF16>(av[i]);
        const float2 y = unpack2<BF16>(gv[i]);
        s += x.x * y.x + x.y * y.y;
      }
    }
  }
#pragma unroll
  for (int m = LPG / 2; m > 0; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
  if (item < total && sub == 0) delta[(static_cast<long long>(bb) * H + hh) * T + t] = s;
}

// ---------------------------------------------------------------------- host
// [B, T, H, hd] view with the given token / batch strides (elements) as a 4-D map (hd, H, T, B); box = 64 columns of
// one head x 128 rows.  Columns past hd are outside the first dimension: loads fill them with zeros.
static int make_tmap_bthd(CUtensorMap* out, const void* base, int B, int T, int H, int hd, long long row_stride,
                          long long batch_stride, int bf16, bool four_d) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((row_stride * 2) & 15) || ((batch_stride * 2) & 15) || (hd & 7)) return -2;
  if (!four_d) {  // plain instantiation: [B, T, H * hd] with all heads' columns in the first dimension
    cuuint64_t dims3[3] = {static_cast<cuuint64_t>(H) * hd, static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(B)};
    cuuint64_t strides3[2] = {static_cast<cuuint64_t>(row_stride) * 2, static_cast<cuuint64_t>(batch_stride) * 2};
    cuuint32_t box3[3] = {64u, static_cast<cuuint32_t>(TILE), 1u};
    return encode_tiled_16bit(out, base, 3, dims3, strides3, box3, bf16) == CUDA_SUCCESS ? 0 : -3;
  }
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(hd), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(T),
                        static_cast<cuuint64_t>(B)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(hd) * 2, static_cast<cuuint64_t>(row_stride) * 2,
                           static_cast<cuuint64_t>(batch_stride) * 2};
  cuuint32_t box[4] = {64u, 1u, static_cast<cuuint32_t>(TILE), 1u};
  return encode_tiled_16bit(out, base, 4, dims, strides, box, bf16) == CUDA_SUCCESS ? 0 : -3;
}

// Work counters of the persistent forward kernel: a pool of {next item, CTAs finished} pairs handed to launches in
// rotation, so that launches which overlap on a device (different streams) do not share a pair.  Zero at module
// load; every launch leaves its pair at zero.
constexpr int ATT_WORK_PAIRS = 64;
__device__ unsigned g_attn_work[2 * ATT_WORK_PAIRS];

static unsigned* next_work_pair() {
  static unsigned* base[64] = {nullptr};
  static unsigned seq = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!base[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_attn_work) != cudaSuccess) return nullptr;
    base[dev] = static_cast<unsigned*>(ptr);
  }
  return base[dev] + 2 * (seq++ % ATT_WORK_PAIRS);
}

template <int HD, bool BF16, bool DROP, bool GEN>
static int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, AttnFwdParams p,
                      int B, cudaStream_t stream) {
  auto kern = flash_fwd_kernel<HD, BF16, DROP, GEN>;
  static bool configured = false;
  static int sms = 0;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdCfg<HD>::SMEM) != cudaSuccess)
      return -10;
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return -10;
    configured = true;
  }
  p.B = B;
  p.n_qblocks = (p.T + TILE - 1) / TILE;
  p.work = next_work_pair();
  if (!p.work) return -10;
  const long long items = static_cast<long long>(p.n_qblocks) * p.H * B;
  if (items > 0x7fffffffLL - 4096) return -2;
  const long long resident = static_cast<long long>(sms) * ((HD == 64) ? 2 : 1);
  const unsigned grid = static_cast<unsigned>(items < resident ? items : resident);
  kern<<<grid, ATT_THREADS, FwdCfg<HD>::SMEM, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

template <bool BF16>
static int launch_fwd128(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, AttnFwdParams p, int B,
                         cudaStream_t stream) {
  auto kern = flash_fwd128_kernel<BF16>;
  static bool configured = false;
  static int sms = 0;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd128Cfg::SMEM) != cudaSuccess) return -10;
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return -10;
    configured = true;
  }
  p.B = B;
  p.n_qblocks = (p.T + 2 * TILE - 1) / (2 * TILE);  // tile pairs
  p.work = next_work_pair();
  if (!p.work) return -10;
  const long long items = static_cast<long long>(p.n_qblocks) * p.H * B;
  if (items > 0x7fffffffLL - 4096) return -2;
  const unsigned grid = static_cast<unsigned>(items < sms ? items : sms);
  kern<<<grid, ATT128_THREADS, Fwd128Cfg::SMEM, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

template <int HD, bool BF16, bool DROP, bool GEN>
static int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                      const CUtensorMap& tdq, AttnBwdParams p, int B, cudaStream_t stream) {
  auto kern = flash_bwd_kernel<HD, BF16, DROP, GEN>;
  static bool configured = false;
  static int sms = 0;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdCfg<HD>::SMEM) != cudaSuccess)
      return -10;
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return -10;
    configured = true;
  }
  p.B = B;
  p.n_kvblocks = (p.T + TILE - 1) / TILE;
  p.work = next_work_pair();
  if (!p.work) return -10;
  const long long items = static_cast<long long>(p.n_kvblocks) * p.H * B;
  if (items > 0x7fffffffLL - 4096) return -2;
  const unsigned grid = static_cast<unsigned>(items < sms ? items : sms);  // one CTA per SM (512 TMEM columns each)
  kern<<<grid, ATT_BWD_THREADS, BwdCfg<HD>::SMEM, stream>>>(tq, tk, tv, tdo, tdq, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Dropout threshold (16 bits) and keep scale for a probability; false when the probability is out of range.
static bool drop_params(float p, uint32_t& threshold16, float& inv_keep) {
  threshold16 = 0u;
  inv_keep = 1.f;
  if (p < 0.f || p >= 1.f) return false;
  threshold16 = static_cast<uint32_t>(p * 65536.f + 0.5f);
  inv_keep = 1.f / (1.f - static_cast<float>(threshold16) / 65536.f);
  return true;
}

}  // namespace msq

static long long* g_attn_prof = nullptr;
static int g_fwd128 = 1;
// Benchmark switch: 0 sends head size 128 through the one-tile forward kernel.
extern "C" void msq_attn_set_fwd128(int on) { g_fwd128 = on; }

// Debug aid: when set to a device buffer of at least 512 int64, CTA (0,0,0) of the next attention
// launches records clock64() at its phase boundaries (forward in [0,256), backward in [256,512)).
extern "C" void msq_attn_set_prof(long long* buf) { g_attn_prof = buf; }

// Head sizes the kernels take: a multiple of 8 up to 128 (64 and 128 exactly; others zero-padded to the next of them).
extern "C" int msq_flash_head_dim_ok(int HD) { return HD >= 8 && HD <= 128 && (HD & 7) == 0; }

// q, k, v: 16-bit [B, T, H, HD] views; *_rs / *_bs are row (token) and batch strides in
// elements.  out: [B, T, H*HD] with its own strides.  lse: fp32 [B, H, T].
// doc_start: int32 [B, T] first position of each token's document, or null (needs `causal`).
// alibi_slopes: fp32 [H] or null.  dropout_p / seed: attention dropout (0 = off); the backward call of the same
// forward must get the same two values.
extern "C" int msq_flash_fwd(const void* q, const void* k, const void* v, long long q_rs, long long q_bs,
                             long long k_rs, long long k_bs, long long v_rs, long long v_bs, void* out,
                             long long o_rs, long long o_bs, float* lse, int B, int T, int H, int HD, float scale,
                             int causal, int bf16, const int* doc_start, const float* alibi_slopes, float dropout_p,
                             unsigned long long seed, int* status, cudaStream_t stream) {
  using namespace msq;
  if (B <= 0 || T <= 0) return 0;
  if (!msq_flash_head_dim_ok(HD)) return -4;
  if (doc_start && !causal) return -6;
  if ((reinterpret_cast<uintptr_t>(out) & 15) || (o_rs & 7) || (o_bs & 7)) return -2;
  CUtensorMap tq, tk, tv;
  int rc;
  const bool gen = doc_start != nullptr || alibi_slopes != nullptr || (HD != 64 && HD != 128);
  if ((rc = make_tmap_bthd(&tq, q, B, T, H, HD, q_rs, q_bs, bf16, gen))) return rc;
  if ((rc = make_tmap_bthd(&tk, k, B, T, H, HD, k_rs, k_bs, bf16, gen))) return rc;
  if ((rc = make_tmap_bthd(&tv, v, B, T, H, HD, v_rs, v_bs, bf16, gen))) return rc;
  AttnFwdParams p;
  p.out = out; p.o_row_stride = o_rs; p.o_batch_stride = o_bs; p.lse = lse;
  p.T = T; p.H = H; p.scale_log2 = scale * LOG2E; p.causal = causal; p.bf16 = bf16; p.status = status;
  p.prof = g_attn_prof;
  p.hd = HD; p.doc_start = doc_start; p.alibi_slopes = alibi_slopes;
  if (!drop_params(dropout_p, p.drop_threshold16, p.inv_keep)) return -2;
  p.seed = seed;
#define MSQ_FWD2(HDV, BF, GN) \
  (p.drop_threshold16 ? launch_fwd<HDV, BF, true, GN>(tq, tk, tv, p, B, stream) : launch_fwd<HDV, BF, false, GN>(tq, tk, tv, p, B, stream))
#define MSQ_FWD(HDV, BF) (gen ? MSQ_FWD2(HDV, BF, true) : MSQ_FWD2(HDV, BF, false))
  if (HD <= 64) return bf16 ? MSQ_FWD(64, true) : MSQ_FWD(64, false);
  if (HD == 128 && !gen && !p.drop_threshold16 && g_fwd128)  // two q tiles per CTA (see flash_fwd128_kernel)
    return bf16 ? launch_fwd128<true>(tq, tk, tv, p, B, stream) : launch_fwd128<false>(tq, tk, tv, p, B, stream);
  return bf16 ? MSQ_FWD(128, true) : MSQ_FWD(128, false);
#undef MSQ_FWD
#undef MSQ_FWD2
}

// delta: fp32 [B, H, T] scratch (written here); dq_accum: fp32 [B, T, H*HD], zeroed by the caller.
extern "C" int msq_flash_bwd(const void* q, const void* k, const void* v, const void* out, const void* d_out,
                             long long q_rs, long long q_bs, long long k_rs, long long k_bs, long long v_rs,
                             long long v_bs, long long o_rs, long long o_bs, long long do_rs, long long do_bs,
                             const float* lse, float* delta, float* dq_accum, void* dk, void* dv, long long dk_rs,
                             long long dk_bs, long long dv_rs, long long dv_bs, int B, int T, int H, int HD,
                             float scale, int causal, int bf16, const int* doc_start, const float* alibi_slopes,
                             float dropout_p, unsigned long long seed, int* status, cudaStream_t stream) {
  using namespace msq;
  if (B <= 0 || T <= 0) return 0;
  if (!msq_flash_head_dim_ok(HD)) return -4;
  if (doc_start && !causal) return -6;
  if (o_rs != do_rs || o_bs != do_bs) return -5;
  if ((dk_rs & 7) || (dk_bs & 7) || (dv_rs & 7) || (dv_bs & 7)) return -2;
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  const bool gen = doc_start != nullptr || alibi_slopes != nullptr || (HD != 64 && HD != 128);
  if ((rc = make_tmap_bthd(&tq, q, B, T, H, HD, q_rs, q_bs, bf16, gen))) return rc;
  if ((rc = make_tmap_bthd(&tk, k, B, T, H, HD, k_rs, k_bs, bf16, gen))) return rc;
  if ((rc = make_tmap_bthd(&tv, v, B, T, H, HD, v_rs, v_bs, bf16, gen))) return rc;
  if ((rc = make_tmap_bthd(&tdo, d_out, B, T, H, HD, do_rs, do_bs, bf16, gen))) return rc;
  CUtensorMap tdq;
  {
    // fp32 [B, T, H, HD] accumulator as a 4-D map (HD, H, T, B), reduced into by 32-row x 32-column boxes of one head
    if (reinterpret_cast<uintptr_t>(dq_accum) & 15) return -2;
    const cuuint64_t cols = static_cast<cuuint64_t>(H) * HD;
    if (!gen) {
      cuuint64_t dims3[3] = {cols, static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(B)};
      cuuint64_t strides3[2] = {cols * 4, cols * 4 * static_cast<cuuint64_t>(T)};
      cuuint32_t box3[3] = {32u, 32u, 1u};
      if (encode_tiled(&tdq, dq_accum, 3, dims3, strides3, box3, CU_TENSOR_MAP_DATA_TYPE_FLOAT32) != CUDA_SUCCESS) return -3;
    } else {
      cuuint64_t dims[4] = {static_cast<cuuint64_t>(HD), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(T),
                            static_cast<cuuint64_t>(B)};
      cuuint64_t strides[3] = {static_cast<cuuint64_t>(HD) * 4, cols * 4, cols * 4 * static_cast<cuuint64_t>(T)};
      cuuint32_t box[4] = {32u, 1u, 32u, 1u};
      if (encode_tiled(&tdq, dq_accum, 4, dims, strides, box, CU_TENSOR_MAP_DATA_TYPE_FLOAT32) != CUDA_SUCCESS) return -3;
    }
  }
  {
    const int lpg = HD <= 64 ? 8 : 16;  // lanes per (b, t, h) row
    const long long nthreads = static_cast<long long>(B) * T * H * lpg;
    const int threads = 256;
    const unsigned blocks = static_cast<unsigned>((nthreads + threads - 1) / threads);
    const uint16_t* po = static_cast<const uint16_t*>(out);
    const uint16_t* pd = static_cast<const uint16_t*>(d_out);
    if ((reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(d_out) & 15) || (o_rs & 7) || (o_bs & 7)) return -2;
    if (lpg == 8) {
      if (bf16) attn_delta_kernel<true, 8><<<blocks, threads, 0, stream>>>(po, pd, o_rs, o_bs, delta, B, T, H, HD);
      else attn_delta_kernel<false, 8><<<blocks, threads, 0, stream>>>(po, pd, o_rs, o_bs, delta, B, T, H, HD);
    } else {
      if (bf16) attn_delta_kernel<true, 16><<<blocks, threads, 0, stream>>>(po, pd, o_rs, o_bs, delta, B, T, H, HD);
      else attn_delta_kernel<false, 16><<<blocks, threads, 0, stream>>>(po, pd, o_rs, o_bs, delta, B, T, H, HD);
    }
  }
  AttnBwdParams p;
  p.lse = lse; p.delta = delta; p.dq_accum = dq_accum; p.dk = dk; p.dv = dv;
  p.dk_row_stride = dk_rs; p.dk_batch_stride = dk_bs; p.dv_row_stride = dv_rs; p.dv_batch_stride = dv_bs;
  p.T = T; p.H = H; p.scale = scale; p.causal = causal; p.bf16 = bf16; p.status = status;
  p.prof = g_attn_prof;
  p.hd = HD; p.doc_start = doc_start; p.alibi_slopes = alibi_slopes;
  if (!drop_params(dropout_p, p.drop_threshold16, p.inv_keep)) return -2;
  p.seed = seed;
#define MSQ_BWD2(HDV, BF, GN) \
  (p.drop_threshold16 ? launch_bwd<HDV, BF, true, GN>(tq, tk, tv, tdo, tdq, p, B, stream) \
                      : launch_bwd<HDV, BF, false, GN>(tq, tk, tv, tdo, tdq, p, B, stream))
#define MSQ_BWD(HDV, BF) (gen ? MSQ_BWD2(HDV, BF, true) : MSQ_BWD2(HDV, BF, false))
  if (HD <= 64) return bf16 ? MSQ_BWD(64, true) : MSQ_BWD(64, false);
  return bf16 ? MSQ_BWD(128, true) : MSQ_BWD(128, false);
#undef MSQ_BWD
#undef MSQ_BWD2
}
