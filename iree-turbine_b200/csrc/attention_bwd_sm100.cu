// Attention backward (head dim 128 or 64, f16 / bf16, grouped-query heads, optional causal mask aligned
// to the bottom-right corner as in the forward kernel):
//   P  = exp(scale * Q K^T - LSE)          dV = P^T dO
//   dP = dO V^T                            dS = P o (dP - delta),  delta[i] = sum_d dO[i, d] O[i, d]
//   dQ = scale * dS K                      dK = scale * dS^T Q
//
// Three launches.  Only the forward's output O is required from the forward call; its row
// log-sum-exp, if the caller kept it, spares the statistics sweep of the second launch:
//   1. attn_bwd_delta_kernel: delta.
//   2. attn_bwd_dq_kernel: one CTA per (batch, query head, tile of 128 queries).  It holds Q and dO
//      and sweeps the visible K/V tiles: first a statistics sweep when no LSE was given, then the
//      gradient sweep (S, dP -> dS -> dQ += dS K).
//   3. attn_bwd_dkv_t_kernel: one CTA per (batch, K/V head, tile of 128 keys).  It holds K and V
//      and sweeps the query tiles of every query head of the group that see these keys, with the
//      keys as the M dimension of every product: S^T, dP^T -> P^T, dS^T -> dV += P^T dO,
//      dK += dS^T Q.
// No atomics: every output element is accumulated by one CTA in a fixed order, so results do not
// depend on the grid or on how heads are sharded over devices.
//
// All products are tcgen05 MMAs (M = 128, fp32 accumulators in tensor memory).  An operand tile in
// shared memory is 128 rows x head-dim 16-bit columns in 64-column blocks of 16 KB with the
// 128-byte swizzle, as TMA writes it, and is described to the tensor core as K-major (contraction
// along the 128-byte rows) or MN-major (contraction along the row index) as the product needs.
// The probabilities and dS never go through shared memory: the threads that computed them store
// them to tensor memory as 16-bit pairs over the columns they were computed from, and the next
// product takes them from there as its A operand (the forward kernel's way of handing P on).
//   S   = Q K^T    A = Q  (TMEM)    B = K  K-major      dQ += dS K     A = dS   (TMEM)  B = K  MN-major
//   dP  = dO V^T   A = dO (TMEM)    B = V  K-major
//   S^T = K Q^T    A = K  K-major   B = Q  K-major      dV += P^T dO   A = P^T  (TMEM)  B = dO MN-major
//   dP^T= V dO^T   A = V  K-major   B = dO K-major      dK += dS^T Q   A = dS^T (TMEM)  B = Q  MN-major
//
// Roles (10 warps): warp 0 TMA producer, warp 1 MMA issuer + tensor-memory owner, warps 2..9 the
// softmax algebra (two threads per lane of tensor memory, 64 columns each), then the epilogue.
// Every wait is bounded.
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace b200k {
namespace {

constexpr int kD = 128;
constexpr int kRows = 128;
constexpr int kBwdThreads = 320;      // TMA warp, MMA warp, eight softmax / epilogue warps
constexpr int kSoftmaxThreads = 256;  // two threads per query row, 64 columns each
constexpr int kTileBytes = kRows * kD * 2;  // 32 KB
constexpr int kHalfBytes = kTileBytes / 2;  // one 64-column block

// Shared-memory tiles of the dQ kernel (32 KB slots): Q and dO (copied to tensor memory in the
// prologue; their slots then become the third K / V buffer), two more K and V buffers (a ring of
// three, so that a tile is loaded an iteration and a half before its score product) and a staging
// tile (statistics exchange, epilogue).
constexpr int kOffQ = 0, kOffDO = kTileBytes, kOffK = 2 * kTileBytes, kOffV = 3 * kTileBytes;
constexpr int kOffK1 = 4 * kTileBytes, kOffDS = 5 * kTileBytes, kOffV1 = 6 * kTileBytes;
constexpr int kDqTiles = 7;
// fix_full, ld_full[3], it_done[3], s_full, s_free, pds_full, dp_full, a_ready
constexpr int kNumDqBars = 12;
constexpr int dq_smem_bytes() { return kDqTiles * kTileBytes + kNumDqBars * 8 + 16 + 1024; }
// Tensor-memory columns.  The dQ kernel has one accumulator and keeps Q and dO in the fourth quarter,
// so that none of its three products reads an A operand from shared memory; the dK / dV kernel has
// two accumulators.
constexpr uint32_t kTmS = 0, kTmDP = 128, kTmAcc0 = 256, kTmAcc1 = 384;
constexpr uint32_t kTmQ = 384, kTmDO = 448;  // dQ kernel: Q and dO as 16-bit pairs (64 columns each at head dim 128)
constexpr float kLog2eBwd = 1.4426950408889634f;
constexpr int kStatusBwdTimeout = 64;

struct BwdParams {
  int32_t batch, q_heads, kv_heads, seq_q, seq_kv;
  int32_t causal, causal_offset;  // query i sees keys j <= i + causal_offset
  int32_t num_q_tiles, num_kv_tiles;
  int32_t bh_group_q, bh_group_kv;  // causal grids: heads whose tiles are interleaved, longest job first (see causal_work_item)
  float scale, scale_log2;
  float* lse2;   // [batch, q_heads, seq_q], log2 domain: log2(sum_j exp2(scale_log2 * s_ij))
  float* delta;  // [batch, q_heads, seq_q]
  const float* lse_in;  // optional: the forward's ln-sum-exp per row (then lse2 is not used)
  int32_t* status;
};

// The forward's row statistic (natural log, -inf for a row without keys) in the form used here:
// log2 domain, +inf for such a row so that exp2(x - lse2) is 0.
__device__ __forceinline__ float lse_to_log2(float lse) { return lse == -INFINITY ? INFINITY : lse * kLog2eBwd; }

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^x for a pair on the FMA pipe instead of the special-function unit (x = j + f, j = rint(x) from
// the low mantissa bits of x + 1.5 * 2^23, 2^f on [-0.5, 0.5] by a degree-3 polynomial, max relative
// error 7.5e-5, far below the rounding of P to 16 bits; exponent added as an integer).  Only used
// where every element is visible, so x is finite; clamped at -125 against exponent underflow.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
  x.x = fmaxf(x.x, -125.f);
  x.y = fmaxf(x.y, -125.f);
  const float2 t = fadd2(x, make_float2(12582912.f, 12582912.f));
  const float2 j = fadd2(t, make_float2(-12582912.f, -12582912.f));
  const float2 f = ffma2(j, make_float2(-1.f, -1.f), x);
  float2 q = ffma2(f, make_float2(0.0551716648f, 0.0551716648f), make_float2(0.2426111251f, 0.2426111251f));
  q = ffma2(q, f, make_float2(0.6932609677f, 0.6932609677f));
  q = ffma2(q, f, make_float2(0.9999280572f, 0.9999280572f));
  float2 r;
  r.x = __int_as_float(__float_as_int(q.x) + (__float_as_int(t.x) << 23));
  r.y = __int_as_float(__float_as_int(q.y) + (__float_as_int(t.y) << 23));
  return r;
}
// Which of every 8 consecutive column pairs take the polynomial (bit i = pair i): the exponentials of
// an iteration (64 per thread, 256 threads) would otherwise occupy the special-function unit for
// 1024 cycles between the score product and the dV product.  Measured on the causal bf16 B4 H32
// S4096 backward: none 2.055 ms, 3 of 8 2.038 ms, 4 of 8 2.023 ms.
constexpr uint32_t kBwdPolyMask = 0x55u;

// Which (batch * head, tile rank) a CTA of a causal grid works on.  A tile's cost grows with its
// rank's complement (rank 0 = the heaviest tile of its head) and CTAs are handed out in blockIdx
// order, so within a group of `group` heads the heaviest tile of every head goes first, then the
// next one, ...: longest job first, which matters at the end of the grid, where a head's heavy
// tiles started late otherwise (dK / dV kernel with grouped heads: 974 -> 909 us).  The groups keep
// the heads in flight few enough for their K / V (dQ kernel) or Q / dO (dK / dV kernel) to stay in
// L2: with all 128 heads of the multi-head bench shape interleaved, every CTA streamed its
// operands from DRAM and the backward took 2.03 ms instead of 1.76.
__device__ __forceinline__ void causal_work_item(int block, int num_bh, int num_tiles, int group, int& bh, int& rank) {
  const int per_group = group * num_tiles;
  const int sg = block / per_group;
  const int g0 = sg * group;
  const int gsize = min(group, num_bh - g0);
  const int r = block - sg * per_group;
  rank = r / gsize;
  bh = g0 + (r - rank * gsize);
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Writes 32 consecutive columns [c0, c0 + 32) of row `r` of a 128 x 128 16-bit tile (two 64-column
// blocks, 128-byte rows, 16-byte chunks XOR-swizzled with the row index as TMA does).
__device__ __forceinline__ void store_row_chunk(uint8_t* tile, int r, int c0, const uint32_t (&w)[16]) {
  uint8_t* row = tile + (c0 >> 6) * kHalfBytes + r * 128;
  const int chunk0 = (c0 & 63) >> 3;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    *reinterpret_cast<uint4*>(row + (((chunk0 + i) ^ (r & 7)) << 4)) =
        make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
}

// D[128 x N] (+)= A * B with both operands in shared memory; KSTEPS steps of K = 16 (8 for a
// contraction over 128 rows or columns, 4 for one over a head dim of 64); N is in the instruction
// descriptor.
// K-major operand: step = 32 bytes inside a 64-column block, second block 16 KB further.
// MN-major operand: step = 16 rows = 2 KB.
template <bool A_MN, bool B_MN, int KSTEPS = 8>
__device__ __forceinline__ void mma_128x128x128(uint32_t d_tmem, uint32_t a_addr, uint32_t b_addr, uint32_t idesc,
                                                bool accumulate) {
  const uint64_t a0 = A_MN ? make_desc_mnmajor_sw128(a_addr, kHalfBytes) : make_desc_kmajor_sw128(a_addr);
  const uint64_t b0 = B_MN ? make_desc_mnmajor_sw128(b_addr, kHalfBytes) : make_desc_kmajor_sw128(b_addr);
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    const uint32_t a_off = A_MN ? ks * (2048 >> 4) : (ks >> 2) * (kHalfBytes >> 4) + (ks & 3) * 2;
    const uint32_t b_off = B_MN ? ks * (2048 >> 4) : (ks >> 2) * (kHalfBytes >> 4) + (ks & 3) * 2;
    umma_f16_ss(d_tmem, a0 + a_off, b0 + b_off, idesc, (accumulate || ks > 0) ? 1u : 0u);
  }
}

// A 128-row x HD-column operand tile: one 64-column block (head dim 64) or two; the tile's slot in
// shared memory is 32 KB either way.
template <int HD>
__device__ __forceinline__ void load_tile_4d(uint8_t* dst, const CUtensorMap* tmap, uint64_t* bar, int row0, int head,
                                             int batch) {
  tma_load_4d(dst, tmap, bar, 0, row0, head, batch);
  if (HD == 128) tma_load_4d(dst + kHalfBytes, tmap, bar, 64, row0, head, batch);
}

// ---------------------------------------------------------------------------------------------
// dQ.  One CTA per (batch, query head, tile of 128 queries) holds Q and dO and sweeps the visible
// K / V tiles: first a statistics sweep when no LSE was given (S = Q K^T only; running row maximum
// and sum -> LSE, kept in registers and written to the workspace), then the gradient sweep
//     S = Q K^T    dP = dO V^T    dS = P o (dP - delta)    dQ += dS K
// Tensor memory holds S | dP | dQ | Q, dO.  The softmax threads copy Q and dO from shared to tensor
// memory once (undoing the 128-byte swizzle), after which all three products take their A operand
// from tensor memory and only the streamed K / V tiles go through the shared-memory port.  The S
// columns are handed back to the MMA warp as soon as the algebra has them in registers, so that the
// next score product runs under the algebra; dS goes back to tensor memory as 16-bit pairs over dP
// and is the A operand of the dQ product there.  K / V tiles stream through a ring of three buffers.
// Measured per-iteration issue order of the MMA warp: dP(i), S(i+1), dQ(i).
// ---------------------------------------------------------------------------------------------
template <typename T, int HD>
__global__ void __launch_bounds__(kBwdThreads, 1)
    attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                       const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                       const __grid_constant__ CUtensorMap tmap_dq, const BwdParams p) {
  static_assert(HD == 128 || HD == 64, "head dim 128 or 64");
  constexpr uint32_t kFmt = std::is_same<T, __half>::value ? kFmtF16 : kFmtBF16;
  constexpr uint32_t kIdKK = make_idesc(kFmt, kFmt, 128, 128, 0, 0);  // S, dP: 128 x 128, contraction over the head dim
  constexpr uint32_t kIdKM = make_idesc(kFmt, kFmt, 128, HD, 0, 1);   // dQ: 128 x HD, B MN-major
  constexpr int kDSteps = HD / 16;                                     // K steps of a contraction over the head dim
  constexpr int kOpBytes = kRows * HD * 2;                             // bytes TMA brings per operand tile
  constexpr int kBufs = 3;  // K / V buffers; the third pair takes over the Q / dO tiles once those are in tensor memory
  auto k_off = [](int b) { return b == 0 ? kOffK : (b == 1 ? kOffK1 : kOffQ); };
  auto v_off = [](int b) { return b == 0 ? kOffV : (b == 1 ? kOffV1 : kOffDO); };

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kDqTiles * kTileBytes);
  uint64_t* fix_full = bars;      // Q and dO have landed in shared memory
  uint64_t* ld_full = bars + 1;   // [buffer] the K (and V) tiles of an iteration have landed
  uint64_t* it_done = bars + 4;   // [buffer] the last MMAs of an iteration that used it have completed
  uint64_t* s_full = bars + 7;    // S is in tensor memory
  uint64_t* s_free = bars + 8;    // every row of S has been read into registers: the next S may be issued
  uint64_t* pds_full = bars + 9;  // all rows of dS stored (and dP read)
  uint64_t* dp_full = bars + 10;  // dP is in tensor memory (gradient iterations)
  uint64_t* a_ready = bars + 11;  // Q and dO have been copied to tensor memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumDqBars);
  volatile uint32_t* abort_word = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int group = p.q_heads / p.kv_heads;

  // ---- work item ----
  // causal: the last query tile of a head is its heaviest
  int bh, tile;
  if (p.causal) {
    int rank;
    causal_work_item(blockIdx.x, gridDim.x / p.num_q_tiles, p.num_q_tiles, p.bh_group_q, bh, rank);
    tile = p.num_q_tiles - 1 - rank;
  } else {
    bh = blockIdx.x / p.num_q_tiles;
    tile = blockIdx.x - bh * p.num_q_tiles;
  }
  const int batch = bh / p.q_heads;
  const int head = bh - batch * p.q_heads;
  const int kvh = head / group;
  const int row0 = tile * kRows;  // first query of the tile
  int n = p.num_kv_tiles;         // visible K / V tiles
  if (p.causal) {
    const int last_col = row0 + kRows - 1 + p.causal_offset;
    n = last_col < 0 ? 0 : min(last_col / kRows + 1, p.num_kv_tiles);
  }
  // a statistics sweep over the n tiles first, unless the caller supplied the forward's LSE
  const int n_stats = p.lse_in == nullptr ? n : 0;
  const int total = n_stats + n;  // iterations

  if (threadIdx.x == 0) {
    mbar_init(fix_full, 1);
    for (int b = 0; b < kBufs; ++b) {
      mbar_init(ld_full + b, 1);
      mbar_init(it_done + b, 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_free, kSoftmaxThreads / 32);
    mbar_init(a_ready, kSoftmaxThreads / 32);
    mbar_init(pds_full, kSoftmaxThreads);
    mbar_init(dp_full, 1);
    *abort_word = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_do);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
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
    // ---------------- TMA producer ----------------
    if (lane == 0 && total > 0) {
      mbar_arrive_expect_tx(fix_full, 2 * kOpBytes);
      load_tile_4d<HD>(smem + kOffQ, &tmap_q, fix_full, row0, head, batch);
      load_tile_4d<HD>(smem + kOffDO, &tmap_do, fix_full, row0, head, batch);
      for (int i = 0; i < total; ++i) {
        const int buf = i % kBufs;
        // the MMAs of the iteration that last used this buffer have finished reading it
        if (i >= kBufs && !mbar_wait(it_done + buf, ((i - kBufs) / kBufs) & 1, abort_word)) break;
        // the third pair of buffers is where Q and dO landed: not before they are in tensor memory
        if (i == kBufs - 1 && !mbar_wait(a_ready, 0, abort_word)) break;
        uint64_t* full = ld_full + buf;
        const bool stats = i < n_stats;
        const int j = stats ? i : i - n_stats;
        mbar_arrive_expect_tx(full, stats ? kOpBytes : 2 * kOpBytes);
        load_tile_4d<HD>(smem + k_off(buf), &tmap_k, full, j * kRows, kvh, batch);
        if (!stats) load_tile_4d<HD>(smem + v_off(buf), &tmap_v, full, j * kRows, kvh, batch);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && total > 0) {
      // D[128 x 128] = A B^T, A (128 x HD, 16-bit pairs) in tensor memory at `a_tmem`, B a K-major tile
      auto mma_ts_k = [&](uint32_t d_tmem, uint32_t a_tmem, uint32_t b_addr) {
        const uint64_t b0 = make_desc_kmajor_sw128(b_addr);
#pragma unroll
        for (int ks = 0; ks < kDSteps; ++ks)
          umma_f16_ts(d_tmem, a_tmem + ks * 8, b0 + (ks >> 2) * (kHalfBytes >> 4) + (ks & 3) * 2, kIdKK, ks > 0 ? 1u : 0u);
      };
      bool ok = mbar_wait(a_ready, 0, abort_word);
      // S of iteration `it`, once its K tile has landed
      auto issue_s = [&](int it) -> bool {
        const int b = it % kBufs;
        if (!mbar_wait(ld_full + b, (it / kBufs) & 1, abort_word)) return false;
        tc_fence_after();
        mma_ts_k(tmem_base + kTmS, tmem_base + kTmQ, smem_u32(smem + k_off(b)));
        umma_commit(s_full);
        return true;
      };
      if (ok) {
        tc_fence_after();
        ok = issue_s(0);
      }
      for (int i = 0; i < total && ok; ++i) {
        const int buf = i % kBufs;
        const bool stats = i < n_stats;
        const uint32_t sk = smem_u32(smem + k_off(buf)), sv = smem_u32(smem + v_off(buf));
        const int gi = i - n_stats;  // index among the gradient iterations
        // The algebra on S starts while dP is still being computed; the next iteration's S is issued
        // as soon as every row of the current one has been read into registers.
        if (!stats) {
          mma_ts_k(tmem_base + kTmDP, tmem_base + kTmDO, sv);
          umma_commit(dp_full);
        }
        if (i + 1 < total) {
          if (!mbar_wait(s_free, i & 1, abort_word)) break;
          if (!issue_s(i + 1)) break;
        }
        if (!mbar_wait(pds_full, i & 1, abort_word)) break;
        tc_fence_after();
        if (!stats) {
          // dQ += dS K, A = dS from tensor memory (keys 0..63 in columns 0..31 of the dP region,
          // keys 64..127 in columns 64..95), B = the K tile read MN-major
          const uint64_t b0 = make_desc_mnmajor_sw128(sk, kHalfBytes);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_f16_ts(tmem_base + kTmAcc0, tmem_base + kTmDP + (ks >> 2) * 64 + (ks & 3) * 8, b0 + ks * (2048 >> 4),
                        kIdKM, (gi > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(it_done + buf);
      }
    }
    __syncwarp();
  } else {
    // ---------------- softmax algebra, then the epilogue: two threads per query row ----------------
    // Warp w may touch tensor-memory lanes 32 (w % 4) ..: warps 2..5 take columns 0..63 of their
    // rows, warps 6..9 columns 64..127.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const float ninf = -INFINITY;
    float m = ninf, l = 0.f, lse2 = INFINITY, dl = 0.f;
    const int q_g = row0 + r;
    const int64_t stat_idx = (static_cast<int64_t>(batch) * p.q_heads + head) * p.seq_q + q_g;
    if (q_g < p.seq_q) {
      dl = __ldg(p.delta + stat_idx);
      if (p.lse_in) lse2 = lse_to_log2(__ldg(p.lse_in + stat_idx));
    }
    // key j (global index) is visible to this row iff j <= col_hi
    int col_hi = -1;
    if (q_g < p.seq_q) {
      col_hi = p.seq_kv - 1;
      if (p.causal) col_hi = min(col_hi, q_g + p.causal_offset);
    }
    // After a wait has given up the loop keeps its shape (arrivals and named barriers) but skips the work.
    bool ok = true;
    // Q and dO are the A operands of S and dP for the whole life of the CTA: they move from the
    // shared-memory tiles TMA wrote into tensor memory once (16-bit pairs, one row per lane), so
    // that those two products read only their B operand from shared memory.
    if (total > 0) {
      ok = mbar_wait(fix_full, 0, abort_word);
      if (ok) {
        constexpr int kChunks = HD / 16;  // 16-byte chunks per thread: 64 (or 32) elements of the row
        const int blk = HD == 128 ? half : 0;
        const int c0 = HD == 128 ? 0 : half * kChunks;
#pragma unroll
        for (int op = 0; op < 2; ++op) {
          const uint8_t* row = smem + (op == 0 ? kOffQ : kOffDO) + blk * kHalfBytes + r * 128;
          uint32_t w[kChunks * 4];
#pragma unroll
          for (int c = 0; c < kChunks; ++c) {
            const uint4 v = *reinterpret_cast<const uint4*>(row + (((c0 + c) ^ (r & 7)) << 4));
            w[4 * c] = v.x;
            w[4 * c + 1] = v.y;
            w[4 * c + 2] = v.z;
            w[4 * c + 3] = v.w;
          }
          const uint32_t dst = lane_base + (op == 0 ? kTmQ : kTmDO) + half * (kChunks * 4);
          if constexpr (HD == 128)
            tmem_st_32x32b_x32(dst, w);
          else
            tmem_st_32x32b_x16(dst, w);
        }
        tmem_wait_st();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(a_ready);
    }
    for (int i = 0; i < total; ++i) {
      const bool stats = i < n_stats;
      const int kv_base = (stats ? i : i - n_stats) * kRows;
      const uint32_t s_base = lane_base + kTmS;
      if (ok && !mbar_wait(s_full, i & 1, abort_word)) ok = false;
      const int gi = i - n_stats;  // index among the gradient iterations
      ok = __all_sync(0xffffffffu, ok);  // one decision per warp
      if (stats) {
        if (ok) {
          tc_fence_after();
#pragma unroll 1
          for (int cc = 0; cc < 2; ++cc) {
            const int c4 = half * 2 + cc;
            uint32_t s[32];
            tmem_ld_32x32b_x32(s_base + c4 * 32, s);
            const int kv0 = kv_base + c4 * 32;
            tmem_wait_ld();
            float cm = ninf;
            const bool all_visible = kv0 + 31 <= col_hi;  // no per-element test then
#pragma unroll
            for (int k = 0; k < 32; ++k) {
              const float x = (all_visible || kv0 + k <= col_hi) ? __uint_as_float(s[k]) * p.scale_log2 : ninf;
              s[k] = __float_as_uint(x);
              cm = fmaxf(cm, x);
            }
            const float m_new = fmaxf(m, cm);
            if (m_new > ninf) {
              float acc = 0.f;
#pragma unroll
              for (int k = 0; k < 32; ++k) acc += ex2_approx(__uint_as_float(s[k]) - m_new);
              l = l * ex2_approx(m - m_new) + acc;
              m = m_new;
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free);  // the scores of this tile have been read
      } else {
        // P from S while the tensor core still computes dP; then dS = P o (dP - delta)
        float pf[64];
        if (!ok && lane == 0) mbar_arrive(s_free);
        if (ok) {
          tc_fence_after();
          uint32_t s64[64];  // this thread's 64 columns in one load
          tmem_ld_32x32b_x64(s_base + half * 64, s64);
          tmem_wait_ld();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(s_free);  // S is in registers: the next score product may overwrite it
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            const int c4 = half * 2 + cc;
            const uint32_t* s = s64 + cc * 32;
            const int kv0 = kv_base + c4 * 32;
            if (kv0 + 31 <= col_hi) {  // the whole chunk is visible to this row: no per-element test
#pragma unroll
              for (int k = 0; k < 32; k += 2) {
                const float x0 = fmaf(__uint_as_float(s[k]), p.scale_log2, -lse2);
                const float x1 = fmaf(__uint_as_float(s[k + 1]), p.scale_log2, -lse2);
                const float2 e = ((kBwdPolyMask >> ((k >> 1) & 7)) & 1u) ? exp2_poly2(make_float2(x0, x1))
                                                                         : make_float2(ex2_approx(x0), ex2_approx(x1));
                pf[cc * 32 + k] = e.x;
                pf[cc * 32 + k + 1] = e.y;
              }
            } else {
#pragma unroll
              for (int k = 0; k < 32; ++k)
                pf[cc * 32 + k] =
                    (kv0 + k <= col_hi) ? ex2_approx(fmaf(__uint_as_float(s[k]), p.scale_log2, -lse2)) : 0.f;
            }
          }
        }
        if (ok && !mbar_wait(dp_full, gi & 1, abort_word)) ok = false;
        if (ok) {
          tc_fence_after();
          uint32_t dp64[64];
          tmem_ld_32x32b_x64(lane_base + kTmDP + half * 64, dp64);
          tmem_wait_ld();
          // dS stays in tensor memory: 16-bit pairs over the first half of this thread's own dP
          // columns, from where the dQ product takes it as its A operand
          uint32_t dsw[32];
#pragma unroll
          for (int k = 0; k < 64; k += 2)
            dsw[k >> 1] = pack2<T>(pf[k] * (__uint_as_float(dp64[k]) - dl), pf[k + 1] * (__uint_as_float(dp64[k + 1]) - dl));
          tmem_st_32x32b_x32(lane_base + kTmDP + half * 64, dsw);
          tmem_wait_st();
        }
      }
      if (stats && i == n_stats - 1) {
        // The two threads of a row combine their (max, sum) through the staging tile, which nothing
        // uses before the epilogue; both evaluate the same expression, so they agree bitwise.
        float2* xchg = reinterpret_cast<float2*>(smem + kOffDS);
        xchg[half * kRows + r] = make_float2(m, l);
        asm volatile("bar.sync 3, 256;" ::: "memory");
        const float2 a0 = xchg[r], a1 = xchg[kRows + r];
        asm volatile("bar.sync 3, 256;" ::: "memory");  // all have read before the tile is written again
        const float mt = fmaxf(a0.x, a1.x);
        const float lt = mt > ninf ? a0.y * exp2f(a0.x - mt) + a1.y * exp2f(a1.x - mt) : 0.f;
        lse2 = lt > 0.f ? mt + log2f(lt) : INFINITY;
        if (half == 0 && q_g < p.seq_q) p.lse2[stat_idx] = lse2;
      }
      tc_fence_before();
      mbar_arrive(pds_full);
    }
    if (ok && total > 0)
      ok = mbar_wait(it_done + (total - 1) % kBufs, ((total - 1) / kBufs) & 1, abort_word);
    // every thread of the eight warps must agree before the named barrier below
    ok = bar_red_and(1, kSoftmaxThreads, ok);
    if (ok) {
      tc_fence_after();
      // accumulator -> 16-bit tile in the staging buffer -> TMA stores
      uint8_t* stage = smem + kOffDS;
#pragma unroll 1
      for (int cc = 0; cc < 2; ++cc) {
        const int c4 = half * 2 + cc;
        if (c4 * 32 >= HD) continue;  // head dim 64: the accumulator has 64 columns
        uint32_t v[32], w[16];
        if (total > 0) {
          tmem_ld_32x32b_x32(lane_base + kTmAcc0 + c4 * 32, v);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int k = 0; k < 32; ++k) v[k] = 0u;  // no key is visible
        }
#pragma unroll
        for (int k = 0; k < 32; k += 2)
          w[k >> 1] = pack2<T>(__uint_as_float(v[k]) * p.scale, __uint_as_float(v[k + 1]) * p.scale);  // dQ carries the softmax scale
        store_row_chunk(stage, r, c4 * 32, w);
      }
      fence_proxy_async_smem();
      asm volatile("bar.sync 2, 256;" ::: "memory");
      if (r == 0 && half == 0) {
        tma_store_4d(&tmap_dq, smem + kOffDS, 0, row0, head, batch);
        if (HD == 128) tma_store_4d(&tmap_dq, smem + kOffDS + kHalfBytes, 64, row0, head, batch);
        tma_store_commit();
        tma_store_wait_read<0>();  // the staging tile has been read: the CTA may go (the writes land before the grid ends)
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0 && threadIdx.x == 0 && p.status) atomicOr(p.status, kStatusBwdTimeout);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------
// dK / dV in the TRANSPOSED orientation.  One CTA per (batch, K/V head, tile of 128 keys) holds K
// and V and sweeps the query tiles of the head group that see these keys.  Every product has the
// keys as its M dimension:
//     S^T  = K Q^T      dP^T = V dO^T      (K, V, Q, dO tiles all K-major in shared memory)
//     dV  += P^T dO     dK  += dS^T Q      (A = P^T / dS^T straight from TENSOR memory, B MN-major)
// so P^T and dS^T never go through shared memory: the thread that owns a key row turns its S^T
// entries into 16-bit probabilities and stores them over its own S^T columns (two threads per
// row, each over the first half of its 64 columns), the way the forward kernel hands P to its
// second product, and likewise dS^T over dP^T.  The row
// statistics belong to the query, i.e. to the COLUMN here; the 128 (lse, delta) pairs of a query
// tile are brought into shared memory once per iteration and read by broadcast.
// MMA order (one in-order stream): dV(i) : S^T(i+1) : dK(i) : dP^T(i+1).  S^T(i+1) may overwrite
// P^T(i) and dP^T(i+1) may overwrite dS^T(i) without a barrier because they are issued behind the
// products that read them.  Shared memory: K, V, two Q buffers, two dO buffers (6 x 32 KB).
// Tensor memory: S^T / P^T | dP^T / dS^T | dV | dK (128 columns each).
// ---------------------------------------------------------------------------------------------
constexpr int kTK = 0, kTV = kTileBytes, kTQ0 = 2 * kTileBytes, kTQ1 = 3 * kTileBytes, kTDO0 = 4 * kTileBytes,
              kTDO1 = 5 * kTileBytes, kTVec = 6 * kTileBytes;  // kTVec: [2 buffers][lse2 128 | delta 128] floats
constexpr int kTVecBytes = 2 * 256 * 4;
// fix_full, ld_full[2], it_done[2], s_full, dp_full, p_full, ds_full
constexpr int kNumDkvtBars = 9;
constexpr int dkvt_smem_bytes() { return 6 * kTileBytes + kTVecBytes + kNumDkvtBars * 8 + 16 + 1024; }

template <typename T, int HD>
__global__ void __launch_bounds__(kBwdThreads, 1)
    attn_bwd_dkv_t_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                          const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                          const __grid_constant__ CUtensorMap tmap_dv, const __grid_constant__ CUtensorMap tmap_dk,
                          const BwdParams p) {
  static_assert(HD == 128 || HD == 64, "head dim 128 or 64");
  constexpr uint32_t kFmt = std::is_same<T, __half>::value ? kFmtF16 : kFmtBF16;
  constexpr uint32_t kIdS = make_idesc(kFmt, kFmt, 128, 128, 0, 0);  // S^T, dP^T: 128 keys x 128 queries
  constexpr uint32_t kIdG = make_idesc(kFmt, kFmt, 128, HD, 0, 1);   // dV, dK: 128 keys x HD, B MN-major
  constexpr int kDSteps = HD / 16;
  constexpr int kOpBytes = kRows * HD * 2;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  float* vec = reinterpret_cast<float*>(smem + kTVec);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kTVec + kTVecBytes);
  uint64_t* fix_full = bars;     // K and V have landed
  uint64_t* ld_full = bars + 1;  // [buffer] Q and dO of an iteration have landed
  uint64_t* it_done = bars + 3;  // [buffer] every product that reads the buffer has completed
  uint64_t* s_full = bars + 5;   // S^T is in tensor memory
  uint64_t* dp_full = bars + 6;  // dP^T is in tensor memory
  uint64_t* p_full = bars + 7;   // all rows of P^T stored (S^T read)
  uint64_t* ds_full = bars + 8;  // all rows of dS^T stored (dP^T read)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumDkvtBars);
  volatile uint32_t* abort_word = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int group = p.q_heads / p.kv_heads;

  // causal: key tile 0 is seen by every query tile, the last one by few
  int bh, tile;
  if (p.causal) {
    causal_work_item(blockIdx.x, gridDim.x / p.num_kv_tiles, p.num_kv_tiles, p.bh_group_kv, bh, tile);
  } else {
    bh = blockIdx.x / p.num_kv_tiles;
    tile = blockIdx.x - bh * p.num_kv_tiles;
  }
  const int batch = bh / p.kv_heads;
  const int kvh = bh - batch * p.kv_heads;
  const int row0 = tile * kRows;  // first key of the tile
  int qt_lo = 0;
  if (p.causal) qt_lo = max(0, row0 - p.causal_offset) / kRows;
  const int n = max(0, p.num_q_tiles - qt_lo);  // query tiles per head that see these keys
  const int total = group * n;

  if (threadIdx.x == 0) {
    mbar_init(fix_full, 1);
    mbar_init(ld_full, 1);
    mbar_init(ld_full + 1, 1);
    mbar_init(it_done, 1);
    mbar_init(it_done + 1, 1);
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_full, kSoftmaxThreads / 32);   // one arrival per warp
    mbar_init(ds_full, kSoftmaxThreads / 32);
    *abort_word = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_do);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
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
    // ---------------- TMA producer ----------------
    if (lane == 0 && total > 0) {
      mbar_arrive_expect_tx(fix_full, 2 * kOpBytes);
      load_tile_4d<HD>(smem + kTK, &tmap_k, fix_full, row0, kvh, batch);
      load_tile_4d<HD>(smem + kTV, &tmap_v, fix_full, row0, kvh, batch);
      for (int i = 0; i < total; ++i) {
        const int b = i & 1;
        if (i >= 2 && !mbar_wait(it_done + b, ((i - 2) >> 1) & 1, abort_word)) break;
        const int g = i / n;
        const int qt = qt_lo + (i - g * n);
        mbar_arrive_expect_tx(ld_full + b, 2 * kOpBytes);
        load_tile_4d<HD>(smem + (b ? kTQ1 : kTQ0), &tmap_q, ld_full + b, qt * kRows, kvh * group + g, batch);
        load_tile_4d<HD>(smem + (b ? kTDO1 : kTDO0), &tmap_do, ld_full + b, qt * kRows, kvh * group + g, batch);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && total > 0) {
      const uint32_t sk = smem_u32(smem + kTK), sv = smem_u32(smem + kTV);
      auto sq = [&](int b) { return smem_u32(smem + (b ? kTQ1 : kTQ0)); };
      auto sdo = [&](int b) { return smem_u32(smem + (b ? kTDO1 : kTDO0)); };
      // D[keys x HD] (+)= A^T-from-tensor-memory * B, B = an MN-major tile (rows = queries): 8 steps of 16 queries
      // The 16-bit A tile sits in two pieces: queries 0..63 in columns 0..31 of the region, queries
      // 64..127 in columns 64..95 (each of the two threads of a row writes over its own S columns).
      auto mma_ts = [&](uint32_t d_tmem, uint32_t a_tmem, uint32_t b_addr, bool accumulate) {
        const uint64_t b0 = make_desc_mnmajor_sw128(b_addr, kHalfBytes);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_f16_ts(d_tmem, a_tmem + (ks >> 2) * 64 + (ks & 3) * 8, b0 + ks * (2048 >> 4), kIdG,
                      (accumulate || ks > 0) ? 1u : 0u);
      };
      bool ok = mbar_wait(fix_full, 0, abort_word);
      if (ok) ok = mbar_wait(ld_full, 0, abort_word);
      if (ok) {
        tc_fence_after();
        mma_128x128x128<false, false, kDSteps>(tmem_base + kTmS, sk, sq(0), kIdS, false);   // S^T(0)
        umma_commit(s_full);
        mma_128x128x128<false, false, kDSteps>(tmem_base + kTmDP, sv, sdo(0), kIdS, false);  // dP^T(0)
        umma_commit(dp_full);
      }
      for (int i = 0; i < total && ok; ++i) {
        const int b = i & 1;
        if (!mbar_wait(p_full, i & 1, abort_word)) break;
        tc_fence_after();
        mma_ts(tmem_base + kTmAcc0, tmem_base + kTmS, sdo(b), i > 0);  // dV += P^T dO
        if (i + 1 < total) {
          if (!mbar_wait(ld_full + (b ^ 1), ((i + 1) >> 1) & 1, abort_word)) break;
          tc_fence_after();
          mma_128x128x128<false, false, kDSteps>(tmem_base + kTmS, sk, sq(b ^ 1), kIdS, false);  // S^T(i+1), behind dV(i)
          umma_commit(s_full);
        }
        if (!mbar_wait(ds_full, i & 1, abort_word)) break;
        tc_fence_after();
        mma_ts(tmem_base + kTmAcc1, tmem_base + kTmDP, sq(b), i > 0);  // dK += dS^T Q
        umma_commit(it_done + b);
        if (i + 1 < total) {
          mma_128x128x128<false, false, kDSteps>(tmem_base + kTmDP, sv, sdo(b ^ 1), kIdS, false);  // dP^T(i+1), behind dK(i)
          umma_commit(dp_full);
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- algebra, then the epilogue: two threads per KEY row ----------------
    // Warps 2..5 take the query columns 0..63 of their rows, warps 6..9 the columns 64..127.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const int tid = threadIdx.x - 64;  // 0 .. 255
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const int key = row0 + r;
    // query q (global index) sees this key iff q >= q_min (and q < seq_q, which the statistics encode)
    const int q_min = (key < p.seq_kv) ? (p.causal ? key - p.causal_offset : INT32_MIN) : INT32_MAX;
    bool ok = true;
    // The (lse2, delta) pairs of the 128 queries of a tile go to shared memory, one value per thread
    // (threads 0..127 the statistic, 128..255 delta).  The values of iteration i + 1 are fetched at
    // the top of iteration i and stored at its end, so the global-memory latency is off the chain.
    auto fetch_stat = [&](int it) -> float {
      float val = (tid < 128) ? INFINITY : 0.f;  // a query past the end: P = exp2(x - inf) = 0
      if (it < total) {
        const int g_ = it / n;
        const int q_g = (qt_lo + (it - g_ * n)) * kRows + (tid & 127);
        if (q_g < p.seq_q) {
          const int64_t idx = (static_cast<int64_t>(batch) * p.q_heads + kvh * group + g_) * p.seq_q + q_g;
          if (tid < 128)
            val = p.lse_in ? lse_to_log2(__ldg(p.lse_in + idx)) : __ldg(p.lse2 + idx);
          else
            val = __ldg(p.delta + idx);
        }
      }
      return val;
    };
    if (total > 0) {
      vec[tid] = fetch_stat(0);
      asm volatile("bar.sync 3, 256;" ::: "memory");
    }
    for (int i = 0; i < total; ++i) {
      const int g = i / n;
      const int qt = qt_lo + (i - g * n);
      const int q_base = qt * kRows;
      const float next_stat = fetch_stat(i + 1);
      const float* lse_v = vec + (i & 1) * 256 + half * 64;
      const float* dl_v = lse_v + 128;
      const int q0 = q_base + half * 64;  // first query column of this thread
      float pf[64];
      if (ok && !mbar_wait(s_full, i & 1, abort_word)) ok = false;
      if (ok) {
        tc_fence_after();
        uint32_t s64[64];
        tmem_ld_32x32b_x64(lane_base + kTmS + half * 64, s64);
        tmem_wait_ld();
        uint32_t pw[32];
        if (q0 >= q_min) {  // every query of the chunk sees this key: no per-element test
#pragma unroll
          for (int c = 0; c < 64; c += 4) {
            const float4 l4 = *reinterpret_cast<const float4*>(lse_v + c);
            const float x0 = fmaf(__uint_as_float(s64[c]), p.scale_log2, -l4.x);
            const float x1 = fmaf(__uint_as_float(s64[c + 1]), p.scale_log2, -l4.y);
            const float x2 = fmaf(__uint_as_float(s64[c + 2]), p.scale_log2, -l4.z);
            const float x3 = fmaf(__uint_as_float(s64[c + 3]), p.scale_log2, -l4.w);
            const float2 e0 = exp2_poly2(make_float2(x0, x1));  // one pair on the FMA pipe, one on the SFU
            pf[c] = e0.x;
            pf[c + 1] = e0.y;
            pf[c + 2] = ex2_approx(x2);
            pf[c + 3] = ex2_approx(x3);
          }
        } else {
#pragma unroll
          for (int c = 0; c < 64; ++c)
            pf[c] = (q0 + c >= q_min) ? ex2_approx(fmaf(__uint_as_float(s64[c]), p.scale_log2, -lse_v[c])) : 0.f;
        }
#pragma unroll
        for (int c = 0; c < 64; c += 2) pw[c >> 1] = pack2<T>(pf[c], pf[c + 1]);
        tmem_st_32x32b_x32(lane_base + kTmS + half * 64, pw);  // over the first half of this thread's own S columns
        tmem_wait_st();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      if (ok && !mbar_wait(dp_full, i & 1, abort_word)) ok = false;
      if (ok) {
        tc_fence_after();
        uint32_t dp64[64];
        tmem_ld_32x32b_x64(lane_base + kTmDP + half * 64, dp64);
        tmem_wait_ld();
        uint32_t dsw[32];
#pragma unroll
        for (int c = 0; c < 64; c += 4) {
          const float4 d4 = *reinterpret_cast<const float4*>(dl_v + c);
          dsw[c >> 1] = pack2<T>(pf[c] * (__uint_as_float(dp64[c]) - d4.x), pf[c + 1] * (__uint_as_float(dp64[c + 1]) - d4.y));
          dsw[(c >> 1) + 1] =
              pack2<T>(pf[c + 2] * (__uint_as_float(dp64[c + 2]) - d4.z), pf[c + 3] * (__uint_as_float(dp64[c + 3]) - d4.w));
        }
        tmem_st_32x32b_x32(lane_base + kTmDP + half * 64, dsw);
        tmem_wait_st();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
      // every thread is done with this iteration's statistics and with the other buffer (read one
      // iteration ago): publish the next ones
      vec[((i + 1) & 1) * 256 + tid] = next_stat;
      asm volatile("bar.sync 3, 256;" ::: "memory");
    }
    if (ok && total > 0) ok = mbar_wait(it_done + ((total - 1) & 1), ((total - 1) >> 1) & 1, abort_word);
    ok = bar_red_and(1, kSoftmaxThreads, ok);
    if (ok) {
      tc_fence_after();
      // accumulators -> 16-bit tiles in the (now unused) Q / dO buffers -> TMA stores
#pragma unroll
      for (int o = 0; o < 2; ++o) {
        uint8_t* stage = smem + (o == 0 ? kTQ0 : kTDO0);
        const uint32_t acc = lane_base + (o == 0 ? kTmAcc0 : kTmAcc1);
        const float f = o == 1 ? p.scale : 1.f;  // dK carries the softmax scale
#pragma unroll 1
        for (int cc = 0; cc < 2; ++cc) {
          const int c4 = half * 2 + cc;
          if (c4 * 32 >= HD) continue;
          uint32_t v[32], w[16];
          if (total > 0) {
            tmem_ld_32x32b_x32(acc + c4 * 32, v);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int k = 0; k < 32; ++k) v[k] = 0u;  // no query sees these keys
          }
#pragma unroll
          for (int k = 0; k < 32; k += 2)
            w[k >> 1] = pack2<T>(__uint_as_float(v[k]) * f, __uint_as_float(v[k + 1]) * f);
          store_row_chunk(stage, r, c4 * 32, w);
        }
      }
      fence_proxy_async_smem();
      asm volatile("bar.sync 2, 256;" ::: "memory");
      if (r == 0 && half == 0) {
        tma_store_4d(&tmap_dv, smem + kTQ0, 0, row0, kvh, batch);
        if (HD == 128) tma_store_4d(&tmap_dv, smem + kTQ0 + kHalfBytes, 64, row0, kvh, batch);
        tma_store_4d(&tmap_dk, smem + kTDO0, 0, row0, kvh, batch);
        if (HD == 128) tma_store_4d(&tmap_dk, smem + kTDO0 + kHalfBytes, 64, row0, kvh, batch);
        tma_store_commit();
        tma_store_wait_read<0>();  // the staging tile has been read: the CTA may go (the writes land before the grid ends)
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0 && threadIdx.x == 0 && p.status) atomicOr(p.status, kStatusBwdTimeout);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b, h, i] = sum_d dO[b, h, i, d] * O[b, h, i, d].  A row of HD 16-bit values is HD / 8 lanes
// of 16 bytes; a warp takes 32 / (HD / 8) rows at a time and eight such groups, all loads issued
// before the first use, so that enough bytes are in flight to run at memory speed.
template <typename T, int HD>
__global__ void attn_bwd_delta_kernel(const T* __restrict__ o, const T* __restrict__ d_o, float* __restrict__ delta,
                                      int64_t rows, int q_heads, int seq_q, int64_t o_sb, int64_t o_sh, int64_t o_ss,
                                      int64_t do_sb, int64_t do_sh, int64_t do_ss) {
  constexpr int kLanesPerRow = HD / 8;
  constexpr int kRowsPerPass = 32 / kLanesPerRow;
  constexpr int kPasses = 8;
  const int lane = threadIdx.x & 31;
  const int sub = lane / kLanesPerRow, col = (lane % kLanesPerRow) * 8;
  const int64_t warp_id = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t row_base = warp_id * (kRowsPerPass * kPasses);
  uint4 ov[kPasses], dv[kPasses];
#pragma unroll
  for (int ps = 0; ps < kPasses; ++ps) {
    const int64_t row = row_base + ps * kRowsPerPass + sub;
    ov[ps] = make_uint4(0, 0, 0, 0);
    dv[ps] = make_uint4(0, 0, 0, 0);
    if (row < rows) {
      const int r32 = static_cast<int>(row);  // the host keeps rows below 2^31: 32-bit divisions
      const int bh = r32 / seq_q;
      const int i = r32 - bh * seq_q;
      const int b = bh / q_heads, h = bh - b * q_heads;
      ov[ps] = *reinterpret_cast<const uint4*>(o + b * o_sb + h * o_sh + i * o_ss + col);
      dv[ps] = *reinterpret_cast<const uint4*>(d_o + b * do_sb + h * do_sh + i * do_ss + col);
    }
  }
#pragma unroll
  for (int ps = 0; ps < kPasses; ++ps) {
    const T* oe = reinterpret_cast<const T*>(&ov[ps]);
    const T* de = reinterpret_cast<const T*>(&dv[ps]);
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) acc += static_cast<float>(oe[k]) * static_cast<float>(de[k]);
#pragma unroll
    for (int sft = kLanesPerRow / 2; sft > 0; sft >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, sft);
    const int64_t row = row_base + ps * kRowsPerPass + sub;
    if (lane % kLanesPerRow == 0 && row < rows) delta[row] = acc;
  }
}

struct BwdMaps {
  CUtensorMap q, d_o, k, v, dq, dk, dv;
};

int encode_bshd(CUtensorMap* out, int dtype, const void* base, int head_dim, int seq, int heads, int batch, int64_t sb,
                int64_t sh, int64_t ss) {
  const uint32_t box[4] = {64, kRows, 1, 1};
  uint64_t dims[4] = {static_cast<uint64_t>(head_dim), static_cast<uint64_t>(seq), static_cast<uint64_t>(heads), static_cast<uint64_t>(batch)};
  uint64_t st[3] = {static_cast<uint64_t>(ss) * 2, static_cast<uint64_t>(sh) * 2, static_cast<uint64_t>(sb) * 2};
  return encode_tmap(out, dtype, 4, const_cast<void*>(base), dims, st, box);
}

template <typename T, int HD>
int launch_bwd_typed(const b200k_attention_bwd_args& a, const BwdMaps& tm, const BwdParams& p, cudaStream_t stream) {
  auto k_dq = attn_bwd_dq_kernel<T, HD>;
  auto k_dkv = attn_bwd_dkv_t_kernel<T, HD>;
  static bool configured_dq[64] = {}, configured_dkv[64] = {};  // per instantiation and device ordinal
  int rc = ensure_dynamic_smem(k_dq, dq_smem_bytes(), configured_dq, "cudaFuncSetAttribute(attention bwd dq smem)");
  if (rc) return rc;
  rc = ensure_dynamic_smem(k_dkv, dkvt_smem_bytes(), configured_dkv, "cudaFuncSetAttribute(attention bwd dkv smem)");
  if (rc) return rc;
  const int64_t rows = static_cast<int64_t>(a.batch) * a.q_heads * a.seq_q;
  if (rows > INT32_MAX) return set_error(B200K_ERR_BAD_SHAPE, "attention_bwd: batch * q_heads * seq_q must be below 2^31");
  const int warps_per_block = 8;
  const int64_t rows_per_block = static_cast<int64_t>(warps_per_block) * (32 / (HD / 8)) * 8;
  attn_bwd_delta_kernel<T, HD><<<static_cast<unsigned>((rows + rows_per_block - 1) / rows_per_block),
                             warps_per_block * 32, 0, stream>>>(
      static_cast<const T*>(a.o), static_cast<const T*>(a.d_o), p.delta, rows, a.q_heads, a.seq_q, a.o_stride_b,
      a.o_stride_h, a.o_stride_s, a.do_stride_b, a.do_stride_h, a.do_stride_s);
  rc = check_cuda(cudaGetLastError(), "attn_bwd_delta_kernel launch");
  if (rc) return rc;
  const int grid_dq = a.batch * a.q_heads * p.num_q_tiles;
  k_dq<<<grid_dq, kBwdThreads, dq_smem_bytes(), stream>>>(tm.q, tm.d_o, tm.k, tm.v, tm.dq, p);
  rc = check_cuda(cudaGetLastError(), "attn_bwd_dq_kernel launch");
  if (rc) return rc;
  const int grid_dkv = a.batch * a.kv_heads * p.num_kv_tiles;
  k_dkv<<<grid_dkv, kBwdThreads, dkvt_smem_bytes(), stream>>>(tm.q, tm.d_o, tm.k, tm.v, tm.dv, tm.dk, p);
  return check_cuda(cudaGetLastError(), "attn_bwd_dkv_t_kernel launch");
}

}  // namespace

uint64_t attention_bwd_workspace_bytes(const b200k_attention_bwd_args& a) {
  if (a.batch <= 0 || a.q_heads <= 0 || a.seq_q <= 0) return 0;
  return 2ull * sizeof(float) * static_cast<uint64_t>(a.batch) * a.q_heads * a.seq_q;
}

int launch_attention_bwd(const b200k_attention_bwd_args& a, cudaStream_t stream) {
  if (!a.q || !a.k || !a.v || !a.o || !a.d_o || !a.d_q || !a.d_k || !a.d_v)
    return set_error(B200K_ERR_NULL, "attention_bwd: q, k, v, o, d_o, d_q, d_k, d_v must be non-NULL");
  if (a.batch <= 0 || a.q_heads <= 0 || a.kv_heads <= 0 || a.seq_q <= 0 || a.seq_kv <= 0)
    return set_error(B200K_ERR_BAD_SHAPE, "attention_bwd: all dimensions must be positive");
  if (a.head_dim != 128 && a.head_dim != 64)
    return set_error(B200K_ERR_BAD_SHAPE, "attention_bwd: head_dim must be 128 or 64");
  if (a.q_heads % a.kv_heads != 0)
    return set_error(B200K_ERR_BAD_SHAPE, "attention_bwd: q_heads must be a multiple of kv_heads");
  if (a.dtype != B200K_F16 && a.dtype != B200K_BF16)
    return set_error(B200K_ERR_BAD_DTYPE, "attention_bwd: dtype must be F16 or BF16");
  const int64_t strides[] = {a.q_stride_b,  a.q_stride_h,  a.q_stride_s,  a.k_stride_b,  a.k_stride_h,  a.k_stride_s,
                             a.v_stride_b,  a.v_stride_h,  a.v_stride_s,  a.o_stride_b,  a.o_stride_h,  a.o_stride_s,
                             a.do_stride_b, a.do_stride_h, a.do_stride_s, a.dq_stride_b, a.dq_stride_h, a.dq_stride_s,
                             a.dk_stride_b, a.dk_stride_h, a.dk_stride_s, a.dv_stride_b, a.dv_stride_h, a.dv_stride_s};
  for (int64_t s : strides)
    if (s <= 0 || s % 8 != 0)
      return set_error(B200K_ERR_BAD_ALIGN, "attention_bwd: every stride must be a positive multiple of 8 elements");
  const void* ptrs[] = {a.q, a.k, a.v, a.o, a.d_o, a.d_q, a.d_k, a.d_v};
  for (const void* ptr : ptrs)
    if (reinterpret_cast<uintptr_t>(ptr) & 15)
      return set_error(B200K_ERR_BAD_ALIGN, "attention_bwd: every tensor must be 16-byte aligned");
  if (!(a.scale > 0.f)) return set_error(B200K_ERR_BAD_SHAPE, "attention_bwd: scale must be positive");
  if (reinterpret_cast<uintptr_t>(a.lse) & 3)
    return set_error(B200K_ERR_BAD_ALIGN, "attention_bwd: lse must be 4-byte aligned");
  const uint64_t need = attention_bwd_workspace_bytes(a);
  if (!a.workspace || a.workspace_bytes < need || (reinterpret_cast<uintptr_t>(a.workspace) & 15))
    return set_error(B200K_ERR_WORKSPACE, "attention_bwd: workspace must be 16-byte aligned and hold %llu bytes",
                     static_cast<unsigned long long>(need));
  int rc = ensure_sm100();
  if (rc) return rc;

  BwdMaps tm;
  rc = encode_bshd(&tm.q, a.dtype, a.q, a.head_dim, a.seq_q, a.q_heads, a.batch, a.q_stride_b, a.q_stride_h, a.q_stride_s);
  if (!rc) rc = encode_bshd(&tm.d_o, a.dtype, a.d_o, a.head_dim, a.seq_q, a.q_heads, a.batch, a.do_stride_b, a.do_stride_h, a.do_stride_s);
  if (!rc) rc = encode_bshd(&tm.k, a.dtype, a.k, a.head_dim, a.seq_kv, a.kv_heads, a.batch, a.k_stride_b, a.k_stride_h, a.k_stride_s);
  if (!rc) rc = encode_bshd(&tm.v, a.dtype, a.v, a.head_dim, a.seq_kv, a.kv_heads, a.batch, a.v_stride_b, a.v_stride_h, a.v_stride_s);
  if (!rc) rc = encode_bshd(&tm.dq, a.dtype, a.d_q, a.head_dim, a.seq_q, a.q_heads, a.batch, a.dq_stride_b, a.dq_stride_h, a.dq_stride_s);
  if (!rc) rc = encode_bshd(&tm.dk, a.dtype, a.d_k, a.head_dim, a.seq_kv, a.kv_heads, a.batch, a.dk_stride_b, a.dk_stride_h, a.dk_stride_s);
  if (!rc) rc = encode_bshd(&tm.dv, a.dtype, a.d_v, a.head_dim, a.seq_kv, a.kv_heads, a.batch, a.dv_stride_b, a.dv_stride_h, a.dv_stride_s);
  if (rc) return rc;

  BwdParams p;
  p.batch = a.batch;
  p.q_heads = a.q_heads;
  p.kv_heads = a.kv_heads;
  p.seq_q = a.seq_q;
  p.seq_kv = a.seq_kv;
  p.causal = a.causal ? 1 : 0;
  p.causal_offset = a.seq_kv - a.seq_q;
  p.num_q_tiles = (a.seq_q + kRows - 1) / kRows;
  p.num_kv_tiles = (a.seq_kv + kRows - 1) / kRows;
  {
    // heads interleaved at a time: about four waves of CTAs (a handful of CTAs per head in flight)
    const int sms = num_sms();
    auto group_for = [&](int tiles, int num_bh) {
      const int g = (4 * sms + tiles - 1) / tiles;
      return g < 1 ? 1 : (g > num_bh ? num_bh : g);
    };
    p.bh_group_q = group_for(p.num_q_tiles, a.batch * a.q_heads);
    p.bh_group_kv = group_for(p.num_kv_tiles, a.batch * a.kv_heads);
  }
  if (static_cast<int64_t>(a.batch) * a.q_heads * p.num_q_tiles > INT32_MAX ||
      static_cast<int64_t>(a.batch) * a.kv_heads * p.num_kv_tiles > INT32_MAX)
    return set_error(B200K_ERR_BAD_SHAPE, "attention_bwd: too many tiles");
  p.scale = a.scale;
  p.scale_log2 = a.scale * kLog2eBwd;
  p.lse_in = a.lse;
  p.lse2 = static_cast<float*>(a.workspace);
  p.delta = p.lse2 + static_cast<int64_t>(a.batch) * a.q_heads * a.seq_q;
  p.status = a.status;
  if (a.head_dim == 64) {
    if (a.dtype == B200K_F16) return launch_bwd_typed<__half, 64>(a, tm, p, stream);
    return launch_bwd_typed<__nv_bfloat16, 64>(a, tm, p, stream);
  }
  if (a.dtype == B200K_F16) return launch_bwd_typed<__half, 128>(a, tm, p, stream);
  return launch_bwd_typed<__nv_bfloat16, 128>(a, tm, p, stream);
}

}  // namespace b200k
