// Attention forward (vanilla and causal) on sm_100a.
//
// One CTA owns 256 query rows of one (batch, head): two 128-row query tiles that ping-pong on
// the tensor core so that the softmax of one tile overlaps the MMAs of the other.
//
//   warps 0..3    softmax + correction + epilogue for query tile 0   (warpgroup 0)
//   warps 4..7    the same for query tile 1                          (warpgroup 1)
//   warp 8        TMA loads: Q tiles once, then K_j and V_j into two 2-stage rings
//   warp 9        issues every tcgen05.mma and owns tensor memory
//   warps 10, 11  idle; they complete warpgroup 2 so that it can hand its registers
//                 (setmaxnreg) to the two softmax warpgroups, which keep a whole score row
//                 (128 fp32) per thread in registers
//
// Tensor memory (512 columns x 128 lanes):  S0 | S1 | O0 | O1, 128 fp32 columns each.  The
// probabilities P (16-bit, two per column) overwrite the first 64 columns of their S tile and
// feed the second MMA directly from tensor memory, so they never touch shared memory.
//
// Per KV tile j and query tile i:  S_i = Q_i K_j^T  ->  softmax warps read S_i (one thread owns
// one row, so row max / row sum need no cross-thread traffic), write P_i  ->  O_i += P_i V_j.
// MMAs issued by one thread complete in order, so "S_i(j+1) is issued after O_i += P_i(j) V_j"
// is all that is needed to let P and S share columns.
//
// The running max is kept in log2 units (scores are multiplied by scale * log2(e) inside the
// exponent's FMA).  O is only rescaled when a row's max grows by more than 2^8; until then the
// stale max is used for both P and the running sum, which is exact after the final division.
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace b200k {
namespace {

constexpr int kAttnThreads = 384;
constexpr int kRegsSoftmax = 216;  // per SM sub-partition the CTA owns 3 warps x 168 registers = 504 per lane at launch;
                                    // setmaxnreg only redistributes that: 2*216 + 72 = 504 (anything larger never completes);
                                    // this split compiles both roles without spills
constexpr int kRegsOther = 72;
constexpr int kTileRows = 128;  // query rows per tile, KV rows per tile
constexpr int kD = 128;
constexpr int kHalfTileBytes = kTileRows * 128;     // one 64-element column block: 16 KB
constexpr int kTileBytes = 2 * kHalfTileBytes;      // 32 KB
constexpr int kQOffset = 0;                         // 2 tiles
constexpr int kKOffset = 2 * kTileBytes;            // 2 stages
constexpr int kVOffset = 4 * kTileBytes;            // 2 stages
constexpr int kBarOffset = 6 * kTileBytes;          // 192 KB
constexpr int kNumBars = 15;
constexpr int kAttnSmem = kBarOffset + kNumBars * 8 + 16 + 1024;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;

struct AttnParams {
  void* o;
  int64_t o_stride_b, o_stride_h, o_stride_s;
  int32_t batch, q_heads, kv_heads, seq_q, seq_kv;
  int32_t causal, causal_offset;
  int32_t num_q_blocks;
  float scale_log2;
  int32_t* status;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^x for a pair on the FMA pipe instead of the special-function unit: x = j + f with j = rint(x)
// taken from the low mantissa bits of x + 1.5 * 2^23, 2^f on [-0.5, 0.5] by a degree-3 polynomial
// (max relative error 7.5e-5, far below the rounding of P to 16 bits), exponent added as an integer.
// Inputs below -125 (including -inf from masking) give about 2^-125, which rounds to nothing in P.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
  x.x = fmaxf(x.x, -125.f);
  x.y = fmaxf(x.y, -125.f);
  const float2 t = fadd2(x, make_float2(12582912.f, 12582912.f));
  const float2 j = fadd2(t, make_float2(-12582912.f, -12582912.f));
  const float2 f = ffma2(j, make_float2(-1.f, -1.f), x);
  float2 p = ffma2(f, make_float2(0.0551716648f, 0.0551716648f), make_float2(0.2426111251f, 0.2426111251f));
  p = ffma2(p, f, make_float2(0.6932609677f, 0.6932609677f));
  p = ffma2(p, f, make_float2(0.9999280572f, 0.9999280572f));
  float2 r;
  r.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23));
  r.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23));
  return r;
}

// Which of every 8 consecutive column pairs take the polynomial instead of ex2.approx (bit i = pair i).
constexpr uint32_t kPolyPairMask = 0x92u;  // 3 of 8

template <typename T>
__device__ __forceinline__ uint32_t pack_pair(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack_pair<__half>(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Number of KV tiles a query tile starting at row r0 has to visit.
__device__ __forceinline__ int kv_tiles_for(int r0, const AttnParams& p, int kv_tiles_total) {
  if (!p.causal) return kv_tiles_total;
  const int last_col = r0 + kTileRows - 1 + p.causal_offset;
  if (last_col < 0) return 0;
  return min(last_col / kTileRows + 1, kv_tiles_total);
}

// Optional timeline capture (compile with -DB200K_ATTN_TRACE): block (0,0,0) records
// (tag, clock64) pairs per role into the buffer passed as the status pointer, 256 events per role:
// role 0 = TMA thread, 1 = MMA thread, 2 = softmax tile 0 (thread 0), 3 = softmax tile 1.
#ifdef B200K_ATTN_TRACE
#define ATTN_TRACE(role, tag)                                                          \
  do {                                                                                 \
    if (trace_on && trace_n < 256) {                                                   \
      long long* tb = reinterpret_cast<long long*>(p.status) + ((role)*256 + trace_n) * 2; \
      tb[0] = (tag);                                                                   \
      tb[1] = clock64();                                                               \
      ++trace_n;                                                                       \
    }                                                                                  \
  } while (0)
#else
#define ATTN_TRACE(role, tag) \
  do {                        \
  } while (0)
#endif

template <typename T>
__global__ void __launch_bounds__(kAttnThreads, 1)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  constexpr uint32_t kFmt = std::is_same<T, __half>::value ? kFmtF16 : kFmtBF16;
  constexpr uint32_t kIdescS = make_idesc(kFmt, kFmt, 128, 128, 0, 0);   // Q, K both K-major
  constexpr uint32_t kIdescPV = make_idesc(kFmt, kFmt, 128, 128, 0, 1);  // V is MN-major

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kBarOffset);
  uint64_t* q_full = bars;         // 1
  uint64_t* k_full = bars + 1;     // 2
  uint64_t* k_empty = bars + 3;    // 2
  uint64_t* v_full = bars + 5;     // 2
  uint64_t* v_empty = bars + 7;    // 2
  uint64_t* s_full = bars + 9;     // 2 (per query tile)
  uint64_t* p_full = bars + 11;    // 2
  uint64_t* o_done = bars + 13;    // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
  volatile uint32_t* abort_word = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
#ifdef B200K_ATTN_TRACE
  const bool trace_on = (blockIdx.x | blockIdx.y | blockIdx.z) == 0 && p.status != nullptr && lane == 0;
  int trace_n = 0;
#endif

  // Heaviest blocks first: under a causal mask the last query rows see the most keys.
  const int qblock = p.num_q_blocks - 1 - static_cast<int>(blockIdx.x);
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int kv_head = head / (p.q_heads / p.kv_heads);
  const int kv_tiles_total = (p.seq_kv + kTileRows - 1) / kTileRows;
  const int n0 = kv_tiles_for(qblock * 256, p, kv_tiles_total);
  const int n1 = kv_tiles_for(qblock * 256 + kTileRows, p, kv_tiles_total);  // n1 >= n0

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(k_full + i, 1);
      mbar_init(k_empty + i, 1);
      mbar_init(v_full + i, 1);
      mbar_init(v_empty + i, 1);
      mbar_init(s_full + i, 1);
      mbar_init(p_full + i, 4);
      mbar_init(o_done + i, 1);
    }
    *abort_word = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= 8) {
    // Warpgroup 2 (TMA, MMA, two idle warps) gives registers back for the softmax warpgroups.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
    if (warp == 8) {
    // ---------------- TMA producer ----------------
    if (lane == 0 && n1 > 0) {
      mbar_arrive_expect_tx(q_full, 2 * kTileBytes);
#pragma unroll
      for (int tile = 0; tile < 2; ++tile)
#pragma unroll
        for (int db = 0; db < 2; ++db)
          tma_load_4d(smem + kQOffset + tile * kTileBytes + db * kHalfTileBytes, &tmap_q, q_full, db * 64,
                      qblock * 256 + tile * kTileRows, head, batch);
      for (int j = 0; j < n1; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(k_empty + st, ph ^ 1, abort_word)) break;
        ATTN_TRACE(0, 100 + j);
        mbar_arrive_expect_tx(k_full + st, kTileBytes);
#pragma unroll
        for (int db = 0; db < 2; ++db)
          tma_load_4d(smem + kKOffset + st * kTileBytes + db * kHalfTileBytes, &tmap_k, k_full + st, db * 64,
                      j * kTileRows, kv_head, batch);
        if (!mbar_wait(v_empty + st, ph ^ 1, abort_word)) break;
        ATTN_TRACE(0, 200 + j);
        mbar_arrive_expect_tx(v_full + st, kTileBytes);
#pragma unroll
        for (int db = 0; db < 2; ++db)
          tma_load_4d(smem + kVOffset + st * kTileBytes + db * kHalfTileBytes, &tmap_v, v_full + st, db * 64,
                      j * kTileRows, kv_head, batch);
      }
    }
    __syncwarp();
    } else if (warp == 9) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && n1 > 0) {
      const uint32_t sq = smem_u32(smem + kQOffset);
      const uint32_t sk = smem_u32(smem + kKOffset);
      const uint32_t sv = smem_u32(smem + kVOffset);
      // The issuing thread runs scalar, latency-bound code, and a 128x128x16 MMA lasts only 64
      // cycles, so the per-MMA issue cost must stay at a handful of instructions: descriptors are
      // split into a constant high word and a low word that is a precomputed base plus a
      // compile-time offset.
      const uint32_t hi_k = static_cast<uint32_t>(make_desc_kmajor_sw128(0) >> 32);
      const uint32_t hi_mn = static_cast<uint32_t>(make_desc_mnmajor_sw128(0, kHalfTileBytes) >> 32);
      const uint32_t q_lo = static_cast<uint32_t>(make_desc_kmajor_sw128(sq));
      const uint32_t k_lo = static_cast<uint32_t>(make_desc_kmajor_sw128(sk));
      const uint32_t v_lo = static_cast<uint32_t>(make_desc_mnmajor_sw128(sv, kHalfTileBytes));
      auto desc = [](uint32_t lo, uint32_t hi) { return (static_cast<uint64_t>(hi) << 32) | lo; };
      // S_tile = Q_tile K^T : 8 k-steps of 16 over the head dimension (two 64-wide blocks).
      auto issue_s = [&](int tile, int kstage) {
        const uint32_t a0 = q_lo + tile * (kTileBytes >> 4);
        const uint32_t b0 = k_lo + kstage * (kTileBytes >> 4);
        const uint32_t d = tmem_base + tile * 128;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = (ks >> 2) * (kHalfTileBytes >> 4) + 2 * (ks & 3);
          umma_f16_ss(d, desc(a0 + off, hi_k), desc(b0 + off, hi_k), kIdescS, ks > 0 ? 1u : 0u);
        }
        umma_commit(s_full + tile);
      };
      // O_tile += P_tile V : 8 k-steps of 16 KV rows; A from tensor memory, B = V (MN-major).
      auto issue_pv = [&](int tile, int vstage, bool first) {
        const uint32_t b0 = v_lo + vstage * (kTileBytes >> 4);
        const uint32_t d = tmem_base + 256 + tile * 128;
        const uint32_t a = tmem_base + tile * 128;
        umma_f16_ts(d, a, desc(b0, hi_mn), kIdescPV, first ? 0u : 1u);
#ifdef B200K_ATTN_TRACE_FINE
        ATTN_TRACE(1, 7000);
#endif
#pragma unroll
        for (int ks = 1; ks < 8; ++ks) {
          umma_f16_ts(d, a + ks * 8, desc(b0 + ks * (2048 >> 4), hi_mn), kIdescPV, 1u);
#ifdef B200K_ATTN_TRACE_FINE
          ATTN_TRACE(1, 7000 + ks);
#endif
        }
        umma_commit(o_done + tile);
      };

      bool ok = mbar_wait(q_full, 0, abort_word) && mbar_wait(k_full + 0, 0, abort_word);
      if (ok) {
        tc_fence_after();
        ATTN_TRACE(1, 1000);
        if (n0 > 0) issue_s(0, 0);
        issue_s(1, 0);
        umma_commit(k_empty + 0);
        ATTN_TRACE(1, 1001);
      }
      for (int j = 0; j < n1 && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const bool has_next = j + 1 < n1;
        const int nst = (j + 1) & 1;
        const uint32_t nph = ((j + 1) >> 1) & 1;
        if (!mbar_wait(v_full + st, ph, abort_word)) { ok = false; break; }
        ATTN_TRACE(1, 2000 + j);  // V_j landed
        if (j < n0) {
          if (!mbar_wait(p_full + 0, j & 1, abort_word)) { ok = false; break; }
          tc_fence_after();
          ATTN_TRACE(1, 3000 + j);  // P0_j ready, issuing PV0_j
          issue_pv(0, st, j == 0);
          ATTN_TRACE(1, 3500 + j);  // PV0_j issued
        }
        if (has_next) {
          if (!mbar_wait(k_full + nst, nph, abort_word)) { ok = false; break; }
          tc_fence_after();
          ATTN_TRACE(1, 4000 + j);  // K_{j+1} landed, issuing S0_{j+1}
          if (j + 1 < n0) issue_s(0, nst);
          ATTN_TRACE(1, 4500 + j);  // S0_{j+1} issued
        }
        if (!mbar_wait(p_full + 1, j & 1, abort_word)) { ok = false; break; }
        tc_fence_after();
        ATTN_TRACE(1, 5000 + j);  // P1_j ready, issuing PV1_j (+ S1_{j+1})
        issue_pv(1, st, j == 0);
        ATTN_TRACE(1, 5500 + j);  // PV1_j issued
        umma_commit(v_empty + st);
        if (has_next) {
          issue_s(1, nst);
          umma_commit(k_empty + nst);
        }
        ATTN_TRACE(1, 6000 + j);
      }
    }
    __syncwarp();
    }
  } else {
    // ---------------- softmax / correction / epilogue ----------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    const int tile = warp >> 2;
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int tile_r0 = qblock * 256 + tile * kTileRows;
    const int q_row = tile_r0 + row_in_tile;
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t t_s = tmem_base + lane_field + tile * 128;
    const uint32_t t_o = tmem_base + lane_field + 256 + tile * 128;
    const int n_mine = tile == 0 ? n0 : n1;
    const float scale_log2 = p.scale_log2;

    float m_used = -INFINITY;
    float2 l2 = make_float2(0.f, 0.f);
    bool ok = true;
    for (int j = 0; j < n_mine; ++j) {
      ok = mbar_wait(s_full + tile, j & 1, abort_word);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (quarter == 0) ATTN_TRACE(2 + tile, 100 + j);  // S_j visible

#ifdef B200K_ATTN_EXPERIMENT_NO_SOFTMAX
      // timing experiment: hand P back immediately (results are meaningless)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full + tile);
      continue;
#endif
      const int col0 = j * kTileRows;
      const bool need_mask =
          (p.causal && col0 + kTileRows - 1 > tile_r0 + p.causal_offset) || (col0 + kTileRows > p.seq_kv);
      int limit = kTileRows;  // columns [0, limit) of this tile are visible to this row
      if (need_mask) {
        int vis = p.seq_kv;
        if (p.causal) vis = min(vis, q_row + p.causal_offset + 1);
        limit = vis - col0;
      }

      // The whole score row (128 fp32) lives in registers: load it in two halves so the max of
      // the first half overlaps the load of the second.
      uint32_t sr[128];
      tmem_ld_32x32b_x64(t_s, sr);
      tmem_wait_ld();
      tmem_ld_32x32b_x64(t_s + 64, sr + 64);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (i >= limit) sr[i] = 0xff800000u;  // -inf
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 64; i += 4) {
        mx0 = fmax3(mx0, __uint_as_float(sr[i]), __uint_as_float(sr[i + 1]));
        mx1 = fmax3(mx1, __uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3]));
      }
      tmem_wait_ld();
      if (need_mask) {
#pragma unroll
        for (int i = 64; i < 128; ++i)
          if (i >= limit) sr[i] = 0xff800000u;
      }
#pragma unroll
      for (int i = 64; i < 128; i += 4) {
        mx0 = fmax3(mx0, __uint_as_float(sr[i]), __uint_as_float(sr[i + 1]));
        mx1 = fmax3(mx1, __uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3]));
      }
      if (quarter == 0) ATTN_TRACE(2 + tile, 200 + j);  // row loaded, max done
      const float m_new = fmaxf(mx0, mx1) * scale_log2;
      const bool grow = m_new > m_used + kRescaleThreshold;  // also true for the first finite max
      float alpha = 1.f;
      if (grow) {
        alpha = ex2(m_used - m_new);  // m_used = -inf gives 0
        m_used = m_new;
      }
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // S_j complete implies O += P V of step j-1 is complete (in-order completion), so O is idle.
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_o + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_32x32b_x32(t_o + c * 32, r);
        }
      }
      l2.x *= alpha;
      l2.y *= alpha;
      const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;
      const float2 scale2 = make_float2(scale_log2, scale_log2);
      const float2 negm2 = make_float2(-m_sub, -m_sub);

      // probabilities -> tensor memory (16-bit pairs over the first 64 columns of S); masked
      // scores are -inf and give exactly 0
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 x = ffma2(make_float2(__uint_as_float(sr[c * 32 + 2 * i]), __uint_as_float(sr[c * 32 + 2 * i + 1])),
                                 scale2, negm2);
          const float2 e = ((kPolyPairMask >> (i & 7)) & 1u) ? exp2_poly2(x) : make_float2(ex2(x.x), ex2(x.y));
          l2 = fadd2(l2, e);
          pk[i] = pack_pair<T>(e.x, e.y);
        }
        tmem_st_32x32b_x16(t_s + c * 16, pk);
      }
      if (quarter == 0) ATTN_TRACE(2 + tile, 300 + j);  // exponentials issued, P stores issued
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full + tile);
      if (quarter == 0) ATTN_TRACE(2 + tile, 400 + j);  // P signalled
    }

    // ---- epilogue: O / l -> global ----
    if (ok && n_mine > 0) {
      ok = mbar_wait(o_done + tile, (n_mine - 1) & 1, abort_word);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const float l = l2.x + l2.y;
      const float inv = (l > 0.f) ? 1.0f / l : 0.f;
      T* orow = reinterpret_cast<T*>(p.o) + batch * p.o_stride_b + head * p.o_stride_h +
                static_cast<int64_t>(q_row) * p.o_stride_s;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        if (n_mine > 0) {
          tmem_ld_32x32b_x32(t_o + c * 32, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (q_row < p.seq_q) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 u;
            u.x = pack_pair<T>(__uint_as_float(r[8 * v + 0]) * inv, __uint_as_float(r[8 * v + 1]) * inv);
            u.y = pack_pair<T>(__uint_as_float(r[8 * v + 2]) * inv, __uint_as_float(r[8 * v + 3]) * inv);
            u.z = pack_pair<T>(__uint_as_float(r[8 * v + 4]) * inv, __uint_as_float(r[8 * v + 5]) * inv);
            u.w = pack_pair<T>(__uint_as_float(r[8 * v + 6]) * inv, __uint_as_float(r[8 * v + 7]) * inv);
            reinterpret_cast<uint4*>(orow + c * 32)[v] = u;
          }
        }
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {
    }
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, kStatusAttnTimeout);
    __syncthreads();
  }
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <typename T>
int launch_typed(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p,
                 cudaStream_t stream) {
  auto kfn = attn_fwd_kernel<T>;
  static bool configured = false;
  if (!configured) {
    int rc = check_cuda(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem),
                        "cudaFuncSetAttribute(attention smem)");
    if (rc) return rc;
    configured = true;
  }
  dim3 grid(p.num_q_blocks, p.q_heads, p.batch);
  kfn<<<grid, kAttnThreads, kAttnSmem, stream>>>(tq, tk, tv, p);
  return check_cuda(cudaGetLastError(), "attn_fwd_kernel launch");
}

}  // namespace

int launch_attention_fwd(const b200k_attention_args& a, cudaStream_t stream) {
  if (!a.q || !a.k || !a.v || !a.o) return set_error(B200K_ERR_NULL, "attention_fwd: q, k, v and o must be non-NULL");
  if (a.batch <= 0 || a.q_heads <= 0 || a.kv_heads <= 0 || a.seq_q <= 0 || a.seq_kv <= 0)
    return set_error(B200K_ERR_BAD_SHAPE, "attention_fwd: all dimensions must be positive");
  if (a.head_dim != kD) return set_error(B200K_ERR_BAD_SHAPE, "attention_fwd: head_dim must be 128");
  if (a.q_heads % a.kv_heads != 0)
    return set_error(B200K_ERR_BAD_SHAPE, "attention_fwd: q_heads must be a multiple of kv_heads");
  if (a.dtype != B200K_F16 && a.dtype != B200K_BF16)
    return set_error(B200K_ERR_BAD_DTYPE, "attention_fwd: dtype must be F16 or BF16");
  if (a.batch > 65535 || a.q_heads > 65535)
    return set_error(B200K_ERR_BAD_SHAPE, "attention_fwd: batch and q_heads must be <= 65535");
  const int64_t strides[] = {a.q_stride_b, a.q_stride_h, a.q_stride_s, a.k_stride_b, a.k_stride_h, a.k_stride_s,
                             a.v_stride_b, a.v_stride_h, a.v_stride_s, a.o_stride_b, a.o_stride_h, a.o_stride_s};
  for (int64_t s : strides)
    if (s <= 0 || s % 8 != 0)
      return set_error(B200K_ERR_BAD_ALIGN, "attention_fwd: every stride must be a positive multiple of 8 elements");
  if ((reinterpret_cast<uintptr_t>(a.q) & 15) || (reinterpret_cast<uintptr_t>(a.k) & 15) ||
      (reinterpret_cast<uintptr_t>(a.v) & 15) || (reinterpret_cast<uintptr_t>(a.o) & 15))
    return set_error(B200K_ERR_BAD_ALIGN, "attention_fwd: q, k, v, o must be 16-byte aligned");
  if (!(a.scale > 0.f)) return set_error(B200K_ERR_BAD_SHAPE, "attention_fwd: scale must be positive");
  int rc = ensure_sm100();
  if (rc) return rc;

  CUtensorMap tq, tk, tv;
  const uint32_t box[4] = {64, kTileRows, 1, 1};
  {
    uint64_t dims[4] = {kD, static_cast<uint64_t>(a.seq_q), static_cast<uint64_t>(a.q_heads),
                        static_cast<uint64_t>(a.batch)};
    uint64_t st[3] = {static_cast<uint64_t>(a.q_stride_s) * 2, static_cast<uint64_t>(a.q_stride_h) * 2,
                      static_cast<uint64_t>(a.q_stride_b) * 2};
    rc = encode_tmap(&tq, a.dtype, 4, const_cast<void*>(a.q), dims, st, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[4] = {kD, static_cast<uint64_t>(a.seq_kv), static_cast<uint64_t>(a.kv_heads),
                        static_cast<uint64_t>(a.batch)};
    uint64_t st[3] = {static_cast<uint64_t>(a.k_stride_s) * 2, static_cast<uint64_t>(a.k_stride_h) * 2,
                      static_cast<uint64_t>(a.k_stride_b) * 2};
    rc = encode_tmap(&tk, a.dtype, 4, const_cast<void*>(a.k), dims, st, box);
    if (rc) return rc;
    uint64_t sv[3] = {static_cast<uint64_t>(a.v_stride_s) * 2, static_cast<uint64_t>(a.v_stride_h) * 2,
                      static_cast<uint64_t>(a.v_stride_b) * 2};
    rc = encode_tmap(&tv, a.dtype, 4, const_cast<void*>(a.v), dims, sv, box);
    if (rc) return rc;
  }

  AttnParams p;
  p.o = a.o;
  p.o_stride_b = a.o_stride_b;
  p.o_stride_h = a.o_stride_h;
  p.o_stride_s = a.o_stride_s;
  p.batch = a.batch;
  p.q_heads = a.q_heads;
  p.kv_heads = a.kv_heads;
  p.seq_q = a.seq_q;
  p.seq_kv = a.seq_kv;
  p.causal = a.causal ? 1 : 0;
  p.causal_offset = a.seq_kv - a.seq_q;
  p.num_q_blocks = (a.seq_q + 255) / 256;
  p.scale_log2 = a.scale * kLog2e;
  p.status = a.status;
  if (a.dtype == B200K_F16) return launch_typed<__half>(tq, tk, tv, p, stream);
  return launch_typed<__nv_bfloat16>(tq, tk, tv, p, stream);
}

}  // namespace b200k
