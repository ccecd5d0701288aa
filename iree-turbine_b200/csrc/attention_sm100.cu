// Attention forward (vanilla and causal) on sm_100a.
//
// Persistent CTAs, one per SM.  A work item is one 128-row query tile of one (batch, head); a CTA
// takes items blockIdx.x, blockIdx.x + gridDim.x, ... from a list ordered (batch, head)-major with
// the heaviest query tiles of a head first, so CTAs that run at the same time share K/V in L2.
//
//   warps 0..3    softmax + correction (one thread = one query row)             warpgroup 0
//   warps 4..7    epilogue: O / rowsum -> global, one item behind the others     warpgroup 1
//   warp 8        TMA loads: Q of the next item, then K_j (3 stages) / V_j (2)    warpgroup 2
//   warp 9        issues every tcgen05.mma and owns tensor memory
//   warps 10, 11  idle (complete warpgroup 2 for the setmaxnreg register hand-off)
//
// Tensor memory (512 columns x 128 lanes):  S[0] | S[1] | O[0] | O[1], 128 fp32 columns each.
//   * Two score buffers: the tensor core computes S(j+1) while the softmax works on S(j), so the
//     softmax never waits for scores and the per-step chain "softmax -> P V -> next scores" of a
//     single-buffer design is gone.  What remains is a throughput balance: about 1230 cycles of
//     softmax instructions per 128 x 128 tile on the four SM sub-partitions against 1024 cycles of
//     MMA (both measured with single-SM micro-benchmarks).
//   * Two output accumulators: the epilogue of item i runs while item i+1 is being computed.
//   * The probabilities P (16-bit, two per column) overwrite the first 64 columns of their score
//     buffer and are the A operand of the second MMA straight from tensor memory.  MMAs issued by
//     one thread complete in order, so issuing S(j+2) after "O += P(j) V(j)" is all that is needed
//     to reuse a buffer.
//
// Epilogue: accumulator -> registers -> 16-bit -> 128-byte-swizzled staging tile in shared memory
// -> two TMA stores (rows past the end of the sequence are clipped by the tensor map).  Direct
// row-per-thread global stores were measured at about 3000 cycles per item and delayed the TMA
// loads of the next item; the staged store is a few hundred.
//
// Softmax: running max in log2 units (scores are multiplied by scale * log2(e) inside the
// exponent's FMA); O is only rescaled when a row's max grows by more than 2^8 (stale max used for
// both P and the running sum, exact after the final division); 3 of every 8 column pairs take a
// degree-3 polynomial on the FMA pipe instead of ex2.approx to balance the special-function unit.
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace b200k {
namespace {

constexpr int kAttnThreads = 384;
// Registers: 3 warps per SM sub-partition x 168 at launch = 504 per lane, redistributed.
constexpr int kRegsSoftmax = 232;
constexpr int kRegsEpilogue = 128;
constexpr int kRegsOther = 72;
static_assert(kRegsSoftmax + kRegsEpilogue + kRegsOther <= 504, "setmaxnreg.inc would never complete");
constexpr int kTileRows = 128;  // query rows per item, KV rows per tile
constexpr int kD = 128;
constexpr int kHalfTileBytes = kTileRows * 128;  // one 64-element column block: 16 KB
constexpr int kTileBytes = 2 * kHalfTileBytes;   // 32 KB
constexpr int kKStages = 3;
constexpr int kVStages = 2;
constexpr int kQOffset = 0;
constexpr int kKOffset = kTileBytes;
constexpr int kVOffset = kKOffset + kKStages * kTileBytes;
constexpr int kOStageOffset = kVOffset + kVStages * kTileBytes;  // epilogue staging tile (layout of a Q tile)
constexpr int kLsumOffset = kOStageOffset + kTileBytes;          // float [2][128]: row sums for the epilogue
constexpr int kBarOffset = kLsumOffset + 2 * kTileRows * 4;
// q_full q_empty | k_full[3] k_empty[3] v_full[2] v_empty[2] | s_full[2] p_full[2] | o_done |
// o_full[2] o_free[2] l_full[2] l_free[2]
constexpr int kNumBars = 2 + 2 * kKStages + 2 * kVStages + 4 + 1 + 8;
constexpr int kAttnSmem = kBarOffset + kNumBars * 8 + 16 + 1024;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;

struct AttnParams {
  void* o;
  int64_t o_stride_b, o_stride_h, o_stride_s;
  int32_t batch, q_heads, kv_heads, seq_q, seq_kv;
  int32_t causal, causal_offset;
  int32_t num_q_tiles;  // ceil(seq_q / 128)
  int32_t num_items;    // batch * q_heads * num_q_tiles
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


struct Item {
  int qtile, head, batch, n;  // n = number of 128-row KV tiles this item visits
};

__device__ __forceinline__ Item decode_item(int idx, const AttnParams& p) {
  Item it;
  const int bh = idx / p.num_q_tiles;
  it.qtile = p.num_q_tiles - 1 - (idx - bh * p.num_q_tiles);  // heaviest tiles of a head first
  it.batch = bh / p.q_heads;
  it.head = bh - it.batch * p.q_heads;
  const int kv_tiles_total = (p.seq_kv + kTileRows - 1) / kTileRows;
  if (!p.causal) {
    it.n = kv_tiles_total;
  } else {
    const int last_col = it.qtile * kTileRows + kTileRows - 1 + p.causal_offset;
    it.n = last_col < 0 ? 0 : min(last_col / kTileRows + 1, kv_tiles_total);
  }
  return it;
}

template <typename T>
__global__ void __launch_bounds__(kAttnThreads, 1)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
                    const AttnParams p) {
  constexpr uint32_t kFmt = std::is_same<T, __half>::value ? kFmtF16 : kFmtBF16;
  constexpr uint32_t kIdescS = make_idesc(kFmt, kFmt, 128, 128, 0, 0);   // Q, K both K-major
  constexpr uint32_t kIdescPV = make_idesc(kFmt, kFmt, 128, 128, 0, 1);  // V is MN-major

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  float* lsum = reinterpret_cast<float*>(smem + kLsumOffset);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kBarOffset);
  uint64_t* q_full = bars;
  uint64_t* q_empty = bars + 1;
  uint64_t* k_full = bars + 2;
  uint64_t* k_empty = k_full + kKStages;
  uint64_t* v_full = k_empty + kKStages;
  uint64_t* v_empty = v_full + kVStages;
  uint64_t* s_full = v_empty + kVStages;  // [score buffer]
  uint64_t* p_full = s_full + 2;          // [score buffer]
  uint64_t* o_done = p_full + 2;          // one phase per "O += P V"
  uint64_t* o_full = o_done + 1;          // [output buffer] last P V of an item complete
  uint64_t* o_free = o_full + 2;          // [output buffer] epilogue has read it
  uint64_t* l_full = o_free + 2;          // [output buffer] row sums written
  uint64_t* l_free = l_full + 2;          // [output buffer] row sums read
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
  volatile uint32_t* abort_word = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
#ifdef B200K_ATTN_TRACE
  const bool trace_on = blockIdx.x == 0 && p.status != nullptr && lane == 0;
  int trace_n = 0;
#endif

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int i = 0; i < kKStages; ++i) {
      mbar_init(k_full + i, 1);
      mbar_init(k_empty + i, 1);
    }
    for (int i = 0; i < kVStages; ++i) {
      mbar_init(v_full + i, 1);
      mbar_init(v_empty + i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(s_full + i, 1);
      mbar_init(p_full + i, 4);
      mbar_init(o_full + i, 1);
      mbar_init(o_free + i, 4);
      mbar_init(l_full + i, 4);
      mbar_init(l_free + i, 4);
    }
    mbar_init(o_done, 1);
    *abort_word = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    prefetch_tmap(&tmap_o);
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int group = p.q_heads / p.kv_heads;

  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
    if (warp == 8) {
      // ---------------- TMA producer ----------------
      if (lane == 0) {
        uint32_t qc = 0, kc = 0, vc = 0;  // Q loads, K tiles, V tiles issued so far
        bool ok = true;
        for (int idx = blockIdx.x; idx < p.num_items && ok; idx += gridDim.x) {
          const Item it = decode_item(idx, p);
          if (it.n == 0) continue;
          const int kv_head = it.head / group;
          if (!mbar_wait(q_empty, (qc & 1) ^ 1, abort_word)) break;
          mbar_arrive_expect_tx(q_full, kTileBytes);
#pragma unroll
          for (int db = 0; db < 2; ++db)
            tma_load_4d(smem + kQOffset + db * kHalfTileBytes, &tmap_q, q_full, db * 64, it.qtile * kTileRows, it.head,
                        it.batch);
          ++qc;
          ATTN_TRACE(0, 9000);
          // Order: K_0, K_1, then V_j followed by K_(j+2): score tiles run two steps ahead of the
          // second MMA, so their operands are requested first.
          auto load_k = [&](int j) {
            const int ks = kc % kKStages;
            if (!mbar_wait(k_empty + ks, ((kc / kKStages) & 1) ^ 1, abort_word)) return false;
            mbar_arrive_expect_tx(k_full + ks, kTileBytes);
#pragma unroll
            for (int db = 0; db < 2; ++db)
              tma_load_4d(smem + kKOffset + ks * kTileBytes + db * kHalfTileBytes, &tmap_k, k_full + ks, db * 64,
                          j * kTileRows, kv_head, it.batch);
            ++kc;
            return true;
          };
          for (int jj = 0; jj < 2 && jj < it.n && ok; ++jj) ok = load_k(jj);
          for (int j = 0; j < it.n && ok; ++j) {
            const int vs = vc % kVStages;
            if (!mbar_wait(v_empty + vs, ((vc / kVStages) & 1) ^ 1, abort_word)) { ok = false; break; }
            mbar_arrive_expect_tx(v_full + vs, kTileBytes);
#pragma unroll
            for (int db = 0; db < 2; ++db)
              tma_load_4d(smem + kVOffset + vs * kTileBytes + db * kHalfTileBytes, &tmap_v, v_full + vs, db * 64,
                          j * kTileRows, kv_head, it.batch);
            ++vc;
            if (j + 2 < it.n) ok = load_k(j + 2);
          }
        }
      }
      __syncwarp();
    } else if (warp == 9) {
      // ---------------- MMA issuer ----------------
      if (lane == 0) {
        const uint32_t sq = smem_u32(smem + kQOffset);
        const uint32_t sk = smem_u32(smem + kKOffset);
        const uint32_t sv = smem_u32(smem + kVOffset);
        // The issuing thread runs scalar, latency-bound code: descriptors are a constant high word
        // plus a low word that is a precomputed base plus a compile-time offset.
        const uint32_t hi_k = static_cast<uint32_t>(make_desc_kmajor_sw128(0) >> 32);
        const uint32_t hi_mn = static_cast<uint32_t>(make_desc_mnmajor_sw128(0, kHalfTileBytes) >> 32);
        const uint32_t q_lo = static_cast<uint32_t>(make_desc_kmajor_sw128(sq));
        const uint32_t k_lo = static_cast<uint32_t>(make_desc_kmajor_sw128(sk));
        const uint32_t v_lo = static_cast<uint32_t>(make_desc_mnmajor_sw128(sv, kHalfTileBytes));
        auto desc = [](uint32_t lo, uint32_t hi) { return (static_cast<uint64_t>(hi) << 32) | lo; };
        // S[buf] = Q K^T : 8 k-steps of 16 over the head dimension (two 64-wide blocks).
        auto issue_s = [&](int buf, int kstage) {
          const uint32_t b0 = k_lo + kstage * (kTileBytes >> 4);
          const uint32_t d = tmem_base + buf * 128;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t off = (ks >> 2) * (kHalfTileBytes >> 4) + 2 * (ks & 3);
            umma_f16_ss(d, desc(q_lo + off, hi_k), desc(b0 + off, hi_k), kIdescS, ks > 0 ? 1u : 0u);
          }
          umma_commit(s_full + buf);
          umma_commit(k_empty + kstage);
        };
        // O[ob] (+)= P[buf] V : 8 k-steps of 16 KV rows; A from tensor memory, B = V (MN-major).
        auto issue_pv = [&](int ob, int buf, int vstage, bool first) {
          const uint32_t b0 = v_lo + vstage * (kTileBytes >> 4);
          const uint32_t d = tmem_base + 256 + ob * 128;
          const uint32_t a = tmem_base + buf * 128;
          umma_f16_ts(d, a, desc(b0, hi_mn), kIdescPV, first ? 0u : 1u);
#pragma unroll
          for (int ks = 1; ks < 8; ++ks) umma_f16_ts(d, a + ks * 8, desc(b0 + ks * (2048 >> 4), hi_mn), kIdescPV, 1u);
          umma_commit(v_empty + vstage);
          umma_commit(o_done);
        };

        uint32_t qc = 0, kc = 0, vc = 0, g = 0, ic = 0;  // Q tiles, K tiles, V tiles, KV steps, items so far
        bool ok = true;
        // Score tiles form one stream over all of this CTA's items and run two KV steps ahead of
        // the second MMA, across item boundaries: while the last two steps of an item finish, the
        // first two score tiles of the next item are already being computed.
        int s_idx = blockIdx.x;  // item the score cursor is in
        int s_j = 0;             // next score tile of that item
        Item s_it = {0, 0, 0, 0};
        auto seek_item = [&]() {  // positions the cursor on the next item that has work
          while (s_idx < p.num_items) {
            s_it = decode_item(s_idx, p);
            if (s_it.n > 0) return;
            s_idx += gridDim.x;
          }
        };
        uint32_t gs = 0;  // score tiles issued so far (global step index of the next one)
        auto issue_next_score = [&]() -> bool {
          if (s_idx >= p.num_items) return true;  // nothing left
          if (s_j == 0) {
            if (!mbar_wait(q_full, qc & 1, abort_word)) return false;
            ++qc;
          }
          const int ks = kc % kKStages;
          if (!mbar_wait(k_full + ks, (kc / kKStages) & 1, abort_word)) return false;
          tc_fence_after();
          ATTN_TRACE(1, 1000 + s_j);
          issue_s(gs & 1, ks);
          ++kc;
          ++gs;
          if (++s_j == s_it.n) {
            umma_commit(q_empty);  // Q is free once the item's last score MMA has run
            s_j = 0;
            s_idx += gridDim.x;
            seek_item();
          }
          return true;
        };
        seek_item();
        ok = issue_next_score() && issue_next_score();  // fill both score buffers
        for (int idx = blockIdx.x; idx < p.num_items && ok; idx += gridDim.x) {
          const Item it = decode_item(idx, p);
          if (it.n == 0) continue;
          const int ob = ic & 1;
          for (int j = 0; j < it.n; ++j, ++g) {
            const int buf = g & 1;
            const int vs = vc % kVStages;
            if (!mbar_wait(v_full + vs, (vc / kVStages) & 1, abort_word)) { ok = false; break; }
            if (!mbar_wait(p_full + buf, (g >> 1) & 1, abort_word)) { ok = false; break; }
            if (j == 0 && !mbar_wait(o_free + ob, ((ic >> 1) & 1) ^ 1, abort_word)) { ok = false; break; }
            tc_fence_after();
            ATTN_TRACE(1, 3000 + j);  // P_j ready
            issue_pv(ob, buf, vs, j == 0);
            ++vc;
            if (j == it.n - 1) umma_commit(o_full + ob);
            // the score buffer just consumed is refilled with the tile two steps ahead
            if (!issue_next_score()) { ok = false; break; }
            ATTN_TRACE(1, 6000 + j);
          }
          ++ic;
        }
      }
      __syncwarp();
    }
  } else if (warp >= 4) {
    // ---------------- epilogue: O / rowsum -> global, one item behind ----------------
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsEpilogue));
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    uint8_t* stage = smem + kOStageOffset;
    const bool store_thread = (warp == 4 && lane == 0);
    auto epi_barrier = [&]() { asm volatile("bar.sync 1, 128;" ::: "memory"); };
    uint32_t ic = 0;
    bool ok = true;
    for (int idx = blockIdx.x; idx < p.num_items && ok; idx += gridDim.x) {
      const Item it = decode_item(idx, p);
      if (it.n == 0) {
        // no visible key: zeros (rare; plain stores)
        const int q_row = it.qtile * kTileRows + row_in_tile;
        if (q_row < p.seq_q) {
          T* orow = reinterpret_cast<T*>(p.o) + it.batch * p.o_stride_b + it.head * p.o_stride_h +
                    static_cast<int64_t>(q_row) * p.o_stride_s;
#pragma unroll
          for (int v = 0; v < 16; ++v) reinterpret_cast<uint4*>(orow)[v] = make_uint4(0u, 0u, 0u, 0u);
        }
        continue;
      }
      const int ob = ic & 1;
      const uint32_t par = (ic >> 1) & 1;
      ok = mbar_wait(o_full + ob, par, abort_word) && mbar_wait(l_full + ob, par, abort_word);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (quarter == 0) ATTN_TRACE(3, 100);
      const float l = lsum[ob * kTileRows + row_in_tile];
      const float inv = (l > 0.f) ? 1.0f / l : 0.f;
      const uint32_t t_o = tmem_base + lane_field + 256 + ob * 128;
      // the staging tile is free once the previous item's TMA stores have read it
      if (store_thread) tma_store_wait_read<0>();
      epi_barrier();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_o + c * 32, r);
        tmem_wait_ld();
        uint8_t* blk = stage + (c >> 1) * kHalfTileBytes + row_in_tile * 128;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 u;
          u.x = pack_pair<T>(__uint_as_float(r[8 * v + 0]) * inv, __uint_as_float(r[8 * v + 1]) * inv);
          u.y = pack_pair<T>(__uint_as_float(r[8 * v + 2]) * inv, __uint_as_float(r[8 * v + 3]) * inv);
          u.z = pack_pair<T>(__uint_as_float(r[8 * v + 4]) * inv, __uint_as_float(r[8 * v + 5]) * inv);
          u.w = pack_pair<T>(__uint_as_float(r[8 * v + 6]) * inv, __uint_as_float(r[8 * v + 7]) * inv);
          const int chunk = (c & 1) * 4 + v;
          *reinterpret_cast<uint4*>(blk + ((chunk ^ (row_in_tile & 7)) << 4)) = u;
        }
      }
      // accumulator and row sums have been read: release them for the item after next
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(o_free + ob);
        mbar_arrive(l_free + ob);
      }
      fence_proxy_async_smem();
      epi_barrier();
      if (store_thread) {
        tma_store_4d(&tmap_o, stage, 0, it.qtile * kTileRows, it.head, it.batch);
        tma_store_4d(&tmap_o, stage + kHalfTileBytes, 64, it.qtile * kTileRows, it.head, it.batch);
        tma_store_commit();
      }
      if (quarter == 0) ATTN_TRACE(3, 200);
      ++ic;
    }
    if (store_thread) tma_store_wait<0>();
  } else {
    // ---------------- softmax / correction ----------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    const float scale_log2 = p.scale_log2;
    uint32_t g = 0, ic = 0;  // KV steps and items so far
    bool ok = true;
    for (int idx = blockIdx.x; idx < p.num_items && ok; idx += gridDim.x) {
      const Item it = decode_item(idx, p);
      if (it.n == 0) continue;
      const int ob = ic & 1;
      const int tile_r0 = it.qtile * kTileRows;
      const int q_row = tile_r0 + row_in_tile;
      const uint32_t t_o = tmem_base + lane_field + 256 + ob * 128;
      float m_used = -INFINITY;
      float2 l2 = make_float2(0.f, 0.f);
      for (int j = 0; j < it.n; ++j, ++g) {
        const int buf = g & 1;
        const uint32_t t_s = tmem_base + lane_field + buf * 128;
        ok = mbar_wait(s_full + buf, (g >> 1) & 1, abort_word);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (quarter == 0) ATTN_TRACE(2, 100 + j);  // S_j visible

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
        if (quarter == 0) ATTN_TRACE(2, 200 + j);  // row loaded, max done
        const float m_new = fmaxf(mx0, mx1) * scale_log2;
        const bool grow = m_new > m_used + kRescaleThreshold;  // also true for the first finite max
        // Every phase of o_done is observed exactly once, in order, and always before P of this
        // step is handed over: a parity wait only works within one phase of the barrier's current
        // one, and the score buffers run ahead of the second MMA.
        bool seen_prev_pv = (g == 0);
        if (j > 0 && __any_sync(0xffffffffu, grow)) {
          float alpha = 1.f;
          if (grow) alpha = ex2(m_used - m_new);  // m_used = -inf gives 0
          ok = mbar_wait(o_done, (g - 1) & 1, abort_word);  // O += P V of the previous step is done
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          seen_prev_pv = true;
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < 8; ++c) {
            uint32_t r[16];
            tmem_ld_32x32b_x16(t_o + c * 16, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32b_x16(t_o + c * 16, r);
          }
          l2.x *= alpha;
          l2.y *= alpha;
        }
        if (grow) m_used = m_new;
        const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;
        const float2 scale2 = make_float2(scale_log2, scale_log2);
        const float2 negm2 = make_float2(-m_sub, -m_sub);

        // probabilities -> tensor memory (16-bit pairs over the first 64 columns of this buffer);
        // masked scores are -inf and give (almost) exactly 0
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
        if (quarter == 0) ATTN_TRACE(2, 300 + j);  // exponentials done, P stores issued
        if (!seen_prev_pv) {
          ok = mbar_wait(o_done, (g - 1) & 1, abort_word);  // long complete by now
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full + buf);
        if (quarter == 0) ATTN_TRACE(2, 400 + j);  // P signalled
      }
      if (!ok) break;
      // hand the row sums to the epilogue warps
      ok = mbar_wait(l_free + ob, ((ic >> 1) & 1) ^ 1, abort_word);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      lsum[ob * kTileRows + row_in_tile] = l2.x + l2.y;
      __syncwarp();
      if (lane == 0) mbar_arrive(l_full + ob);
      ++ic;
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
int launch_typed(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to,
                 const AttnParams& p, cudaStream_t stream) {
  auto kfn = attn_fwd_kernel<T>;
  static bool configured = false;
  if (!configured) {
    int rc = check_cuda(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem),
                        "cudaFuncSetAttribute(attention smem)");
    if (rc) return rc;
    configured = true;
  }
  const int sms = num_sms();
  const int grid = p.num_items < sms ? p.num_items : sms;
  kfn<<<grid, kAttnThreads, kAttnSmem, stream>>>(tq, tk, tv, to, p);
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

  CUtensorMap tq, tk, tv, to;
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

  {
    uint64_t dims[4] = {kD, static_cast<uint64_t>(a.seq_q), static_cast<uint64_t>(a.q_heads),
                        static_cast<uint64_t>(a.batch)};
    uint64_t st[3] = {static_cast<uint64_t>(a.o_stride_s) * 2, static_cast<uint64_t>(a.o_stride_h) * 2,
                      static_cast<uint64_t>(a.o_stride_b) * 2};
    rc = encode_tmap(&to, a.dtype, 4, a.o, dims, st, box);
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
  p.num_q_tiles = (a.seq_q + kTileRows - 1) / kTileRows;
  const int64_t items = static_cast<int64_t>(a.batch) * a.q_heads * p.num_q_tiles;
  if (items > INT32_MAX) return set_error(B200K_ERR_BAD_SHAPE, "attention_fwd: too many query tiles");
  p.num_items = static_cast<int32_t>(items);
  p.scale_log2 = a.scale * kLog2e;
  p.status = a.status;
  if (a.dtype == B200K_F16) return launch_typed<__half>(tq, tk, tv, to, p, stream);
  return launch_typed<__nv_bfloat16>(tq, tk, tv, to, p, stream);
}

}  // namespace b200k
