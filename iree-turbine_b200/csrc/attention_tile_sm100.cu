// Attention forward (vanilla and causal), head dim 128, on sm_100a: the ONE-TILE kernel.
//
// Two kernels share the forward path (launch_attention_fwd in attention_sm100.cu chooses): this one,
// whose work item is a single 128-row query tile served by two softmax warpgroups on alternate KV
// steps with double-buffered score tiles, and the tile-pair kernel in attention_sm100.cu.  This one
// keeps both softmax warpgroups busy all the time and has the finer work granularity: it is the
// faster of the two on non-causal problems and where the pair kernel's units fill the SMs badly.
//
// Persistent CTAs, one per SM.  A work item is one 128-row query tile of one (batch, head); a CTA
// takes items blockIdx.x, blockIdx.x + gridDim.x, ... from a list ordered (batch, head)-major, so
// CTAs that run at the same time share K/V in L2, heaviest query tiles of a head first; a causal
// problem of a few rounds of items interleaves the tiles of all heads instead (see decode_item).
//
//   warps 0..3    softmax + correction of the even KV steps of the CTA (thread = query row)
//   warps 4..7    the same for the odd KV steps
//   warps 8..11   epilogue: O / rowsum -> global, one item behind the others
//   warp 12       TMA loads: Q of the next item, K_j (3 stages), V_j (2 stages)
//   warp 13       issues the score MMAs (S = Q K^T) and owns tensor memory
//   warp 14       issues the second MMAs (O += P V)
//   warp 15       idle (completes the fourth warpgroup for the setmaxnreg register hand-off)
//
// Tensor memory (512 columns x 128 lanes):  S[0] | S[1] (128 fp32 columns each) | P[0] | P[1]
// (64 columns each: 128 16-bit probabilities per row) | O (128 fp32 columns).
//   * Score tile g goes to S[g & 1] and is handled by softmax warpgroup g & 1, which writes P[g & 1].
//     The two warpgroups are half a step apart: while one is in its latency-bound part (wait,
//     tensor-memory load, row max, hand-over) the other runs its exponentials.  They share ONE
//     running row max and ONE accumulator: early in its step a warpgroup reads the running max the
//     other published half a step before, decides whether this tile raises it (by more than 2^8),
//     and publishes the result; only when it does raise it is O rescaled, by that warpgroup, after
//     "O += P V" of the previous step (the other warpgroup's) has completed and before its own P is
//     handed over.  Each warpgroup keeps a partial row sum relative to the running max it last saw;
//     the epilogue brings the two to the final max and adds them.
//   * A softmax thread holds its whole score row in registers, so a score buffer is free
//     again early in the step, as soon as the row has been loaded: S(j+2) is issued then.  The
//     probabilities have buffers of their own for that reason.  The tensor core is never what the
//     softmax waits for: neither the scores of the next step nor "O += P V" of the last one is on
//     its critical path.
//   * Two threads issue MMAs.  A tcgen05.mma does not return until the tensor pipe has room for
//     it, so a group of eight blocks its thread for about as long as it executes (plus some 300
//     cycles when the pipe was idle); with one issuing thread every wait of one kind of MMA
//     delayed the other.
//   * One output accumulator is enough: the first "O = P V" of an item is needed a whole softmax
//     step after the last one of the previous item, and the epilogue reads O in less than that.
//   * P is the A operand of the second MMA straight from tensor memory.
//
// Epilogue: accumulator -> registers -> 16-bit -> 128-byte-swizzled staging block (64 columns) in
// shared memory -> TMA store, twice (rows past the end of the sequence are clipped by the tensor
// map).  Direct row-per-thread global stores were measured at about 3000 cycles per item and delayed the TMA
// loads of the next item; the staged store is a few hundred.
//
// Softmax: running max in log2 units (scores are multiplied by scale * log2(e) inside the
// exponent's FMA); O is only rescaled when a row's max grows by more than 2^8 (stale max used for
// both P and the running sum, exact after the final division).
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace b200k {
namespace {

constexpr int kAttnThreads = 512;
constexpr int kTmaWarp = 12;
constexpr int kScoreWarp = 13;
constexpr int kPvWarp = 14;
// Registers: 4 warps per SM sub-partition x 128 at launch = 512 per lane, redistributed.  A
// setmaxnreg.inc beyond what the others gave up never completes.
constexpr int kRegsSoftmax = 184;
constexpr int kRegsEpilogue = 80;
constexpr int kRegsOther = 64;
static_assert(2 * kRegsSoftmax + kRegsEpilogue + kRegsOther <= 512, "setmaxnreg.inc would never complete");
constexpr int kTileRows = 128;  // query rows per item, KV rows per tile
constexpr int kD = 128;
constexpr int kHalfTileBytes = kTileRows * 128;  // one 64-element column block: 16 KB
constexpr int kTileBytes = 2 * kHalfTileBytes;   // 32 KB
constexpr int kKStages = 3;
constexpr int kVStages = 2;
constexpr int kQOffset = 0;
constexpr int kKOffset = kTileBytes;
constexpr int kVOffset = kKOffset + kKStages * kTileBytes;
constexpr int kOStageOffset = kVOffset + kVStages * kTileBytes;  // epilogue staging: one 64-column block
constexpr int kMaxOffset = kOStageOffset + kHalfTileBytes;   // float [warpgroup][128 rows]: running max it published
constexpr int kLsumOffset = kMaxOffset + 2 * kTileRows * 4;  // float [warpgroup][max, sum][128 rows] for the epilogue
constexpr int kBarOffset = kLsumOffset + 2 * 2 * kTileRows * 4;
// q_full q_empty | k_full[3] k_empty[3] v_full[2] v_empty[2] | s_full[2] s_free[2] p_full[2] x_full[2] |
// o_done[2] | o_full o_free l_full l_free
constexpr int kNumBars = 2 + 2 * kKStages + 2 * kVStages + 8 + 2 + 4;
// tensor memory columns
constexpr uint32_t kTmemS = 0;    // + 128 * buffer
constexpr uint32_t kTmemP = 256;  // + 64 * buffer
constexpr uint32_t kTmemO = 384;
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
  int32_t interleave_heads, item_div;  // order of the item list, see decode_item
  float scale_log2;
  int32_t* status;
  float* lse;  // optional [batch, q_heads, seq_q]: ln sum_j exp(scale * s_ij), -inf for a row without keys
  // Paged K/V (block_table != nullptr): the tensor maps of K and V describe the page pool
  // [num_pages, kv_heads, page_size, 128]; token t of sequence b lives in page
  // block_table[b * block_table_stride + t / page_size], row t % page_size; sequence b has
  // seq_lens[b] <= seq_kv keys and its queries are its last seq_q tokens.
  const int32_t* block_table;
  const int32_t* seq_lens;
  int32_t block_table_stride, page_size, num_pages;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

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


struct Item {
  int qtile, head, batch, n;  // n = number of 128-row KV tiles this item visits
  int kv_len, causal_offset;  // keys of this item's sequence; key j is visible to query i iff j <= i + causal_offset
};

template <bool PAGED>
__device__ __forceinline__ Item decode_item(int idx, const AttnParams& p) {
  Item it;
  // rank 0 = the last query tile of a head, the heaviest one of a causal problem.  The list is
  // (batch, head)-major, except for a causal problem of a few rounds of items (p.interleave_heads, set
  // by the host): there the heaviest tile of EVERY head comes first, then the next one, ...  A CTA
  // takes every gridDim.x-th item, so each gets tiles of every weight and they finish together
  // (head-major, a CTA of a one-round problem got one tile of arbitrary weight: 1 x 8 heads x 8192
  // causal 172 -> 148 us, 4 x 4 x 4096 91 -> 84).  Longer lists are mixed well enough by the stride, and
  // head-major keeps their K / V traffic on few heads.  One division either way: this runs in the
  // single-thread roles between two items.
  const int d = p.item_div;  // heads of all batches when interleaved, else query tiles per head
  const int hi = idx / d, lo = idx - hi * d;
  const int bh = p.interleave_heads ? lo : hi;
  const int rank = p.interleave_heads ? hi : lo;
  it.qtile = p.num_q_tiles - 1 - rank;
  it.batch = bh / p.q_heads;
  it.head = bh - it.batch * p.q_heads;
  // (dense: the two are launch constants and the fields fold away)
  it.kv_len = p.seq_kv;
  if (PAGED) it.kv_len = max(0, min(__ldg(p.seq_lens + it.batch), p.seq_kv));
  it.causal_offset = PAGED ? it.kv_len - p.seq_q : p.causal_offset;
  const int kv_tiles_total = (it.kv_len + kTileRows - 1) / kTileRows;
  if (!p.causal) {
    it.n = kv_tiles_total;
  } else {
    const int last_col = it.qtile * kTileRows + kTileRows - 1 + it.causal_offset;
    it.n = last_col < 0 ? 0 : min(last_col / kTileRows + 1, kv_tiles_total);
  }
  return it;
}

template <typename T, bool PAGED>
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
  float* xmax = reinterpret_cast<float*>(smem + kMaxOffset);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kBarOffset);
  uint64_t* q_full = bars;
  uint64_t* q_empty = bars + 1;
  uint64_t* k_full = bars + 2;
  uint64_t* k_empty = k_full + kKStages;
  uint64_t* v_full = k_empty + kKStages;
  uint64_t* v_empty = v_full + kVStages;
  uint64_t* s_full = v_empty + kVStages;  // [buffer] score tile written
  uint64_t* s_free = s_full + 2;          // [buffer] score tile is in the softmax threads' registers
  uint64_t* p_full = s_free + 2;          // [buffer] probabilities written
  uint64_t* x_full = p_full + 2;          // [warpgroup] it has published the row maxima after its step
  uint64_t* o_done = x_full + 2;          // [step parity] "O += P V" of that step complete
  uint64_t* o_full = o_done + 2;          // last P V of an item complete
  uint64_t* o_free = o_full + 1;          // epilogue has read the accumulator
  uint64_t* l_full = o_free + 1;          // row sums written
  uint64_t* l_free = l_full + 1;          // row sums read
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
  volatile uint32_t* abort_word = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

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
      mbar_init(s_free + i, 4);
      mbar_init(p_full + i, 4);
      mbar_init(x_full + i, 4);
      mbar_init(o_done + i, 1);
    }
    mbar_init(o_full, 1);
    mbar_init(o_free, 4);
    mbar_init(l_full, 8);
    mbar_init(l_free, 4);
    *abort_word = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    prefetch_tmap(&tmap_o);
  }
  if (warp == kScoreWarp) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int group = p.q_heads / p.kv_heads;

  if (warp >= 12) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
    if (warp == kTmaWarp) {
      // ---------------- TMA producer ----------------
      if (lane == 0) {
        uint32_t qc = 0, kc = 0, vc = 0;  // Q loads, K tiles, V tiles issued so far
        bool ok = true;
        // One 128-row K or V tile.  Dense: one box per 64-column block.  Paged: one box per page and
        // block; a page past the sequence's length is replaced by the sequence's first page (those
        // rows are masked; the data only has to be finite), an entry outside the pool is reported
        // and reads as zeros (the tensor map clips it).
        auto load_tile = [&](uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, const Item& it, int j) {
          if (!PAGED) {
#pragma unroll
            for (int db = 0; db < 2; ++db)
              tma_load_4d(dst + db * kHalfTileBytes, tm, bar, db * 64, j * kTileRows, it.head / group, it.batch);
            return;
          }
          const int32_t* row = p.block_table + static_cast<int64_t>(it.batch) * p.block_table_stride;
          const int pages_per_tile = kTileRows / p.page_size;
          const int valid_pages = (it.kv_len + p.page_size - 1) / p.page_size;
          for (int pp = 0; pp < pages_per_tile; ++pp) {
            const int lp = j * pages_per_tile + pp;
            const int page = __ldg(row + (lp < valid_pages ? lp : 0));
            if ((page < 0 || page >= p.num_pages) && p.status) atomicOr(p.status, kStatusDecodeBadPage);
#pragma unroll
            for (int db = 0; db < 2; ++db)
              tma_load_4d(dst + db * kHalfTileBytes + pp * p.page_size * 128, tm, bar, db * 64, 0, it.head / group, page);
          }
        };
        auto load_k = [&](const Item& it, int j) {
          const int ks = kc % kKStages;
          if (!mbar_wait(k_empty + ks, ((kc / kKStages) & 1) ^ 1, abort_word)) return false;
          mbar_arrive_expect_tx(k_full + ks, kTileBytes);
          load_tile(smem + kKOffset + ks * kTileBytes, &tmap_k, k_full + ks, it, j);
          ++kc;
          return true;
        };
        // Q and the first K tiles of an item.  Q's buffer is free once the previous item's last
        // score MMA has run, which is earlier than the release of its last V stage.
        auto load_head = [&](const Item& it) {
          if (!mbar_wait(q_empty, (qc & 1) ^ 1, abort_word)) return false;
          mbar_arrive_expect_tx(q_full, kTileBytes);
#pragma unroll
          for (int db = 0; db < 2; ++db)
            tma_load_4d(smem + kQOffset + db * kHalfTileBytes, &tmap_q, q_full, db * 64, it.qtile * kTileRows, it.head,
                        it.batch);
          ++qc;
          for (int jj = 0; jj < kKStages && jj < it.n; ++jj)
            if (!load_k(it, jj)) return false;
          return true;
        };
        auto next_item = [&](int idx, Item& nx) {  // next item of this CTA that has work; num_items if none
          for (idx += gridDim.x; idx < p.num_items; idx += gridDim.x) {
            nx = decode_item<PAGED>(idx, p);
            if (nx.n > 0) return idx;
          }
          return p.num_items;
        };
        Item it = {};
        int idx = next_item(static_cast<int>(blockIdx.x) - static_cast<int>(gridDim.x), it);
        if (idx < p.num_items) ok = load_head(it);
        while (idx < p.num_items && ok) {
          Item nx = {};
          const int nidx = next_item(idx, nx);
          const bool have_next = nidx < p.num_items;
          // Order within an item: V_j, then K_(j+3); a K stage is released (by the score MMA that
          // read it) earlier than a V stage.  The head of the next item goes before the last V.
          for (int j = 0; j < it.n && ok; ++j) {
            if (j == it.n - 1 && have_next) {
              ok = load_head(nx);
              if (!ok) break;
            }
            const int vs = vc % kVStages;
            if (!mbar_wait(v_empty + vs, ((vc / kVStages) & 1) ^ 1, abort_word)) { ok = false; break; }
            mbar_arrive_expect_tx(v_full + vs, kTileBytes);
            load_tile(smem + kVOffset + vs * kTileBytes, &tmap_v, v_full + vs, it, j);
            ++vc;
            if (j + kKStages < it.n) ok = load_k(it, j + kKStages);
          }
          it = nx;
          idx = nidx;
        }
      }
      __syncwarp();
    } else if (warp == kScoreWarp) {
      // ---------------- score MMAs: S[g & 1] = Q K_g^T for every KV step g of this CTA ----------------
      // Two threads issue MMAs, this one and the one below.  A tcgen05.mma does not return until
      // the tensor pipe has room for it, so a group of eight blocks its thread for about as long
      // as it executes (plus some 300 cycles when the pipe was idle): one thread for both kinds
      // was busy nearly the whole step and every wait of one kind delayed the other.  The streams
      // are independent: each orders itself through barriers (score buffer taken by the softmax,
      // P written, stages loaded), never through issue order.
      if (lane == 0) {
        // The issuing thread runs scalar, latency-bound code: descriptors are a constant high word
        // plus a low word that is a precomputed base plus a compile-time offset.
        const uint32_t hi_k = static_cast<uint32_t>(make_desc_kmajor_sw128(0) >> 32);
        const uint32_t q_lo = static_cast<uint32_t>(make_desc_kmajor_sw128(smem_u32(smem + kQOffset)));
        const uint32_t k_lo = static_cast<uint32_t>(make_desc_kmajor_sw128(smem_u32(smem + kKOffset)));
        auto desc = [](uint32_t lo, uint32_t hi) { return (static_cast<uint64_t>(hi) << 32) | lo; };
        uint32_t g = 0;                // score tiles issued so far
        uint32_t kstage = 0, kpar = 0; // K ring position
        uint32_t qpar = 0;
        bool ok = true;
        for (int idx = blockIdx.x; idx < p.num_items && ok; idx += gridDim.x) {
          const Item it = decode_item<PAGED>(idx, p);
          if (it.n == 0) continue;
          if (!mbar_wait(q_full, qpar, abort_word)) break;
          qpar ^= 1;
          for (int j = 0; j < it.n; ++j, ++g) {
            const uint32_t buf = g & 1;
            if (!mbar_wait(k_full + kstage, kpar, abort_word)) { ok = false; break; }
            // the buffer last held tile g - 2; the softmax threads have it in registers
            // (passes at once for the first two tiles)
            if (!mbar_wait(s_free + buf, ((g >> 1) & 1) ^ 1, abort_word)) { ok = false; break; }
            tc_fence_after();
            const uint32_t b0 = k_lo + kstage * (kTileBytes >> 4);
            const uint32_t d = tmem_base + kTmemS + buf * 128;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {  // 8 k-steps of 16 over the head dimension (two 64-wide blocks)
              const uint32_t off = (ks >> 2) * (kHalfTileBytes >> 4) + 2 * (ks & 3);
              umma_f16_ss(d, desc(q_lo + off, hi_k), desc(b0 + off, hi_k), kIdescS, ks > 0 ? 1u : 0u);
            }
            umma_commit(s_full + buf);
            umma_commit(k_empty + kstage);
            if (j == it.n - 1) umma_commit(q_empty);  // Q is free once the item's last score MMA has run
            if (++kstage == kKStages) {
              kstage = 0;
              kpar ^= 1;
            }
          }
        }
      }
      __syncwarp();
    } else if (warp == kPvWarp) {
      // ---------------- second MMAs: O (+)= P[g & 1] V_g ----------------
      if (lane == 0) {
        const uint32_t hi_mn = static_cast<uint32_t>(make_desc_mnmajor_sw128(0, kHalfTileBytes) >> 32);
        const uint32_t v_lo = static_cast<uint32_t>(make_desc_mnmajor_sw128(smem_u32(smem + kVOffset), kHalfTileBytes));
        auto desc = [](uint32_t lo, uint32_t hi) { return (static_cast<uint64_t>(hi) << 32) | lo; };
        uint32_t g = 0, ic = 0;  // KV steps and items so far
        uint32_t vstage = 0, vpar = 0;
        bool ok = true;
        for (int idx = blockIdx.x; idx < p.num_items && ok; idx += gridDim.x) {
          const Item it = decode_item<PAGED>(idx, p);
          if (it.n == 0) continue;
          for (int j = 0; j < it.n; ++j, ++g) {
            const uint32_t buf = g & 1;
            if (!mbar_wait(v_full + vstage, vpar, abort_word)) { ok = false; break; }
            if (!mbar_wait(p_full + buf, (g >> 1) & 1, abort_word)) { ok = false; break; }
            // the accumulator is read by the epilogue of the previous item
            if (j == 0 && !mbar_wait(o_free, (ic & 1) ^ 1, abort_word)) { ok = false; break; }
            tc_fence_after();
            // 8 k-steps of 16 KV rows; A = P from tensor memory, B = V (MN-major)
            const uint32_t b0 = v_lo + vstage * (kTileBytes >> 4);
            const uint32_t d = tmem_base + kTmemO;
            const uint32_t a = tmem_base + kTmemP + buf * 64;
            umma_f16_ts(d, a, desc(b0, hi_mn), kIdescPV, j == 0 ? 0u : 1u);
#pragma unroll
            for (int ks = 1; ks < 8; ++ks) umma_f16_ts(d, a + ks * 8, desc(b0 + ks * (2048 >> 4), hi_mn), kIdescPV, 1u);
            umma_commit(v_empty + vstage);
            umma_commit(o_done + buf);
            if (j == it.n - 1) umma_commit(o_full);
            if (++vstage == kVStages) {
              vstage = 0;
              vpar ^= 1;
            }
          }
          ++ic;
        }
      }
      __syncwarp();
    }
  } else if (warp >= 8) {
    // ---------------- epilogue: O / rowsum -> global, one item behind ----------------
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsEpilogue));
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    uint8_t* stage = smem + kOStageOffset;
    const bool store_thread = (warp == 8 && lane == 0);
    auto epi_barrier = [&]() { asm volatile("bar.sync 1, 128;" ::: "memory"); };
    uint32_t ic = 0, g0 = 0;  // items so far, KV steps before the current item
    bool ok = true;
    for (int idx = blockIdx.x; idx < p.num_items && ok; idx += gridDim.x) {
      const Item it = decode_item<PAGED>(idx, p);
      if (it.n == 0) {
        // no visible key: zeros (rare; plain stores)
        const int q_row = it.qtile * kTileRows + row_in_tile;
        if (q_row < p.seq_q) {
          T* orow = reinterpret_cast<T*>(p.o) + it.batch * p.o_stride_b + it.head * p.o_stride_h +
                    static_cast<int64_t>(q_row) * p.o_stride_s;
#pragma unroll
          for (int v = 0; v < 16; ++v) reinterpret_cast<uint4*>(orow)[v] = make_uint4(0u, 0u, 0u, 0u);
          if (p.lse) p.lse[(static_cast<int64_t>(it.batch) * p.q_heads + it.head) * p.seq_q + q_row] = -INFINITY;
        }
        continue;
      }
      const uint32_t par = ic & 1;
      ok = mbar_wait(o_full, par, abort_word) && mbar_wait(l_full, par, abort_word);
      // the four warps meet at named barriers below: they give up together or not at all
      ok = bar_red_and(1, 128, ok);
      if (!ok) break;
      tc_fence_after();
      // The two warpgroups' partial row sums, each relative to the running max the warpgroup last
      // used; the accumulator is relative to the larger one.  They are added in the order "the
      // warpgroup that took the item's even steps first", so that the result does not depend on
      // what the CTA processed before this item.
      const int we = g0 & 1, wo = we ^ 1;
      const float m0 = lsum[(we * 2 + 0) * kTileRows + row_in_tile], l0 = lsum[(we * 2 + 1) * kTileRows + row_in_tile];
      const float m1 = lsum[(wo * 2 + 0) * kTileRows + row_in_tile], l1 = lsum[(wo * 2 + 1) * kTileRows + row_in_tile];
      const float mm = fmaxf(m0, m1);
      const float a0 = (m0 == -INFINITY) ? 0.f : ex2(m0 - mm);
      const float a1 = (m1 == -INFINITY) ? 0.f : ex2(m1 - mm);
      const float l = l0 * a0 + l1 * a1;
      const float inv = (l > 0.f) ? 1.0f / l : 0.f;
      if (p.lse) {
        // mm is in the log2 domain (scores times scale * log2 e), l is relative to it
        const int q_row = it.qtile * kTileRows + row_in_tile;
        if (q_row < p.seq_q)
          p.lse[(static_cast<int64_t>(it.batch) * p.q_heads + it.head) * p.seq_q + q_row] =
              (l > 0.f) ? (mm + log2f(l)) * 0.6931471805599453f : -INFINITY;
      }
      const uint32_t t_o = tmem_base + lane_field + kTmemO;
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {  // one 64-column block at a time
        // the staging block is free once the previous TMA store has read it
        if (store_thread) tma_store_wait_read<0>();
        epi_barrier();
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_o + (c2 * 2 + cc) * 32, r);
          tmem_wait_ld();
          uint8_t* blk = stage + row_in_tile * 128;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 u;
            u.x = pack_pair<T>(__uint_as_float(r[8 * v + 0]) * inv, __uint_as_float(r[8 * v + 1]) * inv);
            u.y = pack_pair<T>(__uint_as_float(r[8 * v + 2]) * inv, __uint_as_float(r[8 * v + 3]) * inv);
            u.z = pack_pair<T>(__uint_as_float(r[8 * v + 4]) * inv, __uint_as_float(r[8 * v + 5]) * inv);
            u.w = pack_pair<T>(__uint_as_float(r[8 * v + 6]) * inv, __uint_as_float(r[8 * v + 7]) * inv);
            const int chunk = cc * 4 + v;
            *reinterpret_cast<uint4*>(blk + ((chunk ^ (row_in_tile & 7)) << 4)) = u;
          }
        }
        if (c2 == 1) {
          // accumulator and row sums have been read: release them for the next item
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(o_free);
            mbar_arrive(l_free);
          }
        }
        fence_proxy_async_smem();
        epi_barrier();
        if (store_thread) {
          tma_store_4d(&tmap_o, stage, c2 * 64, it.qtile * kTileRows, it.head, it.batch);
          tma_store_commit();
        }
      }
      ++ic;
      g0 += it.n;
    }
    if (store_thread) tma_store_wait<0>();
  } else {
    // ---------------- softmax / correction: warpgroup w takes the KV steps g with (g & 1) == w ----------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    const int w = warp >> 2;  // also the score buffer and the P buffer this warpgroup works on
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t t_s = tmem_base + lane_field + kTmemS + w * 128;
    const uint32_t t_p = tmem_base + lane_field + kTmemP + w * 64;
    const uint32_t t_o = tmem_base + lane_field + kTmemO;
    float* m_mine = xmax + w * kTileRows + row_in_tile;
    const float* m_theirs = xmax + (w ^ 1) * kTileRows + row_in_tile;
    const float scale_log2 = p.scale_log2;
    const float2 scale2 = make_float2(scale_log2, scale_log2);
    uint32_t g = 0, ic = 0;  // KV steps (of both warpgroups) and items so far
    bool ok = true;
    for (int idx = blockIdx.x; idx < p.num_items && ok; idx += gridDim.x) {
      const Item it = decode_item<PAGED>(idx, p);
      if (it.n == 0) continue;
      const int tile_r0 = it.qtile * kTileRows;
      const int q_row = tile_r0 + row_in_tile;
      const int kv_len = PAGED ? it.kv_len : p.seq_kv;
      const int causal_offset = PAGED ? it.causal_offset : p.causal_offset;
      float m_ref = -INFINITY;  // running max this warpgroup's row sum is relative to
      float2 l2 = make_float2(0.f, 0.f);
      for (int j = 0; j < it.n; ++j, ++g) {
        if ((g & 1u) != static_cast<uint32_t>(w)) continue;
        const uint32_t ph = (g >> 1) & 1;  // phase of this warpgroup's own barriers in this step
        ok = mbar_wait(s_full + w, ph, abort_word);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t sr[128];
        tmem_ld_32x32b_x64(t_s, sr);
        tmem_ld_32x32b_x64(t_s + 64, sr + 64);

        const int col0 = j * kTileRows;
        const bool need_mask =
            (p.causal && col0 + kTileRows - 1 > tile_r0 + causal_offset) || (col0 + kTileRows > kv_len);
        int limit = kTileRows;  // columns [0, limit) of this tile are visible to this row
        if (need_mask) {
          int vis = kv_len;
          if (p.causal) vis = min(vis, q_row + causal_offset + 1);
          limit = vis - col0;
        }
        tmem_wait_ld();
        // the row is in registers: the tensor core may write the tile two steps ahead over it
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free + w);
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (i >= limit) sr[i] = 0xff800000u;  // -inf
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 128; i += 4) {
          mx0 = fmax3(mx0, __uint_as_float(sr[i]), __uint_as_float(sr[i + 1]));
          mx1 = fmax3(mx1, __uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3]));
        }
        const float m_new = fmaxf(mx0, mx1) * scale_log2;
        // The running max after the previous step, published by the other warpgroup early in that
        // step (half a step ago).  Every phase of x_full is observed, also when the value is not
        // needed (first step of an item).
        float m_prev = -INFINITY;
        if (g > 0) {
          ok = mbar_wait(x_full + (w ^ 1), ((g - 1) >> 1) & 1, abort_word);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if (j > 0) m_prev = *m_theirs;
        }
        const bool grow = m_new > m_prev + kRescaleThreshold;  // also true for the first finite max
        const float m_cur = grow ? m_new : m_prev;
        *m_mine = m_cur;
        __syncwarp();
        if (lane == 0) mbar_arrive(x_full + w);
        // this warpgroup's partial row sum follows the running max
        if (m_prev != m_ref) {  // m_prev > m_ref: the other warpgroup raised it
          const float a = ex2(m_ref - m_prev);  // m_ref = -inf gives 0 (and the sum is 0 then)
          l2.x *= a;
          l2.y *= a;
        }
        if (j > 0 && __any_sync(0xffffffffu, grow)) {
          // Rescale O between "O += P V" of the previous step (the other warpgroup's P) and this
          // step's.  Rare after the first steps of an item: the max must grow by 2^8.
          float alpha = 1.f;
          if (grow) alpha = ex2(m_prev - m_new);  // m_prev = -inf gives 0
          ok = mbar_wait(o_done + (w ^ 1), ((g - 1) >> 1) & 1, abort_word);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
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
        m_ref = m_cur;
        const float m_sub = (m_cur == -INFINITY) ? 0.f : m_cur;
        const float2 negm2 = make_float2(-m_sub, -m_sub);
        // this warpgroup's P buffer was last read by "O += P V" two steps ago
        if (g >= 2) {
          ok = mbar_wait(o_done + w, ph ^ 1, abort_word);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }

        // probabilities -> tensor memory (16-bit pairs); masked scores are -inf and give (almost) exactly 0
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float2 x = ffma2(make_float2(__uint_as_float(sr[c * 32 + 2 * i]), __uint_as_float(sr[c * 32 + 2 * i + 1])),
                                   scale2, negm2);
            const float2 e = make_float2(ex2(x.x), ex2(x.y));
            l2 = fadd2(l2, e);
            pk[i] = pack_pair<T>(e.x, e.y);
          }
          tmem_st_32x32b_x16(t_p + c * 16, pk);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full + w);
      }
      if (!ok) break;
      // hand (max, sum) of this warpgroup's steps to the epilogue warps
      ok = mbar_wait(l_free, (ic & 1) ^ 1, abort_word);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      lsum[(w * 2 + 0) * kTileRows + row_in_tile] = m_ref;
      lsum[(w * 2 + 1) * kTileRows + row_in_tile] = l2.x + l2.y;
      __syncwarp();
      if (lane == 0) mbar_arrive(l_full);
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
  if (warp == kScoreWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <typename T, bool PAGED>
int launch_typed(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to,
                 const AttnParams& p, cudaStream_t stream) {
  auto kfn = attn_fwd_kernel<T, PAGED>;
  static bool configured[64] = {};  // per instantiation and device ordinal
  int rc = ensure_dynamic_smem(kfn, kAttnSmem, configured, "cudaFuncSetAttribute(attention smem)");
  if (rc) return rc;
  const int sms = num_sms();
  const int grid = p.num_items < sms ? p.num_items : sms;
  kfn<<<grid, kAttnThreads, kAttnSmem, stream>>>(tq, tk, tv, to, p);
  return check_cuda(cudaGetLastError(), "attn_fwd_kernel launch");
}

}  // namespace

// Arguments have been validated by launch_attention_fwd.
int launch_attention_fwd_tile(const b200k_attention_args& a, cudaStream_t stream) {
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
  if (reinterpret_cast<uintptr_t>(a.lse) & 3) return set_error(B200K_ERR_BAD_ALIGN, "attention_fwd: lse must be 4-byte aligned");
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
  p.interleave_heads = (p.causal && items <= 4 * static_cast<int64_t>(num_sms())) ? 1 : 0;
  p.item_div = p.interleave_heads ? p.num_items / p.num_q_tiles : p.num_q_tiles;
  p.scale_log2 = a.scale * kLog2e;
  p.status = a.status;
  p.lse = a.lse;
  p.block_table = nullptr;
  p.seq_lens = nullptr;
  p.block_table_stride = p.page_size = p.num_pages = 0;
  if (a.dtype == B200K_F16) return launch_typed<__half, false>(tq, tk, tv, to, p, stream);
  return launch_typed<__nv_bfloat16, false>(tq, tk, tv, to, p, stream);
}

// Arguments have been validated by launch_paged_attention_fwd.
int launch_paged_attention_fwd_tile(const b200k_paged_attention_args& a, cudaStream_t stream) {
  if (!a.q || !a.k_cache || !a.v_cache || !a.o || !a.block_table || !a.seq_lens)
    return set_error(B200K_ERR_NULL, "paged_attention_fwd: q, k_cache, v_cache, o, block_table, seq_lens must be non-NULL");
  if (a.batch <= 0 || a.q_heads <= 0 || a.kv_heads <= 0 || a.seq_q <= 0 || a.max_seq_kv <= 0)
    return set_error(B200K_ERR_BAD_SHAPE, "paged_attention_fwd: all dimensions must be positive");
  if (a.head_dim != kD) return set_error(B200K_ERR_BAD_SHAPE, "paged_attention_fwd: head_dim must be 128");
  if (a.q_heads % a.kv_heads != 0)
    return set_error(B200K_ERR_BAD_SHAPE, "paged_attention_fwd: q_heads must be a multiple of kv_heads");
  if (a.dtype != B200K_F16 && a.dtype != B200K_BF16)
    return set_error(B200K_ERR_BAD_DTYPE, "paged_attention_fwd: dtype must be F16 or BF16");
  if (a.page_size < 16 || a.page_size > kTileRows || kTileRows % a.page_size != 0 || a.page_size % 8 != 0)
    return set_error(B200K_ERR_BAD_SHAPE, "paged_attention_fwd: page_size must be 16, 32, 64 or 128");
  if (a.num_pages <= 0 || a.block_table_stride <= 0 ||
      static_cast<int64_t>(a.block_table_stride) * a.page_size < a.max_seq_kv)
    return set_error(B200K_ERR_BAD_SHAPE, "paged_attention_fwd: the block table does not cover max_seq_kv");
  const int64_t strides[] = {a.q_stride_b, a.q_stride_h, a.q_stride_s, a.o_stride_b, a.o_stride_h, a.o_stride_s,
                             a.kv_page_stride, a.kv_head_stride};
  for (int64_t s : strides)
    if (s <= 0 || s % 8 != 0)
      return set_error(B200K_ERR_BAD_ALIGN, "paged_attention_fwd: every stride must be a positive multiple of 8 elements");
  if ((reinterpret_cast<uintptr_t>(a.q) & 15) || (reinterpret_cast<uintptr_t>(a.k_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(a.v_cache) & 15) || (reinterpret_cast<uintptr_t>(a.o) & 15))
    return set_error(B200K_ERR_BAD_ALIGN, "paged_attention_fwd: q, caches and o must be 16-byte aligned");
  if (!(a.scale > 0.f)) return set_error(B200K_ERR_BAD_SHAPE, "paged_attention_fwd: scale must be positive");
  int rc = ensure_sm100();
  if (rc) return rc;

  CUtensorMap tq, tk, tv, to;
  const uint32_t box[4] = {64, kTileRows, 1, 1};
  const uint32_t page_box[4] = {64, static_cast<uint32_t>(a.page_size), 1, 1};
  {
    uint64_t dims[4] = {kD, static_cast<uint64_t>(a.seq_q), static_cast<uint64_t>(a.q_heads),
                        static_cast<uint64_t>(a.batch)};
    uint64_t st[3] = {static_cast<uint64_t>(a.q_stride_s) * 2, static_cast<uint64_t>(a.q_stride_h) * 2,
                      static_cast<uint64_t>(a.q_stride_b) * 2};
    rc = encode_tmap(&tq, a.dtype, 4, const_cast<void*>(a.q), dims, st, box);
    if (rc) return rc;
    uint64_t so[3] = {static_cast<uint64_t>(a.o_stride_s) * 2, static_cast<uint64_t>(a.o_stride_h) * 2,
                      static_cast<uint64_t>(a.o_stride_b) * 2};
    rc = encode_tmap(&to, a.dtype, 4, a.o, dims, so, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[4] = {kD, static_cast<uint64_t>(a.page_size), static_cast<uint64_t>(a.kv_heads),
                        static_cast<uint64_t>(a.num_pages)};
    uint64_t st[3] = {static_cast<uint64_t>(kD) * 2, static_cast<uint64_t>(a.kv_head_stride) * 2,
                      static_cast<uint64_t>(a.kv_page_stride) * 2};
    rc = encode_tmap(&tk, a.dtype, 4, const_cast<void*>(a.k_cache), dims, st, page_box);
    if (rc) return rc;
    rc = encode_tmap(&tv, a.dtype, 4, const_cast<void*>(a.v_cache), dims, st, page_box);
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
  p.seq_kv = a.max_seq_kv;
  p.causal = a.causal ? 1 : 0;
  p.causal_offset = a.max_seq_kv - a.seq_q;
  p.num_q_tiles = (a.seq_q + kTileRows - 1) / kTileRows;
  const int64_t items = static_cast<int64_t>(a.batch) * a.q_heads * p.num_q_tiles;
  if (items > INT32_MAX) return set_error(B200K_ERR_BAD_SHAPE, "paged_attention_fwd: too many query tiles");
  p.num_items = static_cast<int32_t>(items);
  p.interleave_heads = (p.causal && items <= 4 * static_cast<int64_t>(num_sms())) ? 1 : 0;
  p.item_div = p.interleave_heads ? p.num_items / p.num_q_tiles : p.num_q_tiles;
  p.scale_log2 = a.scale * kLog2e;
  p.status = a.status;
  p.lse = nullptr;
  p.block_table = a.block_table;
  p.seq_lens = a.seq_lens;
  p.block_table_stride = a.block_table_stride;
  p.page_size = a.page_size;
  p.num_pages = a.num_pages;
  if (a.dtype == B200K_F16) return launch_typed<__half, true>(tq, tk, tv, to, p, stream);
  return launch_typed<__nv_bfloat16, true>(tq, tk, tv, to, p, stream);
}

}  // namespace b200k
