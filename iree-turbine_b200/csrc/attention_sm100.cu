// Attention forward (vanilla and causal, dense or paged K/V, head dim 128 or 64) on sm_100a: the
// TILE-PAIR kernel, and the entry points that choose between it and the one-tile kernel of
// attention_tile_sm100.cu (see choose_pair_kernel at the end of this file).
//
// Persistent CTAs, one per SM.  A work item is one PAIR of 128-row query tiles (256 consecutive
// query rows) of one (batch, head).  The two tiles of a pair are independent problems that share
// every K/V tile: each has its own score buffer, its own probabilities, its own running max / sum
// and its own output accumulator, and each is served by its own softmax warpgroup.  Nothing is
// exchanged between the two warpgroups; while one of them is busy with its exponentials the
// tensor core works for the other one.
//
//   warps 0..3    softmax of query tile 0 (thread = one query row, the whole score row in registers)
//   warps 4..7    softmax of query tile 1
//   warps 8..11   epilogue: O / rowsum -> global for both tiles, one item behind the others
//   warp 12       TMA loads of K and V: one ring of kKvStages tiles, filled K_0 V_0 K_1 V_1 ...
//   warp 13       issues the MMAs of query tile 0 (one thread) and owns tensor memory
//   warp 14       TMA loads of Q (a thread of its own, so that waiting for a free Q buffer never
//                 holds up K/V loads)
//   warp 15       issues the MMAs of query tile 1 (one thread)
//
// Tensor memory (512 columns x 128 lanes):  S[0] | S[1] (128 fp32 columns each) | O[0] | O[1]
// (head-dim fp32 columns each).  A tile's 128 score columns are TWO buffers of 64: a K/V tile is
// worked through in two half steps of 64 keys, half step h in buffer h & 1.  The probabilities of a
// half step (16-bit, 32 columns) are written over the first half of the scores they came from by the
// thread that has just read that row into registers, and are the A operand of the second MMA
// straight from tensor memory.
//
// Order of the MMAs of query tile t (one in-order stream per tile, issued by its own thread), half step h:
//     S(0) : S(1) : wait P(0) : O += P(0) V[0:64] : S(2) : wait P(1) : O += P(1) V[64:128] : S(3) : ...
// so while the softmax of a tile works on half step h, the scores of half step h + 1 are already
// there or on their way (with one 128-column buffer per tile the next scores could only be issued
// behind the PV product that reads the probabilities, and the softmax waited out both products on
// every step).  S(h + 2) is issued behind O += P(h) V by the same thread, so it may overwrite P(h)
// without a barrier.  A PV group commits to pv_done; the softmax waits there only on the rare step on
// which it has to rescale O in place (the scores it has just read were issued BEFORE the previous
// half step's PV group, so their arrival says nothing about it).  A stream does not stop at item
// boundaries: a tile that has issued its last PV of an item goes on with the first scores of its
// next item as soon as Q and K are there.  The score MMAs have N = 64, so Q is read from shared
// memory twice per K/V tile; measured, that costs less than the waiting it removes.
//
// Causal items: the two tiles of a pair need a different number of KV tiles (n[0] <= n[1]); tile 0
// simply stops taking part once it is past its diagonal.  Work is dealt to CTAs in units that pair
// the heaviest remaining pair of a head with the lightest, so every unit of a causal problem costs
// the same.
//
// Softmax: running max in log2 units (scores are multiplied by scale * log2(e) inside the
// exponent's FMA); O is only rescaled when a row's max grows by more than 2^8 (the stale max is
// used for both P and the running sum, which is exact after the final division).
//
// Epilogue: accumulator -> registers -> 16-bit -> 128-byte-swizzled staging block (64 columns) in
// shared memory -> TMA store (rows past the end of the sequence are clipped by the tensor map).
//
// Every wait is bounded; when one gives up all roles drain to the common teardown, tensor memory
// is freed and the kernel ORs a code into the caller's status word.
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace b200k {
namespace {

constexpr int kAttnThreads = 512;
constexpr int kKvWarp = 12;
constexpr int kMmaWarp = 13;
constexpr int kQWarp = 14;  // (warp 15 issues the MMAs of query tile 1)
// Registers: 4 warps per SM sub-partition x 128 at launch = 512 per lane, redistributed.  A
// setmaxnreg.inc beyond what the others gave up never completes.
constexpr int kRegsSoftmax = 160;
constexpr int kRegsEpilogue = 96;
constexpr int kRegsOther = 96;
static_assert(2 * kRegsSoftmax + kRegsEpilogue + kRegsOther <= 512, "setmaxnreg.inc would never complete");
constexpr int kTileRows = 128;           // query rows per tile, KV rows per tile
constexpr int kPairRows = 2 * kTileRows;  // query rows per work item
constexpr int kHalfTileBytes = kTileRows * 128;  // one 64-element column block of a tile: 16 KB
constexpr int kKvStages = 4;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;

template <int HD>
struct AttnSmem {
  static constexpr int kBlocks = HD / 64;                       // 64-column blocks per tile row
  static constexpr int kTileBytes = kBlocks * kHalfTileBytes;   // 32 KB (HD 128) or 16 KB (HD 64)
  static constexpr int kQOffset = 0;                             // two query tiles
  static constexpr int kKvOffset = 2 * kTileBytes;
  static constexpr int kStageOffset = kKvOffset + kKvStages * kTileBytes;  // epilogue staging: one 64-column block
  static constexpr int kLsumOffset = kStageOffset + kHalfTileBytes;        // float [tile][max, sum][128 rows]
  static constexpr int kBarOffset = kLsumOffset + 2 * 2 * kTileRows * 4;
  // q_full[2] q_empty[2] | kv_full[4] kv_empty[4] | s_full[2][2] p_full[2][2] | o_full[2] o_free[2] | l_full[2] l_free[2] | turn[2] | pv_done[2]
  static constexpr int kNumBars = 4 + 2 * kKvStages + 8 + 4 + 4 + 2 + 2;
  static constexpr int kTotal = kBarOffset + kNumBars * 8 + 16 + 1024;  // + slack for 1024-byte alignment
  // tensor memory columns
  static constexpr uint32_t kTmemS = 0;    // + 128 * tile; P over the first 64 columns
  static constexpr uint32_t kTmemO = 256;  // + HD * tile
};
static_assert(AttnSmem<128>::kTotal <= 232448, "shared memory budget");

struct AttnParams {
  void* o;
  int64_t o_stride_b, o_stride_h, o_stride_s;
  int32_t batch, q_heads, kv_heads, seq_q, seq_kv;
  int32_t causal, causal_offset;
  int32_t num_pairs;       // ceil(seq_q / 256)
  int32_t units_per_head;  // work units per (batch, head): pairs, or (heavy, light) couples of pairs when causal
  int32_t num_units;       // batch * q_heads * units_per_head
  float scale_log2;
  int32_t* status;
  float* lse;  // optional [batch, q_heads, seq_q]: ln sum_j exp(scale * s_ij), -inf for a row without keys
  // Paged K/V (block_table != nullptr): the tensor maps of K and V describe the page pool
  // [num_pages, kv_heads, page_size, head_dim]; token t of sequence b lives in page
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
// The special-function unit delivers 16 results per cycle and SM: 128 x 128 exponentials are 1024
// cycles, as long as the two MMAs of the same tile, so whatever share of them moves to the FMA
// pipe comes off the softmax's critical resource.
constexpr uint32_t kPolyPairMask = 0x00u;

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
  int pair, head, batch;
  int n[2];   // KV tiles query tile t visits (0: the tile has no rows or sees no key)
  int nmax;   // max(n[0], n[1]): KV tiles loaded for the item
  int kv_len, causal_offset;  // keys of this item's sequence; key j is visible to query i iff j <= i + causal_offset
};

template <bool PAGED>
__device__ __forceinline__ Item make_item(int bh, int pair, const AttnParams& p) {
  Item it;
  it.pair = pair;
  it.batch = bh / p.q_heads;
  it.head = bh - it.batch * p.q_heads;
  // (dense: the two are launch constants and the fields fold away)
  it.kv_len = p.seq_kv;
  if (PAGED) it.kv_len = max(0, min(__ldg(p.seq_lens + it.batch), p.seq_kv));
  it.causal_offset = PAGED ? it.kv_len - p.seq_q : p.causal_offset;
  const int kv_tiles_total = (it.kv_len + kTileRows - 1) / kTileRows;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int r0 = pair * kPairRows + t * kTileRows;
    int n = 0;
    if (r0 < p.seq_q) {
      if (!p.causal) {
        n = kv_tiles_total;
      } else {
        const int last_col = r0 + kTileRows - 1 + it.causal_offset;
        n = last_col < 0 ? 0 : min(last_col / kTileRows + 1, kv_tiles_total);
      }
    }
    it.n[t] = n;
  }
  it.nmax = max(it.n[0], it.n[1]);
  return it;
}

// The CTA's items, in the order every role walks them: units blockIdx.x, blockIdx.x + gridDim.x, ...;
// a unit is one pair of a (batch, head), heaviest first, or -- causal -- the k-th heaviest pair
// followed by the k-th lightest of the same head.  Units are numbered (batch, head)-major, so the
// CTAs that run at one time work on a few neighbouring heads and share their K/V in L2.  (Giving
// each CTA a contiguous range of units instead -- one head per CTA at a time -- puts 148 heads'
// K/V in flight at once, more than L2 holds at S = 4096: measured 9 % slower.)
template <bool PAGED>
struct ItemWalk {
  const AttnParams& p;
  int unit, end, part;
  __device__ ItemWalk(const AttnParams& params) : p(params), unit(blockIdx.x), end(params.num_units), part(0) {}
  // Next item, empty ones (nmax == 0) included; false when the CTA has no more.
  __device__ __forceinline__ bool next(Item& it) {
    while (unit < end) {
      const int bh = unit / p.units_per_head;
      const int s = unit - bh * p.units_per_head;
      const int heavy = p.num_pairs - 1 - s;
      if (part == 0) {
        part = 1;
        it = make_item<PAGED>(bh, heavy, p);
        return true;
      }
      part = 0;
      unit += gridDim.x;
      if (p.causal && s < heavy) {
        it = make_item<PAGED>(bh, s, p);
        return true;
      }
    }
    return false;
  }
  // Next item that has work.
  __device__ __forceinline__ bool next_busy(Item& it) {
    while (next(it))
      if (it.nmax > 0) return true;
    return false;
  }
};

template <typename T, int HD, bool PAGED>
__global__ void __launch_bounds__(kAttnThreads, 1)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
                    const AttnParams p) {
  using L = AttnSmem<HD>;
  constexpr int kBlocks = L::kBlocks;
  constexpr int kTileBytes = L::kTileBytes;
  constexpr uint32_t kFmt = std::is_same<T, __half>::value ? kFmtF16 : kFmtBF16;
  constexpr uint32_t kIdescS = make_idesc(kFmt, kFmt, 128, 64, 0, 0);   // Q, K both K-major; 64 keys per half step
  constexpr uint32_t kIdescPV = make_idesc(kFmt, kFmt, 128, HD, 0, 1);  // V is MN-major

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  float* lsum = reinterpret_cast<float*>(smem + L::kLsumOffset);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* q_full = bars;            // [tile] Q tile loaded
  uint64_t* q_empty = q_full + 2;     // [tile] the item's last score MMA of that tile has read Q
  uint64_t* kv_full = q_empty + 2;    // [stage]
  uint64_t* kv_empty = kv_full + kKvStages;
  uint64_t* s_full = kv_empty + kKvStages;  // [tile][half] scores of a half step (64 keys) written
  uint64_t* p_full = s_full + 4;            // [tile][half] probabilities written (and O rescaled if it had to be)
  uint64_t* o_full = p_full + 4;            // [tile] last PV of an item complete
  uint64_t* o_free = o_full + 2;            // [tile] epilogue has read the accumulator
  uint64_t* l_full = o_free + 2;            // [tile] (max, sum) of the item written
  uint64_t* l_free = l_full + 2;            // [tile] ... and read
  uint64_t* turn = l_free + 2;              // [tile] it is this tile's turn to put MMAs into the pipe
  uint64_t* pv_done = turn + 2;             // [tile] one completion per PV group (only waited for before a rescale of O)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile uint32_t* abort_word = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int t = 0; t < 2; ++t) {
      mbar_init(q_full + t, 1);
      mbar_init(q_empty + t, 1);
      for (int hb = 0; hb < 2; ++hb) {
        mbar_init(s_full + 2 * t + hb, 1);
        mbar_init(p_full + 2 * t + hb, 4);
      }
      mbar_init(pv_done + t, 1);
      mbar_init(o_full + t, 1);
      mbar_init(o_free + t, 4);
      mbar_init(l_full + t, 4);
      mbar_init(l_free + t, 4);
      mbar_init(turn + t, 1);
    }
    for (int i = 0; i < kKvStages; ++i) {
      mbar_init(kv_full + i, 1);
      mbar_init(kv_empty + i, 2);
    }
    *abort_word = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    prefetch_tmap(&tmap_o);
  }
  if (warp == kMmaWarp) {
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
    if (warp == kKvWarp) {
      // ---------------- K / V producer: ring entries K_0 V_0 K_1 V_1 ... of every item ----------------
      if (lane == 0) {
        uint32_t e = 0;  // ring entries issued so far
        bool ok = true;
        // One 128-row K or V tile.  Dense: one box per 64-column block.  Paged: one box per page and
        // block; a page past the sequence's length is replaced by the sequence's first page (those
        // rows are masked; the data only has to be finite), an entry outside the pool is reported
        // and reads as zeros (the tensor map clips it).
        auto load_tile = [&](const CUtensorMap* tm, const Item& it, int j) {
          const uint32_t stage = e % kKvStages;
          if (!mbar_wait(kv_empty + stage, ((e / kKvStages) & 1) ^ 1, abort_word)) return false;
          uint8_t* dst = smem + L::kKvOffset + stage * kTileBytes;
          uint64_t* bar = kv_full + stage;
          mbar_arrive_expect_tx(bar, kTileBytes);
          ++e;
          if (!PAGED) {
#pragma unroll
            for (int db = 0; db < kBlocks; ++db)
              tma_load_4d(dst + db * kHalfTileBytes, tm, bar, db * 64, j * kTileRows, it.head / group, it.batch);
            return true;
          }
          const int32_t* row = p.block_table + static_cast<int64_t>(it.batch) * p.block_table_stride;
          const int pages_per_tile = kTileRows / p.page_size;
          const int valid_pages = (it.kv_len + p.page_size - 1) / p.page_size;
          for (int pp = 0; pp < pages_per_tile; ++pp) {
            const int lp = j * pages_per_tile + pp;
            const int page = __ldg(row + (lp < valid_pages ? lp : 0));
            if ((page < 0 || page >= p.num_pages) && p.status) atomicOr(p.status, kStatusDecodeBadPage);
#pragma unroll
            for (int db = 0; db < kBlocks; ++db)
              tma_load_4d(dst + db * kHalfTileBytes + pp * p.page_size * 128, tm, bar, db * 64, 0, it.head / group, page);
          }
          return true;
        };
        ItemWalk<PAGED> walk(p);
        Item it;
        while (ok && walk.next_busy(it)) {
          for (int j = 0; j < it.nmax && ok; ++j) ok = load_tile(&tmap_k, it, j) && load_tile(&tmap_v, it, j);
        }
      }
      __syncwarp();
    } else if (warp == kQWarp) {
      // ---------------- Q producer ----------------
      if (lane == 0) {
        uint32_t ci[2] = {0, 0};  // items of each tile so far
        bool ok = true;
        ItemWalk<PAGED> walk(p);
        Item it, nx;
        bool have = walk.next_busy(it);
        while (ok && have) {
          const bool have_next = walk.next_busy(nx);
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (it.n[t] == 0) continue;
            if (!mbar_wait(q_empty + t, (ci[t] & 1) ^ 1, abort_word)) { ok = false; break; }
            ++ci[t];
            mbar_arrive_expect_tx(q_full + t, kTileBytes);
#pragma unroll
            for (int db = 0; db < kBlocks; ++db)
              tma_load_4d(smem + L::kQOffset + t * kTileBytes + db * kHalfTileBytes, &tmap_q, q_full + t, db * 64,
                          it.pair * kPairRows + t * kTileRows, it.head, it.batch);
          }
          // A Q buffer frees up only a step or so before the next item needs it, less than a trip
          // to HBM: ask for the next item's Q tiles in L2 now, an item ahead.
          if (have_next) {
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              if (nx.n[t] == 0) continue;
#pragma unroll
              for (int db = 0; db < kBlocks; ++db)
                tma_prefetch_4d(&tmap_q, db * 64, nx.pair * kPairRows + t * kTileRows, nx.head, nx.batch);
            }
          }
          it = nx;
          have = have_next;
        }
      }
      __syncwarp();
    } else {
      // ---------------- MMA issue: warp 13 for query tile 0, warp 15 for query tile 1 ----------------
      // One thread per query tile, each with its own in-order stream
      //     wait P(h) : O += P(h) V[half h] : S(h + 2) : ...      (half steps of 64 keys)
      // so neither tile ever waits behind the other's barriers, and a tile that is done with an
      // item runs on into its next item as far as the K/V ring lets it.  A tcgen05.mma does not
      // return until the tensor pipe has room for it, so a thread is busy for about as long as its
      // MMAs execute; with one thread for both tiles every wait of one tile delayed the other.
      // A K/V ring entry is released by BOTH threads (kv_empty counts two arrivals); a thread
      // that does not use an entry still waits for it to be loaded before it lets it go, so its
      // arrival can never be counted towards the stage's previous use.
      if (lane == 0) {
        const uint32_t t = (warp == kMmaWarp) ? 0u : 1u;
        // Scalar, latency-bound code in few registers: descriptors are a constant high word plus a
        // low word that is a precomputed base plus a small offset, and barriers are addressed as
        // one 32-bit base plus an index.
        const uint32_t hi_k = static_cast<uint32_t>(make_desc_kmajor_sw128(0) >> 32);
        const uint32_t hi_mn = static_cast<uint32_t>(make_desc_mnmajor_sw128(0, kHalfTileBytes) >> 32);
        const uint32_t q_lo =
            static_cast<uint32_t>(make_desc_kmajor_sw128(smem_u32(smem + L::kQOffset + t * kTileBytes)));
        const uint32_t k_lo = static_cast<uint32_t>(make_desc_kmajor_sw128(smem_u32(smem + L::kKvOffset)));
        const uint32_t v_lo =
            static_cast<uint32_t>(make_desc_mnmajor_sw128(smem_u32(smem + L::kKvOffset), kHalfTileBytes));
        const uint32_t tmem_s = tmem_base + L::kTmemS + t * 128;
        const uint32_t tmem_o = tmem_base + L::kTmemO + t * HD;
        const uint32_t bar0 = smem_u32(bars);
        // barrier indices in `bars`
        constexpr uint32_t kQFull = 0, kQEmpty = 2, kKvFull = 4, kKvEmpty = 4 + kKvStages, kSFull = 4 + 2 * kKvStages,
                           kPFull = kSFull + 4, kOFull = kSFull + 8, kOFree = kSFull + 10, kTurn = kSFull + 16,
                           kPvDone = kSFull + 18;
        auto desc = [](uint32_t lo, uint32_t hi) { return (static_cast<uint64_t>(hi) << 32) | lo; };
        auto wait = [&](uint32_t index, uint32_t parity) { return mbar_wait_addr(bar0 + 8 * index, parity, abort_word); };
        auto commit = [&](uint32_t index) { umma_commit_addr(bar0 + 8 * index); };
        auto wait_entry = [&](uint32_t e) { return wait(kKvFull + e % kKvStages, (e / kKvStages) & 1); };
        auto free_entry = [&](uint32_t e) { commit(kKvEmpty + e % kKvStages); };  // arrives once this thread's MMAs are done
        // S(half hb) = Q (K rows 64 hb .. 64 hb + 63 of ring entry e)^T, into columns 64 hb .. of the tile's score region
        auto issue_scores = [&](uint32_t e, uint32_t hb) {
          const uint32_t b0 = k_lo + (e % kKvStages) * (kTileBytes >> 4) + hb * (8192u >> 4);
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {  // k-steps of 16 over the head dimension (64-wide blocks)
            const uint32_t off = (ks >> 2) * (kHalfTileBytes >> 4) + 2 * (ks & 3);
            umma_f16_ss(tmem_s + hb * 64, desc(q_lo + off, hi_k), desc(b0 + off, hi_k), kIdescS, ks > 0 ? 1u : 0u);
          }
          commit(kSFull + 2 * t + hb);
        };
        // O (+)= P(half hb) V rows 64 hb .. of ring entry e: 4 k-steps of 16 KV rows; A = P from tensor memory
        auto issue_pv = [&](uint32_t e, uint32_t hb, uint32_t accumulate) {
          const uint32_t b0 = v_lo + (e % kKvStages) * (kTileBytes >> 4) + hb * (4u * (2048u >> 4));
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_f16_ts(tmem_o, tmem_s + hb * 64 + ks * 8, desc(b0 + ks * (2048 >> 4), hi_mn), kIdescPV,
                        ks > 0 ? 1u : accumulate);
          commit(kPvDone + t);
        };
        uint32_t e0 = 0;              // ring entry of K_0 of the current item
        uint32_t cq = 0, ch = 0, co = 0;  // Q tiles, half steps and accumulators of this query tile consumed so far
        // The two threads take turns, tile 0 then tile 1, for every half step.  A thread collects
        // everything its MMAs need BEFORE it asks for its turn, and hands the turn on as soon as its
        // PV MMAs are issued (not completed), so the next group queues up behind them.  Measured on
        // the causal bf16 B4 H32 S4096 problem (same box): turns 1108 TFLOP/s; no order at all 1104
        // on another box against 1151 with turns; a lock taken once the probabilities are there and
        // held for the PV MMAs 1077, held for the score MMAs as well 925; the turn handed on before
        // the PV MMAs 1095, after the score MMAs 852.
        uint32_t ct = 0;  // turns taken
        auto take_turn = [&]() {
          const bool got = wait(kTurn + t, t ? (ct & 1u) : ((ct & 1u) ^ 1u));
          ++ct;
          return got;
        };
        auto pass_turn = [&]() { mbar_arrive(turn + (t ^ 1u)); };
        bool ok = true;
        ItemWalk<PAGED> walk(p);
        Item it;
        while (ok && walk.next_busy(it)) {
          const int n = t ? it.n[1] : it.n[0];
          const int nmax = it.nmax;
          // The first score tile of an item needs no turn: a tile that is done with the previous
          // item starts the next one at once, whatever the other tile is still doing.  Both score
          // buffers are free: the PV groups that read the probabilities in them were issued before.
          if (!wait_entry(e0)) break;
          if (n > 0) {
            if (!wait(kQFull + t, cq & 1u)) break;
            ++cq;
            tc_fence_after();
            issue_scores(e0, 0);
            issue_scores(e0, 1);
            if (n == 1) commit(kQEmpty + t);
          }
          free_entry(e0);
          for (int j = 0; j < nmax && ok; ++j) {
            const uint32_t ev = e0 + 2 * j + 1;  // V_j; K_(j+1) is entry ev + 1
            const bool more = j + 1 < nmax;
            // Everything that is normally there long before the probabilities first (the K/V tiles,
            // the turn), so that the path from "P written" to the first MMA is as short as possible.
            if (!wait_entry(ev) || (more && !wait_entry(ev + 1))) { ok = false; break; }
#pragma unroll
            for (uint32_t hb = 0; hb < 2; ++hb) {
              if (!take_turn()) { ok = false; break; }
              if (j < n) {
                if (j == 0 && hb == 0) {  // the accumulator is read by the epilogue of the tile's previous item
                  if (!wait(kOFree + t, (co & 1u) ^ 1u)) { ok = false; break; }
                  ++co;
                }
                if (!wait(kPFull + 2 * t + hb, (ch >> 1) & 1u)) { ok = false; break; }
                ++ch;
                tc_fence_after();
                issue_pv(ev, hb, (j > 0 || hb > 0) ? 1u : 0u);
                pass_turn();
                if (more && j + 1 < n) {
                  issue_scores(ev + 1, hb);  // over the probabilities the PV group above has just been issued for
                  if (j + 2 == n && hb == 1) commit(kQEmpty + t);  // that was the item's last score MMA of this tile
                }
                if (j == n - 1 && hb == 1) commit(kOFull + t);
              } else {
                pass_turn();  // past this tile's diagonal
              }
            }
            if (!ok) break;
            if (j < n) {
              free_entry(ev);
              if (more) free_entry(ev + 1);
            } else {
              // past this tile's diagonal: let the entries go (they have been loaded, see above)
              mbar_arrive(kv_empty + ev % kKvStages);
              if (more) mbar_arrive(kv_empty + (ev + 1) % kKvStages);
            }
          }
          e0 += 2 * nmax;
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
    uint8_t* stage = smem + L::kStageOffset;
    const bool store_thread = (warp == 8 && lane == 0);
    auto epi_barrier = [&]() { asm volatile("bar.sync 1, 128;" ::: "memory"); };
    uint32_t ci[2] = {0, 0};  // items with work per tile so far
    bool ok = true;
    ItemWalk<PAGED> walk(p);
    Item it;
    while (ok && walk.next(it)) {
#pragma unroll 1
      for (int t = 0; t < 2; ++t) {
        const int tile_r0 = it.pair * kPairRows + t * kTileRows;
        if (tile_r0 >= p.seq_q) continue;
        const int q_row = tile_r0 + row_in_tile;
        if (it.n[t] == 0) {
          // no visible key: zeros (rare; plain stores)
          if (q_row < p.seq_q) {
            T* orow = reinterpret_cast<T*>(p.o) + it.batch * p.o_stride_b + it.head * p.o_stride_h +
                      static_cast<int64_t>(q_row) * p.o_stride_s;
#pragma unroll
            for (int v = 0; v < HD / 8; ++v) reinterpret_cast<uint4*>(orow)[v] = make_uint4(0u, 0u, 0u, 0u);
            if (p.lse) p.lse[(static_cast<int64_t>(it.batch) * p.q_heads + it.head) * p.seq_q + q_row] = -INFINITY;
          }
          continue;
        }
        const uint32_t par = ci[t] & 1;
        ++ci[t];
        ok = mbar_wait(o_full + t, par, abort_word) && mbar_wait(l_full + t, par, abort_word);
        // the four warps meet at named barriers below: they give up together or not at all
        ok = bar_red_and(1, 128, ok);
        if (!ok) break;
        tc_fence_after();
        const float m = lsum[(t * 2 + 0) * kTileRows + row_in_tile];
        const float l = lsum[(t * 2 + 1) * kTileRows + row_in_tile];
        const float inv = (l > 0.f) ? 1.0f / l : 0.f;
        if (p.lse && q_row < p.seq_q) {
          // m is in the log2 domain (scores times scale * log2 e), l is relative to it
          p.lse[(static_cast<int64_t>(it.batch) * p.q_heads + it.head) * p.seq_q + q_row] =
              (l > 0.f) ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
        }
        const uint32_t t_o = tmem_base + lane_field + L::kTmemO + t * HD;
#pragma unroll
        for (int c2 = 0; c2 < kBlocks; ++c2) {  // one 64-column block at a time
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
          if (c2 == kBlocks - 1) {
            // accumulator and row sums have been read: release them for the tile's next item
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              mbar_arrive(o_free + t);
              mbar_arrive(l_free + t);
            }
          }
          fence_proxy_async_smem();
          epi_barrier();
          if (store_thread) {
            tma_store_4d(&tmap_o, stage, c2 * 64, tile_r0, it.head, it.batch);
            tma_store_commit();
          }
        }
      }
    }
    if (store_thread) tma_store_wait<0>();
  } else {
    // ---------------- softmax of query tile t = warp / 4 ----------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    const int t = warp >> 2;
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t t_s = tmem_base + lane_field + L::kTmemS + t * 128;  // scores, and P over their first half
    const uint32_t t_o = tmem_base + lane_field + L::kTmemO + t * HD;
    const float scale_log2 = p.scale_log2;
    const float2 scale2 = make_float2(scale_log2, scale_log2);
    uint32_t cs = 0, ci = 0;  // score tiles and items of this query tile so far
    bool ok = true;
    ItemWalk<PAGED> walk(p);
    Item it;
    while (ok && walk.next_busy(it)) {
      const int n = it.n[t];
      if (n == 0) continue;
      const int tile_r0 = it.pair * kPairRows + t * kTileRows;
      const int q_row = tile_r0 + row_in_tile;
      const int kv_len = it.kv_len;
      const int causal_offset = it.causal_offset;
      float m_ref = -INFINITY;  // the max the row's P and running sum are relative to
      float2 l2 = make_float2(0.f, 0.f);
      for (int h = 0; h < 2 * n; ++h, ++cs) {  // half steps of 64 keys, alternating between the two score buffers
        const uint32_t hb = cs & 1u;
        ok = mbar_wait(s_full + 2 * t + hb, (cs >> 1) & 1u, abort_word);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t sr[64];
        tmem_ld_32x32b_x64(t_s + hb * 64, sr);

        const int col0 = h * 64;
        const bool need_mask = (p.causal && col0 + 63 > tile_r0 + causal_offset) || (col0 + 64 > kv_len);
        int limit = 64;  // columns [0, limit) of this half step are visible to this row
        if (need_mask) {
          int vis = kv_len;
          if (p.causal) vis = min(vis, q_row + causal_offset + 1);
          limit = vis - col0;
        }
        tmem_wait_ld();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (i >= limit) sr[i] = 0xff800000u;  // -inf
        }
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 64; i += 8) {
          mx0 = fmax3(mx0, __uint_as_float(sr[i]), __uint_as_float(sr[i + 1]));
          mx1 = fmax3(mx1, __uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3]));
          mx2 = fmax3(mx2, __uint_as_float(sr[i + 4]), __uint_as_float(sr[i + 5]));
          mx3 = fmax3(mx3, __uint_as_float(sr[i + 6]), __uint_as_float(sr[i + 7]));
        }
        const float m_new = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale_log2;
        const bool grow = m_new > m_ref + kRescaleThreshold;  // also true for the first finite max
        if (h > 0 && __any_sync(0xffffffffu, grow)) {
          // Rescale O in place.  The PV group of the previous half step may still be running (the
          // scores read above were issued before it): wait for its completion, the cs-th of this
          // tile.  The next group waits for p_full below.  Rare after the first steps of an item:
          // the max must grow by 2^8.
          ok = mbar_wait(pv_done + t, (cs - 1u) & 1u, abort_word);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          const float alpha = grow ? ex2(m_ref - m_new) : 1.f;  // m_ref = -inf gives 0
#pragma unroll 1
          for (int c = 0; c < HD / 16; ++c) {
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
        if (grow) m_ref = m_new;
        const float m_sub = (m_ref == -INFINITY) ? 0.f : m_ref;
        const float2 negm2 = make_float2(-m_sub, -m_sub);

        // probabilities -> tensor memory (16-bit pairs) over the first half of the scores they came
        // from; masked scores are -inf and give exactly 0
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float2 x = ffma2(make_float2(__uint_as_float(sr[c * 32 + 2 * i]), __uint_as_float(sr[c * 32 + 2 * i + 1])),
                                   scale2, negm2);
            const float2 e = ((kPolyPairMask >> (i & 7)) & 1u) ? exp2_poly2(x) : make_float2(ex2(x.x), ex2(x.y));
            l2 = fadd2(l2, e);
            pk[i] = pack_pair<T>(e.x, e.y);
          }
          tmem_st_32x32b_x16(t_s + hb * 64 + c * 16, pk);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full + 2 * t + hb);
      }
      if (!ok) break;
      // hand (max, sum) of the item to the epilogue warps
      ok = mbar_wait(l_free + t, (ci & 1) ^ 1, abort_word);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ++ci;
      lsum[(t * 2 + 0) * kTileRows + row_in_tile] = m_ref;
      lsum[(t * 2 + 1) * kTileRows + row_in_tile] = l2.x + l2.y;
      __syncwarp();
      if (lane == 0) mbar_arrive(l_full + t);
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
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <typename T, int HD, bool PAGED>
int launch_typed(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to,
                 const AttnParams& p, cudaStream_t stream) {
  auto kfn = attn_fwd_kernel<T, HD, PAGED>;
  static bool configured[64] = {};  // per instantiation and device ordinal
  int rc = ensure_dynamic_smem(kfn, AttnSmem<HD>::kTotal, configured, "cudaFuncSetAttribute(attention smem)");
  if (rc) return rc;
  const int sms = num_sms();
  const int grid = p.num_units < sms ? p.num_units : sms;
  kfn<<<grid, kAttnThreads, AttnSmem<HD>::kTotal, stream>>>(tq, tk, tv, to, p);
  return check_cuda(cudaGetLastError(), "attn_fwd_kernel launch");
}

template <bool PAGED>
int launch_any(int dtype, int head_dim, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
               const CUtensorMap& to, const AttnParams& p, cudaStream_t stream) {
  if (head_dim == 128) {
    if (dtype == B200K_F16) return launch_typed<__half, 128, PAGED>(tq, tk, tv, to, p, stream);
    return launch_typed<__nv_bfloat16, 128, PAGED>(tq, tk, tv, to, p, stream);
  }
  if (dtype == B200K_F16) return launch_typed<__half, 64, PAGED>(tq, tk, tv, to, p, stream);
  return launch_typed<__nv_bfloat16, 64, PAGED>(tq, tk, tv, to, p, stream);
}

// Work units: see ItemWalk.
int fill_units(AttnParams& p, const char* who) {
  p.num_pairs = (p.seq_q + kPairRows - 1) / kPairRows;
  p.units_per_head = p.causal ? (p.num_pairs + 1) / 2 : p.num_pairs;
  const int64_t units = static_cast<int64_t>(p.batch) * p.q_heads * p.units_per_head;
  if (units > INT32_MAX) return set_error(B200K_ERR_BAD_SHAPE, "%s: too many query tiles", who);
  p.num_units = static_cast<int32_t>(units);
  return B200K_OK;
}

// Which kernel runs a problem (B200K_ATTN_AUTO).  Measured on B200, head dim 128, same box and
// timing loop, one-tile / tile-pair in microseconds.  Non-causal: 8x32x1024 128 / 134, 8x32x2048
// 472 / 473, 4x32x4096 992 / 1030, 1x16x16384 1827 / 2026.  Causal, many rounds of units: 4x32x4096
// 539 / 510, 1x32(8)x16384 2073 / 1995, 2x32(8)x8192 1045 / 1026, but 4x32(8)x2048 155 / 173, where the
// pair kernel's 512 units leave the last of four rounds over 148 SMs half empty, and 4x8x4096 (256
// units, 86 % of two rounds) 152 / 158.  Causal, one or two rounds filled to 86 % (a head shard of
// a long prefill on 8 GPUs): 1x8x8192 144 / 136, 4x4(1)x4096 80 / 76, 1x4x16384 273 / 248, 2x8x8192
// 285 / 269, 1x16(4)x8192 281 / 266, but 4x6(2)x2048 41 / 45, 8x8x1024 40 / 41, 2x4x2048 41 / 43.
// So: head dim 64 only exists in the pair kernel; causal problems take it when its units fill the
// SMs to 90 % or more, or fill one round (two rounds) to 80 % with at least 24 (48) K/V tiles to
// walk; everything else takes the one-tile kernel.
bool choose_pair_kernel(int kernel, int head_dim, bool causal, int64_t pair_units, int64_t kv_tiles) {
  if (head_dim != 128) return true;
  if (kernel == B200K_ATTN_TILE_PAIR) return true;
  if (kernel == B200K_ATTN_ONE_TILE) return false;
  if (!causal) return false;
  const int64_t sms = num_sms();
  const int64_t rounds = (pair_units + sms - 1) / sms;
  if (pair_units * 10 >= rounds * sms * 9) return true;
  return rounds <= 2 && pair_units * 10 >= rounds * sms * 8 && kv_tiles >= (rounds == 1 ? 24 : 48);
}

}  // namespace

int launch_attention_fwd(const b200k_attention_args& a, cudaStream_t stream) {
  if (!a.q || !a.k || !a.v || !a.o) return set_error(B200K_ERR_NULL, "attention_fwd: q, k, v and o must be non-NULL");
  if (a.batch <= 0 || a.q_heads <= 0 || a.kv_heads <= 0 || a.seq_q <= 0 || a.seq_kv <= 0)
    return set_error(B200K_ERR_BAD_SHAPE, "attention_fwd: all dimensions must be positive");
  if (a.head_dim != 128 && a.head_dim != 64)
    return set_error(B200K_ERR_BAD_SHAPE, "attention_fwd: head_dim must be 128 or 64");
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
  if (a.kernel < B200K_ATTN_AUTO || a.kernel > B200K_ATTN_TILE_PAIR)
    return set_error(B200K_ERR_BAD_SHAPE, "attention_fwd: unknown kernel choice %d", a.kernel);
  if (a.kernel == B200K_ATTN_ONE_TILE && a.head_dim != 128)
    return set_error(B200K_ERR_BAD_SHAPE, "attention_fwd: the one-tile kernel covers head_dim 128 only");
  int rc = ensure_sm100();
  if (rc) return rc;
  {
    const int64_t pairs = (a.seq_q + kPairRows - 1) / kPairRows;
    const int64_t units = static_cast<int64_t>(a.batch) * a.q_heads * (a.causal ? (pairs + 1) / 2 : pairs);
    if (!choose_pair_kernel(a.kernel, a.head_dim, a.causal != 0, units, (a.seq_kv + 127) / 128))
      return launch_attention_fwd_tile(a, stream);
  }

  CUtensorMap tq, tk, tv, to;
  const uint32_t box[4] = {64, kTileRows, 1, 1};
  const uint64_t hd = static_cast<uint64_t>(a.head_dim);
  {
    uint64_t dims[4] = {hd, static_cast<uint64_t>(a.seq_q), static_cast<uint64_t>(a.q_heads),
                        static_cast<uint64_t>(a.batch)};
    uint64_t st[3] = {static_cast<uint64_t>(a.q_stride_s) * 2, static_cast<uint64_t>(a.q_stride_h) * 2,
                      static_cast<uint64_t>(a.q_stride_b) * 2};
    rc = encode_tmap(&tq, a.dtype, 4, const_cast<void*>(a.q), dims, st, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[4] = {hd, static_cast<uint64_t>(a.seq_kv), static_cast<uint64_t>(a.kv_heads),
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
    uint64_t dims[4] = {hd, static_cast<uint64_t>(a.seq_q), static_cast<uint64_t>(a.q_heads),
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
  rc = fill_units(p, "attention_fwd");
  if (rc) return rc;
  p.scale_log2 = a.scale * kLog2e;
  p.status = a.status;
  p.lse = a.lse;
  p.block_table = nullptr;
  p.seq_lens = nullptr;
  p.block_table_stride = p.page_size = p.num_pages = 0;
  return launch_any<false>(a.dtype, a.head_dim, tq, tk, tv, to, p, stream);
}

int launch_paged_attention_fwd(const b200k_paged_attention_args& a, cudaStream_t stream) {
  if (!a.q || !a.k_cache || !a.v_cache || !a.o || !a.block_table || !a.seq_lens)
    return set_error(B200K_ERR_NULL, "paged_attention_fwd: q, k_cache, v_cache, o, block_table, seq_lens must be non-NULL");
  if (a.batch <= 0 || a.q_heads <= 0 || a.kv_heads <= 0 || a.seq_q <= 0 || a.max_seq_kv <= 0)
    return set_error(B200K_ERR_BAD_SHAPE, "paged_attention_fwd: all dimensions must be positive");
  if (a.head_dim != 128 && a.head_dim != 64)
    return set_error(B200K_ERR_BAD_SHAPE, "paged_attention_fwd: head_dim must be 128 or 64");
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
  if (a.kernel < B200K_ATTN_AUTO || a.kernel > B200K_ATTN_TILE_PAIR)
    return set_error(B200K_ERR_BAD_SHAPE, "paged_attention_fwd: unknown kernel choice %d", a.kernel);
  if (a.kernel == B200K_ATTN_ONE_TILE && a.head_dim != 128)
    return set_error(B200K_ERR_BAD_SHAPE, "paged_attention_fwd: the one-tile kernel covers head_dim 128 only");
  int rc = ensure_sm100();
  if (rc) return rc;
  {
    const int64_t pairs = (a.seq_q + kPairRows - 1) / kPairRows;
    const int64_t units = static_cast<int64_t>(a.batch) * a.q_heads * (a.causal ? (pairs + 1) / 2 : pairs);
    if (!choose_pair_kernel(a.kernel, a.head_dim, a.causal != 0, units, (a.max_seq_kv + 127) / 128))
      return launch_paged_attention_fwd_tile(a, stream);
  }

  CUtensorMap tq, tk, tv, to;
  const uint32_t box[4] = {64, kTileRows, 1, 1};
  const uint32_t page_box[4] = {64, static_cast<uint32_t>(a.page_size), 1, 1};
  const uint64_t hd = static_cast<uint64_t>(a.head_dim);
  {
    uint64_t dims[4] = {hd, static_cast<uint64_t>(a.seq_q), static_cast<uint64_t>(a.q_heads),
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
    uint64_t dims[4] = {hd, static_cast<uint64_t>(a.page_size), static_cast<uint64_t>(a.kv_heads),
                        static_cast<uint64_t>(a.num_pages)};
    uint64_t st[3] = {hd * 2, static_cast<uint64_t>(a.kv_head_stride) * 2,
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
  rc = fill_units(p, "paged_attention_fwd");
  if (rc) return rc;
  p.scale_log2 = a.scale * kLog2e;
  p.status = a.status;
  p.lse = nullptr;
  p.block_table = a.block_table;
  p.seq_lens = a.seq_lens;
  p.block_table_stride = a.block_table_stride;
  p.page_size = a.page_size;
  p.num_pages = a.num_pages;
  return launch_any<true>(a.dtype, a.head_dim, tq, tk, tv, to, p, stream);
}

}  // namespace b200k
