// GEMM C[M, N] = A[M, K] * B[N, K]^T (f16 / bf16, K contiguous in both operands) with a 256 x 256
// output tile computed by a PAIR of SMs (a cluster of two CTAs, tcgen05 cta_group::2).
//
// Why: with one CTA per tile, a 128 x 256 tile needs 96 bytes of operands per tensor-core cycle
// from L2, more than an SM receives (measured: ~750 instead of 512 cycles per 64-wide k-block), and
// a 256 x 256 tile halves the number of tiles, which leaves SMs idle on mid-sized problems
// (2048^3: 64 tiles on 148 SMs).  In a pair, CTA r loads rows [128 r, 128 r + 128) of the A tile
// and rows [128 r, 128 r + 128) of the B tile (32 KB per k-block instead of 48), and one
// tcgen05.mma.cta_group::2 (M = 256, N = 256) makes both tensor cores multiply their own A half
// with BOTH B halves, reading the peer's half through the cluster's shared memory: 64 bytes per
// tensor-core cycle per SM, with as many CTAs as 128 x 256 tiles would give.
//
// Roles per CTA (6 warps, as in the single-CTA kernel): warp 0 TMA producer (its own halves),
// warp 1 = MMA issuer in the leader CTA (rank 0; idle in the peer), warps 2..5 epilogue (each CTA
// stores its own 128 rows).  Barriers that cross the pair: both producers' TMA loads count their
// bytes on the LEADER's "stage loaded" barrier (cta_group::2 form of the load), so the MMA thread
// waits on one barrier per stage; the peer's epilogue warps arrive on the leader's "accumulator
// drained" barrier through its cluster address; the leader's tcgen05.commit arrives on the
// "stage consumed" / "accumulator ready" barriers of both CTAs (one commit per CTA).  Every wait
// is bounded.  (A first version forwarded "my stage has landed" from a relay thread in the peer
// with mbarrier.arrive.release.cluster: ~1200 cycles per arrival, which made the relay the
// bottleneck -- 2.3x slower than this form.)
//
// Measured (B200, f16, per 64-wide k-block and SM): ~610 cycles against 512 of tensor-core time,
// the same with operands that never leave L2, so the limit is inside the SM.  It fits a shared-
// memory port of 128 bytes per cycle that serves operand reads and TMA writes alike, where each
// CTA's B half is read once per consuming SM: (16 + 16 + 16) KB read + 32 KB written = 80 KB
// -> 640 cycles (a single CTA with a 128 x 256 tile: 48 + 48 KB -> 750, measured ~750).  That is
// the efficiency of the single-CTA 256 x 256 tile at the granularity of 128 x 256 tiles; against
// the single-CTA kernel's own choice of tile it is 0-16 % slower on 12 of 13 shapes tried and 6 %
// faster on 2048 x 2048 x 8192, so it is offered as an explicit choice (tile_m =
// B200K_TILE_SM_PAIR) and not picked automatically.
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace b200k {
namespace {

constexpr int kThreads = 192;
constexpr int kRows = 128;          // A rows and B rows per CTA
constexpr int kPairN = 256;         // output tile is 256 x 256 per pair
constexpr int kStageHalf = kRows * 128;  // 16 KB: 128 rows x 128 bytes
constexpr int kStageBytes = 2 * kStageHalf;
constexpr int kStages = 6;
constexpr int kStagingOffset = kStages * kStageBytes;
constexpr int kStagingBytes = 4 * 2 * 4096;
constexpr int kBarOffset = kStagingOffset + kStagingBytes;
// full[S] empty[S] tfull[2] tempty[2]
constexpr int kNumBars = 2 * kStages + 4;
constexpr int kSmem = kBarOffset + kNumBars * 8 + 16 + 1024;
constexpr uint32_t kTmemCols = 512;  // two accumulator buffers of 256 columns

struct PairParams {
  void* c;
  int64_t ldc;
  int32_t m, n, num_kb;
  int32_t tiles_m, tiles_n;  // in 256 x 256 pair tiles
  int32_t tma_store_ok;
  int32_t* status;
};

// ---- cluster / cta_group::2 wrappers (only this kernel uses them) ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// cluster-wide address of `local` in the CTA with rank `rank`
__device__ __forceinline__ uint32_t map_to_cta(const void* local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(local)), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load of this CTA's box whose completion bytes are counted on a barrier of the pair's LEADER
// CTA (`bar_cluster_addr`, a cluster address): the leader's MMA thread then waits on one barrier
// for both CTAs' halves of a stage.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tmap, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
// Non-blocking test with cluster-scope acquire: barriers that the other CTA (or its TMA loads)
// arrives on are polled by the one thread that waits on them.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// bounded like mbar_wait; for barriers that threads of the other CTA arrive on
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_word) {
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (!mbar_try_wait_cluster(bar, parity)) {
    if ((++spins & 0x3ffu) == 0) {
      if (*abort_word != 0) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > kWaitLimitNs) {
        *abort_word = 1;
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ void umma_pair_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives once on the barrier at `cluster_addr` (in either CTA) when the pair's MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}

template <typename OutT>
__device__ __forceinline__ OutT to_out(float v);
template <>
__device__ __forceinline__ float to_out<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ __half to_out<__half>(float v) {
  return __float2half_rn(v);
}
template <>
__device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

template <bool BF16, typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_c, const PairParams p) {
  constexpr uint32_t kFmt = BF16 ? kFmtBF16 : kFmtF16;
  constexpr uint32_t kIdesc = make_idesc(kFmt, kFmt, 256, kPairN, 0, 0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kBarOffset);  // (leader) stage loaded in both CTAs
  uint64_t* empty = full + kStages;                                 // stage consumed by the pair's MMAs
  uint64_t* tfull = empty + kStages;                                // [buffer] accumulator complete
  uint64_t* tempty = tfull + 2;                                     // (leader) [buffer] drained by both CTAs
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile uint32_t* abort_word = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull + a, 1);
      mbar_init(tempty + a, 8);  // four epilogue warps of each CTA
    }
    *abort_word = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    prefetch_tmap(&tmap_c);
  }
  if (warp == 1) {
    // each CTA allocates its own tensor memory (all 512 columns, so both get base 0); only the
    // MMA and its commit are pair-wide instructions
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_pairs = gridDim.x / 2;
  const int pair = blockIdx.x / 2;
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    // ---------------- TMA producer: this CTA's halves of A and B ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        const int tm = t / p.tiles_n, tn = t - tm * p.tiles_n;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          // in the peer CTA this barrier is signalled from the leader's SM
          if (!(leader ? mbar_wait(empty + stage, phase ^ 1, abort_word)
                       : mbar_wait_cluster(empty + stage, phase ^ 1, abort_word))) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kStageBytes;
          // the bytes of both CTAs are counted on the leader's barrier; the leader announces them
          if (leader) mbar_arrive_expect_tx(full + stage, 2 * kStageBytes);
          const uint32_t bar = map_to_cta(full + stage, 0);
          const int kx = kb * 64;
          tma_load_2d_pair(sa, &tmap_a, bar, kx, tm * 256 + static_cast<int>(rank) * kRows);
          tma_load_2d_pair(sa + kStageHalf, &tmap_b, bar, kx, tn * kPairN + static_cast<int>(rank) * kRows);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ---------------- leader: issues the pair's MMAs ----------------
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      const uint32_t hi = static_cast<uint32_t>(make_desc_kmajor_sw128(0) >> 32);
      const uint32_t lo0 = static_cast<uint32_t>(make_desc_kmajor_sw128(smem_u32(smem)));
      auto desc = [](uint32_t lo, uint32_t h) { return (static_cast<uint64_t>(h) << 32) | lo; };
      for (int t = pair; t < num_tiles && ok; t += num_pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait_cluster(tempty + acc, acc_phase ^ 1, abort_word)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kPairN;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait_cluster(full + stage, phase, abort_word)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_lo = lo0 + stage * (kStageBytes >> 4);
          const uint32_t b_lo = a_lo + (kStageHalf >> 4);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_pair_f16(d_tmem, desc(a_lo + 2 * k, hi), desc(b_lo + 2 * k, hi), kIdesc, (kb | k) != 0 ? 1u : 0u);
          // the stage is free in both CTAs once these MMAs have read it
          umma_commit_pair(map_to_cta(empty + stage, 0));
          umma_commit_pair(map_to_cta(empty + stage, 1));
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) {
          umma_commit_pair(map_to_cta(tfull + acc, 0));
          umma_commit_pair(map_to_cta(tfull + acc, 1));
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue: this CTA's 128 rows of the pair tile ----------------
    const int quarter = warp & 3;
    uint8_t* staging = smem + kStagingOffset + (warp - 2) * (2 * 4096);
    const uint32_t tempty_leader[2] = {map_to_cta(tempty + 0, 0), map_to_cta(tempty + 1, 0)};
    OutT* cbase = reinterpret_cast<OutT*>(p.c);
    uint32_t stg_count = 0;
    int it = 0;
    for (int t = pair; t < num_tiles; t += num_pairs, ++it) {
      const int tm = t / p.tiles_n, tn = t - tm * p.tiles_n;
      const int acc = it & 1;
      bool ok = leader ? mbar_wait(tfull + acc, (it >> 1) & 1, abort_word)
                       : mbar_wait_cluster(tfull + acc, (it >> 1) & 1, abort_word);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row0 = tm * 256 + static_cast<int>(rank) * kRows + quarter * 32;
      const int row = row0 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kPairN;
      constexpr int kCols = 128 / static_cast<int>(sizeof(OutT));
      if (p.tma_store_ok) {
#pragma unroll 1
        for (int c = 0; c < kPairN / kCols; ++c) {
          uint8_t* buf = staging + (stg_count & 1) * 4096;
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
          uint4 v[8];
          if constexpr (sizeof(OutT) == 4) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
          } else {
            uint32_t r[64];
            tmem_ld_32x32b_x64(taddr + c * 64, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              union {
                uint4 u;
                OutT e[8];
              } pk;
#pragma unroll
              for (int j = 0; j < 8; ++j) pk.e[j] = to_out<OutT>(__uint_as_float(r[8 * i + j]));
              v[i] = pk.u;
            }
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) *reinterpret_cast<uint4*>(buf + lane * 128 + ((i ^ (lane & 7)) << 4)) = v[i];
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmap_c, buf, tn * kPairN + c * kCols, row0);
            tma_store_commit();
          }
          ++stg_count;
        }
      } else {
#pragma unroll 2
        for (int c = 0; c < kPairN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c * 32, r);
          tmem_wait_ld();
          const int col = tn * kPairN + c * 32;
          if (row < p.m) {
            OutT* dst = cbase + static_cast<int64_t>(row) * p.ldc + col;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col + i < p.n) dst[i] = to_out<OutT>(__uint_as_float(r[i]));
          }
        }
      }
      // this warp has drained its part of the accumulator: tell the leader's MMA thread
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(tempty_leader[acc]);
    }
    if (lane == 0) tma_store_wait<0>();
    __syncwarp();
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {
    }
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, kStatusGemmTimeout);
    __syncthreads();
  }
  cluster_sync();  // nothing of the peer is touched after this point
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <bool BF16, typename OutT>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const PairParams& p, int grid,
                cudaStream_t stream) {
  auto kfn = gemm_pair_kernel<BF16, OutT>;
  static bool configured[64] = {};  // per instantiation and device ordinal
  int rc = ensure_dynamic_smem(kfn, kSmem, configured, "cudaFuncSetAttribute(pair gemm smem)");
  if (rc) return rc;
  kfn<<<grid, kThreads, kSmem, stream>>>(ta, tb, tc, p);
  return check_cuda(cudaGetLastError(), "gemm_pair_kernel launch");
}

}  // namespace

bool gemm_pair_eligible(const b200k_gemm_args& a) {
  if (a.in_dtype != B200K_F16 && a.in_dtype != B200K_BF16) return false;
  if (a.out_dtype != B200K_F32 && a.out_dtype != a.in_dtype) return false;
  if (a.bias || a.activation != 0 || a.a_km || a.b_kn) return false;
  if (!a.a || !a.b || !a.c || a.m <= 0 || a.n <= 0 || a.k <= 0) return false;
  if (a.m > INT32_MAX || a.n > INT32_MAX || a.k > INT32_MAX) return false;
  const size_t in_es = 2;
  if ((reinterpret_cast<uintptr_t>(a.a) & 15) || (reinterpret_cast<uintptr_t>(a.b) & 15) ||
      (a.lda * in_es) % 16 != 0 || (a.ldb * in_es) % 16 != 0 || a.lda < a.k || a.ldb < a.k || a.ldc < a.n)
    return false;
  return true;
}

int launch_gemm_pair(const b200k_gemm_args& a, cudaStream_t stream) {
  if (!gemm_pair_eligible(a))
    return set_error(B200K_ERR_BAD_SHAPE, "gemm (SM-pair kernel): needs f16 / bf16 NT operands, no fused epilogue");
  int rc = ensure_sm100();
  if (rc) return rc;
  const size_t out_es = dtype_size(a.out_dtype);
  if (reinterpret_cast<uintptr_t>(a.c) % out_es != 0)
    return set_error(B200K_ERR_BAD_ALIGN, "gemm: C is not aligned to its element size");

  CUtensorMap ta, tb, tc;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(a.k), static_cast<uint64_t>(a.m)};
    uint64_t strides[1] = {static_cast<uint64_t>(a.lda) * 2};
    uint32_t box[2] = {64, kRows};
    rc = encode_tmap(&ta, a.in_dtype, 2, const_cast<void*>(a.a), dims, strides, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[2] = {static_cast<uint64_t>(a.k), static_cast<uint64_t>(a.n)};
    uint64_t strides[1] = {static_cast<uint64_t>(a.ldb) * 2};
    uint32_t box[2] = {64, kRows};
    rc = encode_tmap(&tb, a.in_dtype, 2, const_cast<void*>(a.b), dims, strides, box);
    if (rc) return rc;
  }
  PairParams p;
  p.c = a.c;
  p.ldc = a.ldc;
  p.m = static_cast<int32_t>(a.m);
  p.n = static_cast<int32_t>(a.n);
  p.num_kb = static_cast<int32_t>((a.k + 63) / 64);
  p.tiles_m = static_cast<int32_t>((a.m + 255) / 256);
  p.tiles_n = static_cast<int32_t>((a.n + kPairN - 1) / kPairN);
  p.status = a.status;
  p.tma_store_ok = ((reinterpret_cast<uintptr_t>(a.c) & 15) == 0 && (a.ldc * out_es) % 16 == 0) ? 1 : 0;
  if (p.tma_store_ok) {
    uint64_t dims[2] = {static_cast<uint64_t>(a.n), static_cast<uint64_t>(a.m)};
    uint64_t strides[1] = {static_cast<uint64_t>(a.ldc) * out_es};
    uint32_t box[2] = {static_cast<uint32_t>(128 / out_es), 32};
    rc = encode_tmap(&tc, a.out_dtype, 2, a.c, dims, strides, box);
    if (rc) return rc;
  } else {
    tc = ta;  // unused
  }
  const int64_t tiles = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
  const int max_pairs = num_sms() / 2;
  const int pairs = static_cast<int>(tiles < max_pairs ? tiles : max_pairs);
  const int grid = 2 * pairs;
  const bool bf16 = a.in_dtype == B200K_BF16;
  if (a.out_dtype == B200K_F32)
    return bf16 ? launch_pair<true, float>(ta, tb, tc, p, grid, stream) : launch_pair<false, float>(ta, tb, tc, p, grid, stream);
  return bf16 ? launch_pair<true, __nv_bfloat16>(ta, tb, tc, p, grid, stream)
              : launch_pair<false, __half>(ta, tb, tc, p, grid, stream);
}

}  // namespace b200k
