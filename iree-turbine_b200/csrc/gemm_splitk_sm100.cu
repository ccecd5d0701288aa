// Split-K GEMM on sm_100a for problems whose whole output tiles would leave most SMs idle (few
// tiles, long K: weight gradients, narrow projections).
//
// The grid is tiles x split CTAs in thread-block clusters of `split` (2, 4 or 8).  The CTAs of a
// cluster compute the same 128 x BN output tile over consecutive slices of K with the same
// TMA-fed operand ring and tcgen05 MMAs as the whole-tile kernel, then leave their fp32 partial
// tiles in their own shared memory (in the drained ring).  After a cluster barrier every CTA sums
// one band of 128 / split rows over all partials, in rank order, reading its peers through
// distributed shared memory, applies the epilogue and writes the band.  No global scratch and no
// atomics: the result does not depend on timing and is reproducible bit for bit.
//
// CTA = 6 warps as in the whole-tile kernel: warp 0 TMA producer, warp 1 MMA issuer and owner of
// tensor memory, warps 2..5 move the accumulator to shared memory; all six reduce.
#include "common.cuh"
#include "gemm_common.cuh"
#include "ptx.cuh"

namespace b200k {
namespace {

using namespace gemm_detail;

// Stand-in for an absent fp8 scale: the pointer is chosen first and the load is unconditional, so no
// ordering of test and load can touch a null pointer.
__device__ const float kUnitScale = 1.0f;


template <typename OutT>
struct ReduceCtx {
  const GemmParams& p;
  uint32_t smem_base;  // shared-memory address of this CTA's partial tile
  int rank, tm, tn, bz;
};

// CTA `rank` of a cluster of SPLIT sums rows [rank * 128 / SPLIT, (rank + 1) * 128 / SPLIT) of the
// tile over all partial tiles, in rank order, and stores them.  A thread takes four 16-byte chunks
// at a time and issues all their peer loads before the first add, so the latency of distributed
// shared memory is paid once per batch, not once per chunk.
template <int BN, int KIND, typename OutT, int EPI, int SPLIT>
__device__ __forceinline__ void reduce_band(const ReduceCtx<OutT>& c) {
  const GemmParams& p = c.p;
  constexpr int kChunksPerRow = BN / 4;
  constexpr int kRows = kBM / SPLIT;
  constexpr int kUnits = kRows * kChunksPerRow;
  constexpr int kBatch = 4;
  float scale = 1.0f;
  if constexpr (KIND == kKindE4M3) {
    const float* sa = p.scale_a ? p.scale_a : &kUnitScale;
    const float* sb = p.scale_b ? p.scale_b : &kUnitScale;
    scale = *sa * *sb;
  }
  OutT* cbase = reinterpret_cast<OutT*>(p.c) + c.bz * p.c_batch_stride;
  for (int u0 = threadIdx.x; u0 < kUnits; u0 += kGemmThreads * kBatch) {
    float4 sum[kBatch];
    uint32_t off[kBatch];
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      const int u = min(u0 + b * kGemmThreads, kUnits - 1);  // past the end: re-read the last unit, not stored
      const int lr = c.rank * kRows + u / kChunksPerRow;
      const int ch = u % kChunksPerRow;
      off[b] = static_cast<uint32_t>(lr * (BN * 4) + ((ch ^ (lr & 7)) << 4));
      sum[b] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float4 v[SPLIT][kBatch];
#pragma unroll
    for (int s = 0; s < SPLIT; ++s)
#pragma unroll
      for (int b = 0; b < kBatch; ++b)
        v[s][b] = ld_shared_cluster_f32x4(cluster_map_shared(c.smem_base + off[b], static_cast<uint32_t>(s)));
#pragma unroll
    for (int s = 0; s < SPLIT; ++s)
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        sum[b].x += v[s][b].x;
        sum[b].y += v[s][b].y;
        sum[b].z += v[s][b].z;
        sum[b].w += v[s][b].w;
      }
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      const int u = u0 + b * kGemmThreads;
      if (u >= kUnits) break;
      const int lr = c.rank * kRows + u / kChunksPerRow;
      const int ch = u % kChunksPerRow;
      const int row = c.tm * kBM + lr;
      const int col = c.tn * BN + ch * 4;
      if (row >= p.m || col >= p.n) continue;
      uint32_t r[4] = {__float_as_uint(sum[b].x), __float_as_uint(sum[b].y), __float_as_uint(sum[b].z),
                       __float_as_uint(sum[b].w)};
      if constexpr (EPI == 2) {
        // the bias index is clamped, not predicated: every load is in bounds whatever the compiler
        // does with its order (columns past n are not stored)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          r[j] = __float_as_uint(apply_act(
              __uint_as_float(r[j]) * scale + load_bias(p.bias, p.bias_dtype, min(col + j, p.n - 1)), p.act));
      } else if constexpr (EPI == 1) {
#pragma unroll
        for (int j = 0; j < 4; ++j) r[j] = __float_as_uint(apply_act(__uint_as_float(r[j]) * scale, p.act));
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * scale);
      }
      OutT* dst = cbase + static_cast<int64_t>(row) * p.ldc + col;
      if (col + 4 <= p.n && p.vec_store_ok) {
        if constexpr (sizeof(OutT) == 4) {
          *reinterpret_cast<uint4*>(dst) = make_uint4(r[0], r[1], r[2], r[3]);
        } else {
          union {
            uint2 u2;
            OutT e[4];
          } pk;
#pragma unroll
          for (int j = 0; j < 4; ++j) pk.e[j] = to_out<OutT>(__uint_as_float(r[j]));
          *reinterpret_cast<uint2*>(dst) = pk.u2;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (col + j < p.n) dst[j] = to_out<OutT>(__uint_as_float(r[j]));
      }
    }
  }
}

// EPI: 0 = plain store, 1 = activation only, 2 = bias (+ activation).  Separate instantiations, so
// the plain kernel carries no epilogue code and the bias pointer is never tested at run time: the
// activation-only kernel has no bias loads at all (with a run-time null test the compiler was seen
// to issue the loads before the test in this loop, which faults on a null bias).
template <int BN, int KIND, typename OutT, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_splitk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const GemmParams p) {
  using S = GemmSmem<BN, 1>;
  static_assert(kBM * BN * 4 <= S::kStages * S::kStageBytes, "the partial tile must fit in the operand ring");
  constexpr int kElemsPerStage = (KIND == kKindE4M3) ? 128 : 64;  // K elements in 128 bytes
  constexpr uint32_t kFmt = (KIND == kKindBF16) ? kFmtBF16 : (KIND == kKindF16 ? kFmtF16 : kFmtE4M3);
  constexpr uint32_t kIdesc = make_idesc(kFmt, kFmt, kBM, BN, 0, 0);
  constexpr uint32_t kTmemCols = BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty = full + S::kStages;
  uint64_t* tfull = empty + S::kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull + 4);
  volatile uint32_t* abort_word = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::kStages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    mbar_init(tfull, 1);
    *abort_word = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // This CTA: tile of its cluster, slice of the k-blocks by its rank.
  const int rank = static_cast<int>(cluster_ctarank());
  const int tiles_per_problem = p.tiles_m * p.tiles_n;
  const int tile = static_cast<int>(blockIdx.x) / p.split;
  const int bz = tile / tiles_per_problem;
  int tm, tn;
  tile_coords(tile - bz * tiles_per_problem, p.tiles_m, p.tiles_n, tm, tn);
  const int kb_begin = rank * p.kb_per_split;
  const int kb_end = min(p.num_kb, kb_begin + p.kb_per_split);
  const bool a_mn = KIND != kKindE4M3 && p.a_mn != 0;
  const bool b_mn = KIND != kKindE4M3 && p.b_mn != 0;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(empty + stage, phase ^ 1, abort_word)) break;
        uint8_t* sa = smem + stage * S::kStageBytes;
        mbar_arrive_expect_tx(full + stage, S::kStageBytes);
        if (a_mn) {
#pragma unroll
          for (int b = 0; b < kBM / 64; ++b)
            tma_load_3d(sa + b * 8192, &tmap_a, full + stage, tm * kBM + b * 64, kb * kElemsPerStage, bz);
        } else {
          tma_load_3d(sa, &tmap_a, full + stage, kb * kElemsPerStage, tm * kBM, bz);
        }
        if (b_mn) {
#pragma unroll
          for (int b = 0; b < BN / 64; ++b)
            tma_load_3d(sa + S::kABytes + b * 8192, &tmap_b, full + stage, tn * BN + b * 64, kb * kElemsPerStage, bz);
        } else {
          tma_load_3d(sa + S::kABytes, &tmap_b, full + stage, kb * kElemsPerStage, tn * BN, bz);
        }
        if (++stage == S::kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // Per-operand descriptor pieces, chosen once: a K-major operand advances 32 bytes per MMA
      // inside the swizzle atom; an MN-major one ([K, R] storage, 64-element blocks 8 KB apart)
      // advances 16 K-rows = 2 KB and carries its block stride in the low word.
      auto desc = [](uint32_t lo, uint32_t h) { return (static_cast<uint64_t>(h) << 32) | lo; };
      const uint64_t d_k = make_desc_kmajor_sw128(smem_u32(smem));
      const uint64_t d_mn = make_desc_mnmajor_sw128(smem_u32(smem), 8192);
      const uint32_t lo0_a = static_cast<uint32_t>(a_mn ? d_mn : d_k), hi_a = static_cast<uint32_t>((a_mn ? d_mn : d_k) >> 32);
      const uint32_t lo0_b = static_cast<uint32_t>(b_mn ? d_mn : d_k), hi_b = static_cast<uint32_t>((b_mn ? d_mn : d_k) >> 32);
      const uint32_t step_a = a_mn ? (2048u >> 4) : 2u;
      const uint32_t step_b = b_mn ? (2048u >> 4) : 2u;
      const uint32_t idesc = kIdesc | (a_mn ? 1u << 15 : 0u) | (b_mn ? 1u << 16 : 0u);
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(full + stage, phase, abort_word)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_lo = lo0_a + stage * (S::kStageBytes >> 4);
        const uint32_t b_lo = lo0_b + stage * (S::kStageBytes >> 4) + (S::kABytes >> 4);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t accum = (kb != kb_begin || k != 0) ? 1u : 0u;
          if constexpr (KIND == kKindE4M3)
            umma_f8_ss(tmem_base, desc(a_lo + step_a * k, hi_a), desc(b_lo + step_b * k, hi_b), idesc, accum);
          else
            umma_f16_ss(tmem_base, desc(a_lo + step_a * k, hi_a), desc(b_lo + step_b * k, hi_b), idesc, accum);
        }
        umma_commit(empty + stage);  // frees the stage once these MMAs have read it
        if (++stage == S::kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) umma_commit(tfull);  // partial accumulator complete
    }
    __syncwarp();
  } else {
    // ---------------- accumulator -> shared memory ----------------
    // Row r of the fp32 partial tile at r * BN * 4 bytes, its 16-byte chunk c at position
    // c ^ (r & 7): conflict-free for these per-row writes and for the per-chunk reads below.  The
    // operand ring is free: once the accumulator barrier has fired every load has landed and every
    // MMA has read its operands.
    bool ok = mbar_wait(tfull, 0, abort_word);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const int quarter = warp & 3;
      const int lr = quarter * 32 + lane;
      uint8_t* prow = smem + lr * (BN * 4);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 2
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 8; ++i)
          *reinterpret_cast<uint4*>(prow + (((c * 8 + i) ^ (lr & 7)) << 4)) =
              make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
      }
    }
    tc_fence_before();
  }

  // ---------------- reduction over the cluster ----------------
  // Every thread of every CTA reaches both cluster barriers, also after a wait that gave up (the
  // result is then meaningless and the status word says so).
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // all partial tiles are in place
  const bool cluster_ok = cluster_num_ctas() == static_cast<uint32_t>(p.split);
  if (!cluster_ok && threadIdx.x == 0 && p.status) atomicOr(p.status, kStatusGemmNoCluster);
  if (cluster_ok) {
    const ReduceCtx<OutT> ctx{p, smem_u32(smem), rank, tm, tn, bz};
    if (p.split == 2)
      reduce_band<BN, KIND, OutT, EPI, 2>(ctx);
    else if (p.split == 4)
      reduce_band<BN, KIND, OutT, EPI, 4>(ctx);
    else
      reduce_band<BN, KIND, OutT, EPI, 8>(ctx);
  }
  cluster_sync_all();  // no CTA leaves (and frees its shared memory) while a peer still reads it

  // ---------------- teardown ----------------
  if (*abort_word != 0) {
    // A wait gave up: give copies that may still be in flight time to land before the shared
    // memory is released, then report.
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {
    }
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, kStatusGemmTimeout);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

void cluster_config(cudaLaunchConfig_t& cfg, cudaLaunchAttribute& attr, int grid, int split, int smem_bytes,
                    cudaStream_t stream) {
  cfg = cudaLaunchConfig_t{};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
  cfg.stream = stream;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = static_cast<unsigned>(split);
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
}

template <int BN, int KIND, typename OutT, int EPI>
int launch_fused(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream) {
  using S = GemmSmem<BN, 1>;
  auto kfn = gemm_splitk_kernel<BN, KIND, OutT, EPI>;
  static bool configured[64] = {};  // per instantiation and device ordinal
  int rc = ensure_dynamic_smem(kfn, S::kDynamic, configured, "cudaFuncSetAttribute(split-K gemm smem)");
  if (rc) return rc;
  const int64_t ctas = static_cast<int64_t>(p.tiles_m) * p.tiles_n * p.batch * p.split;
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr;
  cluster_config(cfg, attr, static_cast<int>(ctas), p.split, S::kDynamic, stream);
  return check_cuda(cudaLaunchKernelEx(&cfg, kfn, ta, tb, p), "gemm_splitk_kernel launch");
}

template <int BN, int KIND, typename OutT>
int launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream) {
  if (p.bias != nullptr) return launch_fused<BN, KIND, OutT, 2>(ta, tb, p, stream);
  if (p.act != 0) return launch_fused<BN, KIND, OutT, 1>(ta, tb, p, stream);
  return launch_fused<BN, KIND, OutT, 0>(ta, tb, p, stream);
}

template <int BN>
int dispatch_dtype(int in_dtype, int out_dtype, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                   cudaStream_t stream) {
  if (in_dtype == B200K_F16 && out_dtype == B200K_F32) return launch_one<BN, kKindF16, float>(ta, tb, p, stream);
  if (in_dtype == B200K_F16 && out_dtype == B200K_F16) return launch_one<BN, kKindF16, __half>(ta, tb, p, stream);
  if (in_dtype == B200K_BF16 && out_dtype == B200K_F32) return launch_one<BN, kKindBF16, float>(ta, tb, p, stream);
  if (in_dtype == B200K_BF16 && out_dtype == B200K_BF16)
    return launch_one<BN, kKindBF16, __nv_bfloat16>(ta, tb, p, stream);
  if (in_dtype == B200K_E4M3 && out_dtype == B200K_BF16)
    return launch_one<BN, kKindE4M3, __nv_bfloat16>(ta, tb, p, stream);
  if (in_dtype == B200K_E4M3 && out_dtype == B200K_F32) return launch_one<BN, kKindE4M3, float>(ta, tb, p, stream);
  return set_error(B200K_ERR_BAD_DTYPE, "gemm (split-K): unsupported dtype pair in=%d out=%d", in_dtype, out_dtype);
}

template <int BN>
int resident_clusters(int split) {
  using S = GemmSmem<BN, 1>;
  // shared memory and block size do not depend on the data types: one instantiation answers for all
  auto kfn = gemm_splitk_kernel<BN, kKindF16, float, 0>;
  static bool configured[64] = {};
  if (ensure_dynamic_smem(kfn, S::kDynamic, configured, "cudaFuncSetAttribute(split-K gemm smem)") != 0) return 0;
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr;
  cluster_config(cfg, attr, split, split, S::kDynamic, nullptr);
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kfn, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return n;
}

}  // namespace

int launch_gemm_splitk(const CUtensorMap& ta, const CUtensorMap& tb, const gemm_detail::GemmParams& p, int bn,
                       int in_dtype, int out_dtype, cudaStream_t stream) {
  if (p.split != 2 && p.split != 4 && p.split != 8)
    return set_error(B200K_ERR_BAD_SHAPE, "gemm (split-K): split must be 2, 4 or 8");
  if (bn == 256) return dispatch_dtype<256>(in_dtype, out_dtype, ta, tb, p, stream);
  return dispatch_dtype<128>(in_dtype, out_dtype, ta, tb, p, stream);
}

int splitk_resident_clusters(int bn, int split) {
  // The CTAs of a cluster share a GPC, so fewer than SMs / split clusters fit.  Asked once per
  // device, tile width and cluster size.
  static int cache[64][2][9] = {};  // 0 = not asked yet, -1 = cannot launch
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || split < 2 || split > 8) return 0;
  int& slot = cache[dev][bn == 256 ? 1 : 0][split];
  if (slot == 0) {
    const int n = bn == 256 ? resident_clusters<256>(split) : resident_clusters<128>(split);
    slot = n > 0 ? n : -1;
  }
  return slot > 0 ? slot : 0;
}

}  // namespace b200k
