// C[M,N] = A[M,K] * B[N,K]^T on sm_100a: TMA-fed shared-memory ring, tcgen05.mma with fp32
// accumulators in tensor memory, persistent CTAs with double-buffered accumulators so the
// epilogue of one tile overlaps the main loop of the next.
//
// Tile shapes.  A 128 x 256 tile needs 96 bytes of operands per tensor-core cycle, more than an
// SM can pull from L2, so large problems use a 256 x 256 tile: two 128-row halves share each B
// stage (64 bytes per cycle) at the price of a single, not double-buffered, accumulator set.
//
// CTA = 6 warps: warp 0 issues TMA loads, warp 1 owns tensor memory and issues the MMAs,
// warps 2..5 drain accumulators (each warp its own 32-lane quarter of tensor memory).
//
// Data layout.  A and B are K-contiguous, so both are "K-major" UMMA operands.  One pipeline
// stage holds a 128 x 128-byte tile of A and a BN x 128-byte tile of B, written by TMA with the
// 128-byte swizzle; each UMMA consumes 32 bytes of K (16 half-precision or 32 fp8 elements), so
// a stage feeds four MMAs whose descriptors advance by 32 bytes inside the swizzle atom.
#include <cstring>

#include "common.cuh"
#include "gemm_common.cuh"
#include "ptx.cuh"

namespace b200k {
namespace {

using namespace gemm_detail;

// GEN = false: both operands K-major (A [M, K], B [N, K]); the issue path is all compile-time
// offsets.  GEN = true (16-bit types only): either operand may be MN-major, chosen at run time
// (p.a_mn, p.b_mn).  An MN-major operand is stored [K, R] with R contiguous; a pipeline stage holds
// it as R / 64 blocks of 64 K-rows x 128 bytes (128-byte swizzle), one TMA box each; the UMMA
// descriptor has LBO = 8 KB between the 64-element blocks, SBO = 1 KB between 8-row groups, and a
// k-step of 16 rows advances 2 KB.  A stage has the same size either way.
template <int BN, int MT, int KIND, typename OutT, bool GEN>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_nt_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const __grid_constant__ CUtensorMap tmap_c, const GemmParams p,
                   const __grid_constant__ PeerMaps peer_maps) {
  using S = GemmSmem<BN, MT>;
  constexpr int kElemsPerStage = (KIND == kKindE4M3) ? 128 : 64;  // K elements in 128 bytes
  constexpr uint32_t kFmt = (KIND == kKindBF16) ? kFmtBF16 : (KIND == kKindF16 ? kFmtF16 : kFmtE4M3);
  constexpr uint32_t kIdesc = make_idesc(kFmt, kFmt, kBM, BN, 0, 0);
  constexpr uint32_t kTmemCols = 2 * BN;
  // MT == 1: two accumulator buffers of BN columns (epilogue overlaps the next tile's main loop);
  // MT == 2: one buffer holding the two 128-row halves side by side.
  constexpr int kAccBufs = MT == 1 ? 2 : 1;
  constexpr int kTileM = MT * kBM;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty = full + S::kStages;
  uint64_t* tfull = empty + S::kStages;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile uint32_t* abort_word = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::kStages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull + a, 1);
      mbar_init(tempty + a, 4);
    }
    *abort_word = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    prefetch_tmap(&tmap_c);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above touched no global memory, so under a programmatic dependent launch it ran
  // while the previous kernel of the stream was still finishing.  From here on operands are read
  // and C is written: wait for that kernel, then let the next one start its own set-up early (it
  // cannot share an SM with a CTA of this grid, and waits here in turn).
  grid_dependency_wait();
  grid_dependency_trigger();

  const int tiles_per_problem = p.tiles_m * p.tiles_n;
  const int num_tiles = tiles_per_problem * p.batch;  // tile t: problem t / tiles_per_problem

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        const int bz = t / tiles_per_problem;
        tile_coords(t - bz * tiles_per_problem, p.tiles_m, p.tiles_n, tm, tn);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(empty + stage, phase ^ 1, abort_word)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * S::kStageBytes;
          mbar_arrive_expect_tx(full + stage, S::kStageBytes);
          if (GEN && p.a_mn) {
#pragma unroll
            for (int b = 0; b < kTileM / 64; ++b)
              tma_load_3d(sa + b * 8192, &tmap_a, full + stage, tm * kTileM + b * 64, kb * kElemsPerStage, bz);
          } else {
            tma_load_3d(sa, &tmap_a, full + stage, kb * kElemsPerStage, tm * kTileM, bz);
          }
          if (GEN && p.b_mn) {
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
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      // Descriptors: constant high word; low word = precomputed stage base + compile-time offset, so
      // the scalar issue path stays a few instructions per MMA.
      const uint32_t hi = static_cast<uint32_t>(make_desc_kmajor_sw128(0) >> 32);
      const uint32_t lo0 = static_cast<uint32_t>(make_desc_kmajor_sw128(smem_u32(smem)));
      auto desc = [](uint32_t lo, uint32_t h) { return (static_cast<uint64_t>(h) << 32) | lo; };
      // generic kernel: per-operand high word, k-step and instruction descriptor chosen once
      // (the block stride of an MN-major operand, LBO, sits in the LOW word next to the address)
      const uint32_t hi_mn = static_cast<uint32_t>(make_desc_mnmajor_sw128(0, 8192) >> 32);
      const uint32_t lo0_mn = static_cast<uint32_t>(make_desc_mnmajor_sw128(smem_u32(smem), 8192));
      const uint32_t lo0_a = (GEN && p.a_mn) ? lo0_mn : lo0;
      const uint32_t lo0_b = (GEN && p.b_mn) ? lo0_mn : lo0;
      const uint32_t hi_a = (GEN && p.a_mn) ? hi_mn : hi;
      const uint32_t hi_b = (GEN && p.b_mn) ? hi_mn : hi;
      const uint32_t step_a = (GEN && p.a_mn) ? (2048u >> 4) : 2u;
      const uint32_t step_b = (GEN && p.b_mn) ? (2048u >> 4) : 2u;
      const uint32_t idesc = GEN ? (kIdesc | (p.a_mn ? 1u << 15 : 0u) | (p.b_mn ? 1u << 16 : 0u)) : kIdesc;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const int acc = it % kAccBufs;
        const uint32_t acc_phase = (it / kAccBufs) & 1;
        if (!mbar_wait(tempty + acc, acc_phase ^ 1, abort_word)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (MT == 1 ? acc * BN : 0);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(full + stage, phase, abort_word)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_lo = (GEN ? lo0_a : lo0) + stage * (S::kStageBytes >> 4);
          const uint32_t b_lo = (GEN ? lo0_b + stage * (S::kStageBytes >> 4) : a_lo) + (S::kABytes >> 4);
          const uint32_t accum0 = kb != 0 ? 1u : 0u;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t accum = k == 0 ? accum0 : 1u;
#pragma unroll
            for (int h = 0; h < MT; ++h) {
              if constexpr (GEN) {
                const uint64_t a_desc = desc(a_lo + h * ((kBM * kBKBytes) >> 4) + step_a * k, hi_a);
                const uint64_t b_desc = desc(b_lo + step_b * k, hi_b);
                umma_f16_ss(d_tmem + h * BN, a_desc, b_desc, idesc, accum);
              } else {
                const uint64_t a_desc = desc(a_lo + h * ((kBM * kBKBytes) >> 4) + 2 * k, hi);
                const uint64_t b_desc = desc(b_lo + 2 * k, hi);
                if constexpr (KIND == kKindE4M3)
                  umma_f8_ss(d_tmem + h * BN, a_desc, b_desc, kIdesc, accum);
                else
                  umma_f16_ss(d_tmem + h * BN, a_desc, b_desc, kIdesc, accum);
              }
            }
          }
          umma_commit(empty + stage);  // frees the stage once these MMAs have read it
          if (++stage == S::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(tfull + acc);  // accumulator complete
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue warps ----------------
    const int quarter = warp & 3;
    float scale = 1.0f;
    if constexpr (KIND == kKindE4M3) {
      const float sa = p.scale_a ? *p.scale_a : 1.0f;
      const float sb = p.scale_b ? *p.scale_b : 1.0f;
      scale = sa * sb;
    }
    const bool fused = p.bias != nullptr || p.act != 0;  // uniform over the grid
    OutT* cbase = reinterpret_cast<OutT*>(p.c);
    uint8_t* staging = smem + S::kStagingOffset + (warp - 2) * (2 * 4096);
    uint32_t stg_count = 0;
    int it = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
      int tm, tn;
      const int bz = t / tiles_per_problem;
      tile_coords(t - bz * tiles_per_problem, p.tiles_m, p.tiles_n, tm, tn);
      const int acc = it % kAccBufs;
      const uint32_t acc_phase = (it / kAccBufs) & 1;
      bool ok = mbar_wait(tfull + acc, acc_phase, abort_word);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int h = 0; h < MT; ++h) {
        const int row0 = tm * kTileM + h * kBM + quarter * 32;
        const int row = row0 + lane;
        const uint32_t taddr =
            tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + (MT == 1 ? acc * BN : h * BN);
        if (p.num_peers > 0 && !p.peer_tma) {
          // Column shard written straight into every rank's full C (own copy included): registers ->
          // swizzled staging buffer -> each store instruction writes four full 128-byte row segments
          // to one peer, so the NVLink traffic is made of whole lines.
          constexpr int kCols = 128 / static_cast<int>(sizeof(OutT));
#pragma unroll 1
          for (int c = 0; c < BN / kCols; ++c) {
            uint8_t* buf = staging;
            uint4 v[8];
            if constexpr (sizeof(OutT) == 4) {
              uint32_t r[32];
              tmem_ld_32x32b_x32(taddr + c * 32, r);
              tmem_wait_ld();
              float sc = scale;
              if (fused) {
                fused_epilogue<32>(r, scale, p.bias, p.bias_dtype, p.act, tn * BN + c * 32, p.n);
                sc = 1.f;
              }
#pragma unroll
              for (int i = 0; i < 8; ++i)
                v[i] = make_uint4(__float_as_uint(__uint_as_float(r[4 * i]) * sc),
                                  __float_as_uint(__uint_as_float(r[4 * i + 1]) * sc),
                                  __float_as_uint(__uint_as_float(r[4 * i + 2]) * sc),
                                  __float_as_uint(__uint_as_float(r[4 * i + 3]) * sc));
            } else {
              uint32_t r[64];
              tmem_ld_32x32b_x64(taddr + c * 64, r);
              tmem_wait_ld();
              float sc = scale;
              if (fused) {
                fused_epilogue<64>(r, scale, p.bias, p.bias_dtype, p.act, tn * BN + c * 64, p.n);
                sc = 1.f;
              }
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                union {
                  uint4 u;
                  OutT e[8];
                } pk;
#pragma unroll
                for (int j = 0; j < 8; ++j) pk.e[j] = to_out<OutT>(__uint_as_float(r[8 * i + j]) * sc);
                v[i] = pk.u;
              }
            }
            __syncwarp();  // previous chunk's reads of the staging buffer are done
#pragma unroll
            for (int i = 0; i < 8; ++i)
              *reinterpret_cast<uint4*>(buf + lane * 128 + ((i ^ (lane & 7)) << 4)) = v[i];
            __syncwarp();
            const int col = tn * BN + c * kCols;  // column inside the shard
            const int chunk = lane & 7;
            const int ecol = col + chunk * (16 / static_cast<int>(sizeof(OutT)));
#pragma unroll
            for (int rr = 0; rr < 8; ++rr) {
              const int lr = rr * 4 + (lane >> 3);
              const int grow = row0 + lr;
              const uint4 val = *reinterpret_cast<const uint4*>(buf + lr * 128 + ((chunk ^ (lr & 7)) << 4));
              if (grow < p.m && ecol < p.n) {
                const int64_t off = (static_cast<int64_t>(grow) * p.peer_ldc + p.peer_col0 + ecol) *
                                    static_cast<int64_t>(sizeof(OutT));
                if (p.peer_mc) {
                  // one store to the multicast address: the switch writes every rank's copy
                  asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(
                                   reinterpret_cast<uint8_t*>(p.peer_mc) + off),
                               "f"(__uint_as_float(val.x)), "f"(__uint_as_float(val.y)), "f"(__uint_as_float(val.z)),
                               "f"(__uint_as_float(val.w))
                               : "memory");
                } else {
                  int pe = p.peer_first;
                  for (int i = 0; i < p.num_peers; ++i) {
                    *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.peers[pe]) + off) = val;
                    pe = pe + 1 == p.num_peers ? 0 : pe + 1;
                  }
                }
              }
            }
          }
        } else if (p.tma_store_ok || p.peer_tma) {
          // 128 bytes of each of this warp's 32 rows per step: registers -> swizzled staging
          // buffer -> one TMA store (full 128-byte lines, clipped at the matrix edge by the
          // tensor map).  Two buffers per warp; a buffer is reused once its store has been read.
          // Fused all-gather: the same piece goes out once per rank, through that rank's map, as
          // bulk stores to peer-mapped memory; the copy engine of the SM moves the data while the
          // warp prepares the next piece.
          constexpr int kCols = 128 / static_cast<int>(sizeof(OutT));
#pragma unroll 1
          for (int c = 0; c < BN / kCols; ++c) {
            uint8_t* buf = staging + (stg_count & 1) * 4096;
            if (lane == 0) tma_store_wait_read<1>();
            __syncwarp();
            uint4 v[8];
            if constexpr (sizeof(OutT) == 4) {
              uint32_t r[32];
              tmem_ld_32x32b_x32(taddr + c * 32, r);
              tmem_wait_ld();
              float sc = scale;
              if (fused) {
                fused_epilogue<32>(r, scale, p.bias, p.bias_dtype, p.act, tn * BN + c * 32, p.n);
                sc = 1.f;
              }
#pragma unroll
              for (int i = 0; i < 8; ++i)
                v[i] = make_uint4(__float_as_uint(__uint_as_float(r[4 * i]) * sc),
                                  __float_as_uint(__uint_as_float(r[4 * i + 1]) * sc),
                                  __float_as_uint(__uint_as_float(r[4 * i + 2]) * sc),
                                  __float_as_uint(__uint_as_float(r[4 * i + 3]) * sc));
            } else {
              uint32_t r[64];
              tmem_ld_32x32b_x64(taddr + c * 64, r);
              tmem_wait_ld();
              float sc = scale;
              if (fused) {
                fused_epilogue<64>(r, scale, p.bias, p.bias_dtype, p.act, tn * BN + c * 64, p.n);
                sc = 1.f;
              }
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                union {
                  uint4 u;
                  OutT e[8];
                } pk;
#pragma unroll
                for (int j = 0; j < 8; ++j) pk.e[j] = to_out<OutT>(__uint_as_float(r[8 * i + j]) * sc);
                v[i] = pk.u;
              }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
              *reinterpret_cast<uint4*>(buf + lane * 128 + ((i ^ (lane & 7)) << 4)) = v[i];
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (p.num_peers > 0) {
                int pe = p.peer_first;
                for (int i = 0; i < p.num_peers; ++i) {
                  tma_store_2d(&peer_maps.m[pe], buf, tn * BN + c * kCols, row0);
                  pe = pe + 1 == p.num_peers ? 0 : pe + 1;
                }
              } else {
                tma_store_3d(&tmap_c, buf, tn * BN + c * kCols, row0, bz);
              }
              tma_store_commit();
            }
            ++stg_count;
          }
        } else {
#pragma unroll 2
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + c * 32, r);
            tmem_wait_ld();
            const int col = tn * BN + c * 32;
            float sc = scale;
            if (fused) {
              fused_epilogue<32>(r, scale, p.bias, p.bias_dtype, p.act, col, p.n);
              sc = 1.f;
            }
            if (row < p.m && col < p.n) {
              store_chunk<OutT>(cbase + bz * p.c_batch_stride + static_cast<int64_t>(row) * p.ldc + col, r, sc, p.n - col,
                                p.vec_store_ok != 0);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty + acc);
    }
    if (lane == 0) tma_store_wait<0>();  // staging memory must outlive the last stores
    __syncwarp();
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
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

template <int BN, int MT, int KIND, typename OutT, bool GEN = false>
int launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
               const PeerMaps& pm, int grid, cudaStream_t stream) {
  using S = GemmSmem<BN, MT>;
  auto kfn = gemm_nt_kernel<BN, MT, KIND, OutT, GEN>;
  static bool configured[64] = {};  // per instantiation and device ordinal
  int rc = ensure_dynamic_smem(kfn, S::kDynamic, configured, "cudaFuncSetAttribute(gemm smem)");
  if (rc) return rc;
  // Programmatic dependent launch: barrier set-up and the tensor-memory allocation of this kernel
  // overlap the tail of whatever runs before it in the stream (see grid_dependency_wait in the kernel).
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = S::kDynamic;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return check_cuda(cudaLaunchKernelEx(&cfg, kfn, ta, tb, tc, p, pm), "gemm_nt_kernel launch");
}

template <int BN, int MT>
int dispatch_dtype(int in_dtype, int out_dtype, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                   const GemmParams& p, const PeerMaps& pm, int grid, cudaStream_t stream) {
  if (p.a_mn || p.b_mn) {  // generic operand storage: 16-bit types
    if (in_dtype == B200K_F16 && out_dtype == B200K_F32)
      return launch_one<BN, MT, kKindF16, float, true>(ta, tb, tc, p, pm, grid, stream);
    if (in_dtype == B200K_F16 && out_dtype == B200K_F16)
      return launch_one<BN, MT, kKindF16, __half, true>(ta, tb, tc, p, pm, grid, stream);
    if (in_dtype == B200K_BF16 && out_dtype == B200K_F32)
      return launch_one<BN, MT, kKindBF16, float, true>(ta, tb, tc, p, pm, grid, stream);
    if (in_dtype == B200K_BF16 && out_dtype == B200K_BF16)
      return launch_one<BN, MT, kKindBF16, __nv_bfloat16, true>(ta, tb, tc, p, pm, grid, stream);
    return set_error(B200K_ERR_BAD_DTYPE, "gemm: operands stored [K, M] / [K, N] need F16 or BF16 (in=%d out=%d)",
                     in_dtype, out_dtype);
  }
  if (in_dtype == B200K_F16 && out_dtype == B200K_F32)
    return launch_one<BN, MT, kKindF16, float>(ta, tb, tc, p, pm, grid, stream);
  if (in_dtype == B200K_F16 && out_dtype == B200K_F16)
    return launch_one<BN, MT, kKindF16, __half>(ta, tb, tc, p, pm, grid, stream);
  if (in_dtype == B200K_BF16 && out_dtype == B200K_F32)
    return launch_one<BN, MT, kKindBF16, float>(ta, tb, tc, p, pm, grid, stream);
  if (in_dtype == B200K_BF16 && out_dtype == B200K_BF16)
    return launch_one<BN, MT, kKindBF16, __nv_bfloat16>(ta, tb, tc, p, pm, grid, stream);
  if (in_dtype == B200K_E4M3 && out_dtype == B200K_BF16)
    return launch_one<BN, MT, kKindE4M3, __nv_bfloat16>(ta, tb, tc, p, pm, grid, stream);
  if (in_dtype == B200K_E4M3 && out_dtype == B200K_F32)
    return launch_one<BN, MT, kKindE4M3, float>(ta, tb, tc, p, pm, grid, stream);
  return set_error(B200K_ERR_BAD_DTYPE, "gemm_nt: unsupported dtype pair in=%d out=%d", in_dtype, out_dtype);
}

}  // namespace

namespace {
struct PeerTargets {
  int num = 0;
  int first = 0;
  void* c[8] = {};
  void* mc = nullptr;
  bool plain = false;  // 16-byte stores from the epilogue warps instead of bulk tensor stores
  int64_t ldc = 0;
  int64_t col0 = 0;
};
int launch_gemm_impl(const b200k_gemm_args& a, const PeerTargets& peers, cudaStream_t stream);
}  // namespace

int launch_gemm_nt(const b200k_gemm_args& a, cudaStream_t stream) {
  if (!a.c) return set_error(B200K_ERR_NULL, "gemm_nt: a, b and c must be non-NULL");
  return launch_gemm_impl(a, PeerTargets{}, stream);
}

int launch_gemm_nt_allgather(const b200k_gemm_allgather_args& g, cudaStream_t stream) {
  if (g.num_peers < 1 || g.num_peers > 8)
    return set_error(B200K_ERR_BAD_SHAPE, "gemm_nt_allgather: num_peers must be in [1, 8]");
  const size_t out_es = dtype_size(g.gemm.out_dtype);
  if (out_es == 0) return set_error(B200K_ERR_BAD_DTYPE, "gemm_nt_allgather: bad out dtype");
  if (g.col_offset < 0 || g.peer_ldc < g.col_offset + g.gemm.n)
    return set_error(B200K_ERR_BAD_SHAPE, "gemm_nt_allgather: column shard does not fit in the row pitch of the full matrix");
  if ((g.peer_ldc * out_es) % 16 != 0 || (g.col_offset * out_es) % 16 != 0 || (g.gemm.n * out_es) % 16 != 0)
    return set_error(B200K_ERR_BAD_ALIGN, "gemm_nt_allgather: row pitch, column offset and shard width must be multiples of 16 bytes");
  if (g.self_index < 0 || g.self_index >= g.num_peers)
    return set_error(B200K_ERR_BAD_SHAPE, "gemm_nt_allgather: self_index must be in [0, num_peers)");
  if (reinterpret_cast<uintptr_t>(g.multicast_c) & 15)
    return set_error(B200K_ERR_BAD_ALIGN, "gemm_nt_allgather: multicast_c must be 16-byte aligned");
  PeerTargets t;
  t.num = g.num_peers;
  t.first = (g.self_index + 1) % g.num_peers;
  t.mc = g.multicast_c;
  t.plain = g.plain_stores != 0;
  t.ldc = g.peer_ldc;
  t.col0 = g.col_offset;
  for (int i = 0; i < g.num_peers; ++i) {
    if (!g.peer_c[i] || (reinterpret_cast<uintptr_t>(g.peer_c[i]) & 15))
      return set_error(B200K_ERR_BAD_ALIGN, "gemm_nt_allgather: every peer_c must be non-NULL and 16-byte aligned");
    t.c[i] = g.peer_c[i];
  }
  return launch_gemm_impl(g.gemm, t, stream);
}

namespace {
int launch_gemm_impl(const b200k_gemm_args& a, const PeerTargets& peers, cudaStream_t stream) {
  if (!a.a || !a.b) return set_error(B200K_ERR_NULL, "gemm_nt: a, b and c must be non-NULL");
  if (a.m <= 0 || a.n <= 0 || a.k <= 0 || a.m > INT32_MAX || a.n > INT32_MAX || a.k > INT32_MAX)
    return set_error(B200K_ERR_BAD_SHAPE, "gemm_nt: m, n, k must be in [1, 2^31)");
  const size_t in_es = dtype_size(a.in_dtype);
  const size_t out_es = dtype_size(a.out_dtype);
  if (in_es == 0 || out_es == 0 || a.in_dtype == B200K_F32)
    return set_error(B200K_ERR_BAD_DTYPE, "gemm_nt: unsupported dtype in=%d out=%d", a.in_dtype, a.out_dtype);
  const bool a_mn = a.a_km != 0, b_mn = a.b_kn != 0;
  const int64_t batch = a.batch > 1 ? a.batch : 1;
  if (a.batch < 0 || batch > 65535) return set_error(B200K_ERR_BAD_SHAPE, "gemm: batch must be in [0, 65535]");
  if (batch > 1) {
    if (peers.num > 0) return set_error(B200K_ERR_BAD_SHAPE, "gemm_nt_allgather: batched problems are not supported");
    if (a.a_batch_stride <= 0 || a.b_batch_stride <= 0 || a.c_batch_stride <= 0)
      return set_error(B200K_ERR_BAD_SHAPE, "gemm: batch strides must be positive");
    if ((a.a_batch_stride * in_es) % 16 != 0 || (a.b_batch_stride * in_es) % 16 != 0)
      return set_error(B200K_ERR_BAD_ALIGN, "gemm: the A / B batch strides must be multiples of 16 bytes");
  }
  if ((a_mn || b_mn) && a.in_dtype == B200K_E4M3)
    return set_error(B200K_ERR_BAD_DTYPE, "gemm: a_km / b_kn operand storage is for F16 / BF16 only");
  if (a.lda < (a_mn ? a.m : a.k) || a.ldb < (b_mn ? a.n : a.k) || (peers.num == 0 && a.ldc < a.n))
    return set_error(B200K_ERR_BAD_SHAPE, "gemm_nt: leading dimensions smaller than the row length");
  if ((reinterpret_cast<uintptr_t>(a.a) & 15) || (reinterpret_cast<uintptr_t>(a.b) & 15) ||
      (a.lda * in_es) % 16 != 0 || (a.ldb * in_es) % 16 != 0)
    return set_error(B200K_ERR_BAD_ALIGN, "gemm_nt: A/B base and row stride must be multiples of 16 bytes");
  if (peers.num == 0 && reinterpret_cast<uintptr_t>(a.c) % out_es != 0)
    return set_error(B200K_ERR_BAD_ALIGN, "gemm_nt: C is not aligned to its element size");
  if (a.activation < B200K_ACT_NONE || a.activation > B200K_ACT_SILU)
    return set_error(B200K_ERR_BAD_SHAPE, "gemm_nt: unknown activation %d", a.activation);
  if (a.bias && a.bias_dtype != B200K_F32 && a.bias_dtype != B200K_F16 && a.bias_dtype != B200K_BF16)
    return set_error(B200K_ERR_BAD_DTYPE, "gemm_nt: bias must be F32, F16 or BF16");
  if (a.tile_n != 0 && a.tile_n != 128 && a.tile_n != 256)
    return set_error(B200K_ERR_BAD_SHAPE, "gemm_nt: tile_n must be 0, 128 or 256");
  if (a.tile_m != 0 && a.tile_m != 128 && a.tile_m != 256)
    return set_error(B200K_ERR_BAD_SHAPE, "gemm_nt: tile_m must be 0, 128 or 256");
  int rc = ensure_sm100();
  if (rc) return rc;

  const int sms = num_sms();
  // Tile choice: estimated time = waves * tile area / efficiency.  The efficiencies are the
  // measured throughputs of the three shapes on a many-wave problem (f16 8192^3: 1039 / 1375 /
  // 1555 TFLOP/s), relative to one another: a 128-row tile is limited by operand delivery (a
  // 128 x 256 tile needs 96 bytes per tensor-core cycle, a 128 x 128 tile 128), a 256 x 256 tile
  // is not.  (An earlier model with 0.67 / 0.67 / 0.72 chose 128 x 128 tiles for 4096^3, which
  // run at 983 TFLOP/s where 256 x 256 tiles reach 1398.)
  auto cost = [&](int bm, int bn) {
    const int64_t tiles = ((a.m + bm - 1) / bm) * ((a.n + bn - 1) / bn) * batch;
    const int64_t waves = (tiles + sms - 1) / sms;
    const double eff = bm == 256 ? 0.93 : (bn == 256 ? 0.83 : 0.62);
    return static_cast<double>(waves) * bm * bn / eff;
  };
  int bm = a.tile_m, bn = a.tile_n;
  if (bm == 256 && bn == 0) bn = 256;
  if (bn == 0) {
    double best = cost(128, 128);
    bn = 128;
    int best_bm = 128;
    if (a.n > 128 && cost(128, 256) <= best) {
      best = cost(128, 256);
      bn = 256;
    }
    if (bm != 128 && a.n > 128 && a.m > 128 && cost(256, 256) < best) {
      bn = 256;
      best_bm = 256;
    }
    if (bm == 0) bm = best_bm;
  }
  if (bm == 0) bm = 128;
  if (bm == 256 && bn != 256)
    return set_error(B200K_ERR_BAD_SHAPE, "gemm_nt: tile_m 256 requires tile_n 256");
  // Fused all-gather: every tile is also written to the other ranks from the epilogue.  When
  // sending the shard takes longer than computing it (measured on 4 / 8 GPUs: 104 / 56 us of math,
  // about 110 / 190 us of stores), 128-row tiles with their two accumulator sets let the stores of
  // one tile run under the main loop of the next and start after a quarter of the time of a
  // 256 x 256 tile (4 GPUs: 214 us per step against 222).
  if (peers.num > 1 && a.tile_m == 0 && a.tile_n == 0 && a.n > 128) {
    const double send_us = static_cast<double>(peers.num - 1) * a.m * a.n * out_es / 600e3;
    const double peak_tflops = a.in_dtype == B200K_E4M3 ? 3000.0 : 1500.0;
    const double math_us = 2.0 * a.m * a.n * a.k / (peak_tflops * 1e6);
    if (send_us > math_us) {
      bm = 128;
      bn = 256;
    }
  }
  const int k_per_stage = a.in_dtype == B200K_E4M3 ? 128 : 64;
  const int64_t num_kb = (a.k + k_per_stage - 1) / k_per_stage;

  // Split-K over a cluster (128-row tiles, gemm_splitk_sm100.cu): worth it when the whole tiles
  // leave most SMs idle and K is long.  Estimated cycles = waves * k-blocks per CTA * cycles per
  // k-block (measured with operands from HBM: 568 / 750 / 1250 for 128x128 / 128x256 / 256x256
  // tiles) + the part of the epilogue nothing overlaps; a split adds the cluster launch, two
  // cluster barriers, the partial-tile write and the reduction through peer shared memory
  // (measured: about 4 to 6 us more than an un-split launch of the same k-blocks).
  if (a.split_k != 0 && a.split_k != 1 && a.split_k != 2 && a.split_k != 4 && a.split_k != 8)
    return set_error(B200K_ERR_BAD_SHAPE, "gemm: split_k must be 0, 1, 2, 4 or 8");
  int split = 1;
  if (a.split_k > 1) {
    if (peers.num > 0) return set_error(B200K_ERR_BAD_SHAPE, "gemm_nt_allgather: split_k is not supported");
    if (a.tile_m == 256) return set_error(B200K_ERR_BAD_SHAPE, "gemm: split_k needs 128-row tiles (tile_m 0 or 128)");
    if (num_kb < a.split_k) return set_error(B200K_ERR_BAD_SHAPE, "gemm: split_k exceeds the number of k-blocks");
    bm = 128;
    split = a.split_k;
    if (splitk_resident_clusters(bn, split) == 0)
      return set_error(B200K_ERR_UNSUPPORTED_ARCH, "gemm: clusters of %d CTAs cannot be launched", split);
  } else if (a.split_k == 0 && peers.num == 0) {
    auto cycles_kb = [](int tm, int tn) { return tm == 256 ? 1250.0 : (tn == 256 ? 750.0 : 568.0); };
    auto split_cost = [](int tn, int s) { return tn == 256 ? 10000.0 + 2000.0 * s : 8000.0 + 1200.0 * s; };
    auto tail = [](int tm, int tn) { return tm == 256 ? 6000.0 : (tn == 256 ? 3000.0 : 1500.0); };
    const int64_t tiles0 = ((a.m + bm - 1) / bm) * ((a.n + bn - 1) / bn) * batch;
    const int64_t waves0 = (tiles0 + sms - 1) / sms;
    double best = static_cast<double>(waves0) * num_kb * cycles_kb(bm, bn) + tail(bm, bn);
    best *= 0.9;  // a split has to win clearly
    if (tiles0 * 2 <= sms && a.tile_m != 256) {
      for (int tn = 128; tn <= 256; tn += 128) {
        if (a.tile_n != 0 && a.tile_n != tn) continue;
        if (tn == 256 && a.n <= 128) continue;
        const int64_t tiles = ((a.m + 127) / 128) * ((a.n + tn - 1) / tn) * batch;
        for (int s = 2; s <= 8; s *= 2) {
          if (num_kb < 4 * s) continue;  // at least four k-blocks per slice
          const int resident = splitk_resident_clusters(tn, s);
          if (resident == 0) continue;
          const int64_t waves = (tiles + resident - 1) / resident;
          const int64_t per = (num_kb + s - 1) / s;
          const double t = static_cast<double>(waves) * per * cycles_kb(128, tn) + tail(128, tn) + split_cost(tn, s);
          if (t < best) {
            best = t;
            split = s;
            bm = 128;
            bn = tn;
          }
        }
      }
    }
  }
  const int tiles_m = static_cast<int>((a.m + bm - 1) / bm);
  const int tiles_n = static_cast<int>((a.n + bn - 1) / bn);

  CUtensorMap ta, tb;
  {
    // K-major: rows of the stored matrix are rows of the tile; MN-major ([K, M] storage): one box
    // is 64 contiguous M-elements x 64 K-rows
    uint64_t dims[3] = {static_cast<uint64_t>(a_mn ? a.m : a.k), static_cast<uint64_t>(a_mn ? a.k : a.m),
                        static_cast<uint64_t>(batch)};
    uint64_t strides[2] = {static_cast<uint64_t>(a.lda) * in_es,
                           static_cast<uint64_t>(batch > 1 ? a.a_batch_stride : a.lda) * in_es};
    uint32_t box[3] = {static_cast<uint32_t>(a_mn ? 64 : k_per_stage), static_cast<uint32_t>(a_mn ? 64 : bm), 1u};
    rc = encode_tmap(&ta, a.in_dtype, 3, const_cast<void*>(a.a), dims, strides, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[3] = {static_cast<uint64_t>(b_mn ? a.n : a.k), static_cast<uint64_t>(b_mn ? a.k : a.n),
                        static_cast<uint64_t>(batch)};
    uint64_t strides[2] = {static_cast<uint64_t>(a.ldb) * in_es,
                           static_cast<uint64_t>(batch > 1 ? a.b_batch_stride : a.ldb) * in_es};
    uint32_t box[3] = {static_cast<uint32_t>(b_mn ? 64 : k_per_stage), static_cast<uint32_t>(b_mn ? 64 : bn), 1u};
    rc = encode_tmap(&tb, a.in_dtype, 3, const_cast<void*>(a.b), dims, strides, box);
    if (rc) return rc;
  }

  GemmParams p;
  p.c = a.c;
  p.scale_a = a.scale_a;
  p.scale_b = a.scale_b;
  p.status = a.status;
  p.bias = a.bias;
  p.bias_dtype = a.bias_dtype;
  p.act = a.activation;
  p.a_mn = a_mn ? 1 : 0;
  p.b_mn = b_mn ? 1 : 0;
  p.ldc = a.ldc;
  p.m = static_cast<int32_t>(a.m);
  p.n = static_cast<int32_t>(a.n);
  p.tiles_m = tiles_m;
  p.tiles_n = tiles_n;
  p.num_kb = static_cast<int32_t>(num_kb);
  p.kb_per_split = static_cast<int32_t>((num_kb + split - 1) / split);
  // every slice must hold at least one k-block (an empty one would leave an accumulator unwritten)
  while (split > 1 && static_cast<int64_t>(p.kb_per_split) * (split - 1) >= num_kb) {
    split /= 2;
    p.kb_per_split = static_cast<int32_t>((num_kb + split - 1) / split);
  }
  p.split = split;
  p.batch = static_cast<int32_t>(batch);
  p.c_batch_stride = batch > 1 ? a.c_batch_stride : 0;
  p.vec_store_ok = ((reinterpret_cast<uintptr_t>(a.c) & 15) == 0 && (a.ldc * out_es) % 16 == 0 &&
                    (p.c_batch_stride * out_es) % 16 == 0) ? 1 : 0;
  p.num_peers = peers.num;
  p.peer_first = peers.first;
  p.peer_mc = peers.mc;
  p.peer_ldc = peers.ldc;
  p.peer_col0 = peers.col0;
  for (int i = 0; i < 8; ++i) p.peers[i] = peers.c[i];
  if (peers.num > 0) p.vec_store_ok = 0;

  p.tma_store_ok = p.vec_store_ok;
  CUtensorMap tc;
  memset(&tc, 0, sizeof(tc));
  if (p.tma_store_ok) {
    uint64_t dims[3] = {static_cast<uint64_t>(a.n), static_cast<uint64_t>(a.m), static_cast<uint64_t>(batch)};
    uint64_t strides[2] = {static_cast<uint64_t>(a.ldc) * out_es,
                           static_cast<uint64_t>(batch > 1 ? a.c_batch_stride : a.ldc) * out_es};
    uint32_t box[3] = {static_cast<uint32_t>(128 / out_es), 32u, 1u};
    rc = encode_tmap(&tc, a.out_dtype, 3, a.c, dims, strides, box);
    if (rc) return rc;
  }
  // Fused all-gather by bulk tensor stores: one map per rank over this rank's columns of that
  // rank's matrix (validated above: bases, column offset and row pitch are multiples of 16 bytes).
  static const PeerMaps kNoPeerMaps = {};
  PeerMaps peer_maps;
  p.peer_tma = (peers.num > 0 && peers.mc == nullptr && !peers.plain) ? 1 : 0;
  if (p.peer_tma) {
    memset(&peer_maps, 0, sizeof(peer_maps));
    for (int i = 0; i < peers.num; ++i) {
      uint64_t dims[2] = {static_cast<uint64_t>(a.n), static_cast<uint64_t>(a.m)};
      uint64_t strides[1] = {static_cast<uint64_t>(peers.ldc) * out_es};
      uint32_t box[2] = {static_cast<uint32_t>(128 / out_es), 32u};
      void* base = static_cast<uint8_t*>(peers.c[i]) + peers.col0 * static_cast<int64_t>(out_es);
      rc = encode_tmap(&peer_maps.m[i], a.out_dtype, 2, base, dims, strides, box);
      if (rc) return rc;
    }
  }
  const PeerMaps& pm = p.peer_tma ? peer_maps : kNoPeerMaps;
  const int64_t num_tiles = static_cast<int64_t>(tiles_m) * tiles_n * batch;
  if (num_tiles > INT32_MAX) return set_error(B200K_ERR_BAD_SHAPE, "gemm: too many tiles");
  if (split > 1) {
    if (num_tiles * split > INT32_MAX) return set_error(B200K_ERR_BAD_SHAPE, "gemm: too many tiles");
    return launch_gemm_splitk(ta, tb, p, bn, a.in_dtype, a.out_dtype, stream);
  }
  const int grid = static_cast<int>(num_tiles < sms ? num_tiles : sms);
  if (bm == 256) return dispatch_dtype<256, 2>(a.in_dtype, a.out_dtype, ta, tb, tc, p, pm, grid, stream);
  if (bn == 256) return dispatch_dtype<256, 1>(a.in_dtype, a.out_dtype, ta, tb, tc, p, pm, grid, stream);
  return dispatch_dtype<128, 1>(a.in_dtype, a.out_dtype, ta, tb, tc, p, pm, grid, stream);
}
}  // namespace

}  // namespace b200k
