// Pieces shared by the GEMM kernels (the persistent whole-tile kernel and the split-K cluster
// kernel): tile constants, the kernel parameter block, the shared-memory layout of the operand
// ring, tile rasterisation and the epilogue helpers.
#pragma once
#include "common.cuh"
#include "ptx.cuh"

namespace b200k {
namespace gemm_detail {

constexpr int kBM = 128;
constexpr int kBKBytes = 128;
constexpr int kGemmThreads = 192;
constexpr int kGroupM = 16;  // m-tiles per rasterisation group (keeps one wave's operands L2-resident)

enum GemmKind : int { kKindF16 = 0, kKindBF16 = 1, kKindE4M3 = 2 };

struct GemmParams {
  void* c;
  const float* scale_a;
  const float* scale_b;
  int32_t* status;
  int64_t ldc;
  int32_t m, n;
  int32_t tiles_m, tiles_n, num_kb;  // tiles_m counts MT * 128-row tiles
  int32_t batch;                     // independent problems (tensor maps are 3-D: [batch][rows][k])
  int32_t split;                     // split-K kernel only: CTAs per tile (= cluster size) ...
  int32_t kb_per_split;              // ... each summing this many consecutive k-blocks
  int64_t c_batch_stride;            // elements between the C matrices of consecutive problems
  // Optional fused epilogue: y = act(acc * scale + bias[col]); bias == nullptr and act == 0 leave
  // the plain path untouched.
  const void* bias;
  int32_t bias_dtype;  // B200K_F32 | B200K_F16 | B200K_BF16
  int32_t act;         // B200K_ACT_*
  // Operand storage (generic kernel only): a_mn = A is stored [K, M] (M contiguous), b_mn = B is
  // stored [K, N] (N contiguous); 0 = the contraction dimension K is the contiguous one.
  int32_t a_mn, b_mn;
  int32_t vec_store_ok;
  int32_t tma_store_ok;  // C is 16-byte aligned with a 16-byte-multiple row pitch: epilogue uses TMA stores
  // Fused all-gather of a column shard: when num_peers > 0 every output tile is written with plain
  // 16-byte stores into each peer's full matrix (peer-mapped memory) at column peer_col0.
  int32_t num_peers;
  int32_t peer_first;  // index of the first peer written (the rank after this one); own copy last
  int64_t peer_ldc;
  int64_t peer_col0;
  void* peers[8];
  void* peer_mc;  // NVSwitch multicast address of the matrix, or nullptr
  int32_t peer_tma;  // the pieces go out as bulk tensor stores through PeerMaps (one per rank)
};

// Tensor maps over this rank's column shard inside every rank's full matrix (fused all-gather):
// map i covers columns [col0, col0 + n) of rank i's matrix, so a store is clipped at the shard's edge.
struct PeerMaps {
  CUtensorMap m[8];
};

template <int BN, int MT>
struct GemmSmem {
  static constexpr int kStages = MT == 2 ? 3 : (BN == 256 ? 4 : 6);
  static constexpr int kABytes = MT * kBM * kBKBytes;
  static constexpr int kBBytes = BN * kBKBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // epilogue staging: per epilogue warp two 32-row x 128-byte buffers (TMA store source)
  static constexpr int kStagingOffset = kStages * kStageBytes;
  static constexpr int kStagingBytes = 4 * 2 * 32 * 128;
  static constexpr int kBarOffset = kStagingOffset + kStagingBytes;
  static constexpr int kNumBars = 2 * kStages + 4;
  static constexpr int kTotal = kBarOffset + kNumBars * 8 + 16;
  static constexpr int kDynamic = kTotal + 1024;  // slack for 1024-byte alignment of the tiles
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int group_size = kGroupM * tiles_n;
  const int group = t / group_size;
  const int first_m = group * kGroupM;
  const int gm = min(tiles_m - first_m, kGroupM);
  const int r = t - group * group_size;
  tm = first_m + r % gm;
  tn = r / gm;
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

__device__ __forceinline__ float apply_act(float x, int act) {
  switch (act) {
    case B200K_ACT_RELU:
      return fmaxf(x, 0.f);
    case B200K_ACT_GELU:  // exact (erf) form, the default of aten::gelu
      return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
    case B200K_ACT_SILU:
      return x / (1.f + __expf(-x));
    default:
      return x;
  }
}

__device__ __forceinline__ float load_bias(const void* bias, int dtype, int col) {
  if (dtype == B200K_F32) return __ldg(reinterpret_cast<const float*>(bias) + col);
  if (dtype == B200K_F16) return __half2float(__ldg(reinterpret_cast<const __half*>(bias) + col));
  return __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16*>(bias) + col));
}

// A bias of zero for calls without one (see fused_epilogue).
static __device__ const float kZeroBias = 0.0f;

// Fused epilogue on N accumulator values of one row (columns col0 .. col0 + N - 1), in place:
// r = act(r * scale + bias).  Every lane of a warp reads the same bias element (one broadcast
// load per column).  Afterwards the caller's own scaling must be 1.
// No load here is guarded by a test the compiler could move it across: without a bias the pointer
// is switched to a zero that lives in device memory, and the column index is clamped to the vector
// instead of predicated (columns past n are never stored).  A guarded form of this loop was seen to
// fault on a null bias in one kernel, its loads having been issued ahead of the null test.
template <int N>
__device__ __forceinline__ void fused_epilogue(uint32_t (&r)[N], float scale, const void* bias, int bias_dtype, int act,
                                               int col0, int n) {
  const bool has_bias = bias != nullptr;
  const void* b = has_bias ? bias : static_cast<const void*>(&kZeroBias);
  const int dt = has_bias ? bias_dtype : static_cast<int>(B200K_F32);
  const int last = has_bias ? n - 1 : 0;
#pragma unroll
  for (int j = 0; j < N; ++j) {
    const float x = __uint_as_float(r[j]) * scale + load_bias(b, dt, min(col0 + j, last));
    r[j] = __float_as_uint(apply_act(x, act));
  }
}

// Stores 32 consecutive columns of one output row.
template <typename OutT>
__device__ __forceinline__ void store_chunk(OutT* dst, const uint32_t (&r)[32], float scale, int valid_cols,
                                            bool vec_ok) {
  if (valid_cols >= 32 && vec_ok) {
    if constexpr (sizeof(OutT) == 4) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float4 v = make_float4(__uint_as_float(r[4 * i]) * scale, __uint_as_float(r[4 * i + 1]) * scale,
                               __uint_as_float(r[4 * i + 2]) * scale, __uint_as_float(r[4 * i + 3]) * scale);
        reinterpret_cast<float4*>(dst)[i] = v;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        union {
          uint4 u;
          OutT h[8];
        } pk;
#pragma unroll
        for (int j = 0; j < 8; ++j) pk.h[j] = to_out<OutT>(__uint_as_float(r[8 * i + j]) * scale);
        reinterpret_cast<uint4*>(dst)[i] = pk.u;
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < valid_cols) dst[i] = to_out<OutT>(__uint_as_float(r[i]) * scale);
  }
}

}  // namespace gemm_detail

// Split-K kernel (gemm_splitk_sm100.cu).  Tensor maps as for the whole-tile kernel with 128-row A
// boxes; p.split in {2, 4, 8}, grid = tiles * p.split.
int launch_gemm_splitk(const CUtensorMap& ta, const CUtensorMap& tb, const gemm_detail::GemmParams& p, int bn,
                       int in_dtype, int out_dtype, cudaStream_t stream);
// Clusters of `split` CTAs of that kernel the current device holds at once (0 = cannot launch).
int splitk_resident_clusters(int bn, int split);

}  // namespace b200k
