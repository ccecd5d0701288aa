// Decode and paged-decode attention: one query token per sequence against its KV history,
// grouped-query heads, split over KV chunks (phase 1) and merged by a reduction kernel.
//
// The path is HBM-bandwidth bound (about 4 flop per byte of KV), so the design goal is bytes
// in flight, not math throughput:
//   * a CTA owns one (sequence, kv head, KV chunk); its 4 warps each own every 4th 16-token
//     tile of the chunk and run a private cp.async ring (no CTA-wide barrier in the main loop);
//   * every global access to K/V is a 16-byte cp.async, a warp's 32 lanes covering 512
//     contiguous bytes of a page slab; the page id comes from the block table once per tile;
//   * all query heads of the group share each K/V tile through mma.sync.m16n8k16 with the
//     group's heads as (zero-padded) rows, so issue slots stay free for the loads;
//   * head dim 128 or 64 (template parameter HD): everything below scales with the row length;
//   * softmax state is fp32; row max / sum are reduced across the quad with warp shuffles.
//
// Shared memory tile layout: 16 rows (tokens) x HD halves (256 or 128 bytes); the 16-byte chunk c of
// row r is stored at chunk position c ^ (r & 7) so ldmatrix reads are bank-conflict free.
#include <mutex>
#include <type_traits>

#include "common.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace b200k {
namespace {

constexpr int kTileTokens = 16;
constexpr int kDecodeWarps = 4;
constexpr int kDecodeThreads = kDecodeWarps * 32;
constexpr int kDecodeStages = 3;
// per head dim HD (128 or 64): a tile is 16 tokens x HD halves for K and the same for V
template <int HD>
struct DecodeTile {
  static constexpr int kRowBytes = HD * 2;
  static constexpr int kBytes = kTileTokens * kRowBytes;                        // 4 KB (HD 128) or 2 KB
  static constexpr int kSmem = kDecodeWarps * kDecodeStages * 2 * kBytes;       // 96 KB or 48 KB
  static constexpr int kChunksPerRow = kRowBytes / 16;                          // 16-byte pieces per row
};
constexpr float kLog2e = 1.4426950408889634f;

struct DecodeParams {
  const void* q;
  const void* k;
  const void* v;
  const int32_t* block_table;
  const int32_t* seq_lens;
  float* ws_o;    // [num_seqs * q_heads * max_chunks][128]
  float2* ws_ml;  // [num_seqs * q_heads * max_chunks]  (max in log2 units, sum)
  void* o;
  int32_t num_seqs, q_heads, kv_heads, group;
  int32_t page_size, num_pages, block_table_stride;
  int32_t chunk_tokens, max_chunks;
  int32_t max_seq_len;  // seq_lens entries are clamped to [0, max_seq_len]
  int32_t* status;      // optional device status word
  int64_t kv_batch_stride, kv_head_stride, kv_page_stride;
  float scale_log2;
};

// Address (in elements) of row `token` of kv head `head` for sequence `seq`.  Returns -1 when the
// block-table entry is outside the pool.  This single function defines the paged layout for the
// decode kernel and for the gather check kernel.
template <bool PAGED>
__device__ __forceinline__ int64_t kv_row_offset(const int32_t* __restrict__ block_table, int32_t block_table_stride,
                                                 int32_t page_size, int32_t num_pages, int64_t kv_page_stride,
                                                 int64_t kv_head_stride, int64_t kv_batch_stride, int32_t head_dim,
                                                 int32_t seq, int32_t head, int32_t token) {
  if constexpr (PAGED) {
    const int32_t logical_page = token / page_size;
    const int32_t in_page = token - logical_page * page_size;
    const int32_t page = __ldg(block_table + static_cast<int64_t>(seq) * block_table_stride + logical_page);
    if (page < 0 || page >= num_pages) return -1;
    return static_cast<int64_t>(page) * kv_page_stride + static_cast<int64_t>(head) * kv_head_stride +
           static_cast<int64_t>(in_page) * head_dim;
  } else {
    return static_cast<int64_t>(seq) * kv_batch_stride + static_cast<int64_t>(head) * kv_head_stride +
           static_cast<int64_t>(token) * head_dim;
  }
}

__device__ __forceinline__ void cp_async_16(uint32_t smem_dst, const void* gsrc, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

template <typename T>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ------------------------------------------------------------------------------------------
// phase 1
// ------------------------------------------------------------------------------------------
template <typename T, bool PAGED, int HD>
__global__ void __launch_bounds__(kDecodeThreads, 2) decode_splitkv_kernel(const DecodeParams p) {
  constexpr int kHeadDim = HD;
  constexpr int kTileBytes = DecodeTile<HD>::kBytes;
  constexpr int kRowBytes = DecodeTile<HD>::kRowBytes;
  constexpr int kChunks = DecodeTile<HD>::kChunksPerRow;
  constexpr int kKSteps = HD / 16;  // k-steps of the score product = 16-dim slices of the head dim
  const int chunk = blockIdx.x;
  const int kvh = blockIdx.y;
  const int seq = blockIdx.z;
  // seq_lens is device data the host cannot validate: a length beyond what the grid, the workspace
  // and the block table were sized for is cut to max_seq_len (and reported), a negative one to 0.
  const int len_given = __ldg(p.seq_lens + seq);
  const int len = max(0, min(len_given, p.max_seq_len));
  if (len_given > p.max_seq_len && chunk == 0 && kvh == 0 && threadIdx.x == 0 && p.status)
    atomicOr(p.status, kStatusDecodeLenClamped);
  const int chunk_start = chunk * p.chunk_tokens;
  if (chunk_start >= len) return;
  const int chunk_end = min(len, chunk_start + p.chunk_tokens);
  const int n_tiles = (chunk_end - chunk_start + kTileTokens - 1) / kTileTokens;

  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;  // fragment row
  const int t = lane & 3;   // fragment column pair
  const int G = p.group;

  uint8_t* warp_smem = smem + warp * (kDecodeStages * 2 * kTileBytes);
  const uint32_t warp_smem_u32 = static_cast<uint32_t>(__cvta_generic_to_shared(warp_smem));
  const T* kbase = reinterpret_cast<const T*>(p.k);
  const T* vbase = reinterpret_cast<const T*>(p.v);

  // Query fragments: rows = heads of the group (zero beyond G), HD / 16 k-steps of 16 dims.
  uint32_t qf[kKSteps][4];
  {
    const T* qrow0 = reinterpret_cast<const T*>(p.q) + (static_cast<int64_t>(seq) * p.q_heads + kvh * G) * kHeadDim;
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks) {
      const int col = ks * 16 + 2 * t;
      qf[ks][0] = (g < G) ? *reinterpret_cast<const uint32_t*>(qrow0 + g * kHeadDim + col) : 0u;
      qf[ks][1] = (g + 8 < G) ? *reinterpret_cast<const uint32_t*>(qrow0 + (g + 8) * kHeadDim + col) : 0u;
      qf[ks][2] = (g < G) ? *reinterpret_cast<const uint32_t*>(qrow0 + g * kHeadDim + col + 8) : 0u;
      qf[ks][3] = (g + 8 < G) ? *reinterpret_cast<const uint32_t*>(qrow0 + (g + 8) * kHeadDim + col + 8) : 0u;
    }
  }

  // Issues this lane's cp.async of one tile (HD / 16 for K, as many for V).
  auto issue_tile = [&](int tile, int stage) {
    const int tok0 = chunk_start + tile * kTileTokens;
    const uint32_t sk = warp_smem_u32 + stage * (2 * kTileBytes);
    const uint32_t sv = sk + kTileBytes;
    // All 16 rows of the tile sit in one page (page_size is a multiple of 16), so one table read.
    const int64_t base = kv_row_offset<PAGED>(p.block_table, p.block_table_stride, p.page_size, p.num_pages,
                                              p.kv_page_stride, p.kv_head_stride, p.kv_batch_stride, kHeadDim, seq,
                                              kvh, tok0);
#pragma unroll
    for (int i = 0; i < kKSteps; ++i) {
      const int id = i * 32 + lane;  // 16-byte chunk id inside the slab
      const int row = id / kChunks;
      const int c = id % kChunks;
      const bool valid = (base >= 0) && (tok0 + row < len);
      const int64_t off = valid ? base + row * kHeadDim + c * 8 : 0;
      const uint32_t dst = row * kRowBytes + ((c ^ (row & 7)) << 4);
      cp_async_16(sk + dst, kbase + off, valid ? 16u : 0u);
      cp_async_16(sv + dst, vbase + off, valid ? 16u : 0u);
    }
  };

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  const int my_tiles = (n_tiles > warp) ? (n_tiles - warp + kDecodeWarps - 1) / kDecodeWarps : 0;

#pragma unroll
  for (int s = 0; s < kDecodeStages - 1; ++s) {
    if (s < my_tiles) issue_tile(warp + s * kDecodeWarps, s);
    cp_async_commit();
  }

  for (int j = 0; j < my_tiles; ++j) {
    {
      const int jn = j + kDecodeStages - 1;
      if (jn < my_tiles) issue_tile(warp + jn * kDecodeWarps, jn % kDecodeStages);
      cp_async_commit();
    }
    cp_async_wait<kDecodeStages - 1>();
    __syncwarp();

    const int stage = j % kDecodeStages;
    const uint32_t sk = warp_smem_u32 + stage * (2 * kTileBytes);
    const uint32_t sv = sk + kTileBytes;
    const int tok0 = chunk_start + (warp + j * kDecodeWarps) * kTileTokens;

    // ---- S = Q K^T : 16 (heads) x 16 (tokens) ----
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    {
      const int mi = lane >> 3;
      const int row = (lane & 7) + ((mi >> 1) << 3);
#pragma unroll
      for (int ks = 0; ks < kKSteps; ++ks) {
        const int c = ks * 2 + (mi & 1);
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4(sk + row * kRowBytes + ((c ^ (row & 7)) << 4), r0, r1, r2, r3);
        mma_16816<T>(s[0], qf[ks], r0, r1);
        mma_16816<T>(s[1], qf[ks], r2, r3);
      }
    }

    // ---- online softmax (log2 domain) ----
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int tok = tok0 + i * 8 + 2 * t;
      s[i][0] = (tok < chunk_end) ? s[i][0] * p.scale_log2 : -INFINITY;
      s[i][1] = (tok + 1 < chunk_end) ? s[i][1] * p.scale_log2 : -INFINITY;
      s[i][2] = (tok < chunk_end) ? s[i][2] * p.scale_log2 : -INFINITY;
      s[i][3] = (tok + 1 < chunk_end) ? s[i][3] * p.scale_log2 : -INFINITY;
      mx_lo = fmaxf(mx_lo, fmaxf(s[i][0], s[i][1]));
      mx_hi = fmaxf(mx_hi, fmaxf(s[i][2], s[i][3]));
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    const float ms_lo = (mn_lo == -INFINITY) ? 0.f : mn_lo;
    const float ms_hi = (mn_hi == -INFINITY) ? 0.f : mn_hi;
    const float a_lo = fast_exp2(m_lo - ms_lo), a_hi = fast_exp2(m_hi - ms_hi);
    m_lo = mn_lo;
    m_hi = mn_hi;
    float ps_lo = 0.f, ps_hi = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      s[i][0] = fast_exp2(s[i][0] - ms_lo);
      s[i][1] = fast_exp2(s[i][1] - ms_lo);
      s[i][2] = fast_exp2(s[i][2] - ms_hi);
      s[i][3] = fast_exp2(s[i][3] - ms_hi);
      ps_lo += s[i][0] + s[i][1];
      ps_hi += s[i][2] + s[i][3];
    }
    l_lo = l_lo * a_lo + ps_lo;
    l_hi = l_hi * a_hi + ps_hi;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      o[i][0] *= a_lo;
      o[i][1] *= a_lo;
      o[i][2] *= a_hi;
      o[i][3] *= a_hi;
    }

    // ---- O += P V : 16 (heads) x HD (dims), k = 16 tokens ----
    uint32_t pf[4];
    pf[0] = pack2<T>(s[0][0], s[0][1]);
    pf[1] = pack2<T>(s[0][2], s[0][3]);
    pf[2] = pack2<T>(s[1][0], s[1][1]);
    pf[3] = pack2<T>(s[1][2], s[1][3]);
    {
      const int mi = lane >> 3;
      const int row = (lane & 7) + ((mi & 1) << 3);
#pragma unroll
      for (int dn = 0; dn < HD / 16; ++dn) {
        const int c = dn * 2 + (mi >> 1);
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4_trans(sv + row * kRowBytes + ((c ^ (row & 7)) << 4), r0, r1, r2, r3);
        mma_16816<T>(o[2 * dn], pf, r0, r1);
        mma_16816<T>(o[2 * dn + 1], pf, r2, r3);
      }
    }
    __syncwarp();
  }
  cp_async_wait<0>();

  // ---- merge the four warps' partial states and write the chunk's partial result ----
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  __syncthreads();  // every warp is done with its ring; reuse shared memory
  float* sm_o = reinterpret_cast<float*>(smem);                 // [warps][16][HD]
  float* sm_m = sm_o + kDecodeWarps * 16 * kHeadDim;            // [warps][16]
  float* sm_l = sm_m + kDecodeWarps * 16;                       // [warps][16]
  {
    float* wo = sm_o + warp * 16 * kHeadDim;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      const int col = i * 8 + 2 * t;
      if (g < G) *reinterpret_cast<float2*>(wo + g * kHeadDim + col) = make_float2(o[i][0], o[i][1]);
      if (g + 8 < G) *reinterpret_cast<float2*>(wo + (g + 8) * kHeadDim + col) = make_float2(o[i][2], o[i][3]);
    }
    if (t == 0) {
      sm_m[warp * 16 + g] = m_lo;
      sm_m[warp * 16 + g + 8] = m_hi;
      sm_l[warp * 16 + g] = l_lo;
      sm_l[warp * 16 + g + 8] = l_hi;
    }
  }
  __syncthreads();
  {
    const int d = threadIdx.x;  // one thread per output dim (the upper half idles at HD 64)
    for (int r = 0; r < G && d < kHeadDim; ++r) {
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < kDecodeWarps; ++w) M = fmaxf(M, sm_m[w * 16 + r]);
      const float Ms = (M == -INFINITY) ? 0.f : M;
      float L = 0.f, acc = 0.f;
#pragma unroll
      for (int w = 0; w < kDecodeWarps; ++w) {
        const float f = fast_exp2(sm_m[w * 16 + r] - Ms);
        L += sm_l[w * 16 + r] * f;
        acc += sm_o[(w * 16 + r) * kHeadDim + d] * f;
      }
      const int64_t slot = (static_cast<int64_t>(seq) * p.q_heads + kvh * G + r) * p.max_chunks + chunk;
      p.ws_o[slot * kHeadDim + d] = acc;
      if (d == 0) p.ws_ml[slot] = make_float2(M, L);
    }
  }
}

// ------------------------------------------------------------------------------------------
// phase 2: merge chunks
// ------------------------------------------------------------------------------------------
template <typename T, int HD>
__global__ void __launch_bounds__(HD) decode_reduce_kernel(const DecodeParams p) {
  constexpr int kHeadDim = HD;
  const int qh = blockIdx.x;
  const int seq = blockIdx.y;
  const int d = threadIdx.x;
  const int len = max(0, min(__ldg(p.seq_lens + seq), p.max_seq_len));  // same clamp as phase 1
  const int n_chunks = (len + p.chunk_tokens - 1) / p.chunk_tokens;      // <= max_chunks
  const int64_t slot0 = (static_cast<int64_t>(seq) * p.q_heads + qh) * p.max_chunks;
  float M = -INFINITY;
  for (int c = 0; c < n_chunks; ++c) M = fmaxf(M, p.ws_ml[slot0 + c].x);
  const float Ms = (M == -INFINITY) ? 0.f : M;
  float L = 0.f, acc = 0.f;
  for (int c = 0; c < n_chunks; ++c) {
    const float2 ml = p.ws_ml[slot0 + c];
    const float f = fast_exp2(ml.x - Ms);
    L += ml.y * f;
    acc += p.ws_o[(slot0 + c) * kHeadDim + d] * f;
  }
  const float out = (L > 0.f) ? acc / L : 0.f;
  T* o = reinterpret_cast<T*>(p.o) + (static_cast<int64_t>(seq) * p.q_heads + qh) * kHeadDim + d;
  if constexpr (sizeof(T) == 2 && std::is_same<T, __half>::value)
    *o = __float2half_rn(out);
  else
    *o = __float2bfloat16_rn(out);
}

// ------------------------------------------------------------------------------------------
// gather check kernel: copies rows through the block table with kv_row_offset<true>
// ------------------------------------------------------------------------------------------
__global__ void paged_gather_kernel(const uint8_t* __restrict__ cache, const int32_t* __restrict__ block_table,
                                    const int32_t* __restrict__ seq_lens, uint8_t* __restrict__ out, int32_t kv_heads,
                                    int32_t head_dim, int32_t page_size, int32_t num_pages, int32_t block_table_stride,
                                    int32_t max_seq_len, int64_t kv_page_stride, int64_t kv_head_stride,
                                    int32_t elem_bytes) {
  const int seq = blockIdx.z;
  const int head = blockIdx.y;
  const int len = min(__ldg(seq_lens + seq), max_seq_len);
  const int row_bytes = head_dim * elem_bytes;
  const int chunks_per_row = row_bytes / 16;
  for (int token = blockIdx.x; token < len; token += gridDim.x) {
    const int64_t off = kv_row_offset<true>(block_table, block_table_stride, page_size, num_pages, kv_page_stride,
                                            kv_head_stride, 0, head_dim, seq, head, token);
    if (off < 0) continue;
    const uint4* src = reinterpret_cast<const uint4*>(cache + off * elem_bytes);
    uint4* dst = reinterpret_cast<uint4*>(
        out + ((static_cast<int64_t>(seq) * kv_heads + head) * max_seq_len + token) * row_bytes);
    for (int c = threadIdx.x; c < chunks_per_row; c += blockDim.x) dst[c] = src[c];
  }
}

int validate_decode(const b200k_decode_args& a) {
  if (!a.q || !a.k_cache || !a.v_cache || !a.seq_lens || !a.o)
    return set_error(B200K_ERR_NULL, "decode_attention: q, k_cache, v_cache, seq_lens and o must be non-NULL");
  if (a.num_seqs <= 0 || a.q_heads <= 0 || a.kv_heads <= 0 || a.max_seq_len <= 0)
    return set_error(B200K_ERR_BAD_SHAPE, "decode_attention: num_seqs, q_heads, kv_heads, max_seq_len must be > 0");
  if (a.head_dim != 128 && a.head_dim != 64)
    return set_error(B200K_ERR_BAD_SHAPE, "decode_attention: head_dim must be 128 or 64");
  if (a.q_heads % a.kv_heads != 0 || a.q_heads / a.kv_heads > 16)
    return set_error(B200K_ERR_BAD_SHAPE, "decode_attention: q_heads must be a multiple (<= 16x) of kv_heads");
  if (a.dtype != B200K_F16 && a.dtype != B200K_BF16)
    return set_error(B200K_ERR_BAD_DTYPE, "decode_attention: dtype must be F16 or BF16");
  if (a.chunk_tokens < 0 || a.chunk_tokens % 64 != 0)
    return set_error(B200K_ERR_BAD_SHAPE, "decode_attention: chunk_tokens must be 0 or a multiple of 64");
  if (a.num_seqs > 65535 || a.kv_heads > 65535)
    return set_error(B200K_ERR_BAD_SHAPE, "decode_attention: num_seqs and kv_heads must be <= 65535");
  if (a.block_table) {
    if (a.page_size <= 0 || a.page_size % 16 != 0)
      return set_error(B200K_ERR_BAD_SHAPE, "decode_attention: page_size must be a positive multiple of 16");
    if (a.num_pages <= 0 || a.block_table_stride <= 0)
      return set_error(B200K_ERR_BAD_SHAPE, "decode_attention: num_pages and block_table_stride must be > 0");
    if (static_cast<int64_t>(a.block_table_stride) * a.page_size < a.max_seq_len)
      return set_error(B200K_ERR_BAD_SHAPE, "decode_attention: block table row too short for max_seq_len");
    if (a.kv_page_stride % 8 != 0 || a.kv_head_stride % 8 != 0)
      return set_error(B200K_ERR_BAD_ALIGN, "decode_attention: page and head strides must be multiples of 8 elements");
  } else {
    if (a.kv_batch_stride % 8 != 0 || a.kv_head_stride % 8 != 0)
      return set_error(B200K_ERR_BAD_ALIGN, "decode_attention: batch and head strides must be multiples of 8 elements");
  }
  if ((reinterpret_cast<uintptr_t>(a.k_cache) & 15) || (reinterpret_cast<uintptr_t>(a.v_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(a.q) & 15) || (reinterpret_cast<uintptr_t>(a.o) & 15))
    return set_error(B200K_ERR_BAD_ALIGN, "decode_attention: q, o, k_cache, v_cache must be 16-byte aligned");
  return B200K_OK;
}

template <typename T, int HD>
int launch_decode_typed(const DecodeParams& p, bool paged, int num_seqs, cudaStream_t stream) {
  dim3 grid(p.max_chunks, p.kv_heads, num_seqs);
  constexpr int kSmem = DecodeTile<HD>::kSmem;
  int rc;
  if (paged) {
    auto kfn = decode_splitkv_kernel<T, true, HD>;
    static bool configured[64] = {};
    rc = ensure_dynamic_smem(kfn, kSmem, configured, "cudaFuncSetAttribute(decode smem)");
    if (rc) return rc;
    kfn<<<grid, kDecodeThreads, kSmem, stream>>>(p);
  } else {
    auto kfn = decode_splitkv_kernel<T, false, HD>;
    static bool configured[64] = {};
    rc = ensure_dynamic_smem(kfn, kSmem, configured, "cudaFuncSetAttribute(decode smem)");
    if (rc) return rc;
    kfn<<<grid, kDecodeThreads, kSmem, stream>>>(p);
  }
  rc = check_cuda(cudaGetLastError(), "decode_splitkv_kernel launch");
  if (rc) return rc;
  decode_reduce_kernel<T, HD><<<dim3(p.q_heads, num_seqs), HD, 0, stream>>>(p);
  return check_cuda(cudaGetLastError(), "decode_reduce_kernel launch");
}

}  // namespace

int32_t decode_default_chunk(const b200k_decode_args& a) {
  if (a.chunk_tokens > 0) return a.chunk_tokens;
  if (a.max_seq_len <= 0 || a.num_seqs <= 0 || a.kv_heads <= 0) return 64;
  const int64_t want = 8ll * 148;  // enough CTAs to fill every SM several times over
  int32_t ch = 512;
  while (ch > 64 &&
         static_cast<int64_t>(a.num_seqs) * a.kv_heads * ((a.max_seq_len + ch - 1) / ch) < want)
    ch /= 2;
  return ch;
}

uint64_t decode_workspace_bytes(const b200k_decode_args& a) {
  if (a.num_seqs <= 0 || a.q_heads <= 0 || a.max_seq_len <= 0) return 0;
  const int32_t ch = decode_default_chunk(a);
  const uint64_t max_chunks = (static_cast<uint64_t>(a.max_seq_len) + ch - 1) / ch;
  const uint64_t slots = static_cast<uint64_t>(a.num_seqs) * a.q_heads * max_chunks;
  return slots * static_cast<uint64_t>(a.head_dim > 0 ? a.head_dim : 128) * sizeof(float) + slots * sizeof(float2);
}

int launch_decode(const b200k_decode_args& a, cudaStream_t stream) {
  int rc = validate_decode(a);
  if (rc) return rc;
  const uint64_t need = decode_workspace_bytes(a);
  if (!a.workspace || a.workspace_bytes < need)
    return set_error(B200K_ERR_WORKSPACE, "decode_attention: workspace of %llu bytes required, %llu given",
                     static_cast<unsigned long long>(need), static_cast<unsigned long long>(a.workspace_bytes));
  if (reinterpret_cast<uintptr_t>(a.workspace) & 255)
    return set_error(B200K_ERR_BAD_ALIGN, "decode_attention: workspace must be 256-byte aligned");
  rc = ensure_sm100();
  if (rc) return rc;

  DecodeParams p;
  p.q = a.q;
  p.k = a.k_cache;
  p.v = a.v_cache;
  p.block_table = a.block_table;
  p.seq_lens = a.seq_lens;
  p.o = a.o;
  p.num_seqs = a.num_seqs;
  p.q_heads = a.q_heads;
  p.kv_heads = a.kv_heads;
  p.group = a.q_heads / a.kv_heads;
  p.page_size = a.block_table ? a.page_size : 16;
  p.num_pages = a.num_pages;
  p.block_table_stride = a.block_table_stride;
  p.chunk_tokens = decode_default_chunk(a);
  p.max_chunks = (a.max_seq_len + p.chunk_tokens - 1) / p.chunk_tokens;
  p.max_seq_len = a.max_seq_len;
  p.status = a.status;
  p.kv_batch_stride = a.kv_batch_stride;
  p.kv_head_stride = a.kv_head_stride;
  p.kv_page_stride = a.kv_page_stride;
  p.scale_log2 = a.scale * kLog2e;
  const uint64_t slots = static_cast<uint64_t>(a.num_seqs) * a.q_heads * p.max_chunks;
  p.ws_o = reinterpret_cast<float*>(a.workspace);
  p.ws_ml = reinterpret_cast<float2*>(reinterpret_cast<uint8_t*>(a.workspace) + slots * a.head_dim * sizeof(float));
  if (p.max_chunks > 65535 * 32)
    return set_error(B200K_ERR_BAD_SHAPE, "decode_attention: too many chunks (raise chunk_tokens)");
  const bool paged = a.block_table != nullptr;
  if (a.head_dim == 128) {
    if (a.dtype == B200K_F16) return launch_decode_typed<__half, 128>(p, paged, a.num_seqs, stream);
    return launch_decode_typed<__nv_bfloat16, 128>(p, paged, a.num_seqs, stream);
  }
  if (a.dtype == B200K_F16) return launch_decode_typed<__half, 64>(p, paged, a.num_seqs, stream);
  return launch_decode_typed<__nv_bfloat16, 64>(p, paged, a.num_seqs, stream);
}

int launch_paged_gather(const void* cache, const int32_t* block_table, const int32_t* seq_lens, void* out,
                        int32_t num_seqs, int32_t kv_heads, int32_t head_dim, int32_t page_size, int32_t num_pages,
                        int32_t block_table_stride, int32_t max_seq_len, int64_t kv_page_stride, int64_t kv_head_stride,
                        int32_t elem_bytes, cudaStream_t stream) {
  if (!cache || !block_table || !seq_lens || !out) return set_error(B200K_ERR_NULL, "paged_gather: NULL pointer");
  if (num_seqs <= 0 || kv_heads <= 0 || head_dim <= 0 || page_size <= 0 || num_pages <= 0 || max_seq_len <= 0 ||
      block_table_stride <= 0 || num_seqs > 65535 || kv_heads > 65535)
    return set_error(B200K_ERR_BAD_SHAPE, "paged_gather: bad dimensions");
  if (elem_bytes <= 0 || (head_dim * elem_bytes) % 16 != 0 || (kv_page_stride * elem_bytes) % 16 != 0 ||
      (kv_head_stride * elem_bytes) % 16 != 0 || (reinterpret_cast<uintptr_t>(cache) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return set_error(B200K_ERR_BAD_ALIGN, "paged_gather: rows, strides and bases must be multiples of 16 bytes");
  int rc = ensure_sm100();
  if (rc) return rc;
  const int gx = max_seq_len < 1024 ? max_seq_len : 1024;
  paged_gather_kernel<<<dim3(gx, kv_heads, num_seqs), 32, 0, stream>>>(
      reinterpret_cast<const uint8_t*>(cache), block_table, seq_lens, reinterpret_cast<uint8_t*>(out), kv_heads,
      head_dim, page_size, num_pages, block_table_stride, max_seq_len, kv_page_stride, kv_head_stride, elem_bytes);
  return check_cuda(cudaGetLastError(), "paged_gather_kernel launch");
}

// ------------------------------------------------------------------------------------------
// KV-cache append: the step before decode.  Row t of new_rows[s] goes to token position
// positions[s] + t of sequence s, through the block table, with kv_row_offset<true> (the address
// function of the decode kernel).  One warp per (token, head) row; 16-byte stores; rows whose
// block-table entry is outside the pool are dropped and reported through the status word.
// ------------------------------------------------------------------------------------------
__global__ void kv_append_kernel(const uint8_t* __restrict__ k_new, const uint8_t* __restrict__ v_new,
                                 uint8_t* __restrict__ k_cache, uint8_t* __restrict__ v_cache,
                                 const int32_t* __restrict__ block_table, const int32_t* __restrict__ positions,
                                 int32_t new_tokens, int32_t kv_heads, int32_t head_dim, int32_t page_size,
                                 int32_t num_pages, int32_t block_table_stride, int64_t kv_page_stride,
                                 int64_t kv_head_stride, int32_t elem_bytes, int32_t* status) {
  const int seq = blockIdx.z;
  const int head = blockIdx.y;
  const int row_bytes = head_dim * elem_bytes;
  const int chunks_per_row = row_bytes / 16;
  const int pos0 = __ldg(positions + seq);
  const int warps = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int t = blockIdx.x * warps + warp; t < new_tokens; t += gridDim.x * warps) {
    const int token = pos0 + t;
    int64_t off = -1;
    if (pos0 >= 0 && token / page_size < block_table_stride)
      off = kv_row_offset<true>(block_table, block_table_stride, page_size, num_pages, kv_page_stride, kv_head_stride, 0,
                                head_dim, seq, head, token);
    if (off < 0) {
      if (lane == 0 && status) atomicOr(status, kStatusDecodeBadPage);
      continue;
    }
    const int64_t src = ((static_cast<int64_t>(seq) * new_tokens + t) * kv_heads + head) * row_bytes;
    const uint4* ks = reinterpret_cast<const uint4*>(k_new + src);
    const uint4* vs = reinterpret_cast<const uint4*>(v_new + src);
    uint4* kd = reinterpret_cast<uint4*>(k_cache + off * elem_bytes);
    uint4* vd = reinterpret_cast<uint4*>(v_cache + off * elem_bytes);
    for (int c = lane; c < chunks_per_row; c += 32) {
      kd[c] = __ldg(ks + c);
      vd[c] = __ldg(vs + c);
    }
  }
}

int launch_kv_append(const void* k_new, const void* v_new, void* k_cache, void* v_cache, const int32_t* block_table,
                     const int32_t* positions, int32_t num_seqs, int32_t new_tokens, int32_t kv_heads, int32_t head_dim,
                     int32_t page_size, int32_t num_pages, int32_t block_table_stride, int64_t kv_page_stride,
                     int64_t kv_head_stride, int32_t elem_bytes, int32_t* status, cudaStream_t stream) {
  if (!k_new || !v_new || !k_cache || !v_cache || !block_table || !positions)
    return set_error(B200K_ERR_NULL, "kv_append: NULL pointer");
  if (num_seqs <= 0 || new_tokens <= 0 || kv_heads <= 0 || head_dim <= 0 || page_size <= 0 || num_pages <= 0 ||
      block_table_stride <= 0 || num_seqs > 65535 || kv_heads > 65535)
    return set_error(B200K_ERR_BAD_SHAPE, "kv_append: bad dimensions");
  if (elem_bytes <= 0 || (head_dim * elem_bytes) % 16 != 0 || (kv_page_stride * elem_bytes) % 16 != 0 ||
      (kv_head_stride * elem_bytes) % 16 != 0 || (reinterpret_cast<uintptr_t>(k_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(v_cache) & 15) || (reinterpret_cast<uintptr_t>(k_new) & 15) ||
      (reinterpret_cast<uintptr_t>(v_new) & 15))
    return set_error(B200K_ERR_BAD_ALIGN, "kv_append: rows, strides and bases must be multiples of 16 bytes");
  int rc = ensure_sm100();
  if (rc) return rc;
  const int warps = 4;
  int gx = (new_tokens + warps - 1) / warps;
  if (gx > 1024) gx = 1024;
  kv_append_kernel<<<dim3(gx, kv_heads, num_seqs), warps * 32, 0, stream>>>(
      reinterpret_cast<const uint8_t*>(k_new), reinterpret_cast<const uint8_t*>(v_new),
      reinterpret_cast<uint8_t*>(k_cache), reinterpret_cast<uint8_t*>(v_cache), block_table, positions, new_tokens,
      kv_heads, head_dim, page_size, num_pages, block_table_stride, kv_page_stride, kv_head_stride, elem_bytes, status);
  return check_cuda(cudaGetLastError(), "kv_append_kernel launch");
}

// ------------------------------------------------------------------------------------------
// Decode with scratch that lives inside the library.
//
// Some callers have no way to hand over scratch memory: a host runtime that gives a plug-in
// kernel only its input and output buffers and keeps every device allocation to itself, or a
// serving loop that runs inside a fixed, pre-planned memory budget where cudaMalloc (which may
// synchronize the device, and may fail once memory is fragmented) is not allowed on the request
// path.  For them the split-KV partials go into the fixed array below instead of a caller
// buffer.  The array is part of the loaded module, so every GPU that loads this library keeps
// B200K_DECODE_STATIC_SCRATCH_BYTES of device memory reserved until the process exits.
//
// In host code `g_decode_scratch` is only a handle for the runtime, not a device address, so it
// is never passed to a kernel directly: the address is looked up once per device with
// cudaGetSymbolAddress (with that device current) and cached.
// ------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_decode_scratch[B200K_DECODE_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_scratch_mu;
void* g_scratch_addr[64] = {};  // indexed by device ordinal

int static_scratch_for_current_device(void** out) {
  int dev = -1;
  int rc = check_cuda(cudaGetDevice(&dev), "decode_attention_static: cudaGetDevice");
  if (rc) return rc;
  if (dev < 0 || dev >= 64) return set_error(B200K_ERR_CUDA, "decode_attention_static: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (!g_scratch_addr[dev]) {
    void* addr = nullptr;
    rc = check_cuda(cudaGetSymbolAddress(&addr, g_decode_scratch), "decode_attention_static: cudaGetSymbolAddress");
    if (rc) return rc;
    if (!addr) return set_error(B200K_ERR_CUDA, "decode_attention_static: scratch symbol resolved to NULL");
    g_scratch_addr[dev] = addr;
  }
  *out = g_scratch_addr[dev];
  return B200K_OK;
}
}  // namespace

int launch_decode_static(const b200k_decode_args& a, cudaStream_t stream) {
  int rc = validate_decode(a);
  if (rc) return rc;
  const uint64_t need = decode_workspace_bytes(a);
  if (need > B200K_DECODE_STATIC_SCRATCH_BYTES)
    return set_error(B200K_ERR_WORKSPACE,
                     "decode_attention_static: this problem needs %llu bytes of scratch but the built-in array holds "
                     "%llu; use a larger chunk_tokens, fewer sequences per call, or b200k_decode_attention with a "
                     "caller-provided workspace",
                     static_cast<unsigned long long>(need),
                     static_cast<unsigned long long>(B200K_DECODE_STATIC_SCRATCH_BYTES));
  rc = ensure_sm100();
  if (rc) return rc;
  void* scratch = nullptr;
  rc = static_scratch_for_current_device(&scratch);
  if (rc) return rc;
  // Nothing in the scratch has to start at zero: the reduction reads only the slots of chunks
  // below ceil(len / chunk) of each sequence, and phase 1 of the same call writes exactly those.
  b200k_decode_args with_scratch = a;
  with_scratch.workspace = scratch;
  with_scratch.workspace_bytes = B200K_DECODE_STATIC_SCRATCH_BYTES;
  return launch_decode(with_scratch, stream);
}

}  // namespace b200k
