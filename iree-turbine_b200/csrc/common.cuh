// Shared host/device declarations for the kernel translation units and the C-ABI layer.
#pragma once
#include <cstdint>
#include <cstddef>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/b200k.h"

namespace b200k {

// Codes OR-ed into the caller's device status word by kernels whose bounded waits gave up.
enum : int32_t {
  kStatusGemmTimeout = 1,
  kStatusAttnTimeout = 2,
  kStatusDecodeBadPage = 4,
  kStatusDecodeLenClamped = 8,
  kStatusSelftestTimeout = 16,
  kStatusGemmNoCluster = 32,  // split-K kernel found itself in a cluster of another size than asked for
};

// ---- host-side error plumbing (abi.cu) ----
int set_error(int status, const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);
int ensure_sm100();
int num_sms();

// Encodes a tiled tensor map with 128-byte swizzle.  dims/strides innermost-first; strides in
// bytes for dimensions 1..rank-1.
int encode_tmap(CUtensorMap* out, int dtype, int rank, void* base, const uint64_t* dims, const uint64_t* strides_bytes,
                const uint32_t* box, bool swizzle128 = true);

// ---- launchers implemented next to their kernels ----
int launch_gemm_nt(const b200k_gemm_args& a, cudaStream_t stream);
int launch_gemm_nt_allgather(const b200k_gemm_allgather_args& g, cudaStream_t stream);
int launch_attention_fwd(const b200k_attention_args& a, cudaStream_t stream);
int launch_attention_fwd_tile(const b200k_attention_args& a, cudaStream_t stream);  // attention_tile_sm100.cu
int launch_paged_attention_fwd_tile(const b200k_paged_attention_args& a, cudaStream_t stream);
int launch_paged_attention_fwd(const b200k_paged_attention_args& a, cudaStream_t stream);
int launch_decode(const b200k_decode_args& a, cudaStream_t stream);
int launch_decode_static(const b200k_decode_args& a, cudaStream_t stream);
uint64_t decode_workspace_bytes(const b200k_decode_args& a);
int32_t decode_default_chunk(const b200k_decode_args& a);
int launch_paged_gather(const void* cache, const int32_t* block_table, const int32_t* seq_lens, void* out,
                        int32_t num_seqs, int32_t kv_heads, int32_t head_dim, int32_t page_size, int32_t num_pages,
                        int32_t block_table_stride, int32_t max_seq_len, int64_t kv_page_stride, int64_t kv_head_stride,
                        int32_t elem_bytes, cudaStream_t stream);
int launch_kv_append(const void* k_new, const void* v_new, void* k_cache, void* v_cache, const int32_t* block_table,
                     const int32_t* positions, int32_t num_seqs, int32_t new_tokens, int32_t kv_heads, int32_t head_dim,
                     int32_t page_size, int32_t num_pages, int32_t block_table_stride, int64_t kv_page_stride,
                     int64_t kv_head_stride, int32_t elem_bytes, int32_t* status, cudaStream_t stream);
int launch_bounded_wait_selftest(int32_t* status, uint32_t limit_us, cudaStream_t stream);
int launch_quantize_e4m3(const float* x, void* y, float* scale_out, uint32_t* amax_scratch, int64_t n,
                         cudaStream_t stream);

// Opts a kernel into more than 48 KB of dynamic shared memory.  The attribute belongs to the
// (function, device) pair, so it is set once per device ordinal: `done` is the caller's table, one
// per kernel instantiation.  Setting it twice is harmless, which is why the table needs no lock.
template <typename Kernel>
inline int ensure_dynamic_smem(Kernel kfn, int bytes, bool (&done)[64], const char* what) {
  int dev = -1;
  int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
  if (rc) return rc;
  if (dev < 0 || dev >= 64) return set_error(B200K_ERR_CUDA, "%s: device ordinal %d out of range", what, dev);
  if (done[dev]) return B200K_OK;
  rc = check_cuda(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes), what);
  if (rc) return rc;
  done[dev] = true;
  return B200K_OK;
}

inline size_t dtype_size(int dt) {
  switch (dt) {
    case B200K_F16:
    case B200K_BF16:
      return 2;
    case B200K_F32:
      return 4;
    case B200K_E4M3:
      return 1;
    default:
      return 0;
  }
}

}  // namespace b200k
