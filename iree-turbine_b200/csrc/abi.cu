// extern "C" surface of the library (declared in include/b200k.h): argument plumbing, error
// reporting, tensor-map encoding through the driver entry point, host-buffer variants.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace b200k {

namespace {
thread_local char g_last_error[512] = "";

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}
}  // namespace

int set_error(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return status;
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return B200K_OK;
  return set_error(B200K_ERR_CUDA, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

namespace {
struct DeviceInfo {
  int major = -1;
  int sms = 0;
};
DeviceInfo query_device() {
  // Cached per device ordinal; small fixed table (a box has at most 8 GPUs, allow 64).
  static DeviceInfo table[64];
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return DeviceInfo{};
  std::lock_guard<std::mutex> lock(mu);
  if (table[dev].major < 0) {
    int major = 0, sms = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return DeviceInfo{};
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return DeviceInfo{};
    table[dev].major = major;
    table[dev].sms = sms;
  }
  return table[dev];
}
}  // namespace

int ensure_sm100() {
  DeviceInfo d = query_device();
  if (d.major < 0) {
    cudaGetLastError();
    return set_error(B200K_ERR_CUDA, "no usable CUDA device (cudaGetDevice / attribute query failed)");
  }
  if (d.major != 10)
    return set_error(B200K_ERR_UNSUPPORTED_ARCH, "kernels are built for sm_100a only; device has compute capability %d.x",
                     d.major);
  return B200K_OK;
}

int num_sms() {
  DeviceInfo d = query_device();
  return d.sms > 0 ? d.sms : 148;
}

int encode_tmap(CUtensorMap* out, int dtype, int rank, void* base, const uint64_t* dims, const uint64_t* strides_bytes,
                const uint32_t* box, bool swizzle128) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return set_error(B200K_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMapDataType dt;
  switch (dtype) {
    case B200K_F16:
      dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
      break;
    case B200K_BF16:
      dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
      break;
    case B200K_E4M3:
      dt = CU_TENSOR_MAP_DATA_TYPE_UINT8;
      break;
    case B200K_F32:
      dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
      break;
    default:
      return set_error(B200K_ERR_BAD_DTYPE, "encode_tmap: dtype %d", dtype);
  }
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i > 0) gstrides[i - 1] = strides_bytes[i - 1];
  }
  auto encode = [&]() {
    return fn(out, dt, static_cast<cuuint32_t>(rank), base, gdims, gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult r = encode();
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // A thread that has made no runtime call that needs the device yet (an autograd worker thread
    // running a backward op first thing) has no current driver context: bind the primary one.
    cudaFree(nullptr);
    r = encode();
  }
  if (r != CUDA_SUCCESS)
    return set_error(B200K_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dims %llu x %llu)",
                     static_cast<int>(r), rank, static_cast<unsigned long long>(dims[0]),
                     static_cast<unsigned long long>(rank > 1 ? dims[1] : 1));
  return B200K_OK;
}

// Copy-back stream of the host-buffer entry points, one per device, created on first use and kept
// for the life of the process (a stream and two events; no device memory).  Results go back to the
// host on this stream while the caller's stream is already uploading the next slice, so the two
// copy directions overlap.
struct SideStream {
  cudaStream_t stream = nullptr;
  cudaEvent_t ready = nullptr;  // a slice's result is complete on the caller's stream
  cudaEvent_t done = nullptr;   // all copy-backs are complete on the side stream
};

int get_side_stream(SideStream* out) {
  static std::mutex mu;
  static SideStream cache[64];
  int dev = 0;
  int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
  if (rc) return rc;
  if (dev < 0 || dev >= 64) return set_error(B200K_ERR_CUDA, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  SideStream& c = cache[dev];
  if (!c.stream) {
    SideStream n;
    rc = check_cuda(cudaStreamCreateWithFlags(&n.stream, cudaStreamNonBlocking), "create copy-back stream");
    if (rc) return rc;
    rc = check_cuda(cudaEventCreateWithFlags(&n.ready, cudaEventDisableTiming), "create event");
    if (rc) return rc;
    rc = check_cuda(cudaEventCreateWithFlags(&n.done, cudaEventDisableTiming), "create event");
    if (rc) return rc;
    c = n;
  }
  *out = c;
  return 0;
}

}  // namespace b200k

namespace b200k {
// attention_bwd_sm100.cu
int launch_attention_bwd(const b200k_attention_bwd_args& a, cudaStream_t stream);
uint64_t attention_bwd_workspace_bytes(const b200k_attention_bwd_args& a);
}  // namespace b200k

using namespace b200k;

extern "C" {

int b200k_abi_version(void) { return B200K_ABI_VERSION; }

const char* b200k_last_error(void) { return g_last_error; }

const char* b200k_status_string(int status) {
  switch (status) {
    case B200K_OK:
      return "OK";
    case B200K_ERR_BAD_SHAPE:
      return "BAD_SHAPE";
    case B200K_ERR_BAD_ALIGN:
      return "BAD_ALIGN";
    case B200K_ERR_BAD_DTYPE:
      return "BAD_DTYPE";
    case B200K_ERR_UNSUPPORTED_ARCH:
      return "UNSUPPORTED_ARCH";
    case B200K_ERR_CUDA:
      return "CUDA_ERROR";
    case B200K_ERR_NULL:
      return "NULL_POINTER";
    case B200K_ERR_TIMEOUT:
      return "TIMEOUT";
    case B200K_ERR_WORKSPACE:
      return "WORKSPACE_TOO_SMALL";
    default:
      return "UNKNOWN";
  }
}

int b200k_gemm_nt(const b200k_gemm_args* args, void* stream) {
  if (!args) return set_error(B200K_ERR_NULL, "gemm_nt: args is NULL");
  return launch_gemm_nt(*args, static_cast<cudaStream_t>(stream));
}

int b200k_gemm_nt_allgather(const b200k_gemm_allgather_args* args, void* stream) {
  if (!args) return set_error(B200K_ERR_NULL, "gemm_nt_allgather: args is NULL");
  return launch_gemm_nt_allgather(*args, static_cast<cudaStream_t>(stream));
}

uint64_t b200k_attention_bwd_workspace_bytes(const b200k_attention_bwd_args* args) {
  return args ? attention_bwd_workspace_bytes(*args) : 0;
}

int b200k_attention_bwd(const b200k_attention_bwd_args* args, void* stream) {
  if (!args) return set_error(B200K_ERR_NULL, "attention_bwd: args is NULL");
  return launch_attention_bwd(*args, static_cast<cudaStream_t>(stream));
}

int b200k_attention_fwd(const b200k_attention_args* args, void* stream) {
  if (!args) return set_error(B200K_ERR_NULL, "attention_fwd: args is NULL");
  return launch_attention_fwd(*args, static_cast<cudaStream_t>(stream));
}

uint64_t b200k_decode_workspace_bytes(const b200k_decode_args* args) {
  if (!args) return 0;
  return decode_workspace_bytes(*args);
}

int32_t b200k_decode_default_chunk(const b200k_decode_args* args) {
  if (!args) return 0;
  return decode_default_chunk(*args);
}

int b200k_decode_attention(const b200k_decode_args* args, void* stream) {
  if (!args) return set_error(B200K_ERR_NULL, "decode_attention: args is NULL");
  return launch_decode(*args, static_cast<cudaStream_t>(stream));
}

int b200k_decode_attention_static(const b200k_decode_args* args, void* stream) {
  if (!args) return set_error(B200K_ERR_NULL, "decode_attention_static: args is NULL");
  return launch_decode_static(*args, static_cast<cudaStream_t>(stream));
}

int b200k_paged_gather(const void* cache, const int32_t* block_table, const int32_t* seq_lens, void* out,
                       int32_t num_seqs, int32_t kv_heads, int32_t head_dim, int32_t page_size, int32_t num_pages,
                       int32_t block_table_stride, int32_t max_seq_len, int64_t kv_page_stride,
                       int64_t kv_head_stride, int32_t elem_bytes, void* stream) {
  return launch_paged_gather(cache, block_table, seq_lens, out, num_seqs, kv_heads, head_dim, page_size, num_pages,
                             block_table_stride, max_seq_len, kv_page_stride, kv_head_stride, elem_bytes,
                             static_cast<cudaStream_t>(stream));
}

int b200k_paged_attention_fwd(const b200k_paged_attention_args* args, void* stream) {
  if (!args) return set_error(B200K_ERR_NULL, "paged_attention_fwd: args is NULL");
  return launch_paged_attention_fwd(*args, static_cast<cudaStream_t>(stream));
}

int b200k_kv_append(const void* k_new, const void* v_new, void* k_cache, void* v_cache, const int32_t* block_table,
                    const int32_t* positions, int32_t num_seqs, int32_t new_tokens, int32_t kv_heads, int32_t head_dim,
                    int32_t page_size, int32_t num_pages, int32_t block_table_stride, int64_t kv_page_stride,
                    int64_t kv_head_stride, int32_t elem_bytes, int32_t* status, void* stream) {
  return launch_kv_append(k_new, v_new, k_cache, v_cache, block_table, positions, num_seqs, new_tokens, kv_heads,
                          head_dim, page_size, num_pages, block_table_stride, kv_page_stride, kv_head_stride, elem_bytes,
                          status, static_cast<cudaStream_t>(stream));
}

int b200k_selftest_bounded_wait(int32_t* status, uint32_t limit_us, void* stream) {
  return launch_bounded_wait_selftest(status, limit_us, static_cast<cudaStream_t>(stream));
}

int b200k_quantize_e4m3(const float* x, void* y, float* scale_out, uint32_t* amax_scratch, int64_t n, void* stream) {
  return launch_quantize_e4m3(x, y, scale_out, amax_scratch, n, static_cast<cudaStream_t>(stream));
}

int b200k_gemm_nt_host(const b200k_gemm_args* host, const b200k_gemm_args* dev, void* stream) {
  if (!host || !dev) return set_error(B200K_ERR_NULL, "gemm_nt_host: args is NULL");
  if (!host->a || !host->b || !host->c || !dev->a || !dev->b || !dev->c)
    return set_error(B200K_ERR_NULL, "gemm_nt_host: host and device a, b, c must be non-NULL");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t in_es = dtype_size(dev->in_dtype), out_es = dtype_size(dev->out_dtype);
  if (in_es == 0 || out_es == 0) return set_error(B200K_ERR_BAD_DTYPE, "gemm_nt_host: bad dtype");
  if (dev->m <= 0 || dev->n <= 0 || dev->k <= 0) return set_error(B200K_ERR_BAD_SHAPE, "gemm_nt_host: bad shape");
  // The row-block slicing below assumes A stored [M, K] and B stored [N, K].
  if (dev->a_km || dev->b_kn || host->a_km || host->b_kn)
    return set_error(B200K_ERR_BAD_SHAPE, "gemm_nt_host: operands stored [K, M] / [K, N] are not supported on the host-buffer path");
  if (dev->lda < dev->k || dev->ldb < dev->k || dev->ldc < dev->n || host->lda < dev->k || host->ldb < dev->k ||
      host->ldc < dev->n)
    return set_error(B200K_ERR_BAD_SHAPE, "gemm_nt_host: a row pitch of the host or device image is smaller than the row");
  // Row pitches may differ between the host and device images.  B goes up first; then A is
  // uploaded, multiplied and C copied back in row blocks, the copy-back of one block (on the
  // library's copy-back stream) overlapping the upload of the next.
  SideStream side;
  int rc = get_side_stream(&side);
  if (rc) return rc;
  rc = check_cuda(cudaMemcpy2DAsync(const_cast<void*>(dev->b), dev->ldb * in_es, host->b, host->ldb * in_es,
                                    dev->k * in_es, dev->n, cudaMemcpyHostToDevice, s),
                  "gemm_nt_host: copy B");
  if (rc) return rc;
  // blocks of whole 256-row tiles, at least 8 MB of A each so that a block keeps every SM busy
  int64_t rows = dev->m;
  const int64_t min_rows = ((int64_t(8) << 20) / (dev->k * int64_t(in_es)) + 255) / 256 * 256;
  if (dev->m >= 2 * min_rows) rows = min_rows > 1024 ? min_rows : 1024;
  for (int64_t r0 = 0; r0 < dev->m; r0 += rows) {
    const int64_t nr = dev->m - r0 < rows ? dev->m - r0 : rows;
    b200k_gemm_args blk = *dev;
    blk.m = nr;
    blk.a = static_cast<const char*>(dev->a) + r0 * dev->lda * in_es;
    blk.c = static_cast<char*>(dev->c) + r0 * dev->ldc * out_es;
    rc = check_cuda(cudaMemcpy2DAsync(const_cast<void*>(blk.a), dev->lda * in_es,
                                      static_cast<const char*>(host->a) + r0 * host->lda * in_es, host->lda * in_es,
                                      dev->k * in_es, nr, cudaMemcpyHostToDevice, s),
                    "gemm_nt_host: copy A");
    if (rc) return rc;
    rc = launch_gemm_nt(blk, s);
    if (rc) return rc;
    rc = check_cuda(cudaEventRecord(side.ready, s), "record");
    if (rc) return rc;
    rc = check_cuda(cudaStreamWaitEvent(side.stream, side.ready, 0), "wait");
    if (rc) return rc;
    rc = check_cuda(cudaMemcpy2DAsync(static_cast<char*>(host->c) + r0 * host->ldc * out_es, host->ldc * out_es, blk.c,
                                      dev->ldc * out_es, dev->n * out_es, nr, cudaMemcpyDeviceToHost, side.stream),
                    "gemm_nt_host: copy C");
    if (rc) return rc;
  }
  // the caller's stream completes only when every copy-back has
  rc = check_cuda(cudaEventRecord(side.done, side.stream), "record");
  if (rc) return rc;
  return check_cuda(cudaStreamWaitEvent(s, side.done, 0), "wait");
}

int b200k_attention_fwd_host(const b200k_attention_args* host, const b200k_attention_args* dev, void* stream) {
  if (!host || !dev) return set_error(B200K_ERR_NULL, "attention_fwd_host: args is NULL");
  if (!host->q || !host->k || !host->v || !host->o || !dev->q || !dev->k || !dev->v || !dev->o)
    return set_error(B200K_ERR_NULL, "attention_fwd_host: q, k, v, o must be non-NULL");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t es = dtype_size(dev->dtype);
  if (es != 2) return set_error(B200K_ERR_BAD_DTYPE, "attention_fwd_host: dtype must be F16 or BF16");
  // The host image must be densely packed [b, h, s, d] and so must the device image.
  const size_t qn = static_cast<size_t>(dev->batch) * dev->q_heads * dev->seq_q * dev->head_dim * es;
  const size_t kn = static_cast<size_t>(dev->batch) * dev->kv_heads * dev->seq_kv * dev->head_dim * es;
  auto dense = [&](const b200k_attention_args* a) {
    return a->q_stride_s == a->head_dim && a->q_stride_h == int64_t(a->seq_q) * a->head_dim &&
           a->q_stride_b == int64_t(a->q_heads) * a->seq_q * a->head_dim && a->k_stride_s == a->head_dim &&
           a->k_stride_h == int64_t(a->seq_kv) * a->head_dim &&
           a->k_stride_b == int64_t(a->kv_heads) * a->seq_kv * a->head_dim && a->v_stride_s == a->k_stride_s &&
           a->v_stride_h == a->k_stride_h && a->v_stride_b == a->k_stride_b && a->o_stride_s == a->q_stride_s &&
           a->o_stride_h == a->q_stride_h && a->o_stride_b == a->q_stride_b;
  };
  if (!dense(dev) || !dense(host))
    return set_error(B200K_ERR_BAD_SHAPE, "attention_fwd_host: host and device images must be dense [b,h,s,d]");
  // One batch element at a time: upload, compute, and copy the result back on the library's
  // copy-back stream while the next element is being uploaded.
  SideStream side;
  int rc = get_side_stream(&side);
  if (rc) return rc;
  const size_t q1 = qn / dev->batch, k1 = kn / dev->batch;
  for (int32_t b = 0; b < dev->batch; ++b) {
    b200k_attention_args one = *dev;
    one.batch = 1;
    one.q = static_cast<const char*>(dev->q) + b * q1;
    one.k = static_cast<const char*>(dev->k) + b * k1;
    one.v = static_cast<const char*>(dev->v) + b * k1;
    one.o = static_cast<char*>(dev->o) + b * q1;
    if (dev->lse) one.lse = dev->lse + static_cast<size_t>(b) * dev->q_heads * dev->seq_q;  // stays on the device
    rc = check_cuda(cudaMemcpyAsync(const_cast<void*>(one.q), static_cast<const char*>(host->q) + b * q1, q1,
                                    cudaMemcpyHostToDevice, s), "copy Q");
    if (rc) return rc;
    rc = check_cuda(cudaMemcpyAsync(const_cast<void*>(one.k), static_cast<const char*>(host->k) + b * k1, k1,
                                    cudaMemcpyHostToDevice, s), "copy K");
    if (rc) return rc;
    rc = check_cuda(cudaMemcpyAsync(const_cast<void*>(one.v), static_cast<const char*>(host->v) + b * k1, k1,
                                    cudaMemcpyHostToDevice, s), "copy V");
    if (rc) return rc;
    rc = launch_attention_fwd(one, s);
    if (rc) return rc;
    rc = check_cuda(cudaEventRecord(side.ready, s), "record");
    if (rc) return rc;
    rc = check_cuda(cudaStreamWaitEvent(side.stream, side.ready, 0), "wait");
    if (rc) return rc;
    rc = check_cuda(cudaMemcpyAsync(static_cast<char*>(host->o) + b * q1, one.o, q1, cudaMemcpyDeviceToHost,
                                    side.stream), "copy O");
    if (rc) return rc;
  }
  // the caller's stream completes only when every copy-back has
  rc = check_cuda(cudaEventRecord(side.done, side.stream), "record");
  if (rc) return rc;
  return check_cuda(cudaStreamWaitEvent(s, side.done, 0), "wait");
}

}  // extern "C"
